"""Python face of the hand-written CUDA kernels.

Every function here launches a kernel from ``csrc/`` on the current CUDA stream (matrix products
of the bf16 path may go to cuBLAS, as the reference's do:
``ginfer/core/op/kernels/cuda/gemm_kernel/gemm_kernel.cu:93-156``).  There is no CPU path: a
tensor that is not on a CUDA device is an error, and so is a library that cannot be built.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import BuildError, build_all, load_library, set_pdl  # noqa: F401

_CODES = {torch.float32: 0, torch.bfloat16: 1}


def _code(dt: torch.dtype) -> int:
    try:
        return _CODES[dt]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 activations, not {dt}") from None


def _p(t):
    """The device address of a tensor for a kernel (``None`` stays ``None``).  A tensor that is
    not on a CUDA device is refused here: its address would mean nothing to a kernel."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("ginfer_b200 kernels run on a CUDA device only; got a tensor on "
                           f"{t.device}")
    return c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("ginfer_b200 kernels run on a CUDA device only; got a tensor on "
                               f"{t.device}")


def _ok(rc: int, what: str):
    if rc > 0:
        raise RuntimeError(f"{what}: CUDA error {rc} at launch")
    if rc < 0:
        raise RuntimeError(f"{what}: the kernel refused its arguments (code {rc})")


class _Counter:
    """Kernel launches made through this module (each entry point launches one kernel unless it
    says otherwise); read by the benchmark."""
    launches = 0


_fns: dict = {}


def _fn(lib_name: str, fn_name: str, argtypes, defines=(), kernels: int = 1):
    key = (lib_name, tuple(defines), fn_name)
    g = _fns.get(key)
    if g is None:
        lib = load_library(lib_name, tuple(defines))
        f = getattr(lib, fn_name)
        f.argtypes = argtypes
        f.restype = c_int

        def g(*args, _f=f, _k=kernels):
            _Counter.launches += _k
            return _f(*args)
        _fns[key] = g
    return g


def launch_count() -> int:
    return _Counter.launches


# ----------------------------------------------------------------------------- embedding
def embedding(token_ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    _cuda(token_ids, weight)
    assert token_ids.dtype == torch.int32 and token_ids.is_contiguous()
    T, (V, H) = token_ids.numel(), weight.shape
    out = torch.empty((T, H), dtype=weight.dtype, device=weight.device)
    f = _fn("elementwise", "gf_embedding",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _ok(f(_p(token_ids), _p(weight), _p(out), T, H, _code(weight.dtype), _stream()), "embedding")
    return out


def embedding_scaled(token_ids: torch.Tensor, weight: torch.Tensor, scale: float,
                     want_act: bool):
    """``x = float(W[ids]) * scale`` as the fp32 residual stream; with ``want_act`` also its
    rounding to the weight's dtype (what the first sublayer's products read), else ``None``."""
    _cuda(token_ids, weight)
    assert token_ids.dtype == torch.int32 and token_ids.is_contiguous() and weight.is_contiguous()
    T, (V, H) = token_ids.numel(), weight.shape
    out = torch.empty((T, H), dtype=torch.float32, device=weight.device)
    act = torch.empty((T, H), dtype=weight.dtype, device=weight.device) if want_act else None
    f = _fn("stream_ops", "gf_embedding_scaled",
            [c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
             c_void_p])
    _ok(f(_p(token_ids), _p(weight), _code(weight.dtype), float(scale), _p(out), _p(act),
          _code(weight.dtype), T, H, _stream()), "embedding_scaled")
    return out, act


def outnorm_add(x: torch.Tensor, y: torch.Tensor, gamma: torch.Tensor, eps: float,
                act_dtype: torch.dtype, want_act: bool = True):
    """``x' = x + y * gamma / rms(y)`` (fp32; ``x`` the fp32 stream, ``y`` a sublayer's output in
    fp32 or the activation dtype, ``gamma`` fp32) and, with ``want_act``, ``x'`` rounded to
    ``act_dtype`` for the next sublayer's products."""
    _cuda(x, y, gamma)
    assert x.dtype == torch.float32 and gamma.dtype == torch.float32
    assert x.dim() == 2 and x.is_contiguous() and y.is_contiguous() and y.shape == x.shape
    R, H = x.shape
    out = torch.empty_like(x)
    act = torch.empty((R, H), dtype=act_dtype, device=x.device) \
        if want_act and act_dtype != torch.float32 else None
    f = _fn("stream_ops", "gf_outnorm_add",
            [c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
             c_int, c_void_p])
    rc = f(_p(x), _p(y), _code(y.dtype), _p(gamma), float(eps), _p(out), _p(act),
           _code(act_dtype), R, H, _stream())
    if rc == -4:
        raise ValueError(f"rows of {H} channels do not fit the norm kernel's shared memory")
    _ok(rc, "outnorm_add")
    return out, (out if act_dtype == torch.float32 else act)


def clamped_glu(gate_up: torch.Tensor, limit: float, alpha: float, up_shift: float
                ) -> torch.Tensor:
    """``gate_up [T, 2 I]`` with gate and up interleaved -> ``min(g, limit) * sigmoid(alpha *
    min(g, limit)) * (clamp(u, -limit, limit) + up_shift)``, ``[T, I]``."""
    _cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    T, I = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("stream_ops", "gf_clamped_glu",
            [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float, c_int, c_void_p])
    _ok(f(_p(gate_up), _p(out), T, I, float(limit), float(alpha), float(up_shift),
          _code(gate_up.dtype), _stream()), "clamped_glu")
    return out


def postnorm(x: torch.Tensor, y: torch.Tensor, alpha: float, gamma: torch.Tensor, eps: float,
             act_dtype: torch.dtype, want_act: bool = True, pairs=None):
    """Norm after the sum: ``x' = s * gamma / rms(s)`` with ``s = alpha * x + y`` (fp32; ``x`` the
    fp32 stream, ``y`` a sublayer's output in fp32 or the activation dtype, ``gamma`` fp32) and,
    with ``want_act``, ``x'`` rounded to ``act_dtype``.  ``pairs = (pos_of_pair, weights or None,
    top)``: ``y`` holds a row per (token, choice) pair of a routed feed-forward and the kernel
    adds a token's rows up itself."""
    _cuda(x, y, gamma)
    assert x.dtype == torch.float32 and gamma.dtype == torch.float32
    assert x.dim() == 2 and x.is_contiguous() and y.is_contiguous() and y.shape[1] == x.shape[1]
    R, H = x.shape
    pos = wgt = None
    top = 0
    if pairs is not None:
        pos, wgt, top = pairs
        assert pos.numel() == R * top and y.dtype == torch.float32
    else:
        assert y.shape == x.shape
    out = torch.empty_like(x)
    act = torch.empty((R, H), dtype=act_dtype, device=x.device) \
        if want_act and act_dtype != torch.float32 else None
    f = _fn("stream_ops", "gf_postnorm",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_float,
             c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    rc = f(_p(x), _p(y), _code(y.dtype), _p(pos), _p(wgt), int(top), float(alpha), _p(gamma),
           float(eps), _p(out), _p(act), _code(act_dtype), R, H, _stream())
    if rc == -4:
        raise ValueError(f"rows of {H} channels do not fit the norm kernel's shared memory")
    _ok(rc, "postnorm")
    return out, (out if act_dtype == torch.float32 else act)


def qk_wide_prepare(qkv: torch.Tensor, nh: int, nkv: int, hd: int, vd: int, k_off: int,
                    v_off: int, q_w, k_w, eps: float, freqs, rot: int, positions: torch.Tensor,
                    slot_mapping, kpages: torch.Tensor, vpages: torch.Tensor, v_first=None,
                    mix=None) -> None:
    """A token's q | k | v row before attention where q and k are normed over the whole
    projection: ``q / rms(q) * q_w`` over all heads at once (``k`` likewise; no norm without
    weights), rotation of the first ``rot`` channels of every head in pairs ``(i, i + rot/2)`` by
    ``float(position) * freqs[i]``, values mixed with ``v_first`` (``(1 - mix) v + mix v_first``,
    ``mix`` a one-element fp32 tensor on the device); q in place, k and v into the cache slot
    ``slot_mapping`` names (``None``: nothing is written)."""
    _cuda(qkv, q_w, k_w, freqs, positions, slot_mapping, kpages, vpages, v_first, mix)
    assert qkv.dim() == 2 and qkv.stride(1) == 1
    assert kpages.is_contiguous() and vpages.is_contiguous() and kpages.dtype == qkv.dtype
    assert tuple(kpages.shape[-2:]) == (nkv, hd) and tuple(vpages.shape[-2:]) == (nkv, vd)
    if v_first is not None:
        assert v_first.dtype == qkv.dtype and v_first.stride(1) == 1 and mix.dtype == torch.float32
        assert v_first.shape == (qkv.shape[0], nkv * vd)
    f = _fn("qk_wide", "gf_qk_wide_prepare",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
             c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_int, c_void_p])
    rc = f(_p(qkv), qkv.stride(0), qkv.shape[0], nh, nkv, hd, vd, int(k_off), int(v_off), _p(q_w),
           _p(k_w), float(eps), _p(freqs), int(rot), _p(positions), _p(slot_mapping), _p(kpages),
           _p(vpages), _p(v_first), v_first.stride(0) if v_first is not None else 0, _p(mix),
           _code(qkv.dtype), _stream())
    if rc == -3:
        raise ValueError(f"{rot} rotated channels must be an even number within the head of {hd}")
    _ok(rc, "qk_wide_prepare")


# ----------------------------------------------------------------------------- add + rmsnorm
def add_rmsnorm(x: torch.Tensor, delta, gamma: torch.Tensor, eps: float, rows=None,
                want_sum: bool = True, out_dtype=None):
    """``s = x + delta`` in fp32; returns ``(s or None, s * gamma / rms(s))``.  ``x`` is the fp32
    residual stream or an activation; ``delta`` and the normed output have the activation dtype
    (``out_dtype``, else that of ``delta``, else of ``x``).  Without ``delta`` and ``rows`` the
    returned ``s`` is ``x`` itself."""
    _cuda(x, delta, gamma, rows)
    assert x.dim() == 2 and x.is_contiguous()
    H = x.shape[1]
    act = out_dtype or (x.dtype if delta is None else delta.dtype)
    if delta is not None:
        assert delta.shape == x.shape and delta.is_contiguous()
    assert gamma.numel() == H and gamma.is_contiguous()
    R = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    normed = torch.empty((R, H), dtype=act, device=x.device)
    s = None
    if want_sum:
        if delta is None and rows is None:
            s = x
        elif delta is None:
            s = x.index_select(0, rows.long())
        else:
            s = torch.empty((R, H), dtype=torch.float32, device=x.device)
    f = _fn("elementwise", "gf_add_rmsnorm",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_void_p])
    sum_ptr = _p(s) if (want_sum and delta is not None) else None
    _ok(f(_p(x), _code(x.dtype), _p(delta), _p(gamma), _code(gamma.dtype), float(eps), _p(rows),
          sum_ptr, _p(normed), R, H, _code(act), _stream()), "add_rmsnorm")
    return s, normed


# ----------------------------------------------------------------------------- rope + KV write
def rope_kv_write(qkv: torch.Tensor, table, rotary_dim: int, positions: torch.Tensor,
                  slot_mapping, pages: torch.Tensor, nh: int, nkv: int, hd: int) -> None:
    """Rotate the q and k heads of ``qkv [T, (nh + 2 nkv) hd]`` (q in place) and, when
    ``slot_mapping`` is given, write k and v into ``pages [2, num_pages, page, nkv, hd]``."""
    _cuda(qkv, table, positions, slot_mapping, pages)
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == (nh + 2 * nkv) * hd
    assert pages.is_contiguous() and pages.dtype == qkv.dtype and pages.shape[0] == 2
    assert tuple(pages.shape[3:]) == (nkv, hd)
    if table is not None:
        assert table.dtype == torch.float32 and table.is_contiguous()
        assert table.shape[1] == rotary_dim and rotary_dim % 2 == 0 and rotary_dim <= hd
    T = qkv.shape[0]
    f = _fn("elementwise", "gf_rope_kv_write",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_void_p])
    _ok(f(_p(qkv), qkv.stride(0), _p(table), int(rotary_dim), _p(positions), _p(slot_mapping),
          _p(pages[0]), _p(pages[1]), T, nh, nkv, hd, _code(qkv.dtype), _stream()),
        "rope_kv_write")


# ----------------------------------------------------------------------------- silu * up
def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``gate_up [T, 2 I]`` with gate and up interleaved (g0, u0, g1, u1, ...) -> ``[T, I]``."""
    _cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    T, I = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((T, I), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("elementwise", "gf_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _ok(f(_p(gate_up), _p(out), T, I, _code(gate_up.dtype), _stream()), "silu_mul")
    return out


def activation_(x: torch.Tensor, kind: str, c: float = 0.0) -> torch.Tensor:
    """In place, fp32 arithmetic: ``kind`` ``"relu2"``: ``relu(x)^2``; ``"softcap"``:
    ``c * tanh(x / c)``."""
    _cuda(x)
    assert x.is_contiguous()
    f = _fn("elementwise", "gf_activation",
            [c_void_p, c_longlong, c_int, c_float, c_int, c_void_p])
    rc = f(_p(x), x.numel(), {"relu2": 0, "softcap": 1}[kind], float(c), _code(x.dtype), _stream())
    if rc == -3:
        raise ValueError(f"activation {kind!r} with constant {c}")
    _ok(rc, "activation")
    return x


# ----------------------------------------------------------------------------- attention
def mask_span(window: int = 0, chunk: int = 0) -> int:
    """How the attention kernels are told their mask, as one integer: 0 = every earlier key,
    ``window`` > 0 = the last ``window`` keys, ``-chunk`` = the keys of the query's own chunk of
    ``chunk`` positions (chunks are counted from position 0 of the sequence)."""
    if window and chunk:
        raise ValueError("a mask is a sliding window or chunks, not both")
    return int(window) if window else -int(chunk)


def paged_attention_simt(qkv, pages, block_table, seq_of_token, positions, nh, nkv, hd, scale,
                         window, page_size, vd=None, softcap: float = 0.0, slopes=None):
    """``window``: the mask as :func:`mask_span` gives it.  ``vd``: the values' head size where
    it is not the keys' (``pages`` is then a pair of tensors).  ``softcap`` > 0: scores pass
    ``cap * tanh(s / cap)``; ``slopes`` (fp32, a head): ``slope * (p - c)`` is taken off the score
    of the key at ``c`` for the query at ``p``, after the cap."""
    _cuda(qkv, pages[0], pages[1], block_table, seq_of_token, positions, slopes)
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == nh
                              and slopes.is_contiguous())
    T = qkv.shape[0]
    vd = hd if vd is None else int(vd)
    out = torch.empty((T, nh * vd), dtype=qkv.dtype, device=qkv.device)
    f = _fn("attention_simt", "gf_paged_attention_simt",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_int,
             c_void_p])
    rc = f(_p(qkv), qkv.stride(0), _p(pages[0]), _p(pages[1]), _p(block_table),
           block_table.stride(0), _p(seq_of_token), _p(positions), _p(out), T, nh, nkv, hd, vd,
           page_size, int(window), float(scale), float(softcap or 0.0), _p(slopes),
           _code(qkv.dtype), _stream())
    if rc == -3:
        raise ValueError(f"attention kernels take head sizes up to 256 and head counts that are "
                         f"a multiple of the kv head count; got head_dim={hd}, heads={nh}, "
                         f"kv_heads={nkv}")
    _ok(rc, "paged_attention_simt")
    return out


def attention_fuses_rope(qkv: torch.Tensor, ctx, nh: int, nkv: int, hd: int) -> bool:
    """True if :func:`paged_attention` can rotate q and k and write the new k and v itself for
    this step (pass ``rope=`` then, and skip :func:`rope_kv_write`)."""
    from . import attention_bf16
    return attention_bf16.fuses_rope(qkv, ctx, hd, nh, nkv)


def paged_attention(qkv: torch.Tensor, pages, block_table: torch.Tensor, ctx,
                    nh: int, nkv: int, hd: int, scale: float, window: int, page_size: int,
                    rope=None, vd: int | None = None, softcap: float = 0.0,
                    slopes=None) -> torch.Tensor:
    """Attention of the step's queries (first ``nh * hd`` columns of ``qkv``) over the paged
    cache; returns ``[T, nh * hd]``.  Picks the kernel by dtype, head size and batch shape.
    ``rope = (table or None, rotary_dim, write)`` where :func:`attention_fuses_rope`: q and k are
    still unrotated and the new k and v not yet in the cache.  ``window``: the mask as
    :func:`mask_span` gives it.  ``vd``: the values' head size if it differs from ``hd``
    (``pages`` is then the pair of the cache's two planes; the result is ``[T, nh * vd]``).
    ``softcap``, ``slopes``: a soft cap on the scores and a distance bias a head, see
    :func:`paged_attention_simt`."""
    from . import attention_bf16
    shaped = dict(softcap=float(softcap or 0.0), slopes=slopes)
    if vd is not None and vd != hd:        # keys and values of different widths: the plain kernel
        assert rope is None
        return paged_attention_simt(qkv, pages, block_table, ctx.seq_of_token, ctx.positions, nh,
                                    nkv, hd, scale, window, page_size, vd=vd, **shaped)
    if qkv.dtype == torch.bfloat16:
        out = attention_bf16.try_run(qkv, pages, block_table, ctx, nh, nkv, hd, scale, window,
                                     page_size, rope=rope, **shaped)
        if out is not None:
            return out
    assert rope is None
    return paged_attention_simt(qkv, pages, block_table, ctx.seq_of_token, ctx.positions, nh, nkv,
                                hd, scale, window, page_size, **shaped)


# ----------------------------------------------------------------------------- sampling
_argmax_scratch: dict = {}


def argmax(logits: torch.Tensor) -> torch.Tensor:
    _cuda(logits)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    words = 2 * R * (-(-V // 4096))
    if torch.cuda.is_current_stream_capturing():
        scratch = torch.empty(words, dtype=torch.int32, device=logits.device)
    else:
        scratch = _argmax_scratch.get(logits.device)
        if scratch is None or scratch.numel() < words:
            scratch = torch.empty(max(words, 1 << 16), dtype=torch.int32, device=logits.device)
            _argmax_scratch[logits.device] = scratch
    f = _fn("sampling", "gf_argmax", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    rc = f(_p(logits), _p(out), R, V, _p(scratch), _stream())
    if rc == -5:
        raise ValueError(f"argmax takes at most 4096 rows at a time, got {R}")
    _ok(rc, "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """Row ``r``: arg-max if ``temperature[r] <= 0`` else the first index whose cumulative
    ``softmax(logits / temperature)`` reaches ``u[r]``."""
    _cuda(logits, temperature, u)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    R, V = logits.shape
    assert temperature.dtype == torch.float32 and u.dtype == torch.float32
    assert temperature.numel() == R and u.numel() == R
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _fn("sampling", "gf_sample",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _ok(f(_p(logits), _p(temperature), _p(u), _p(out), R, V, _stream()), "sample")
    return out


def scatter_tokens(dst: torch.Tensor, dst_idx: torch.Tensor, src: torch.Tensor,
                   src_idx: torch.Tensor) -> None:
    """``dst[dst_idx[i]] = src[src_idx[i]]`` (all int32, on the device)."""
    _cuda(dst, dst_idx, src, src_idx)
    assert all(t.dtype == torch.int32 for t in (dst, dst_idx, src, src_idx))
    n = dst_idx.numel()
    assert src_idx.numel() == n
    f = _fn("sampling", "gf_scatter_tokens",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _ok(f(_p(dst), _p(dst_idx), _p(src), _p(src_idx), n, _stream()), "scatter_tokens")


def qkv_rope_write(x, linear, table, rot, positions, slot_mapping, pages, nh, nkv, hd):
    """``linear(x)`` with q and k rotated and k and v written to the cache by the product's own
    epilogue, where that is served (bf16, many tokens; see ``gemm_prefill.qkv_rope_write``), else
    ``None``."""
    if (getattr(linear, "dtype", None) != torch.bfloat16 or x.dtype != torch.bfloat16
            or linear.out_dtype != torch.bfloat16):
        return None
    from . import gemm_prefill
    return gemm_prefill.qkv_rope_write(x, linear.weight, linear._bias_f32, table, rot, positions,
                                       slot_mapping, pages, nh, nkv, hd)


def bmm_f32_out(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched product ``[B, M, K] @ [B, K, N]`` with an fp32 result (fp32 accumulation; from
    fp32 operands a true 32-bit product: the reduced-precision matrix modes stay off)."""
    _cuda(a, b)
    if a.dtype == torch.float32:
        assert not torch.backends.cuda.matmul.allow_tf32
        return torch.bmm(a, b)
    return torch.bmm(a, b, out_dtype=torch.float32)


from .linear import GatedLinear, Linear, add_to  # noqa: E402,F401
from . import prenorm  # noqa: E402,F401
from . import depth  # noqa: E402,F401
