"""Python face of ``csrc/depth_stream.cu``: a 32-bit residual stream with norms on both sides of
every sublayer and a weighted average over the depth of the model."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import _code, _cuda, _fn, _ok, _p, _stream


def embedding_positions(token_ids: torch.Tensor, positions: torch.Tensor, weight: torch.Tensor,
                        pos_table: torch.Tensor, out: torch.Tensor | None = None,
                        norm_weight=None, norm_eps: float = 0.0, act_dtype=None):
    """``x[t] = float(weight[ids[t]]) + float(pos_table[positions[t]])`` as the fp32 stream
    (written into ``out`` if given); with ``norm_weight`` (fp32) also its RMS norm in
    ``act_dtype``.  Returns ``(x, normed or None)``."""
    _cuda(token_ids, positions, weight, pos_table, out, norm_weight)
    assert token_ids.dtype == torch.int32 and token_ids.is_contiguous()
    assert positions.dtype == torch.int32 and positions.is_contiguous()
    assert weight.is_contiguous() and pos_table.is_contiguous()
    assert weight.dtype == pos_table.dtype and weight.shape[1] == pos_table.shape[1]
    T, H = token_ids.numel(), weight.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=weight.device)
    assert out.dtype == torch.float32 and out.shape == (T, H) and out.is_contiguous()
    act = act_dtype or weight.dtype
    normed = None
    if norm_weight is not None:
        assert norm_weight.dtype == torch.float32 and norm_weight.numel() == H
        normed = torch.empty((T, H), dtype=act, device=weight.device)
    f = _fn("depth_stream", "gf_embedding_pos",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p,
             c_int, c_int, c_int, c_void_p])
    rc = f(_p(token_ids), _p(positions), _p(weight), _p(pos_table), _code(weight.dtype), _p(out),
           _p(norm_weight), float(norm_eps), _p(normed), _code(act), T, H, _stream())
    if rc == -4:
        raise ValueError(f"rows of {H} channels do not fit the kernel's shared memory")
    _ok(rc, "embedding_positions")
    return out, normed


def sandwich_update(x: torch.Tensor, y: torch.Tensor, gamma_b: torch.Tensor, eps: float,
                    act_dtype: torch.dtype, *, history=None, mix_weights=None, n_before: int = 0,
                    next_weight=None, next_eps: float = 0.0, want_out: bool = True, y_bias=None):
    """The end of a sublayer on the fp32 stream ``x [R, H]``: ``v = x + y * gamma_b / rms(y)``
    (``y_bias``, fp32 ``[H]``: added to every row of ``y`` first).
    With ``history [states, R, H]`` and ``mix_weights [n_before + 1]`` (fp32), ``v`` is stored as
    state ``n_before`` of the history and the stream becomes ``sum_j mix_weights[j] * state_j``
    over the states ``0 .. n_before``.  With ``next_weight`` (fp32 ``[H]``) the RMS norm of the new
    stream is formed in the same pass.  Returns ``(stream or None, normed in act_dtype or
    None)``."""
    _cuda(x, y, gamma_b, history, mix_weights, next_weight, y_bias)
    assert y_bias is None or (y_bias.dtype == torch.float32 and y_bias.numel() == x.shape[1]
                              and y_bias.is_contiguous())
    assert x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous()
    assert y.shape == x.shape and y.is_contiguous()
    R, H = x.shape
    assert gamma_b.dtype == torch.float32 and gamma_b.numel() == H and gamma_b.is_contiguous()
    hist = keep = None
    stride = 0
    if mix_weights is not None:
        assert history is not None and history.dtype == torch.float32 and history.is_contiguous()
        assert history.shape[1:] == (R, H) and 0 < n_before < history.shape[0]
        assert mix_weights.dtype == torch.float32 and mix_weights.numel() == n_before + 1
        assert mix_weights.is_contiguous()
        hist, keep, stride = history, history[n_before], R * H
    out = torch.empty_like(x) if want_out else None
    normed = None
    if next_weight is not None:
        assert next_weight.dtype == torch.float32 and next_weight.numel() == H
        normed = torch.empty((R, H), dtype=act_dtype, device=x.device)
    f = _fn("depth_stream", "gf_sandwich_update",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_longlong,
             c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p])
    rc = f(_p(x), _p(y), _code(y.dtype), _p(y_bias), _p(gamma_b), float(eps), _p(hist), _p(mix_weights),
           int(n_before), stride, _p(keep), _p(out), _p(next_weight), float(next_eps), _p(normed),
           _code(act_dtype), R, H, _stream())
    if rc == -4:
        raise ValueError(f"rows of {H} channels do not fit the kernel's shared memory")
    _ok(rc, "sandwich_update")
    return out, normed
