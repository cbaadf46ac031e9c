"""Linear recurrences with decays over per-request state (``csrc/decay_state.cu``): the
convolution and step sizes of a state-space mixer, the decays of gated linear attention, the
recurrence both share, and the gated norm of its output."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import _code, _cuda, _fn, _ok, _p, _stream


def ssd_prepare(proj: torch.Tensor, conv_col: int, dt_col: int, conv_w: torch.Tensor,
                conv_b: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor,
                state: torch.Tensor, ctx, H: int, channels: int, taps: int, conv_off: int):
    """``proj [T, ...]``: ``channels`` convolved columns from ``conv_col`` on, ``H`` step sizes
    from ``dt_col`` on.  Convolves over time (reading the slots' last inputs, and bringing them up
    to date afterwards), adds the bias, applies SiLU; ``dt = softplus(dt + dt_bias)``, decay
    ``exp(-exp(A_log) dt)``.  Returns fp32 ``(xbc [T, channels], rates [T, 2 H])``, decays in the
    first ``H`` columns of ``rates``, step sizes in the others."""
    _cuda(proj, conv_w, conv_b, dt_bias, A_log, state)
    T = proj.shape[0]
    assert proj.dim() == 2 and proj.stride(1) == 1
    assert state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    assert conv_w.dtype == torch.float32 and conv_w.shape == (channels, taps)
    assert conv_w.is_contiguous() and conv_b.dtype == torch.float32 and conv_b.numel() == channels
    assert dt_bias.dtype == torch.float32 and A_log.dtype == torch.float32
    xbc = torch.empty((T, channels), dtype=torch.float32, device=proj.device)
    rates = torch.empty((T, 2 * H), dtype=torch.float32, device=proj.device)
    f = _fn("decay_state", "gf_ssd_prepare",
            [c_void_p, c_int, c_int, c_int] + [c_void_p] * 8 + [c_int] * 7 +
            [c_void_p, c_void_p, c_int, c_void_p], kernels=2)
    rc = f(_p(proj), proj.stride(0), int(conv_col), int(dt_col), _p(conv_w), _p(conv_b),
           _p(dt_bias), _p(A_log), _p(state), _p(ctx.seq_of_token), _p(ctx.cu_seqlens_q),
           _p(ctx.slot_ids), T, ctx.num_seqs, H, channels, taps, state.stride(0), int(conv_off),
           _p(xbc), _p(rates), _code(proj.dtype), _stream())
    _ok(rc, "ssd_prepare")
    return xbc, rates


def gla_prepare(proj: torch.Tensor, z: torch.Tensor, HD: int, HV: int, q_scale: float,
                tau: float) -> torch.Tensor:
    """``proj [T, >= 2 HD + HV]`` (q | k | v first), ``z [T, HD]`` fp32 -> fp32 ``[T, 3 HD + HV]``
    laid out ``q * q_scale | k | sigmoid(z)^(1/tau) | v``."""
    _cuda(proj, z)
    T = proj.shape[0]
    assert proj.stride(1) == 1 and z.dtype == torch.float32 and z.is_contiguous()
    assert z.shape == (T, HD)
    out = torch.empty((T, 3 * HD + HV), dtype=torch.float32, device=proj.device)
    f = _fn("decay_state", "gf_gla_prepare",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p, c_int,
             c_void_p])
    _ok(f(_p(proj), proj.stride(0), _p(z), T, HD, HV, float(q_scale), 1.0 / float(tau), _p(out),
          _code(proj.dtype), _stream()), "gla_prepare")
    return out


def silu_f32(proj: torch.Tensor, width: int) -> torch.Tensor:
    """``silu`` of the first ``width`` columns of ``proj [T, ...]`` as fp32 ``[T, width]``: the
    operands of a linear attention whose q, k and v pass an activation and nothing else."""
    _cuda(proj)
    T = proj.shape[0]
    assert proj.dim() == 2 and proj.stride(1) == 1 and width <= proj.shape[1]
    out = torch.empty((T, width), dtype=torch.float32, device=proj.device)
    f = _fn("decay_state", "gf_silu_f32",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p])
    _ok(f(_p(proj), proj.stride(0), T, int(width), _p(out), _code(proj.dtype), _stream()),
        "silu_f32")
    return out


# The recurrence keeps a column's rows of the state in registers: key sizes up to this.
MAX_KEY_SIZE = 256

# With fewer blocks of four lanes a column than this (requests x heads x tiles of 32 columns), long
# portions take sixteen lanes a column: four times the blocks, each with a shorter chain a token.
# Measured on a B200 with 2,048-token portions and key sizes 64 and 128: sixteen lanes win up to 64
# such blocks (430 against 605 us at 32, 540 against 605 us at 64), are level at 96 and lose from
# 128 on (710 against 605 us), where four lanes a column already give every SM a block.
WIDE_BELOW_BLOCKS = 96
WIDE_MIN_TOKENS = 64


def recurrence(q, k, v, g, state: torch.Tensor, ctx, H: int, G: int, D: int, Vd: int,
               k_scale=None, skip=None) -> torch.Tensor:
    """Advance every request's state ``S [H, D, Vd]`` (first in its slot) over its tokens of this
    step: ``S <- diag(g_t) S + (c_t k_t) v_t^T``, ``o_t = S^T q_t + skip_h v_t``.  ``q``, ``k``:
    fp32 rows of ``G`` heads of ``D`` (views with a row stride are fine); ``v``: rows of ``H`` heads
    of ``Vd``; ``g``: rows of ``H * D`` decays, or of ``H`` (one a head); ``k_scale``: rows of
    ``H`` factors ``c`` or ``None``; ``skip``: ``[H]`` or ``None``.  Returns ``o [T, H * Vd]``."""
    _cuda(q, k, v, g, k_scale, skip, state)
    T = v.shape[0]
    for t in (q, k, v, g, k_scale):
        assert t is None or (t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1)
    assert q.shape[1] == G * D and k.shape[1] == G * D and v.shape[1] == H * Vd
    gD = g.shape[1] // H
    assert g.shape[1] == H * gD and gD in (1, D)
    assert state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    o = torch.empty((T, H * Vd), dtype=torch.float32, device=v.device)
    blocks = ctx.num_seqs * H * (-(-Vd // 32))
    wide = int(blocks < WIDE_BELOW_BLOCKS and ctx.max_q_len >= WIDE_MIN_TOKENS)
    f = _fn("decay_state", "gf_decay_recurrence",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
             c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 5 +
            [c_void_p, c_int, c_int, c_void_p])
    rc = f(_p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(g), g.stride(0), gD,
           _p(k_scale), k_scale.stride(0) if k_scale is not None else 0, _p(skip), _p(state),
           state.stride(0), _p(ctx.cu_seqlens_q), _p(ctx.slot_ids), ctx.num_seqs, H, G, D, Vd,
           _p(o), o.stride(0), wide, _stream())
    if rc == -3:
        raise ValueError(f"the recurrence takes key sizes up to 256 and heads that are a multiple "
                         f"of the groups; got key size {D}, {H} heads, {G} groups")
    _ok(rc, "decay_recurrence")
    return o


def gated_norm(o: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, group_size: int,
               gate_first: bool, eps: float, dtype: torch.dtype, sigmoid_gate: bool = False
               ) -> torch.Tensor:
    """RMS norm of ``o [T, C]`` (fp32) in groups of ``group_size`` channels with a SiLU gate (a
    plain sigmoid with ``sigmoid_gate``):
    ``gate_first``: ``y = o silu(gate)``, then ``y / rms(y) * w``; else ``o / rms(o) * w *
    silu(gate)``.  ``w`` has ``C`` weights, or ``group_size`` shared by the groups.  ``gate``:
    ``[T, C]``, fp32 or the activation dtype, rows may be strided.  Returns ``[T, C]`` in
    ``dtype``."""
    _cuda(o, gate, w)
    T, C = o.shape
    assert o.dtype == torch.float32 and o.is_contiguous() and C % group_size == 0
    assert gate.shape == (T, C) and gate.stride(1) == 1
    assert w.dtype == torch.float32 and w.numel() in (C, group_size) and w.is_contiguous()
    out = torch.empty((T, C), dtype=dtype, device=o.device)
    f = _fn("decay_state", "gf_gated_norm",
            [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_int,
             c_int, c_int, c_int, c_void_p])
    shared = int(w.numel() == group_size and C != group_size)
    _ok(f(_p(o), _p(gate), gate.stride(0), _code(gate.dtype), _p(w), shared, int(bool(gate_first)) | (2 if sigmoid_gate else 0),
          float(eps), _p(out), T, C // group_size, int(group_size), _code(dtype), _stream()),
        "gated_norm")
    return out
