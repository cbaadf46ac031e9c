"""Python face of ``csrc/prenorm_stream.cu``: updates of a 32-bit residual stream with the norm of
the next sublayer in the same pass, q/k norm + pair rotation + cache write, the per-head output
gate and the gated gather of a token table."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import _code, _cuda, _fn, _ok, _p, _stream

NORM_NONE, NORM_LAYER, NORM_RMS = 0, 1, 2


def stream_update(x: torch.Tensor, act_dtype: torch.dtype, *, y=None, scale=None, mult: float = 1.0,
                  y_rms_eps: float | None = None, add_full=None, add_row=None, rows=None,
                  want_out: bool = True, want_act: bool = False, norm: int = NORM_NONE,
                  norm_weight=None, norm_bias=None, norm_eps: float = 0.0, pairs=None):
    """``x' = x (+ add_full) (+ add_row) + mult * f(y)`` on the fp32 stream ``x [R, H]``, with
    ``f(y) = y * scale`` (``scale`` fp32 ``[H]`` or ``None``) or, with ``y_rms_eps``,
    ``y / sqrt(mean(y^2) + y_rms_eps) * scale``.  ``rows`` (int32) selects rows of the inputs
    first.  Returns ``(x' fp32 or None, x' in act_dtype or None, norm(x') in act_dtype or None)``
    where the norm is a layer norm (``NORM_LAYER``: weight and optional bias) or an RMS norm
    (``NORM_RMS``), all sums in 32-bit.  ``pairs = (pos_of_pair [R * top] int32, weights [R, top]
    fp32 or None, top)``: ``y`` holds a row per (token, choice) pair and a token's ``y`` is the
    sum of its pairs' rows (times their weights), added up in the order chosen."""
    _cuda(x, y, scale, add_full, add_row, rows, norm_weight, norm_bias)
    pos_of_pair, pair_w, top = pairs if pairs is not None else (None, None, 0)
    _cuda(pos_of_pair, pair_w)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous()
    H = x.shape[1]
    R = x.shape[0] if rows is None else rows.numel()
    for v in (scale, add_row, norm_weight, norm_bias):
        assert v is None or (v.dtype == torch.float32 and v.numel() == H and v.is_contiguous())
    if pairs is not None:
        assert y is not None and rows is None and y.is_contiguous() and y.shape[1] == H
        assert pos_of_pair.dtype == torch.int32 and pos_of_pair.numel() == R * top
        assert pair_w is None or (pair_w.dtype == torch.float32 and pair_w.numel() == R * top
                                  and pair_w.is_contiguous())
    elif y is not None:
        assert y.shape == x.shape and y.is_contiguous()
    if add_full is not None:
        assert add_full.shape == x.shape and add_full.dtype == torch.float32 \
            and add_full.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    ymode = 0 if y is None else (2 if y_rms_eps is not None else 1)
    dev = x.device
    out = torch.empty((R, H), dtype=torch.float32, device=dev) if want_out else None
    act = None
    if want_act:
        act = out if (act_dtype == torch.float32 and out is not None) \
            else torch.empty((R, H), dtype=act_dtype, device=dev)
    normed = torch.empty((R, H), dtype=act_dtype, device=dev) if norm else None
    f = _fn("prenorm_stream", "gf_stream_update",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_float, c_float, c_void_p,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
             c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    rc = f(_p(x), _p(rows), _p(y), _code(y.dtype) if y is not None else 0, ymode, _p(scale),
           float(mult), float(y_rms_eps or 0.0), _p(add_full), _p(add_row), _p(out),
           _p(act) if act is not out else None, _code(act_dtype), int(norm), _p(norm_weight),
           _p(norm_bias), float(norm_eps), _p(normed), R, H, _p(pos_of_pair), _p(pair_w), int(top),
           _stream())
    if rc == -4:
        raise ValueError(f"rows of {H} channels do not fit the stream kernel's shared memory")
    _ok(rc, "stream_update")
    return out, act, normed


def qk_norm_rope(qkv: torch.Tensor, nh: int, nkv: int, hd: int, k_off: int, v_off: int, q_weight,
                 k_weight, eps: float, freqs, interleaved: bool, positions: torch.Tensor,
                 slot_mapping, pages: torch.Tensor, q_temp=None) -> None:
    """Per head of ``qkv [T, ...]`` (q heads from column 0, k heads from ``k_off``): RMS norm with
    the weight of its kind (``None``: no norm), rotation of the first ``2 len(freqs)`` channels in
    pairs by ``position * freqs[i]`` (neighbours ``(2i, 2i+1)`` if ``interleaved``, else halves);
    q in place; with ``slot_mapping`` k goes to ``pages[0]`` and the values (columns from
    ``v_off``, unchanged) to ``pages[1]``.  ``q_temp = (coef, every)``: the normed queries at
    position ``p`` are multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``."""
    _cuda(qkv, q_weight, k_weight, freqs, positions, slot_mapping, pages)
    assert qkv.dim() == 2 and qkv.stride(1) == 1
    assert pages.is_contiguous() and pages.dtype == qkv.dtype and pages.shape[0] == 2
    assert tuple(pages.shape[3:]) == (nkv, hd)
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == hd and w.is_contiguous())
    n_pairs = 0 if freqs is None else freqs.numel()
    if freqs is not None:
        assert freqs.dtype == torch.float32 and freqs.is_contiguous()
    f = _fn("prenorm_stream", "gf_qk_norm_rope",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
             c_float, c_int,
             c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    qt_coef, qt_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    _ok(f(_p(qkv), qkv.stride(0), qkv.shape[0], nh, nkv, hd, int(k_off), int(v_off), _p(q_weight),
          _p(k_weight), float(eps), qt_coef, qt_every, _p(freqs), n_pairs, int(bool(interleaved)), _p(positions),
          _p(slot_mapping), _p(pages[0]), _p(pages[1]), _code(qkv.dtype), _stream()),
        "qk_norm_rope")


def head_gate(o: torch.Tensor, gates: torch.Tensor, nh: int, hd: int) -> torch.Tensor:
    """``o [T, nh * hd]`` in place: head ``h`` times ``sigmoid(gates[t, h])`` (``gates`` a view
    with any row stride)."""
    _cuda(o, gates)
    assert o.is_contiguous() and o.shape[1] == nh * hd and gates.dtype == o.dtype
    assert gates.stride(1) == 1 and gates.shape == (o.shape[0], nh)
    f = _fn("prenorm_stream", "gf_head_gate",
            [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _ok(f(_p(o), _p(gates), gates.stride(0), o.shape[0], nh, hd, _code(o.dtype), _stream()),
        "head_gate")
    return o


def token_gate(z: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, offset: int
               ) -> torch.Tensor:
    """``gelu_tanh(z[t, j]) * table[token_ids[t], offset + j]`` in the table's dtype; ``z [T, dim]``
    fp32 or of that dtype."""
    _cuda(z, token_ids, table)
    assert z.dim() == 2 and z.is_contiguous() and table.stride(1) == 1
    assert token_ids.dtype == torch.int32 and token_ids.is_contiguous()
    T, dim = z.shape
    assert 0 <= offset and offset + dim <= table.shape[1]
    out = torch.empty((T, dim), dtype=table.dtype, device=z.device)
    f = _fn("prenorm_stream", "gf_token_gate",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int,
             c_void_p])
    _ok(f(_p(z), _code(z.dtype), _p(token_ids), _p(table), table.stride(0), int(offset), dim,
          _p(out), T, _code(table.dtype), _stream()), "token_gate")
    return out
