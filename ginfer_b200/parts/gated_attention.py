"""Grouped-query attention with normed queries and keys and a gate on every head's output.

``q = W_q h``, ``k = W_k h``; the values are the keys as projected (before norm and rotation), or
``W_v h`` with ``value_projection``.  Each head of q and k is RMS-normed over its channels with
one weight vector for all heads (``q.norm``, ``k.norm``), then rotated by the position encoding
(pairs of channels).  ``score = q.k * scale`` over the keys ``j`` with ``0 <= p - j < window``
(all earlier keys without a window), softmax, query head ``n`` reads kv head
``n / (heads / kv_heads)``.  Head ``n``'s output is multiplied by ``sigmoid(W_g h)_n`` before
``W_o``.

Options for designs without rotation: ``position = None`` (positions enter only through what
follows); ``q_temp = (coef, every)``: the normed query at position ``p`` is multiplied by ``1 + coef
* ln(floor((p + 1) / every) + 1)``; ``softcap``: ``score <- cap * tanh(score / cap)`` after the
scale; ``distance_slope_base = b``: head ``n`` of ``H`` takes ``2^(-b (n + 1) / H) * (p - j)`` off the
score of key ``j`` (after the cap, before the softmax).

One product over the joined matrices gives q, k, (v) and the gates; one kernel norms and rotates q
in place and writes the normed, rotated k and the values to their cache slots; the attention
kernels of the plain grouped-query mixer run over that cache; one kernel applies the gates.
Norms, angles, scores, softmax and the gates' sigmoids are 32-bit arithmetic in both paths.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import prenorm
from .base import Mixer, PagedKVSpec, TensorSpec, make_part, register_mixer
from .plan import PartSpec


class NormedGatedAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, position: PartSpec | None, window: int = 0, qk_norm: bool = True,
                 qk_norm_eps: float = 1e-6, value_projection: bool = False,
                 head_gate: bool = True, prefix: str = "mix", q_temp=None,
                 softcap: float | None = None, distance_slope_base: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size = int(hidden_size)
        self.nh, self.nkv, self.hd = int(num_heads), int(num_kv_heads), int(head_dim)
        self.scale, self.window = float(scale), int(window)
        self.qk_norm, self.eps = bool(qk_norm), float(qk_norm_eps)
        self.value_projection, self.gated = bool(value_projection), bool(head_gate)
        self.prefix = prefix + "." if prefix else ""
        self.position = make_part("position", position) if position is not None else None
        if self.position is not None:
            if not hasattr(self.position, "frequencies"):
                raise ValueError("this mixer rotates channel pairs by frequencies; its position "
                                 "encoding must give them (kind 'pair_rotary')")
            if self.position.dims > self.hd:
                raise ValueError(f"{self.position.dims} rotated channels do not fit a head of "
                                 f"{self.hd}")
        self.q_temp = None
        if q_temp is not None:
            coef, every = float(q_temp[0]), int(q_temp[1])
            if every <= 0:
                raise ValueError(f"q_temp: 'every' must be positive, got {every}")
            self.q_temp = (coef, every)
        self.softcap = float(softcap) if softcap else 0.0
        if self.softcap < 0:
            raise ValueError(f"softcap must be positive, got {softcap}")
        self.slope_base = None if distance_slope_base is None else float(distance_slope_base)
        self.slopes = None

    def _n(self, name):
        return self.prefix + name

    def tensor_specs(self):
        W, nh, nkv, hd = self.hidden_size, self.nh, self.nkv, self.hd
        out = [TensorSpec(self._n("q"), (nh * hd, W)), TensorSpec(self._n("k"), (nkv * hd, W))]
        if self.value_projection:
            out.append(TensorSpec(self._n("v"), (nkv * hd, W)))
        if self.qk_norm:
            out += [TensorSpec(self._n("q.norm"), (hd,), "norm32"),
                    TensorSpec(self._n("k.norm"), (hd,), "norm32")]
        if self.gated:
            out.append(TensorSpec(self._n("g"), (nh, W)))
        out.append(TensorSpec(self._n("o"), (W, nh * hd)))
        return out + (self.position.tensor_specs() if self.position is not None else [])

    def load(self, tensors, dtype, device):
        nh, nkv, hd = self.nh, self.nkv, self.hd
        parts = [tensors[self._n("q")], tensors[self._n("k")]]
        self.k_off = nh * hd
        self.v_off = self.k_off
        cols = (nh + nkv) * hd
        if self.value_projection:
            parts.append(tensors[self._n("v")])
            self.v_off, cols = cols, cols + nkv * hd
        self.g_off = cols
        if self.gated:
            parts.append(tensors[self._n("g")])
            cols += nh
        if cols % 8:      # rows of the product stay 16-byte aligned in bfloat16
            parts.append(torch.zeros((8 - cols % 8, self.hidden_size), dtype=parts[0].dtype,
                                     device=parts[0].device))
        self.qkv = ops.Linear(torch.cat(parts, dim=0))
        self.q_w = tensors[self._n("q.norm")].float().contiguous() if self.qk_norm else None
        self.k_w = tensors[self._n("k.norm")].float().contiguous() if self.qk_norm else None
        self.out = ops.Linear(tensors[self._n("o")], None, out_dtype=torch.float32)
        if self.position is not None:
            self.position.load(tensors, dtype, device)
        if self.slope_base is not None:
            self.slopes = torch.tensor([2.0 ** (-self.slope_base * (n + 1) / nh)
                                        for n in range(nh)], dtype=torch.float32, device=device)

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.hd, self.window)

    def forward(self, x, ctx, cache):
        nh, nkv, hd = self.nh, self.nkv, self.hd
        qkv = self.qkv(x)
        pos = self.position
        prenorm.qk_norm_rope(qkv, nh, nkv, hd, self.k_off, self.v_off, self.q_w, self.k_w,
                             self.eps, pos.frequencies() if pos is not None else None,
                             pos.interleaved if pos is not None else False,
                             ctx.positions, cache.slot_mapping if cache.write else None,
                             cache.pages, q_temp=self.q_temp)
        o = ops.paged_attention(qkv, cache.pages, cache.block_table, ctx, nh, nkv, hd, self.scale,
                                cache.window, cache.page_size, softcap=self.softcap,
                                slopes=self.slopes)
        if self.gated:
            prenorm.head_gate(o, qkv[:, self.g_off:self.g_off + nh], nh, hd)
        return self.out(o)


register_mixer("qknorm_attention", NormedGatedAttention)
