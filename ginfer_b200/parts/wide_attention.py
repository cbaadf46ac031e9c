"""Grouped-query attention whose queries and keys are normed over the whole projection.

``q = W_q h + b_q``, ``k = W_k h + b_k``, ``v = W_v h + b_v`` (``H`` query heads and ``G`` key/value
heads; keys of ``D`` channels, values of ``Vd``).  ``q`` is RMS-normed over all its ``H D``
channels at once with a weight of that size (``k`` likewise), before it is split into heads; then
every head's first ``dims`` channels are rotated by the position encoding (pairs ``(i, i +
dims/2)``).  ``score = q.k * scale`` over the keys the mask lets the query see (everything before
it, a sliding window, or the query's own chunk of ``chunk`` positions counted from position 0 of
the sequence), softmax; query head ``n`` reads kv head ``n // (H / G)``.

**Value mixing** (``value_mix``): the layer that is the ``"source"`` (the first layer of a model
that mixes) leaves its values of the step's tokens in ``ctx.extras`` (under ``value_mix_key``);
every layer with ``"mix"`` replaces its own by ``(1 - lambda) v + lambda v_first`` with its scalar
tensor ``vmix``, and caches the mixed values.  (The source owns a ``vmix`` too and does not use
it.)  Which layer is which is the plan's to say: a step's context may be run more than once.

One product over the joined matrices gives q, k and v; one kernel norms, rotates, mixes and writes
the cache; the attention kernels of the plain grouped-query mixer run over that cache where keys
and values have one width.  Norms, angles, the mix, scores and softmax are fp32 arithmetic.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, PagedKVSpec, TensorSpec, make_part, register_mixer
from .plan import PartSpec


class WideNormAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_dim: int, scale: float, position: PartSpec, window: int = 0, chunk: int = 0,
                 qk_norm: bool = True, qk_norm_eps: float = 1e-6, bias: bool = True,
                 value_mix: str | None = None, value_mix_key: str = "value_mix",
                 prefix: str = "mix"):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        if window and chunk:
            raise ValueError("a mask is a sliding window or chunks, not both")
        self.hidden_size = int(hidden_size)
        self.nh, self.nkv = int(num_heads), int(num_kv_heads)
        self.hd, self.vd = int(head_dim), int(v_dim)
        self.scale, self.window, self.chunk = float(scale), int(window), int(chunk)
        self.qk_norm, self.eps, self.bias = bool(qk_norm), float(qk_norm_eps), bool(bias)
        if value_mix not in (None, "source", "mix"):
            raise ValueError(f"value_mix is None, 'source' or 'mix', not {value_mix!r}")
        self.value_mix, self.mix_key = value_mix, value_mix_key
        self.prefix = prefix + "." if prefix else ""
        self.position = make_part("position", position)
        if not hasattr(self.position, "frequencies") or self.position.interleaved:
            raise ValueError("this mixer rotates the pairs (i, i + dims/2) by frequencies; its "
                             "position encoding must be 'pair_rotary' with interleaved=False")
        if self.position.dims > self.hd:
            raise ValueError(f"{self.position.dims} rotated channels do not fit a head of {self.hd}")

    def _n(self, name):
        return self.prefix + name

    def tensor_specs(self):
        W, nh, nkv, hd, vd = self.hidden_size, self.nh, self.nkv, self.hd, self.vd
        out = [TensorSpec(self._n("q"), (nh * hd, W)), TensorSpec(self._n("k"), (nkv * hd, W)),
               TensorSpec(self._n("v"), (nkv * vd, W))]
        if self.bias:
            out += [TensorSpec(self._n("q.b"), (nh * hd,), "bias"),
                    TensorSpec(self._n("k.b"), (nkv * hd,), "bias"),
                    TensorSpec(self._n("v.b"), (nkv * vd,), "bias")]
        if self.qk_norm:
            out += [TensorSpec(self._n("q.norm"), (nh * hd,), "norm32"),
                    TensorSpec(self._n("k.norm"), (nkv * hd,), "norm32")]
        if self.value_mix:
            out.append(TensorSpec(self._n("vmix"), (), "f32"))
        out.append(TensorSpec(self._n("o"), (W, nh * vd)))
        return out + self.position.tensor_specs()

    def load(self, tensors, dtype, device):
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        parts = [tensors[self._n(p)] for p in "qkv"]
        self.k_off, self.v_off = nh * hd, (nh + nkv) * hd
        cols = self.v_off + nkv * vd
        b = None
        if self.bias:
            b = torch.cat([tensors[self._n(p + ".b")].float() for p in "qkv"])
        if cols % 8:      # rows of the product stay 16-byte aligned in bfloat16
            pad = 8 - cols % 8
            parts.append(torch.zeros((pad, self.hidden_size), dtype=parts[0].dtype,
                                     device=parts[0].device))
            if b is not None:
                b = torch.cat([b, torch.zeros(pad, dtype=b.dtype, device=b.device)])
        self.qkv = ops.Linear(torch.cat(parts, dim=0), b)
        self.q_w = tensors[self._n("q.norm")].float().contiguous() if self.qk_norm else None
        self.k_w = tensors[self._n("k.norm")].float().contiguous() if self.qk_norm else None
        self.mix = tensors[self._n("vmix")].float().reshape(1).contiguous() \
            if self.value_mix else None
        self.out = ops.Linear(tensors[self._n("o")], None, out_dtype=torch.float32)
        self.position.load(tensors, dtype, device)

    def cache_spec(self):
        if self.vd == self.hd:
            return PagedKVSpec(self.nkv, self.hd, self.window, chunk=self.chunk)
        return PagedKVSpec(self.nkv, self.hd, self.window, chunk=self.chunk,
                           planes=((self.nkv, self.hd), (self.nkv, self.vd)))

    def forward(self, x, ctx, cache):
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        qkv = self.qkv(x)
        v_first = None
        if self.value_mix == "source":        # its values are what the later layers mix in
            ctx.extras[self.mix_key] = qkv[:, self.v_off:self.v_off + nkv * vd]
        elif self.value_mix == "mix":
            v_first = ctx.extras[self.mix_key]
            if v_first.shape != (qkv.shape[0], nkv * vd):
                raise ValueError("layers that mix their values must agree on the values' size")
        ops.qk_wide_prepare(qkv, nh, nkv, hd, vd, self.k_off, self.v_off, self.q_w, self.k_w,
                            self.eps, self.position.frequencies(), self.position.dims,
                            ctx.positions, cache.slot_mapping if cache.write else None,
                            cache.pages[0], cache.pages[1], v_first, self.mix)
        o = ops.paged_attention(qkv, cache.pages, cache.block_table, ctx, nh, nkv, hd, self.scale,
                                ops.mask_span(cache.window, cache.chunk), cache.page_size, vd=vd)
        return self.out(o)


register_mixer("widenorm_attention", WideNormAttention)
