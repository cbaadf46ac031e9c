"""RMS normalisation, with the preceding residual addition fused in.

Formula as the reference computes it (``ginfer/core/op/kernels/cuda/rmsnorm_kernel.cu:27-66``):
``ss = sum_j x_j^2``, ``rms = sqrtf(ss / H + eps)``, ``out_j = x_j * gamma_j / rms``, all in fp32
with one cast at the end.  The reference adds residuals in a separate kernel
(``ginfer/core/layer/transformer/encoder.cc:35,39``); here the addition happens in the same
kernel, in fp32, and the sum is written once in the activation dtype.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import LazyNorm, Norm, TensorSpec, register_norm


class RMSNorm(Norm):
    """``weight_offset``: the stored weight is an offset from this value (1.0 for weights stored
    around zero: the norm multiplies by ``1 + w``); the sum is formed once, in 32-bit, at load."""

    def __init__(self, size: int, eps: float, weight_name: str = "weight",
                 weight_offset: float = 0.0):
        self.size = int(size)
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight_offset = float(weight_offset)
        self.weight: torch.Tensor | None = None
        self._w32: torch.Tensor | None = None      # the weight in 32-bit, made when first needed

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.size,),
                           "f32" if self.weight_offset else "norm")]

    def load(self, tensors, dtype, device):
        self.weight = tensors[self.weight_name]
        self._w32 = None
        if self.weight_offset:
            self.weight = (self.weight.float() + self.weight_offset).contiguous()

    def weight32(self) -> torch.Tensor:
        """The weight in 32-bit (made once), for kernels that apply this norm inside a pass of
        their own."""
        if self._w32 is None:
            self._w32 = self.weight.float().contiguous()
        return self._w32

    def add_output(self, x, y, act_dtype, want_act=True):
        """For blocks whose norms sit on the sublayers' outputs: ``x' = x + norm(y)`` on the fp32
        stream ``x``; returns ``(x', x' in act_dtype or None)``."""
        w = self.weight if self.weight.dtype == torch.float32 else self.weight.float()
        return ops.outnorm_add(x, y, w, self.eps, act_dtype, want_act)

    def post(self, x, y, alpha, act_dtype, want_act=True, pairs=None):
        """For blocks whose norms sit behind the sums: ``x' = norm(alpha * x + y)`` on the fp32
        stream ``x``; returns ``(x', x' in act_dtype or None)``.  ``pairs``: see
        :func:`ginfer_b200.ops.postnorm`."""
        if self._w32 is None:
            self._w32 = self.weight.float().contiguous()
        return ops.postnorm(x, y, alpha, self._w32, self.eps, act_dtype, want_act, pairs)

    def forward(self, x, delta=None, rows=None, want_sum=True, out_dtype=None):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, rows=rows, want_sum=want_sum,
                               out_dtype=out_dtype)

    def lazy(self, summed, dtype):
        return LazyNorm(summed, self.weight, self.eps, dtype)

    def fold_weight(self):
        return self.weight if not self.weight_offset else None


    def fused(self):
        if self.weight_offset or self.weight.dtype != torch.float32:
            return None
        return ops.prenorm.NORM_RMS, self.weight, None, self.eps


register_norm("rmsnorm", RMSNorm)


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w + b`` with the variance as the mean of the squared
    deviations; mean, variance and the result in 32-bit, weight and bias kept in 32-bit.  The
    input is the fp32 residual stream; a ``delta`` still to be added is added in the same pass."""

    def __init__(self, size: int, eps: float, weight_name: str = "weight",
                 bias_name: str | None = "bias"):
        self.size, self.eps = int(size), float(eps)
        self.weight_name, self.bias_name = weight_name, bias_name
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def tensor_specs(self):
        out = [TensorSpec(self.weight_name, (self.size,), "norm32")]
        if self.bias_name:
            out.append(TensorSpec(self.bias_name, (self.size,), "f32"))
        return out

    def load(self, tensors, dtype, device):
        self.weight = tensors[self.weight_name].float().contiguous()
        self.bias = tensors[self.bias_name].float().contiguous() if self.bias_name else None

    def fused(self):
        return ops.prenorm.NORM_LAYER, self.weight, self.bias, self.eps

    def forward(self, x, delta=None, rows=None, want_sum=True, out_dtype=None):
        act = out_dtype or (x.dtype if delta is None else delta.dtype)
        if x.dtype != torch.float32:
            x = x.float()
        plain = delta is None and rows is None      # then the sum is x itself
        s, _, n = ops.prenorm.stream_update(
            x, act, y=delta, rows=rows, want_out=want_sum and not plain,
            norm=ops.prenorm.NORM_LAYER, norm_weight=self.weight, norm_bias=self.bias,
            norm_eps=self.eps)
        return (x if plain and want_sum else s), n


register_norm("layernorm", LayerNorm)
