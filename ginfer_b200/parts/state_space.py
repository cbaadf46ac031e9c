"""State-space mixer in its dual form (a linear recurrence with one decay per head).

``W_in h`` is laid out ``z [inner] | x [inner] | B [G N] | C [G N] | dt [H]`` with ``inner = H *
Vd``.  ``x``, ``B`` and ``C`` together pass a causal convolution over time per channel (``taps``
taps, the last one the current token's, zeros before the sequence's start) with a bias, then SiLU.
``dt = softplus(dt + dt_bias)``.  Per head ``n`` (reading group ``n // (H / G)`` of ``B`` and
``C``): ``S_t = exp(-exp(A_log_n) dt) S_(t-1) + dt B_t x_t^T`` (``S`` is ``N x Vd``), ``y_t = S_t^T
C_t + D_n x_t``.  ``y`` (heads side by side) times ``silu(z)`` is RMS-normed in ``norm_groups``
equal parts, times the norm weight, and projected by ``W_o``.

State per request (one fp32 row of a slot): ``S [H, N, Vd]``, then the convolution's last
``taps - 1`` inputs ``[taps - 1, inner + 2 G N]``.  The first product leaves in 32-bit (its step
sizes feed exponentials); convolution, step sizes, decays, recurrence and norm are fp32 arithmetic
in both paths.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import decay
from .base import Mixer, StateSpec, TensorSpec, register_mixer


class StateSpaceDual(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, v_dim: int, state_dim: int, groups: int,
                 conv_taps: int, norm_groups: int = 1, norm_eps: float = 1e-6,
                 prefix: str = "mix"):
        self.hidden_size, self.H, self.Vd = int(hidden_size), int(num_heads), int(v_dim)
        self.N, self.G, self.taps = int(state_dim), int(groups), int(conv_taps)
        self.norm_groups, self.eps = int(norm_groups), float(norm_eps)
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} groups")
        self.inner = self.H * self.Vd
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} channels cannot be normed in {self.norm_groups} "
                             "equal parts")
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        if self.N > decay.MAX_KEY_SIZE:
            raise ValueError(f"a state size of {self.N} is over the recurrence kernel's "
                             f"{decay.MAX_KEY_SIZE}")
        self.channels = self.inner + 2 * self.G * self.N
        self.state_floats = self.H * self.N * self.Vd
        self.prefix = prefix + "." if prefix else ""

    def _n(self, name):
        return self.prefix + name

    def tensor_specs(self):
        W, H = self.hidden_size, self.H
        return [TensorSpec(self._n("in"), (2 * self.inner + 2 * self.G * self.N + H, W)),
                TensorSpec(self._n("conv"), (self.channels, self.taps), "f32"),
                TensorSpec(self._n("conv.b"), (self.channels,), "f32"),
                TensorSpec(self._n("dt_bias"), (H,), "f32"),
                TensorSpec(self._n("A_log"), (H,), "f32"),
                TensorSpec(self._n("D"), (H,), "f32"),
                TensorSpec(self._n("norm"), (self.inner,), "norm32"),
                TensorSpec(self._n("o"), (W, self.inner))]

    def load(self, tensors, dtype, device):
        w = tensors[self._n("in")]
        pad = -w.shape[0] % 8               # rows of the product stay 16-byte aligned
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)])
        self.first = ops.Linear(w, None, out_dtype=torch.float32)
        self.out = ops.Linear(tensors[self._n("o")], None, out_dtype=torch.float32)
        self.conv_w = tensors[self._n("conv")].float().contiguous()
        self.conv_b = tensors[self._n("conv.b")].float().contiguous()
        self.dt_bias = tensors[self._n("dt_bias")].float().contiguous()
        self.A_log = tensors[self._n("A_log")].float().contiguous()
        self.D = tensors[self._n("D")].float().contiguous()
        self.norm_w = tensors[self._n("norm")].float().contiguous()

    def cache_spec(self):
        return StateSpec((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, ctx, cache):
        H, G, N, Vd, inner = self.H, self.G, self.N, self.Vd, self.inner
        state = cache.state
        p = self.first(x)                               # fp32 [T, z | x | B | C | dt (| pad)]
        xbc, rates = decay.ssd_prepare(p, inner, inner + self.channels, self.conv_w, self.conv_b,
                                       self.dt_bias, self.A_log, state, ctx, H, self.channels,
                                       self.taps, self.state_floats)
        gn = G * N
        y = decay.recurrence(xbc[:, inner + gn:], xbc[:, inner:inner + gn], xbc[:, :inner],
                             rates[:, :H], state, ctx, H, G, N, Vd, k_scale=rates[:, H:],
                             skip=self.D)
        y = decay.gated_norm(y, p[:, :inner], self.norm_w, inner // self.norm_groups, True,
                             self.eps, ctx.dtype)
        return self.out(y)


register_mixer("state_space_dual", StateSpaceDual)
