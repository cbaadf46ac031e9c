"""Gated linear attention: a linear recurrence with one decay per head and key channel.

``q = W_q h * D^-1/2``, ``k = W_k h`` (``H`` heads of ``D``), ``v = W_v h`` (``H`` heads of
``Vd``).  Decay ``alpha = sigmoid(z)^(1/tau)`` with ``z = W_a2 (W_a1 h) + b_a2`` laid out heads x
``D``.  Per head ``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``.  Each head's
``o`` is RMS-normed over its ``Vd`` channels with one weight vector shared by the heads; the heads
side by side are multiplied by ``silu(W_g h)`` and projected by ``W_o``.

State per request (one fp32 row of a slot): ``S [H, D, Vd]``.  The decay's second product leaves
in 32-bit; its logarithm and exponential, the recurrence and the norm are fp32 arithmetic in both
paths.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import decay
from .base import Mixer, StateSpec, TensorSpec, register_mixer


class GatedLinearAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, v_dim: int, tau: float,
                 norm_eps: float = 1e-6, decay_rank: int = -1, prefix: str = "mix"):
        self.hidden_size, self.H = int(hidden_size), int(num_heads)
        self.D, self.Vd, self.tau = int(key_dim), int(v_dim), float(tau)
        if not (self.tau > 0):
            raise ValueError(f"tau must be > 0, got {tau}")
        if self.D > decay.MAX_KEY_SIZE:
            raise ValueError(f"a key size of {self.D} is over the recurrence kernel's "
                             f"{decay.MAX_KEY_SIZE}")
        self.eps, self.decay_rank = float(norm_eps), int(decay_rank)     # -1: the file's
        self.prefix = prefix + "." if prefix else ""

    def _n(self, name):
        return self.prefix + name

    def tensor_specs(self):
        W, HD, HV, r = self.hidden_size, self.H * self.D, self.H * self.Vd, self.decay_rank
        return [TensorSpec(self._n("q"), (HD, W)), TensorSpec(self._n("k"), (HD, W)),
                TensorSpec(self._n("v"), (HV, W)), TensorSpec(self._n("g"), (HV, W)),
                TensorSpec(self._n("o"), (W, HV)),
                TensorSpec(self._n("norm"), (self.Vd,), "norm32"),
                TensorSpec(self._n("a1"), (r, W)), TensorSpec(self._n("a2"), (HD, r)),
                TensorSpec(self._n("a2.b"), (HD,), "f32")]

    def load(self, tensors, dtype, device):
        t = {k: tensors[self._n(k)] for k in ("q", "k", "v", "g", "o", "norm", "a1", "a2", "a2.b")}
        r = t["a1"].shape[0]
        if t["a2"].shape[1] != r:
            raise ValueError(f"{self.prefix}a1 and a2 disagree on their inner size")
        rows = [t["q"], t["k"], t["v"], t["g"], t["a1"]]       # one product for all that reads h
        n = sum(x.shape[0] for x in rows)
        if -n % 8:
            rows.append(torch.zeros((-n % 8, self.hidden_size), dtype=rows[0].dtype, device=device))
        self.first = ops.Linear(torch.cat(rows, dim=0))
        HD, HV = self.H * self.D, self.H * self.Vd
        self.g_off = 2 * HD + HV
        self.a1_off, self.r = self.g_off + HV, r
        self.decay = ops.Linear(t["a2"], t["a2.b"].float(), out_dtype=torch.float32)
        self.out = ops.Linear(t["o"], None, out_dtype=torch.float32)
        self.norm_w = t["norm"].float().contiguous()

    def cache_spec(self):
        return StateSpec((self.H * self.D * self.Vd,), torch.float32)

    def forward(self, x, ctx, cache):
        H, D, Vd = self.H, self.D, self.Vd
        HD, HV = H * D, H * Vd
        p = self.first(x)                                   # [T, q | k | v | g | a1 (| pad)]
        z = self.decay(p[:, self.a1_off:self.a1_off + self.r].contiguous())      # fp32 [T, H D]
        f = decay.gla_prepare(p, z, HD, HV, D ** -0.5, self.tau)     # fp32 q | k | decays | v
        o = decay.recurrence(f[:, :HD], f[:, HD:2 * HD], f[:, 3 * HD:], f[:, 2 * HD:3 * HD],
                             cache.state, ctx, H, H, D, Vd)
        y = decay.gated_norm(o, p[:, self.g_off:self.g_off + HV], self.norm_w, Vd, False, self.eps,
                             ctx.dtype)
        return self.out(y)


register_mixer("gated_linear_attention", GatedLinearAttention)


class DecayLinearAttention(Mixer):
    """Linear attention with ONE fixed decay a head.  ``q = silu(W_q h)``, ``k = silu(W_k h)``
    (``H`` heads of ``D``), ``v = silu(W_v h)`` (``H`` heads of ``Vd``); per head ``S_t = a_n
    S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` with the constants ``decays[n]`` and no other scale.
    All heads' outputs side by side are RMS-normed TOGETHER with a weight of ``H Vd``, multiplied by
    ``sigmoid(W_g h)`` and projected by ``W_o``.

    State per request (one fp32 row of a slot): ``S [H, D, Vd]``, zero at the start.  One product
    gives q | k | v | g; the activations leave in 32-bit and the recurrence, the norm and the gate
    are fp32 arithmetic in both paths.  The recurrence is the one the other decaying mixers use
    (``ops.decay.recurrence`` with a decay a head)."""

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, v_dim: int, decays,
                 norm_eps: float = 1e-6, prefix: str = "mix"):
        self.hidden_size, self.H = int(hidden_size), int(num_heads)
        self.D, self.Vd = int(key_dim), int(v_dim)
        self.decays = [float(a) for a in decays]
        if len(self.decays) != self.H:
            raise ValueError(f"{len(self.decays)} decays for {self.H} heads")
        if self.D > decay.MAX_KEY_SIZE:
            raise ValueError(f"a key size of {self.D} is over the recurrence kernel's "
                             f"{decay.MAX_KEY_SIZE}")
        self.eps = float(norm_eps)
        self.prefix = prefix + "." if prefix else ""

    def _n(self, name):
        return self.prefix + name

    def tensor_specs(self):
        W, HD, HV = self.hidden_size, self.H * self.D, self.H * self.Vd
        return [TensorSpec(self._n("q"), (HD, W)), TensorSpec(self._n("k"), (HD, W)),
                TensorSpec(self._n("v"), (HV, W)), TensorSpec(self._n("g"), (HV, W)),
                TensorSpec(self._n("o"), (W, HV)), TensorSpec(self._n("norm"), (HV,), "norm32")]

    def load(self, tensors, dtype, device):
        rows = [tensors[self._n(k)] for k in ("q", "k", "v", "g")]
        n = sum(x.shape[0] for x in rows)
        if -n % 8:        # rows of the product stay 16-byte aligned in bfloat16
            rows.append(torch.zeros((-n % 8, self.hidden_size), dtype=rows[0].dtype, device=device))
        self.first = ops.Linear(torch.cat(rows, dim=0))
        self.out = ops.Linear(tensors[self._n("o")], None, out_dtype=torch.float32)
        self.norm_w = tensors[self._n("norm")].float().contiguous()
        self.decay_row = torch.tensor(self.decays, dtype=torch.float32, device=device)[None, :]

    def cache_spec(self):
        return StateSpec((self.H * self.D * self.Vd,), torch.float32)

    def forward(self, x, ctx, cache):
        H, D, Vd = self.H, self.D, self.Vd
        HD, HV = H * D, H * Vd
        p = self.first(x)                                   # [T, q | k | v | g (| pad)]
        f = decay.silu_f32(p, 2 * HD + HV)                  # fp32 q | k | v through SiLU
        g = self.decay_row.expand(p.shape[0], H)            # every token's decays: the constants
        o = decay.recurrence(f[:, :HD], f[:, HD:2 * HD], f[:, 2 * HD:], g, cache.state, ctx,
                             H, H, D, Vd)
        y = decay.gated_norm(o, p[:, 2 * HD + HV:2 * HD + 2 * HV], self.norm_w, HV, False,
                             self.eps, ctx.dtype, sigmoid_gate=True)
        return self.out(y)


register_mixer("decay_linear_attention", DecayLinearAttention)
