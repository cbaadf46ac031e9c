"""Routed feed-forward (mixture of experts).

Router logits ``z = h W_r^T`` in 32-bit (float32 path: from the fp32 stream; bfloat16 path: from
the bfloat16 rounding of ``h`` and the bfloat16 router matrix, whose products are exact in 32-bit
and are added up in 32-bit by the tensor cores), scores ``softmax(z)`` over ALL experts, the ``top_k`` largest chosen; a token's output is the sum of the chosen experts' outputs
weighted by their scores (as they are, or renormalised over the chosen ones with
``renormalize``: the softmax over the chosen logits alone).  An expert is a clamped GLU (see
:class:`ClampedGLU`; an infinite limit, ``alpha`` 1 and no shift make it ``silu(g) * u``) without
biases, stored as ``<prefix>.e<i>.gate|up|down``.

Nothing returns to the host inside a step: the pairs (token, expert) are sorted by expert on the
device and two grouped products walk over them.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import moe
from .base import FeedForward, PairSum, TensorSpec, register_feed_forward


class RoutedGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, num_experts: int,
                 top_k: int, renormalize: bool = False, alpha: float = 1.702,
                 up_shift: float = 1.0, prefix: str = "mlp"):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.E, self.top = int(num_experts), int(top_k)
        if not (0 < self.top <= self.E):
            raise ValueError(f"{self.top} of {self.E} experts cannot be chosen")
        self.limit, self.alpha, self.up_shift = float(limit), float(alpha), float(up_shift)
        self.renormalize = bool(renormalize)
        self.prefix = prefix + "." if prefix else ""

    def tensor_specs(self):
        h, f = self.hidden_size, self.intermediate_size
        out = []
        for e in range(self.E):
            p = f"{self.prefix}e{e}."
            out += [TensorSpec(p + "gate", (f, h)), TensorSpec(p + "up", (f, h)),
                    TensorSpec(p + "down", (h, f))]
        out.append(TensorSpec(self.prefix + "router", (self.E, h)))
        return out

    def load(self, tensors, dtype, device):
        f, h = self.intermediate_size, self.hidden_size
        gu = [torch.stack([tensors[f"{self.prefix}e{e}.gate"], tensors[f"{self.prefix}e{e}.up"]],
                          dim=1).reshape(2 * f, h) for e in range(self.E)]
        self.w_gate_up = torch.stack(gu).contiguous()                       # [E, 2 F, H]
        self.w_down = torch.stack([tensors[f"{self.prefix}e{e}.down"]
                                   for e in range(self.E)]).contiguous()    # [E, H, F]
        self.router = ops.Linear(tensors[self.prefix + "router"], None, out_dtype=torch.float32)
        self.act = torch.tensor([self.limit, self.alpha, self.up_shift], dtype=torch.float32,
                                device=device)

    can_defer_sum = True

    def forward(self, x, ctx, defer_sum: bool = False):
        T = x.shape[0]
        idx, wgt = moe.route(self.router(x), self.top, self.renormalize)
        plan = moe.Plan(idx, self.E, moe.kernel_for(
            x, T * self.top, (self.hidden_size, self.intermediate_size),
            (self.intermediate_size, self.hidden_size)))
        y = moe.grouped_glu(x, self.w_gate_up, plan, self.limit, self.alpha, self.up_shift,
                            act=self.act)
        rows = moe.grouped_down(y, self.w_down, plan)
        if defer_sum:
            return PairSum(rows, plan.pos_of_pair, wgt, self.top,
                           lambda: moe.combine(rows, plan, wgt, T))
        return moe.combine(rows, plan, wgt, T)


register_feed_forward("routed_glu", RoutedGLU)


class RoutedExperts(FeedForward):
    """Experts of two matrices, ``W_down act(W_up h)`` with ``act = relu^2``, stored as
    ``<prefix>.e<i>.up|down``; no biases.  Router scores ``sigmoid(W_r h)`` (or the softmax over all
    experts) in 32-bit, the ``top_k`` largest chosen (lowest index among equals), the scores as
    weights, as they are or renormalised over the chosen ones.  ``weight_on="input"``: the weight
    multiplies what the expert reads, ``sum_e expert_e(w_e h)``; the first grouped product scales
    its accumulator by ``w_e`` before the activation, which is that product.  ``"output"``:
    ``sum_e w_e expert_e(h)``."""

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top_k: int,
                 score: str = "sigmoid", renormalize: bool = False, weight_on: str = "input",
                 prefix: str = "mlp"):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.E, self.top = int(num_experts), int(top_k)
        if not (0 < self.top <= self.E):
            raise ValueError(f"{self.top} of {self.E} experts cannot be chosen")
        if score not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError(f"score {score!r} / weight_on {weight_on!r} are not known")
        self.score, self.renormalize, self.weight_on = score, bool(renormalize), weight_on
        self.prefix = prefix + "." if prefix else ""

    def tensor_specs(self):
        h, f = self.hidden_size, self.intermediate_size
        out = []
        for e in range(self.E):
            p = f"{self.prefix}e{e}."
            out += [TensorSpec(p + "up", (f, h)), TensorSpec(p + "down", (h, f))]
        out.append(TensorSpec(self.prefix + "router", (self.E, h)))
        return out

    def load(self, tensors, dtype, device):
        p = self.prefix
        self.w_up = torch.stack([tensors[f"{p}e{e}.up"] for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[f"{p}e{e}.down"] for e in range(self.E)]).contiguous()
        self.router = ops.Linear(tensors[p + "router"], None, out_dtype=torch.float32)

    can_defer_sum = True

    def forward(self, x, ctx, defer_sum: bool = False):
        T = x.shape[0]
        idx, wgt = moe.route(self.router(x), self.top, self.renormalize, self.score)
        plan = moe.Plan(idx, self.E, moe.kernel_for(
            x, T * self.top, (self.hidden_size, self.intermediate_size),
            (self.intermediate_size, self.hidden_size)))
        on_input = self.weight_on == "input"
        y = moe.grouped_relu2(x, self.w_up, plan, wgt if on_input else None)
        rows, w = moe.grouped_down(y, self.w_down, plan), None if on_input else wgt
        if defer_sum:
            return PairSum(rows, plan.pos_of_pair, w, self.top,
                           lambda: moe.combine(rows, plan, w, T))
        return moe.combine(rows, plan, w, T)


register_feed_forward("routed_experts", RoutedExperts)
