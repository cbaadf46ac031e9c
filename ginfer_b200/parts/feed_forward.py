"""Feed-forward parts.

SwiGLU as the reference computes it (``ginfer/core/layer/transformer/feedforward.cc:22-25``,
``ginfer/core/op/kernels/cuda/swiglu_kernel.cu:24-27``): ``g = y W_g^T``, ``u = y W_u^T``,
``z = (g * 1/(1+exp(-g))) * u`` in fp32, ``m = z W_d^T``; no biases.  Gate and up weights are
joined at load into one matrix so that one product reads ``y`` once.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, Summed, TensorSpec, register_feed_forward


class SwiGLU(FeedForward):
    takes_lazy_norm = True
    adds_residual = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "mlp",
                 gate_name: str = "gate_proj", up_name: str = "up_proj",
                 down_name: str = "down_proj"):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        p = prefix + "." if prefix else ""
        self.gate_key = f"{p}{gate_name}.weight"
        self.up_key = f"{p}{up_name}.weight"
        self.down_key = f"{p}{down_name}.weight"
        self.gate_up = None
        self.down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return [TensorSpec(self.gate_key, (i, h)), TensorSpec(self.up_key, (i, h)),
                TensorSpec(self.down_key, (h, i))]

    def load(self, tensors, dtype, device):
        self.gate_up = ops.GatedLinear(tensors[self.gate_key], tensors[self.up_key])
        self.down = ops.Linear(tensors[self.down_key])

    def forward(self, x, ctx, residual=None, then=None):
        z = self.gate_up(x)            # silu(gate) * up, [T, intermediate]
        if residual is not None:
            s = ops.add_to(self.down, z, residual,
                           then.fold_weight() if then is not None else None)
            if s is not None:
                return Summed(*s)
        return self.down(z)


register_feed_forward("swiglu", SwiGLU)


class ClampedGLU(FeedForward):
    """``g = min(x W_g^T, limit)``, ``u = clamp(x W_u^T, -limit, limit)``,
    ``z = g * sigmoid(alpha g) * (u + up_shift)``, ``m = z W_d^T``; no biases.  The defaults
    (``alpha`` 1.702: the sigmoid form of GELU; ``up_shift`` 1) are those of the designs that use
    it so far.  The output leaves in fp32 for the norm that follows it."""

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float,
                 alpha: float = 1.702, up_shift: float = 1.0, prefix: str = "mlp",
                 gate_name: str = "gate", up_name: str = "up", down_name: str = "down"):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.alpha, self.up_shift = float(limit), float(alpha), float(up_shift)
        p = prefix + "." if prefix else ""
        self.gate_key, self.up_key, self.down_key = p + gate_name, p + up_name, p + down_name

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return [TensorSpec(self.gate_key, (i, h)), TensorSpec(self.up_key, (i, h)),
                TensorSpec(self.down_key, (h, i))]

    def load(self, tensors, dtype, device):
        self.gate_up = ops.GatedLinear(tensors[self.gate_key], tensors[self.up_key],
                                       clamped=(self.limit, self.alpha, self.up_shift))
        self.down = ops.Linear(tensors[self.down_key], None, out_dtype=torch.float32)

    def forward(self, x, ctx):
        return self.down(self.gate_up(x))


register_feed_forward("clamped_glu", ClampedGLU)


class DenseActivationMLP(FeedForward):
    """Two matrices with an activation between them: ``W_down act(W_up x + b_up) + b_down`` with
    ``act = relu^2`` (the only one so far); biases optional.  The output leaves in fp32 for the
    norm that follows it."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu2",
                 bias: bool = True, prefix: str = "mlp", up_name: str = "up",
                 down_name: str = "down"):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        if activation != "relu2":
            raise ValueError(f"activation {activation!r}: only 'relu2' is there")
        self.activation, self.bias = activation, bool(bias)
        p = prefix + "." if prefix else ""
        self.up_key, self.down_key = p + up_name, p + down_name

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        out = [TensorSpec(self.up_key, (i, h)), TensorSpec(self.down_key, (h, i))]
        if self.bias:
            out += [TensorSpec(self.up_key + ".b", (i,), "bias"),
                    TensorSpec(self.down_key + ".b", (h,), "bias")]
        return out

    def load(self, tensors, dtype, device):
        b = (lambda k: tensors[k + ".b"].float().contiguous()) if self.bias else (lambda k: None)
        self.up = ops.Linear(tensors[self.up_key], b(self.up_key), activation=self.activation)
        self.down = ops.Linear(tensors[self.down_key], b(self.down_key), out_dtype=torch.float32)

    can_defer_bias = True

    def forward(self, x, ctx, defer_bias: bool = False):
        """``defer_bias``: returns ``(y, b)`` whose sum is the result, ``b`` the down-projection's
        bias where the caller's next kernel can add it for nothing (else ``None``)."""
        if defer_bias:
            return self.down.deferring_bias(self.up(x))
        return self.down(self.up(x))


register_feed_forward("dense_mlp", DenseActivationMLP)
