"""Token embedding and output head.

Embedding: ``h[t, :] = E[ids[t], :]`` (``ginfer/core/op/kernels/cuda/embedding_kernel.cu:16-24``).
Head: the rows that want logits are selected first and only those are projected
(``ginfer/core/layer/transformer/lmhead.cc:15-27``); a tied head shares the embedding matrix
(``ginfer/model/qwen2.cc:42-46``).  Logits leave in fp32.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, TensorSpec, register_part


class TokenEmbedding(Embedding):
    """``scale``: the rows are multiplied by it and leave as the fp32 residual stream (their
    rounding to the activation dtype is left in ``ctx.extras["act_copy"]`` for the first block)."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "model.embed_tokens.weight",
                 scale: float | None = None):
        self.vocab_size, self.hidden_size, self.name = int(vocab_size), int(hidden_size), name
        self.scale = None if scale is None else float(scale)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), "embedding")]

    def load(self, tensors, dtype, device):
        self.weight = tensors[self.name]

    def forward(self, token_ids, ctx):
        if self.scale is None:
            return ops.embedding(token_ids, self.weight)
        x, act = ops.embedding_scaled(token_ids, self.weight, self.scale,
                                      want_act=self.weight.dtype != torch.float32)
        ctx.extras["act_copy"] = (x, x if act is None else act)
        return x


class PositionedEmbedding(Embedding):
    """``x[t] = E[token] + P[position]`` with a learned table ``P [max_positions, hidden]``, not
    scaled; the fp32 residual stream.  ``keep_states`` > 0: the model averages over its depth, and
    the stream's states (this output, then one a layer) live in one buffer ``[keep_states, T,
    hidden]`` that is made here and travels in ``ctx.extras["depth_history"]``; the output is its
    first state."""

    def __init__(self, vocab_size: int, hidden_size: int, max_positions: int,
                 name: str = "embed", position_name: str = "pos", keep_states: int = 0):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.max_positions, self.keep_states = int(max_positions), int(keep_states)
        self.name, self.position_name = name, position_name
        self.weight: torch.Tensor | None = None
        self.table: torch.Tensor | None = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), "embedding"),
                TensorSpec(self.position_name, (self.max_positions, self.hidden_size),
                           "embedding")]

    def load(self, tensors, dtype, device):
        self.weight = tensors[self.name]
        self.table = tensors[self.position_name]

    def forward(self, token_ids, ctx):
        out = None
        if self.keep_states:
            hist = torch.empty((self.keep_states, token_ids.numel(), self.hidden_size),
                               dtype=torch.float32, device=self.weight.device)
            ctx.extras["depth_history"] = hist
            out = hist[0]
        x, _ = ops.depth.embedding_positions(token_ids, ctx.positions, self.weight, self.table,
                                             out=out)
        return x


class LinearHead(Head):
    """``tied_to`` names the tensor of another part (the embedding) to share; otherwise the head
    has a matrix ``name`` of its own.  ``softcap``: the logits pass ``cap * tanh(logits / cap)``
    (fp32)."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "lm_head.weight",
                 tied_to: str | None = None, softcap: float | None = None):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.name, self.tied_to = name, tied_to
        self.softcap = float(softcap) if softcap else None    # logits <- cap * tanh(logits / cap)
        self.proj = None

    def tensor_specs(self):
        if self.tied_to:
            return []
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), "matrix")]

    def load(self, tensors, dtype, device):
        self.proj = ops.Linear(tensors[self.tied_to or self.name], None, out_dtype=torch.float32)

    def forward(self, x, ctx):
        logits = self.proj(x)
        if self.softcap is not None:
            ops.activation_(logits, "softcap", self.softcap)
        return logits


register_part("embedding", "token", TokenEmbedding)
register_part("embedding", "token_positions", PositionedEmbedding)
register_part("head", "linear", LinearHead)
