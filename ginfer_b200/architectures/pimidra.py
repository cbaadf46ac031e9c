"""Pimidra as a plan of parts.

A decoder whose layers differ: each has a state-space mixer in its dual form (``mamba2``), a
grouped-query attention with whole-projection q/k norms, partly rotated heads, a chunked mask and
values mixed with the first such layer's (``attention``), or gated linear attention (``gla``),
followed by a dense feed-forward (``relu(gate) * up``) or a mixture of experts (``silu(gate) *
up``, the softmax over the chosen logits as weights), or by none.  The norms follow the sums:
``x <- norm(alpha * x + sublayer(x))``.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

import math

from ..config.pimidra_config import PimidraConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, sequential_run

# Positions are exact in 32-bit floats up to here; nothing else bounds a sequence's length.
MAX_POSITIONS = 1 << 24

# ``alpha`` of the clamped gated activation below zero: the gate's sigmoid as a step, i.e. relu
RELU_GATE = -1.0


def _mixer(cfg: PimidraConfig, kind: str, m, value_mix=None) -> PartSpec:
    if kind == "mamba2":
        return PartSpec("state_space_dual", dict(
            hidden_size=cfg.width, num_heads=m["heads"], v_dim=m["vdim"], state_dim=m["state"],
            groups=m["groups"], conv_taps=m["conv"], norm_groups=m.get("norm_groups", 1),
            norm_eps=cfg.norm_eps, prefix="mix"))
    if kind == "gla":
        # the inner size of the decay's low-rank projection is the tensors' own; a configuration
        # may name it (``decay_rank``) so that random weights can be drawn
        return PartSpec("gated_linear_attention", dict(
            hidden_size=cfg.width, num_heads=m["heads"], key_dim=m["dim"], v_dim=m["vdim"],
            tau=m["tau"], norm_eps=cfg.norm_eps, decay_rank=m.get("decay_rank", -1),
            prefix="mix"))
    rot = m.get("rot")
    position = PartSpec("pair_rotary", dict(
        dims=rot["dims"] if rot else 0, base=rot["base"] if rot else 1.0, interleaved=False,
        linear_factor=(rot.get("scaling") or {}).get("factor", 1.0) if rot else 1.0))
    return PartSpec("widenorm_attention", dict(
        hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
        head_dim=m["dim"], v_dim=m["vdim"], scale=m["scale"], position=position,
        chunk=m["mask"]["size"] if m.get("mask") is not None else 0,
        qk_norm_eps=cfg.norm_eps, value_mix=value_mix, prefix="mix"))


def _feed_forward(cfg: PimidraConfig, mlp) -> PartSpec | None:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("clamped_glu", dict(hidden_size=cfg.width, intermediate_size=mlp["ff"],
                                            limit=math.inf, alpha=RELU_GATE, up_shift=0.0,
                                            prefix="mlp"))
    return PartSpec("routed_glu", dict(
        hidden_size=cfg.width, intermediate_size=mlp["expert"]["ff"], limit=math.inf, alpha=1.0,
        up_shift=0.0, num_experts=mlp["router"]["experts"], top_k=mlp["router"]["top"],
        renormalize=True, prefix="mlp"))


def pimidra_plan(cfg: PimidraConfig) -> ModelPlan:
    def norm(name):
        return PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.norm_eps, weight_name=name))
    layers, mixing = [], False
    for i, L in enumerate(cfg.layers):
        ff = _feed_forward(cfg, L.mlp)
        role = None
        if L.type == "attention" and L.mixer.get("v_mix"):
            # the first layer that mixes its values is the one whose values the others mix in
            role, mixing = ("mix" if mixing else "source"), True
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=_mixer(cfg, L.type, L.mixer, role), feed_forward=ff,
            mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2") if ff else None,
            block=PartSpec("postnorm", dict(alpha=cfg.postln_alpha))))
    return ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab, hidden_size=cfg.width,
                                         name="embed", scale=1.0)),
        layers=tuple(layers), run=sequential_run(len(layers)), final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, name="head")),
        eos_token_ids=tuple(cfg.eos_token_ids))


register_architecture("Pimidra", PimidraConfig, pimidra_plan, model_types=("pimidra",))
