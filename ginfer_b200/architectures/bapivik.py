"""Bapivik as a plan of parts.

A decoder on a 32-bit residual stream whose layers differ: each has linear attention with a fixed
decay a head (``lightning``), latent attention without positions whose queries pass a latent of
their own and whose heads are gated, possibly over ANOTHER layer's cached latent vectors
(``latent_attention``), or grouped-query attention whose values are its keys, with normed heads, a
query temperature, a soft cap, a distance bias and a sliding window (``attention``), followed by a
dense relu^2 feed-forward with biases or by none.  Every sublayer has a norm in front and a norm
behind; every layer ends with a weighted average over the embedding output and all layers' results
so far.  Positions come from a learned table added to the token embedding; the head is the
embedding matrix, with a soft cap on the logits.

Tensor names: ``embed``, ``pos``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.dwa``, ``final.norm``.
"""
from __future__ import annotations

from ..config.bapivik_config import BapivikConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, RunEntry

# The distance bias of the attention mixer: head n of H takes 2^(-SLOPE_BASE (n + 1) / H) a position.
SLOPE_BASE = 8.0


def _mixer(cfg: BapivikConfig, kind: str, m) -> PartSpec:
    if kind == "lightning":
        return PartSpec("decay_linear_attention", dict(
            hidden_size=cfg.width, num_heads=m["heads"], key_dim=m["dim"], v_dim=m["vdim"],
            decays=tuple(float(a) for a in m["decay"]), norm_eps=cfg.norm_eps, prefix="mix"))
    if kind == "latent_attention":
        return PartSpec("latent_attention", dict(
            hidden_size=cfg.width, num_heads=m["heads"], nope_dim=m["dim"], rope_dim=0,
            v_dim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"], latent_eps=cfg.norm_eps,
            q_rank=m["q_rank"], head_gate=True, own_latent=m.get("kv_from") is None,
            prefix="mix"))
    qt = m.get("q_temp")
    return PartSpec("qknorm_attention", dict(
        hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
        head_dim=m["dim"], scale=m["scale"], position=None,
        window=m["mask"]["size"] if m.get("mask") is not None else 0,
        qk_norm_eps=cfg.norm_eps, value_projection=False, head_gate=False,
        q_temp=(qt["coef"], qt["every"]) if qt else None, softcap=m.get("softcap"),
        distance_slope_base=SLOPE_BASE, prefix="mix"))


def bapivik_plan(cfg: BapivikConfig) -> ModelPlan:
    def norm(name):
        return PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.norm_eps, weight_name=name))
    layers, run = [], []
    for i, L in enumerate(cfg.layers):
        ff = None
        if L.mlp is not None:
            ff = PartSpec("dense_mlp", dict(hidden_size=cfg.width, intermediate_size=L.mlp["ff"],
                                            activation="relu2", bias=True, prefix="mlp"))
        layers.append(LayerSpec(
            prefix=f"l{i}", mixer=_mixer(cfg, L.type, L.mixer), feed_forward=ff,
            mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2") if ff else None,
            block=PartSpec("sandwich", dict(
                mixer_out_norm=norm("norm1b"),
                feed_forward_out_norm=norm("norm2b") if ff else None,
                depth_states=i + 2, depth_name="dwa"))))
        src = L.mixer.get("kv_from") if L.type == "latent_attention" else None
        # a layer without latent vectors of its own reads the cache of the layer it names
        run.append(RunEntry(layer=i, cache=i) if src is None
                   else RunEntry(layer=i, cache=src, write_cache=False))
    return ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_positions", dict(
            vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=cfg.max_positions,
            name="embed", position_name="pos", keep_states=len(layers) + 1)),
        layers=tuple(layers), run=tuple(run), final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=cfg.width,
                                     tied_to="embed", softcap=cfg.logit_softcap)),
        eos_token_ids=tuple(cfg.eos_token_ids))


register_architecture("Bapivik", BapivikConfig, bapivik_plan, model_types=("bapivik",))
