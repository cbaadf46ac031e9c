"""Typed configuration of the Pimidra design, read from its own ``config.json`` keys.

A Pimidra folder names its design under ``architecture`` and describes every layer on its own:
``layers[i] = {"type": "mamba2" | "attention" | "gla", "mixer": its sizes and constants, "mlp":
feed-forward or null}``.  Beside the layers: ``width``, ``vocab``, ``norm.eps`` and
``postln_alpha`` (the factor on the stream inside the sums that the norms follow).  Every size and
constant of a model comes from this object.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_config import ConfigError
from .vilepel_config import _eos, _need, _plain, _positive_int

MIXER_KEYS = {
    "mamba2": ("heads", "vdim", "state", "groups", "conv"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "gla": ("heads", "dim", "vdim", "tau"),
}


@dataclass(frozen=True)
class PimidraLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": _plain(self.mixer), "mlp": _plain(self.mlp)}


@dataclass(frozen=True)
class PimidraConfig:
    width: int
    vocab: int
    norm_eps: float
    postln_alpha: float
    layers: tuple[PimidraLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "PimidraConfig":
        width = _positive_int(_need(d, "width", "the model"), "width")
        vocab = _positive_int(_need(d, "vocab", "the model"), "vocab")
        eps = float(_need(_need(d, "norm", "the model"), "eps", "norm"))
        alpha = float(_need(d, "postln_alpha", "the model"))
        raw_layers = _need(d, "layers", "the model")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where} has type {kind!r}; known mixers are "
                                  f"{sorted(MIXER_KEYS)}")
            mixer = _need(L, "mixer", where)
            for k in MIXER_KEYS[kind]:
                _need(mixer, k, f"{where}.mixer")
            mlp = L.get("mlp")
            if mlp is not None:
                mk = _need(mlp, "kind", f"{where}.mlp")
                if mk == "dense":
                    _positive_int(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff")
                elif mk == "moe":
                    ex = _need(mlp, "expert", f"{where}.mlp")
                    _positive_int(_need(ex, "ff", f"{where}.mlp.expert"), f"{where}.mlp.expert.ff")
                    ro = _need(mlp, "router", f"{where}.mlp")
                    n = _positive_int(_need(ro, "experts", f"{where}.mlp.router"), "experts")
                    top = _positive_int(_need(ro, "top", f"{where}.mlp.router"), "top")
                    if top > n:
                        raise ConfigError(f"config.json: {where} chooses {top} of {n} experts")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mk!r} is not 'dense' or "
                                      "'moe'")
            layers.append(PimidraLayer(kind, mixer, mlp))
        cfg = cls(width=width, vocab=vocab, norm_eps=eps, postln_alpha=alpha,
                  layers=tuple(layers), eos_token_ids=_eos(d.get("eos_token_id"), vocab),
                  torch_dtype=str(d.get("torch_dtype", "bfloat16")),
                  extra={k: v for k, v in d.items()
                         if k not in ("architecture", "width", "vocab", "norm", "postln_alpha",
                                      "layers", "eos_token_id", "torch_dtype")})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not (self.norm_eps > 0):
            raise ConfigError(f"config.json: norm.eps must be > 0, got {self.norm_eps}")
        mixed = None
        for i, L in enumerate(self.layers):
            m, where = L.mixer, f"layers[{i}].mixer"
            for k in ("heads", "vdim"):
                _positive_int(m[k], f"{where}.{k}")
            if L.type == "mamba2":
                for k in ("state", "groups", "conv"):
                    _positive_int(m[k], f"{where}.{k}")
                if m["heads"] % m["groups"]:
                    raise ConfigError(f"config.json: layers[{i}] has {m['heads']} heads for "
                                      f"{m['groups']} groups")
                parts = _positive_int(m.get("norm_groups", 1), f"{where}.norm_groups")
                if (m["heads"] * m["vdim"]) % parts:
                    raise ConfigError(f"config.json: layers[{i}] norms {m['heads'] * m['vdim']} "
                                      f"channels in {parts} parts")
            elif L.type == "gla":
                _positive_int(m["dim"], f"{where}.dim")
                if not (float(m["tau"]) > 0):
                    raise ConfigError(f"config.json: {where}.tau must be > 0")
            else:
                _positive_int(m["dim"], f"{where}.dim")
                _positive_int(m["kv_heads"], f"{where}.kv_heads")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: layers[{i}] has {m['heads']} heads for "
                                      f"{m['kv_heads']} kv heads")
                if m.get("mask") is not None:          # no mask: every earlier token is seen
                    _positive_int(_need(m["mask"], "size", f"{where}.mask"), "mask.size")
                rot = m.get("rot")
                if rot is not None:                    # no rot: queries and keys are not rotated
                    dims = _positive_int(_need(rot, "dims", f"{where}.rot"), "rot.dims")
                    if dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"config.json: layers[{i}] rotates {dims} of {m['dim']} "
                                          "channels; it must be an even number of them")
                    if not (float(_need(rot, "base", f"{where}.rot")) > 0):
                        raise ConfigError(f"config.json: {where}.rot.base must be > 0")
                    sc = rot.get("scaling")
                    if sc is not None and not (float(_need(sc, "factor", f"{where}.rot.scaling"))
                                               > 0):
                        raise ConfigError(f"config.json: {where}.rot.scaling.factor must be > 0")
                if m.get("v_mix"):
                    size = m["kv_heads"] * m["vdim"]
                    if mixed is not None and mixed != size:
                        raise ConfigError(f"config.json: layers[{i}] mixes values of {size} "
                                          f"channels with the first mixing layer's {mixed}")
                    mixed = size

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = dict(self.extra)
        d.update(architecture="Pimidra", width=self.width, vocab=self.vocab,
                 norm={"eps": self.norm_eps}, postln_alpha=self.postln_alpha,
                 layers=[L.to_dict() for L in self.layers], torch_dtype=self.torch_dtype)
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
