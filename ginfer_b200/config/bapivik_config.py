"""Typed configuration of the Bapivik design, read from its own ``config.json`` keys.

A Bapivik folder names its design under ``architecture`` and describes every layer on its own:
``layers[i] = {"type": "lightning" | "latent_attention" | "attention", "mixer": its sizes and
constants, "mlp": {"kind": "dense", "ff": n} or null}``.  Beside the layers: ``width``, ``vocab``,
``max_positions`` (rows of the learned position table), ``norm.eps`` and ``logit_softcap``.  Every
size and constant of a model comes from this object.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_config import ConfigError
from .vilepel_config import _eos, _need, _plain, _positive_int

MIXER_KEYS = {
    "lightning": ("heads", "dim", "vdim", "decay"),
    "latent_attention": ("heads", "dim", "vdim", "kv_rank", "q_rank", "scale"),
    "attention": ("heads", "kv_heads", "dim", "scale"),
}


@dataclass(frozen=True)
class BapivikLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": _plain(self.mixer), "mlp": _plain(self.mlp)}


@dataclass(frozen=True)
class BapivikConfig:
    width: int
    vocab: int
    max_positions: int
    norm_eps: float
    layers: tuple[BapivikLayer, ...]
    logit_softcap: float | None = None
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BapivikConfig":
        width = _positive_int(_need(d, "width", "the model"), "width")
        vocab = _positive_int(_need(d, "vocab", "the model"), "vocab")
        max_pos = _positive_int(_need(d, "max_positions", "the model"), "max_positions")
        eps = float(_need(_need(d, "norm", "the model"), "eps", "norm"))
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
                if mk != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mk!r} is not 'dense'")
                _positive_int(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff")
            layers.append(BapivikLayer(kind, mixer, mlp))
        cap = d.get("logit_softcap")
        cfg = cls(width=width, vocab=vocab, max_positions=max_pos, norm_eps=eps,
                  layers=tuple(layers), logit_softcap=None if cap is None else float(cap),
                  eos_token_ids=_eos(d.get("eos_token_id"), vocab),
                  torch_dtype=str(d.get("torch_dtype", "bfloat16")),
                  extra={k: v for k, v in d.items()
                         if k not in ("architecture", "width", "vocab", "max_positions", "norm",
                                      "layers", "logit_softcap", "eos_token_id", "torch_dtype")})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not (self.norm_eps > 0):
            raise ConfigError(f"config.json: norm.eps must be > 0, got {self.norm_eps}")
        if self.logit_softcap is not None and not (self.logit_softcap > 0):
            raise ConfigError(f"config.json: logit_softcap must be > 0, got {self.logit_softcap}")
        for i, L in enumerate(self.layers):
            m, where = L.mixer, f"layers[{i}].mixer"
            for k in ("heads", "dim"):
                _positive_int(m[k], f"{where}.{k}")
            if L.type == "lightning":
                _positive_int(m["vdim"], f"{where}.vdim")
                dec = m["decay"]
                if not isinstance(dec, (list, tuple)) or len(dec) != m["heads"]:
                    raise ConfigError(f"config.json: {where}.decay must list one decay for each "
                                      f"of the {m['heads']} heads")
            elif L.type == "latent_attention":
                for k in ("vdim", "kv_rank", "q_rank"):
                    _positive_int(m[k], f"{where}.{k}")
                src = m.get("kv_from")
                if src is not None:
                    if not isinstance(src, int) or not (0 <= src < i):
                        raise ConfigError(f"config.json: {where}.kv_from must name an earlier "
                                          f"layer, got {src!r}")
                    S = self.layers[src]
                    if S.type != "latent_attention" or S.mixer.get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}.kv_from names layer {src}, which "
                                          "has no latent vectors of its own")
                    if S.mixer["kv_rank"] != m["kv_rank"]:
                        raise ConfigError(f"config.json: layers[{i}] reads latent vectors of "
                                          f"{S.mixer['kv_rank']} channels as {m['kv_rank']}")
            else:
                _positive_int(m["kv_heads"], f"{where}.kv_heads")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: layers[{i}] has {m['heads']} heads for "
                                      f"{m['kv_heads']} kv heads")
                if m.get("vdim", m["dim"]) != m["dim"]:
                    raise ConfigError(f"config.json: layers[{i}]: the values are the keys, so "
                                      f"vdim {m['vdim']} must equal dim {m['dim']}")
                if m.get("mask") is not None:          # no mask: every earlier token is seen
                    _positive_int(_need(m["mask"], "size", f"{where}.mask"), "mask.size")
                qt = m.get("q_temp")
                if qt is not None:
                    float(_need(qt, "coef", f"{where}.q_temp"))
                    _positive_int(_need(qt, "every", f"{where}.q_temp"), "q_temp.every")
                cap = m.get("softcap")
                if cap is not None and not (float(cap) > 0):
                    raise ConfigError(f"config.json: {where}.softcap must be > 0")

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = dict(self.extra)
        d.update(architecture="Bapivik", width=self.width, vocab=self.vocab,
                 max_positions=self.max_positions, norm={"eps": self.norm_eps},
                 layers=[L.to_dict() for L in self.layers], torch_dtype=self.torch_dtype)
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
