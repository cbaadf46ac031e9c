"""Tiny Pimidra configurations and model folders for the tests.  The folders' weights are drawn at
random and then shaped so that faults show: queries are scaled up (peaked attention: a key that is
wrongly seen or missed moves the logits), the decays of the recurrent mixers are slow (a token far
back still matters), norm weights and biases are not small, routers choose clearly."""
from __future__ import annotations

import copy
import json
import os

import torch

from ginfer_b200.config.registry import resolve_architecture
from ginfer_b200.parts.model import DecoderModel
from ginfer_b200.weights.random_init import random_tensors
from ginfer_b200.weights.safetensors_io import write_safetensors


def attention(heads=4, kv_heads=2, dim=16, vdim=16, chunk=37, rot_dims=8, base=1000.0, factor=4.0,
              scale=None, v_mix=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else dim ** -0.5}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if factor:
            m["rot"]["scaling"] = {"factor": factor}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def mamba2(heads=4, vdim=12, state=20, groups=2, conv=3, norm_groups=3):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state,
                                        "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def gla(heads=3, dim=10, vdim=14, tau=8.0, decay_rank=5):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau,
                                     "decay_rank": decay_rank}}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=40):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp):
    return dict(copy.deepcopy(mixer), mlp=copy.deepcopy(mlp))


def config(layers, width=48, vocab=211, eps=2e-5, alpha=1.7):
    return {"architecture": "Pimidra", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "postln_alpha": alpha, "layers": layers, "torch_dtype": "float32"}


# sizes chosen so that nothing is a power of two where it need not be: kv heads fewer than heads,
# a layer whose values are narrower than its keys (the cache keeps two planes), part of a head /
# the whole head / nothing rotating, with and without a stretch of the positions, chunks that are
# no multiple of a page, a layer without mask, a layer without feed-forward, three layers that mix
# their values, one / several groups of a state-space layer, norms in one and in three parts
MIXED = config([
    layer(attention(), moe()),
    layer(mamba2(), dense()),
    layer(gla(), None),
    layer(attention(heads=2, kv_heads=2, dim=24, vdim=16, chunk=21, rot_dims=24, factor=None),
          moe(experts=3, top=1, ff=24)),
    layer(attention(heads=3, kv_heads=1, dim=12, vdim=20, chunk=0, rot_dims=0, v_mix=False),
          dense(ff=56)),
    layer(mamba2(heads=2, vdim=28, state=9, groups=2, conv=2, norm_groups=1), moe()),
    layer(attention(heads=6, kv_heads=2, dim=8, vdim=16, chunk=16, rot_dims=4, base=77.0,
                    factor=1.5), None),
    layer(gla(heads=1, dim=33, vdim=7, tau=3.0, decay_rank=2), dense(ff=40)),
])

# other sizes: all experts chosen, five taps, one group, chunks of ONE token (a token sees itself
# only), one kv head, an alpha below one, a head size the tensor-core kernels take
OTHER = config([
    layer(gla(heads=2, dim=36, vdim=40, tau=30.0, decay_rank=3), moe(experts=4, top=4, ff=32)),
    layer(attention(heads=5, kv_heads=5, dim=32, vdim=32, chunk=64, rot_dims=16, base=50.0,
                    factor=2.0), dense(ff=100)),
    layer(mamba2(heads=3, vdim=16, state=40, groups=1, conv=5, norm_groups=1), None),
    layer(attention(heads=2, kv_heads=1, dim=16, vdim=160, chunk=1, rot_dims=0), dense(ff=64)),
], width=80, vocab=173, eps=1e-6, alpha=0.6)

# head size 64 with equal key and value widths: the kernels of large layers run under replay
# (tcgen05 prompt attention, decode tiles by TMA); chunks longer and shorter than a key tile
WIDE = config([
    layer(attention(heads=4, kv_heads=2, dim=64, vdim=64, chunk=100, rot_dims=32, factor=8.0),
          moe(experts=6, top=2, ff=48)),
    layer(attention(heads=2, kv_heads=2, dim=64, vdim=64, chunk=48, rot_dims=64, factor=None),
          dense(ff=96)),
    layer(mamba2(heads=4, vdim=32, state=64, groups=1, conv=4, norm_groups=2), None),
    layer(gla(heads=2, dim=64, vdim=64, tau=16.0, decay_rank=8), None),
], width=128, vocab=197, eps=1e-5, alpha=2.0)

SSD_ONLY = config([layer(mamba2(), None)], width=40, vocab=97)
GLA_ONLY = config([layer(gla(), None)], width=40, vocab=97)
ATTENTION_ONLY = config([layer(attention(chunk=19, v_mix=False), None)], width=40, vocab=97)
VALUE_MIX = config([layer(attention(chunk=0), None), layer(attention(chunk=0), None)], width=40,
                   vocab=97)
DENSE_FF = config([layer(gla(), dense())], width=40, vocab=97)
ROUTED_FF = config([layer(gla(), moe(experts=7, top=3))], width=40, vocab=97)


def shaped_tensors(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    arch = resolve_architecture(cfg)
    model = DecoderModel(arch.build_plan(arch.config_cls.from_dict(cfg)))
    t = random_tensors(model, seed, torch.float32)
    g = torch.Generator().manual_seed(seed + 1)
    kinds = {f"l{i}": L["type"] for i, L in enumerate(cfg["layers"])}

    def rnd(like, std):
        return torch.randn(like.shape, generator=g) * std
    for name in list(t):
        x = t[name]
        head, _, leaf = name.partition(".")
        kind = kinds.get(head)
        if leaf in ("norm1", "norm2", "mix.norm", "mix.q.norm", "mix.k.norm") \
                or name == "final.norm":
            t[name] = 1.0 + rnd(x, 0.3)
        elif leaf == "mix.A_log":
            t[name] = -3.0 + rnd(x, 1.0)                 # slow decays: far tokens matter
        elif leaf in ("mix.dt_bias", "mix.D"):
            t[name] = rnd(x, 1.0)
        elif leaf == "mix.conv":
            t[name] = rnd(x, 0.6)
        elif leaf == "mix.conv.b":
            t[name] = rnd(x, 0.3)
        elif leaf == "mix.a2.b":
            t[name] = 3.0 + rnd(x, 1.0)                  # decays near one
        elif leaf == "mix.vmix":
            t[name] = torch.rand((), generator=g) * 0.4 + 0.3
        elif leaf in ("mix.q.b", "mix.k.b", "mix.v.b"):
            t[name] = rnd(x, 0.5)
        elif leaf == "mix.q" and kind == "attention":
            t[name] = x * 30.0                           # peaked attention
        elif leaf == "mlp.router":
            t[name] = x * 20.0                           # clear choices
        elif x.dim() == 2:
            t[name] = x * 4.0
    return t


def write_folder(path: str, cfg: dict, seed: int = 0, storage=torch.float32, tensors=None) -> str:
    os.makedirs(path, exist_ok=True)
    out = dict(cfg, torch_dtype="bfloat16" if storage == torch.bfloat16 else "float32")
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f)
    tensors = tensors if tensors is not None else shaped_tensors(cfg, seed)
    tensors = {k: (v if not v.is_floating_point() else v.to(storage)) for k, v in tensors.items()}
    write_safetensors(os.path.join(path, "model.safetensors"), tensors, metadata={"format": "pt"})
    return path


# ----------------------------------------------------------------------------- a key that stands out
EDGE_WIDTH = 32
TARGET, PROBE = 1, 2           # token ids: the key that stands out, and the query that asks for it


def edge_model(chunk: int, vocab: int = 40):
    """A one-layer attention model, made by hand, in which the token PROBE asks for the token
    TARGET and for nothing else: its query is the target's key direction, every other token's
    query is zero (it averages what it sees) and every other key is orthogonal to the probe's
    query.  Seen, the target's value is the probe's answer; unseen, the average of the chunk."""
    W = EDGE_WIDTH
    cfg = config([layer(attention(heads=1, kv_heads=1, dim=W, vdim=W, chunk=chunk, rot_dims=0,
                                  scale=1.0, v_mix=False), None)], width=W, vocab=vocab, eps=1e-6,
                 alpha=0.5)
    g = torch.Generator().manual_seed(chunk)
    a = torch.zeros(W)
    a[0] = 1.0
    b = torch.zeros(W)
    b[1] = 1.0
    embed = torch.randn(vocab, W, generator=g)
    embed[:, :2] = 0.0                                   # fillers: orthogonal to a and b
    embed[TARGET] = a
    embed[PROBE] = b
    t = {"embed": embed, "l0.norm1": 1.0 + torch.randn(W, generator=g) * 0.2,
         "final.norm": torch.ones(W), "head": torch.randn(vocab, W, generator=g),
         "l0.mix.q": torch.outer(a, b) * 4.0, "l0.mix.k": torch.eye(W), "l0.mix.v": torch.eye(W),
         "l0.mix.q.b": torch.zeros(W), "l0.mix.k.b": torch.zeros(W), "l0.mix.v.b": torch.zeros(W),
         "l0.mix.q.norm": torch.ones(W), "l0.mix.k.norm": torch.ones(W),
         "l0.mix.o": torch.randn(W, W, generator=g)}
    return cfg, t
