"""Tiny Bapivik configurations and model folders for the tests.  The folders' weights are drawn at
random and then shaped so that faults show: queries are scaled up (peaked attention: a key that is
wrongly seen or missed moves the logits), norm weights, biases and the weights of the depth
average are not small, and the configurations give slow decays (a token far back still matters)."""
from __future__ import annotations

import copy
import json
import os

import torch

from ginfer_b200.config.registry import resolve_architecture
from ginfer_b200.parts.model import DecoderModel
from ginfer_b200.weights.random_init import random_tensors
from ginfer_b200.weights.safetensors_io import write_safetensors


def attention(heads=4, kv_heads=2, dim=16, window=37, q_temp=(0.4, 16), softcap=15.0, scale=None):
    # normed queries and keys: the scores' spread is set by the scale alone, and a scale of three
    # times the usual one brings them under the cap's bend
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
         "scale": scale if scale is not None else 3.0 * dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=16, vdim=12, kv_rank=32, q_rank=24, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale if scale is not None else dim ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def lightning(heads=3, dim=10, vdim=14, decay=(0.7, 0.95, 0.999)):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                                           "decay": list(decay)}}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp):
    return dict(copy.deepcopy(mixer), mlp=copy.deepcopy(mlp))


def config(layers, width=48, vocab=211, eps=2e-5, max_positions=400, logit_softcap=12.0):
    d = {"architecture": "Bapivik", "width": width, "vocab": vocab, "norm": {"eps": eps},
         "max_positions": max_positions, "layers": layers, "torch_dtype": "float32"}
    if logit_softcap:
        d["logit_softcap"] = logit_softcap
    return d


# sizes chosen so that nothing is a power of two where it need not be: kv heads fewer than heads,
# values narrower and wider than keys, two layers with latent vectors of their own and two that
# read the FIRST one's (not the nearest), a window that is no multiple of a page, an attention
# layer without window, temperature and cap, layers without feed-forward, one head and several
MIXED = config([
    layer(latent(), dense()),
    layer(attention(), dense(ff=56)),
    layer(latent(heads=2, dim=8, vdim=20, kv_rank=32, q_rank=10), None),
    layer(lightning(), dense(ff=40)),
    layer(attention(heads=3, kv_heads=3, dim=24, window=0, q_temp=None, softcap=None), None),
    layer(latent(heads=4, dim=12, vdim=8, kv_rank=32, q_rank=16, kv_from=0), dense()),
    layer(lightning(heads=1, dim=33, vdim=7, decay=(0.99,)), None),
    layer(latent(heads=1, dim=20, vdim=24, kv_rank=32, q_rank=7, kv_from=0), None),
])

# other sizes: a recurrent layer first, windows of ONE and of two tokens (a token sees itself
# only), one kv head, a latent size that fits no tensor-core tile, a temperature that changes
# every token, a decay of exactly one, no cap on the logits, a head size the tensor-core kernels take
OTHER = config([
    layer(lightning(heads=2, dim=36, vdim=40, decay=(1.0, 0.5)), dense(ff=100)),
    layer(attention(heads=5, kv_heads=5, dim=32, window=64, q_temp=(1.5, 1), softcap=4.0), None),
    layer(latent(heads=5, dim=6, vdim=10, kv_rank=20, q_rank=33), dense(ff=64)),
    layer(attention(heads=2, kv_heads=1, dim=16, window=1, q_temp=None, softcap=30.0), dense(ff=32)),
    layer(latent(heads=2, dim=24, vdim=4, kv_rank=20, q_rank=5, kv_from=2), None),
    layer(attention(heads=6, kv_heads=2, dim=8, window=2, q_temp=(0.2, 50), softcap=None), None),
], width=80, vocab=173, eps=1e-6, max_positions=300, logit_softcap=None)

# head size 64, latent and key sizes in multiples of 16: the kernels of large layers run under
# replay; windows longer and shorter than a key tile
WIDE = config([
    layer(attention(heads=4, kv_heads=2, dim=64, window=100, q_temp=(0.3, 32), softcap=25.0),
          dense(ff=96)),
    layer(latent(heads=4, dim=64, vdim=32, kv_rank=64, q_rank=48), None),
    layer(attention(heads=2, kv_heads=2, dim=64, window=48, q_temp=None, softcap=None), dense(ff=48)),
    layer(lightning(heads=2, dim=64, vdim=64, decay=(0.9, 0.995)), None),
    layer(latent(heads=2, dim=32, vdim=64, kv_rank=64, q_rank=32, kv_from=1), dense(ff=64)),
], width=128, vocab=197, eps=1e-5, max_positions=700, logit_softcap=20.0)

# a width that is no multiple of four and sizes that are no multiple of eight anywhere: the scalar
# paths of the row kernels and the products that leave for the library
ODD = config([
    layer(lightning(heads=2, dim=12, vdim=9, decay=(0.9, 0.99)), dense(ff=37)),
    layer(latent(heads=3, dim=10, vdim=7, kv_rank=18, q_rank=11), dense(ff=50)),
    layer(attention(heads=3, kv_heads=1, dim=14, window=21), None),
    layer(latent(heads=2, dim=6, vdim=5, kv_rank=18, q_rank=9, kv_from=1), dense(ff=20)),
    layer(attention(heads=2, kv_heads=2, dim=16, window=40, softcap=None), dense(ff=33)),
], width=50, vocab=101, eps=1e-5, max_positions=200, logit_softcap=9.0)

LIGHTNING_ONLY = config([layer(lightning(), None)], width=40, vocab=97)
LATENT_ONLY = config([layer(latent(), None)], width=40, vocab=97)
SHARED_LATENT = config([layer(latent(), None), layer(latent(kv_rank=32, kv_from=0), None)], width=40,
                       vocab=97)
ATTENTION_ONLY = config([layer(attention(window=19), None)], width=40, vocab=97)
DENSE_FF = config([layer(lightning(), dense())], width=40, vocab=97)


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
        if name == "final.norm":                         # logits that reach their cap's bend
            t[name] = (1.0 + rnd(x, 0.3)) * 8.0
        elif name == "embed":                            # tokens weigh more than positions
            t[name] = x * 5.0
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b", "mix.norm", "mix.q.norm", "mix.k.norm",
                      "mix.dq.norm", "mix.dkv.norm"):
            t[name] = 1.0 + rnd(x, 0.3)
        elif leaf == "dwa":                              # every earlier state counts
            w = 0.15 + 0.2 * torch.rand(x.shape, generator=g)
            w[-1] = 0.8
            t[name] = w
        elif leaf in ("mlp.up.b", "mlp.down.b"):
            t[name] = rnd(x, 0.5)
        elif name == "pos":
            t[name] = rnd(x, 0.05)
        elif leaf == "mix.q" and kind == "attention":
            t[name] = x * 30.0                           # peaked attention
        elif leaf == "mix.uq":
            t[name] = x * 400.0
        elif leaf in ("mix.uk", "mix.dkv", "mix.dq"):
            t[name] = x * 10.0
        elif x.dim() == 2 and name != "embed":
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


def _edge_common(W, vocab, g, max_positions):
    a = torch.zeros(W)
    a[0] = 1.0
    b = torch.zeros(W)
    b[1] = 1.0
    embed = torch.randn(vocab, W, generator=g)
    embed[:, :2] = 0.0                                   # fillers: orthogonal to a and b
    embed[TARGET] = a * 6.0
    embed[PROBE] = b * 6.0
    t = {"embed": embed, "pos": torch.zeros(max_positions, W),
         "l0.norm1": torch.ones(W), "l0.norm1b": 1.0 + torch.randn(W, generator=g) * 0.2,
         "l0.dwa": torch.tensor([0.3, 1.0]), "final.norm": torch.ones(W),
         "l0.mix.o": torch.randn(W, W, generator=g)}
    return a, b, t


def edge_attention_model(window: int, vocab: int = 40, max_positions: int = 512):
    """A one-layer attention model, made by hand, in which the token PROBE asks for the token
    TARGET and for nothing else: its query is the target's key direction, every other token's
    query is zero (it averages what it sees, but for the distance bias) and every other key is
    orthogonal to the probe's query.  Seen, the target's value is the probe's answer; unseen, a
    mixture of the window."""
    W = EDGE_WIDTH
    cfg = config([layer(attention(heads=1, kv_heads=1, dim=W, window=window, q_temp=(0.5, 64),
                                  softcap=50.0, scale=1.0), None)], width=W, vocab=vocab, eps=1e-6,
                 max_positions=max_positions, logit_softcap=None)
    g = torch.Generator().manual_seed(window)
    a, b, t = _edge_common(W, vocab, g, max_positions)
    t.update({"l0.mix.q": torch.outer(a, b) * 4.0, "l0.mix.k": torch.eye(W),
              "l0.mix.q.norm": torch.ones(W), "l0.mix.k.norm": torch.ones(W)})
    return cfg, t


def edge_latent_model(vocab: int = 40, max_positions: int = 512):
    """The same for latent attention (every earlier key is seen): the probe asks for the target,
    however far back it is, and two layers read the same latent vectors."""
    W = EDGE_WIDTH
    cfg = config([layer(latent(heads=1, dim=W, vdim=W, kv_rank=W, q_rank=W, scale=1.0), None)],
                 width=W, vocab=vocab, eps=1e-6, max_positions=max_positions, logit_softcap=None)
    g = torch.Generator().manual_seed(7)
    a, b, t = _edge_common(W, vocab, g, max_positions)
    t.update({"l0.mix.dq": torch.outer(a, b) * 4.0, "l0.mix.dq.norm": torch.ones(W),
              "l0.mix.uq": torch.eye(W), "l0.mix.dkv": torch.eye(W),
              "l0.mix.dkv.norm": torch.ones(W), "l0.mix.uk": torch.eye(W),
              "l0.mix.uv": torch.eye(W), "l0.mix.g": torch.randn(1, W, generator=g) * 0.1})
    return cfg, t
