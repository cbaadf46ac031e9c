"""Bapivik without a GPU: configuration, the plan, tensor names, caches, and the plain
implementation's own mechanisms on hand-made cases."""
import copy
import math

import pytest
import torch

import plain_bapivik as plain
import tiny_bapivik as tb
from ginfer_b200.config import ConfigError, resolve_architecture
from ginfer_b200.parts.base import PagedKVSpec, StateSpec
from ginfer_b200.parts.model import DecoderModel

F64 = torch.float64


def build(cfg):
    arch = resolve_architecture(cfg)
    return arch, arch.config_cls.from_dict(cfg)


def test_registry_and_round_trip():
    arch, cfg = build(tb.MIXED)
    assert arch.name == "Bapivik" and cfg.width == 48 and len(cfg.layers) == 8
    assert cfg.max_positions == 400 and cfg.norm_eps == 2e-5 and cfg.logit_softcap == 12.0
    assert build(cfg.to_dict())[1] == cfg
    assert build(tb.OTHER)[1].logit_softcap is None


def test_run_list_caches_states_and_tensor_names():
    arch, cfg = build(tb.MIXED)
    plan = arch.build_plan(cfg)
    assert plan.max_positions == 400
    # the layers that read another layer's latent vectors read ITS cache and write none
    assert [(e.layer, e.cache, e.write_cache) for e in plan.run] == [
        (0, 0, True), (1, 1, True), (2, 2, True), (3, 3, True), (4, 4, True), (5, 0, False),
        (6, 6, True), (7, 0, False)]
    model = DecoderModel(plan)
    specs = model.cache_specs()
    assert set(specs) == {0, 1, 2, 3, 4, 6}
    assert specs[0] == PagedKVSpec(1, 32, 0, ((1, 32),)) == specs[2]     # one latent vector a token
    assert specs[1] == PagedKVSpec(2, 16, 37) and specs[4] == PagedKVSpec(3, 24, 0)
    assert specs[3] == StateSpec((3 * 10 * 14,)) and specs[6] == StateSpec((33 * 7,))
    shapes = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert shapes["embed"] == (211, 48) and shapes["pos"] == (400, 48)
    assert "head" not in shapes                                          # the head is the embedding
    assert shapes["l0.mix.dq"] == (24, 48) and shapes["l0.mix.uq"] == (48, 24)
    assert shapes["l0.mix.dkv"] == (32, 48) and shapes["l0.mix.dkv.norm"] == (32,)
    assert shapes["l0.mix.uk"] == (48, 32) and shapes["l0.mix.uv"] == (36, 32)
    assert shapes["l0.mix.g"] == (3, 48) and shapes["l0.mix.o"] == (48, 36)
    assert "l5.mix.dkv" not in shapes and "l5.mix.dkv.norm" not in shapes
    assert shapes["l5.mix.uk"] == (48, 32) and shapes["l5.mix.dq.norm"] == (16,)
    assert shapes["l1.mix.q"] == (64, 48) and shapes["l1.mix.k"] == (32, 48)
    assert "l1.mix.v" not in shapes and shapes["l1.mix.q.norm"] == (16,)
    assert shapes["l3.mix.norm"] == (42,) and shapes["l3.mix.g"] == (42, 48)
    assert shapes["l3.mix.q"] == (30, 48) and shapes["l3.mix.o"] == (48, 42)
    assert [shapes[f"l{i}.dwa"] for i in range(8)] == [(i + 2,) for i in range(8)]
    assert shapes["l0.mlp.up.b"] == (72,) and shapes["l0.mlp.down.b"] == (48,)
    assert "l2.norm2" not in shapes and "l2.norm2b" not in shapes and "l2.norm1b" in shapes
    assert not any(n.startswith("l2.mlp") for n in shapes)


def test_every_constant_reaches_the_parts():
    arch, cfg = build(tb.OTHER)
    plan = arch.build_plan(cfg)
    li, at, la, a1, sh, a2 = plan.layers
    assert plan.embedding.params["keep_states"] == 7 and plan.head.params["softcap"] is None
    assert plan.head.params["tied_to"] == "embed"
    assert li.mixer.params["decays"] == (1.0, 0.5) and li.mixer.params["norm_eps"] == 1e-6
    assert at.mixer.params["q_temp"] == (1.5, 1) and at.mixer.params["softcap"] == 4.0
    assert at.mixer.params["window"] == 64 and a1.mixer.params["window"] == 1
    assert a1.mixer.params["q_temp"] is None and a2.mixer.params["softcap"] is None
    assert at.mixer.params["distance_slope_base"] == 8.0 and at.mixer.params["position"] is None
    assert la.mixer.params["q_rank"] == 33 and la.mixer.params["own_latent"] is True
    assert sh.mixer.params["own_latent"] is False and sh.mixer.params["kv_rank"] == 20
    assert la.mixer.params["rope_dim"] == 0 and la.mixer.params["head_gate"] is True
    for i, L in enumerate(plan.layers):
        assert L.block.kind == "sandwich" and L.block.params["depth_states"] == i + 2
        assert L.mixer_norm.params["eps"] == 1e-6
    assert build(tb.WIDE)[0].build_plan(build(tb.WIDE)[1]).head.params["softcap"] == 20.0


def test_refusals():
    def bad(change, text):
        cfg = copy.deepcopy(tb.MIXED)
        change(cfg)
        with pytest.raises(ConfigError, match=text):
            build(cfg)
    bad(lambda c: c["layers"][0].update(type="conv"), "known mixers")
    bad(lambda c: c["layers"][3]["mixer"].update(decay=[0.5]), "one decay")
    bad(lambda c: c["layers"][5]["mixer"].update(kv_from=7), "earlier")
    bad(lambda c: c["layers"][5]["mixer"].update(kv_from=1), "no latent vectors")
    bad(lambda c: c["layers"][7]["mixer"].update(kv_from=5), "no latent vectors")
    bad(lambda c: c["layers"][5]["mixer"].update(kv_rank=16), "channels")
    bad(lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv heads")
    bad(lambda c: c["layers"][1]["mixer"].update(vdim=8), "values are the keys")
    bad(lambda c: c["layers"][0]["mlp"].update(kind="moe"), "dense")
    bad(lambda c: c.pop("max_positions"), "max_positions")
    bad(lambda c: c.update(logit_softcap=0.0), "logit_softcap")


# ----------------------------------------------------------------------------- the oracle itself
def test_visibility_and_temperature_by_hand():
    v = plain.visible(5, 2)
    assert v.tolist() == [[True, False, False, False, False], [True, True, False, False, False],
                          [False, True, True, False, False], [False, False, True, True, False],
                          [False, False, False, True, True]]
    assert plain.visible(3, 0).tolist() == [[True, False, False], [True, True, False],
                                            [True, True, True]]
    assert plain.visible(3, 1).tolist() == [[True, False, False], [False, True, False],
                                            [False, False, True]]
    t = plain.query_temperature(9, 0.5, 4)            # floor((p + 1) / 4): 0 0 0 1 1 1 1 2 2
    want = [1.0] * 3 + [1 + 0.5 * math.log(2)] * 4 + [1 + 0.5 * math.log(3)] * 2
    assert torch.allclose(t, torch.tensor(want, dtype=F64))


def test_lightning_recurrence_by_hand():
    """One head with one key channel and two value channels: the state is a geometric sum."""
    m = {"heads": 1, "dim": 1, "vdim": 2, "decay": [0.5]}
    one = torch.tensor([[1.0]], dtype=F64)
    P = {"q": one, "k": one, "v": torch.tensor([[1.0], [2.0]], dtype=F64),
         "g": torch.zeros(2, 1, dtype=F64), "o": torch.eye(2, dtype=F64),
         "norm": torch.tensor([2.0, 3.0], dtype=F64)}
    hs = [1.0, 2.0, -1.0]
    s = lambda z: z / (1 + math.exp(-z))               # noqa: E731
    S = [0.0, 0.0]
    want = []
    for x in hs:
        S = [0.5 * S[c] + s(x) * s((c + 1) * x) for c in range(2)]
        o = [s(x) * S[c] for c in range(2)]
        rms = math.sqrt((o[0] ** 2 + o[1] ** 2) / 2 + 1e-9)
        want.append([o[0] / rms * 2.0 * 0.5, o[1] / rms * 3.0 * 0.5])   # the gate is sigmoid(0)
    out = plain.lightning(torch.tensor(hs, dtype=F64)[:, None], P, "", m, 1e-9)
    assert torch.allclose(out, torch.tensor(want, dtype=F64))


def test_attention_values_are_the_unnormed_keys_and_bias_counts_the_distance():
    torch.manual_seed(0)
    W, D = 6, 4
    m = {"heads": 2, "kv_heads": 1, "dim": D, "scale": 0.0}     # scale 0: only the bias is left
    P = {"q": torch.randn(2 * D, W, dtype=F64), "k": torch.randn(D, W, dtype=F64),
         "q.norm": torch.ones(D, dtype=F64), "k.norm": torch.full((D,), 9.0, dtype=F64),
         "o": torch.eye(2 * D, dtype=F64)}
    h = torch.randn(3, W, dtype=F64)
    out = plain.attention(h, P, "", m, 1e-6).reshape(3, 2, D)
    k = h @ P["k"].T
    for n in range(2):
        slope = 2.0 ** (-8.0 * (n + 1) / 2)
        w = torch.softmax(torch.tensor([-2 * slope, -slope, 0.0], dtype=F64), 0)
        assert torch.allclose(out[2, n], w @ k)                  # values: k as projected
    assert torch.allclose(out[0, 0], k[0])


def test_depth_average_and_shared_latents_by_hand():
    """Two layers whose sublayers are switched off (zero output matrices): the stream after layer
    i is the weighted sum of equal states, and a layer that names another's latent vectors gives
    the same result as the oracle reading them directly."""
    cfg = tb.SHARED_LATENT
    t = {k: v.double() for k, v in tb.shaped_tensors(cfg, 3).items()}
    toks = [5, 9, 1, 33]
    t0 = dict(t)
    t0["l0.mix.o"] = torch.zeros_like(t["l0.mix.o"])
    t0["l1.mix.o"] = torch.zeros_like(t["l1.mix.o"])
    layers = []
    plain.forward(cfg, t0, toks, layers_out=layers)
    x0 = plain.embed(toks, t0)
    assert torch.allclose(layers[0], t0["l0.dwa"].sum() * x0)
    x1 = layers[0]                                               # layer 1's input and its result
    assert torch.allclose(layers[1], (t0["l1.dwa"][0] + t0["l1.dwa"][1]) * x0 + t0["l1.dwa"][2] * x1)
    # without the average the second layer's latent source matters through its own weights only
    a = plain.forward(cfg, t, toks)
    b = plain.forward(cfg, t, toks, without=("dwa",))
    assert not torch.allclose(a, b)
