"""Pimidra without a GPU: configuration, the plan, tensor names, caches, and the plain
implementation's own mechanisms on hand-made cases."""
import copy
import math

import pytest
import torch

import plain_pimidra as plain
import tiny_pimidra as tp
from ginfer_b200.config import ConfigError, resolve_architecture
from ginfer_b200.parts.base import PagedKVSpec, StateSpec
from ginfer_b200.parts.model import DecoderModel


def build(cfg):
    arch = resolve_architecture(cfg)
    return arch, arch.config_cls.from_dict(cfg)


def test_registry_and_round_trip():
    arch, cfg = build(tp.MIXED)
    assert arch.name == "Pimidra" and cfg.width == 48 and len(cfg.layers) == 8
    assert cfg.postln_alpha == 1.7 and cfg.norm_eps == 2e-5
    assert build(cfg.to_dict())[1] == cfg


def test_caches_states_and_tensor_names():
    arch, cfg = build(tp.MIXED)
    plan = arch.build_plan(cfg)
    model = DecoderModel(plan)
    specs = model.cache_specs()
    assert specs[0] == PagedKVSpec(2, 16, 0, None, 37)
    assert specs[3] == PagedKVSpec(2, 24, 0, ((2, 24), (2, 16)), 21)      # keys wider than values
    assert specs[4] == PagedKVSpec(1, 12, 0, ((1, 12), (1, 20)), 0)       # no mask
    # S [heads, state, vdim], then the last (taps - 1) inputs of x | B | C
    assert specs[1] == StateSpec((4 * 20 * 12 + 2 * (4 * 12 + 2 * 2 * 20),))
    assert specs[5] == StateSpec((2 * 9 * 28 + 1 * (2 * 28 + 2 * 2 * 9),))
    assert specs[2] == StateSpec((3 * 10 * 14,)) and specs[7] == StateSpec((33 * 7,))
    shapes = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert shapes["l1.mix.in"] == (2 * 48 + 2 * 2 * 20 + 4, 48)
    assert shapes["l1.mix.conv"] == (48 + 80, 3) and shapes["l1.mix.norm"] == (48,)
    assert shapes["l0.mix.q.norm"] == (64,) and shapes["l0.mix.k.norm"] == (32,)
    assert shapes["l0.mix.vmix"] == () and "l4.mix.vmix" not in shapes
    assert shapes["l3.mix.o"] == (48, 2 * 16) and shapes["l3.mix.v.b"] == (2 * 16,)
    assert shapes["l2.mix.a1"] == (5, 48) and shapes["l2.mix.a2"] == (30, 5)
    assert shapes["l2.mix.norm"] == (14,) and shapes["l2.mix.g"] == (42, 48)
    assert "l2.norm2" not in shapes and not any(n.startswith("l2.mlp") for n in shapes)
    assert {"embed", "head", "final.norm", "l0.mlp.e4.down", "l0.mlp.router", "l1.mlp.gate",
            "l7.mix.a2.b", "l5.mix.dt_bias", "l5.mix.D", "l5.mix.conv.b"} <= set(shapes)


def test_every_constant_reaches_the_parts():
    arch, cfg = build(tp.OTHER)
    plan = arch.build_plan(cfg)
    g, a, s, one = plan.layers
    assert all(L.block.kind == "postnorm" and L.block.params["alpha"] == 0.6 for L in plan.layers)
    assert g.mixer.params["tau"] == 30.0 and g.mixer.params["norm_eps"] == 1e-6
    assert g.feed_forward.params["top_k"] == 4 and g.feed_forward.params["renormalize"] is True
    assert math.isinf(g.feed_forward.params["limit"]) and g.feed_forward.params["alpha"] == 1.0
    assert a.mixer.params["chunk"] == 64 and a.mixer.params["scale"] == 32 ** -0.5
    pos = a.mixer.params["position"].params
    assert (pos["dims"], pos["base"], pos["linear_factor"], pos["interleaved"]) == (16, 50.0, 2.0, False)
    assert a.feed_forward.params["alpha"] < 0 and a.feed_forward.params["up_shift"] == 0.0
    assert s.mixer.params["conv_taps"] == 5 and s.mixer.params["groups"] == 1
    assert s.mixer.params["state_dim"] == 40 and s.feed_forward is None
    assert one.mixer.params["chunk"] == 1 and one.mixer.params["position"].params["dims"] == 0
    # the first layer that mixes its values is the source, the others mix
    assert [L.mixer.params.get("value_mix") for L in plan.layers] == [None, "source", None, "mix"]
    roles = [L.mixer.params.get("value_mix") for L in arch.build_plan(build(tp.MIXED)[1]).layers]
    assert roles == ["source", None, None, "mix", None, None, "mix", None]
    assert a.mixer_norm.params["eps"] == 1e-6 and plan.embedding.params["scale"] == 1.0


def test_frequencies_are_divided_by_the_factor():
    from ginfer_b200.parts.position import PairRotary
    f = PairRotary(dims=8, base=100.0, interleaved=False, linear_factor=4.0).host_frequencies()
    want = [100.0 ** (-2 * i / 8) / 4.0 for i in range(4)]
    assert f.dtype.name == "float32" and max(abs(float(a) - b) for a, b in zip(f, want)) < 1e-8


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].__setitem__("type", "latent"), "known mixers"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("groups", 3), "groups"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("norm_groups", 5), "parts"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), "even"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "positive"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("vdim", 20), "mixes values"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("tau", 0), "tau"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "chooses"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "glu"), "dense"),
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
])
def test_refusals(edit, text):
    cfg = copy.deepcopy(tp.MIXED)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        build(cfg)


def test_key_sizes_over_the_recurrences_limit_are_refused_when_the_model_is_built():
    for i, key in ((1, "state"), (2, "dim")):
        cfg = copy.deepcopy(tp.MIXED)
        cfg["layers"][i]["mixer"][key] = 257
        arch, typed = build(cfg)
        with pytest.raises(ValueError, match="recurrence kernel"):
            DecoderModel(arch.build_plan(typed))


def test_mask_span_encoding():
    from ginfer_b200.ops import mask_span
    assert (mask_span(), mask_span(window=7), mask_span(chunk=5)) == (0, 7, -5)
    with pytest.raises(ValueError):
        mask_span(3, 4)


# ----------------------------------------------------------------------------- the oracle's own mechanisms
def test_chunks_are_counted_from_position_zero():
    ok = plain.visible(7, 3)
    assert ok[2].tolist() == [True, True, True, False, False, False, False]
    assert ok[3].tolist() == [False, False, False, True, False, False, False]
    assert ok[5].tolist() == [False, False, False, True, True, True, False]
    assert plain.visible(3, 0).tolist() == [[True, False, False], [True, True, False], [True] * 3]
    assert plain.visible(3, 1).tolist() == [[True, False, False], [False, True, False],
                                            [False, False, True]]


def test_half_rotation_pairs_and_partial_heads():
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0                                     # pairs with channel 2 when dims = 4
    x[:, 0, 5] = 7.0                                     # beyond the rotated channels
    y = plain.rotate_half(x, 4, 10.0, 2.0)
    for p in range(3):
        a = p * 1.0 / 2.0                                # f_0 = 1, divided by the factor
        assert torch.allclose(y[p, 0, [0, 2]], torch.tensor([math.cos(a), math.sin(a)], dtype=torch.float64))
        assert float(y[p, 0, 5]) == 7.0 and float(y[p, 0, 1]) == 0.0 and float(y[p, 0, 3]) == 0.0


def test_causal_taps_and_router():
    u = torch.arange(1.0, 5.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)          # the last tap is the current token's
    out = plain.causal_conv(u, w, torch.tensor([0.5], dtype=torch.float64))
    assert out[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5]
    idx, wgt = plain.route(torch.tensor([[0.0, 2.0, 2.0, -1.0]], dtype=torch.float64), 2)
    assert idx.tolist() == [[1, 2]] and wgt.tolist() == [[0.5, 0.5]]
    idx, wgt = plain.route(torch.tensor([[1.0, 3.0, 0.0]], dtype=torch.float64), 2)
    e = math.exp(-2.0)
    assert idx.tolist() == [[1, 0]] and abs(float(wgt[0, 1]) - e / (1 + e)) < 1e-12


def test_state_space_recurrence_by_hand():
    """One head, one state channel, no convolution reach: S_t = a_t S + dt_t B_t x_t."""
    m = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    P = {"in": torch.eye(5, dtype=torch.float64), "conv": torch.ones(3, 1, dtype=torch.float64),
         "conv.b": torch.zeros(3, dtype=torch.float64), "dt_bias": torch.zeros(1, dtype=torch.float64),
         "A_log": torch.zeros(1, dtype=torch.float64), "D": torch.tensor([0.5], dtype=torch.float64),
         "norm": torch.ones(1, dtype=torch.float64), "o": torch.ones(1, 1, dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0, 1.0, 1.0, 0.3], [1.0, -1.0, 2.0, 0.5, -0.2]], dtype=torch.float64)
    y = plain.mamba2(h, {"p." + k: v for k, v in P.items()}, "p.", m, 0.0)
    x, B, C = plain.silu(h[:, 1]), plain.silu(h[:, 2]), plain.silu(h[:, 3])
    dt = plain.softplus(h[:, 4])
    S0 = dt[0] * B[0] * x[0]
    S1 = torch.exp(-dt[1]) * S0 + dt[1] * B[1] * x[1]
    raw = torch.stack([S0 * C[0] + 0.5 * x[0], S1 * C[1] + 0.5 * x[1]]) * plain.silu(h[:, 0])
    assert torch.allclose(y[:, 0], raw / raw.abs())      # a norm over one channel leaves the sign
