"""Bapivik on the device against the plain implementation (``plain_bapivik``): every mechanism
alone, whole prompts against token-by-token decoding, portions down to two tokens, batches of
unequal requests, pages and slots used again, keys just inside and just outside a window in prompts
and decoded, a far key among hundreds at page borders, far tokens of the recurrent layers, the
first tokens of a sequence, long decoding through CUDA graphs, other sizes, and greedy generation
through the entry point."""
import json
import math
import os
import random

import numpy as np
import pytest
import torch

import plain_bapivik as plain
import replay
import tiny_bapivik as tb

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64
_folders: dict = {}
_expected: dict = {}


def folder(tmp_path_factory, name, cfg, dtype, tensors=None):
    key = (name, dtype)
    if key not in _folders:
        path = str(tmp_path_factory.mktemp(f"bapivik_{name}_{dtype}"))
        _folders[key] = tb.write_folder(path, cfg, seed=len(name), storage=DTYPES[dtype],
                                        tensors=tensors)
    return _folders[key]


def stored(model_dir):
    """The folder's tensors as float64 (what the file holds, not what was drawn)."""
    from ginfer_b200.weights.safetensors_io import open_model_tensors
    out = {}
    for n, (f, k) in open_model_tensors(model_dir).items():
        t = f.get(k)
        out[n] = t.double() if t.is_floating_point() else t
    return out


def prompts(vocab, lengths, seed=0):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def expected(model_dir, cfg, requests, **kw):
    out = {}
    W = None
    for rid, toks in requests.items():
        key = (model_dir, tuple(toks), tuple(sorted(kw.items())))
        if key not in _expected:
            W = W or stored(model_dir)
            _expected[key] = plain.forward(cfg, W, toks, **kw).numpy()
        out[rid] = _expected[key]
    return out


def make_runner(model_dir, dtype, max_tokens, page_size=16, eager=True, max_live=4):
    from ginfer_b200.engine.loading import load_model
    from ginfer_b200.engine.runner import ModelRunner
    model, _ = load_model(model_dir, dtype, "cuda:0")
    budget = -(-max_tokens // 64) * 64
    return ModelRunner(model, page_size=page_size, max_num_seqs=max_live, max_seq_len=budget,
                       num_pages=budget // page_size, max_num_batched_tokens=budget,
                       enforce_eager=eager)


def rel(row, ref):
    d = row.astype(np.float64) - ref
    d = d - d.mean()
    return float(np.sqrt((d * d).mean()) / np.sqrt(((ref - ref.mean()) ** 2).mean()))


def row_errors(rows, want):
    """Per row: rms of the difference (mean taken off) over the rms of the expected logits."""
    worst, where, errs = 0.0, None, []
    for (rid, pos), row in sorted(rows.items()):
        e = rel(row, want[rid][pos])
        errs.append(e)
        if not e <= worst:
            worst, where = e, (rid, pos)
    return worst, where, float(np.mean(errs)), errs


# float32: differences of summation order.  bfloat16: the folders' peaked attention amplifies the
# format's rounding, so single rows may be off (at most one in thirty) while the mean stays small;
# a misplaced page, a lost state or a window off by one puts most rows near one.
LIMIT = {"float32": (1e-4, 2e-5), "bfloat16": (0.3, 0.05)}


def check(rows, want, dtype, requests):
    assert len(rows) == sum(len(t) for t in requests.values()), "a logits row is missing"
    worst, where, mean, errs = row_errors(rows, want)
    if dtype == "bfloat16":
        over = sum(e > LIMIT[dtype][0] for e in errs)
        assert over <= len(errs) // 30, f"{over} of {len(errs)} rows are off; worst {where}: {worst:.3e}"
    else:
        assert worst <= LIMIT[dtype][0], f"worst row {where}: relative error {worst:.3e}"
    assert mean <= LIMIT[dtype][1], f"mean relative error {mean:.3e}"


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("name", ["LIGHTNING_ONLY", "LATENT_ONLY", "SHARED_LATENT",
                                  "ATTENTION_ONLY", "DENSE_FF"])
def test_each_mechanism_alone(tmp_path_factory, name):
    cfg = getattr(tb, name)
    d = folder(tmp_path_factory, name, cfg, "float32")
    reqs = prompts(cfg["vocab"], [70, 3, 1])
    steps = replay.cut_whole(reqs)
    rows = replay.run_in_process(make_runner(d, "float32", replay.peak_tokens(steps)), steps)
    check(rows, expected(d, cfg, reqs), "float32", reqs)


@pytest.mark.parametrize("without", ["pos", "dwa", "norm_b", "gate", "shared", "q_temp", "softcap",
                                     "slopes", "window", "logit_cap"])
def test_the_oracle_without_a_mechanism_is_far_from_the_oracle(tmp_path_factory, without):
    """Passing the comparisons means the mechanism was computed: leaving it out moves the logits by
    much more than any limit."""
    cfg = tb.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [90], seed=11)
    full = expected(d, cfg, reqs)["r0"]
    less = expected(d, cfg, reqs, without=(without,))["r0"]
    rows = {("r0", p): less[p].astype(np.float32) for p in range(40, 90)}
    assert row_errors(rows, {"r0": full})[2] > 0.01        # the float32 limit is 1e-4


# ----------------------------------------------------------------------------- cuts of the same work
LENGTHS = [150, 97, 41, 5, 1, 66]


def cuts(reqs):
    mixed, _ = replay.cut_mixed(reqs, seed=3, decode_tail=20)
    singles, _ = replay.cut_mixed(reqs, seed=5, decode_tail=9, singles_first=True,
                                  sizes=(2, 2, 3, 17, 40))
    # portions long enough for the tensor-core prompt kernels beside single tokens, in both orders
    long_a, _ = replay.cut_mixed(reqs, seed=9, decode_tail=10, singles_first=True,
                                 sizes=replay.LONG_SIZES)
    long_b, _ = replay.cut_mixed(reqs, seed=10, decode_tail=6, sizes=(64, 80, 65))
    return {"whole": replay.cut_whole(reqs), "decode": replay.cut_tail_decode(reqs, tail=40),
            "portions": replay.cut_portions(reqs), "mixed": mixed, "mixed_singles_first": singles,
            "mixed_long_singles_first": long_a, "mixed_long": long_b}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["MIXED", "OTHER", "WIDE", "ODD"])
def test_cuts_agree_with_plain(tmp_path_factory, name, dtype):
    cfg = getattr(tb, name)
    d = folder(tmp_path_factory, name, cfg, dtype)
    reqs = prompts(cfg["vocab"], LENGTHS, seed=1)
    want = expected(d, cfg, reqs)
    got = {}
    for cut, steps in cuts(reqs).items():
        # the pool holds what the live requests hold and no more: pages and slots are used again
        runner = make_runner(d, dtype, replay.peak_tokens(steps), page_size=8 if name == "OTHER" else 16)
        got[cut] = replay.run_in_process(runner, steps)
        check(got[cut], want, dtype, reqs)
    # how the work was cut changes the logits by rounding only
    for cut in got:
        for key, row in got[cut].items():
            ref = got["whole"][key]
            scale = float(np.abs(ref - ref.mean()).max())
            if dtype == "float32":
                assert float(np.abs(row - ref).max()) <= 1e-3 * scale, (cut, key)


def test_the_first_tokens_of_a_sequence(tmp_path_factory):
    """Positions 0, 1, 2: one key, an empty state, a window that is not yet full, the first rows of
    the position table; as a prompt of their own, as the start of a longer one, one by one, and
    behind another request that left its slot and pages."""
    cfg = tb.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [50, 3, 2, 1], seed=21)
    want = expected(d, cfg, reqs)
    for steps in (replay.cut_whole(reqs), replay.cut_tail_decode(reqs, tail=60),
                  replay.cut_portions(reqs, sizes=(1, 2, 1, 1, 40))):
        runner = make_runner(d, "float32", 64, max_live=1)
        rows = replay.run_in_process(runner, steps)
        check(rows, want, "float32", reqs)
        for rid in reqs:
            for p in range(min(3, len(reqs[rid]))):
                assert rel(rows[(rid, p)], want[rid][p]) <= 1e-4, (rid, p)


@pytest.mark.parametrize("name, dtype", [("MIXED", "float32"), ("WIDE", "bfloat16")])
def test_long_decoding_past_windows_and_pages_through_graphs(tmp_path_factory, name, dtype):
    cfg = getattr(tb, name)
    d = folder(tmp_path_factory, name, cfg, dtype)
    reqs = prompts(cfg["vocab"], [230], seed=2)
    steps = replay.cut_tail_decode(reqs, tail=200)       # 30 in one step, then 200 single tokens
    runner = make_runner(d, dtype, replay.peak_tokens(steps), eager=False)
    check(replay.run_in_process(runner, steps), expected(d, cfg, reqs), dtype, reqs)
    assert runner.graph_launches > 0


@pytest.mark.parametrize("name", ["WIDE", "MIXED"])
def test_equal_prompts_replay_a_graph_of_the_whole_step(tmp_path_factory, name):
    """Prompts of one length, one a step: from the second on the step is captured and replayed
    (latent attention over keys formed for the block table's whole width, the tensor-core prompt
    kernels), then decoded tokens follow; pages and slots are used again."""
    cfg = getattr(tb, name)
    d = folder(tmp_path_factory, name, cfg, "bfloat16")
    reqs = prompts(cfg["vocab"], [300, 300, 300, 300, 300], seed=31)
    steps = []
    for rid, toks in reqs.items():
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": rid, "tokens": toks[:288], "want": list(range(288))}]})
        for i in range(288, 300):
            steps.append({"step": len(steps), "end": [rid] if i == 299 else [], "entries": [
                {"id": rid, "tokens": [toks[i]], "want": [0]}]})
    runner = make_runner(d, "bfloat16", replay.peak_tokens(steps), eager=False)
    rows = replay.run_in_process(runner, steps)
    check(rows, expected(d, cfg, reqs), "bfloat16", reqs)
    assert any(isinstance(k[0], str) for k in runner._graphs), "no portion step was captured"


def test_trace_program(tmp_path_factory, tmp_path):
    cfg = tb.OTHER
    d = folder(tmp_path_factory, "OTHER", cfg, "float32")
    reqs = prompts(cfg["vocab"], [90, 33, 2, 47, 64], seed=4)
    steps, peak = replay.cut_mixed(reqs, seed=7)
    os.makedirs(tmp_path / "out")
    rows = run_trace(d, steps, peak, str(tmp_path / "out"), cfg["vocab"])
    check(rows, expected(d, cfg, reqs), "float32", reqs)


def run_trace(model_dir, steps, max_tokens, out_dir, vocab):
    import subprocess
    import sys
    cmd = [sys.executable, os.path.join(replay.ROOT, "bin", "trace_run"), "--model", model_dir,
           "--dtype", "float32", "--out", out_dir, "--max-tokens", str(max_tokens)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            assert p.stdout.readline().strip() == f"done {s['step']}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    return replay.collect(steps, lambda i: np.fromfile(os.path.join(out_dir, f"{i}.f32"),
                                                       dtype="<f4").reshape(-1, vocab))


# ----------------------------------------------------------------------------- a key at a window's edge
def _edge_cuts(reqs, before, around):
    return (replay.cut_whole(reqs), replay.cut_tail_decode(reqs, tail=1),
            replay.cut_tail_decode(reqs, tail=around + 3),
            replay.cut_portions(reqs, sizes=(max(1, before), 5, 2, 3, max(2, around), 7)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window, page", [(37, 16), (16, 16), (48, 8), (2, 16), (5, 4), (64, 16),
                                          (100, 32)])
def test_a_key_just_inside_and_just_outside_the_window(tmp_path_factory, window, page, dtype):
    """The probing token asks for the target token alone.  The target sits ``window - 1`` tokens
    before the probe (the last key the window keeps) or ``window`` before it (the first one it has
    lost); the probe is a row of the whole prompt, of a later portion, and decoded alone, with the
    target decoded as well or part of the prompt."""
    cfg, tensors = tb.edge_attention_model(window)
    d = folder(tmp_path_factory, f"EDGE{window}", cfg, dtype, tensors)
    W = stored(d)
    rng = random.Random(window)
    probe_at = 2 * window + 70
    answers = {}
    for place, target_at in (("in", probe_at - window + 1), ("out", probe_at - window)):
        toks = [rng.randrange(3, cfg["vocab"]) for _ in range(probe_at + 1)]
        toks[target_at], toks[probe_at] = tb.TARGET, tb.PROBE
        want = plain.forward(cfg, W, toks).numpy()
        answers[place] = want[probe_at]
        reqs = {"e": toks}
        for cut in _edge_cuts(reqs, target_at - 2, window):
            runner = make_runner(d, dtype, len(toks) + 64, page_size=page)
            rows = replay.run_in_process(runner, cut)
            err = rel(rows[("e", probe_at)], want[probe_at])
            assert err <= (2e-4 if dtype == "float32" else 0.05), (place, err)
    # the two places give different answers: the probe reads the target's value or it does not
    dlt = answers["in"] - answers["out"]
    assert np.sqrt((dlt ** 2).mean()) > 0.2 * np.sqrt((answers["in"] ** 2).mean())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("target_at, page", [(0, 16), (15, 16), (16, 16), (17, 16), (255, 8),
                                             (256, 32), (3, 4)])
def test_latent_attention_finds_a_far_key_among_hundreds(tmp_path_factory, target_at, page, dtype):
    """Latent attention sees every earlier key: the probe, 600 tokens on, asks for a target at the
    sequence's start, at a page's last and first place, and the answer differs from the one
    without the target."""
    cfg, tensors = tb.edge_latent_model(max_positions=700)
    d = folder(tmp_path_factory, "EDGE_LATENT", cfg, dtype, tensors)
    W = stored(d)
    rng = random.Random(target_at)
    probe_at = 600
    toks = [rng.randrange(3, cfg["vocab"]) for _ in range(probe_at + 1)]
    toks[probe_at] = tb.PROBE
    without = plain.forward(cfg, W, toks).numpy()[probe_at]
    toks[target_at] = tb.TARGET
    want = plain.forward(cfg, W, toks).numpy()
    assert rel(without.astype(np.float32), want[probe_at]) > 0.2
    reqs = {"e": toks}
    for cut in _edge_cuts(reqs, target_at + 1, 30):
        runner = make_runner(d, dtype, len(toks) + 64, page_size=page)
        rows = replay.run_in_process(runner, cut)
        err = rel(rows[("e", probe_at)], want[probe_at])
        assert err <= (2e-4 if dtype == "float32" else 0.05), err


def test_two_layers_read_the_same_latent_vectors_and_only_the_owner_writes_them(tmp_path_factory):
    """A model whose second layer reads the first one's latent vectors against the same model
    whose second layer reads its OWN (the oracle with ``without=shared`` is far), under cuts that
    use pages again."""
    cfg = tb.SHARED_LATENT
    d = folder(tmp_path_factory, "SHARED_LATENT", cfg, "float32")
    reqs = prompts(cfg["vocab"], [100, 37, 64, 5], seed=8)
    want = expected(d, cfg, reqs)
    steps, peak = replay.cut_mixed(reqs, seed=2, max_live=2)
    rows = replay.run_in_process(make_runner(d, "float32", peak, page_size=8, max_live=2), steps)
    check(rows, want, "float32", reqs)


# ----------------------------------------------------------------------------- generation
@pytest.mark.parametrize("pages", [None, 14])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, pages):
    from ginfer_b200.engine.llm import Engine
    from ginfer_b200.sampling import SamplingParams
    cfg = tb.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [40, 9, 75, 1, 23], seed=6)
    eng = Engine(d, dtype="float32", max_num_seqs=3, max_num_batched_tokens=64, max_seq_len=128,
                 num_kvcache_blocks=pages, kvcache_block_size=8)
    outs = eng.generate(list(reqs.values()), SamplingParams(temperature=0.0, max_tokens=10,
                                                             ignore_eos=True))
    W = stored(d)
    for toks, out in zip(reqs.values(), outs):
        assert len(out) == 10
        seq = list(toks)
        for t in out:
            logits = plain.forward(cfg, W, seq)[-1]
            if int(torch.argmax(logits)) != t:           # only a close call may differ
                assert float(logits.max() - logits[t]) < 1e-3 * float(logits.abs().max()), (seq, t)
            seq.append(t)
    if pages is not None:
        eng.runner.cache.check()


def test_generation_from_the_command_line(tmp_path_factory, tmp_path):
    import subprocess
    import sys
    cfg = tb.OTHER
    d = folder(tmp_path_factory, "OTHER", cfg, "float32")
    reqs = prompts(cfg["vocab"], [6, 11], seed=10)
    f = tmp_path / "prompts.txt"
    f.write_text("\n".join(json.dumps(t) for t in reqs.values()) + "\n")
    r = subprocess.run([sys.executable, os.path.join(replay.ROOT, "bin", "ginfer_generate"),
                        "--model-path", d, "--dtype", "float32", "--prompt-ids", str(f),
                        "--max-tokens", "5", "--ignore-eos", "--max-num-seqs", "2",
                        "--max-seq-len", "64", "--num-kvcache-blocks", "8"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.strip().splitlines()]
    W = stored(d)
    for toks, line in zip(reqs.values(), lines):
        seq = list(toks)
        assert len(line["output_ids"]) == 5
        for t in line["output_ids"]:
            logits = plain.forward(cfg, W, seq)[-1]
            if int(torch.argmax(logits)) != t:
                assert float(logits.max() - logits[t]) < 1e-3 * float(logits.abs().max())
            seq.append(t)


# ----------------------------------------------------------------------------- kernels alone
class _Ctx:
    extras: dict = {}


def rms(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


@pytest.mark.parametrize("store", [torch.float32, torch.bfloat16])
def test_embedding_with_learned_positions(store):
    from ginfer_b200.ops import depth
    g = torch.Generator().manual_seed(0)
    for H in (40, 328, 1030):
        E = torch.randn(57, H, generator=g).to(store)
        P = torch.randn(91, H, generator=g).to(store)
        ids = torch.randint(0, 57, (23,), generator=g).int()
        pos = torch.randint(0, 91, (23,), generator=g).int()
        w = torch.rand(H, generator=g) + 0.5
        hist = torch.zeros(3, 23, H, device="cuda")
        x, n = depth.embedding_positions(ids.cuda(), pos.cuda(), E.cuda(), P.cuda(), out=hist[0],
                                         norm_weight=w.cuda(), norm_eps=1e-4, act_dtype=store)
        want = E.double()[ids.long()] + P.double()[pos.long()]
        assert torch.allclose(x.double().cpu(), want, atol=1e-6)
        assert x.data_ptr() == hist.data_ptr() and float(hist[1:].abs().max()) == 0.0
        tol = 1e-5 if store == torch.float32 else 2e-2
        assert torch.allclose(n.double().cpu(), rms(want, w.double(), 1e-4), atol=tol, rtol=tol)
        x2, none = depth.embedding_positions(ids.cuda(), pos.cuda(), E.cuda(), P.cuda())
        assert none is None and torch.equal(x2, x)


@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [48, 50, 1024, 2050])
def test_sublayer_end_norm_sum_average_and_next_norm(ydt, H):
    """``x + norm_b(y)``, kept as a state of the history, the weighted sum over the states, and the
    norm in front of what follows, in one kernel; with and without the average and the next norm;
    widths that take four channels an access and widths that do not."""
    from ginfer_b200.ops import depth
    g = torch.Generator().manual_seed(H)
    R, states = 19, 5
    x = torch.randn(R, H, generator=g)
    y = (torch.randn(R, H, generator=g) * 3).to(ydt)
    wb, wn = torch.rand(H, generator=g) + 0.5, torch.rand(H, generator=g) + 0.5
    v = x.double() + rms(y.double(), wb.double(), 1e-3)
    out, n = depth.sandwich_update(x.cuda(), y.cuda(), wb.cuda(), 1e-3, ydt)
    assert n is None and torch.allclose(out.double().cpu(), v, atol=1e-5)
    yb = torch.randn(H, generator=g)                  # a bias left for this kernel to add
    out, n = depth.sandwich_update(x.cuda(), y.cuda(), wb.cuda(), 1e-3, ydt, y_bias=yb.cuda())
    vb = x.double() + rms(y.double() + yb.double(), wb.double(), 1e-3)
    assert torch.allclose(out.double().cpu(), vb, atol=1e-5)
    out, n = depth.sandwich_update(x.cuda(), y.cuda(), wb.cuda(), 1e-3, ydt, next_weight=wn.cuda(),
                                   next_eps=1e-5)
    tol = 1e-5 if ydt == torch.float32 else 2e-2
    assert torch.allclose(out.double().cpu(), v, atol=1e-5)
    assert n.dtype == ydt and torch.allclose(n.double().cpu(), rms(v, wn.double(), 1e-5), atol=tol,
                                             rtol=tol)
    for nb in (1, 2, states - 1):
        hist0 = torch.randn(states, R, H, generator=g)
        hist = hist0.clone().cuda()
        mix = torch.randn(nb + 1, generator=g)
        out, n = depth.sandwich_update(x.cuda(), y.cuda(), wb.cuda(), 1e-3, ydt, history=hist,
                                       mix_weights=mix.cuda(), n_before=nb,
                                       next_weight=wn.cuda(), next_eps=1e-5)
        want = (mix.double()[:nb, None, None] * hist0.double()[:nb]).sum(0) + float(mix[nb]) * v
        assert torch.allclose(out.double().cpu(), want, atol=2e-5)
        assert torch.allclose(n.double().cpu(), rms(want, wn.double(), 1e-5), atol=tol, rtol=tol)
        assert torch.allclose(hist[nb].double().cpu(), v, atol=1e-5)      # the layer's own result
        keep = [j for j in range(states) if j != nb]
        assert torch.equal(hist[keep].cpu(), hist0[keep])
        out2, n2 = depth.sandwich_update(x.cuda(), y.cuda(), wb.cuda(), 1e-3, ydt,
                                         history=hist0.clone().cuda(), mix_weights=mix.cuda(),
                                         n_before=nb)
        assert n2 is None and torch.allclose(out2, out, atol=1e-6)


def test_activations_in_place():
    from ginfer_b200 import ops
    g = torch.Generator().manual_seed(1)
    for dt in (torch.float32, torch.bfloat16):
        x = (torch.randn(37, 53, generator=g) * 4).to(dt)
        tol = 1e-6 if dt == torch.float32 else 1e-2
        y = ops.activation_(x.clone().cuda(), "relu2").double().cpu()
        assert torch.allclose(y, torch.relu(x.double()) ** 2, atol=tol, rtol=tol)
        y = ops.activation_((x * 20).clone().cuda(), "softcap", 7.5).double().cpu()
        assert torch.allclose(y, 7.5 * torch.tanh((x * 20).double() / 7.5), atol=tol, rtol=tol)
        assert float(y.abs().max()) <= 7.5


def test_silu_operands_and_the_norm_over_all_heads_with_a_sigmoid_gate():
    from ginfer_b200.ops import decay
    g = torch.Generator(device="cuda").manual_seed(3)
    for act in (torch.float32, torch.bfloat16):
        for C in (42, 96, 1100, 2048):
            T = 17
            p = (torch.randn(T, C + C + 8, generator=g, device="cuda") * 3).to(act)
            f = decay.silu_f32(p, C)
            z = p[:, :C].double()
            assert f.dtype == torch.float32 and torch.allclose(f.double(), z * torch.sigmoid(z),
                                                               atol=1e-6, rtol=1e-6)
            o = torch.randn(T, C, generator=g, device="cuda") * 2
            w = torch.rand(C, generator=g, device="cuda") + 0.5
            y = decay.gated_norm(o, p[:, C:2 * C], w, C, False, 1e-4, act, sigmoid_gate=True)
            want = rms(o.double(), w.double(), 1e-4) * torch.sigmoid(p[:, C:2 * C].double())
            tol = 1e-5 if act == torch.float32 else 2e-2
            assert torch.allclose(y.double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("H, D, Vd", [(3, 10, 14), (1, 33, 7), (4, 64, 64), (2, 128, 96)])
def test_fixed_decays_keep_a_far_token_and_fade_it_by_the_decay(H, D, Vd):
    """One row of decays (a head each) serves every token: a value written at the first token under
    a key that no later token uses is read back 300 tokens later, faded by ``decay^299``, in one
    portion, token by token or in uneven portions, and the state of other slots stays."""
    from ginfer_b200.ops import decay
    T = 300
    g0 = torch.Generator().manual_seed(D)
    k = torch.zeros(T, H, D)
    k[0, :, 0] = 1.0
    for t in range(1, T):
        k[t, :, 1 + t % (D - 1)] = 1.0
    q = torch.zeros(T, H, D)
    q[:, :, 0] = 1.0
    v = torch.randn(T, H, Vd, generator=g0)
    rates = torch.tensor([1.0, 0.99, 0.999, 0.5][:H])
    want = v[0].double() * (rates.double() ** (T - 1))[:, None]
    for cut in ([T], [1] * T, [7, 2, 100, 1, 190]):
        state = torch.zeros(3, H * D * Vd, device="cuda")
        ctx = _Ctx()
        ctx.num_seqs = 1
        ctx.slot_ids = torch.tensor([1], dtype=torch.int32, device="cuda")
        at, last = 0, None
        for n in cut:
            ctx.cu_seqlens_q = torch.tensor([0, n], dtype=torch.int32, device="cuda")
            ctx.max_q_len = n
            sl = slice(at, at + n)
            gt = rates.cuda()[None, :].expand(n, H)            # the same row for every token
            last = decay.recurrence(q[sl].reshape(n, -1).cuda(), k[sl].reshape(n, -1).cuda(),
                                    v[sl].reshape(n, -1).cuda(), gt, state, ctx, H, H, D, Vd)
            at += n
        assert torch.allclose(last[-1].double().cpu().reshape(H, Vd), want, atol=1e-4), cut[:3]
        assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


def test_latent_norms_and_the_cache_write():
    from ginfer_b200.ops import latent
    g = torch.Generator().manual_seed(2)
    for dt in (torch.float32, torch.bfloat16):
        for Q, C in ((24, 32), (33, 20), (88, 136), (0, 64), (768, 512)):
            T, slots = 11, 30
            ld = Q + C + 8
            proj = (torch.randn(T, ld, generator=g) * 2).to(dt)
            qw, cw = torch.rand(Q, generator=g) + 0.5, torch.rand(C, generator=g) + 0.5
            slot = torch.randperm(slots, generator=g)[:T].int()
            pages = torch.zeros(slots, 1, C, dtype=dt).cuda()
            cq = latent.norms(proj.cuda(), 0, Q, qw.cuda() if Q else None, Q, C, cw.cuda(), 1e-5,
                              slot.cuda(), pages)
            tol = 1e-5 if dt == torch.float32 else 2e-2
            if Q:
                assert torch.allclose(cq.double().cpu(), rms(proj[:, :Q].double(), qw.double(), 1e-5),
                                      atol=tol, rtol=tol)
            else:
                assert cq is None
            want = rms(proj[:, Q:Q + C].double(), cw.double(), 1e-5)
            assert torch.allclose(pages[slot.long(), 0].double().cpu(), want, atol=tol, rtol=tol)
            rest = [s for s in range(slots) if s not in set(slot.tolist())]
            assert float(pages[rest].abs().max()) == 0.0
            # a layer that reads another layer's latent vectors writes none
            pages2 = torch.zeros_like(pages)
            latent.norms(proj.cuda(), 0, Q, qw.cuda() if Q else None, Q, C, cw.cuda(), 1e-5, None,
                         pages2)
            assert float(pages2.abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, D, qt", [(4, 2, 16, (0.4, 16)), (3, 3, 24, None), (5, 5, 32, (1.5, 1)),
                                            (6, 2, 10, (0.2, 50)), (16, 4, 128, (0.25, 256))])
def test_head_norms_query_temperature_and_values_that_are_the_raw_keys(dtype, nh, nkv, D, qt):
    from ginfer_b200.ops import prenorm
    g = torch.Generator().manual_seed(D)
    T, slots = 13, 40
    cols = (nh + nkv) * D
    ld = cols + (-cols % 8)
    qk = (torch.randn(T, ld, generator=g) * 2).to(dtype)
    qw, kw = torch.rand(D, generator=g) + 0.5, torch.rand(D, generator=g) + 0.5
    # positions on both sides of the places where the temperature steps
    every = qt[1] if qt else 7
    pos = torch.tensor([0, 1, every - 2, every - 1, every, 2 * every - 2, 2 * every - 1, 2 * every,
                        3 * every - 1, 5 * every, 777, 778, 1023][:T]).clamp(min=0).int()
    slot = torch.randperm(slots, generator=g)[:T].int()
    pages = torch.zeros(2, slots, 1, nkv, D, dtype=dtype).cuda()
    dev = qk.clone().cuda()
    prenorm.qk_norm_rope(dev, nh, nkv, D, nh * D, nh * D, qw.cuda(), kw.cuda(), 1e-5, None, False,
                         pos.cuda(), slot.cuda(), pages, q_temp=qt)
    x = qk.double()
    q = rms(x[:, :nh * D].reshape(T, nh, D), qw.double(), 1e-5)
    if qt:
        temp = 1.0 + qt[0] * torch.log(torch.floor((pos.double() + 1) / qt[1]) + 1)
        q = q * temp[:, None, None]
    k_raw = x[:, nh * D:cols].reshape(T, nkv, D)
    k = rms(k_raw, kw.double(), 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(dev[:, :nh * D].double().cpu().reshape(T, nh, D), q, atol=tol, rtol=tol)
    assert torch.allclose(pages[0][slot.long(), 0].double().cpu(), k, atol=tol, rtol=tol)
    assert torch.equal(pages[1][slot.long(), 0].cpu(), qk[:, nh * D:cols].reshape(T, nkv, D))
    assert torch.equal(dev[:, nh * D:].cpu(), qk[:, nh * D:])         # k stays as projected
    gates = torch.randn(T, nh + 3, generator=g).to(dtype).cuda()
    o = torch.randn(T, nh * D, generator=g).to(dtype)
    got = prenorm.head_gate(o.clone().cuda(), gates[:, 2:2 + nh], nh, D).double().cpu()
    want = o.double().reshape(T, nh, D) * torch.sigmoid(gates[:, 2:2 + nh].double().cpu())[:, :, None]
    assert torch.allclose(got.reshape(T, nh, D), want, atol=tol, rtol=tol)


def _paged_kv(keys, page, nkv, D, dtype, g):
    npages = -(-keys // page)
    order = torch.randperm(npages + 3, generator=g)[:npages]
    k = torch.randn(keys, nkv, D, generator=g).to(dtype)
    v = torch.randn(keys, nkv, D, generator=g).to(dtype)
    pages = torch.zeros(2, npages + 3, page, nkv, D, dtype=dtype)
    for j in range(keys):
        pages[0, order[j // page], j % page] = k[j]
        pages[1, order[j // page], j % page] = v[j]
    return k.double(), v.double(), pages.cuda(), order


def _shaped_reference(q, k, v, p, nh, nkv, scale, window, cap, slopes):
    lo = max(0, p - window + 1) if window > 0 else 0
    out = []
    for n in range(nh):
        s = (k[lo:p + 1, n // (nh // nkv)] @ q[n]) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        if slopes is not None:
            s = s - float(slopes[n]) * (p - torch.arange(lo, p + 1)).double()
        out.append(torch.softmax(s, 0) @ v[lo:p + 1, n // (nh // nkv)])
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, D, window, cap, sloped", [
    (4, 2, 64, 100, 25.0, True), (2, 2, 64, 48, 0.0, True), (16, 4, 128, 0, 30.0, True),
    (3, 1, 16, 37, 4.0, False), (6, 2, 24, 19, 15.0, True), (20, 1, 64, 70, 10.0, True),
    (4, 2, 48, 33, 20.0, True), (2, 2, 80, 72, 20.0, True)])
def test_attention_with_capped_scores_and_a_distance_bias(dtype, nh, nkv, D, window, cap, sloped):
    """The step's queries over a paged cache in shuffled pages, with a cap on the scores and a
    bias a head by the distance: every row of a prompt (the tensor-core prompt kernel in bfloat16
    where the head size allows: tcgen05 from 64 rows, ``mma.sync`` below; the fp32-arithmetic
    kernel elsewhere), single decoded rows of
    several requests (the split decode kernel), and single rows in front of a portion."""
    from ginfer_b200 import ops
    g = torch.Generator().manual_seed(D + window)
    keys, page = 200, 8
    k, v, pages, order = _paged_kv(keys, page, nkv, D, dtype, g)
    q = (torch.randn(keys, nh, D, generator=g) * 3).to(dtype)
    slopes = torch.tensor([2.0 ** (-8.0 * (n + 1) / nh) for n in range(nh)]) if sloped else None
    scale = D ** -0.5
    table1 = order.int().cuda()[None, :]
    tol = 1e-4 if dtype == torch.float32 else 3e-2

    def run(rows_of, starts):
        """rows_of[b]: the positions of request b's rows (all requests read the same cache)."""
        B = len(rows_of)
        rows = [p for r in rows_of for p in r]
        ctx = _Ctx()
        ctx.extras = {}
        ctx.num_seqs, ctx.num_tokens = B, len(rows)
        ctx.q_lens_host = [len(r) for r in rows_of]
        ctx.max_q_len = max(ctx.q_lens_host)
        ctx.decode_only = ctx.max_q_len == 1
        ctx.max_kv_len = max(r[-1] + 1 for r in rows_of)
        i32 = dict(dtype=torch.int32, device="cuda")
        ctx.positions = torch.tensor(rows, **i32)
        ctx.seq_of_token = torch.tensor([b for b, r in enumerate(rows_of) for _ in r], **i32)
        ctx.cu_seqlens_q = torch.tensor([0] + list(np.cumsum(ctx.q_lens_host)), **i32)
        ctx.kv_lens = torch.tensor([r[-1] + 1 for r in rows_of], **i32)
        out = ops.paged_attention(q[rows].reshape(len(rows), nh * D).cuda().contiguous(), pages,
                                  table1.expand(B, -1).contiguous(), ctx, nh, nkv, D, scale, window,
                                  page, softcap=cap, slopes=slopes.cuda() if sloped else None)
        out = out.double().cpu().reshape(len(rows), nh, D)
        for i, p in enumerate(rows):
            want = _shaped_reference(q[p].double(), k, v, p, nh, nkv, scale, window, cap, slopes)
            assert torch.allclose(out[i], want, atol=tol, rtol=tol), (p, starts)
    run([list(range(keys))], "prompt")                                   # a whole prompt
    run([list(range(130, keys))], "portion")                             # a later portion
    run([list(range(150, keys))], "short portion")                       # under the tcgen05 kernel's rows
    run([[keys - 1], [5], [window if window else 63], [0], [77]], "decode")
    run([[keys - 1], [40], list(range(90, 175))], "mixed")               # single rows, then a portion


@pytest.mark.parametrize("M", [1, 8, 16, 33, 64, 100, 700])
def test_squared_relu_in_the_products_epilogue(M):
    """``relu(x W^T + b)^2`` from the tcgen05 kernel (direct tiles and K splits added up inside a
    cluster, by the token count) and from the library product with the kernel behind it, rows of
    exactly zero and negative ones included; in 32-bit from the FMA product."""
    from ginfer_b200 import ops
    from ginfer_b200.ops import gemm_bf16
    g = torch.Generator(device="cuda").manual_seed(M)
    for K, N in ((192, 328), (4096, 136), (64, 1000)):
        x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
        w[:5] = 0
        b = torch.randn(N, generator=g, device="cuda")
        b[:3] = 0
        for bias in (b, None):
            want = torch.relu(x.double() @ w.double().T + (bias.double() if bias is not None else 0)) ** 2
            for out in (torch.bfloat16, torch.float32):
                y = ops.Linear(w, bias, out_dtype=out, activation="relu2")(x)
                assert y.dtype == out and y.shape == (M, N)
                tol = 0.02 if out == torch.bfloat16 else 2e-3
                assert float((y.double() - want).abs().max()) <= tol * float(want.abs().max())
                assert float(y[:, :3].abs().max()) == 0.0 or bias is not None
            y32 = ops.Linear(w.float(), bias, activation="relu2")(x.float())
            assert torch.allclose(y32.double(), want, atol=1e-3, rtol=1e-4)
    gemm_bf16.check_errors("cuda:0")


def test_latent_vectors_gathered_by_the_block_tables():
    from ginfer_b200.ops import latent
    g = torch.Generator().manual_seed(4)
    for dt in (torch.bfloat16, torch.float32):
        for C, page in ((32, 4), (20, 8), (512, 16), (6, 2)):
            pool = 9
            pages = torch.randn(pool, page, 1, C, generator=g).to(dt)
            table = torch.randint(0, pool, (5, 7), generator=g).int()
            table[1, 3] = -1                              # behind a request's last page
            table[2, 4] = pool + 5
            for B, W in ((3, 5), (5, 7), (1, 1)):
                c, own = latent.gather_pages(pages.cuda(), table.cuda(), B, W)
                assert c.shape == (B * W * page, C) and own.shape == (B, W)
                assert torch.equal(own.cpu(), torch.arange(B * W, dtype=torch.int32).view(B, W))
                want = pages[table[:B, :W].clamp(0, pool - 1).long()].reshape(B * W * page, C)
                assert torch.equal(c.cpu(), want)
