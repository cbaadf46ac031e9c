"""Pimidra on the device against the plain implementation (``plain_pimidra``): every mechanism
alone, whole prompts against token-by-token decoding, portions down to two tokens, batches of
unequal requests, pages and slots used again, keys at the edges of chunks and pages, far tokens of
the recurrent layers, long decoding through CUDA graphs, other sizes, and greedy generation
through the entry point."""
import json
import os
import random

import numpy as np
import pytest
import torch

import plain_pimidra as plain
import replay
import tiny_pimidra as tp

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_folders: dict = {}
_expected: dict = {}


def folder(tmp_path_factory, name, cfg, dtype, tensors=None):
    key = (name, dtype)
    if key not in _folders:
        path = str(tmp_path_factory.mktemp(f"pimidra_{name}_{dtype}"))
        _folders[key] = tp.write_folder(path, cfg, seed=len(name), storage=DTYPES[dtype],
                                        tensors=tensors)
    return _folders[key]


def stored(model_dir):
    from ginfer_b200.weights.safetensors_io import open_model_tensors
    return {n: f.get(k) for n, (f, k) in open_model_tensors(model_dir).items()}


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
            _expected[key] = plain.forward(cfg, W, toks, **kw)[0].numpy()
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


def row_errors(rows, want):
    """Per row: rms of the difference (mean taken off) over the rms of the expected logits."""
    worst, where, errs = 0.0, None, []
    for (rid, pos), row in sorted(rows.items()):
        ref = want[rid][pos]
        d = row.astype(np.float64) - ref
        d = d - d.mean()
        e = float(np.sqrt((d * d).mean()) / np.sqrt(((ref - ref.mean()) ** 2).mean()))
        errs.append(e)
        if not e <= worst:
            worst, where = e, (rid, pos)
    return worst, where, float(np.mean(errs)), errs


# float32: differences of summation order.  bfloat16: the folders' peaked attention and clear
# routing amplify the format's rounding, so single rows may be off while the mean stays small, and
# a row whose router scores were close may choose another expert (at most one row in thirty may be
# off for that); a misplaced page, a lost state or a chunk off by one puts most rows near one.
LIMIT = {"float32": (3e-4, 5e-5), "bfloat16": (0.3, 0.1)}


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
@pytest.mark.parametrize("name", ["SSD_ONLY", "GLA_ONLY", "ATTENTION_ONLY", "VALUE_MIX", "DENSE_FF",
                                  "ROUTED_FF"])
def test_each_mechanism_alone(tmp_path_factory, name):
    cfg = getattr(tp, name)
    d = folder(tmp_path_factory, name, cfg, "float32")
    reqs = prompts(cfg["vocab"], [70, 3, 1])
    steps = replay.cut_whole(reqs)
    rows = replay.run_in_process(make_runner(d, "float32", replay.peak_tokens(steps)), steps)
    check(rows, expected(d, cfg, reqs), "float32", reqs)


@pytest.mark.parametrize("without", ["alpha", "chunk", "vmix", "scaling"])
def test_the_oracle_without_a_mechanism_is_far_from_the_oracle(tmp_path_factory, without):
    """Passing the comparisons means the mechanism was computed: leaving it out moves the logits by
    much more than any limit."""
    cfg = tp.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "float32")
    reqs = prompts(cfg["vocab"], [90], seed=11)
    full = expected(d, cfg, reqs)["r0"]
    less = expected(d, cfg, reqs, without=(without,))["r0"]
    rows = {("r0", p): less[p].astype(np.float32) for p in range(40, 90)}
    assert row_errors(rows, {"r0": full})[2] > 0.01        # the float32 limit is 3e-4


# ----------------------------------------------------------------------------- cuts of the same work
LENGTHS = [150, 97, 41, 5, 1, 66]


def cuts(reqs):
    mixed, _ = replay.cut_mixed(reqs, seed=3, decode_tail=20)
    singles, _ = replay.cut_mixed(reqs, seed=5, decode_tail=9, singles_first=True,
                                  sizes=(2, 2, 3, 17, 40))
    return {"whole": replay.cut_whole(reqs), "decode": replay.cut_tail_decode(reqs, tail=40),
            "portions": replay.cut_portions(reqs), "mixed": mixed, "mixed_singles_first": singles}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["MIXED", "OTHER", "WIDE"])
def test_cuts_agree_with_plain(tmp_path_factory, name, dtype):
    cfg = getattr(tp, name)
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


def test_a_long_portion_takes_the_tcgen05_grouped_products(tmp_path_factory):
    """Six hundred tokens in one step are 1,200 (token, expert) pairs in the routed layers that
    choose two experts: the grouped products run on tcgen05 (with the SiLU gate in the epilogue),
    the long portion takes the recurrence with sixteen lanes a column, and the norm behind the sum
    adds up the pairs' rows; a short request follows it."""
    from ginfer_b200.ops import moe
    cfg = tp.MIXED
    d = folder(tmp_path_factory, "MIXED", cfg, "bfloat16")
    reqs = prompts(cfg["vocab"], [600, 70], seed=12)
    assert 600 * 2 >= moe.TCGEN05_MIN_PAIRS
    steps = replay.cut_whole(reqs)
    rows = replay.run_in_process(make_runner(d, "bfloat16", replay.peak_tokens(steps)), steps)
    check(rows, expected(d, cfg, reqs), "bfloat16", reqs)


@pytest.mark.parametrize("name, dtype", [("MIXED", "float32"), ("WIDE", "bfloat16")])
def test_long_decoding_past_chunks_and_pages_through_graphs(tmp_path_factory, name, dtype):
    cfg = getattr(tp, name)
    d = folder(tmp_path_factory, name, cfg, dtype)
    reqs = prompts(cfg["vocab"], [230], seed=2)
    steps = replay.cut_tail_decode(reqs, tail=200)       # 30 in one step, then 200 single tokens
    runner = make_runner(d, dtype, replay.peak_tokens(steps), eager=False)
    check(replay.run_in_process(runner, steps), expected(d, cfg, reqs), dtype, reqs)
    assert runner.graph_launches > 0


def test_trace_program(tmp_path_factory, tmp_path):
    cfg = tp.OTHER
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


# ----------------------------------------------------------------------------- a key at a chunk's edge
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk, page", [(37, 16), (16, 16), (48, 8), (1, 16), (5, 4)])
def test_a_key_just_inside_and_just_outside_the_chunk(tmp_path_factory, chunk, page, dtype):
    """The probing token asks for the target token alone.  The target sits on the first position of
    the probe's chunk (seen) or on the last one of the chunk before (not seen), the probe on the
    chunk's last position, as a row of the whole prompt, of a later portion, and decoded alone."""
    cfg, tensors = tp.edge_model(chunk)
    d = folder(tmp_path_factory, f"EDGE{chunk}", cfg, dtype, tensors)
    W = stored(d)
    rng = random.Random(chunk)
    start = 3 * chunk                                    # the chunk the probe sits in
    probe_at = start + chunk - 1
    answers = {}
    for place, target_at in (("in", start), ("out", start - 1)):
        if chunk == 1 and place == "in":
            continue                                     # the probe's only key is itself
        toks = [rng.randrange(3, cfg["vocab"]) for _ in range(probe_at + 1)]
        toks[target_at], toks[probe_at] = tp.TARGET, tp.PROBE
        want = plain.forward(cfg, W, toks)[0].numpy()
        answers[place] = want[probe_at]
        reqs = {"e": toks}
        for cut in (replay.cut_whole(reqs), replay.cut_tail_decode(reqs, tail=1),
                    replay.cut_portions(reqs, sizes=(start - 2, 5, 2, 3, chunk, 7))):
            runner = make_runner(d, dtype, len(toks) + 64, page_size=page)
            rows = replay.run_in_process(runner, cut)
            ref = want[probe_at]
            dlt = rows[("e", probe_at)].astype(np.float64) - ref
            err = np.sqrt(((dlt - dlt.mean()) ** 2).mean()) / np.sqrt(((ref - ref.mean()) ** 2).mean())
            assert err <= (2e-4 if dtype == "float32" else 0.05), (place, err)
    if len(answers) == 2:                                # the two places give different answers
        dlt = answers["in"] - answers["out"]
        assert np.sqrt((dlt ** 2).mean()) > 0.2 * np.sqrt((answers["in"] ** 2).mean())


# ----------------------------------------------------------------------------- generation
@pytest.mark.parametrize("pages", [None, 14])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, pages):
    from ginfer_b200.engine.llm import Engine
    from ginfer_b200.sampling import SamplingParams
    cfg = tp.MIXED
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
            logits = plain.forward(cfg, W, seq)[0][-1]
            top2 = torch.topk(logits, 2).values
            if int(torch.argmax(logits)) != t:           # only a close call may differ
                assert float(top2[0] - logits[t]) < 1e-3 * float(logits.abs().max()), (seq, t)
            seq.append(t)
    if pages is not None:
        eng.runner.cache.check()


def test_generation_from_the_command_line(tmp_path_factory, tmp_path):
    import subprocess
    import sys
    cfg = tp.OTHER
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
            logits = plain.forward(cfg, W, seq)[0][-1]
            if int(torch.argmax(logits)) != t:
                assert float(logits.max() - logits[t]) < 1e-3 * float(logits.abs().max())
            seq.append(t)


# ----------------------------------------------------------------------------- kernels alone
class _Ctx:
    pass


def test_norm_behind_the_sum_and_its_pair_sum():
    from ginfer_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    for act in (torch.float32, torch.bfloat16):
        for H in (88, 50, 1024, 4100):
            x = torch.randn(37, H, generator=g, device="cuda")
            y = (torch.randn(37, H, generator=g, device="cuda") * 3).to(act)
            w = torch.randn(H, generator=g, device="cuda")
            out, a = ops.postnorm(x, y, 2.5, w, 1e-3, act)
            want = plain.rms_norm(2.5 * x.double() + y.double(), w.double(), 1e-3)
            assert torch.allclose(out.double(), want, atol=1e-5, rtol=1e-5)
            assert a.dtype == act and torch.equal(a, out.to(act))
            # rows of (token, choice) pairs in shuffled places, weighted
            top = 3
            rows = torch.randn(37 * top, H, generator=g, device="cuda")
            pos = torch.randperm(37 * top, generator=g, device="cuda").int()
            wg = torch.rand(37, top, generator=g, device="cuda")
            for weights in (wg, None):
                out, _ = ops.postnorm(x, rows, 0.7, w, 1e-3, act, pairs=(pos, weights, top))
                y2 = rows.double()[pos.long()].reshape(37, top, H)
                y2 = (y2 * wg.double()[:, :, None]).sum(1) if weights is not None else y2.sum(1)
                want = plain.rms_norm(0.7 * x.double() + y2, w.double(), 1e-3)
                assert torch.allclose(out.double(), want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("T", [1, 8, 40, 100, 800, 1100])
def test_relu_gate_in_the_products_epilogues(T):
    """``relu(gate) * up`` as the step form of the clamped sigmoid-gated activation (no limit, a
    negative alpha), inside the three gated product paths, zero gates included."""
    from ginfer_b200 import ops
    from ginfer_b200.ops import gemm_bf16
    g = torch.Generator(device="cuda").manual_seed(T)
    K, I = 192, 328
    x = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
    wg = (torch.randn(I, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    wg[:7] = 0                                           # gates of exactly zero
    wu = (torch.randn(I, K, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    z = ops.GatedLinear(wg, wu, clamped=(float("inf"), -1.0, 0.0))(x)
    gate = (x.double() @ wg.double().T).to(torch.bfloat16).double()
    up = (x.double() @ wu.double().T).to(torch.bfloat16).double()
    want = torch.relu(gate) * up
    assert z.shape == (T, I) and not torch.isnan(z).any()
    assert float((z.double() - want).abs().max()) <= 0.03 * float(want.abs().max())
    z32 = ops.clamped_glu(torch.stack([gate, up], -1).reshape(T, 2 * I).float(), float("inf"),
                          -1.0, 0.0)
    assert torch.allclose(z32.double(), want, atol=1e-5)
    gemm_bf16.check_errors("cuda:0")


def test_router_weights_are_the_softmax_over_the_chosen_logits():
    from ginfer_b200.ops import moe
    g = torch.Generator(device="cuda").manual_seed(1)
    for E, top in ((5, 2), (12, 4), (3, 1), (4, 4), (70, 6)):
        z = torch.randn(41, E, generator=g, device="cuda") * 3
        z[0] = 0.0                                       # equal logits: the lowest indices win
        idx, w = moe.route(z, top, True)
        wi, ww = plain.route(z.double().cpu(), top)
        assert torch.equal(idx.long().cpu(), wi)
        assert torch.allclose(w.double().cpu(), ww, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, D, Vd, rot", [(4, 2, 16, 16, 8), (3, 1, 12, 20, 0), (2, 2, 64, 64, 64),
                                                 (5, 5, 24, 8, 6), (3, 1, 32, 24, 16), (2, 1, 10, 6, 4),
                                                 (16, 4, 128, 128, 64)])
def test_whole_projection_norm_rotation_mix_and_cache_write(dtype, nh, nkv, D, Vd, rot):
    # sizes in multiples of four take the kernel with four channels an access (but the 16-channel
    # heads, whose rows of values to mix in start anywhere), the others a channel a thread
    from ginfer_b200 import ops
    g = torch.Generator().manual_seed(D + rot)
    T, slots = 9, 40
    cols = (nh + nkv) * D + nkv * Vd
    ld = cols + (-cols % 8)
    qkv = (torch.randn(T, ld, generator=g) * 2).to(dtype)
    vf = torch.randn(T, nkv * Vd + (3 if D == 16 else 4), generator=g).to(dtype)
    qw, kw = torch.rand(nh * D, generator=g) + 0.5, torch.rand(nkv * D, generator=g) + 0.5
    freqs = torch.rand(rot // 2, generator=g)
    pos = torch.randint(0, 900, (T,), generator=g).int()
    slot = torch.randperm(slots, generator=g)[:T].int()
    lam = torch.tensor([0.37])
    kp = torch.zeros(slots, nkv, D, dtype=dtype).cuda()
    vp = torch.zeros(slots, nkv, Vd, dtype=dtype).cuda()
    dev = qkv.clone().cuda()
    ops.qk_wide_prepare(dev, nh, nkv, D, Vd, nh * D, (nh + nkv) * D, qw.cuda(), kw.cuda(), 1e-5,
                        freqs.cuda(), rot, pos.cuda(), slot.cuda(), kp, vp,
                        vf.cuda()[:, :nkv * Vd], lam.cuda())
    x = qkv.double()
    q = plain.rms_norm(x[:, :nh * D], qw.double(), 1e-5).reshape(T, nh, D)
    k = plain.rms_norm(x[:, nh * D:(nh + nkv) * D], kw.double(), 1e-5).reshape(T, nkv, D)
    half = rot // 2
    for t in range(T):
        a = (pos[t].float() * freqs).double()            # the angle is a 32-bit product
        for y in (q, k):
            u, v = y[t, :, :half].clone(), y[t, :, half:rot].clone()
            y[t, :, :half] = u * torch.cos(a) - v * torch.sin(a)
            y[t, :, half:rot] = v * torch.cos(a) + u * torch.sin(a)
    v = 0.63 * x[:, (nh + nkv) * D:cols] + 0.37 * vf.double()[:, :nkv * Vd]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(dev[:, :nh * D].double().cpu(), q.reshape(T, -1), atol=tol, rtol=tol)
    assert torch.allclose(kp[slot.long()].double().cpu(), k, atol=tol, rtol=tol)
    assert torch.allclose(vp[slot.long()].double().cpu().reshape(T, -1), v, atol=tol, rtol=tol)
    assert torch.equal(dev[:, nh * D:].cpu(), qkv[:, nh * D:])      # k and v stay as projected
    untouched = [s for s in range(slots) if s not in set(slot.tolist())]
    assert float(kp[untouched].abs().max()) == 0.0 and float(vp[untouched].abs().max()) == 0.0


def _paged(keys, page, width, heads, dtype, g):
    npages = -(-keys // page)
    order = torch.randperm(npages + 3, generator=g)[:npages]
    vals = torch.randn(keys, heads, width, generator=g)
    pages = torch.zeros(npages + 3, page, heads, width)
    for j in range(keys):
        pages[order[j // page], j % page] = vals[j]
    return vals, pages.to(dtype).cuda(), order


@pytest.mark.parametrize("span", [-37, -16, -1, -64, 23, 0])
@pytest.mark.parametrize("hd, vd", [(16, 16), (24, 40), (64, 64)])
def test_plain_attention_sees_its_chunk_and_nothing_else(span, hd, vd):
    """Every row of a prompt and single decoded rows, keys and values of different widths, pages in
    shuffled order: against softmax over exactly the keys the mask allows."""
    from ginfer_b200 import ops
    g = torch.Generator().manual_seed(hd + span)
    nh, nkv, keys, page = 4, 2, 150, 8
    k, kp, order = _paged(keys, page, hd, nkv, torch.float32, g)
    g2 = torch.Generator().manual_seed(7)
    v = torch.randn(keys, nkv, vd, generator=g2)
    vp = torch.zeros(kp.shape[0], page, nkv, vd)
    for j in range(keys):
        vp[order[j // page], j % page] = v[j]
    vp = vp.cuda()
    q = torch.randn(keys, nh * hd, generator=g) * 2
    table = order.int().cuda()[None, :]
    for rows in (list(range(keys)), [keys - 1], [36, 37, 74, 111]):
        T = len(rows)
        out = ops.paged_attention_simt(
            q[rows].cuda().contiguous(), (kp, vp), table,
            torch.zeros(T, dtype=torch.int32, device="cuda"),
            torch.tensor(rows, dtype=torch.int32, device="cuda"), nh, nkv, hd, 0.3, span, page,
            vd=vd).cpu().reshape(T, nh, vd)
        for i, p in enumerate(rows):
            lo = max(0, p - span + 1) if span > 0 else (p // -span * -span if span < 0 else 0)
            for n in range(nh):
                s = (k[lo:p + 1, n // 2] @ q[p].reshape(nh, hd)[n]).double() * 0.3
                want = torch.softmax(s, 0) @ v[lo:p + 1, n // 2].double()
                assert torch.allclose(out[i, n].double(), want, atol=1e-4), (p, n)


@pytest.mark.parametrize("H, G, D, Vd, per_channel", [(2, 1, 12, 20, True), (3, 3, 10, 7, True),
                                                      (4, 2, 64, 40, False), (2, 2, 130, 9, True),
                                                      (1, 1, 33, 33, False)])
def test_recurrence_keeps_a_far_token_and_forgets_by_its_decays(H, G, D, Vd, per_channel):
    """With decays of one a value written at the first token under a key that no later token uses
    is read back hundreds of tokens later, in one portion, token by token or in uneven portions;
    with a decay below one on a head it fades by exactly that factor."""
    from ginfer_b200.ops import decay
    T = 300
    g0 = torch.Generator().manual_seed(D)
    k = torch.zeros(T, G, D)
    k[0, :, 0] = 1.0
    for t in range(1, T):
        k[t, :, 1 + t % (D - 1)] = 1.0
    q = torch.zeros(T, G, D)
    q[:, :, 0] = 1.0
    v = torch.randn(T, H, Vd, generator=g0)
    for rate in (1.0, 0.99):
        gt = torch.ones(T, H, D if per_channel else 1)
        gt[:, H - 1] = rate
        want = v[0].clone()
        want[H - 1] *= rate ** (T - 1)
        for cut in ([T], [1] * T, [7, 2, 100, 1, 190]):
            state = torch.zeros(3, H * D * Vd + 11, device="cuda")
            ctx = _Ctx()
            ctx.num_seqs = 1
            ctx.slot_ids = torch.tensor([1], dtype=torch.int32, device="cuda")
            at, last = 0, None
            for n in cut:
                ctx.cu_seqlens_q = torch.tensor([0, n], dtype=torch.int32, device="cuda")
                ctx.max_q_len = n
                sl = slice(at, at + n)
                last = decay.recurrence(q[sl].reshape(n, -1).cuda(), k[sl].reshape(n, -1).cuda(),
                                        v[sl].reshape(n, -1).cuda(), gt[sl].reshape(n, -1).cuda(),
                                        state, ctx, H, G, D, Vd)
                at += n
            assert torch.allclose(last[-1].cpu().reshape(H, Vd), want, atol=1e-4), (rate, cut[:3])
            assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0
            assert float(state[1, H * D * Vd:].abs().max()) == 0.0


@pytest.mark.parametrize("B, H, G, D, Vd, per_channel", [(40, 8, 4, 24, 36, True), (3, 2, 2, 130, 9, False),
                                                         (50, 6, 1, 64, 32, False), (2, 3, 3, 48, 64, True)])
def test_recurrence_batches_against_a_loop(B, H, G, D, Vd, per_channel):
    """Many requests of unequal lengths in one launch (both widths of the kernel), states in
    shuffled slots, factors on the keys and a skip weight, against a loop in float64."""
    from ginfer_b200.ops import decay
    g0 = torch.Generator().manual_seed(B)
    lens = [1 + (7 * b) % 5 for b in range(B)] if B > 3 else [70 + 9 * b for b in range(B)]
    T = sum(lens)
    q = torch.randn(T, G * D, generator=g0) / D ** 0.5
    k = torch.randn(T, G * D, generator=g0) / D ** 0.5
    v = torch.randn(T, H * Vd, generator=g0)
    gD = D if per_channel else 1
    gt = torch.rand(T, H * gD, generator=g0) * 0.5 + 0.5
    c = torch.rand(T, H, generator=g0) + 0.2
    skip = torch.randn(H, generator=g0)
    slots = torch.randperm(B + 3, generator=g0)[:B]
    state0 = torch.randn(B + 3, H * D * Vd + 5, generator=g0)
    state = state0.clone().cuda()
    ctx = _Ctx()
    ctx.num_seqs, ctx.max_q_len = B, max(lens)
    ctx.slot_ids = slots.int().cuda()
    cu = torch.tensor([0] + lens).cumsum(0)
    ctx.cu_seqlens_q = cu.int().cuda()
    # operands as strided views of wider rows, as the mixers hand them over
    wide = torch.cat([q, k, v], dim=1).cuda()
    o = decay.recurrence(wide[:, :G * D], wide[:, G * D:2 * G * D], wide[:, 2 * G * D:], gt.cuda(),
                         state, ctx, H, G, D, Vd, k_scale=c.cuda(), skip=skip.cuda()).cpu()
    per = H // G
    for b in range(B):
        S = state0[slots[b], :H * D * Vd].double().reshape(H, D, Vd).clone()
        for t in range(int(cu[b]), int(cu[b + 1])):
            for n in range(H):
                kt = k[t].reshape(G, D)[n // per].double()
                qt = q[t].reshape(G, D)[n // per].double()
                vt = v[t].reshape(H, Vd)[n].double()
                S[n] = gt[t].reshape(H, gD)[n].double()[:, None] * S[n] + \
                    float(c[t, n]) * torch.outer(kt, vt)
                want = S[n].T @ qt + float(skip[n]) * vt
                assert torch.allclose(o[t].reshape(H, Vd)[n].double(), want, atol=2e-4)
        got = state[slots[b]].cpu()
        assert torch.allclose(got[:H * D * Vd].double(), S.reshape(-1), atol=2e-4)
        assert torch.equal(got[H * D * Vd:], state0[slots[b], H * D * Vd:])
    untouched = [s for s in range(B + 3) if s not in set(slots.tolist())]
    assert torch.equal(state[untouched].cpu(), state0[untouched])


@pytest.mark.parametrize("taps, cut", [(4, [50]), (4, [1] * 12), (5, [2, 2, 3, 1, 30]), (2, [7, 1, 9]),
                                       (1, [5, 5])])
def test_convolution_step_sizes_and_the_slots_last_inputs(taps, cut):
    """The state-space layer's preparation in portions shorter than the convolution reaches,
    against the whole sequence convolved at once."""
    from ginfer_b200.ops import decay
    g0 = torch.Generator().manual_seed(taps)
    H, CH, T = 3, 37, sum(cut)
    ld = 8 + CH + H + 5
    proj = torch.randn(T, ld, generator=g0)
    w, b = torch.randn(CH, taps, generator=g0), torch.randn(CH, generator=g0)
    dt_bias, A_log = torch.randn(H, generator=g0), torch.randn(H, generator=g0)
    want = plain.silu(plain.causal_conv(proj[:, 8:8 + CH].double(), w.double(), b.double()))
    dt = plain.softplus(proj[:, 8 + CH:8 + CH + H].double() + dt_bias.double())
    S0 = 11
    state = torch.zeros(4, S0 + (taps - 1) * CH, device="cuda")
    ctx = _Ctx()
    ctx.num_seqs = 1
    ctx.slot_ids = torch.tensor([2], dtype=torch.int32, device="cuda")
    at = 0
    for n in cut:
        ctx.cu_seqlens_q = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        ctx.seq_of_token = torch.zeros(n, dtype=torch.int32, device="cuda")
        xbc, rates = decay.ssd_prepare(proj[at:at + n].cuda(), 8, 8 + CH, w.cuda(), b.cuda(),
                                       dt_bias.cuda(), A_log.cuda(), state, ctx, H, CH, taps, S0)
        assert torch.allclose(xbc.double().cpu(), want[at:at + n], atol=1e-5)
        assert torch.allclose(rates[:, H:].double().cpu(), dt[at:at + n], atol=1e-5)
        assert torch.allclose(rates[:, :H].double().cpu(),
                              torch.exp(-torch.exp(A_log.double()) * dt[at:at + n]), atol=1e-5)
        at += n
    assert float(state[:, :S0].abs().max()) == 0.0


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
# a warp a group; a block a group with four channels an access, and with one
@pytest.mark.parametrize("groups,gs", [(3, 20), (2, 520), (1, 1100), (2, 4096), (2, 522)])
def test_gated_norm_both_orders(act, groups, gs):
    from ginfer_b200.ops import decay
    g = torch.Generator(device="cuda").manual_seed(3)
    T = 21
    o = torch.randn(T, groups * gs, generator=g, device="cuda") * 2
    gate_wide = torch.randn(T, groups * gs + 8, generator=g, device="cuda")
    for gate in (gate_wide[:, 8:], gate_wide[:, 8:].to(act)):
        z = gate.double()
        sz = z * torch.sigmoid(z)
        w_full = torch.rand(groups * gs, generator=g, device="cuda") + 0.5
        w_one = torch.rand(gs, generator=g, device="cuda") + 0.5
        y = decay.gated_norm(o, gate, w_full, gs, True, 1e-4, act)
        t = (o.double() * sz).reshape(T, groups, gs)
        want = (t / torch.sqrt((t * t).mean(-1, keepdim=True) + 1e-4)).reshape(T, -1) * w_full.double()
        tol = 1e-5 if act == torch.float32 else 2e-2
        assert torch.allclose(y.double(), want, atol=tol, rtol=tol)
        y = decay.gated_norm(o, gate, w_one, gs, False, 1e-4, act)
        t = o.double().reshape(T, groups, gs)
        want = (t / torch.sqrt((t * t).mean(-1, keepdim=True) + 1e-4) * w_one.double()).reshape(T, -1) * sz
        assert torch.allclose(y.double(), want, atol=tol, rtol=tol)


def test_decays_of_gated_linear_attention():
    from ginfer_b200.ops import decay
    g = torch.Generator(device="cuda").manual_seed(5)
    T, HD, HV = 13, 24, 20
    proj = torch.randn(T, 2 * HD + HV + 8, generator=g, device="cuda")
    z = torch.randn(T, HD, generator=g, device="cuda") * 20           # far into both tails
    f = decay.gla_prepare(proj, z, HD, HV, 0.25, 16.0).double()
    assert torch.allclose(f[:, :HD], proj[:, :HD].double() * 0.25, atol=1e-6)
    assert torch.equal(f[:, HD:2 * HD].float(), proj[:, HD:2 * HD])
    assert torch.equal(f[:, 3 * HD:].float(), proj[:, 2 * HD:2 * HD + HV])
    want = torch.sigmoid(z.double()) ** (1 / 16.0)
    assert torch.allclose(f[:, 2 * HD:3 * HD], want, atol=1e-6, rtol=1e-5)
