"""The Mananex design through the engine against the plain implementation, in every
way of cutting the work, on four small models that differ in every size and constant
(and from layer to layer): dense, routed and absent feed-forwards in different orders,
groups of query heads, values narrower and wider than keys, rotations of a whole head,
of a part and none, windows from one token to longer than any request with none, few
and more than a page of kept first tokens, heads that take the tcgen05 and TMA attention
kernels, the mma.sync ones and the plain one, widths that are no multiple of eight.  The
random weights are reshaped so that faults show: attention sharp enough that a window
one token off or a lost first token moves the result, sinks that matter, forget gates
that keep and that forget, routers that are far from uniform, gates away from a half."""
import json
import os

import pytest
import torch

from conftest import random_tokens
from helpers import run_batch, run_chunks, run_schedule, run_tail_decoded, run_whole
from plain import mananex as plain

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
ROW_BAR = 0.08


def assert_close(got, want, dtype, what=""):
    """32-bit: element by element, at 1e-4 + 1e-3 |want|.  bfloat16: a rounding that
    flips an expert or moves a sharp attention weight changes single rows visibly while
    the rows as a whole stay close; the bar is on the median and the upper quartile of
    the rows' differences (root mean square, mean taken off) as a share of the logits'
    spread.  A lost mechanism, a wrong page or a lost state moves every row after it by
    more than 0.3."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    if dtype == "float32":
        err = (got - want).abs()
        assert bool((err <= 1e-4 + 1e-3 * want.abs()).all()), (
            f"{what}: max err {float(err.max()):.3g} at {int(err.argmax())}")
        return
    d = got - want
    d = d - d.mean(dim=-1, keepdim=True)
    spread = float((want - want.mean(dim=-1, keepdim=True)).pow(2).mean().sqrt())
    rows = d.pow(2).mean(dim=-1).sqrt() / spread
    med, q3 = float(rows.median()), float(rows.quantile(0.75))
    assert med <= ROW_BAR and q3 <= 3 * ROW_BAR, (
        f"{what}: median row differs by {med:.3f} of the logits' spread, upper quartile {q3:.3f}, "
        f"worst {float(rows.max()):.3f} (row {int(rows.argmax())})")


def _left(heads, kv_heads, dim, vdim, scale, rot=None, mask=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if mask:
        m["mask"] = {"size": mask[0]}
        if mask[1] is not None:
            m["mask"]["keep_first"] = mask[1]
    return m


def _mix(left, right, ls, rs):
    return dict(left=left, right=dict(heads=right[0], dim=right[1], vdim=right[2]), left_scale=ls,
                right_scale=rs)


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(mixer, mlp):
    return dict(type="parallel", mixer=mixer, mlp=mlp)


MAN = {
    # groups of two query heads, a window shorter than a page with two kept tokens, then one of a
    # single token (a token sees itself and the first); routed first, a layer without feed-forward
    "P": dict(architecture="Mananex", vocab=211, width=64, norm={"eps": 1e-5}, layers=[
        _layer(_mix(_left(4, 2, 16, 16, 0.6, (10000.0, 8), (7, 2)), (2, 8, 16), 0.7, 1.3), _moe(6, 2, 24)),
        _layer(_mix(_left(2, 1, 32, 16, 0.5, (500.0, 32), (1, 1)), (4, 16, 8), 1.0, 0.5), None),
        _layer(_mix(_left(4, 4, 16, 32, 0.7, None, (9, 0)), (1, 24, 40), 1.2, 0.9), {"kind": "dense", "ff": 96})]),
    # heads of 64 (the tcgen05 prompt kernel, the TMA decode kernel from 64 pairs on): a window longer
    # than a page with five kept tokens; a second layer that keeps more than a page of first tokens
    "Q": dict(architecture="Mananex", vocab=300, width=128, norm={"eps": 3e-6}, layers=[
        _layer(_mix(_left(4, 4, 64, 64, 0.3, (1e6, 64), (70, 5)), (2, 64, 32), 0.9, 0.8), {"kind": "dense", "ff": 200}),
        _layer(_mix(_left(4, 1, 64, 64, 0.25, (1e4, 16), (130, 70)), (4, 32, 32), 0.5, 1.1), _moe(5, 1, 40))]),
    # values narrower and wider than keys, heads too wide or too odd for the tensor-core kernels, no
    # window, a window longer than every request, every expert chosen
    "R": dict(architecture="Mananex", vocab=160, width=96, norm={"eps": 1e-6}, layers=[
        _layer(_mix(_left(6, 3, 24, 8, 0.4, (1e5, 4), None), (3, 40, 12), 1.0, 1.0), _moe(3, 3, 16)),
        _layer(_mix(_left(2, 2, 40, 40, 0.3, (1e3, 40), (400, 3)), (6, 8, 16), 0.8, 0.9), None),
        _layer(_mix(_left(2, 1, 144, 16, 0.15, (1e4, 20), (33, None)), (2, 100, 24), 1.5, 0.3), {"kind": "dense", "ff": 64}),
        _layer(_mix(_left(3, 3, 16, 48, 0.5, None, (64, 64)), (2, 12, 20), 0.6, 0.6), _moe(9, 4, 8))]),
    # nothing a multiple of eight; one expert; a window of three that keeps one
    "S": dict(architecture="Mananex", vocab=173, width=100, norm={"eps": 2e-5}, layers=[
        _layer(_mix(_left(3, 3, 20, 28, 0.45, (1e4, 6), (3, 1)), (5, 12, 20), 0.9, 1.1), _moe(1, 1, 52)),
        _layer(_mix(_left(5, 1, 12, 12, 0.6, (50.0, 12), (65, 0)), (2, 30, 18), 1.1, 0.7), {"kind": "dense", "ff": 52})]),
}
SEEDS = {"P": 11, "Q": 13, "R": 17, "S": 19}
LENGTHS = {"P": [1, 5, 70, 150], "Q": [2, 64, 129, 300], "R": [3, 131, 270], "S": [1, 66, 200]}


def _sharpen(tensors):
    g = torch.Generator().manual_seed(1)
    out = {}
    for name, t in tensors:
        f = t.float()
        if name == "embed":
            f = f * 10.0
        elif name.endswith(".left.q") or name.endswith(".left.k"):
            f = f * 8.0                                         # sharp attention: single keys carry a row
        elif name.endswith(".left.sink"):
            f = f * 20.0
        elif name.endswith(".left.g") or name.endswith(".rg1") or name.endswith(".rg2"):
            f = f * 6.0
        elif name.endswith(".left.o") or name.endswith(".right.o") or name.endswith(".left.v"):
            f = f * 3.0
        elif name.endswith(".right.f"):
            f = f * 30.0                                        # channels that keep and channels that forget
        elif name.endswith(".right.q") or name.endswith(".right.v"):
            f = f * 5.0
        elif name.endswith(".router"):
            f = f * 10.0
        elif name.endswith(".lower"):
            f = torch.rand(f.shape, generator=g) * 0.9
        elif name.endswith(".dwa"):
            f = f * 3.0
        elif ".mlp.e" in name or name.endswith((".mlp.gate", ".mlp.up", ".mlp.down")):
            f = f * 5.0                                         # feed-forwards that weigh as much as the mixers
        elif name.endswith(".router.b"):
            f = f * 15.0
        elif name.endswith(".b"):
            f = f * 3.0
        out[name] = f.to(t.dtype)
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (folder, config dict, {tensor name: CPU tensor})."""
    import grout_b200.architectures  # noqa: F401
    from grout_b200.config import resolve_architecture
    from grout_b200.engine.model import expected_tensors
    from grout_b200.weights import random_tensors, write_safetensors
    base = tmp_path_factory.mktemp("mananex")
    out = {}
    for name, cfg in MAN.items():
        arch = resolve_architecture(cfg)
        exp = expected_tensors(arch.plan(arch.config_cls.from_dict(cfg)))
        w = _sharpen(random_tensors(exp, SEEDS[name]))
        folder = str(base / name)
        os.makedirs(folder)
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(cfg, fh)
        write_safetensors(os.path.join(folder, "model.safetensors"), list(w.items()))
        out[name] = (folder, cfg, w)
    return out


@pytest.fixture(scope="module")
def engines(models):
    from grout_b200.engine import Engine
    made = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in made:
            made[key] = Engine.load(models[name][0], dtype=dtype, max_tokens=4096, max_batch=8,
                                    max_seq_len=512, **kw)
        return made[key]
    return get


@pytest.fixture(scope="module")
def oracle(models):
    memo = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in memo:
            _d, cfg, w = models[name]
            memo[key] = plain.logits(w, cfg, list(tokens))
        return memo[key]
    return get


def test_the_sharpened_weights_do_what_they_are_for(models):
    """Models on which a window one token off, a lost kept token, a lost rotation, sink,
    gate, lower bound, bias or depth average shows in the logits."""
    def moved(name, t, cfg2=None, w2=None):
        """The largest change of a logit, as a share of the logits' spread."""
        _d, c0, w0 = models[name]
        ref = plain.logits(w0, c0, t)
        return float((plain.logits(w2 or w0, cfg2 or c0, t) - ref).abs().max() / ref.std())

    def edit(name, fn):
        c = json.loads(json.dumps(models[name][1]))
        fn(c)
        return c

    tp = random_tokens(60, MAN["P"]["vocab"], 1)
    tq = random_tokens(300, MAN["Q"]["vocab"], 2)      # longer than the second layer's window and kept tokens
    for size in (6, 8):
        assert moved("P", tp, edit("P", lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=size))) > 0.2
    for keep in (1, 3):
        assert moved("P", tp, edit("P", lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=keep))) > 0.2
    for size in (69, 71):
        assert moved("Q", tq, edit("Q", lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=size))) > 0.1
    for keep in (4, 6):
        assert moved("Q", tq, edit("Q", lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=keep))) > 0.1
    assert moved("P", tp, edit("P", lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=0))) > 0.2
    assert moved("P", tp, edit("P", lambda c: c["layers"][0]["mixer"].update(left_scale=0.8))) > 0.05
    w = models["P"][2]
    for part in (".sink", ".left.g", ".lower", ".f.b", ".rg1.b", "router.b", ".norm1"):
        assert moved("P", tp, w2={k: (v * 0 if k.endswith(part) else v) for k, v in w.items()}) > 0.1, part
    flat = {k: (torch.cat([v[:-1] * 0, v[-1:] * 0 + 1]) if k.endswith(".dwa") else v) for k, v in w.items()}
    assert moved("P", tp, w2=flat) > 0.2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(MAN))
def test_each_request_alone_and_whole(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    for i, n in enumerate(LENGTHS[name]):
        toks = random_tokens(n, MAN[name]["vocab"], 100 + i)
        assert_close(run_whole(eng, toks), oracle(name, toks), dtype, f"{name} whole, {n} tokens")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(MAN))
def test_prefill_against_token_by_token(engines, oracle, name, dtype):
    """The tail decoded across a window's edge and a page's; then everything but the first
    token decoded, so that every window edge and the end of the kept first tokens are passed
    in single steps too."""
    eng = engines(name, dtype)
    n = LENGTHS[name][-1]
    toks = random_tokens(n, MAN[name]["vocab"], 200)
    assert_close(run_tail_decoded(eng, toks, tail=40), oracle(name, toks), dtype, f"{name} tail")
    short = toks[:90]
    got = run_tail_decoded(eng, short, tail=89)
    assert_close(got, oracle(name, short), dtype, f"{name} decoded from the first token")
    if dtype == "float32":
        assert (got - run_whole(eng, short)).abs().max().item() < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(MAN))
def test_a_prompt_fed_in_portions(engines, oracle, name, dtype):
    """Portions of two tokens and of one (shorter than the windows and than the kept first
    tokens); portions that end one short of a page, on it and beyond it."""
    eng = engines(name, dtype)
    for i, chunks in enumerate([[2] * 12 + [1, 3], [63, 1, 64, 2], [60, 10, 70, 61], [1, 1, 1, 2, 1, 30, 1, 1]]):
        toks = random_tokens(sum(chunks), MAN[name]["vocab"], 700 + i)
        got = run_chunks(eng, toks, chunks)
        assert_close(got, oracle(name, toks), dtype, f"{name} portions {chunks}")
        if dtype == "float32":
            assert (got - run_whole(eng, toks)).abs().max().item() < 2e-5, chunks
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(MAN))
def test_unequal_batches_one_after_another(engines, oracle, name, dtype):
    """Three batches in a row on one engine: slots (and with them the linear attention's
    state rows) and pages of an earlier batch are used again by a later one, and within a
    batch the shorter requests end earlier."""
    eng = engines(name, dtype)
    V = MAN[name]["vocab"]
    plans = [[(5, 3), (11, 9), (17, 1)],
             [(1, 20), (7, 2), (30, 11), (64, 5), (130, 33), (200, 80)],
             [(65, 4), (2, 4), (128, 70)]]
    for b, plan in enumerate(plans):
        reqs = [random_tokens(p + d, V, 300 + 10 * b + i) for i, (p, d) in enumerate(plan)]
        got = run_batch(eng, reqs, [p for p, _ in plan])
        for i, r in enumerate(reqs):
            assert_close(got[i], oracle(name, r), dtype, f"{name} batch {b} request {i}")
            if dtype == "float32":
                assert (got[i] - run_whole(eng, r)).abs().max().item() < 2e-5, (b, i)
        eng.cache.check()
        assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_first_tokens_and_long_decoding(engines, oracle, name, dtype):
    """A prompt of one token and 330 decoded ones: the first positions (a window that is not
    full yet, kept tokens that are still inside it, an empty state) and a long run of single
    steps across page boundaries, with a windowed store that gives pages back but for those
    of the kept first tokens."""
    eng = engines(name, dtype)
    toks = random_tokens(331, MAN[name]["vocab"], 400)
    assert_close(run_tail_decoded(eng, toks, tail=330), oracle(name, toks), dtype, "long decoding")
    eng.cache.check()


def test_a_windowed_store_keeps_the_first_pages_and_gives_the_others_back(engines):
    eng = engines("Q", "float32")
    toks = random_tokens(500, MAN["Q"]["vocab"], 410)
    s = eng.open_sequence()
    eng.step([(s, toks)], [[0]])
    # layer 0: window 70, 5 kept (page 0 and the window's two or three pages); layer 1: window 130, 70
    # kept (pages 0 and 1 and the window's three or four)
    held = sorted(st.stores[0].pool.n_held for st in eng.cache.stores)
    assert held[0] <= 1 + 3 and held[1] <= 2 + 4 and held[0] >= 3 and held[1] >= 5, held
    eng.close_sequence(s)
    eng.cache.check()
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(MAN))
def test_steps_that_mix_one_and_many_tokens(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    lengths = [20 + 5 + 1 + 3 + 1, 9 + 1 + 1 + 1 + 1 + 1, 70 + 1 + 2]
    schedule = [{0: 20, 1: 9}, {0: 5, 1: 1}, {0: 1, 1: 1, 2: 70}, {0: 3, 1: 1, 2: 1},
                {0: 1, 1: 1, 2: 2}, {1: 1}]
    reqs = [random_tokens(n, MAN[name]["vocab"], 720 + i) for i, n in enumerate(lengths)]
    got = run_schedule(eng, reqs, schedule)
    for i, r in enumerate(reqs):
        assert_close(got[i], oracle(name, r), dtype, f"{name} mixed steps, request {i}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_steps_against_steps_launched_one_by_one(engines, oracle, dtype):
    reqs = [random_tokens(n, MAN["Q"]["vocab"], 740 + i) for i, n in enumerate((90, 33, 140))]
    outs = {}
    for use in (True, False):
        eng = engines("Q", dtype, use_graphs=use)
        outs[use] = run_batch(eng, reqs, [60, 30, 100])
    for i, r in enumerate(reqs):
        assert_close(outs[True][i], oracle("Q", r), dtype, f"captured, request {i}")
        assert_close(outs[False][i], oracle("Q", r), dtype, f"launched, request {i}")
        if dtype == "float32":
            assert torch.allclose(outs[True][i], outs[False][i], atol=1e-5, rtol=1e-4)


def test_many_sequences_take_the_tma_decode_kernel(models, oracle):
    """Sixteen sequences of four kv heads are 64 (sequence, kv head) pairs: decode steps of
    heads of 64 then run on the TMA kernel, over windows with kept first tokens."""
    from grout_b200.engine import Engine
    folder, cfg, _w = models["Q"]
    eng = Engine.load(folder, dtype="bfloat16", max_tokens=16 * 512, max_batch=16, max_seq_len=512)
    reqs = [random_tokens(150 + 7 * i, cfg["vocab"], 760 + i) for i in range(16)]
    got = run_batch(eng, reqs, [len(r) - 12 for r in reqs])
    for i in (0, 5, 15):
        assert_close(got[i], oracle("Q", reqs[i]), "bfloat16", f"request {i} of 16")
    eng.cache.check()


@pytest.mark.parametrize("name", sorted(MAN))
def test_greedy_generation_through_the_engine(models, name):
    """Engine.generate (its scheduler, cache and device sampler) against the plain
    loop, in 32-bit, where the argmax is the same token."""
    from grout_b200.engine import Engine
    folder, cfg, w = models[name]
    eng = Engine.load(folder, dtype="float32", max_tokens=2048, max_batch=3)
    prompts = [random_tokens(n, cfg["vocab"], 800 + i) for i, n in enumerate((1, 7, 30, 64, 5))]
    want = [plain.greedy_generate(w, cfg, p, 10) for p in prompts]
    outs = eng.generate(prompts, 10, ignore_eos=True)          # five requests on three slots
    assert [o.token_ids for o in outs] == want
    stop = want[1][3]
    outs = eng.generate(prompts, 10, stop_ids=[stop])
    assert [o.token_ids for o in outs] == [plain.greedy_generate(w, cfg, p, 10, stop_ids=(stop,))
                                           for p in prompts]
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


def test_generation_in_bfloat16_and_the_command_line(models, tmp_path):
    """bfloat16 generation runs through captured steps; its tokens are the plain
    loop's wherever the plain logits leave no doubt.  And the command line serves
    the design as it serves the others."""
    import subprocess
    import sys
    from conftest import ROOT
    from grout_b200.engine import Engine
    folder, cfg, w = models["Q"]
    eng = Engine.load(folder, dtype="bfloat16", max_tokens=2048, max_batch=4)
    prompt = random_tokens(70, cfg["vocab"], 820)
    got = eng.generate([prompt], 10, ignore_eos=True)[0].token_ids
    seq = list(prompt)
    for tok in got:
        row = plain.logits(w, cfg, seq, rows=[len(seq) - 1])[0]
        top2 = torch.topk(row, 2).values
        if float(top2[0] - top2[1]) > 0.1 * float(row.std()):
            assert tok == int(torch.argmax(row)), len(seq)
        seq.append(tok)
    out = tmp_path / "out.json"
    ids = ",".join(str(t) for t in prompt[:9])
    r = subprocess.run([sys.executable, "-m", "grout_b200", "--model", folder, "--prompt-ids", ids,
                        "--max-new-tokens", "6", "--ignore-eos", "--fp32", "--device-argmax",
                        "--output-json", str(out), "--quiet"], cwd=ROOT, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.load(open(out))["token_ids"] == plain.greedy_generate(w, cfg, prompt[:9], 6)


def test_trace_replay_serves_the_design(models, tmp_path):
    """bin/trace_run on a Mananex folder: a prompt, then single tokens, two requests."""
    import subprocess
    import sys
    import numpy as np
    from conftest import ROOT
    folder, cfg, w = models["P"]
    a, b = random_tokens(40, cfg["vocab"], 840), random_tokens(9, cfg["vocab"], 841)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:37], "want": [0, 36]},
                                     {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[37]], "want": []},
                                     {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[38]], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[39]], "want": [0]}], "end": ["a"]}]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    la, lb = plain.logits(w, cfg, a), plain.logits(w, cfg, b)
    want = {0: torch.stack([la[0], la[36], lb[7]]), 1: lb[8:9], 2: la[38:39], 3: la[39:40]}
    for i, wnt in want.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        assert_close(got, wnt, "float32", f"step {i}")
