"""The Zutazen design through the engine against the plain implementation, in
every way of cutting the work, on four small models that differ in every size and
constant (and from layer to layer): the order of the three kinds of mixer, layers
that run another layer's tensors, layers without feed-forward, windows from one
token to longer than any request, latent rows that take the tensor-core attention
kernels and rows that take the plain one, widths that are no multiple of eight.
The random weights are reshaped so that faults show: attention sharp enough that
a window one token off moves the result, slow and fast decays side by side,
routers that are far from uniform, biases that matter."""
import json
import os

import pytest
import torch

from conftest import random_tokens
from helpers import run_batch, run_chunks, run_schedule, run_tail_decoded, run_whole
from plain import zutazen as plain

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


def _ret(heads, dim, vdim, dims, base=10000.0, lo=0.8, hi=0.9995):
    return dict(heads=heads, dim=dim, vdim=vdim, rot={"base": base, "dims": dims},
                decay=[lo + (hi - lo) * i / max(heads - 1, 1) for i in range(heads)])


def _lat(heads, dim, rot_dim, vdim, kv_rank, scale, window, base=10000.0):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
             rot={"base": base, "dims": rot_dim})
    if window:
        m["mask"] = {"size": window}
    return m


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(kind, mixer, mlp, **kw):
    return dict(type=kind, mixer=mixer, mlp=mlp, **kw)


_P0 = _layer("latent_attention", _lat(4, 16, 8, 16, 24, 0.2, 7), {"kind": "dense", "ff": 96})
_Q0 = _layer("retention", _ret(2, 64, 32, 64, base=1e6), _moe(5, 1, 40))
_S1 = _layer("retention", _ret(5, 30, 18, 10), _moe(7, 3, 20))
ZUT = {
    # attention first; the last layer runs the first one's tensors; a window shorter than a page
    "P": dict(architecture="Zutazen", vocab=211, width=64, norm={"eps": 1e-5}, embedding={"scale": 0.5},
              layers=[_P0, _layer("retention", _ret(4, 16, 8, 8), _moe(6, 2, 24)),
                      _layer("rglru", dict(width=48, blocks=3, conv=3), None),
                      dict(_P0, weights_of=0)]),
    # latent rows of 64 (the tcgen05 prompt kernel), a window longer than a page, one tap, one part
    "Q": dict(architecture="Zutazen", vocab=300, width=128, norm={"eps": 3e-6}, embedding={"scale": 1.7},
              layers=[_Q0,
                      _layer("latent_attention", _lat(4, 64, 16, 64, 48, 0.1, 70, base=5e5), {"kind": "dense", "ff": 200}),
                      _layer("rglru", dict(width=128, blocks=1, conv=1), None),
                      dict(_Q0, weights_of=0)]),
    # rows of 128 after filling up, a window longer than every request, no window at all with rows
    # too wide for the tensor-core kernels, values narrower than keys, five taps
    "R": dict(architecture="Zutazen", vocab=160, width=96, norm={"eps": 1e-6}, embedding={"scale": 12.0},
              layers=[_layer("rglru", dict(width=60, blocks=5, conv=5), _moe(9, 3, 16)),
                      _layer("latent_attention", _lat(6, 24, 4, 8, 120, 0.15, 400), {"kind": "dense", "ff": 64}),
                      _layer("retention", _ret(6, 40, 12, 20), None),
                      _layer("latent_attention", _lat(2, 128, 32, 128, 110, 0.08, None), None)]),
    # nothing a multiple of eight; a window of one token (a token sees itself only); a later
    # layer's tensors used twice
    "S": dict(architecture="Zutazen", vocab=173, width=100, norm={"eps": 2e-5}, embedding={"scale": 1.0},
              layers=[_layer("latent_attention", _lat(3, 40, 6, 56, 21, 0.2, 1), {"kind": "dense", "ff": 52}),
                      _S1,
                      dict(_S1, weights_of=1),
                      _layer("rglru", dict(width=50, blocks=2, conv=2), {"kind": "dense", "ff": 52}),
                      _layer("latent_attention", _lat(5, 12, 2, 20, 30, 0.3, 65), None)]),
}
SEEDS = {"P": 11, "Q": 13, "R": 17, "S": 19}
LENGTHS = {"P": [1, 5, 70, 150], "Q": [2, 64, 129, 300], "R": [3, 131, 270], "S": [1, 66, 200]}


def _sharpen(tensors):
    g = torch.Generator().manual_seed(1)
    tensors = list(tensors)
    latent = {n[:-len("dkv")] for n, _ in tensors if n.endswith(".mix.dkv")}     # prefixes of latent mixers
    out = {}
    for name, t in tensors:
        f = t.float()
        if name.endswith(".lam"):
            f = torch.linspace(-6.0, 1.0, f.numel())           # channels that keep and channels that forget
        elif name.endswith(".conv"):
            f = torch.randn(f.shape, generator=g) * 0.6
        elif name.endswith(".router"):
            f = f * 10.0
        elif name.endswith(".mix.dkv") or (name.endswith(".mix.q") and name[:-1] in latent):
            f = f * 6.0                                         # sharp attention: single keys carry a row
        elif name == "embed":
            f = f * 10.0
        elif name.endswith(".mix.g") or name.endswith(".mix.y") or name.endswith(".mix.x"):
            f = f * 5.0
        elif name.endswith(".mix.o"):
            f = f * 3.0
        elif name.endswith(".mix.uk"):
            f = f * 20.0
        elif name.endswith(".mix.uv"):
            f = f * 10.0
        elif name.endswith(".ra") or name.endswith(".ri"):
            f = f * 20.0
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
    base = tmp_path_factory.mktemp("zutazen")
    out = {}
    for name, cfg in ZUT.items():
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
    """Models on which a window one token off, a lost rotation, a lost decay, a lost tail,
    bias, gate or embedding scale shows in the logits."""
    _d, cfg, w = models["P"]
    toks = random_tokens(60, cfg["vocab"], 1)
    full = plain.logits(w, cfg, toks)

    def moved(cfg2=None, w2=None, name="P", t=toks, ref=None):
        """The largest change of a logit, as a share of the logits' spread."""
        _d2, c0, w0 = models[name]
        ref = plain.logits(w0, c0, t) if ref is None else ref
        return float((plain.logits(w2 or w0, cfg2 or c0, t) - ref).abs().max() / ref.std())

    def edit(name, fn):
        c = json.loads(json.dumps(models[name][1]))
        fn(c)
        return c

    def window(size):
        def fn(c):
            for i in (0, 3):
                c["layers"][i]["mixer"]["mask"]["size"] = size
        return fn
    assert moved(edit("P", window(8)), ref=full) > 0.2 and moved(edit("P", window(6)), ref=full) > 0.2
    tq = random_tokens(150, models["Q"][1]["vocab"], 2)
    for size in (69, 71):
        assert moved(edit("Q", lambda c: c["layers"][1]["mixer"]["mask"].update(size=size)), name="Q", t=tq) > 0.2

    def no_rot(c):
        c["layers"][1]["mixer"]["rot"]["dims"] = 0
    assert moved(edit("P", no_rot), ref=full) > 0.2

    def decay(c):
        c["layers"][1]["mixer"]["decay"] = [0.5] * 4
    assert moved(edit("P", decay), ref=full) > 0.2
    assert moved(edit("P", lambda c: c["embedding"].update(scale=0.6)), ref=full) > 0.2
    tail_off = {k: v.clone() for k, v in w.items()}
    tail_off["l2.mix.conv"][:, :-1] = 0
    assert moved(w2=tail_off, ref=full) > 0.2
    assert moved(w2={k: (v * 0 if k.endswith(".b") else v) for k, v in w.items()}, ref=full) > 0.2
    assert moved(w2={k: (v * 0 if k.endswith("mix.g") else v) for k, v in w.items()}, ref=full) > 0.2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ZUT))
def test_each_request_alone_and_whole(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    for i, n in enumerate(LENGTHS[name]):
        toks = random_tokens(n, ZUT[name]["vocab"], 100 + i)
        assert_close(run_whole(eng, toks), oracle(name, toks), dtype, f"{name} whole, {n} tokens")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.tokens_held() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ZUT))
def test_prefill_against_token_by_token(engines, oracle, name, dtype):
    """The tail decoded across a window's edge and a page's; then everything but the first
    token decoded, so that every window edge is passed in single steps too."""
    eng = engines(name, dtype)
    n = LENGTHS[name][-1]
    toks = random_tokens(n, ZUT[name]["vocab"], 200)
    assert_close(run_tail_decoded(eng, toks, tail=40), oracle(name, toks), dtype, f"{name} tail")
    short = toks[:90]
    got = run_tail_decoded(eng, short, tail=89)
    assert_close(got, oracle(name, short), dtype, f"{name} decoded from the first token")
    if dtype == "float32":
        assert (got - run_whole(eng, short)).abs().max().item() < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ZUT))
def test_a_prompt_fed_in_portions(engines, oracle, name, dtype):
    """Portions of two tokens and of one (shorter than the convolution's tail and than the
    windows); portions that end one short of a page, on it and beyond it."""
    eng = engines(name, dtype)
    for i, chunks in enumerate([[2] * 12 + [1, 3], [63, 1, 64, 2], [60, 10, 70], [1, 1, 1, 2, 1, 30, 1, 1]]):
        toks = random_tokens(sum(chunks), ZUT[name]["vocab"], 700 + i)
        got = run_chunks(eng, toks, chunks)
        assert_close(got, oracle(name, toks), dtype, f"{name} portions {chunks}")
        if dtype == "float32":
            assert (got - run_whole(eng, toks)).abs().max().item() < 2e-5, chunks
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ZUT))
def test_unequal_batches_one_after_another(engines, oracle, name, dtype):
    """Three batches in a row on one engine: slots (and with them the recurrent layers'
    state rows) and pages of an earlier batch are used again by a later one, and within a
    batch the shorter requests end earlier."""
    eng = engines(name, dtype)
    V = ZUT[name]["vocab"]
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
    """A prompt of one token and 250 decoded ones: the first positions (a window that is
    not full yet, a convolution that still sees zeros, an empty state) and a long run of
    single steps across page boundaries, with a windowed store that gives pages back."""
    eng = engines(name, dtype)
    toks = random_tokens(251, ZUT[name]["vocab"], 400)
    assert_close(run_tail_decoded(eng, toks, tail=250), oracle(name, toks), dtype, "long decoding")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(ZUT))
def test_steps_that_mix_one_and_many_tokens(engines, oracle, name, dtype):
    eng = engines(name, dtype)
    lengths = [20 + 5 + 1 + 3 + 1, 9 + 1 + 1 + 1 + 1 + 1, 70 + 1 + 2]
    schedule = [{0: 20, 1: 9}, {0: 5, 1: 1}, {0: 1, 1: 1, 2: 70}, {0: 3, 1: 1, 2: 1},
                {0: 1, 1: 1, 2: 2}, {1: 1}]
    reqs = [random_tokens(n, ZUT[name]["vocab"], 720 + i) for i, n in enumerate(lengths)]
    got = run_schedule(eng, reqs, schedule)
    for i, r in enumerate(reqs):
        assert_close(got[i], oracle(name, r), dtype, f"{name} mixed steps, request {i}")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_steps_against_steps_launched_one_by_one(engines, oracle, dtype):
    """Both within the plain implementation's bar; in 32-bit equal to each other up to the
    rounding of sums taken in another order (a captured prompt step knows only an upper
    bound of the rows its sequences bring, so retention may go chunk by chunk there and row
    by row in the launched step)."""
    reqs = [random_tokens(n, ZUT["Q"]["vocab"], 740 + i) for i, n in enumerate((90, 33, 140))]
    outs = {}
    for use in (True, False):
        eng = engines("Q", dtype, use_graphs=use)
        outs[use] = run_batch(eng, reqs, [60, 30, 100])
    for i, r in enumerate(reqs):
        assert_close(outs[True][i], oracle("Q", r), dtype, f"captured, request {i}")
        assert_close(outs[False][i], oracle("Q", r), dtype, f"launched, request {i}")
        if dtype == "float32":
            assert torch.allclose(outs[True][i], outs[False][i], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("name", sorted(ZUT))
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
    """bin/trace_run on a Zutazen folder: a prompt, then single tokens, two requests."""
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
