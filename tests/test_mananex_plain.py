"""What needs no GPU of the Mananex design: its configuration and plan, the plain
implementation's reading of each mechanism against hand computation, and the cache's
bookkeeping for windows that keep a sequence's first tokens and for layers with two
needs."""
import json
import math

import pytest
import torch

from plain import mananex as plain

CFG = dict(architecture="Mananex", vocab=50, width=16, norm={"eps": 1e-5}, layers=[
    dict(type="parallel", mlp={"kind": "dense", "ff": 24}, mixer=dict(
        left=dict(heads=2, kv_heads=1, dim=8, vdim=4, scale=0.3, rot={"base": 100.0, "dims": 4},
                  mask={"size": 3, "keep_first": 1}),
        right=dict(heads=2, dim=4, vdim=6), left_scale=0.5, right_scale=2.0)),
    dict(type="parallel", mlp={"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 4, "top": 2}},
         mixer=dict(left=dict(heads=1, kv_heads=1, dim=4, vdim=4, scale=0.5),
                    right=dict(heads=1, dim=2, vdim=2), left_scale=1.0, right_scale=1.0)),
    dict(type="parallel", mlp=None, mixer=dict(
        left=dict(heads=2, kv_heads=2, dim=4, vdim=8, scale=0.5, mask={"size": 5}),
        right=dict(heads=1, dim=2, vdim=2), left_scale=1.0, right_scale=1.0))])


def _weights(cfg, seed=0):
    import grout_b200.architectures  # noqa: F401
    from grout_b200.config import resolve_architecture
    from grout_b200.engine.model import expected_tensors
    from grout_b200.weights import random_tensors
    arch = resolve_architecture(cfg)
    exp = expected_tensors(arch.plan(arch.config_cls.from_dict(cfg)))
    return exp, dict(random_tensors(exp, seed))


def test_configuration_names_every_problem():
    import grout_b200.architectures  # noqa: F401
    from grout_b200.config import ConfigError, MananexConfig, resolve_architecture
    assert resolve_architecture(CFG).name == "Mananex"
    MananexConfig.from_dict(CFG)
    bad = json.loads(json.dumps(CFG))
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 3          # two heads cannot share three
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 10      # more than a head has
    bad["layers"][1]["mlp"]["router"]["top"] = 5               # more than there are experts
    bad["layers"][2]["mixer"]["left"]["mask"] = {"size": 0}
    bad["layers"][2]["type"] = "serial"
    del bad["norm"]["eps"]
    with pytest.raises(ConfigError) as e:
        MananexConfig.from_dict(bad)
    assert len(e.value.problems) == 5, e.value.problems
    bad2 = json.loads(json.dumps(CFG))
    del bad2["layers"][0]["mixer"]["right"]
    bad2["layers"][1]["mixer"]["left_scale"] = "1"
    with pytest.raises(ConfigError) as e:
        MananexConfig.from_dict(bad2)
    assert len(e.value.problems) == 2, e.value.problems


def test_plan_reads_exactly_the_designs_tensors():
    exp, _w = _weights(CFG)
    shapes = {n: tuple(s.shape) for n, s in exp.items()}
    assert shapes["embed"] == (50, 16) and shapes["final.norm"] == (16,) and "head" not in shapes
    assert shapes["l0.mix.left.q"] == (16, 16) and shapes["l0.mix.left.k"] == (8, 16)
    assert shapes["l0.mix.left.v"] == (4, 16) and shapes["l0.mix.left.o"] == (16, 8)
    assert shapes["l0.mix.left.g"] == (2, 16) and shapes["l0.mix.left.sink"] == (2,)
    assert shapes["l0.mix.right.q"] == (8, 16) and shapes["l0.mix.right.f.b"] == (8,)
    assert shapes["l0.mix.right.lower"] == (8,) and shapes["l0.mix.right.v"] == (12, 16)
    assert shapes["l0.mix.right.norm"] == (6,) and shapes["l0.mix.right.o"] == (16, 12)
    assert shapes["l0.mlp.gate.b"] == (24,) and shapes["l0.mlp.down"] == (16, 24)
    assert shapes["l1.mlp.router"] == (4, 16) and shapes["l1.mlp.router.b"] == (4,)
    assert shapes["l1.mlp.e3.down"] == (16, 8)
    assert shapes["l0.rg1"] == (16, 16) and shapes["l0.rg2.b"] == (16,)
    assert "l2.rg2" not in shapes and "l2.rg1" in shapes and not any(n.startswith("l2.mlp") for n in shapes)
    assert [shapes[f"l{i}.dwa"] for i in range(3)] == [(2,), (3,), (4,)]


def test_plan_needs_of_the_cache():
    import grout_b200.architectures  # noqa: F401
    from grout_b200.cache import KVSpec, SideBySideSpec, StateSpec
    from grout_b200.config import resolve_architecture
    from grout_b200.engine.model import Model
    from grout_b200.parts import BuildContext
    arch = resolve_architecture(CFG)
    model = Model(arch.plan(arch.config_cls.from_dict(CFG)), BuildContext(torch.float32, torch.device("cpu")))
    specs = [b.cache_spec() for b in model.blocks]
    assert specs[0] == SideBySideSpec((KVSpec(1, 8, 3, keep_first=1), StateSpec((2 * 4 * 6,))))
    assert specs[1] == SideBySideSpec((KVSpec(1, 4, None), StateSpec((4,))))
    assert specs[2].specs[0] == KVSpec(2, 8, 5)            # a window without kept tokens; rows as wide as the values
    assert len(model.cache_layout().groups) == 3


def test_a_windowed_store_keeps_the_pages_of_the_first_tokens():
    from grout_b200.cache import CacheLayout, KVSpec, SequenceCache, SideBySideSpec, StateSpec
    spec = SideBySideSpec((KVSpec(1, 8, 100, keep_first=70), StateSpec((4,))))
    cache = SequenceCache(CacheLayout.from_specs([spec, KVSpec(1, 8, 100)]), max_tokens=64 * 40, max_slots=4,
                          max_seq_len=2048, dtype=torch.float32, device="cpu", allocate=False)
    s = cache.open()
    held = []
    for n in (64, 64, 64, 200, 1, 300):
        cache.reserve(s, n)
        cache.advance(s, n)
        held.append([st.tokens_held() // 64 for st in cache.stores])
        cache.check()
    # 693 tokens: positions 594.. are in reach of the next query: pages 9 and 10, and with kept tokens pages 0, 1
    assert held[-1] == [4, 2], held
    assert held[2] == [3, 2]            # 192 tokens: page 0 is out of the window, but kept in the first store
    pages = cache.stores[0].stores[0].pages_of[s]
    assert pages[0] is not None and pages[1] is not None and pages[2] is None and pages[-1] is not None
    other = cache.open()
    cache.reserve(other, 130)
    cache.close(s)
    cache.check()
    assert [st.tokens_held() // 64 for st in cache.stores] == [3, 3]
    cache.close(other)
    assert cache.tokens_held() == 0


def test_visibility_is_the_window_or_the_first_tokens():
    assert plain.visible(10, 10, 1, 0) and not plain.visible(10, 9, 1, 0) and not plain.visible(3, 4, 9, 9)
    assert plain.visible(10, 8, 3, 0) and not plain.visible(10, 7, 3, 0)
    assert plain.visible(10, 1, 3, 2) and not plain.visible(10, 2, 3, 2) and plain.visible(10, 0, 3, 2)
    assert plain.visible(99, 0, None, 0)
    pos = list(range(40, 75))
    for size, keep in ((1, 0), (7, 2), (7, 50), (None, 3), (100, 0)):
        want = torch.tensor([[plain.visible(i, j, size, keep) for j in pos] for i in pos])
        assert torch.equal(plain.visibility(pos, size, keep), want)


def test_rotation_turns_neighbours_and_keeps_lengths():
    x = torch.arange(24, dtype=torch.float64).view(2, 1, 12) + 1
    y = plain.rotate_neighbours(x, [0, 3], 100.0, 4)
    assert torch.equal(y[0], x[0]) and torch.equal(y[1, 0, 4:], x[1, 0, 4:])
    a0, a1 = 3 * 1.0, 3 * 100.0 ** -0.5
    u, v = float(x[1, 0, 0]), float(x[1, 0, 1])
    assert math.isclose(float(y[1, 0, 0]), u * math.cos(a0) - v * math.sin(a0))
    assert math.isclose(float(y[1, 0, 1]), v * math.cos(a0) + u * math.sin(a0))
    u, v = float(x[1, 0, 2]), float(x[1, 0, 3])
    assert math.isclose(float(y[1, 0, 2]), u * math.cos(a1) - v * math.sin(a1))
    assert math.isclose(float(y[1, 0, 0] ** 2 + y[1, 0, 1] ** 2), float(x[1, 0, 0] ** 2 + x[1, 0, 1] ** 2))


def test_attention_by_hand_sink_gate_and_kept_token():
    """One head, values of one element, keys equal to the queries' direction: three tokens, a window of
    one that keeps the first token."""
    w = {"q": torch.tensor([[1.0]]), "k": torch.tensor([[1.0]]), "v": torch.tensor([[1.0]]),
         "o": torch.tensor([[1.0]]), "sink": torch.tensor([math.log(2.0)]), "g": torch.tensor([[0.0]])}
    m = dict(heads=1, kv_heads=1, dim=1, vdim=1, scale=1.0, mask={"size": 1, "keep_first": 1})
    h = torch.tensor([[1.0], [2.0], [0.0]], dtype=torch.float64)
    out = plain.windowed_attention(h, [0, 1, 2], w, m)
    # token 0: sees itself: e / (e + 2) * 1, gate 0.5
    assert math.isclose(float(out[0]), 0.5 * math.e / (math.e + 2))
    # token 1: scores 2 * 1 (token 0, kept) and 2 * 2 (itself)
    e2, e4 = math.exp(2), math.exp(4)
    assert math.isclose(float(out[1]), 0.5 * (e2 * 1 + e4 * 2) / (e2 + e4 + 2))
    # token 2: q = 0: scores 0 for token 0 (kept) and itself; token 1 is outside the window
    assert math.isclose(float(out[2]), 0.5 * (1 * 1 + 1 * 0) / (1 + 1 + 2))


def test_forget_gate_by_hand():
    """f at its lower bound writes 1 - low of the value and keeps low of the state."""
    w = {"q": torch.tensor([[1.0]]), "f": torch.tensor([[0.0]]), "f.b": torch.tensor([-50.0]),
         "lower": torch.tensor([0.25]), "v": torch.tensor([[1.0], [2.0]]), "norm": torch.ones(2),
         "o": torch.eye(2)}
    h = torch.tensor([[1.0], [1.0]], dtype=torch.float64)
    out, S = plain.forgetful_linear_attention(h, w, dict(heads=1, dim=1, vdim=2), 0.0)
    # S_1 = 0.75 [1, 2]; S_2 = 0.25 S_1 + 0.75 [1, 2] = 0.9375 [1, 2]; o is normalised over the two values
    assert torch.allclose(S[0, 0], torch.tensor([0.9375, 1.875], dtype=torch.float64))
    r = math.sqrt((1 + 4) / 2)
    assert torch.allclose(out[1], torch.tensor([1 / r, 2 / r], dtype=torch.float64))
    # the sigmoid fully open: f = 1, nothing is written
    w["f.b"] = torch.tensor([50.0])
    _out, S = plain.forgetful_linear_attention(h, w, dict(heads=1, dim=1, vdim=2), 0.0)
    assert float(S.abs().max()) < 1e-12


def test_router_weighs_the_chosen_by_their_own_softmax():
    w = {"m.router": torch.tensor([[1.0], [3.0], [2.0], [-1.0]]), "m.router.b": torch.tensor([0.0, 0.0, 0.0, 5.0])}
    idx, wt = plain.route(torch.tensor([[1.0]], dtype=torch.float64), w, "m.", 2)
    assert idx.tolist() == [[3, 1]]                              # the bias lifts the last expert to the top
    assert math.isclose(float(wt[0, 0]), math.exp(4) / (math.exp(4) + math.exp(3)))
    assert math.isclose(float(wt.sum()), 1.0)


def test_depth_average_and_the_norm_around_zero():
    hist = [torch.full((2, 3), 1.0, dtype=torch.float64), torch.full((2, 3), 10.0, dtype=torch.float64)]
    assert torch.allclose(plain.depth_average(hist, torch.tensor([0.5, 2.0])), torch.full((2, 3), 20.5, dtype=torch.float64))
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = plain.norm_around_zero(x, torch.tensor([0.0, 1.0]), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3 / r, 8 / r]], dtype=torch.float64))


def test_the_whole_model_is_causal_and_uses_every_tensor():
    exp, w = _weights(CFG, seed=3)
    toks = [3, 14, 15, 9, 2, 6, 5, 35, 8, 9, 7, 9]
    full = plain.logits(w, CFG, toks)
    assert tuple(full.shape) == (12, 50)
    assert torch.allclose(plain.logits(w, CFG, toks[:7]), full[:7], atol=1e-12)
    unused = []
    for name in exp:
        w2 = dict(w)
        w2[name] = w[name].float() * 0.5 + 0.25
        if float((plain.logits(w2, CFG, toks) - full).abs().max()) <= 1e-9:
            unused.append(name)
    # only an expert that no token of these twelve chose may go unnoticed
    assert all(".mlp.e" in n for n in unused) and len({n.split(".")[2] for n in unused}) <= 2, unused
