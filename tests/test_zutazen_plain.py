"""The Zutazen design without a GPU: its configuration, its plan (tensor names,
the order of layer runs, which runs share tensors) and hand computations that pin
the plain implementation's reading of each mechanism."""
import math

import pytest
import torch

from plain import zutazen as plain

RET = dict(heads=2, dim=8, vdim=6, decay=[0.9, 0.99], rot={"base": 100.0, "dims": 4})
REC = dict(width=12, blocks=3, conv=3)
LAT = dict(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=10, scale=0.3, rot={"base": 50.0, "dims": 4},
           mask={"size": 5})
MOE = {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 5, "top": 2}}
CFG = dict(architecture="Zutazen", vocab=50, width=24, norm={"eps": 1e-5}, embedding={"scale": 1.7},
           layers=[{"type": "retention", "mixer": RET, "mlp": {"kind": "dense", "ff": 40}},
                   {"type": "latent_attention", "mixer": LAT, "mlp": MOE},
                   {"type": "rglru", "mixer": REC, "mlp": None},
                   {"type": "latent_attention", "mixer": LAT, "mlp": MOE, "weights_of": 1}])


def test_configuration_reads_and_refuses():
    import grout_b200.architectures  # noqa: F401
    from grout_b200.config import ConfigError, resolve_architecture
    arch = resolve_architecture(CFG)
    cfg = arch.config_cls.from_dict(CFG)
    assert arch.name == "Zutazen" and cfg.weights_layer(3) == 1 and cfg.weights_layer(2) == 2
    bad = dict(CFG, layers=[dict(CFG["layers"][0], type="conv")])
    with pytest.raises(ConfigError, match="type"):
        arch.config_cls.from_dict(bad)
    bad = dict(CFG, layers=CFG["layers"][:3] + [dict(CFG["layers"][3], weights_of=3)])
    with pytest.raises(ConfigError, match="weights_of"):
        arch.config_cls.from_dict(bad)
    bad = dict(CFG, layers=[dict(CFG["layers"][0], mixer=dict(RET, decay=[0.9]))])
    with pytest.raises(ConfigError, match="decay"):
        arch.config_cls.from_dict(bad)
    bad = dict(CFG, layers=[dict(CFG["layers"][2], mixer=dict(REC, blocks=5))])
    with pytest.raises(ConfigError, match="equal parts"):
        arch.config_cls.from_dict(bad)
    bad = dict(CFG, layers=[dict(CFG["layers"][1], mixer=dict(LAT, rot={"base": 50.0, "dims": 2}))])
    with pytest.raises(ConfigError, match="rot_dim"):
        arch.config_cls.from_dict(bad)
    with pytest.raises(ConfigError, match="embedding"):
        arch.config_cls.from_dict({k: v for k, v in CFG.items() if k != "embedding"})


def test_plan_names_tensors_and_orders_layer_runs():
    import grout_b200.architectures  # noqa: F401
    from grout_b200.cache.spec import KVSpec, StateSpec
    from grout_b200.config import resolve_architecture
    from grout_b200.engine.model import Model, expected_tensors
    from grout_b200.parts.base import BuildContext
    arch = resolve_architecture(CFG)
    plan = arch.plan(arch.config_cls.from_dict(CFG))
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 1]          # the fourth run uses layer 1's tensors
    assert all(e.cache_of is None for e in plan.schedule)            # on a cache of its own
    exp = expected_tensors(plan)
    assert exp["l0.mix.q"].shape == (16, 24) and exp["l0.mix.g"].shape == (12, 24)
    assert exp["l0.mlp.gate.b"].shape == (40,) and exp["l0.mlp.down.b"].shape == (24,)
    assert exp["l1.mix.q"].shape == (36, 24) and exp["l1.mix.dkv"].shape == (14, 24)
    assert exp["l1.mix.uk"].shape == (24, 10) and exp["l1.mix.uv"].shape == (18, 10)
    assert exp["l1.mix.dkv.norm"].shape == (10,) and exp["l1.mlp.router"].shape == (5, 24)
    assert exp["l2.mix.ra"].shape == (3, 4, 4) and exp["l2.mix.conv"].shape == (12, 3)
    assert exp["l2.mix.ri.b"].shape == (3, 4) and exp["l2.mix.o"].shape == (24, 12)
    assert "l2.norm2" not in exp and "l1.mlp.correction" not in exp
    assert not any(n.startswith("l3.") for n in exp)
    specs = [Model(plan, BuildContext(torch.float32, torch.device("cpu"))).blocks[e.layer].cache_spec()
             for e in plan.schedule]
    assert specs[0] == StateSpec((2 * 8 * 6,), torch.float32) and specs[2] == StateSpec((3 * 12,), torch.float32)
    assert specs[1] == KVSpec(1, 14, 5, values_in_keys=True) == specs[3]


def test_retention_by_hand():
    """o_t = sum_{s <= t} decay^(t - s) (q_t . k_s) v_s, no softmax and no denominator."""
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(6, 4, generator=g), torch.randn(6, 4, generator=g)
    v = torch.randn(6, 3, generator=g)
    o, S = plain.retention_head(q, k, v, 0.8)
    for t in range(6):
        want = sum(0.8 ** (t - s) * float(q[t].double() @ k[s].double()) * v[s].double() for s in range(t + 1))
        assert torch.allclose(o[t], want, atol=1e-12)
    # a state handed on continues the sequence
    o2, _ = plain.retention_head(q[4:], k[4:], v[4:], 0.8, S=plain.retention_head(q[:4], k[:4], v[:4], 0.8)[1])
    assert torch.allclose(o2, o[4:], atol=1e-12)


def test_rotations_by_hand():
    """Half-split pairs (i, i + dims/2) and neighbouring pairs (2i, 2i + 1); elements
    beyond ``dims`` pass; position 0 changes nothing."""
    x = torch.arange(1.0, 7.0).view(1, 6).repeat(2, 1)
    for inter, pairs in ((False, [(0, 2), (1, 3)]), (True, [(0, 1), (2, 3)])):
        y = plain.rotate(x, [0, 3], 10.0, 4, inter)
        assert torch.equal(y[0], x[0].double()) and torch.equal(y[1, 4:], x[1, 4:].double())
        for i, (a, b) in enumerate(pairs):
            ang = 3 * 10.0 ** (-2.0 * i / 4)
            assert math.isclose(float(y[1, a]), float(x[1, a]) * math.cos(ang) - float(x[1, b]) * math.sin(ang), abs_tol=1e-12)
            assert math.isclose(float(y[1, b]), float(x[1, b]) * math.cos(ang) + float(x[1, a]) * math.sin(ang), abs_tol=1e-12)


def test_gated_recurrence_by_hand():
    """The first token is no special case: S_0 = sqrt(1 - a^2) i u; the convolution's last
    column is the current token's."""
    u = torch.tensor([[2.0], [1.0]])
    r = torch.tensor([[0.5], [0.25]])
    i = torch.tensor([[0.5], [1.0]])
    lam = torch.tensor([0.3], dtype=torch.float64)
    sp = math.log1p(math.exp(0.3))
    a0, a1 = math.exp(-8 * 0.5 * sp), math.exp(-8 * 0.25 * sp)
    S = plain.gated_recurrence(u, r, i, lam)
    s0 = math.sqrt(1 - a0 * a0) * 0.5 * 2.0
    assert math.isclose(float(S[0]), s0, rel_tol=1e-12)
    assert math.isclose(float(S[1]), a1 * s0 + math.sqrt(1 - a1 * a1), rel_tol=1e-12)
    x = torch.tensor([[1.0], [10.0], [100.0]])
    y = plain.causal_conv(x, torch.tensor([[3.0, 2.0]]), torch.tensor([0.5]))
    assert y.flatten().tolist() == [2.5, 23.5, 230.5]
    bd = plain.block_diagonal(torch.tensor([[1.0, 2.0, 3.0, 4.0]]),
                              torch.tensor([[[1.0, 0.0], [1.0, 1.0]], [[0.0, 2.0], [1.0, 0.0]]]),
                              torch.zeros(2, 2))
    assert bd.flatten().tolist() == [1.0, 3.0, 8.0, 3.0]


def test_window_and_router_by_hand():
    q = torch.zeros(4, 2)
    v = torch.eye(4)
    out = plain.windowed_softmax_attention(q, torch.zeros(4, 2), v, 1.0, 2)
    assert torch.allclose(out[0], torch.tensor([1.0, 0, 0, 0]).double())
    assert torch.allclose(out[3], torch.tensor([0, 0, 0.5, 0.5]).double())     # itself and one before it
    idx, w = plain.route(torch.tensor([[1.0, 0.0]]), torch.tensor([[0.0, 1.0], [2.0, 0.0], [-1.0, 0.0], [1.0, 5.0]]), 2)
    assert idx.tolist() == [[1, 3]]
    assert torch.allclose(w, torch.sigmoid(torch.tensor([[2.0, 1.0]])).double())   # scores as they are
    # the weight multiplies the expert's input: with top 1, out = expert(s h), not s expert(h)
    g = torch.Generator().manual_seed(1)
    W = {"p.router": torch.tensor([[4.0, 0.0, 0.0]]), "p.e0.gate": torch.randn(5, 3, generator=g),
         "p.e0.up": torch.randn(5, 3, generator=g), "p.e0.down": torch.randn(3, 5, generator=g)}
    h = torch.tensor([[0.5, -1.0, 2.0]])
    s = float(torch.sigmoid(torch.tensor(2.0)))
    got = plain.routed_ff(h, W, "p.", {"router": {"experts": 1, "top": 1}})
    assert torch.allclose(got, plain.expert_ff(s * h.double(), W, "p.e0."), atol=1e-12)
    assert not torch.allclose(got, s * plain.expert_ff(h.double(), W, "p.e0."), atol=1e-3)
