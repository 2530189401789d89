"""Each mechanism that the Zutazen design brought, alone, against the plain
implementation's function for it: the scaled embedding, the gated feed-forward
with biases, retention (state carried over steps, slots used again, a planted
pair read back far away under a slow decay and lost under a fast one, partial
rotation), the gated linear recurrence (convolution tail across portions shorter
than it, parts of the channels, one tap), the per-head products of latent
attention, and experts chosen by sigmoid scores that weigh their input."""
import math

import pytest
import torch

from plain import zutazen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: dict(atol=3e-5, rtol=3e-4), torch.bfloat16: dict(atol=0.03, rtol=0.03)}


def close(got, want, dtype, what=""):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = (got - want).abs()
    bound = TOL[dtype]["atol"] + TOL[dtype]["rtol"] * want.abs()
    assert bool((err <= bound).all()), f"{what}: max err {err.max().item():.3g} at {int(err.argmax())}"


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def step_of(seqs):
    """The fields of a step that the kernels read, for sequences given as (slot, start, n)."""
    from grout_b200.engine.batch import make_context
    return make_context([(s, st, [0] * n) for s, st, n in seqs], None, DEV)


g32 = lambda t: t.float().to(DEV).contiguous()


# ------------------------------------------------------------------ small pieces
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scaled_embedding_is_32_bit(dtype):
    from grout_b200.kernels import ops
    table = rnd(37, 72, seed=1).to(dtype)
    ids = torch.tensor([3, 36, 0, 3], dtype=torch.int32)
    got = ops.embed_scaled(table.to(DEV), ids.to(DEV), 1.7)
    assert got.dtype == torch.float32
    close(got, table.double()[ids.long()] * 1.7, torch.float32)      # not rounded to the table's type


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [3, 64, 300])
def test_gated_feed_forward_with_biases(dtype, rows):
    """relu gate, three biases, every product choice; the result leaves as 32-bit sums."""
    from grout_b200.parts import BuildContext, PartSpec, ProductChoice, build_part
    W, F = 64, 96
    names = {"gate": "gate", "up": "up", "down": "down", "gate_bias": "gate.b", "up_bias": "up.b", "down_bias": "down.b"}
    w = {"gate": rnd(F, W, seed=1, scale=0.3), "up": rnd(F, W, seed=2, scale=0.3), "down": rnd(W, F, seed=3, scale=0.2),
         "gate.b": rnd(F, seed=4, scale=0.5), "up.b": rnd(F, seed=5, scale=0.5), "down.b": rnd(W, seed=6, scale=0.5)}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = rnd(rows, W, seed=7).to(dtype)
    want = plain.dense_ff(x, {"m." + k: v for k, v in w.items()}, "m.")
    no_bias = plain.dense_ff(x, {"m." + k: (v * 0 if k.endswith(".b") else v) for k, v in w.items()}, "m.")
    assert float((want - no_bias).abs().max()) > 0.3                  # the biases matter here
    choices = [ProductChoice()] if dtype == torch.float32 else \
        [ProductChoice("tc", "auto"), ProductChoice("tc", "pair"), ProductChoice("skinny", "library")]
    for choice in choices:
        part = build_part("feedforward", PartSpec("gated_mlp", dict(
            hidden=W, intermediate=F, activation="relu", bias=True, names=names)),
            BuildContext(dtype, torch.device(DEV), choice))
        part.load({k: v.to(DEV) for k, v in w.items()})
        got = part.forward(x.to(DEV), None)
        assert got.dtype == torch.float32 and got.dim() == 3
        got = got.sum(0).double().cpu()
        if dtype == torch.float32:
            close(got, want, dtype)
        else:
            assert float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) < 0.01, (rows, choice)


def test_relu_gate_without_biases():
    from grout_b200.kernels import ops
    gu = rnd(5, 2 * 24, seed=1, scale=2.0)
    close(ops.relu_mul(gu.to(DEV), 0), torch.relu(gu[:, :24].double()) * gu[:, 24:].double(), torch.float32)


# ------------------------------------------------------------------ retention
def _ret_weights(m, W, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    return {"q": r(H * dk, W, sc=0.3), "k": r(H * dk, W, sc=0.3), "v": r(H * dv, W, sc=0.3),
            "g": r(H * dv, W, sc=0.3)}


def _ret_run(w, m, xs, cuts, dtype, state=None, slot=0, n_slots=3, first_pos=0):
    """Feeds rows xs [T, W] through the kernels in steps of the given sizes."""
    from grout_b200.kernels import ops
    from grout_b200.parts.position import scaled_inverse_frequencies
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    rd = m["rot"]["dims"]
    inv = torch.from_numpy(scaled_inverse_frequencies(rd, m["rot"]["base"], None)).float().to(DEV) if rd else None
    wp = torch.cat([w[k] for k in ("q", "k", "v", "g")], 0).double()
    if state is None:
        state = torch.zeros(n_slots + 1, H * dk * dv, device=DEV)
    decay = torch.tensor(m["decay"], dtype=torch.float32, device=DEV)
    outs, start = [], first_pos
    for n in cuts:
        step = step_of([(slot, start, n)])
        proj = g32(xs[start - first_pos:start - first_pos + n].double() @ wp.T)
        y = ops.retention_forward(proj, state, decay, inv, H=H, dk=dk, dv=dv, rot_dim=rd, k_scale=dk ** -0.5,
                                  norm_eps=1e-5, token_pos=step.token_pos, cu_q=step.cu_q, slots=step.slots,
                                  dtype=dtype, max_rows=step.max_q_len)
        outs.append(y.float().cpu())
        start += n
    return torch.cat(outs), state


def _ret_plain(w, m, xs, first_pos=0):
    W = dict({"m." + k: v for k, v in w.items()})
    W["m.o"] = torch.eye(m["heads"] * m["vdim"])          # the read-out before the o projection
    return plain.retention_mixer(xs, W, "m.", m, 1e-5, first_pos=first_pos)


def _ret(heads, dim, vdim, dims, base=10000.0, lo=0.7, hi=0.999):
    return dict(heads=heads, dim=dim, vdim=vdim, rot={"base": base, "dims": dims},
                decay=[lo + (hi - lo) * i / max(heads - 1, 1) for i in range(heads)])


RET_SHAPES = [_ret(4, 16, 8, 16), _ret(3, 40, 20, 12),     # a head that fills no lane group, a part rotated
              _ret(2, 64, 48, 64, base=1e6), _ret(1, 128, 16, 32), _ret(2, 30, 10, 0),   # no rotation at all
              _ret(1, 256, 40, 256), _ret(5, 8, 3, 2), _ret(2, 20, 130, 20)]


@pytest.mark.parametrize("m", RET_SHAPES)
def test_retention_whole_in_portions_and_token_by_token(m):
    W, T = 24, 150
    w = _ret_weights(m, W, seed=3)
    xs = rnd(T, W, seed=4)
    want = _ret_plain(w, m, xs)
    whole, _ = _ret_run(w, m, xs, [T], torch.float32)
    close(whole, want, torch.float32, "whole")
    for cuts in ([2] * 75, [1] * T, [1, 2, 3, 100, 44], [149, 1]):
        got, _ = _ret_run(w, m, xs, cuts, torch.float32)      # the same sums, in another order at most
        close(got, whole, torch.float32, str(cuts))
    half, _ = _ret_run(w, m, xs, [T], torch.bfloat16)
    close(half, want, torch.bfloat16, "bfloat16 output")


def test_retention_positions_far_from_zero():
    """Angles are position times frequency in 32-bit: a sequence that goes on at position 3000."""
    m = _ret(2, 32, 16, 32, base=1e4)
    w, xs = _ret_weights(m, 24, seed=5), rnd(20, 24, seed=6)
    got, _ = _ret_run(w, m, xs, [20], torch.float32, first_pos=3000)
    want = _ret_plain(w, m, xs, first_pos=3000)
    assert float((got.double() - want).abs().max()) < 2e-3           # 32-bit angles at 3000 radians


def test_retention_batches_slots_used_again_and_padding():
    from grout_b200.kernels import ops
    from grout_b200.parts.position import scaled_inverse_frequencies
    m = RET_SHAPES[0]
    H, dk, dv, W = m["heads"], m["dim"], m["vdim"], 24
    w = _ret_weights(m, W, seed=5)
    xa, xb = rnd(40, W, seed=6), rnd(9, W, seed=7)
    alone_a, _ = _ret_run(w, m, xa, [40], torch.float32)
    alone_b, _ = _ret_run(w, m, xb, [9], torch.float32)
    wp = torch.cat([w[k] for k in ("q", "k", "v", "g")], 0).double()
    inv = torch.from_numpy(scaled_inverse_frequencies(16, m["rot"]["base"], None)).float().to(DEV)
    decay = torch.tensor(m["decay"], dtype=torch.float32, device=DEV)
    state = torch.zeros(4, H * dk * dv, device=DEV)
    run = lambda step, rows: ops.retention_forward(
        g32(rows.double() @ wp.T), state, decay, inv, H=H, dk=dk, dv=dv, rot_dim=16, k_scale=dk ** -0.5,
        norm_eps=1e-5, token_pos=step.token_pos, cu_q=step.cu_q, slots=step.slots, dtype=torch.float32,
        max_rows=step.max_q_len).cpu()
    # a in slot 2 and b in slot 1 start together with a padding sequence between them
    y = run(step_of([(2, 0, 30), (-1, 0, 3), (1, 0, 8)]), torch.cat([xa[:30], rnd(3, W, seed=8), xb[:8]]))
    close(y[:30], alone_a[:30], torch.float32); close(y[33:], alone_b[:8], torch.float32)
    assert float(state[3].abs().max()) == 0.0 and float(state[0].abs().max()) == 0.0   # padding rows store nothing
    y = run(step_of([(1, 8, 1), (2, 30, 1)]), torch.cat([xb[8:9], xa[30:31]]))         # decoded together, other order
    close(y[0], alone_b[8], torch.float32); close(y[1], alone_a[30], torch.float32)
    state[1].zero_()                                                  # b ends; its slot serves a new request
    y = run(step_of([(2, 31, 9), (1, 0, 9)]), torch.cat([xa[31:], xb]))
    close(y[:9], alone_a[31:], torch.float32); close(y[9:], alone_b, torch.float32)


def test_retention_reads_a_far_pair():
    """What was written 400 tokens ago comes back under a slow decay when its key is asked
    for, scaled by decay^400, and is gone under a fast one; there is no softmax that would
    renormalise it."""
    W = 32
    m = dict(heads=1, dim=16, vdim=8, rot={"base": 1e4, "dims": 0}, decay=[0.999])
    w = {"q": torch.eye(16, W) * 4, "k": torch.eye(16, W) * 4, "v": torch.zeros(8, W), "g": torch.zeros(8, W)}
    w["v"][:, 16:24] = torch.eye(8)
    w["g"][:, 24] = 1.0
    xs = torch.zeros(402, W)
    xs[:, 24] = 2.0
    xs[:, 3], xs[:, 16] = 0.02, 0.05                                  # every token writes a little under key 3
    xs[0, 5], xs[0, 16:24] = 5.0, torch.arange(1.0, 9.0)              # the planted pair: key 5 -> value
    xs[401, 5] = 5.0                                                  # the last token asks for key 5
    for decay, keeps in ((0.999, True), (0.9, False)):
        m["decay"] = [decay]
        got, _ = _ret_run(w, m, xs, [300, 101, 1], torch.float32)
        close(got, _ret_plain(w, m, xs), torch.float32, f"decay {decay}")
        x2 = xs.clone()
        x2[0, 16:24] = 0.0
        other, _ = _ret_run(w, m, x2, [402], torch.float32)
        moved = float((got[401] - other[401]).abs().max())
        assert (moved > 0.1) == keeps, (decay, moved)


# ------------------------------------------------------------------ the gated linear recurrence
def _rec_weights(m, W, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    C, nb, taps = m["width"], m["blocks"], m["conv"]
    bw = C // nb
    return {"y": r(C, W, sc=0.3), "y.b": r(C, sc=0.3), "x": r(C, W, sc=0.3), "x.b": r(C, sc=0.3),
            "conv": r(C, taps, sc=0.6), "conv.b": r(C, sc=0.3),
            "ra": r(nb, bw, bw, sc=1.5 / math.sqrt(bw)), "ra.b": r(nb, bw, sc=0.5),
            "ri": r(nb, bw, bw, sc=1.5 / math.sqrt(bw)), "ri.b": r(nb, bw, sc=0.5),
            "lam": torch.linspace(-6.0, 1.0, C)}                     # channels that keep and channels that forget


def _rec_run(w, m, xs, cuts, dtype, state=None, slot=0, n_slots=3):
    from grout_b200.kernels import ops
    C, nb, taps = m["width"], m["blocks"], m["conv"]
    wp = torch.cat([w["y"], w["x"]], 0).double()
    if state is None:
        state = torch.zeros(n_slots + 1, taps * C, device=DEV)
    outs, start = [], 0
    for n in cuts:
        step = step_of([(slot, start, n)])
        y = ops.rglru_forward(g32(xs[start:start + n].double() @ wp.T), state, g32(torch.cat([w["y.b"], w["x.b"]])),
                              g32(w["conv"]), g32(w["conv.b"]), g32(w["ra"].transpose(1, 2)), g32(w["ra.b"].reshape(-1)),
                              g32(w["ri"].transpose(1, 2)), g32(w["ri.b"].reshape(-1)), g32(w["lam"]), blocks=nb,
                              taps=taps, factor=8.0, token_seq=step.token_seq, cu_q=step.cu_q, slots=step.slots,
                              dtype=dtype, max_rows=step.max_q_len)
        outs.append(y.float().cpu())
        start += n
    return torch.cat(outs), state


def _rec_plain(w, m, xs):
    W = dict({"m." + k: v for k, v in w.items()})
    W["m.o"] = torch.eye(m["width"])
    return plain.rglru_mixer(xs, W, "m.", m)


REC_SHAPES = [dict(width=24, blocks=3, conv=4), dict(width=40, blocks=1, conv=1), dict(width=30, blocks=5, conv=2),
              dict(width=512, blocks=2, conv=5), dict(width=66, blocks=66, conv=3)]


@pytest.mark.parametrize("m", REC_SHAPES)
def test_recurrence_whole_in_portions_and_token_by_token(m):
    W, T = 24, 150
    w, xs = _rec_weights(m, W, seed=3), rnd(T, W, seed=4)
    want = _rec_plain(w, m, xs)
    whole, _ = _rec_run(w, m, xs, [T], torch.float32)
    close(whole, want, torch.float32, "whole")
    # portions shorter than the convolution's tail, which then holds rows of several steps
    for cuts in ([2] * 75, [1] * T, [1, 2, 3, 100, 44], [149, 1], [64, 65, 21], [33, 117]):
        got, _ = _rec_run(w, m, xs, cuts, torch.float32)
        close(got, whole, torch.float32, str(cuts))
    half, _ = _rec_run(w, m, xs, [T], torch.bfloat16)
    close(half, want, torch.bfloat16, "bfloat16 output")


def test_recurrence_first_token_decays_and_tail():
    """The first token is scaled like every other (S_0 = sqrt(1 - a^2) i u, not i u); a slow
    channel still holds its first input after 300 tokens, a fast one does not; the tail of
    the convolution matters."""
    m = dict(width=8, blocks=2, conv=3)
    W = 16
    w, xs = _rec_weights(m, W, seed=9), rnd(301, W, seed=10)
    w["lam"] = torch.tensor([-9.0, -9.0, 3.0, 3.0, -9.0, 3.0, -9.0, 3.0])
    got, state = _rec_run(w, m, xs, [1, 200, 100], torch.float32)
    want = _rec_plain(w, m, xs)
    close(got, want, torch.float32)
    x2 = xs.clone()
    x2[0] = -xs[0]
    _other, state2 = _rec_run(w, m, x2, [301], torch.float32)
    S_a, S_b = state[0, 2 * 8:].cpu(), state2[0, 2 * 8:].cpu()
    moved = (S_a - S_b).abs()
    assert float(moved[[0, 1, 4, 6]].min()) > 1e-4 and float(moved[[2, 3, 5, 7]].max()) < 1e-6
    no_tail = dict(w, conv=torch.cat([torch.zeros(8, 2), w["conv"][:, 2:]], 1))
    assert float((_rec_plain(no_tail, m, xs) - want).abs().max()) > 0.05


def test_recurrence_batches_slots_used_again_and_padding():
    from grout_b200.kernels import ops
    m, W = REC_SHAPES[0], 24
    C, nb, taps = m["width"], m["blocks"], m["conv"]
    w = _rec_weights(m, W, seed=5)
    xa, xb = rnd(40, W, seed=6), rnd(9, W, seed=7)
    alone_a, _ = _rec_run(w, m, xa, [40], torch.float32)
    alone_b, _ = _rec_run(w, m, xb, [9], torch.float32)
    wp = torch.cat([w["y"], w["x"]], 0).double()
    state = torch.zeros(4, taps * C, device=DEV)
    run = lambda step, rows: ops.rglru_forward(
        g32(rows.double() @ wp.T), state, g32(torch.cat([w["y.b"], w["x.b"]])), g32(w["conv"]), g32(w["conv.b"]),
        g32(w["ra"].transpose(1, 2)), g32(w["ra.b"].reshape(-1)), g32(w["ri"].transpose(1, 2)),
        g32(w["ri.b"].reshape(-1)), g32(w["lam"]), blocks=nb, taps=taps, factor=8.0, token_seq=step.token_seq,
        cu_q=step.cu_q, slots=step.slots, dtype=torch.float32, max_rows=step.max_q_len).cpu()
    y = run(step_of([(2, 0, 30), (-1, 0, 3), (1, 0, 8)]), torch.cat([xa[:30], rnd(3, W, seed=8), xb[:8]]))
    close(y[:30], alone_a[:30], torch.float32); close(y[33:], alone_b[:8], torch.float32)
    assert float(state[3].abs().max()) == 0.0                         # padding rows store nothing
    y = run(step_of([(1, 8, 1), (2, 30, 1)]), torch.cat([xb[8:9], xa[30:31]]))
    close(y[0], alone_b[8], torch.float32); close(y[1], alone_a[30], torch.float32)
    state[1].zero_()
    y = run(step_of([(2, 31, 9), (1, 0, 9)]), torch.cat([xa[31:], xb]))
    close(y[:9], alone_a[31:], torch.float32); close(y[9:], alone_b, torch.float32)


# ------------------------------------------------------------------ latent attention's pieces
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 3, 8, 10), (70, 2, 64, 96), (33, 7, 30, 17), (1, 1, 128, 128)])
def test_product_per_head_with_and_without_gate(dtype, shape):
    from grout_b200.kernels import ops
    T, H, K, N = shape
    x = rnd(T, H, K + 6, seed=1).to(dtype)                            # rows wider than what is read
    w = rnd(H, N, K, seed=2, scale=K ** -0.5).to(dtype)
    want = torch.einsum("thk,hnk->thn", x[..., :K].double(), w.double())
    out = torch.full((T, H, N + 3), 7.0, dtype=dtype, device=DEV)
    got = ops.heads_mm(x.to(DEV), w.to(DEV), out)
    close(got[..., :N], want, dtype)
    assert bool((got[..., N:] == 7.0).all())                          # columns beyond N are left alone
    gate = rnd(T, 5 + H * N, seed=3)
    got = ops.heads_mm(x.to(DEV), w.to(DEV), gate=gate.to(DEV), gate_col=5)
    close(got, want * torch.sigmoid(gate[:, 5:].double()).view(T, H, N), dtype, "gated")


# ------------------------------------------------------------------ routed experts
def _moe_weights(E, F, W, seed, router_scale=3.0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    w = {"router": r(E, W, sc=router_scale / math.sqrt(W))}
    for j in range(E):
        w[f"e{j}.gate"], w[f"e{j}.up"] = r(F, W, sc=2.0 / math.sqrt(W)), r(F, W, sc=2.0 / math.sqrt(W))
        w[f"e{j}.down"] = r(W, F, sc=1.0 / math.sqrt(F))
    return w


def _moe_run(w, E, top, x, dtype):
    from grout_b200.kernels import ops
    stack = lambda what: torch.stack([w[f"e{j}.{what}"] for j in range(E)]).to(dtype).to(DEV).contiguous()
    return ops.moe_forward(x.to(dtype).to(DEV), g32(w["router"]), None, stack("gate"), stack("up"), stack("down"),
                           top=top, slope=1.0, up_offset=0.0, score_fn="sigmoid", weigh_input=True, want_choice=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(12, 1, 64, 32, 40), (5, 2, 24, 40, 3), (3, 3, 17, 9, 70), (8, 2, 128, 64, 600)])
def test_experts_with_sigmoid_scores_that_weigh_their_input(dtype, shape):
    E, top, W, F, T = shape
    w = _moe_weights(E, F, W, seed=E + T)
    w = {k: (v.to(dtype).float() if k != "router" else v) for k, v in w.items()}
    x = rnd(T, W, seed=2).to(dtype).float()
    out, ids, wts = _moe_run(w, E, top, x, dtype)
    want_ids, want_w = plain.route(x, w["router"], top)
    assert torch.equal(ids.cpu().long(), want_ids)
    close(wts, want_w, torch.float32, "scores, as they are")
    assert float(wts.sum(-1).max()) > 1.05 or top == 1               # not renormalised
    want = plain.routed_ff(x, {"m." + k: v for k, v in w.items()}, "m.", {"router": {"experts": E, "top": top}})
    got = out.sum(0).double().cpu()
    if dtype == torch.float32:
        close(got, want, dtype)
    else:
        assert float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) < 0.02
    # weighing the output instead would be another function
    wrong = torch.zeros_like(want)
    for t in range(T):
        for e, s in zip(want_ids[t].tolist(), want_w[t]):
            wrong[t] += s * plain.expert_ff(x[t:t + 1].double(), {"m." + k: v for k, v in w.items()}, f"m.e{e}.")[0]
    assert float((wrong - want).abs().max()) > 10 * float((got - want).abs().max())


def test_a_tokens_experts_do_not_depend_on_its_batch():
    E, top, W, F = 6, 2, 32, 16
    w = _moe_weights(E, F, W, seed=4)
    x = rnd(50, W, seed=5)
    whole, _, _ = _moe_run(w, E, top, x, torch.float32)
    for rows in ([0], [49, 3, 17], list(range(20, 37))):
        part, _, _ = _moe_run(w, E, top, x[rows], torch.float32)
        assert torch.equal(part.cpu(), whole[:, rows].cpu())


# ------------------------------------------------------------------ steps of many rows, steps of one row
def _rec_call(w, m, rows, step, state, dtype=torch.float32):
    from grout_b200.kernels import ops
    wp = torch.cat([w["y"], w["x"]], 0).double()
    return ops.rglru_forward(
        g32(rows.double() @ wp.T), state, g32(torch.cat([w["y.b"], w["x.b"]])), g32(w["conv"]), g32(w["conv.b"]),
        g32(w["ra"].transpose(1, 2)), g32(w["ra.b"].reshape(-1)), g32(w["ri"].transpose(1, 2)),
        g32(w["ri.b"].reshape(-1)), g32(w["lam"]), blocks=m["blocks"], taps=m["conv"], factor=8.0,
        token_seq=step.token_seq, cu_q=step.cu_q, slots=step.slots, dtype=dtype, max_rows=step.max_q_len).float().cpu()


@pytest.mark.parametrize("m", [dict(width=48, blocks=3, conv=4), dict(width=200, blocks=2, conv=2)])
def test_recurrence_long_sequences_go_chunk_by_chunk(m):
    """Sequences of more rows than a chunk of the scan, with lengths at a chunk's edge, in one
    step beside short ones and a padding sequence: each as alone, the kept state as token by
    token, and the next step goes on from it."""
    W, C, taps = 24, m["width"], m["conv"]
    w = _rec_weights(m, W, seed=11)
    lens = [130, 1, 64, 65, 200, 63, 128]
    xs = [rnd(n + 2, W, seed=20 + i) for i, n in enumerate(lens)]
    want = [_rec_plain(w, m, x) for x in xs]
    state = torch.zeros(len(lens) + 2, taps * C, device=DEV)
    state[1:] = 7.0                                                # slots that held something else before
    state[1:len(lens) + 1].zero_()
    seqs = [(i + 1, 0, n) for i, n in enumerate(lens)]
    seqs.insert(3, (-1, 0, 70))
    rows = [x[:n] for x, n in zip(xs, lens)]
    rows.insert(3, rnd(70, W, seed=40))
    y = _rec_call(w, m, torch.cat(rows), step_of(seqs), state)
    at = 0
    for (slot, _, n) in seqs:
        if slot > 0:
            close(y[at:at + n], want[slot - 1][:n], torch.float32, f"length {n}")
            _, by_one = _rec_run(w, m, xs[slot - 1][:n], [1] * n, torch.float32)
            close(state[slot], by_one[0], torch.float32, f"state after {n}")
        at += n
    assert float((state[len(lens) + 1] - 7.0).abs().max()) == 0.0  # a padding sequence stores nothing
    # two more rows each (a step of few rows) from the kept state
    y = _rec_call(w, m, torch.cat([x[n:] for x, n in zip(xs, lens)]),
                  step_of([(i + 1, n, 2) for i, n in enumerate(lens)]), state)
    for i, n in enumerate(lens):
        close(y[2 * i:2 * i + 2], want[i][n:], torch.float32, f"after {n}")


@pytest.mark.parametrize("m", [_ret(3, 40, 20, 12), _ret(2, 64, 130, 64), _ret(1, 256, 256, 32), _ret(5, 8, 3, 2),
                               _ret(2, 24, 300, 0)])
def test_retention_step_of_one_row_a_sequence(m):
    """A step in which every sequence brings one row against the same rows walked by the
    kernels for steps of any shape: read-outs and states, a padding sequence among them."""
    from grout_b200.kernels import ops
    from grout_b200.parts.position import scaled_inverse_frequencies
    H, dk, dv, W = m["heads"], m["dim"], m["vdim"], 24
    rd = m["rot"]["dims"]
    w = _ret_weights(m, W, seed=12)
    wp = torch.cat([w[k] for k in ("q", "k", "v", "g")], 0).double()
    inv = torch.from_numpy(scaled_inverse_frequencies(rd, m["rot"]["base"], None)).float().to(DEV) if rd else None
    decay = torch.tensor(m["decay"], dtype=torch.float32, device=DEV)
    starts = [5, 0, 700, 31]
    step = step_of([(2, starts[0], 1), (-1, starts[1], 1), (0, starts[2], 1), (3, starts[3], 1)])
    rows = rnd(4, W, seed=13)
    before = rnd(5, H * dk * dv, seed=14).to(DEV)
    outs = []
    for max_rows in (None, 1):
        state = before.clone()
        y = ops.retention_forward(g32(rows.double() @ wp.T), state, decay, inv, H=H, dk=dk, dv=dv, rot_dim=rd,
                                  k_scale=dk ** -0.5, norm_eps=1e-5, token_pos=step.token_pos, cu_q=step.cu_q,
                                  slots=step.slots, dtype=torch.float32, max_rows=max_rows)
        outs.append((y.cpu(), state.cpu()))
    close(outs[1][0], outs[0][0], torch.float32, "read-outs")
    close(outs[1][1], outs[0][1], torch.float32, "states")
    assert torch.equal(outs[1][1][[1, 4]], before.cpu()[[1, 4]])      # slots of no sequence stay
    assert not torch.equal(outs[1][1][0], before.cpu()[0])


@pytest.mark.parametrize("m", [_ret(3, 40, 20, 12), _ret(2, 64, 130, 64, lo=0.9), _ret(1, 128, 128, 128, lo=0.97),
                               _ret(2, 20, 140, 0, lo=0.5, hi=0.9999)])
def test_retention_long_sequences_go_chunk_by_chunk(m):
    """Sequences of more rows than the chunks of the scan, with lengths at a chunk's edge, in
    one step beside short ones and a padding sequence, from states that an earlier portion
    left: each as alone in the plain implementation, the read-outs and the kept states as
    the row-by-row kernels give them, and a step of few rows goes on from the kept state."""
    from grout_b200.kernels import ops
    from grout_b200.parts.position import scaled_inverse_frequencies
    H, dk, dv, W = m["heads"], m["dim"], m["vdim"], 24
    rd = m["rot"]["dims"]
    w = _ret_weights(m, W, seed=21)
    wp = torch.cat([w[k] for k in ("q", "k", "v", "g")], 0).double()
    inv = torch.from_numpy(scaled_inverse_frequencies(rd, m["rot"]["base"], None)).float().to(DEV) if rd else None
    decay = torch.tensor(m["decay"], dtype=torch.float32, device=DEV)
    lens = [256, 3, 257, 383, 1, 384, 385, 127, 129, 300]
    head = [0, 0, 5, 0, 2, 130, 0, 0, 1, 0]                        # rows that an earlier step brought
    xs = [rnd(h + n + 2, W, seed=50 + i) for i, (h, n) in enumerate(zip(head, lens))]
    want = [_ret_plain(w, m, x) for x in xs]

    def run(state, seqs, rows, max_rows):
        step = step_of(seqs)
        return ops.retention_forward(
            g32(torch.cat(rows).double() @ wp.T), state, decay, inv, H=H, dk=dk, dv=dv, rot_dim=rd,
            k_scale=dk ** -0.5, norm_eps=1e-5, token_pos=step.token_pos, cu_q=step.cu_q, slots=step.slots,
            dtype=torch.float32, max_rows=step.max_q_len if max_rows == "known" else max_rows).float().cpu()

    states = []
    for max_rows in ("known", None):                               # chunk by chunk, then row by row
        state = torch.full((len(lens) + 2, H * dk * dv), 7.0, device=DEV)
        state[1:len(lens) + 1].zero_()
        with_head = [(i + 1, 0, h) for i, h in enumerate(head) if h]
        run(state, with_head, [xs[s - 1][:h] for s, _, h in with_head], None)
        seqs = [(i + 1, h, n) for i, (h, n) in enumerate(zip(head, lens))]
        rows = [x[h:h + n] for x, h, n in zip(xs, head, lens)]
        seqs.insert(4, (-1, 0, 260))
        rows.insert(4, rnd(260, W, seed=49))
        y = run(state, seqs, rows, max_rows)
        at = 0
        for slot, h, n in seqs:
            if slot > 0:
                close(y[at:at + n], want[slot - 1][h:h + n], torch.float32, f"{max_rows}: {h} then {n} rows")
            at += n
        assert float((state[[0, len(lens) + 1]] - 7.0).abs().max()) == 0.0   # a padding sequence stores nothing
        states.append(state.clone())
        y = run(state, [(i + 1, h + n, 2) for i, (h, n) in enumerate(zip(head, lens))],
                [x[h + n:] for x, h, n in zip(xs, head, lens)], "known")
        for i, (h, n) in enumerate(zip(head, lens)):
            close(y[2 * i:2 * i + 2], want[i][h + n:], torch.float32, f"{max_rows}: after {h} and {n} rows")
    close(states[0], states[1], torch.float32, "kept states")


@pytest.mark.parametrize("act", ["relu", "silu", "gelu_tanh"])
@pytest.mark.parametrize("rows,F,W", [(5, 48, 64), (64, 96, 40), (300, 160, 72), (513, 32, 256)])
def test_gate_epilogue_with_biases_of_the_tensor_core_products(act, rows, F, W):
    """act(x Wg^T + bg) * (x Wu^T + bu) as the epilogue of the product for few rows and of
    the product for many, against the same in double precision from the same bfloat16
    operands; a bias large enough that leaving it out, or adding it behind the gate, shows."""
    from grout_b200.kernels import ops
    g, u = rnd(F, W, seed=1, scale=0.3).bfloat16(), rnd(F, W, seed=2, scale=0.3).bfloat16()
    bg, bu = rnd(F, seed=3, scale=1.5), rnd(F, seed=4, scale=1.5)
    x = rnd(rows, W, seed=5).bfloat16()
    fused = torch.stack([g.view(-1, 8, W), u.view(-1, 8, W)], dim=1).reshape(2 * F, W).contiguous().to(DEV)
    bias = torch.stack([bg.view(-1, 8), bu.view(-1, 8)], dim=1).reshape(-1).contiguous().to(DEV)
    zg, zu = x.double() @ g.double().T + bg.double(), x.double() @ u.double().T + bu.double()
    fn = {"relu": torch.relu, "silu": torch.nn.functional.silu,
          "gelu_tanh": lambda z: torch.nn.functional.gelu(z, approximate="tanh")}[act]
    want = fn(zg) * zu
    assert float((want - fn(zg - bg.double()) * (zu - bu.double())).abs().max()) > 1.0
    got = [ops.gemm_tc2_bf16(x.to(DEV), fused, torch.bfloat16, silu_mul=True, gate_act=act, bias=bias)]
    if rows <= ops.SKINNY_MAX_ROWS:
        got.append(ops.gemm_tc_bf16(x.to(DEV), fused, torch.bfloat16, swap=True, silu_mul=True, gate_act=act, bias=bias))
    for y in got:
        close(y.float(), want, torch.bfloat16, f"{act} {rows}x{F}x{W}")


# ------------------------------------------------------------------ latent attention, through its part
def _lat_weights(m, W, seed, sharp):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sc=1.0: torch.randn(*s, generator=g) * sc
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    return {"q": r(H * (dn + dr), W, sc=sharp / math.sqrt(W)), "dkv": r(R + dr, W, sc=1 / math.sqrt(W)),
            "dkv.norm": 1 + r(R, sc=0.2), "uk": r(H * dn, R, sc=sharp / math.sqrt(R)),
            "uv": r(H * dv, R, sc=1 / math.sqrt(R)), "g": r(H * dv, W, sc=1 / math.sqrt(W)),
            "o": r(W, H * dv, sc=1 / math.sqrt(H * dv))}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(3, 16, 8, 16, 24, 64), (20, 32, 16, 32, 48, 65), (2, 24, 0, 40, 40, 5),
                                   (17, 64, 32, 64, 96, 130), (1, 8, 4, 8, 300, 63)])
def test_latent_attention_windows_pages_and_cuts(dtype, shape):
    """Through the mixer part and a paged cache: windows of a page, of one more and of one
    less, and longer than two pages, passing over a prompt and over decoded tokens; the same
    rows in other cuts; the scores are sharp enough that a window one token off, in either
    direction, would show in the rows behind the window."""
    from grout_b200.cache import CacheLayout, SequenceCache
    from grout_b200.parts import BuildContext, PartSpec, build_part
    H, dn, dr, dv, R, window = shape
    W, T, eps = 48, 210, 1e-5
    m = dict(heads=H, dim=dn, rot_dim=dr, vdim=dv, kv_rank=R, scale=(dn + dr) ** -0.5,
             rot={"base": 1e4, "dims": dr}, mask={"size": window})
    w = {k: v.to(dtype) for k, v in _lat_weights(m, W, seed=31, sharp=4.0).items()}
    x = rnd(T, W, seed=32).to(dtype)
    pw = {"m." + k: v for k, v in w.items()}
    want = plain.latent_attention_mixer(x, pw, "m.", m, eps)
    for other in (window - 1, window + 1):
        if other > 0:
            off = plain.latent_attention_mixer(x, pw, "m.", dict(m, mask={"size": other}), eps)
            assert float((off - want)[window:].abs().max()) > 0.1 * float(want.abs().max())
            assert float((off - want)[:min(window, other) - 1].abs().max()) < 1e-9 if min(window, other) > 1 else True
    position = (PartSpec("rotary_interleaved", dict(head_dim=dr, theta=1e4, rot_dim=dr, exact_table=True))
                if dr else PartSpec("none", {}))
    part = build_part("mixer", PartSpec("latent_attention", dict(
        hidden=W, n_heads=H, head_dim=dn, rot_dim=dr, v_head_dim=dv, kv_rank=R, position=position,
        scale=m["scale"], norm_eps=eps, window=window, gated=True)), BuildContext(dtype, torch.device(DEV)))
    part.load({k: v.to(DEV) for k, v in w.items()})
    cache = SequenceCache(CacheLayout.from_specs([part.cache_spec()]), max_tokens=1024, max_slots=3,
                          max_seq_len=256, dtype=dtype, device=DEV)
    first = None
    for cuts in ([T], [window + 2] + [1] * (T - window - 2) if window + 2 < T else [T - 1, 1],
                 [63, 2, 64, 1, 70, 1, 1, 8], [2] * (T // 2)):
        held = cache.open()                                   # another request holds pages in between
        cache.reserve(held, 70)
        slot = cache.open()
        outs, start = [], 0
        for n in cuts:
            cache.reserve(slot, n)
            cache.flush()
            step = make_step([(slot, start, n)])
            y = part.forward(x[start:start + n].to(DEV), step, cache.view(0))
            outs.append((y.sum(0) if y.dim() == 3 else y).float().cpu())
            cache.advance(slot, n)
            start += n
        cache.close(held)
        cache.close(slot)                                     # the pages serve the next cut
        got = torch.cat(outs)
        if dtype == torch.float32:
            close(got, want, dtype, str(cuts[:4]))
        else:
            d = got.double() - want
            assert float(d.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) < 0.03, cuts[:4]
            assert float(d.abs().max()) < 0.15 * float(want.abs().max()), cuts[:4]
        if first is None:
            first = got
        elif dtype == torch.float32:
            close(got, first, dtype, "cut against whole")


def make_step(seqs):
    from grout_b200.engine.batch import make_context
    return make_context([(s, st, [0] * n) for s, st, n in seqs], None, DEV)
