"""Each mechanism that the Mananex design brought, alone, against the plain
implementation's function for it: the forget-gate linear attention (state carried over
steps, slots used again, padding rows, a planted value read back far away through a gate
that keeps and lost through one that forgets), attention windows that keep a sequence's
first tokens (planted keys just inside and just outside the window and the kept tokens,
at page borders, in prompts and in single steps, through every attention kernel), the
sigmoid gate per head, the rotation of neighbouring pairs, the gated sum with the depth
average and the norm, and routers with a bias that weigh the chosen by the softmax over
their logits alone."""
import math

import pytest
import torch

from plain import mananex as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: dict(atol=3e-5, rtol=3e-4), torch.bfloat16: dict(atol=0.03, rtol=0.03)}


def close(got, want, dtype, what=""):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = (got - want).abs()
    bound = TOL[dtype]["atol"] + TOL[dtype]["rtol"] * want.abs()
    assert bool((err <= bound).all()), f"{what}: max err {err.max().item():.3g} at {int(err.argmax())}"


def close_to_scale(got, want, dtype, what=""):
    """The same with the absolute part of the bar taken from the largest value: sums of many terms
    of that size cancel, and their 32-bit rounding is what is left where the result is near zero."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = (got - want).abs()
    bound = TOL[dtype]["atol"] * max(1.0, float(want.abs().max())) + TOL[dtype]["rtol"] * want.abs()
    assert bool((err <= bound).all()), f"{what}: max err {err.max().item():.3g} at {int(err.argmax())}"


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def make_step(seqs):
    """The fields of a step that the kernels read, for sequences given as (slot, start, n)."""
    from grout_b200.engine.batch import make_context
    return make_context([(s, st, [0] * n) for s, st, n in seqs], None, DEV)


g32 = lambda t: t.float().to(DEV).contiguous()


# ------------------------------------------------------------------ forget-gate linear attention
def _fg_weights(m, W, seed, f_scale=1.0):
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    return {"q": rnd(H * dk, W, seed=seed, scale=0.4), "f": rnd(H * dk, W, seed=seed + 1, scale=0.5 * f_scale),
            "f.b": rnd(H * dk, seed=seed + 2, scale=1.0), "lower": torch.sigmoid(rnd(H * dk, seed=seed + 3)),
            "v": rnd(H * dv, W, seed=seed + 4, scale=0.4), "norm": 1 + rnd(dv, seed=seed + 5, scale=0.2),
            "o": torch.eye(H * dv)}


def _fg_run(w, m, xs, cuts, dtype, state=None, slot=0, n_slots=2, mult=1.0, wide=0):
    """The kernel on the 32-bit sums of the plain products, fed in portions; returns (the read-outs
    before the o projection, the state rows)."""
    from grout_b200.kernels import ops
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    wp = torch.cat([w[k] for k in ("q", "f", "v")], 0).double()
    if state is None:
        state = torch.zeros(n_slots + 1, H * dk * dv, device=DEV)
    outs, start = [], 0
    for n in cuts:
        step = make_step([(slot, start, n)])
        proj = g32(xs[start:start + n].double() @ wp.T)
        if wide:          # the sums as columns of a wider product
            big = torch.full((n, wide + proj.shape[1] + 3), float("nan"), device=DEV)
            big[:, wide:wide + proj.shape[1]] = proj
            proj = big[:, wide:wide + proj.shape[1]]
        y = ops.hgrn2_forward(proj, state, g32(w["f.b"]), g32(w["lower"]), g32(w["norm"]), H=H, dk=dk, dv=dv,
                              q_col=0, f_col=H * dk, v_col=2 * H * dk, norm_eps=1e-5, cu_q=step.cu_q,
                              slots=step.slots, dtype=dtype, out_scale=mult)
        outs.append(y.float().cpu())
        start += n
    return torch.cat(outs), state


def _fg_plain(w, m, xs, state=None):
    out, S = plain.forgetful_linear_attention(xs.double(), {"m." + k: v for k, v in w.items()}, m, 1e-5, "m.", state)
    return out, S


FG_SHAPES = [dict(heads=4, dim=16, vdim=8), dict(heads=3, dim=40, vdim=20), dict(heads=2, dim=64, vdim=48),
             dict(heads=1, dim=128, vdim=16), dict(heads=2, dim=30, vdim=10), dict(heads=1, dim=256, vdim=40),
             dict(heads=5, dim=8, vdim=3), dict(heads=2, dim=20, vdim=130), dict(heads=1, dim=1, vdim=1),
             dict(heads=2, dim=100, vdim=24)]


@pytest.mark.parametrize("m", FG_SHAPES)
def test_forget_gate_attention_whole_in_portions_and_token_by_token(m):
    W, T = 24, 150
    w = _fg_weights(m, W, seed=3)
    xs = rnd(T, W, seed=4)
    want, S_want = _fg_plain(w, m, xs)
    whole, state = _fg_run(w, m, xs, [T], torch.float32)
    close(whole, want, torch.float32, "whole")
    close(state[0].view(m["heads"], m["dim"], m["vdim"]), S_want, torch.float32, "state")
    for cuts in ([2] * 75, [1] * T, [1, 2, 3, 100, 44], [149, 1]):
        got, st = _fg_run(w, m, xs, cuts, torch.float32)
        assert torch.equal(got, whole), cuts                  # the same sums in the same order
        assert torch.equal(st[0], state[0]), cuts
    half, _ = _fg_run(w, m, xs, [T], torch.bfloat16)
    close(half, want, torch.bfloat16, "bfloat16 output")
    scaled, _ = _fg_run(w, m, xs, [T], torch.float32, mult=0.7, wide=5)
    close(scaled, 0.7 * want, torch.float32, "a factor, and sums that are part of a wider row")


@pytest.mark.parametrize("m", [dict(heads=2, dim=64, vdim=48), dict(heads=3, dim=20, vdim=130),
                               dict(heads=1, dim=100, vdim=24)])
def test_forget_gate_attention_long_sequences_go_chunk_by_chunk(m):
    """A sequence that brings 256 rows or more in a step goes chunk by chunk: the same sums in another
    order.  Lengths at the chunks' edges; a state that is there already; another sequence of a few rows,
    a padding sequence and one more long sequence in the same step; gates that forget at once and gates
    that keep nearly everything side by side."""
    from grout_b200.kernels import ops
    H, dk, dv, W = m["heads"], m["dim"], m["vdim"], 24
    w = _fg_weights(m, W, seed=61, f_scale=4.0)
    wp = torch.cat([w[k] for k in ("q", "f", "v")], 0).double()
    for T in (256, 257, 320, 383, 1000):
        xs = rnd(40 + T, W, seed=62)
        want, S_want = _fg_plain(w, m, xs)
        got, state = _fg_run(w, m, xs, [40, T], torch.float32)      # 40 rows row by row first, then the long step
        close(got, want, torch.float32, f"{T} rows after 40")
        close(state[0].view(H, dk, dv), S_want, torch.float32, "state")
    a, b, c = rnd(300, W, seed=63), rnd(5, W, seed=64), rnd(450, W, seed=65)
    pad = rnd(70, W, seed=66)
    state = torch.zeros(5, H * dk * dv, device=DEV)
    rows = torch.cat([a, b, pad, c])
    step = make_step([(1, 0, 300), (3, 0, 5), (-1, 0, 70), (0, 0, 450)])
    y = ops.hgrn2_forward(g32(rows.double() @ wp.T), state, g32(w["f.b"]), g32(w["lower"]), g32(w["norm"]),
                          H=H, dk=dk, dv=dv, q_col=0, f_col=H * dk, v_col=2 * H * dk, norm_eps=1e-5,
                          cu_q=step.cu_q, slots=step.slots, dtype=torch.float32, max_rows=step.max_q_len).cpu()
    for xs, (lo, hi), slot in ((a, (0, 300), 1), (b, (300, 305), 3), (c, (375, 825), 0)):
        want, S_want = _fg_plain(w, m, xs)
        close(y[lo:hi], want, torch.float32, f"rows {lo}..{hi}")
        close(state[slot].view(H, dk, dv).cpu(), S_want, torch.float32, f"state of slot {slot}")
    assert float(state[2].abs().max()) == 0.0 and float(state[4].abs().max()) == 0.0


def test_forget_gate_attention_batches_slots_used_again_and_padding():
    """Three sequences of unequal length in one step with a padding sequence between them; then a
    slot is zeroed and used by another sequence, which must not see what was there."""
    from grout_b200.kernels import ops
    m = dict(heads=3, dim=24, vdim=16)
    H, dk, dv, W = 3, 24, 16, 32
    w = _fg_weights(m, W, seed=11)
    wp = torch.cat([w[k] for k in ("q", "f", "v")], 0).double()
    seqs = [rnd(n, W, seed=20 + i) for i, n in enumerate((7, 1, 40))]
    pad = rnd(5, W, seed=30)
    state = torch.zeros(4 + 1, H * dk * dv, device=DEV)
    state[4] = float("nan") * 0 + 7.0         # the padding row's place holds something
    rows = torch.cat([seqs[0], pad, seqs[1], seqs[2]])
    step = make_step([(2, 0, 7), (-1, 0, 5), (0, 0, 1), (3, 0, 40)])
    y = ops.hgrn2_forward(g32(rows.double() @ wp.T), state, g32(w["f.b"]), g32(w["lower"]), g32(w["norm"]),
                          H=H, dk=dk, dv=dv, q_col=0, f_col=H * dk, v_col=2 * H * dk, norm_eps=1e-5,
                          cu_q=step.cu_q, slots=step.slots, dtype=torch.float32).cpu()
    at = {0: (0, 7), 1: (12, 13), 2: (13, 53)}
    for i, (a, b) in at.items():
        close(y[a:b], _fg_plain(w, m, seqs[i])[0], torch.float32, f"sequence {i}")
    assert float(state[1].abs().max()) == 0.0               # no sequence had slot 1
    # continue sequence 0 (slot 2) alone, then reuse slot 3 for a new sequence after zeroing
    more = rnd(9, W, seed=40)
    step = make_step([(2, 7, 9)])
    y2 = ops.hgrn2_forward(g32(more.double() @ wp.T), state, g32(w["f.b"]), g32(w["lower"]), g32(w["norm"]),
                           H=H, dk=dk, dv=dv, q_col=0, f_col=H * dk, v_col=2 * H * dk, norm_eps=1e-5,
                           cu_q=step.cu_q, slots=step.slots, dtype=torch.float32).cpu()
    close(y2, _fg_plain(w, m, torch.cat([seqs[0], more]))[0][7:], torch.float32, "continued")
    state[3].zero_()
    fresh = rnd(6, W, seed=41)
    step = make_step([(3, 0, 6)])
    y3 = ops.hgrn2_forward(g32(fresh.double() @ wp.T), state, g32(w["f.b"]), g32(w["lower"]), g32(w["norm"]),
                           H=H, dk=dk, dv=dv, q_col=0, f_col=H * dk, v_col=2 * H * dk, norm_eps=1e-5,
                           cu_q=step.cu_q, slots=step.slots, dtype=torch.float32).cpu()
    close(y3, _fg_plain(w, m, fresh)[0], torch.float32, "a slot used again")


def test_forget_gate_attention_reads_a_far_value():
    """One channel's gate is held at its lower bound of nearly one for 400 tokens (the value written
    at the first token is still there), another's near zero (it is gone after a few): the read-out of
    the last token tells them apart, in one step and token by token."""
    m = dict(heads=1, dim=2, vdim=4)
    W, T = 8, 400
    w = _fg_weights(m, W, seed=50)
    w["f"] = torch.zeros(2, W)
    w["f.b"] = torch.tensor([-20.0, -20.0])                 # the sigmoid is 0: f is its lower bound
    w["lower"] = torch.tensor([0.9999, 0.05])
    w["q"] = torch.zeros(2, W)
    w["q"][:, 0] = 5.0
    w["v"] = torch.zeros(4, W)
    w["v"][:, 1] = 1.0
    w["norm"] = torch.ones(4)
    xs = torch.zeros(T, W)
    xs[:, 0] = 1.0                                          # q is the same everywhere
    xs[0, 1] = 50.0                                         # a value only the first token writes
    want, S = _fg_plain(w, m, xs)
    assert float(S[0, 0].abs().max()) > 1e-3 and float(S[0, 1].abs().max()) < 1e-12
    whole, state = _fg_run(w, m, xs, [T], torch.float32)
    close(state[0].view(1, 2, 4), S, torch.float32, "state after 400 tokens")
    steps, state1 = _fg_run(w, m, xs, [1] * T, torch.float32)     # (the whole went chunk by chunk)
    close(state1[0].view(1, 2, 4), S, torch.float32, "state, token by token")
    close(steps, want, torch.float32, "read-outs, token by token")
    close(whole, want, torch.float32, "read-outs")


# ------------------------------------------------------------------ windows that keep first tokens
def _attention_part(dtype, H, G, D, Dv, window, keep, rot_dims, gate=True, base=1e4):
    from grout_b200.parts import BuildContext, PartSpec, build_part
    position = (PartSpec("rotary_interleaved", dict(head_dim=D, theta=base, rot_dim=rot_dims, exact_table=True))
                if rot_dims else PartSpec("none", {}))
    return build_part("mixer", PartSpec("gqa_attention", dict(
        hidden=48, n_heads=H, n_kv_heads=G, head_dim=D, v_head_dim=Dv, position=position, scale=D ** -0.5,
        window=window, keep_first=keep, sinks=True, head_gate=gate,
        names={"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink", "g": "g"})),
        BuildContext(dtype, torch.device(DEV)))


def _attention_weights(H, G, D, Dv, W, seed, sharp):
    return {"q": rnd(H * D, W, seed=seed, scale=0.3 * sharp), "k": rnd(G * D, W, seed=seed + 1, scale=0.3 * sharp),
            "v": rnd(G * Dv, W, seed=seed + 2, scale=0.5), "sink": rnd(H, seed=seed + 3, scale=1.5),
            "g": rnd(H, W, seed=seed + 4, scale=0.5), "o": rnd(W, H * Dv, seed=seed + 5, scale=0.3)}


def _attention_plain(x, w, H, G, D, Dv, window, keep, rot_dims, positions=None, base=1e4):
    m = dict(heads=H, kv_heads=G, dim=D, vdim=Dv, scale=D ** -0.5)
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    positions = list(range(x.shape[0])) if positions is None else positions
    return plain.windowed_attention(x.double(), positions, {"m." + k: v for k, v in w.items()}, m, "m.")


ATT_SHAPES = [  # heads, kv heads, dim, vdim, window, kept, rotated
    (4, 2, 16, 16, 7, 2, 8), (2, 2, 64, 64, 64, 1, 64), (2, 1, 64, 64, 65, 64, 16), (2, 2, 128, 128, 63, 65, 32),
    (3, 3, 40, 40, 10, 3, 40), (2, 1, 24, 8, 70, 5, 4), (2, 2, 16, 48, 1, 1, 0), (4, 2, 96, 96, 130, 70, 32),
    (2, 2, 32, 32, 300, 4, 32), (2, 2, 32, 32, 5, 0, 6), (1, 1, 144, 16, 33, 2, 20)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", ATT_SHAPES)
def test_attention_windows_kept_tokens_pages_and_cuts(dtype, shape):
    """Through the mixer part and a paged cache: the window and the kept first tokens pass over a
    prompt and over decoded tokens, across page borders; the same rows in other cuts, with another
    request's pages in between and pages used again; the scores are sharp enough that a window or
    a count of kept tokens that is one off, in either direction, shows in the rows behind it."""
    from grout_b200.cache import CacheLayout, SequenceCache
    H, G, D, Dv, window, keep, rot = shape
    W, T = 48, 210
    w = {k: v.to(dtype) for k, v in _attention_weights(H, G, D, Dv, W, seed=31, sharp=1.0).items()}
    x = rnd(T, W, seed=32).to(dtype)
    want = _attention_plain(x, w, H, G, D, Dv, window, keep, rot)
    if window + keep < 100:      # (the long ones are held to their edges by the planted keys below)
        for dw, dk in ((-1, 0), (1, 0), (0, -1), (0, 1)):
            if window + dw > 0 and keep + dk >= 0:
                off = _attention_plain(x, w, H, G, D, Dv, window + dw, keep + dk, rot)
                assert float((off - want).abs().max()) > 0.02 * float(want.abs().max()), (dw, dk)
    part = _attention_part(dtype, H, G, D, Dv, window, keep, rot)
    part.load({k: v.to(DEV) for k, v in w.items()})
    cache = SequenceCache(CacheLayout.from_specs([part.cache_spec()]), max_tokens=1024, max_slots=3,
                          max_seq_len=256, dtype=dtype, device=DEV)
    first = None
    for cuts in ([T], [min(window + 2, T - 1)] + [1] * (T - min(window + 2, T - 1)),
                 [63, 2, 64, 1, 70, 1, 1, 8], [2] * (T // 2), [1] * T):
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
        cache.check()
        got = torch.cat(outs)
        if dtype == torch.float32:
            close_to_scale(got, want, dtype, str(cuts[:4]))
        else:
            d = got.double() - want
            assert float(d.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()) < 0.03, cuts[:4]
            assert float(d.abs().max()) < 0.15 * float(want.abs().max()), cuts[:4]
        if first is None:
            first = got
        elif dtype == torch.float32:
            close_to_scale(got, first, dtype, "cut against whole")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128, 96, 40])
def test_a_planted_key_at_every_edge(dtype, D):
    """One query far down the sequence and one key that matches it among 330 that do not: placed
    just inside and just outside the window, just inside and just outside the kept first tokens, and
    on both sides of the page borders next to them, it carries the row or is not seen at all; the
    sinks' share of the denominator is there in both cases.  As a prompt's row and as a single step,
    with enough sequences in the step that the decode kernels with many pairs take it."""
    from grout_b200.kernels import ops
    H = G = 2
    window, keep, T, page = 70, 66, 330, 64
    n_seqs = 40 if dtype == torch.bfloat16 else 2
    scale = 1.0
    cases = {"inside the window": T - window, "outside the window": T - window - 1,
             "last kept": keep - 1, "first not kept": keep, "page border kept": page - 1,
             "page border, kept in the second page": page, "first token": 0, "far and not kept": 150,
             "the query's own key": T - 1}
    sink = torch.tensor([0.5, -1.0])
    for what, at in cases.items():
        k = rnd(T, G, D, seed=3, scale=0.05)
        q = rnd(1, H, D, seed=4, scale=0.05)
        k[at] += 3.0 * q[0] / q[0].norm(dim=-1, keepdim=True)      # a score that stands out ...
        q = q * 40.0
        v = rnd(T, G, D, seed=5)
        seen = plain.visible(T - 1, at, window, keep)
        s = torch.einsum("hd,thd->ht", q[0].double(), k.double()) * scale
        mask = torch.tensor([plain.visible(T - 1, j, window, keep) for j in range(T)])
        s = s.masked_fill(~mask[None, :], -math.inf)
        top = torch.maximum(s.max(dim=-1).values, sink.double())
        e = torch.exp(s - top[:, None])
        p = e / (e.sum(-1) + torch.exp(sink.double() - top))[:, None]
        want = torch.einsum("ht,thd->hd", p, v.double())
        assert (float(p[0, at]) > 0.5) == seen, what               # ... and decides the row, if it is seen
        # a cache of n_seqs sequences that all hold these keys; pages in no particular order
        n_pages = (T + page - 1) // page
        kp = torch.zeros(n_seqs * n_pages + 1, G, page, D, dtype=dtype)
        vp = torch.zeros_like(kp)
        order = torch.randperm(n_seqs * n_pages, generator=torch.Generator().manual_seed(7)) + 1
        table = order.view(n_seqs, n_pages).to(torch.int32)
        for sq in range(n_seqs):
            for pg in range(n_pages):
                rows = slice(pg * page, min(T, (pg + 1) * page))
                n = rows.stop - rows.start
                kp[table[sq, pg], :, :n] = k[rows].transpose(0, 1).to(dtype)
                vp[table[sq, pg], :, :n] = v[rows].transpose(0, 1).to(dtype)
        kp, vp, table = kp.to(DEV), vp.to(DEV), table.to(DEV)
        # as single steps of all sequences
        step = make_step([(sq, T - 1, 1) for sq in range(n_seqs)])
        qd = q.to(dtype).expand(n_seqs, H, D).contiguous().to(DEV)
        got = ops.attention(qd, kp, vp, table, step=step, page=page, scale=scale, window=window,
                            sinks=sink.to(DEV), keep_first=keep).float().cpu()
        # as the last row of a prompt's portion of 100 rows (the rows before it are not looked at)
        step = make_step([(0, T - 100, 100)])
        qp = torch.zeros(100, H, D, dtype=dtype)
        qp[-1] = q[0].to(dtype)
        gotp = ops.attention(qp.to(DEV), kp, vp, table, step=step, page=page, scale=scale, window=window,
                             sinks=sink.to(DEV), keep_first=keep).float().cpu()
        for name, g in (("decode", got[0]), ("decode, last sequence", got[-1]), ("prompt", gotp[-1])):
            if dtype == torch.float32:
                close_to_scale(g, want, dtype, f"{what}, {name}")
            else:
                assert float((g.double() - want).abs().max()) < 0.06 * float(want.abs().max()) + 0.02, (what, name)


# ------------------------------------------------------------------ small pieces
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(37, 3, 32, 20, 7, 5), (70, 4, 64, 48, 16, 8), (5, 2, 128, 128, 0, 0)])
def test_gate_per_head_drops_the_filling_and_writes_into_a_wider_row(dtype, sizes):
    from grout_b200.kernels import ops
    T, H, Ds, Dv, before, after = sizes         # (odd sizes take single values, the others 16-byte pieces)
    x = rnd(T, H, Ds, seed=1).to(dtype)
    logits = rnd(T, H + 2, seed=2, scale=2.0)
    wide = torch.full((T, before + H * Dv + after), 9.0, dtype=dtype, device=DEV)
    out = ops.head_gate(x.to(DEV), logits.to(DEV)[:, 1:1 + H], Dv, 0.8, into=wide[:, before:before + H * Dv])
    want = x.double()[:, :, :Dv] * torch.sigmoid(logits.double()[:, 1:1 + H])[:, :, None] * 0.8
    close(out.float().cpu(), want.reshape(T, H * Dv), dtype)
    assert bool((wide[:, :before] == 9.0).all()) and bool((wide[:, before + H * Dv:] == 9.0).all())
    plain_out = ops.head_gate(x.to(DEV), None, Dv)
    close(plain_out.float().cpu(), x.double()[:, :, :Dv].reshape(T, H * Dv), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 2, 24, 8), (4, 4, 128, 128), (2, 1, 128, 32), (3, 3, 40, 6), (2, 2, 64, 64)])
def test_rotation_of_neighbouring_pairs_in_the_qk_kernel(dtype, shape):
    """q and k leave the q/k kernel turned pair by pair (2j with 2j + 1) on their first elements, the
    rest passes; positions far from zero; few rows and many (the kernels differ)."""
    from grout_b200.kernels import ops
    from grout_b200.parts.position import scaled_inverse_frequencies
    H, G, D, rot = shape
    inv = torch.from_numpy(scaled_inverse_frequencies(rot, 1e4, None)).float().to(DEV)
    for T, start in ((3, 0), (200, 1000)):
        qkv = rnd(T, (H + 2 * G) * D, seed=T).to(dtype)
        step = make_step([(-1, start, T)])
        q, kv = ops.qk_prepare(qkv.to(DEV), H, G, D, inv_freq=inv, rot_dim=rot, token_seq=step.token_seq,
                               token_pos=step.token_pos, slots=step.slots, want_kv_out=True, interleaved=True)
        pos = list(range(start, start + T))
        src = qkv.double().view(T, H + 2 * G, D)
        # (the angle position * frequency is a 32-bit product: at position 1,000 it is good to 1e-4)
        far = dict(atol=1e-3, rtol=0.0) if dtype == torch.float32 and start else None
        for got, want, nm in ((q, src[:, :H], "q"), (kv[:, :G], src[:, H:H + G], "k")):
            want = plain.rotate_neighbours(want, pos, 1e4, rot)
            if far:
                assert torch.allclose(got.double().cpu(), want, **far), nm
            else:
                close(got.float().cpu(), want, dtype, nm)
        close(kv[:, G:].float().cpu(), src[:, H + G:], dtype, "v passes")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(19, 100, 2), (8, 1024, 0), (100, 1024, 4), (3, 4096, 0)])
def test_gated_sums_depth_average_and_norm_in_one_kernel(dtype, sizes):
    """X = x + sigmoid(g1 + b1) d1 + sigmoid(g2 + b2) d2 is stored among the earlier results, the
    stream becomes their weighted sum and is normalised; terms as activations and as stacks of
    partial sums, one term, no gate, no average, a row list."""
    from grout_b200.kernels import ops
    (T, N, g0), n_hist = sizes, 11       # (rows that are no multiple of four take single loads; few rows of a
    x = rnd(T, N, seed=1)                #  wide stream a cluster of blocks each; more than eight earlier results)
    d1, d2 = rnd(T, N, seed=2).to(dtype), rnd(3, T, N, seed=3)
    gates = rnd(T, 2 * N + 8, seed=4, scale=2.0)
    b1, b2 = rnd(N, seed=5), rnd(N, seed=6)
    hist = rnd(n_hist + 2, T, N, seed=7)
    aw, nw = rnd(n_hist + 1, seed=8), 1 + rnd(N, seed=9, scale=0.2)
    X = (x.double() + torch.sigmoid(gates.double()[:, g0:g0 + N] + b1.double()) * d1.double()
         + torch.sigmoid(gates.double()[:, g0 + N:g0 + 2 * N] + b2.double()) * d2.double().sum(0))
    avg = plain.depth_average(list(hist[:n_hist].double()) + [X], aw)
    y_want = plain.rms(avg, 1e-5) * nw.double()
    hd, gd = hist.to(DEV).clone(), gates.to(DEV)
    res, y = ops.gated_norm(x.to(DEV).clone(), [(d1.to(DEV), gd[:, g0:g0 + N], b1.to(DEV)),
                                                (d2.to(DEV), gd[:, g0 + N:g0 + 2 * N], b2.to(DEV))],
                            dtype=dtype, hist=hd, n_hist=n_hist, avg_w=aw.to(DEV), norm_w=nw.to(DEV), eps=1e-5)
    close(hd[n_hist].cpu(), X, torch.float32, "the layer's result among the earlier ones")
    assert torch.equal(hd[n_hist + 1].cpu(), hist[n_hist + 1])
    close(res.cpu(), avg, torch.float32, "the stream")
    close(y.float().cpu(), y_want, dtype, "normalised")
    rows = torch.tensor([2, 0, T - 1], dtype=torch.int32)
    hd2 = hist.to(DEV).clone()
    res2, y2 = ops.gated_norm(x.to(DEV), [(d1.to(DEV), gd[:, g0:g0 + N], b1.to(DEV)),
                                          (d2.to(DEV), gd[:, g0 + N:g0 + 2 * N], b2.to(DEV))],
                              dtype=dtype, hist=hd2, n_hist=n_hist, avg_w=aw.to(DEV), rows=rows.to(DEV),
                              norm_w=nw.to(DEV), eps=1e-5)
    close(res2.cpu(), avg[rows.long()], torch.float32, "picked rows")
    close(y2.float().cpu(), y_want[rows.long()], dtype, "picked rows, normalised")
    assert torch.equal(hd2.cpu(), hist)                       # a gather stores nothing
    # one ungated term, no average, no norm: the sum itself, rounded
    res3, y3 = ops.gated_norm(x.to(DEV).clone(), [(d1.to(DEV), None, None)], dtype=dtype)
    close(res3.cpu(), x.double() + d1.double(), torch.float32)
    close(y3.float().cpu(), x.double() + d1.double(), dtype)


def test_the_norm_part_resolves_what_its_kernel_does_not_take():
    """A depth average in front of a norm without a kernel for it, and contributions that carry a
    factor of their own: resolved step by step to the same numbers."""
    from grout_b200.parts import Averaged, BuildContext, Contribution, PartSpec, build_part
    T, N = 6, 40
    ctx = BuildContext(torch.float32, torch.device(DEV))
    norm = build_part("norm", PartSpec("rmsnorm", dict(dim=N, eps=1e-5, name="w", unit_offset=True)), ctx)
    wz = rnd(N, seed=1, scale=0.3)
    norm.load({"w": wz.to(DEV)})
    x, d = rnd(T, N, seed=2), rnd(T, N, seed=3)
    g = rnd(T, N, seed=4)
    hist = rnd(3, T, N, seed=5).to(DEV)
    aw = rnd(3, seed=6)
    X = x.double() + 0.5 * torch.sigmoid(g.double()) * d.double()
    avg = plain.depth_average([hist[0].double().cpu(), hist[1].double().cpu(), X], aw)
    pending = Averaged((Contribution(d.to(DEV), mult=0.5, gate=g.to(DEV)),), hist, 2, aw.to(DEV))
    res, y = norm.add_norm(x.to(DEV).clone(), pending)
    close(res.cpu(), avg, torch.float32)
    close(y.cpu(), plain.norm_around_zero(avg, wz, 1e-5), torch.float32)
    layer = build_part("norm", PartSpec("layernorm", dict(dim=N, eps=1e-5)), ctx)
    layer.load({"weight": torch.ones(N, device=DEV), "bias": torch.zeros(N, device=DEV)})
    hist2 = hist.clone()
    res2, _y = layer.add_norm(x.to(DEV).clone(), Averaged((Contribution(d.to(DEV), mult=0.5, gate=g.to(DEV)),),
                                                          hist2, 2, aw.to(DEV)))
    close(res2.cpu(), avg, torch.float32)


# ------------------------------------------------------------------ routed experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(6, 2, 24, 64), (1, 1, 16, 40), (9, 9, 8, 48), (64, 3, 16, 32)])
def test_experts_chosen_by_logits_and_weighed_by_the_softmax_over_the_chosen(dtype, shape):
    from grout_b200.parts import BuildContext, PartSpec, build_part
    E, top, F, W = shape
    T = 70
    w = {"router": rnd(E, W, seed=1, scale=0.5), "router.b": rnd(E, seed=2, scale=2.0)}
    for e in range(E):
        w[f"e{e}.gate"] = rnd(F, W, seed=10 + 3 * e, scale=0.3)
        w[f"e{e}.up"] = rnd(F, W, seed=11 + 3 * e, scale=0.3)
        w[f"e{e}.down"] = rnd(W, F, seed=12 + 3 * e, scale=0.3)
    w = {k: v.to(dtype) for k, v in w.items()}
    x = rnd(T, W, seed=5).to(dtype)
    mlp = {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": top}}
    pw = {"m." + k: v for k, v in w.items()}
    want = plain.experts_feed_forward(x.double(), pw, mlp, "m.")
    if E > top:
        no_bias = plain.experts_feed_forward(x.double(), dict(pw, **{"m.router.b": w["router.b"] * 0}), mlp, "m.")
        assert float((no_bias - want).abs().max()) > 0.1 * float(want.abs().max())      # the bias chooses
    part = build_part("feedforward", PartSpec("routed_experts", dict(
        hidden=W, intermediate=F, n_experts=E, top=top, limit=None, gate_slope=1.0, up_offset=0.0,
        score_fn="softmax_top", correction=False, router_bias=True, router_bias_name="router.b")),
        BuildContext(dtype, torch.device(DEV)))
    part.load({k: v.to(DEV) for k, v in w.items()})
    got = part.forward(x.to(DEV), None)
    assert got.dtype == torch.float32 and tuple(got.shape) == (top, T, W)
    got = got.sum(0).double().cpu()
    if dtype == torch.float32:
        close(got, want, dtype)
    else:
        # a near tie between two experts may fall the other way after rounding: most rows agree
        rows = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
        assert float(rows.median()) < 0.02 and float((rows < 0.05).double().mean()) > 0.9
    # a token's result does not depend on the rows around it
    alone = part.forward(x[11:12].to(DEV), None).sum(0).double().cpu()
    assert torch.allclose(alone[0], got[11], atol=1e-5 if dtype == torch.float32 else 2e-2, rtol=1e-3)
