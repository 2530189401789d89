"""Plain Mananex decoder: whole sequences, no cache, one function per mechanism.

Mananex is a decoder of "parallel" layers on a depth-averaged stream.  With X_0 the
embedded tokens, layer i reads x (the average that the layer before it left, or X_0),
computes h = N(x) once, and both of its sublayers read h:

    X_(i+1) = x + sigmoid(R1 h + r1) * M(h) + sigmoid(R2 h + r2) * F(h)
    x      <- sum over j = 0 .. i+1 of a_i[j] * X_j          (a_i: the layer's learned weights)

N is an RMS norm whose weight is stored around zero (x / rms * (1 + w)).  The mixer M
runs two mixers side by side on the same h and adds them with constant factors:

* left: grouped-query attention with a rotation of neighbouring pairs on the first
  ``rot.dims`` elements of every q and k head, a sliding window that also keeps the
  sequence's first ``keep_first`` tokens, a learned sink per head in the softmax's
  denominator, and a sigmoid gate per head (one number a head) on the output;
* right: a linear attention whose forget gate f (bounded below by a learned floor)
  also decides what is written: S <- diag(f) S + (1 - f) v^T, o = S^T q with
  q = silu(Wq h), then an RMS norm per head.

F is a silu-gated feed-forward with biases or a mixture of small silu-gated experts
whose router (with a bias) takes the ``top`` largest logits and weighs the chosen
experts by the softmax over those logits alone.  The logits come from the embedding
table itself after a last norm.

All arithmetic is float64 on the CPU.  Inputs are a dict ``name -> tensor`` with the
checkpoint's tensor names and the raw ``config.json`` dict.  Nothing here is shared
with the product package.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def rms(x, eps):
    x = x.to(DT)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + float(eps))


def norm_around_zero(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w)."""
    return rms(x, eps) * (1.0 + w.to(DT))


def norm_plain(x, w, eps):
    return rms(x, eps) * w.to(DT)


def silu(z):
    return z * torch.sigmoid(z)


def rotate_neighbours(x, positions, base, dims):
    """Turns elements (2i, 2i+1), i < dims/2, of the last axis of x [T, heads, D] by
    the angle p * base^(-2i/dims); elements from ``dims`` on pass unchanged."""
    x = x.to(DT).clone()
    if not dims:
        return x
    half = dims // 2
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    ang = torch.as_tensor(positions, dtype=DT)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2].clone(), x[..., 1:dims:2].clone()
    x[..., 0:dims:2] = u * c - v * s
    x[..., 1:dims:2] = v * c + u * s
    return x


def visible(i, j, size, keep_first):
    """Whether the query at position i sees the key at position j."""
    return j <= i and ((size is None or i - j < size) or j < keep_first)


def visibility(positions, size, keep_first):
    """[T, T] bool: row i, column j is ``visible(positions[i], positions[j], ...)``."""
    p = torch.as_tensor(positions, dtype=torch.long)
    i, j = p[:, None], p[None, :]
    near = torch.ones_like(i - j, dtype=torch.bool) if size is None else (i - j < size)
    return (j <= i) & (near | (j < keep_first))


def windowed_attention(h, positions, w, m, prefix=""):
    """The left mixer on h [T, width] with the tensors ``prefix + q/k/v/o/sink/g``."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].to(DT).T).view(T, H, D)
    k = (h @ w[prefix + "k"].to(DT).T).view(T, G, D)
    v = (h @ w[prefix + "v"].to(DT).T).view(T, G, Dv)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = rotate_neighbours(q, positions, rot["base"], rot["dims"])
        k = rotate_neighbours(k, positions, rot["base"], rot["dims"])
    mask = m.get("mask") or {}
    size, keep = mask.get("size"), int(mask.get("keep_first", 0))
    see = visibility(positions, size, keep)
    sink = w[prefix + "sink"].to(DT)
    gate = torch.sigmoid(h @ w[prefix + "g"].to(DT).T)                  # [T, H]
    out = torch.zeros(T, H, Dv, dtype=DT)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~see, -math.inf)
        top = torch.maximum(s.max(dim=-1).values, sink[a].expand(T))
        e = torch.exp(s - top[:, None])
        p = e / (e.sum(dim=-1) + torch.exp(sink[a] - top))[:, None]
        out[:, a] = (p @ v[:, g]) * gate[:, a:a + 1]
    return out.reshape(T, H * Dv) @ w[prefix + "o"].to(DT).T


def forgetful_linear_attention(h, w, m, eps, prefix="", state=None):
    """The right mixer.  Returns (output [T, width], the state after the last row)."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[prefix + "q"].to(DT).T).view(T, H, dk)
    v = (h @ w[prefix + "v"].to(DT).T).view(T, H, dv)
    low = w[prefix + "lower"].to(DT)
    f = low + (1.0 - low) * torch.sigmoid(h @ w[prefix + "f"].to(DT).T + w[prefix + "f.b"].to(DT))
    f = f.view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=DT) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=DT)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = norm_plain(o, w[prefix + "norm"], eps)
    return o.reshape(T, H * dv) @ w[prefix + "o"].to(DT).T, S


def two_mixers(h, positions, w, m, eps, prefix):
    left = windowed_attention(h, positions, w, m["left"], prefix + "left.")
    right, _ = forgetful_linear_attention(h, w, m["right"], eps, prefix + "right.")
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def dense_feed_forward(h, w, prefix):
    g = h @ w[prefix + "gate"].to(DT).T + w[prefix + "gate.b"].to(DT)
    u = h @ w[prefix + "up"].to(DT).T + w[prefix + "up.b"].to(DT)
    return (silu(g) * u) @ w[prefix + "down"].to(DT).T + w[prefix + "down.b"].to(DT)


def route(h, w, prefix, top):
    """(chosen experts [T, top], their weights [T, top])."""
    z = h @ w[prefix + "router"].to(DT).T + w[prefix + "router.b"].to(DT)
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def experts_feed_forward(h, w, mlp, prefix):
    idx, wt = route(h, w, prefix, int(mlp["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(idx[t].tolist(), wt[t]):
            pre = f"{prefix}e{e}."
            g = w[pre + "gate"].to(DT) @ h[t]
            u = w[pre + "up"].to(DT) @ h[t]
            out[t] += p * (w[pre + "down"].to(DT) @ (silu(g) * u))
    return out


def feed_forward(h, w, mlp, prefix):
    if mlp["kind"] == "dense":
        return dense_feed_forward(h, w, prefix)
    return experts_feed_forward(h, w, mlp, prefix)


def residual_gate(h, w, name):
    return torch.sigmoid(h @ w[name].to(DT).T + w[name + ".b"].to(DT))


def layer(x, positions, w, cfg, i):
    """X_(i+1) from the layer's input x."""
    spec, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    h = norm_around_zero(x, w[p + "norm1"], eps)
    out = x + residual_gate(h, w, p + "rg1") * two_mixers(h, positions, w, spec["mixer"], eps, p + "mix.")
    if spec.get("mlp") is not None:
        out = out + residual_gate(h, w, p + "rg2") * feed_forward(h, w, spec["mlp"], p + "mlp.")
    return out


def depth_average(history, weights):
    """sum_j weights[j] * history[j]."""
    return sum(float(a) * X for a, X in zip(weights.to(DT), history))


def forward(tokens, w, cfg, positions=None, streams=None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) receives the stream
    after every layer."""
    T = len(tokens)
    positions = list(range(T)) if positions is None else positions
    x = w["embed"].to(DT)[torch.as_tensor(tokens, dtype=torch.long)]
    history = [x]
    for i in range(len(cfg["layers"])):
        history.append(layer(x, positions, w, cfg, i))
        x = depth_average(history, w[f"l{i}.dwa"])
        if streams is not None:
            streams.append(x)
    h = norm_around_zero(x, w["final.norm"], cfg["norm"]["eps"])
    return h @ w["embed"].to(DT).T


def logits(w, cfg, tokens, rows=None):
    out = forward(tokens, w, cfg)
    return out if rows is None else out[list(rows)]


def greedy_generate(w, cfg, prompt, n_new, stop_ids=()):
    """The first-maximum token after each step, the whole sequence run again every time."""
    seq, new = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(logits(w, cfg, seq, rows=[len(seq) - 1])[0]))
        if tok in stop_ids:          # a stop token ends the request and is not part of its output
            break
        new.append(tok)
        seq.append(tok)
    return new
