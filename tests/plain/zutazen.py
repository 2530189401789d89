"""Plain Zutazen decoder: whole sequences, no cache, one function per mechanism.

Zutazen is a pre-norm decoder, x <- x + M(N1(x)); x <- x + F(N2(x)) (the second
line only where the layer has an F), whose stream starts as E[token] * c.  A
layer's mixer M is one of

* retention: a matrix-valued state per head that fades by a fixed factor a
  token and is read without a softmax,
* a gated linear recurrence per channel behind a short causal convolution
  (two branches, the second a gelu gate), whose decay and input gate come from
  block-diagonal matrices,
* attention over a window of the last tokens whose keys and values are both
  expanded from one small latent vector per token, plus one short rotated key
  that all heads share, with a sigmoid gate on the heads' output.

F is a gated feed-forward with biases (relu gate) or a mixture of small gated
experts without biases (silu gate) whose router scores are sigmoids and weigh
the expert's *input*.  A layer may run another layer's weights on a state of
its own.

All arithmetic is float64 on the CPU.  Inputs are a dict ``name -> tensor`` with
the checkpoint's tensor names and the raw ``config.json`` dict.  Nothing here is
shared with the product package.
"""
from __future__ import annotations

import math

import torch

DT = torch.float64
LOG_DECAY_FACTOR = 8.0        # log a = -8 r softplus(lam) in the gated recurrence


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w (w may be None)."""
    x = x.to(DT)
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + float(eps))
    return y if w is None else y * w.to(DT)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, positions, base, dims, interleaved):
    """Turns the first ``dims`` elements of the last axis of x [T, ..., D] by
    p * base^(-2i/dims).  Element i goes with element i + dims/2, or, when
    ``interleaved``, element 2i with element 2i + 1."""
    x = x.to(DT).clone()
    if not dims:
        return x
    half = dims // 2
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    ang = torch.as_tensor(positions, dtype=DT)[:, None] * f[None, :]         # [T, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    if interleaved:
        u, v = x[..., 0:dims:2].clone(), x[..., 1:dims:2].clone()
        x[..., 0:dims:2] = u * c - v * s
        x[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half].clone(), x[..., half:dims].clone()
        x[..., :half] = u * c - v * s
        x[..., half:dims] = v * c + u * s
    return x


def retention_head(q, k, v, decay, S=None):
    """One head.  q, k [T, dk]; v [T, dv]; S <- decay S + k v^T; o = S^T q."""
    q, k, v = q.to(DT), k.to(DT), v.to(DT)
    S = torch.zeros(k.shape[1], v.shape[1], dtype=DT) if S is None else S.to(DT)
    out = []
    for t in range(q.shape[0]):
        S = float(decay) * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out), S


def retention_mixer(h, W, prefix, m, eps, first_pos=0):
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    h = h.to(DT)
    g = lambda n: W[prefix + n].to(DT)
    T = h.shape[0]
    pos = torch.arange(first_pos, first_pos + T)
    rot = m["rot"]
    q = rotate((h @ g("q").T).view(T, H, dk), pos, rot["base"], rot["dims"], False)
    k = rotate((h @ g("k").T).view(T, H, dk), pos, rot["base"], rot["dims"], False) * dk ** -0.5
    v = (h @ g("v").T).view(T, H, dv)
    gate = silu(h @ g("g").T).view(T, H, dv)
    outs = []
    for i in range(H):
        o, _S = retention_head(q[:, i], k[:, i], v[:, i], m["decay"][i])
        outs.append(rms_norm(o, None, eps) * gate[:, i])
    return torch.cat(outs, dim=-1) @ g("o").T


def causal_conv(x, taps_w, bias):
    """x [T, C], taps_w [C, taps]; y[t, c] = bias[c] + sum_j taps_w[c, taps-1-j] x[t-j, c]."""
    T, C = x.shape
    taps = taps_w.shape[1]
    y = torch.zeros(T, C, dtype=DT) + bias.to(DT)
    for j in range(min(taps, T)):
        y[j:] += taps_w.to(DT)[:, taps - 1 - j] * x.to(DT)[:T - j]
    return y


def block_diagonal(u, w, b):
    """u [T, C] cut into w.shape[0] equal parts; part i is multiplied by w[i] [out, in]."""
    nb, bw = w.shape[0], w.shape[1]
    parts = u.to(DT).view(u.shape[0], nb, bw)
    return (torch.einsum("tbi,boi->tbo", parts, w.to(DT)) + b.to(DT)).reshape(u.shape[0], nb * bw)


def gated_recurrence(u, r, i, lam):
    """Per channel: a = exp(-8 r softplus(lam)); S <- a S + sqrt(1 - a^2) i u, from S = 0."""
    log_a = -LOG_DECAY_FACTOR * r.to(DT) * torch.nn.functional.softplus(lam.to(DT))
    a = torch.exp(log_a)
    x = torch.sqrt(1.0 - a * a) * i.to(DT) * u.to(DT)
    S = torch.zeros(u.shape[1], dtype=DT)
    out = []
    for t in range(u.shape[0]):
        S = a[t] * S + x[t]
        out.append(S)
    return torch.stack(out)


def rglru_mixer(h, W, prefix, m):
    h = h.to(DT)
    g = lambda n: W[prefix + n].to(DT)
    y = gelu_tanh(h @ g("y").T + g("y.b"))
    u = causal_conv(h @ g("x").T + g("x.b"), g("conv"), g("conv.b"))
    r = torch.sigmoid(block_diagonal(u, g("ra"), g("ra.b")))
    i = torch.sigmoid(block_diagonal(u, g("ri"), g("ri.b")))
    S = gated_recurrence(u, r, i, g("lam"))
    return (S * y) @ g("o").T


def windowed_softmax_attention(q, k, v, scale, window):
    """One head.  Row i sees rows j with 0 <= i - j < window."""
    q, k, v = q.to(DT), k.to(DT), v.to(DT)
    T = q.shape[0]
    s = (q @ k.T) * float(scale)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    s = s.masked_fill(~((i - j >= 0) & (i - j < int(window))), -math.inf)
    return torch.softmax(s, dim=-1) @ v


def latent_attention_mixer(h, W, prefix, m, eps, first_pos=0):
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    h = h.to(DT)
    g = lambda n: W[prefix + n].to(DT)
    T = h.shape[0]
    pos = torch.arange(first_pos, first_pos + T)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    window = m["mask"]["size"] if m.get("mask") else T + 1
    q = (h @ g("q").T).view(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate(q[..., dn:], pos, rot["base"], rot["dims"], True)
    down = h @ g("dkv").T
    c = rms_norm(down[:, :R], g("dkv.norm"), eps)
    k_rot = rotate(down[:, R:], pos, rot["base"], rot["dims"], True)              # [T, dr], all heads
    k_plain = (c @ g("uk").T).view(T, H, dn)
    v = (c @ g("uv").T).view(T, H, dv)
    gate = torch.sigmoid(h @ g("g").T).view(T, H, dv)
    outs = []
    for i in range(H):
        qi = torch.cat([q_plain[:, i], q_rot[:, i]], dim=-1)
        ki = torch.cat([k_plain[:, i], k_rot], dim=-1)
        outs.append(windowed_softmax_attention(qi, ki, v[:, i], m["scale"], window) * gate[:, i])
    return torch.cat(outs, dim=-1) @ g("o").T


def dense_ff(h, W, prefix):
    h = h.to(DT)
    g = lambda n: W[prefix + n].to(DT)
    a = torch.relu(h @ g("gate").T + g("gate.b"))
    return (a * (h @ g("up").T + g("up.b"))) @ g("down").T + g("down.b")


def route(h, router_w, top):
    """Sigmoid scores, the ``top`` largest, the scores themselves as weights."""
    s = torch.sigmoid(h.to(DT) @ router_w.to(DT).T)
    w, idx = torch.topk(s, int(top), dim=-1)
    return idx, w


def expert_ff(h, W, prefix):
    g = lambda n: W[prefix + n].to(DT)
    return (silu(h @ g("gate").T) * (h @ g("up").T)) @ g("down").T


def routed_ff(h, W, prefix, mlp):
    h = h.to(DT)
    idx, w = route(h, W[prefix + "router"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(idx[t].tolist(), w[t]):
            out[t] += expert_ff((we * h[t])[None], W, f"{prefix}e{e}.")[0]
    return out


def forward(tokens, W, cfg, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token."""
    eps = cfg["norm"]["eps"]
    x = W["embed"].to(DT)[torch.as_tensor(tokens)] * float(cfg["embedding"]["scale"])
    after = []
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        layer = cfg["layers"][src]
        p = f"l{src}."
        h = rms_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "retention":
            x = x + retention_mixer(h, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "rglru":
            x = x + rglru_mixer(h, W, p + "mix.", layer["mixer"])
        else:
            x = x + latent_attention_mixer(h, W, p + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            x = x + (dense_ff(h, W, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, W, p + "mlp.", mlp))
        after.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].to(DT).T
    return (logits, torch.stack(after)) if return_layers else logits


def logits(W, cfg, tokens, rows=None):
    out = forward(list(tokens), W, cfg)
    return out if rows is None else out[list(rows)]


def greedy_generate(W, cfg, prompt, n_new, stop_ids=()):
    """The plain loop: the whole sequence is recomputed for every new token."""
    seq, made = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(seq, W, cfg)[-1]))
        if tok in stop_ids:          # a stop token ends the request and is not part of its output
            break
        made.append(tok)
        seq.append(tok)
    return made
