"""Mixers that carry a state of fixed size from token to token instead of keys
and values.  Their cache need is a ``StateSpec``: one row of 32-bit floats per
sequence and layer, zero when the sequence starts; the rows of a sequence are
walked in order (``step.cu_q``), so the state after a prompt is the same
whether its tokens came in one step, in portions or one by one.
"""
from __future__ import annotations

import torch

from ..cache.spec import StateSpec
from ..kernels import ops
from .base import BuildContext, ParamSpec, PartSpec, build_part, register_part
from .linear import Linear
from .mixer import Mixer
from .position import PositionEncoding


@register_part("mixer", "gated_delta")
class GatedDelta(Mixer):
    """The gated delta rule.  With h the mixer's input,

        q = Wq h, k = Wk h  (n_kv_heads x key_dim),  v = Wv h  (n_heads x value_dim)
        each through a causal convolution over time of ``conv_taps`` taps per channel
        (no bias, zeros before the sequence's start; the last tap is the current
        token's), then silu;  q and k made unit vectors per head,
        x / sqrt(sum(x^2) + unit_eps), q also times key_dim^(-1/2)
        beta = sigmoid(Wb h),  g = exp(-exp(A_log) softplus(Wa h + dt_bias))   per head
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q            per head
        y = Wo [ o / sqrt(mean(o^2) + norm_eps) * w * silu(Wg h) ]

    Head i reads q and k of kv head i // (n_heads / n_kv_heads); the norm's weight
    w [value_dim] is shared by the heads.  S [key_dim, value_dim] starts at zero and
    is kept, with the last ``conv_taps - 1`` inputs of the convolutions, per
    sequence.  The six projections are one product, which leaves 32-bit sums; all
    that follows up to y is 32-bit whatever the activation type.  ``names``
    replaces local tensor names (keys q, k, v, q_conv, k_conv, v_conv, b, a, A_log,
    dt_bias, g, norm, o)."""

    NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv",
             "v_conv": "v.conv", "b": "b", "a": "a", "A_log": "A_log", "dt_bias": "dt_bias",
             "g": "g", "norm": "norm", "o": "o"}

    def __init__(self, ctx: BuildContext, hidden: int, n_heads: int, n_kv_heads: int, key_dim: int,
                 value_dim: int, conv_taps: int, norm_eps: float, unit_eps: float = 1e-6,
                 names=None):
        super().__init__(ctx)
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} kv heads")
        if conv_taps < 1:
            raise ValueError("a convolution has at least one tap")
        self.hidden, self.H, self.G = int(hidden), int(n_heads), int(n_kv_heads)
        self.dk, self.dv, self.taps = int(key_dim), int(value_dim), int(conv_taps)
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.names = dict(self.NAMES, **(names or {}))
        self.proj = self.o = None
        self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def param_specs(self):
        W, H, G, dk, dv, nm = self.hidden, self.H, self.G, self.dk, self.dv, self.names
        return {nm["q"]: ParamSpec((G * dk, W)), nm["k"]: ParamSpec((G * dk, W)),
                nm["v"]: ParamSpec((H * dv, W)), nm["g"]: ParamSpec((H * dv, W)),
                nm["b"]: ParamSpec((H, W)), nm["a"]: ParamSpec((H, W)),
                nm["q_conv"]: ParamSpec((G * dk, self.taps), "vector"),
                nm["k_conv"]: ParamSpec((G * dk, self.taps), "vector"),
                nm["v_conv"]: ParamSpec((H * dv, self.taps), "vector"),
                nm["A_log"]: ParamSpec((H,), "offset"), nm["dt_bias"]: ParamSpec((H,), "offset"),
                nm["norm"]: ParamSpec((dv,), "vector"), nm["o"]: ParamSpec((W, H * dv))}

    def load(self, params):
        nm = self.names
        ws = [params[nm[k]] for k in ("q", "k", "v", "g", "b", "a")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the projections of one mixer must be stored in one dtype to be fused")
        self.proj = Linear(torch.cat(ws, dim=0), self.ctx.products)
        self.o = Linear(params[nm["o"]], self.ctx.products)
        # what enters the recurrence is 32-bit whatever the checkpoint stores
        f32 = lambda t: t.float().contiguous()
        self.conv_w = f32(torch.cat([params[nm[k]] for k in ("q_conv", "k_conv", "v_conv")], dim=0))
        self.a_log, self.dt_bias = f32(params[nm["A_log"]]), f32(params[nm["dt_bias"]])
        self.norm_w = f32(params[nm["norm"]])

    def kernel_modules(self):
        return ("delta",) + self.proj.kernel_modules() + self.o.kernel_modules()

    def cache_spec(self):
        return StateSpec((ops.delta_state_floats(self.H, self.G, self.dk, self.dv, self.taps),),
                         torch.float32)

    def captures_prompts(self):
        return True

    def forward(self, x, step, cache):
        if cache is None or tuple(cache.spec.shape) != tuple(self.cache_spec().shape):
            raise ValueError(f"the gated delta rule was given the cache "
                             f"{None if cache is None else cache.spec}")
        proj = self.proj(x, out_dtype=torch.float32)
        y = ops.delta_forward(proj, cache.state, self.conv_w, self.a_log, self.dt_bias,
                              self.norm_w, H=self.H, G=self.G, dk=self.dk, dv=self.dv,
                              taps=self.taps, unit_eps=self.unit_eps, norm_eps=self.norm_eps,
                              token_seq=step.token_seq, cu_q=step.cu_q, slots=step.slots,
                              dtype=self.ctx.dtype, max_rows=step.max_q_len)
        return self.o(y, partial_ok=True)


@register_part("mixer", "retention")
class Retention(Mixer):
    """Linear attention with a fixed decay per head and neither softmax nor
    denominator.  With h the mixer's input,

        q = Wq h, k = Wk h  (n_heads x key_dim),  v = Wv h  (n_heads x value_dim)
        q, k rotated by ``position`` (a rotation of half-split pairs), k then times ``k_scale``
        S <- decay_i S + k v^T;  o = S^T q                                    per head i
        y = Wo [ o / sqrt(mean(o^2) + norm_eps) * silu(Wg h) ]                (no norm weight)

    ``decay`` holds one constant per head.  S [key_dim, value_dim] starts at zero and
    is kept per sequence in 32-bit.  The four projections are one product, which leaves
    32-bit sums; all that follows up to y is 32-bit whatever the activation type.
    ``names`` replaces local tensor names (keys q, k, v, g, o)."""

    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}

    def __init__(self, ctx: BuildContext, hidden: int, n_heads: int, key_dim: int, value_dim: int,
                 decay, position: PartSpec, norm_eps: float, k_scale: float = None, names=None):
        super().__init__(ctx)
        self.hidden, self.H, self.dk, self.dv = int(hidden), int(n_heads), int(key_dim), int(value_dim)
        self.decay_values = tuple(float(d) for d in decay)
        if len(self.decay_values) != self.H:
            raise ValueError(f"{len(self.decay_values)} decays for {self.H} heads")
        self.norm_eps = float(norm_eps)
        self.k_scale = float(k_scale) if k_scale is not None else self.dk ** -0.5
        self.names = dict(self.NAMES, **(names or {}))
        self.position = build_part("position", position, ctx)
        rot = self.position.rotary()
        if rot is None and type(self.position).apply_qk is not PositionEncoding.apply_qk:
            raise ValueError("retention takes a rotation (or no position encoding)")
        if rot is not None and (rot.interleaved or rot.rot_dim > self.dk):
            raise ValueError("retention rotates half-split pairs within a head's keys")
        self.proj = self.o = self.decay = None

    def children(self):
        return (self.position,)

    def param_specs(self):
        W, H, dk, dv, nm = self.hidden, self.H, self.dk, self.dv, self.names
        return {nm["q"]: ParamSpec((H * dk, W)), nm["k"]: ParamSpec((H * dk, W)),
                nm["v"]: ParamSpec((H * dv, W)), nm["g"]: ParamSpec((H * dv, W)),
                nm["o"]: ParamSpec((W, H * dv))}

    def load(self, params):
        nm = self.names
        ws = [params[nm[k]] for k in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the projections of one mixer must be stored in one dtype to be fused")
        self.proj = Linear(torch.cat(ws, dim=0), self.ctx.products)
        self.o = Linear(params[nm["o"]], self.ctx.products)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=ws[0].device)

    def kernel_modules(self):
        return ("retention",) + self.proj.kernel_modules() + self.o.kernel_modules()

    def cache_spec(self):
        return StateSpec((self.H * self.dk * self.dv,), torch.float32)

    def captures_prompts(self):
        return True

    def forward(self, x, step, cache):
        if cache is None or tuple(cache.spec.shape) != tuple(self.cache_spec().shape):
            raise ValueError(f"retention was given the cache {None if cache is None else cache.spec}")
        rot = self.position.rotary()
        proj = self.proj(x, out_dtype=torch.float32)
        y = ops.retention_forward(proj, cache.state, self.decay, rot.inv_freq if rot else None,
                                  H=self.H, dk=self.dk, dv=self.dv, rot_dim=rot.rot_dim if rot else 0,
                                  k_scale=self.k_scale, norm_eps=self.norm_eps,
                                  token_pos=step.token_pos, cu_q=step.cu_q, slots=step.slots,
                                  dtype=self.ctx.dtype, max_rows=step.max_q_len)
        return self.o(y, partial_ok=True)


@register_part("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    """The recurrent block of Griffin: two branches of ``width`` channels,

        y = gelu_tanh(Wy h + by);   u = conv(Wx h + bx)
        (a causal convolution per channel of ``conv_taps`` taps with a bias, zeros
        before the sequence's start, the last tap the current token's, no activation)
        r = sigmoid(Wa_b u_b + ba),  i = sigmoid(Wi_b u_b + bi)
        (the channels form ``blocks`` equal parts, part b with square matrices of its own)
        a = exp(-log_decay_factor r softplus(lam));   S <- a S + sqrt(1 - a^2) i u
        out = Wo (S * y)

    S starts at zero (the first token is no special case) and is kept per sequence in
    32-bit together with the convolution's last ``conv_taps - 1`` inputs.  The two
    branches are one product that leaves 32-bit sums; all that follows up to S * y is
    32-bit.  ``names`` replaces local tensor names (keys y, y_bias, x, x_bias, conv,
    conv_bias, a, a_bias, i, i_bias, lam, o)."""

    NAMES = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv",
             "conv_bias": "conv.b", "a": "ra", "a_bias": "ra.b", "i": "ri", "i_bias": "ri.b",
             "lam": "lam", "o": "o"}

    def __init__(self, ctx: BuildContext, hidden: int, width: int, blocks: int, conv_taps: int,
                 log_decay_factor: float = 8.0, names=None):
        super().__init__(ctx)
        self.hidden, self.C, self.blocks, self.taps = int(hidden), int(width), int(blocks), int(conv_taps)
        if self.blocks < 1 or self.C % self.blocks:
            raise ValueError(f"{self.C} channels do not form {self.blocks} equal parts")
        if self.taps < 1:
            raise ValueError("a convolution has at least one tap")
        self.factor = float(log_decay_factor)
        self.names = dict(self.NAMES, **(names or {}))
        self.proj = self.o = None
        self.bias = self.conv_w = self.conv_b = self.wa_t = self.wi_t = self.ba = self.bi = self.lam = None

    def param_specs(self):
        W, C, nb, nm = self.hidden, self.C, self.blocks, self.names
        bw = C // nb
        return {nm["y"]: ParamSpec((C, W)), nm["y_bias"]: ParamSpec((C,), "offset"),
                nm["x"]: ParamSpec((C, W)), nm["x_bias"]: ParamSpec((C,), "offset"),
                nm["conv"]: ParamSpec((C, self.taps), "vector"), nm["conv_bias"]: ParamSpec((C,), "offset"),
                nm["a"]: ParamSpec((nb, bw, bw)), nm["a_bias"]: ParamSpec((nb, bw), "offset"),
                nm["i"]: ParamSpec((nb, bw, bw)), nm["i_bias"]: ParamSpec((nb, bw), "offset"),
                nm["lam"]: ParamSpec((C,), "offset"), nm["o"]: ParamSpec((W, C))}

    def load(self, params):
        nm = self.names
        wy, wx = params[nm["y"]], params[nm["x"]]
        if wy.dtype != wx.dtype:
            raise ValueError("the two branches must be stored in one dtype to be fused")
        self.proj = Linear(torch.cat([wy, wx], dim=0), self.ctx.products)
        self.o = Linear(params[nm["o"]], self.ctx.products)
        # what enters the recurrence is 32-bit whatever the checkpoint stores
        f32 = lambda t: t.float().contiguous()
        self.bias = f32(torch.cat([params[nm["y_bias"]].float(), params[nm["x_bias"]].float()]))
        self.conv_w, self.conv_b = f32(params[nm["conv"]]), f32(params[nm["conv_bias"]])
        # [part, out, in] -> [part, in, out]: a warp's threads read neighbouring outputs
        self.wa_t = f32(params[nm["a"]].float().transpose(1, 2))
        self.wi_t = f32(params[nm["i"]].float().transpose(1, 2))
        self.ba, self.bi = f32(params[nm["a_bias"]].reshape(-1)), f32(params[nm["i_bias"]].reshape(-1))
        self.lam = f32(params[nm["lam"]])

    def kernel_modules(self):
        return ("rglru",) + self.proj.kernel_modules() + self.o.kernel_modules()

    def cache_spec(self):
        return StateSpec((self.taps * self.C,), torch.float32)

    def captures_prompts(self):
        return True

    def forward(self, x, step, cache):
        if cache is None or tuple(cache.spec.shape) != tuple(self.cache_spec().shape):
            raise ValueError(f"the gated linear recurrence was given the cache "
                             f"{None if cache is None else cache.spec}")
        proj = self.proj(x, out_dtype=torch.float32)
        y = ops.rglru_forward(proj, cache.state, self.bias, self.conv_w, self.conv_b, self.wa_t,
                              self.ba, self.wi_t, self.bi, self.lam, blocks=self.blocks,
                              taps=self.taps, factor=self.factor, token_seq=step.token_seq,
                              cu_q=step.cu_q, slots=step.slots, dtype=self.ctx.dtype,
                              max_rows=step.max_q_len)
        return self.o(y, partial_ok=True)


@register_part("mixer", "forget_gate_attention")
class ForgetGateAttention(Mixer):
    """Linear attention in which the forget gate also decides what is written (HGRN2).
    With h the mixer's input,

        q = silu(Wq h)  (n_heads x key_dim),   v = Wv h  (n_heads x value_dim)
        f = low + (1 - low) * sigmoid(Wf h + bf)      per head and channel; ``low`` is a learned
                                                      lower bound of the gate, inside [0, 1)
        S <- diag(f) S + (1 - f) v^T;   o = S^T q     per head: there is no key, 1 - f stands
                                                      where one would, and no other scale
        y = Wo [ o / sqrt(mean(o^2) + norm_eps) * w ] the norm per head over value_dim, its
                                                      weight w [value_dim] shared by the heads

    S [key_dim, value_dim] starts at zero and is kept per sequence in 32-bit.  The three
    projections are one product that leaves 32-bit sums; all that follows up to y is 32-bit
    whatever the activation type.  ``names`` replaces local tensor names (keys q, f, f_bias,
    lower, v, norm, o).  The mixer can run beside another one (``SideBySide``)."""

    NAMES = {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o"}

    def __init__(self, ctx: BuildContext, hidden: int, n_heads: int, key_dim: int, value_dim: int,
                 norm_eps: float, names=None):
        super().__init__(ctx)
        self.hidden, self.H, self.dk, self.dv = int(hidden), int(n_heads), int(key_dim), int(value_dim)
        self.norm_eps = float(norm_eps)
        self.names = dict(self.NAMES, **(names or {}))
        self.beside = False          # set by a SideBySide parent before load
        self.proj = self.o = self.side_w = self.o_w = None
        self.f_bias = self.lower = self.norm_w = None

    def param_specs(self):
        W, H, dk, dv, nm = self.hidden, self.H, self.dk, self.dv, self.names
        return {nm["q"]: ParamSpec((H * dk, W)), nm["f"]: ParamSpec((H * dk, W)),
                nm["f_bias"]: ParamSpec((H * dk,), "offset"), nm["lower"]: ParamSpec((H * dk,), "fraction"),
                nm["v"]: ParamSpec((H * dv, W)), nm["norm"]: ParamSpec((dv,), "vector"),
                nm["o"]: ParamSpec((W, H * dv))}

    def load(self, params):
        nm = self.names
        ws = [params[nm[k]] for k in ("q", "f", "v")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the projections of one mixer must be stored in one dtype to be fused")
        side = torch.cat(ws, dim=0)
        if self.beside:              # the parent multiplies: one product for all its mixers
            self.side_w, self.o_w = side, params[nm["o"]]
        else:
            self.proj = Linear(side, self.ctx.products)
            self.o = Linear(params[nm["o"]], self.ctx.products)
        # what enters the recurrence is 32-bit whatever the checkpoint stores
        f32 = lambda t: t.float().contiguous()
        self.f_bias, self.lower = f32(params[nm["f_bias"]]), f32(params[nm["lower"]])
        self.norm_w = f32(params[nm["norm"]])

    def kernel_modules(self):
        mods = ("hgrn2",)
        for lin in (self.proj, self.o):
            mods += lin.kernel_modules() if lin else ()
        return mods

    def cache_spec(self):
        return StateSpec((self.H * self.dk * self.dv,), torch.float32)

    def captures_prompts(self):
        return True

    # -- beside another mixer ------------------------------------------------
    @property
    def inner_width(self) -> int:
        return self.H * self.dv

    def side_weight(self):
        return self.side_w

    def out_weight(self):
        return self.o_w

    def inner(self, x, step, cache, sums=None, out=None, mult: float = 1.0):
        """The o projection's input [T, n_heads * value_dim], times ``mult``, from ``sums``,
        the 32-bit products of ``side_weight`` (q | f | v rows) with x."""
        if cache is None or tuple(cache.spec.shape) != tuple(self.cache_spec().shape):
            raise ValueError(f"forget-gate attention was given the cache "
                             f"{None if cache is None else cache.spec}")
        H, dk, dv = self.H, self.dk, self.dv
        return ops.hgrn2_forward(sums, cache.state, self.f_bias, self.lower, self.norm_w, H=H, dk=dk,
                                 dv=dv, q_col=0, f_col=H * dk, v_col=2 * H * dk,
                                 norm_eps=self.norm_eps, cu_q=step.cu_q, slots=step.slots,
                                 dtype=self.ctx.dtype, out_scale=mult, into=out, max_rows=step.max_q_len)

    def forward(self, x, step, cache):
        y = self.inner(x, step, cache, self.proj(x, out_dtype=torch.float32))
        return self.o(y, partial_ok=True)
