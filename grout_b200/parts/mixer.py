"""Mixers: the part of a layer that lets tokens see other tokens.

Interface of the family:

* ``cache_spec()`` — ``KVSpec``, ``StateSpec`` or None: what one layer of this
  mixer keeps per sequence.  The cache groups layers with equal needs.
* ``forward(x, step, cache) -> y`` — ``x`` [T, hidden] in the compute dtype
  (``y`` may be a stack of 32-bit partial sums [S, T, hidden]: see ``Norm.add_norm``),
  ``step`` the ``StepContext`` (which sequence and position each row has),
  ``cache`` the layer's view of its store (``KVLayerView`` / ``StateLayerView``).
  It must store what later steps need (keys, values, state) for the rows of
  sequences whose slot is not negative, and return [T, hidden].
  A mixer with a recurrence walks each sequence's rows in order, using
  ``step.cu_q``; it must give the same state whether the tokens come in one
  step or one by one.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..cache.spec import KVSpec, SideBySideSpec
from ..kernels import ops
from .base import BuildContext, ParamSpec, Part, PartSpec, build_part, register_part
from .linear import Linear
from .position import PositionEncoding


class Mixer(Part):
    family = "mixer"

    def cache_spec(self):
        return None

    def forward(self, x, step, cache):
        raise NotImplementedError


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    """Causal grouped-query attention over the paged cache.

    q, k, v projections without bias (fused into one product at load, as the
    reference fuses them, src/model.rs:1396, 6021-6073); optional RMSNorm of
    every q and k head over head_dim with one weight vector shared by the heads,
    before the rotation (src/training.rs:318-331); the position encoding of the
    given spec; k and v stored at the token's position; scores q.k * scale with
    scale = 1/sqrt(head_dim) unless given (src/model.rs:2398); query head h reads
    kv head h // (heads / kv_heads) (src/kernels.rs:1166); keys up to the query's
    own position, or the last ``window`` of them; o projection.

    Further terms, each absent by default: ``softcap`` c replaces a score s by
    c * tanh(s / c) (after the scaling); ``sinks`` gives every query head a learned
    logit (tensor ``sink`` [heads]) that stands in the softmax's denominator as
    exp(sink) beside the keys' terms and has no value; ``values_are_keys`` takes
    the values to be the keys as projected, before the rotation (there is no v
    projection; the cache still holds both, the keys rotated).  ``sink_logit`` puts
    the same constant logit into every head's denominator instead of a learned one
    (0.0: one is added to the sum of exponentials).  ``q_temp`` = (coef, every)
    multiplies the query at position p, after its norm, by
    1 + coef * ln(floor((p + 1) / every) + 1).  ``v_head_dim``: values of another
    size than queries and keys; the cache, the queries and the attention's output
    are then as wide as the larger of the two, filled up with zeros, and the o
    projection's columns likewise, so that every attention kernel serves.
    ``keep_first`` F: with a window, the sequence's first F tokens stay visible to every
    later query, at their own positions (their pages are kept).  ``head_gate``: every
    head's output is multiplied by sigmoid(Wg h)_head, one number a head (tensor ``g``
    [heads, hidden]; 32-bit sums, 32-bit sigmoid), before the o projection.  A rotation
    of neighbouring pairs (``rotary_interleaved``) is folded into the q/k kernel as the
    half-split one is.
    ``names`` replaces local tensor names (keys: q, k, v, o, q_norm, k_norm, sink, g).

    The mixer can run beside another one on the same input (``SideBySide``): it then names
    the rows whose 32-bit products with the input it needs (``side_weight``: the head gate's),
    leaves the o projection's input in a view it is given (``inner``) and hands out its o
    weight (``out_weight``) instead of multiplying by it.
    """

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight",
             "o": "o_proj.weight", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight",
             "sink": "sink", "g": "g"}

    def __init__(self, ctx: BuildContext, hidden: int, n_heads: int, n_kv_heads: int,
                 head_dim: int, position: PartSpec, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, scale: Optional[float] = None,
                 shares_kv: bool = False, softcap: Optional[float] = None, sinks: bool = False,
                 values_are_keys: bool = False, names: Optional[dict] = None,
                 v_head_dim: Optional[int] = None, q_temp: Optional[tuple] = None,
                 sink_logit: Optional[float] = None, keep_first: int = 0, head_gate: bool = False):
        super().__init__(ctx)
        self.keep_first = int(keep_first or 0) if window else 0
        self.head_gate = bool(head_gate)
        self.beside = False          # set by a SideBySide parent before load
        self.g = self.g_w = self.o_w = None
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} kv heads")
        self.hidden, self.nq, self.nkv, self.D = int(hidden), int(n_heads), int(n_kv_heads), int(head_dim)
        self.Dv = int(v_head_dim) if v_head_dim else self.D
        # the width of a cached row, of a query and of the attention's output
        self.Ds = max(self.D, self.Dv)
        if self.Ds != self.D or self.Ds != self.Dv:
            if values_are_keys or shares_kv:
                raise ValueError("values of another size than the keys go with a v projection "
                                 "and a cache of the layer's own")
            if ctx.dtype == torch.bfloat16:       # the tensor-core kernels take multiples of 16
                self.Ds = (self.Ds + 15) // 16 * 16
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        if self.q_temp and self.q_temp[1] <= 0:
            raise ValueError("q_temp = (coef, every) with every >= 1")
        if sink_logit is not None and sinks:
            raise ValueError("either learned sinks or one constant sink logit")
        self.sink_logit = None if sink_logit is None else float(sink_logit)
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.D)
        # a layer that attends over another layer's keys and values projects
        # queries only, stores nothing and owns no cache (the schedule says whose
        # cache it is given)
        self.shares_kv = bool(shares_kv)
        self.softcap = float(softcap) if softcap else None
        self.has_sinks, self.values_are_keys = bool(sinks), bool(values_are_keys)
        if self.values_are_keys and (self.shares_kv or qk_norm_eps is not None):
            raise ValueError("values that are the keys go with a cache of the layer's own and "
                             "with keys that are not normalised")
        self.names = dict(self.NAMES, **(names or {}))
        self.sink = None
        self.position = build_part("position", position, ctx)
        self.qkv = self.o = None
        self.q_norm_w = self.k_norm_w = None

    def children(self):
        return (self.position,)

    def param_specs(self):
        H, nq, nkv, D, nm = self.hidden, self.nq, self.nkv, self.D, self.names
        specs = {nm["q"]: ParamSpec((nq * D, H)), nm["o"]: ParamSpec((H, nq * self.Dv))}
        if not self.shares_kv:
            specs[nm["k"]] = ParamSpec((nkv * D, H))
            if not self.values_are_keys:
                specs[nm["v"]] = ParamSpec((nkv * self.Dv, H))
        if self.qk_norm_eps is not None:
            specs[nm["q_norm"]] = ParamSpec((D,), "vector")
            if not self.shares_kv:
                specs[nm["k_norm"]] = ParamSpec((D,), "vector")
        if self.has_sinks:
            specs[nm["sink"]] = ParamSpec((nq,), "offset")
        if self.head_gate:
            specs[nm["g"]] = ParamSpec((nq, H))
        return specs

    def load(self, params):
        nm = self.names
        ws = [params[nm["q"]]]
        if not self.shares_kv:
            ws += [params[nm["k"]]] + ([] if self.values_are_keys else [params[nm["v"]]])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("q, k and v projections must be stored in one dtype to be fused")
        self.qkv = Linear(torch.cat(ws, dim=0) if len(ws) > 1 else ws[0], self.ctx.products)
        o = params[nm["o"]]
        if self.beside:             # the parent multiplies: by one weight for all its mixers
            self.o_w, self.g_w = o, (params[nm["g"]] if self.head_gate else None)
        elif self.head_gate:        # the gate's kernel also drops what fills up a head
            self.o = Linear(o, self.ctx.products)
            self.g = Linear(params[nm["g"]], self.ctx.products)
        else:
            if self.Ds != self.Dv:      # zero columns where the attention's output is filled up
                wide = o.new_zeros((self.hidden, self.nq, self.Ds))
                wide[:, :, :self.Dv] = o.view(self.hidden, self.nq, self.Dv)
                o = wide.view(self.hidden, self.nq * self.Ds)
            self.o = Linear(o, self.ctx.products)
        if self.sink_logit is not None:
            self.sink = torch.full((self.nq,), self.sink_logit, dtype=torch.float32, device=o.device)
        if self.qk_norm_eps is not None:
            self.q_norm_w = params[nm["q_norm"]].contiguous()
            if not self.shares_kv:
                self.k_norm_w = params[nm["k_norm"]].contiguous()
        if self.has_sinks:       # 32-bit, as the scores are
            self.sink = params[nm["sink"]].float().contiguous()

    def kernel_modules(self):
        mods = ("qk_prepare", "attn_generic") + self.qkv.kernel_modules()
        mods += self.o.kernel_modules() if self.o else ()
        if self.head_gate or self.beside:
            mods += ("elementwise",)
        if self.ctx.dtype == torch.bfloat16:
            mods += ops.fast_attention_modules(self.Ds, self.nq, self.nkv)
        return mods

    def cache_spec(self):
        if self.shares_kv:
            return None
        if self.keep_first:
            return KVSpec(self.nkv, self.Ds, self.window, keep_first=self.keep_first)
        return KVSpec(self.nkv, self.Ds, self.window)

    # -- beside another mixer ------------------------------------------------
    @property
    def inner_width(self) -> int:
        return self.nq * self.Dv

    def side_weight(self):
        return self.g_w

    def out_weight(self):
        return self.o_w

    def inner(self, x, step, cache, sums=None, out=None, mult: float = 1.0):
        """The o projection's input [T, heads * v_head_dim], times ``mult``: the heads'
        outputs under their gates (``sums``: the 32-bit products of ``side_weight`` with
        x), written into ``out`` when given."""
        attn = self._attend(x, step, cache)
        return ops.head_gate(attn, sums if self.head_gate else None, self.Dv, mult, into=out)

    def captures_prompts(self):
        # an encoding with arithmetic of its own runs between two kernels here and
        # answers for itself
        return True

    def forward(self, x, step, cache):
        T = x.shape[0]
        if self.head_gate:
            y = self.inner(x, step, cache, self.g(x, out_dtype=torch.float32))
            return self.o(y, partial_ok=True)
        attn = self._attend(x, step, cache)
        return self.o(attn.view(T, self.nq * self.Ds), partial_ok=True)

    def _attend(self, x, step, cache):
        """The heads' outputs [T, heads, Ds] (keys and values of the step's rows stored)."""
        T = x.shape[0]
        rot = self.position.rotary()
        if cache is None or (cache.spec.n_kv_heads, cache.spec.head_dim) != (self.nkv, self.Ds):
            raise ValueError(f"attention with {self.nkv} kv heads of {self.Ds} was given the cache "
                             f"{None if cache is None else cache.spec}")
        fused = rot is not None or type(self.position).apply_qk is PositionEncoding.apply_qk
        if not fused and (self.Ds != self.D or self.q_temp):
            raise ValueError("a position encoding with arithmetic of its own goes with neither "
                             "values of another size nor a query temperature")
        # the q/k preparation can add the partial sums of a split-K projection itself
        qkv = self.qkv(x, partial_ok=fused and x.dtype == torch.bfloat16 and not self.shares_kv)
        if self.shares_kv:
            q, _ = ops.qk_prepare(qkv, self.nq, 0, self.D, q_w=self.q_norm_w,
                                  eps=self.qk_norm_eps or 0.0,
                                  inv_freq=rot.inv_freq if rot else None,
                                  rot_dim=rot.rot_dim if rot else 0, token_seq=step.token_seq,
                                  token_pos=step.token_pos, slots=step.slots, q_temp=self.q_temp,
                                  interleaved=bool(rot and rot.interleaved))
            if rot is None:
                q, _k = self.position.apply_qk(q, q[:, :0], step.token_pos)
            return ops.attention(q.contiguous(), cache.k_pages, cache.v_pages, cache.block_table,
                                 step=step, page=cache.page, scale=self.scale, window=self.window,
                                 softcap=self.softcap, sinks=self.sink, keep_first=self.keep_first)
        common = dict(q_w=self.q_norm_w, k_w=self.k_norm_w, eps=self.qk_norm_eps or 0.0,
                      values_are_keys=self.values_are_keys, token_seq=step.token_seq, token_pos=step.token_pos, slots=step.slots)
        if fused:
            q, _ = ops.qk_prepare(qkv, self.nq, self.nkv, self.D,
                                  inv_freq=rot.inv_freq if rot else None,
                                  rot_dim=rot.rot_dim if rot else 0,
                                  block_table=cache.block_table, k_pages=cache.k_pages,
                                  v_pages=cache.v_pages, page=cache.page, v_dim=self.Dv,
                                  q_temp=self.q_temp, interleaved=bool(rot and rot.interleaved),
                                  **common)
        else:
            # a position encoding with its own arithmetic: normalise, hand q and k
            # over, then store
            q, kv = ops.qk_prepare(qkv, self.nq, self.nkv, self.D, want_kv_out=True, **common)
            k, v = kv[:, :self.nkv], kv[:, self.nkv:]
            q, k = self.position.apply_qk(q, k, step.token_pos)
            kv = torch.cat([k, v], dim=1).contiguous()
            ops.kv_write(kv, self.nkv, self.D, token_seq=step.token_seq, token_pos=step.token_pos,
                         slots=step.slots, block_table=cache.block_table, k_pages=cache.k_pages,
                         v_pages=cache.v_pages, page=cache.page)
            q = q.contiguous()
        return ops.attention(q, cache.k_pages, cache.v_pages, cache.block_table, step=step,
                             page=cache.page, scale=self.scale, window=self.window,
                             softcap=self.softcap, sinks=self.sink, keep_first=self.keep_first)


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    """Mixers that read the same input side by side; the result is the sum of theirs,
    each times a constant:  y = sum_i scale_i * mixer_i(h).

    ``mixers`` is a tuple of (name, PartSpec, scale); a mixer's tensors lie under
    ``<name>.``.  Each mixer must be able to run beside another (``side_weight``,
    ``inner``, ``out_weight``, ``inner_width``: see ``GQAAttention``): the rows whose 32-bit
    products with h the mixers need are one product, every mixer leaves the input of its
    output projection, already times its constant, in its part of one wide row, and the
    output projections are one product over that row.  The layer's cache need is the
    tuple of the mixers' needs (``SideBySideSpec``)."""

    def __init__(self, ctx: BuildContext, hidden: int, mixers):
        super().__init__(ctx)
        self.hidden = int(hidden)
        self.names = [m[0] for m in mixers]
        self.scales = [float(m[2]) for m in mixers]
        self.parts = [build_part("mixer", m[1], ctx) for m in mixers]
        if len(set(self.names)) != len(self.names) or not self.parts:
            raise ValueError("mixers side by side need names of their own")
        for n, p in zip(self.names, self.parts):
            if not all(hasattr(p, a) for a in ("side_weight", "inner", "out_weight", "inner_width")):
                raise ValueError(f"mixer '{n}' ({type(p).__name__}) cannot run beside another")
            p.beside = True
        self.side = self.o = None
        self.side_cols = []           # per mixer (first column, count) in the side product
        self.inner_cols = []          # per mixer (first column, count) in the wide row

    def children(self):
        return tuple(self.parts)

    def param_specs(self):
        return {f"{n}.{local}": spec for n, p in zip(self.names, self.parts)
                for local, spec in p.param_specs().items()}

    def load(self, params):
        side, outs, at_s, at_i = [], [], 0, 0
        self.side_cols, self.inner_cols = [], []
        for n, p in zip(self.names, self.parts):
            p.load({local: params[f"{n}.{local}"] for local in p.param_specs()})
            w = p.side_weight()
            self.side_cols.append((at_s, 0 if w is None else w.shape[0]))
            if w is not None:
                side.append(w)
                at_s += w.shape[0]
            self.inner_cols.append((at_i, p.inner_width))
            outs.append(p.out_weight())
            at_i += p.inner_width
        if len({w.dtype for w in side + outs}) != 1:
            raise ValueError("mixers side by side must be stored in one dtype to be fused")
        self.side = Linear(torch.cat(side, dim=0), self.ctx.products) if side else None
        self.o = Linear(torch.cat(outs, dim=1), self.ctx.products)
        for p in self.parts:          # the fused copies serve from here on
            p.o_w = p.g_w = p.side_w = None

    def kernel_modules(self):
        mods = self.o.kernel_modules() if self.o else ()
        return mods + (self.side.kernel_modules() if self.side else ())

    def lend_side_weight(self):
        """The rows of the side product, for a block that multiplies h by rows of its own in
        32-bit anyway and takes these along (it then passes ``sums`` to ``forward``); None when
        there are none.  The mixer's own product is given up."""
        if self.side is None:
            return None
        w, self.side = self.side.weight, None
        return w

    def keep_side_weight(self, w) -> None:
        self.side = Linear(w, self.ctx.products)

    def cache_spec(self):
        return SideBySideSpec(tuple(p.cache_spec() for p in self.parts))

    def captures_prompts(self):
        return True

    def forward(self, x, step, cache, sums=None):
        if not isinstance(cache, tuple) or len(cache) != len(self.parts):
            raise ValueError(f"{len(self.parts)} mixers side by side were given the cache {cache!r}")
        T = x.shape[0]
        if sums is None and self.side is not None:
            sums = self.side(x, out_dtype=torch.float32)
        wide = torch.empty((T, self.o.in_features), dtype=self.ctx.dtype, device=x.device)
        for p, view, scale, (s0, sn), (i0, n) in zip(self.parts, cache, self.scales, self.side_cols,
                                                     self.inner_cols):
            p.inner(x, step, view, sums[:, s0:s0 + sn] if sn else None, wide[:, i0:i0 + n], scale)
        return self.o(wide, partial_ok=True)


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Attention whose keys and values are expanded from one latent vector per token.

        q = Wq h                      per head ``head_dim`` plain and ``rot_dim`` rotated elements
        d = Wdkv h                    ``kv_rank`` + ``rot_dim`` numbers
        c = rmsnorm(d[:kv_rank]) * w  the latent (``norm_eps`` under the root)
        k_rot = rot(d[kv_rank:])      one rotated key part shared by all heads
        head i:  k = [Wuk_i c | k_rot],  v = Wuv_i c  (``v_head_dim``)
        score = (q_plain . Wuk_i c + rot(q_rot) . k_rot) * scale;  softmax over the keys the
        query sees (its own position and the ``window`` - 1 before it, or all before it)
        y = Wo [ heads * sigmoid(Wg h) ]           (the gate only with ``gated``)

    The cache keeps [c | k_rot] per token, once for all heads; Wuk is folded into
    the query ((Wuk_i^T q_plain) . c) and Wuv applied to the attention's output over
    the latents, so the attention kernels see query heads that all read one kv head of
    kv_rank + rot_dim elements whose values are its keys.  ``position`` rotates the
    rot_dim part (neighbouring pairs).  Norm, rotation and gate are 32-bit on the
    projection's 32-bit sums.  ``names`` replaces local tensor names (keys q, dkv,
    dkv_norm, uk, uv, g, o)."""

    NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "g": "g", "o": "o"}

    def __init__(self, ctx: BuildContext, hidden: int, n_heads: int, head_dim: int, rot_dim: int,
                 v_head_dim: int, kv_rank: int, position: PartSpec, scale: float, norm_eps: float,
                 window: Optional[int] = None, gated: bool = True, names: Optional[dict] = None):
        super().__init__(ctx)
        self.hidden, self.H, self.dn, self.dr = int(hidden), int(n_heads), int(head_dim), int(rot_dim)
        self.dv, self.R = int(v_head_dim), int(kv_rank)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.window = int(window) if window else None
        self.gated = bool(gated)
        self.names = dict(self.NAMES, **(names or {}))
        self.position = build_part("position", position, ctx)
        rot = self.position.rotary()
        if self.dr and (rot is None or not rot.interleaved or rot.rot_dim != self.dr):
            raise ValueError("latent attention rotates the whole rotated part in neighbouring pairs")
        # the width of a cached row, of a query and of the attention's output
        self.Ds = self.R + self.dr
        if ctx.dtype == torch.bfloat16:           # the tensor-core kernels take multiples of 16
            self.Ds = (self.Ds + 15) // 16 * 16
        self.proj = self.o = self.uk_t = self.uv = self.norm_w = None

    def children(self):
        return (self.position,)

    def param_specs(self):
        W, H, nm = self.hidden, self.H, self.names
        specs = {nm["q"]: ParamSpec((H * (self.dn + self.dr), W)),
                 nm["dkv"]: ParamSpec((self.R + self.dr, W)),
                 nm["dkv_norm"]: ParamSpec((self.R,), "vector"),
                 nm["uk"]: ParamSpec((H * self.dn, self.R)), nm["uv"]: ParamSpec((H * self.dv, self.R)),
                 nm["o"]: ParamSpec((W, H * self.dv))}
        if self.gated:
            specs[nm["g"]] = ParamSpec((H * self.dv, W))
        return specs

    def load(self, params):
        nm = self.names
        ws = [params[nm["q"]], params[nm["dkv"]]] + ([params[nm["g"]]] if self.gated else [])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the projections of one mixer must be stored in one dtype to be fused")
        self.proj = Linear(torch.cat(ws, dim=0), self.ctx.products)
        self.o = Linear(params[nm["o"]], self.ctx.products)
        dt = self.ctx.dtype
        # [H dn, R] -> per head [R, dn]: the product that folds Wuk into the query
        self.uk_t = params[nm["uk"]].view(self.H, self.dn, self.R).transpose(1, 2).to(dt).contiguous()
        self.uv = params[nm["uv"]].view(self.H, self.dv, self.R).to(dt).contiguous()
        self.norm_w = params[nm["dkv_norm"]].float().contiguous()

    def kernel_modules(self):
        mods = ("latent", "attn_generic") + self.proj.kernel_modules() + self.o.kernel_modules()
        if self.ctx.dtype == torch.bfloat16:
            mods += ops.fast_attention_modules(self.Ds, min(self.H, self.GROUP), 1)
        return mods

    def cache_spec(self):
        return KVSpec(1, self.Ds, self.window, values_in_keys=True)

    GROUP = 16       # the most query heads that the tensor-core decode kernels let share a kv head

    def _attend(self, q, step, cache):
        """Attention of all heads over the one shared row per token.  More heads than the
        tensor-core kernels let share a kv head go in groups, each a call of its own."""
        kw = dict(step=step, page=cache.page, scale=self.scale, window=self.window)
        if (self.H <= self.GROUP or q.dtype != torch.bfloat16
                or not ops.fast_attention_takes(self.Ds, self.GROUP, 1, cache.page)):
            return ops.attention(q, cache.k_pages, cache.v_pages, cache.block_table, **kw)
        return ops.join_heads([ops.attention(ops.head_group(q, a, min(self.GROUP, self.H - a)), cache.k_pages,
                                             cache.v_pages, cache.block_table, **kw)
                               for a in range(0, self.H, self.GROUP)])

    def captures_prompts(self):
        return True

    def forward(self, x, step, cache):
        if cache is None or cache.spec != self.cache_spec():
            raise ValueError(f"latent attention with rows of {self.Ds} was given the cache "
                             f"{None if cache is None else cache.spec}")
        T, H = x.shape[0], self.H
        rot = self.position.rotary()
        proj = self.proj(x, out_dtype=torch.float32)
        q_plain, q = ops.latent_prepare(
            proj, self.norm_w, rot.inv_freq if rot else None, H=H, dn=self.dn, dr=self.dr, R=self.R,
            dv=self.dv if self.gated else 0, eps=self.norm_eps, token_seq=step.token_seq,
            token_pos=step.token_pos, slots=step.slots, block_table=cache.block_table,
            pages=cache.k_pages, page=cache.page, dtype=self.ctx.dtype)
        ops.heads_mm(q_plain, self.uk_t, q)
        attn = self._attend(q, step, cache)
        y = ops.heads_mm(attn, self.uv, gate=proj if self.gated else None,
                         gate_col=H * (self.dn + self.dr) + self.R + self.dr)
        return self.o(y.view(T, H * self.dv), partial_ok=True)
