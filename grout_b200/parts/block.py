"""Blocks: how a layer's norm, mixer and feed-forward are arranged.

Interface of the family: ``forward(res, pending, step, cache) -> (res, pending)``.
The hidden state travels between blocks as a pair: ``res``, the residual stream
in 32-bit ([T, hidden], None before the first block), and ``pending``, a
contribution in the compute dtype that has not been added yet.  Leaving the last
sum pending lets the next norm do it in the same kernel that normalises (the
reference defers the MLP's residual add into the next layer's norm in the same
way, src/model.rs:3151-3164).
"""
from __future__ import annotations

from typing import Dict

from typing import Optional

from .base import BuildContext, ParamSpec, Part, PartSpec, build_part, register_part
from .linear import Linear
from .norm import Contribution, stream_add


class Block(Part):
    family = "block"

    def forward(self, res, pending, step, cache):
        raise NotImplementedError

    def cache_spec(self):
        return None


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += feedforward(norm2(x)) (src/training.rs:303-349).
    The second line is absent when the layer has no feed-forward (neither ``norm2``
    nor ``feedforward`` is given)."""

    roles = ("norm1", "mixer", "norm2", "feedforward")

    def __init__(self, ctx: BuildContext, norm1: PartSpec, mixer: PartSpec,
                 norm2: Optional[PartSpec] = None, feedforward: Optional[PartSpec] = None):
        super().__init__(ctx)
        if (norm2 is None) != (feedforward is None):
            raise ValueError("a feed-forward comes with its norm, or neither is given")
        self.norm1 = build_part("norm", norm1, ctx)
        self.mixer = build_part("mixer", mixer, ctx)
        self.norm2 = build_part("norm", norm2, ctx) if norm2 else None
        self.feedforward = build_part("feedforward", feedforward, ctx) if feedforward else None

    def children(self):
        return tuple(self.named_parts().values())

    def named_parts(self) -> Dict[str, Part]:
        return {r: getattr(self, r) for r in self.roles if getattr(self, r) is not None}

    def cache_spec(self):
        return self.mixer.cache_spec()

    def captures_prompts(self):
        return True

    def forward(self, res, pending, step, cache):
        res, n = self.norm1.add_norm(res, pending)
        a = self.mixer.forward(n, step, cache)
        if self.feedforward is None:
            return res, a
        res, m = self.norm2.add_norm(res, a)
        return res, self.feedforward.forward(m, step)


@register_part("block", "sandwich")
class SandwichBlock(Block):
    """A norm in front of every sublayer and another behind it, whose output
    enters the stream times ``mult``:

        x += mult * norm1b(mixer(norm1(x)));  x += mult * norm2b(feedforward(norm2(x)))

    The second line is absent when the layer has no feed-forward.  A sublayer's
    output leaves here as a ``Contribution`` (its norm and factor still to be
    applied), so the norm that reads the stream next does the normalising, the
    scaling, the 32-bit sum and its own normalising in one kernel."""

    def __init__(self, ctx: BuildContext, norm1: PartSpec, mixer: PartSpec, norm1b: PartSpec,
                 norm2: Optional[PartSpec] = None, feedforward: Optional[PartSpec] = None,
                 norm2b: Optional[PartSpec] = None, mult: float = 1.0):
        super().__init__(ctx)
        if (feedforward is None) != (norm2 is None) or (feedforward is None) != (norm2b is None):
            raise ValueError("a feed-forward comes with both of its norms, or none of the three")
        self.mult = float(mult)
        self.norm1 = build_part("norm", norm1, ctx)
        self.mixer = build_part("mixer", mixer, ctx)
        self.norm1b = build_part("norm", norm1b, ctx)
        self.norm2 = build_part("norm", norm2, ctx) if norm2 else None
        self.feedforward = build_part("feedforward", feedforward, ctx) if feedforward else None
        self.norm2b = build_part("norm", norm2b, ctx) if norm2b else None

    def named_parts(self) -> Dict[str, Part]:
        roles = ("norm1", "mixer", "norm1b", "norm2", "feedforward", "norm2b")
        return {r: getattr(self, r) for r in roles if getattr(self, r) is not None}

    def children(self):
        return tuple(self.named_parts().values())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def captures_prompts(self):
        return True

    def forward(self, res, pending, step, cache):
        res, n = self.norm1.add_norm(res, pending)
        a = Contribution(self.mixer.forward(n, step, cache), self.norm1b, self.mult)
        if self.feedforward is None:
            return res, a
        res, m = self.norm2.add_norm(res, a)
        return res, Contribution(self.feedforward.forward(m, step), self.norm2b, self.mult)


@register_part("block", "postnorm")
class PostNormBlock(Block):
    """A norm behind every sublayer and none in front of it: the sublayers read
    the stream as it is, and what they return is normalised, multiplied channel
    by channel by a learned vector ("layer scale") and added:

        x += scale1 * norm1(mixer(x));  x += scale2 * norm2(feedforward(x))

    The second line is absent when the layer has no feed-forward; a scale is
    absent when its tensor's name is None.  ``scale1`` / ``scale2`` are the
    tensors' names under the layer's prefix.  A sublayer's output leaves here as a
    ``Contribution``, so each sublayer boundary is one kernel: normalise, scale,
    add in 32-bit, round for the next reader."""

    def __init__(self, ctx: BuildContext, mixer: PartSpec, norm1: PartSpec,
                 scale1: Optional[str] = None, feedforward: Optional[PartSpec] = None,
                 norm2: Optional[PartSpec] = None, scale2: Optional[str] = None):
        super().__init__(ctx)
        if (feedforward is None) != (norm2 is None):
            raise ValueError("a feed-forward comes with its norm, or neither is there")
        self.mixer = build_part("mixer", mixer, ctx)
        self.norm1 = build_part("norm", norm1, ctx)
        self.feedforward = build_part("feedforward", feedforward, ctx) if feedforward else None
        self.norm2 = build_part("norm", norm2, ctx) if norm2 else None
        self.scale_names = (scale1, scale2 if feedforward else None)
        self.scale1 = self.scale2 = None
        self.width = self.norm1.dim

    def named_parts(self) -> Dict[str, Part]:
        roles = ("mixer", "norm1", "feedforward", "norm2")
        return {r: getattr(self, r) for r in roles if getattr(self, r) is not None}

    def children(self):
        return tuple(self.named_parts().values())

    def param_specs(self):
        return {n: ParamSpec((self.width,), "vector") for n in self.scale_names if n}

    def load(self, params):
        # 32-bit whatever the checkpoint stores: the sum into the stream is 32-bit
        s1, s2 = self.scale_names
        self.scale1 = params[s1].float().contiguous() if s1 else None
        self.scale2 = params[s2].float().contiguous() if s2 else None

    def kernel_modules(self):
        return ("norm",)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def captures_prompts(self):
        return True

    def forward(self, res, pending, step, cache):
        res, x = stream_add(res, pending, self.ctx.dtype)
        a = Contribution(self.mixer.forward(x, step, cache), self.norm1, scale=self.scale1)
        if self.feedforward is None:
            return res, a
        res, x = stream_add(res, a, self.ctx.dtype)
        return res, Contribution(self.feedforward.forward(x, step), self.norm2, scale=self.scale2)


@register_part("block", "parallel")
class ParallelBlock(Block):
    """One norm, and both sublayers read its output side by side:

        h = norm1(x);   x += gate1 * mixer(h) + gate2 * feedforward(h)

    The feed-forward's term is absent when the layer has none.  With ``gated`` each
    sublayer's result is multiplied element by element by sigmoid(W h + b) ("gated
    residual"), W and b being the tensors ``gate1`` / ``gate2`` (local names; the bias is
    the name + ``bias_suffix``) under the layer's prefix; both gates' logits come from one
    product with 32-bit sums, which also takes the rows that the mixer wants multiplied with h in
    32-bit, if it has some to lend (``lend_side_weight``).  The sublayers' results leave as a tuple of
    ``Contribution``s, so the sum into the stream is done by the kernel of whoever reads
    the stream next (the next layer's norm, or the model's last one)."""

    def __init__(self, ctx: BuildContext, norm1: PartSpec, mixer: PartSpec,
                 feedforward: Optional[PartSpec] = None, gated: bool = False,
                 gate1: str = "rg1", gate2: str = "rg2", bias_suffix: str = ".b"):
        super().__init__(ctx)
        self.norm1 = build_part("norm", norm1, ctx)
        self.mixer = build_part("mixer", mixer, ctx)
        self.feedforward = build_part("feedforward", feedforward, ctx) if feedforward else None
        self.gated = bool(gated)
        self.gate_names = (gate1, gate2 if feedforward else None) if self.gated else (None, None)
        self.bias_suffix = bias_suffix
        self.width = self.norm1.dim
        self.gates = None
        self.gate_bias = (None, None)
        self.n_gate_cols, self.mixer_sums = 0, False

    def named_parts(self) -> Dict[str, Part]:
        roles = ("norm1", "mixer", "feedforward")
        return {r: getattr(self, r) for r in roles if getattr(self, r) is not None}

    def children(self):
        return tuple(self.named_parts().values())

    def param_specs(self):
        specs = {}
        for n in self.gate_names:
            if n:
                specs[n] = ParamSpec((self.width, self.width))
                specs[n + self.bias_suffix] = ParamSpec((self.width,), "offset")
        return specs

    def load(self, params):
        import torch
        names = [n for n in self.gate_names if n]
        ws = [params[n] for n in names]
        if len({w.dtype for w in ws}) > 1:
            raise ValueError("the two residual gates must be stored in one dtype to be fused")
        # a mixer that needs 32-bit products with h of its own (``SideBySide``) hands its rows over:
        # one product then serves the gates and the mixer
        self.n_gate_cols = sum(w.shape[0] for w in ws)
        side = self.mixer.lend_side_weight() if hasattr(self.mixer, "lend_side_weight") else None
        if side is not None and side.dtype == ws[0].dtype:
            ws = ws + [side]
        elif side is not None:
            self.mixer.keep_side_weight(side)
        self.mixer_sums = side is not None and len(ws) > len(names)
        self.gates = Linear(torch.cat(ws, dim=0) if len(ws) > 1 else ws[0], self.ctx.products)
        # 32-bit whatever the checkpoint stores: the sum into the stream is 32-bit
        self.gate_bias = tuple(params[n + self.bias_suffix].float().contiguous() if n else None
                               for n in self.gate_names)

    def kernel_modules(self):
        return ("gated_norm",) + (self.gates.kernel_modules() if self.gates else ())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def captures_prompts(self):
        return True

    def forward(self, res, pending, step, cache):
        import torch
        res, h = self.norm1.add_norm(res, pending)
        W = self.width
        logits = self.gates(h, out_dtype=torch.float32) if self.gated else None
        if self.gated and self.mixer_sums:
            a = self.mixer.forward(h, step, cache, sums=logits[:, self.n_gate_cols:])
        else:
            a = self.mixer.forward(h, step, cache)
        terms = [Contribution(a, gate=logits[:, :W] if self.gated else None, gate_bias=self.gate_bias[0])]
        if self.feedforward is not None:
            m = self.feedforward.forward(h, step)
            terms.append(Contribution(m, gate=logits[:, W:2 * W] if self.gated else None,
                                      gate_bias=self.gate_bias[1]))
        return res, tuple(terms)
