"""The two ends of the model: token embedding and output head."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import BuildContext, ParamSpec, Part, register_part
from .linear import Linear


class Embedding(Part):
    family = "embedding"
    #: True when ``forward`` returns the 32-bit residual stream itself instead of
    #: a first contribution to it in the compute dtype
    starts_stream = False

    def forward(self, tokens, step):
        raise NotImplementedError


@register_part("embedding", "token")
class TokenEmbedding(Embedding):
    """x[t] = E[ids[t]], no scaling (src/training.rs:278-282).  With ``scale`` the row
    is multiplied by that constant in 32-bit, and the result is the 32-bit residual
    stream itself (``starts_stream``) instead of a first contribution to it."""

    def __init__(self, ctx: BuildContext, vocab: int, hidden: int, name: str = "weight",
                 scale: Optional[float] = None):
        super().__init__(ctx)
        self.vocab, self.hidden, self.name = int(vocab), int(hidden), name
        self.scale = None if scale is None else float(scale)
        self.starts_stream = self.scale is not None
        self.weight = None

    def param_specs(self):
        return {self.name: ParamSpec((self.vocab, self.hidden))}

    def load(self, params):
        self.weight = params[self.name].contiguous()

    def kernel_modules(self):
        return ("embed", "elementwise")

    def captures_prompts(self):
        return True

    def forward(self, tokens, step, out=None):
        if self.scale is not None:
            return ops.embed_scaled(self.weight, tokens, self.scale, into=out)
        x = ops.embed(self.weight, tokens)
        return ops.cast(x, self.ctx.dtype) if x.dtype != self.ctx.dtype else x


@register_part("embedding", "token_positional")
class TokenPositionalEmbedding(Embedding):
    """x[t] = N(E[ids[t]] + P[pos[t]]): a token table, a learned table of position
    vectors (positions count from 0 in every sequence; neither term is scaled)
    and an RMS norm over the sum (weight as it is, ``eps`` inside the root).  The
    sum and the norm are 32-bit and the result is the 32-bit residual stream
    itself (``starts_stream``), not a contribution to it.  ``names``: the tensors'
    local names (keys token, position, norm)."""

    starts_stream = True

    def __init__(self, ctx: BuildContext, vocab: int, hidden: int, max_positions: int, eps: float,
                 names: Optional[dict] = None):
        super().__init__(ctx)
        self.vocab, self.hidden, self.max_positions = int(vocab), int(hidden), int(max_positions)
        self.eps = float(eps)
        self.names = dict({"token": "weight", "position": "position.weight", "norm": "norm.weight"},
                          **(names or {}))
        self.weight = self.positions = self.norm_w = None

    def param_specs(self):
        nm = self.names
        return {nm["token"]: ParamSpec((self.vocab, self.hidden)),
                nm["position"]: ParamSpec((self.max_positions, self.hidden)),
                nm["norm"]: ParamSpec((self.hidden,), "vector")}

    def load(self, params):
        nm = self.names
        self.weight = params[nm["token"]].contiguous()
        self.positions = params[nm["position"]].contiguous()
        if self.positions.dtype != self.weight.dtype:
            raise ValueError("the token and position tables must be stored in one dtype")
        self.norm_w = params[nm["norm"]].float().contiguous()

    def kernel_modules(self):
        return ("embed",)

    def captures_prompts(self):
        return True

    def forward(self, tokens, step):
        return ops.embed_pos_norm(self.weight, self.positions, tokens, step.token_pos,
                                  self.norm_w, self.eps)


class Head(Part):
    family = "head"

    def forward(self, h):
        raise NotImplementedError


@register_part("head", "linear")
class LinearHead(Head):
    """logits = h W^T in 32-bit; W is the embedding table when ``tied``
    (src/training.rs:352-362).  With ``scale`` the logits are multiplied by it, and
    with ``softcap`` c they then become c * tanh(logit / c); both in 32-bit.
    ``name``: the weight's local name."""

    def __init__(self, ctx: BuildContext, vocab: int, hidden: int, tied: bool,
                 scale: Optional[float] = None, softcap: Optional[float] = None,
                 name: str = "weight"):
        super().__init__(ctx)
        self.vocab, self.hidden, self.tied = int(vocab), int(hidden), bool(tied)
        self.scale = float(scale) if scale is not None else 1.0
        self.softcap = float(softcap) if softcap else None
        self.name = name
        self.proj: Optional[Linear] = None

    def param_specs(self):
        return {} if self.tied else {self.name: ParamSpec((self.vocab, self.hidden))}

    def load(self, params):
        if not self.tied:
            self.proj = Linear(params[self.name], self.ctx.products)

    def tie(self, table: torch.Tensor) -> None:
        self.proj = Linear(table, self.ctx.products)   # shares the allocation (src/model.rs:1375-1377)

    def kernel_modules(self):
        mods = self.proj.kernel_modules() if self.proj else ()
        return mods + (("elementwise",) if self.scale != 1.0 or self.softcap else ())

    def captures_prompts(self):
        return True

    def forward(self, h):
        logits = self.proj(h, out_dtype=torch.float32)
        if self.scale != 1.0 or self.softcap:
            ops.scale_softcap_(logits, self.scale, self.softcap)
        return logits
