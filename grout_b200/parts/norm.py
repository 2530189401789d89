"""Norms.  Interface of the family:

* ``forward(x) -> y``: normalises rows of ``x`` [T, N] (compute dtype).
* ``add_norm(res, delta, rows=None) -> (res, y)``: adds ``delta`` (compute
  dtype, may be None) into the 32-bit residual stream ``res`` (may be None on
  the first layer), optionally keeps only ``rows``, and returns the updated
  stream with its normalised rows.  ``delta`` may also arrive as a stack of
  32-bit partial sums [S, T, N] (a split-K projection leaves its reduction to
  the norm); they are added in order.  The default does the steps one after the
  other; RMSNorm does all of it in one kernel.  ``delta`` may, thirdly, be a
  ``Contribution``: a sublayer's output that passes through a norm of its own and
  a constant factor on its way into the stream ("sandwich" layers), with, if the
  model has one, a vector that is added to every row on the same occasion.
  ``LayerNorm`` does all of that in its one kernel as well, and so does ``RMSNorm``
  for a contribution whose own norm is an RMS norm (with, if the layer has one, a
  learned per-channel scale behind it); every other combination is resolved
  first and goes on as above.
* ``stream_add(res, delta, dtype) -> (res, x)``: the same sum without a norm
  behind it, for sublayers that read the stream as it is: ``x`` is the updated
  stream in the compute dtype.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from dataclasses import dataclass

from ..kernels import ops
from .base import BuildContext, ParamSpec, Part, register_part


@dataclass
class Contribution:
    """What is about to be added to the residual stream: ``mult * scale * norm(delta)``
    (just ``delta`` without a norm; nothing when ``delta`` is None) plus
    ``offset`` on every row.  ``delta`` is [T, N] in the compute dtype or a stack of
    32-bit partial sums [S, T, N]; ``offset`` and ``scale`` (a learned factor per
    channel, "layer scale") are 32-bit vectors [N]."""
    delta: Optional[torch.Tensor]
    norm: Optional["Norm"] = None
    mult: float = 1.0
    offset: Optional[torch.Tensor] = None
    scale: Optional[torch.Tensor] = None
    #: a gated residual: ``delta`` is multiplied element by element by
    #: sigmoid(gate + gate_bias); ``gate`` is a 32-bit [T, N] view of logits (it may be
    #: part of a wider row), ``gate_bias`` a 32-bit vector [N] or None
    gate: Optional[torch.Tensor] = None
    gate_bias: Optional[torch.Tensor] = None

    def resolved(self) -> Optional[torch.Tensor]:
        """The contribution as one 32-bit tensor [T, N] (step by step, for norms
        without a kernel that takes it whole); None when there is nothing."""
        d = self.delta
        if d is not None and d.dim() == 3:
            d = d.sum(dim=0)
        if d is not None and self.norm is not None:
            d = self.norm.forward(d if d.dtype == self.norm.ctx.dtype
                                  else ops.cast(d, self.norm.ctx.dtype))
        if d is not None:
            d = d.float() * self.mult if self.mult != 1.0 else d.float()
            if self.scale is not None:
                d = d * self.scale.float()[None, :]
            if self.gate is not None:
                g = self.gate.float()
                d = d * torch.sigmoid(g if self.gate_bias is None else g + self.gate_bias.float()[None, :])
        if self.offset is not None:
            d = self.offset.float()[None, :] if d is None else d + self.offset.float()[None, :]
        return d


@dataclass
class Averaged:
    """What a model with a depth-averaged stream hands to the next norm: the layer's
    contributions ``terms`` (a tensor, a ``Contribution`` or a tuple of them; sublayers
    that run side by side leave one each) are still to be added to the stream, which
    gives the layer's result X; X becomes entry ``index`` of ``history`` [n, T, N]
    (32-bit: the embedding's output and every earlier layer's result lie before it), and
    the stream that goes on is sum_j weights[j] * history[j], j = 0 .. index."""
    terms: object
    history: torch.Tensor
    index: int
    weights: torch.Tensor          # 32-bit [index + 1]

    def resolve(self, res: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Step by step, for norms without a kernel that takes all of it: the new stream
        (of ``rows`` only, when given)."""
        x = residual_add(res, resolve_terms(self.terms))
        self.history[self.index].copy_(x)
        hist = self.history[:self.index + 1]
        if rows is not None:
            hist = hist.index_select(1, rows.long())
        return (self.weights.float()[:, None, None] * hist).sum(dim=0)


def as_terms(pending):
    """``pending`` as a tuple of ``Contribution``s (tensors are wrapped, None is dropped)."""
    if pending is None:
        return ()
    items = pending if isinstance(pending, (tuple, list)) else (pending,)
    return tuple(p if isinstance(p, Contribution) else Contribution(p) for p in items if p is not None)


def resolve_terms(pending) -> Optional[torch.Tensor]:
    """The sum of all pending contributions as one 32-bit tensor (None: nothing)."""
    total = None
    for c in as_terms(pending):
        d = c.resolved()
        if d is not None:
            total = d if total is None else total + d
    return total


def with_offset(pending, offset: torch.Tensor) -> Contribution:
    """``pending`` (a tensor, a ``Contribution`` or None) with ``offset`` added to
    every row as well."""
    if isinstance(pending, Contribution):
        if pending.offset is not None:
            offset = pending.offset + offset
        return Contribution(pending.delta, pending.norm, pending.mult, offset, pending.scale)
    return Contribution(pending, None, 1.0, offset)


class Norm(Part):
    family = "norm"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, res: Optional[torch.Tensor], delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        if isinstance(delta, Averaged):
            res, delta = delta.resolve(res, rows), None
            return res, self.forward(ops.cast(res, self.ctx.dtype))
        if isinstance(delta, (Contribution, tuple, list)):
            delta = resolve_terms(delta)
        res = residual_add(res, delta, rows)
        return res, self.forward(ops.cast(res, self.ctx.dtype))


def residual_add(res, delta, rows=None) -> torch.Tensor:
    """32-bit residual sum for norms without a fused kernel (a library call on
    small tensors; parts of this package use the fused kernel instead)."""
    if delta is not None and delta.dim() == 3:      # partial sums of a split-K product
        delta = delta.sum(dim=0)
    if res is None:
        if delta is None:
            raise ValueError("neither a residual stream nor a contribution to it")
        out = delta.float()
    elif delta is None:
        out = res
    else:
        out = res + delta.float()
    return out if rows is None else out.index_select(0, rows.long())


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * w; the weight multiplies as it is
    (src/kernels.rs:316-341, src/training.rs:233-238)."""

    def __init__(self, ctx: BuildContext, dim: int, eps: float, name: str = "weight",
                 unit_offset: bool = False):
        """``unit_offset``: the tensor is stored around zero and the norm multiplies by
        1 + w (the sum is taken in 32-bit at load)."""
        super().__init__(ctx)
        self.dim, self.eps, self.name = int(dim), float(eps), name
        self.unit_offset = bool(unit_offset)
        self.weight = None
        self._weight32 = None

    def param_specs(self):
        return {self.name: ParamSpec((self.dim,), "offset" if self.unit_offset else "vector")}

    def load(self, params):
        w = params[self.name]
        self.weight = (1.0 + w.float()).contiguous() if self.unit_offset else w.contiguous()
        self._weight32 = None

    def weight32(self) -> torch.Tensor:
        """The weight in 32-bit, as the kernels that take a whole contribution read it."""
        if self._weight32 is None:
            self._weight32 = self.weight.float().contiguous()
        return self._weight32

    def captures_prompts(self):
        return True

    def forward(self, x):
        _res, y = ops.add_rmsnorm(None, x, self.weight, self.eps, dtype=self.ctx.dtype,
                                  write_res=False)
        return y

    def kernel_modules(self):
        return ("norm",)

    def add_norm(self, res, delta, rows=None):
        if isinstance(delta, (Averaged, tuple, list)) or (isinstance(delta, Contribution)
                                                          and delta.gate is not None):
            return self._add_gated(res, delta, rows)
        if isinstance(delta, Contribution):
            if _one_kernel(delta):
                return _add_contribution(res, delta, self.ctx.dtype, rows, self)
            # resolved step by step, added in 32-bit
            res, delta = residual_add(res, delta.resolved()), None
        return ops.add_rmsnorm(res, delta, self.weight, self.eps, dtype=self.ctx.dtype, rows=rows)

    def _add_gated(self, res, pending, rows):
        """Gated contributions of sublayers that ran side by side and, for a model with a
        depth-averaged stream, the average over the earlier layers' results, in the one
        kernel that also normalises (``ops.gated_norm``).  Contributions that carry more
        than a gate (a norm, a factor, a vector of their own) are resolved first."""
        avg = pending if isinstance(pending, Averaged) else None
        terms = as_terms(avg.terms if avg else pending)
        plain = all(c.norm is None and c.mult == 1.0 and c.offset is None and c.scale is None
                    for c in terms)
        if not plain or len(terms) > 2:
            res, terms = residual_add(res, resolve_terms(terms)), ()
        return ops.gated_norm(res, [(c.delta, c.gate, c.gate_bias) for c in terms],
                              dtype=self.ctx.dtype, hist=avg.history if avg else None,
                              n_hist=avg.index if avg else 0, avg_w=avg.weights if avg else None,
                              rows=rows, norm_w=self.weight32(), eps=self.eps)


def _one_kernel(c: Contribution) -> bool:
    """Whether ``ops.add_postnorm`` takes the contribution whole."""
    return c.mult == 1.0 and c.offset is None and (c.norm is None or type(c.norm) is RMSNorm)


def _add_contribution(res, c: Contribution, dtype, rows, norm: Optional[RMSNorm]):
    post = c.norm if c.delta is not None else None
    return ops.add_postnorm(res, c.delta, dtype=dtype, rows=rows,
                            post_weight=post.weight32() if post else None,
                            post_eps=post.eps if post else 0.0,
                            scale=c.scale if c.delta is not None else None,
                            weight=norm.weight32() if norm else None,
                            eps=norm.eps if norm else 0.0)


def stream_add(res, delta, dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """Adds ``delta`` (a tensor in the compute dtype, a stack of partial sums, a
    ``Contribution`` or None) into the 32-bit stream ``res`` (None: the stream
    starts with the contribution) and returns the stream with its rounding to
    ``dtype``, which is what a sublayer without a norm in front of it reads."""
    if not isinstance(delta, Contribution):
        delta = Contribution(delta)
    if not _one_kernel(delta):
        res, delta = residual_add(res, delta.resolved()), Contribution(None)
    return _add_contribution(res, delta, dtype, None, None)


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * w + b over the last axis, var the mean
    of the squared deviations; mean, variance and the scaling are 32-bit.  The
    bias may be absent (``bias=False``), and with ``center=False`` the mean is not
    taken off (x / sqrt(mean(x^2) + eps) * w + b).  ``weight_name`` and
    ``bias_name`` are the tensors' local names."""

    def __init__(self, ctx: BuildContext, dim: int, eps: float, bias: bool = True,
                 center: bool = True, weight_name: str = "weight", bias_name: str = "bias"):
        super().__init__(ctx)
        self.dim, self.eps = int(dim), float(eps)
        self.has_bias, self.center = bool(bias), bool(center)
        self.weight_name, self.bias_name = weight_name, bias_name
        self.weight = self.bias = None

    def param_specs(self):
        specs = {self.weight_name: ParamSpec((self.dim,), "vector")}
        if self.has_bias:
            specs[self.bias_name] = ParamSpec((self.dim,), "offset")
        return specs

    def load(self, params):
        # 32-bit whatever the checkpoint stores: the norm's arithmetic is 32-bit
        self.weight = params[self.weight_name].float().contiguous()
        self.bias = params[self.bias_name].float().contiguous() if self.has_bias else None

    def kernel_modules(self):
        return ("layernorm",)

    def captures_prompts(self):
        return True

    def forward(self, x):
        _res, y = ops.add_layernorm(None, x, self.weight, self.bias, self.eps, self.center,
                                    dtype=self.ctx.dtype, write_res=False)
        return y

    def add_norm(self, res, delta, rows=None):
        post = None
        mult, offset = 1.0, None
        if isinstance(delta, Averaged):          # resolved step by step, then normalised
            res, delta, rows = delta.resolve(res, rows), None, None
        elif isinstance(delta, (tuple, list)) or (isinstance(delta, Contribution) and delta.gate is not None):
            res, delta = residual_add(res, resolve_terms(delta)), None
        if isinstance(delta, Contribution):
            c, delta = delta, delta.delta
            mult, offset = c.mult, c.offset
            if c.norm is not None and delta is not None:
                if not isinstance(c.norm, LayerNorm):
                    delta, mult = Contribution(delta, c.norm, mult).resolved(), 1.0
                    res, delta = residual_add(res, delta), None
                else:
                    post = c.norm
        return ops.add_layernorm(res, delta, self.weight, self.bias, self.eps, self.center,
                                 dtype=self.ctx.dtype, rows=rows, mult=mult, offset=offset,
                                 post_weight=post.weight if post else None,
                                 post_bias=post.bias if post else None,
                                 post_eps=post.eps if post else 0.0,
                                 post_center=post.center if post else True)
