"""Position encodings.  Interface of the family:

* ``rotary() -> RotaryTable | None``: an encoding that is a rotation of the
  first ``rot_dim`` elements of every query and key head by angle
  ``pos * inv_freq[j]`` returns its table, and attention folds it into the
  kernel that also normalises q and k and writes the cache.
* ``apply_qk(q, k, token_pos) -> (q, k)``: any other encoding of queries and
  keys ([T, heads, D]); attention calls it between its projection and the
  cache write when ``rotary()`` is None.

An encoding that is added to the embeddings is not of this family: it is an
``embedding`` part, whose ``forward(tokens, step)`` has every row's position in
``step.token_pos``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .base import BuildContext, Part, register_part


@dataclass
class RotaryTable:
    inv_freq: torch.Tensor   # float32 [rot_dim / 2] on the device
    rot_dim: int
    interleaved: bool = False   # element 2j goes with 2j + 1 instead of j with j + rot_dim / 2


class PositionEncoding(Part):
    family = "position"

    def rotary(self) -> Optional[RotaryTable]:
        return None

    def apply_qk(self, q, k, token_pos):
        return q, k


@register_part("position", "none")
class NoPosition(PositionEncoding):
    def __init__(self, ctx: BuildContext):
        super().__init__(ctx)

    def captures_prompts(self):
        return True


def scaled_inverse_frequencies(rot_dim: int, theta: float, scaling: Optional[dict]) -> np.ndarray:
    """theta^(-2j / rot_dim) for j < rot_dim / 2 in float64, with the band-wise
    scaling of ``RotaryHalfSplit`` when ``scaling`` is given."""
    j = np.arange(rot_dim // 2, dtype=np.float64)
    f = np.power(np.float64(theta), -2.0 * j / rot_dim)
    if scaling:
        factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wave = 2.0 * np.pi / f
        s = (original / wave - low) / (high - low)
        mixed = (1.0 - s) * f / factor + s * f
        f = np.where(wave < original / high, f, np.where(wave > original / low, f / factor, mixed))
    return f


@register_part("position", "rotary_half_split")
class RotaryHalfSplit(PositionEncoding):
    """Half-split ("NeoX") rotation: element j pairs with j + rot_dim/2;
    inv_freq[j] = 1 / theta^(2j / rot_dim), computed in float32 on the host and
    uploaded (src/model.rs:5992-5997); the angle pos * inv_freq[j] and its sine
    and cosine are float32 in the kernel (src/kernels.rs:3640-3648).

    ``scaling`` = dict(factor, low, high, original) stretches the slow
    frequencies for contexts longer than the ``original`` one, band by band (the
    rule that Llama 3.1 introduced): with wavelength l = 2 pi / f, a frequency
    with l < original / high stays, one with l > original / low becomes
    f / factor, and between the two f / factor and f are mixed with weights
    1 - s and s, s = (original / l - low) / (high - low).  With ``scaling``, or
    with ``exact_table``, the table is computed in float64 and rounded once."""

    def __init__(self, ctx: BuildContext, head_dim: int, theta: float,
                 rot_dim: Optional[int] = None, scaling: Optional[dict] = None,
                 exact_table: bool = False):
        super().__init__(ctx)
        self.head_dim = int(head_dim)
        self.rot_dim = int(rot_dim if rot_dim is not None else head_dim)
        if self.rot_dim % 2 or not 0 < self.rot_dim <= self.head_dim:
            raise ValueError(f"rot_dim={self.rot_dim} must be even and at most head_dim={head_dim}")
        self.theta = float(theta)
        i = np.arange(0, self.rot_dim, 2, dtype=np.float32)
        p = i / np.float32(self.rot_dim)
        inv = (np.float32(1.0) / np.power(np.float32(self.theta), p, dtype=np.float32))
        self.scaling = dict(scaling) if scaling else None
        if self.scaling or exact_table:
            inv = scaled_inverse_frequencies(self.rot_dim, self.theta, self.scaling)
        self._table = RotaryTable(torch.from_numpy(inv.astype(np.float32)).to(ctx.device),
                                  self.rot_dim)

    def rotary(self):
        return self._table

    def captures_prompts(self):
        return True


@register_part("position", "rotary_interleaved")
class RotaryInterleaved(RotaryHalfSplit):
    """The same rotation with neighbours as pairs: element 2j goes with element
    2j + 1, j < rot_dim / 2, and the pair turns by pos * inv_freq[j].  ``gqa_attention``
    folds it into its q/k kernel as it does the half-split rotation;
    ``latent_attention`` rotates in a kernel of its own."""

    def __init__(self, ctx: BuildContext, head_dim: int, theta: float,
                 rot_dim: Optional[int] = None, scaling: Optional[dict] = None,
                 exact_table: bool = False):
        super().__init__(ctx, head_dim, theta, rot_dim, scaling, exact_table)
        self._table.interleaved = True
