"""What a layer asks of the cache.

A need is a frozen (hashable, comparable) object with one method,
``make_store(n_layers, sizes, dtype, device, allocate)``, which returns the
storage for a group of ``n_layers`` layers that all have this need.  Layers
whose needs compare equal share a store.  A store has the methods of
``stores.Store``: ``open``, ``reserve``, ``trim``, ``close``, ``flush``,
``tokens_held``, ``layer(index)`` (what the layer's part is handed as its
``cache`` argument) and ``check``.  The cache itself knows no kind of need: a
mixer that keeps something else (keys and values of different widths, a
compressed latent) brings its own spec and store.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

PAGE_TOKENS = 64   # tokens per page of a key/value store; requests hold whole pages


@dataclass(frozen=True)
class StoreSizes:
    """The limits a cache was built with, handed to every ``make_store``."""
    n_pages: int               # pages of PAGE_TOKENS tokens in a paged store
    max_slots: int             # sequences alive at once
    max_pages_per_seq: int     # pages of the longest sequence
    max_seq_len: int


@dataclass(frozen=True)
class KVSpec:
    """Keys and values of ``n_kv_heads`` heads of ``head_dim`` for every token
    (``window`` None) or for the last ``window`` tokens.  ``values_in_keys``: a
    token's value is read from its key row (a latent that serves as both), so the
    store holds one tensor and hands it out as keys and as values.  ``keep_first``:
    with a window, a sequence's first ``keep_first`` tokens stay visible to every
    later query, so the pages that hold them are never given back."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    values_in_keys: bool = False
    keep_first: int = 0

    def make_store(self, n_layers: int, sizes: StoreSizes, dtype, device, allocate: bool = True):
        from .stores import KVStore
        return KVStore(self, n_layers, sizes.n_pages, sizes.max_slots, sizes.max_pages_per_seq,
                       dtype, device, allocate)


@dataclass(frozen=True)
class StateSpec:
    """Per-sequence state of fixed size: one tensor of ``shape`` per sequence and
    layer, zero when the sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def make_store(self, n_layers: int, sizes: StoreSizes, dtype, device, allocate: bool = True):
        from .stores import StateStore
        return StateStore(self, n_layers, sizes.max_slots, device, allocate)


@dataclass(frozen=True)
class SideBySideSpec:
    """The needs of mixers that run side by side in one layer (keys and values for one,
    a state for the other, ...): a store of each, opened, grown, trimmed and closed
    together; the layer is handed the tuple of their views, in the order of ``specs``."""
    specs: Tuple[object, ...]

    def make_store(self, n_layers: int, sizes: StoreSizes, dtype, device, allocate: bool = True):
        from .stores import SideBySideStore
        return SideBySideStore(self, [s.make_store(n_layers, sizes, dtype, device, allocate)
                                      for s in self.specs])


class CacheFull(RuntimeError):
    """No free slot or page is left."""
