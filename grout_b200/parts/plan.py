"""The layout of a model as data: which parts, in which order, reading which
tensors.  An architecture's ``plan(config)`` returns a ``ModelPlan``; the engine
builds every model from one, so a new architecture is a new plan and, where it
needs them, new parts.

* ``layers`` — one ``LayerPlan`` per set of weights: the block's kind, the spec
  of each of its parts, and under which checkpoint prefix each part's tensors
  lie.  Layers are independent, so different layers may have different mixers
  or feed-forwards.
* ``schedule`` — the order in which layers run, as data: a list of
  ``ScheduleEntry(layer, cache_of)``.  A layer may be named twice (its weights
  run twice; each run that owns a cache has its own), and an entry may read
  another entry's cache instead of owning one (``cache_of`` = index into the
  schedule).  ``add`` = (name, row) adds row ``row`` of the model-level tensor
  ``name`` (declared in ``ModelPlan.stream_vectors``) to every row of the
  residual stream right before the entry's layer runs: what a model that goes
  through a run of layers several times adds in front of each pass.
  ``average`` = a tensor's name: the stream that goes on after the entry is a learned
  weighted sum over the embedding's output and the results of all entries up to this one
  ("depth-weighted average"); entry k's tensor holds k + 2 weights, the embedding's first.
  Either every entry of a schedule has one or none has.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from .base import PartSpec


@dataclass(frozen=True)
class LayerPlan:
    block: PartSpec                       # family "block"; its args name the parts' specs
    prefix: str                           # e.g. "model.layers.3."
    part_prefix: Dict[str, str]           # block role -> sub-prefix, e.g. {"mixer": "self_attn."}


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int
    cache_of: Optional[int] = None        # schedule index whose cache this entry uses
    add: Optional[Tuple[str, int]] = None # (stream vector's tensor name, row) added before it runs
    average: Optional[str] = None         # tensor [index + 2]: weights of the depth average behind it


@dataclass(frozen=True)
class ModelPlan:
    embedding: PartSpec
    embedding_prefix: str                 # "model.embed_tokens."
    layers: Tuple[LayerPlan, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str                # "model.norm."
    head: PartSpec
    head_prefix: str                      # "lm_head."
    vocab_size: int
    max_position: int                     # longest sequence the architecture allows
    stop_tokens: Tuple[int, ...] = ()
    stream_vectors: Tuple[Tuple[str, Tuple[int, int]], ...] = ()   # (tensor name, [rows, hidden])
    # tensors that a checkpoint may hold although nothing reads them (name, shape)
    unread_tensors: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()

    def validate(self) -> None:
        n = len(self.layers)
        vectors = dict(self.stream_vectors)
        averaged = [e.average is not None for e in self.schedule]
        if any(averaged) and not all(averaged):
            raise ValueError("a depth-averaged stream needs weights behind every schedule entry")
        for i, e in enumerate(self.schedule):
            if e.add is not None and (e.add[0] not in vectors or
                                      not 0 <= e.add[1] < vectors[e.add[0]][0]):
                raise ValueError(f"schedule entry {i} adds row {e.add[1]} of '{e.add[0]}', which "
                                 f"the plan does not declare")
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule entry {i} names layer {e.layer} of {n}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < len(self.schedule) or e.cache_of == i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                                     f"which owns none")
