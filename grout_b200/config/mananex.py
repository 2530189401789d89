"""Configuration of the Mananex decoder.

The file names the design under ``architecture`` and describes the model layer by
layer: ``layers`` is a list of objects ``{"type", "mixer", "mlp"}`` (``mlp`` null: the
layer has no feed-forward).  Nothing that the arithmetic needs is defaulted; a term
whose key is absent (``rot``, ``mask``, ``mask.keep_first``) is absent from the model.

    vocab, width                  sizes of the embedding table (which is also the head) and the stream
    norm.eps                      epsilon of every RMS norm
    layers[i].type                "parallel": two mixers side by side
    layers[i].mixer               left, right, left_scale, right_scale
    layers[i].mixer.left          heads, kv_heads, dim, vdim, scale, rot.{base, dims},
                                  mask.{size, keep_first}
    layers[i].mixer.right         heads, dim, vdim
    layers[i].mlp                 {"kind": "dense", "ff"} or {"kind": "moe",
                                  "expert": {"ff"}, "router": {"experts", "top"}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ModelConfig

_LAYER_TYPES = ("parallel",)
_MLP_KINDS = ("dense", "moe")


def _number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _positive_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v > 0


def _count(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v >= 0


@dataclass(frozen=True)
class MananexConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[dict, ...]
    norm: dict
    architecture: str = "Mananex"
    eos_token_id: Optional[int] = None

    def validate(self):
        for key in ("vocab", "width"):
            if not _positive_int(getattr(self, key)):
                yield f"'{key}' must be a positive integer, found {getattr(self, key)!r}"
        if not _number(self.norm.get("eps")) or not self.norm["eps"] > 0:
            yield f"'norm.eps' must be a positive number, found {self.norm.get('eps')!r}"
        if not self.layers:
            yield "'layers' is empty"
        for i, layer in enumerate(self.layers):
            yield from self._layer_problems(i, layer)

    def _layer_problems(self, i, layer):
        where = f"layers[{i}]"
        if not isinstance(layer, dict):
            yield f"{where} is not an object"
            return
        if layer.get("type") not in _LAYER_TYPES:
            yield f"{where}.type={layer.get('type')!r}: this design has {list(_LAYER_TYPES)}"
            return
        m = layer.get("mixer")
        if not isinstance(m, dict) or not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
            yield f"{where}.mixer needs the objects 'left' and 'right'"
            return
        for key in ("left_scale", "right_scale"):
            if not _number(m.get(key)):
                yield f"{where}.mixer.{key} must be a number, found {m.get(key)!r}"
        yield from self._left_problems(where + ".mixer.left", m["left"])
        yield from self._right_problems(where + ".mixer.right", m["right"])
        yield from self._mlp_problems(where, layer.get("mlp"))

    def _left_problems(self, where, m):
        for key in ("heads", "kv_heads", "dim", "vdim"):
            if not _positive_int(m.get(key)):
                yield f"{where}.{key} must be a positive integer, found {m.get(key)!r}"
                return
        if m["heads"] % m["kv_heads"]:
            yield f"{where}: {m['heads']} heads cannot share {m['kv_heads']} kv heads"
        if not _number(m.get("scale")):
            yield f"{where}.scale must be a number, found {m.get('scale')!r}"
        rot = m.get("rot")
        if rot is not None:
            if not (isinstance(rot, dict) and _number(rot.get("base")) and rot["base"] > 0
                    and _count(rot.get("dims")) and rot["dims"] % 2 == 0):
                yield f"{where}.rot needs a positive 'base' and an even 'dims', found {rot!r}"
            elif rot["dims"] > m["dim"]:
                yield f"{where}.rot.dims={rot['dims']} exceeds the head's {m['dim']} elements"
        mask = m.get("mask")
        if mask is not None:
            if not (isinstance(mask, dict) and _positive_int(mask.get("size"))
                    and _count(mask.get("keep_first", 0))):
                yield (f"{where}.mask needs a positive integer 'size' and, if given, a count "
                       f"'keep_first', found {mask!r}")

    def _right_problems(self, where, m):
        for key in ("heads", "dim", "vdim"):
            if not _positive_int(m.get(key)):
                yield f"{where}.{key} must be a positive integer, found {m.get(key)!r}"

    def _mlp_problems(self, where, mlp):
        if mlp is None:
            return
        if not isinstance(mlp, dict) or mlp.get("kind") not in _MLP_KINDS:
            yield f"{where}.mlp.kind={mlp!r}: this design has {list(_MLP_KINDS)}"
            return
        if mlp["kind"] == "dense":
            if not _positive_int(mlp.get("ff")):
                yield f"{where}.mlp.ff must be a positive integer, found {mlp.get('ff')!r}"
            return
        ex, r = mlp.get("expert"), mlp.get("router")
        if not (isinstance(ex, dict) and _positive_int(ex.get("ff"))):
            yield f"{where}.mlp.expert needs a positive integer 'ff', found {ex!r}"
        if not (isinstance(r, dict) and _positive_int(r.get("experts")) and _positive_int(r.get("top"))):
            yield f"{where}.mlp.router needs positive integers 'experts' and 'top', found {r!r}"
        elif r["top"] > r["experts"]:
            yield f"{where}.mlp.router.top={r['top']} exceeds its {r['experts']} experts"

    # ---- derived -------------------------------------------------------
    def eos_token_ids(self) -> Tuple[int, ...]:
        return () if self.eos_token_id is None else (int(self.eos_token_id),)
