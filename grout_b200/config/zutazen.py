"""Configuration of the Zutazen decoder.

The file names the design under ``architecture`` and describes the model layer
by layer: ``layers`` is a list of objects ``{"type", "mixer", "mlp"}`` (``mlp``
null: the layer has no feed-forward).  A layer with ``weights_of: j`` has no
tensors of its own and runs layer j's (its sizes and constants are layer j's), on
a cache or state of its own.  Nothing that the arithmetic needs is defaulted.

    vocab, width                  sizes of the embedding table, the head and the stream
    embedding.scale               factor of the embedded token
    norm.eps                      epsilon of every RMS norm
    layers[i].type                "retention" | "rglru" | "latent_attention"
    layers[i].mixer (retention)   heads, dim, vdim, decay [heads], rot.{base, dims}
    layers[i].mixer (rglru)       width, blocks, conv (taps)
    layers[i].mixer (latent_attention)
                                  heads, dim, rot_dim, vdim, kv_rank, scale,
                                  rot.{base, dims}, mask.size
    layers[i].mlp                 {"kind": "dense", "ff"} or {"kind": "moe",
                                  "expert": {"ff"}, "router": {"experts", "top"}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ModelConfig

_MIXER_TYPES = ("retention", "rglru", "latent_attention")
_MLP_KINDS = ("dense", "moe")


def _number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _positive_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v > 0


def _count(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v >= 0


def _rot_problems(where, rot, limit):
    if not (isinstance(rot, dict) and _number(rot.get("base")) and rot["base"] > 0
            and _count(rot.get("dims")) and rot["dims"] % 2 == 0):
        yield f"{where}.rot needs a positive 'base' and an even 'dims', found {rot!r}"
    elif rot["dims"] > limit:
        yield f"{where}.rot.dims={rot['dims']} exceeds the {limit} elements it can turn"


@dataclass(frozen=True)
class ZutazenConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[dict, ...]
    norm: dict
    embedding: dict
    architecture: str = "Zutazen"
    eos_token_id: Optional[int] = None

    def validate(self):
        for key in ("vocab", "width"):
            if not _positive_int(getattr(self, key)):
                yield f"'{key}' must be a positive integer, found {getattr(self, key)!r}"
        if not _number(self.norm.get("eps")) or not self.norm["eps"] > 0:
            yield f"'norm.eps' must be a positive number, found {self.norm.get('eps')!r}"
        if not _number(self.embedding.get("scale")):
            yield f"'embedding.scale' must be a number, found {self.embedding.get('scale')!r}"
        if not self.layers:
            yield "'layers' is empty"
        for i, layer in enumerate(self.layers):
            yield from self._layer_problems(i, layer)

    def _layer_problems(self, i, layer):
        where = f"layers[{i}]"
        if not isinstance(layer, dict):
            yield f"{where} is not an object"
            return
        if layer.get("type") not in _MIXER_TYPES:
            yield f"{where}.type={layer.get('type')!r}: this design has {list(_MIXER_TYPES)}"
            return
        src = layer.get("weights_of")
        if src is not None:
            if not _count(src) or src >= len(self.layers) or src == i or \
                    not isinstance(self.layers[src], dict) or "weights_of" in self.layers[src]:
                yield f"{where}.weights_of={src!r} must name another layer that has tensors of its own"
            elif layer["type"] != self.layers[src].get("type"):
                yield f"{where} uses the weights of layer {src}, which is of another type"
            return
        m = layer.get("mixer")
        if not isinstance(m, dict):
            yield f"{where}.mixer is missing"
            return
        yield from getattr(self, "_" + layer["type"] + "_problems")(where + ".mixer", m)
        yield from self._mlp_problems(where, layer.get("mlp"))

    def _retention_problems(self, where, m):
        for key in ("heads", "dim", "vdim"):
            if not _positive_int(m.get(key)):
                yield f"{where}.{key} must be a positive integer, found {m.get(key)!r}"
                return
        d = m.get("decay")
        if not (isinstance(d, (list, tuple)) and len(d) == m["heads"]
                and all(_number(v) and 0 < v <= 1 for v in d)):
            yield f"{where}.decay needs one factor in (0, 1] per head, found {d!r}"
        yield from _rot_problems(where, m.get("rot"), m["dim"])

    def _rglru_problems(self, where, m):
        for key in ("width", "blocks", "conv"):
            if not _positive_int(m.get(key)):
                yield f"{where}.{key} must be a positive integer, found {m.get(key)!r}"
                return
        if m["width"] % m["blocks"]:
            yield f"{where}: {m['width']} channels do not form {m['blocks']} equal parts"

    def _latent_attention_problems(self, where, m):
        for key in ("heads", "dim", "vdim", "kv_rank"):
            if not _positive_int(m.get(key)):
                yield f"{where}.{key} must be a positive integer, found {m.get(key)!r}"
                return
        if not _count(m.get("rot_dim")) or m["rot_dim"] % 2:
            yield f"{where}.rot_dim must be an even count, found {m.get('rot_dim')!r}"
            return
        if not _number(m.get("scale")):
            yield f"{where}.scale must be a number, found {m.get('scale')!r}"
        if m["rot_dim"]:
            yield from _rot_problems(where, m.get("rot"), m["rot_dim"])
            if isinstance(m.get("rot"), dict) and m["rot"].get("dims") != m["rot_dim"]:
                yield f"{where}.rot.dims={m['rot'].get('dims')!r} must equal rot_dim={m['rot_dim']}"
        mask = m.get("mask")
        if mask is not None and not (isinstance(mask, dict) and _positive_int(mask.get("size"))):
            yield f"{where}.mask needs a positive integer 'size', found {mask!r}"

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
    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer i runs."""
        return int(self.layers[i].get("weights_of", i))

    def eos_token_ids(self) -> Tuple[int, ...]:
        return () if self.eos_token_id is None else (int(self.eos_token_id),)
