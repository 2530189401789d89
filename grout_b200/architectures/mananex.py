"""The Mananex decoder as a plan.

"Parallel" layers on a depth-averaged stream: a layer takes one RMS norm (weight stored
around zero) of the stream, its mixer and its feed-forward both read that, and each
result is multiplied by a sigmoid gate computed from the same input before it is added;
what goes on to the next layer is a learned weighted sum over the embedding's output and
the results of all layers so far.  The mixer is two mixers side by side, added with
constant factors: grouped-query attention (rotation of neighbouring pairs on part of a
head, a sliding window that keeps the sequence's first tokens, a learned sink per head, a
sigmoid gate per head) and a linear attention whose forget gate also decides what is
written.  The feed-forward is a silu-gated one with biases or a mixture of small experts
whose router weighs the chosen by the softmax over their logits alone.  The head is the
embedding table.  This file holds the checkpoint's tensor names and the order of the
parts; every size and constant comes from the configuration.

Tensor names: ``embed``, ``final.norm`` and per layer i ``l<i>.norm1``, ``l<i>.rg1`` /
``rg2`` each with ``.b``, ``l<i>.dwa``; ``l<i>.mix.left.{q,k,v,sink,g,o}``;
``l<i>.mix.right.{q,f,f.b,lower,v,norm,o}``; ``l<i>.mlp.{gate,up,down}`` each with ``.b``, or
``l<i>.mlp.e<j>.{gate,up,down}`` with ``router`` and ``router.b``.
"""
from __future__ import annotations

from ..config import MananexConfig, register_architecture
from ..parts.base import PartSpec
from ..parts.plan import LayerPlan, ModelPlan, ScheduleEntry

NO_POSITION_LIMIT = 1 << 30       # nothing in the design bounds a sequence's length


def _norm(dim: int, eps: float) -> PartSpec:
    return PartSpec("rmsnorm", dict(dim=dim, eps=eps, name="", unit_offset=True))


def _left(width: int, m: dict) -> PartSpec:
    rot, mask = m.get("rot"), m.get("mask")
    position = (PartSpec("rotary_interleaved", dict(head_dim=m["dim"], theta=float(rot["base"]),
                                                    rot_dim=int(rot["dims"]), exact_table=True))
                if rot and rot["dims"] else PartSpec("none", {}))
    return PartSpec("gqa_attention", dict(
        hidden=width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
        v_head_dim=m["vdim"], position=position, scale=float(m["scale"]),
        window=int(mask["size"]) if mask else None,
        keep_first=int(mask.get("keep_first", 0)) if mask else 0,
        sinks=True, head_gate=True,
        names={"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink", "g": "g"}))


def _right(width: int, m: dict, eps: float) -> PartSpec:
    return PartSpec("forget_gate_attention", dict(
        hidden=width, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"], norm_eps=eps))


def _mixer(width: int, m: dict, eps: float) -> PartSpec:
    return PartSpec("side_by_side", dict(hidden=width, mixers=(
        ("left", _left(width, m["left"]), float(m["left_scale"])),
        ("right", _right(width, m["right"], eps), float(m["right_scale"])))))


def _feedforward(width: int, mlp: dict) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", dict(
            hidden=width, intermediate=int(mlp["ff"]), activation="silu", bias=True,
            names={"gate": "gate", "up": "up", "down": "down", "gate_bias": "gate.b",
                   "up_bias": "up.b", "down_bias": "down.b"}))
    r, ex = mlp["router"], mlp["expert"]
    return PartSpec("routed_experts", dict(
        hidden=width, intermediate=int(ex["ff"]), n_experts=int(r["experts"]), top=int(r["top"]),
        limit=None, gate_slope=1.0, up_offset=0.0, score_fn="softmax_top", correction=False,
        router_bias=True, router_bias_name="router.b"))


def mananex_plan(cfg: MananexConfig) -> ModelPlan:
    W, eps = cfg.width, float(cfg.norm["eps"])
    layers = []
    for i, layer in enumerate(cfg.layers):
        args = dict(norm1=_norm(W, eps), mixer=_mixer(W, layer["mixer"], eps), gated=True,
                    gate1="rg1", gate2="rg2", bias_suffix=".b")
        if layer.get("mlp") is not None:
            args["feedforward"] = _feedforward(W, layer["mlp"])
        layers.append(LayerPlan(PartSpec("parallel", args), f"l{i}.", {
            "norm1": "norm1", "mixer": "mix.", "feedforward": "mlp."}))
    schedule = tuple(ScheduleEntry(i, average=f"l{i}.dwa") for i in range(len(cfg.layers)))
    return ModelPlan(
        embedding=PartSpec("token", dict(vocab=cfg.vocab, hidden=W, name="embed", scale=1.0)),
        embedding_prefix="",
        layers=tuple(layers),
        schedule=schedule,
        final_norm=_norm(W, eps),
        final_norm_prefix="final.norm",
        head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=W, tied=True)),
        head_prefix="",
        vocab_size=cfg.vocab,
        max_position=NO_POSITION_LIMIT,
        stop_tokens=cfg.eos_token_ids(),
    )


register_architecture("Mananex", MananexConfig, mananex_plan, model_types=("mananex",))
