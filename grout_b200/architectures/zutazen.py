"""The Zutazen decoder as a plan.

Pre-norm layers, x <- x + M(N1(x)); x <- x + F(N2(x)) with RMS norms, on a stream
that starts as the embedded token times a constant.  A layer's mixer M is
retention (a fading matrix-valued state per head, read without a softmax), a
gated linear recurrence per channel behind a short convolution, or attention
over a window of the last tokens whose keys and values come from one latent
vector per token.  Its feed-forward F, if it has one, is a gated one with biases
and a relu gate, or a mixture of small experts with silu gates whose router
scores are sigmoids that weigh the expert's input.  A layer may run another
layer's tensors on a cache or state of its own.  This file holds the
checkpoint's tensor names, the constants the design fixes and the order of the
parts; every size and every other constant comes from the configuration.

Tensor names: ``embed``, ``final.norm``, ``head`` and per layer i ``l<i>.norm1`` /
``norm2``; a retention mixer's ``l<i>.mix.{q,k,v,g,o}``; a recurrence's
``l<i>.mix.{y,x,conv,ra,ri}`` each with ``.b``, ``lam``, ``o``; a latent attention's
``l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}``; ``l<i>.mlp.{gate,up,down}`` each with ``.b``,
or ``l<i>.mlp.e<j>.{gate,up,down}`` and ``router``.
"""
from __future__ import annotations

from ..config import ZutazenConfig, register_architecture
from ..parts.base import PartSpec
from ..parts.plan import LayerPlan, ModelPlan, ScheduleEntry

LOG_DECAY_FACTOR = 8.0            # log a = -8 r softplus(lam) in the gated recurrence
NO_POSITION_LIMIT = 1 << 30       # nothing in the design bounds a sequence's length


def _rms(dim: int, eps: float, name: str) -> PartSpec:
    return PartSpec("rmsnorm", dict(dim=dim, eps=eps, name=name))


def _mixer(kind: str, width: int, m: dict, eps: float) -> PartSpec:
    if kind == "retention":
        rot = m["rot"]
        position = (PartSpec("rotary_half_split", dict(head_dim=m["dim"], theta=float(rot["base"]),
                                                       rot_dim=int(rot["dims"]), exact_table=True))
                    if rot["dims"] else PartSpec("none", {}))
        return PartSpec("retention", dict(
            hidden=width, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
            decay=tuple(float(d) for d in m["decay"]), position=position, norm_eps=eps,
            k_scale=float(m["dim"]) ** -0.5))
    if kind == "rglru":
        return PartSpec("gated_linear_recurrence", dict(
            hidden=width, width=m["width"], blocks=m["blocks"], conv_taps=m["conv"],
            log_decay_factor=LOG_DECAY_FACTOR))
    dr = int(m["rot_dim"])
    position = (PartSpec("rotary_interleaved", dict(head_dim=dr, theta=float(m["rot"]["base"]),
                                                    rot_dim=dr, exact_table=True))
                if dr else PartSpec("none", {}))
    mask = m.get("mask")
    return PartSpec("latent_attention", dict(
        hidden=width, n_heads=m["heads"], head_dim=m["dim"], rot_dim=dr, v_head_dim=m["vdim"],
        kv_rank=m["kv_rank"], position=position, scale=float(m["scale"]), norm_eps=eps,
        window=int(mask["size"]) if mask else None, gated=True))


def _feedforward(width: int, mlp: dict) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", dict(
            hidden=width, intermediate=int(mlp["ff"]), activation="relu", bias=True,
            names={"gate": "gate", "up": "up", "down": "down", "gate_bias": "gate.b",
                   "up_bias": "up.b", "down_bias": "down.b"}))
    r, ex = mlp["router"], mlp["expert"]
    return PartSpec("routed_experts", dict(
        hidden=width, intermediate=int(ex["ff"]), n_experts=int(r["experts"]), top=int(r["top"]),
        limit=None, gate_slope=1.0, up_offset=0.0, score_fn="sigmoid", correction=False,
        weigh_input=True))


def zutazen_plan(cfg: ZutazenConfig) -> ModelPlan:
    W, eps = cfg.width, float(cfg.norm["eps"])
    own = [i for i in range(len(cfg.layers)) if cfg.weights_layer(i) == i]
    index = {layer: n for n, layer in enumerate(own)}
    layers = []
    for i in own:
        layer = cfg.layers[i]
        args = dict(mixer=_mixer(layer["type"], W, layer["mixer"], eps), norm1=_rms(W, eps, ""))
        if layer.get("mlp") is not None:
            args.update(feedforward=_feedforward(W, layer["mlp"]), norm2=_rms(W, eps, ""))
        layers.append(LayerPlan(PartSpec("prenorm", args), f"l{i}.", {
            "norm1": "norm1", "norm2": "norm2", "mixer": "mix.", "feedforward": "mlp."}))
    # a layer that runs another's tensors is one more run of that layer, with a
    # cache or state of its own
    schedule = tuple(ScheduleEntry(index[cfg.weights_layer(i)]) for i in range(len(cfg.layers)))
    return ModelPlan(
        embedding=PartSpec("token", dict(vocab=cfg.vocab, hidden=W, name="embed",
                                         scale=float(cfg.embedding["scale"]))),
        embedding_prefix="",
        layers=tuple(layers),
        schedule=schedule,
        final_norm=_rms(W, eps, ""),
        final_norm_prefix="final.norm",
        head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=W, tied=False, name="head")),
        head_prefix="",
        vocab_size=cfg.vocab,
        max_position=NO_POSITION_LIMIT,
        stop_tokens=cfg.eos_token_ids(),
    )


register_architecture("Zutazen", ZutazenConfig, zutazen_plan, model_types=("zutazen",))
