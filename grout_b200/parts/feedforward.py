"""Feed-forward parts.  Interface of the family: ``forward(x, step) -> y`` with
``x`` and ``y`` [T, hidden] in the compute dtype (``y`` may be a stack of 32-bit
partial sums [S, T, hidden], which the next norm adds: see ``Norm.add_norm``).  A feed-forward with experts
routes inside ``forward``; the rows' packing is the step's and does not change.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import BuildContext, ParamSpec, Part, register_part
from .linear import Linear


class FeedForward(Part):
    family = "feedforward"

    def forward(self, x, step):
        raise NotImplementedError


@register_part("feedforward", "swiglu")
class SwiGLU(FeedForward):
    """d = (silu(x Wg^T) * (x Wu^T)) Wd^T, no biases (src/training.rs:344-349).
    Gate and up are fused into one product at load (src/model.rs:1401)."""

    def __init__(self, ctx: BuildContext, hidden: int, intermediate: int):
        super().__init__(ctx)
        self.hidden, self.intermediate = int(hidden), int(intermediate)
        self.gate_up = self.down = None
        self.interleave = 0

    def param_specs(self):
        return {"gate_proj.weight": ParamSpec((self.intermediate, self.hidden)),
                "up_proj.weight": ParamSpec((self.intermediate, self.hidden)),
                "down_proj.weight": ParamSpec((self.hidden, self.intermediate))}

    def load(self, params):
        g, u = params["gate_proj.weight"], params["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError("gate and up projections must be stored in one dtype to be fused")
        # bf16: rows interleaved in groups of 8 (8 gates, their 8 ups, ...) so that
        # the decode product holds a gate and its up in one tile and can apply
        # silu(gate) * up before it stores
        self.interleave = 8 if (g.dtype == torch.bfloat16 and self.intermediate % 8 == 0
                                and self.hidden % 8 == 0) else 0
        if self.interleave:
            k = self.interleave
            fused = torch.stack([g.view(-1, k, self.hidden), u.view(-1, k, self.hidden)], dim=1)
            self.gate_up = Linear(fused.reshape(2 * self.intermediate, self.hidden), self.ctx.products)
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0), self.ctx.products)
        self.down = Linear(params["down_proj.weight"], self.ctx.products)

    def kernel_modules(self):
        return ("elementwise",) + self.gate_up.kernel_modules() + self.down.kernel_modules()

    def captures_prompts(self):
        return True

    def forward(self, x, step):
        return self.down(self.gate_up.silu_mul(x, self.interleave), partial_ok=True)


@register_part("feedforward", "relu2_mlp")
class ReluSquaredMLP(FeedForward):
    """d = (max(x Wu^T, 0))^2 Wd^T, no biases, no gate.  The square of the relu
    is taken in 32-bit on the product's accumulator where the product's kernel
    has that epilogue, else by a kernel of its own.  ``names``: the local names of
    the two tensors (keys up, down)."""

    def __init__(self, ctx: BuildContext, hidden: int, intermediate: int, names=None):
        super().__init__(ctx)
        self.hidden, self.intermediate = int(hidden), int(intermediate)
        self.names = dict({"up": "up_proj.weight", "down": "down_proj.weight"}, **(names or {}))
        self.up = self.down = None

    def param_specs(self):
        return {self.names["up"]: ParamSpec((self.intermediate, self.hidden)),
                self.names["down"]: ParamSpec((self.hidden, self.intermediate))}

    def load(self, params):
        self.up = Linear(params[self.names["up"]], self.ctx.products)
        self.down = Linear(params[self.names["down"]], self.ctx.products)

    def kernel_modules(self):
        return ("elementwise",) + self.up.kernel_modules() + self.down.kernel_modules()

    def captures_prompts(self):
        return True

    def forward(self, x, step):
        return self.down(self.up.relu_squared(x), partial_ok=True)


@register_part("feedforward", "gated_mlp")
class GatedMLP(FeedForward):
    """d = (act(x Wg^T) * (x Wu^T)) Wd^T with ``activation`` "silu", "gelu_tanh"
    (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))) or "relu".  Gate and up are
    one product; the activation and the multiplication are taken in 32-bit on its
    result.  With ``bias`` each of the three projections has a bias,
    d = (act(x Wg^T + bg) * (x Wu^T + bu)) Wd^T + bd: the biases are added to the
    products' 32-bit sums, and the result leaves as 32-bit sums for the next norm to
    add.  ``names``: the tensors' local names (keys gate, up, down and, with biases,
    gate_bias, up_bias, down_bias)."""

    ACTIVATIONS = ("silu", "gelu_tanh", "relu")

    def __init__(self, ctx: BuildContext, hidden: int, intermediate: int,
                 activation: str = "silu", names=None, bias: bool = False):
        super().__init__(ctx)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"activation '{activation}': one of {list(self.ACTIVATIONS)}")
        self.hidden, self.intermediate, self.activation = int(hidden), int(intermediate), activation
        self.has_bias = bool(bias)
        self.names = dict({"gate": "gate_proj.weight", "up": "up_proj.weight",
                           "down": "down_proj.weight", "gate_bias": "gate_proj.bias",
                           "up_bias": "up_proj.bias", "down_bias": "down_proj.bias"}, **(names or {}))
        self.gate_up = self.down = self.gate_up_bias = self.down_bias = None
        self.interleave = 0

    def param_specs(self):
        nm = self.names
        specs = {nm["gate"]: ParamSpec((self.intermediate, self.hidden)),
                 nm["up"]: ParamSpec((self.intermediate, self.hidden)),
                 nm["down"]: ParamSpec((self.hidden, self.intermediate))}
        if self.has_bias:
            specs.update({nm["gate_bias"]: ParamSpec((self.intermediate,), "offset"),
                          nm["up_bias"]: ParamSpec((self.intermediate,), "offset"),
                          nm["down_bias"]: ParamSpec((self.hidden,), "offset")})
        return specs

    def load(self, params):
        g, u = params[self.names["gate"]], params[self.names["up"]]
        if g.dtype != u.dtype:
            raise ValueError("gate and up projections must be stored in one dtype to be fused")
        # bf16: rows interleaved in groups of 8 (8 gates, their 8 ups, ...), the layout in
        # which the tcgen05 products apply the activation before they store
        self.interleave = 8 if (g.dtype == torch.bfloat16 and self.intermediate % 8 == 0
                                and self.hidden % 8 == 0) else 0
        if self.interleave:
            k = self.interleave
            fused = torch.stack([g.view(-1, k, self.hidden), u.view(-1, k, self.hidden)], dim=1)
            self.gate_up = Linear(fused.reshape(2 * self.intermediate, self.hidden), self.ctx.products)
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0), self.ctx.products)
        self.down = Linear(params[self.names["down"]], self.ctx.products)
        if self.has_bias:       # 32-bit, in the fused product's order of rows
            bg, bu = params[self.names["gate_bias"]].float(), params[self.names["up_bias"]].float()
            if self.interleave:
                k = self.interleave
                fused_b = torch.stack([bg.view(-1, k), bu.view(-1, k)], dim=1).reshape(-1)
            else:
                fused_b = torch.cat([bg, bu])
            self.gate_up_bias = fused_b.contiguous()
            self.down_bias = params[self.names["down_bias"]].float().contiguous()

    def kernel_modules(self):
        return ("elementwise",) + self.gate_up.kernel_modules() + self.down.kernel_modules()

    def captures_prompts(self):
        return True

    def forward(self, x, step):
        if self.has_bias:
            # the biases join the product's 32-bit sums: in its epilogue where it has one
            inner = self.gate_up.silu_mul(x, self.interleave, self.activation, bias=self.gate_up_bias)
            d = self.down(inner, out_dtype=torch.float32, partial_ok=True)
            # partial sums: the bias joins the first; else one 32-bit term for the norm to add
            d = d if d.dim() == 3 else d.unsqueeze(0)
            ops.add_bias_(d[0], self.down_bias)
            return d
        return self.down(self.gate_up.silu_mul(x, self.interleave, self.activation), partial_ok=True)


@register_part("feedforward", "routed_experts")
class RoutedExperts(FeedForward):
    """``n_experts`` small gated feed-forwards of which every token uses ``top``.

        z = Wr x (32-bit), s = softmax(z) over all n_experts + n_identity outputs
        (``score_fn`` "sigmoid": s = sigmoid(z), every output by itself; "softmax_top": the
        logits z themselves choose, and the chosen weigh in with the softmax over their own
        logits alone; ``router_bias``: z = Wr x + b, b the tensor ``router_bias_name``)
        c = s + correction (``correction`` False: there is none, c = s);  the outputs form ``n_groups`` equal groups of neighbours,
        a group's score is its largest c, only outputs of the ``keep_groups`` best
        groups can be chosen; the ``top`` largest c are chosen and weigh in with s
        expert:  g = min(Wg x, limit), u = clamp(Wu x, -limit, limit),
                 y = Wd (g sigmoid(gate_slope g) (u + 1))
        the last ``n_identity`` outputs stand for experts that return x itself
        out = sum of s * y over the chosen; the weights are not renormalised
        ``limit`` None clamps nothing; ``up_offset`` is the 1 of (u + 1);
        ``weigh_input``: the weight multiplies the expert's input instead of its
        result, out = sum of expert(s x)

    Tensors: ``router`` [n_experts + n_identity, hidden], ``correction``, and per
    expert j ``e<j>.gate`` / ``e<j>.up`` [intermediate, hidden], ``e<j>.down``.  The
    result leaves as ``top`` weighted 32-bit partial sums, which the next norm adds."""

    def __init__(self, ctx: BuildContext, hidden: int, intermediate: int, n_experts: int, top: int,
                 limit: Optional[float], gate_slope: float, n_identity: int = 0, n_groups: int = 1,
                 keep_groups: int = 1, score_fn: str = "softmax", correction: bool = True,
                 weigh_input: bool = False, up_offset: float = 1.0, router_bias: bool = False,
                 router_bias_name: str = "router.b"):
        super().__init__(ctx)
        self.hidden, self.intermediate = int(hidden), int(intermediate)
        self.E, self.n_identity, self.top = int(n_experts), int(n_identity), int(top)
        self.n_groups, self.keep_groups = int(n_groups), int(keep_groups)
        self.limit = math.inf if limit is None else float(limit)
        self.gate_slope, self.up_offset = float(gate_slope), float(up_offset)
        if score_fn not in ops.MOE_SCORE_FNS:
            raise ValueError(f"score function '{score_fn}': one of {sorted(ops.MOE_SCORE_FNS)}")
        self.score_fn, self.has_correction, self.weigh_input = score_fn, bool(correction), bool(weigh_input)
        self.has_router_bias, self.router_bias_name = bool(router_bias), router_bias_name
        self.router_b = None
        n_all = self.E + self.n_identity
        if n_all % self.n_groups or not 1 <= self.keep_groups <= self.n_groups:
            raise ValueError(f"{n_all} router outputs do not form {self.n_groups} equal groups "
                             f"of which {self.keep_groups} are kept")
        if not 1 <= self.top <= self.keep_groups * (n_all // self.n_groups):
            raise ValueError(f"top={self.top} exceeds what {self.keep_groups} groups hold")
        self.router_w = self.correction = self.w_gate = self.w_up = self.w_down = None

    def param_specs(self):
        n_all = self.E + self.n_identity
        specs = {"router": ParamSpec((n_all, self.hidden))}
        if self.has_correction:
            specs["correction"] = ParamSpec((n_all,), "offset")
        if self.has_router_bias:
            specs[self.router_bias_name] = ParamSpec((n_all,), "offset")
        for j in range(self.E):
            specs[f"e{j}.gate"] = ParamSpec((self.intermediate, self.hidden))
            specs[f"e{j}.up"] = ParamSpec((self.intermediate, self.hidden))
            specs[f"e{j}.down"] = ParamSpec((self.hidden, self.intermediate))
        return specs

    def load(self, params):
        # the router is 32-bit whatever the checkpoint stores
        self.router_w = params["router"].float().contiguous()
        self.correction = params["correction"].float().contiguous() if self.has_correction else None
        self.router_b = (params[self.router_bias_name].float().contiguous()
                         if self.has_router_bias else None)
        stack = lambda what: torch.stack([params[f"e{j}.{what}"] for j in range(self.E)]).to(
            self.ctx.dtype).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")

    def kernel_modules(self):
        return ("moe",)

    def captures_prompts(self):
        return True

    def forward(self, x, step):
        return ops.moe_forward(x, self.router_w, self.correction, self.w_gate, self.w_up,
                               self.w_down, top=self.top, n_identity=self.n_identity,
                               n_groups=self.n_groups, keep_groups=self.keep_groups,
                               limit=self.limit, slope=self.gate_slope, score_fn=self.score_fn,
                               weigh_input=self.weigh_input, up_offset=self.up_offset,
                               router_bias=self.router_b)
