"""Feed-forwards without a SwiGLU: the dense up/act/down layer and the routed mixture of clamped gated experts."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..registry import FEED_FORWARDS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(Part):
    """down(act(up(x))) with the tanh form of GELU.  Tensors: up, down."""
    kernels = ("moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.activation != "gelu_tanh":
            raise ValueError(f"dense_mlp knows the activation gelu_tanh, not {spec.activation!r}")
        self.spec = spec
        self.up = self.down = None

    def param_specs(self):
        s = self.spec
        return {"up": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX, normal_init(s.hidden_size ** -0.5)),
                "down": ParamSpec((s.hidden_size, s.intermediate_size), MATRIX, normal_init(2.0 * s.intermediate_size ** -0.5))}

    def bind(self, t):
        self.up, self.down = t["up"], t["down"]

    def setup(self, rt) -> None:
        pass

    def forward(self, x: torch.Tensor):
        return K.linear(K.gelu_tanh(K.linear(x, self.up)), self.down)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(Part):
    """down(g~ sigmoid(act_alpha g~) (u~ + 1)) with g~ = min(gate(x), limit), u~ = clamp(up(x), -limit, limit): the
    clamped gated expert as a dense layer.  The gate and up products are one (merged at bind time).  Tensors: gate, up, down."""
    kernels = ("moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        self.gate_up = self.down = None

    def param_specs(self):
        s = self.spec
        fan = normal_init(s.hidden_size ** -0.5)
        return {"gate": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX, fan),
                "up": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX, fan),
                "down": ParamSpec((s.hidden_size, s.intermediate_size), MATRIX, normal_init(2.0 * s.intermediate_size ** -0.5))}

    def bind(self, t):
        self.gate_up = torch.cat([t["gate"], t["up"]], 0).contiguous()
        self.down = t["down"]

    def setup(self, rt) -> None:
        pass

    def forward(self, x: torch.Tensor):
        s = self.spec
        return K.linear(K.moe_activation(K.linear(x, self.gate_up), None, 1, s.limit, s.act_alpha), self.down)


@FEED_FORWARDS.register("routed_mlp")
class RoutedMLP(Part):
    """`num_experts` gated experts and `num_identity` identity experts behind one router (the softmax form is described;
    `spec.score = "sigmoid"` scores every output by itself, `spec.expert = "silu"` with `spec.weigh = "input"` makes the
    expert down(silu(gate(w h)) * up(w h)), computed as silu(w g) * (w u) from the products g, u of the unweighted input).

    Router (32-bit): s = softmax(W_r h) over all outputs; the choice is made on s + correction among the experts of
    the `keep_groups` best of `num_groups` groups of neighbours; the `top` chosen ones weigh in with s * route_scale.
    Expert: g = min(W_gate h, limit), u = clamp(W_up h, +-limit), y = g sigmoid(act_alpha g) (u + 1), output W_down y.
    An identity expert's output is h itself.

    All experts' gate and up matrices are one stacked matrix, and so are their down matrices; the activation kernel
    multiplies every expert's y by the token's weight for that expert (0: not chosen), so the one stacked down product
    is already the weighted sum over the experts.  `forward` returns (rows, h, identity weight per row): the norm that
    follows adds weight * h in 32-bit.  Tensors: router, correction, e<i>.gate, e<i>.up, e<i>.down."""
    kernels = ("moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.score not in ("softmax", "sigmoid") or spec.expert not in ("clamped", "silu") or spec.weigh not in ("output", "input"):
            raise ValueError("routed_mlp knows the scores softmax | sigmoid, the experts clamped | silu, weights on output | input")
        if (spec.expert, spec.weigh) not in (("clamped", "output"), ("silu", "input")):
            raise ValueError("routed_mlp has kernels for clamped experts weighted at the output and silu experts weighted at the input")
        self.spec = spec
        self.router = self.correction = self.gate_up = self.down = None

    def param_specs(self):
        s = self.spec
        n = s.num_experts + s.num_identity
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        specs = {"router": ParamSpec((n, s.hidden_size), VECTOR, normal_init(1.5 * s.hidden_size ** -0.5))}
        if s.correction:
            specs["correction"] = ParamSpec((n,), VECTOR, normal_init(0.05))
        for e in range(s.num_experts):
            specs[f"e{e}.gate"] = ParamSpec((s.expert_size, s.hidden_size), MATRIX, fan)
            specs[f"e{e}.up"] = ParamSpec((s.expert_size, s.hidden_size), MATRIX, fan)
            specs[f"e{e}.down"] = ParamSpec((s.hidden_size, s.expert_size), MATRIX, normal_init(3.0 * s.expert_size ** -0.5))
        return specs

    def bind(self, t):
        s = self.spec
        self.router, self.correction = t["router"], t.get("correction")
        self.gate_up = torch.cat([t[f"e{e}.{n}"] for e in range(s.num_experts) for n in ("gate", "up")], 0).contiguous()
        self.down = torch.cat([t[f"e{e}.down"] for e in range(s.num_experts)], 1).contiguous()

    def setup(self, rt) -> None:
        pass

    def forward(self, x: torch.Tensor):
        s = self.spec
        dense, _, _, id_weight = K.moe_route(x, self.router, self.correction, s.num_experts, s.top, s.num_groups,
                                             s.keep_groups, s.route_scale, sigmoid_scores=s.score == "sigmoid")
        if s.num_experts == 0:
            return torch.zeros_like(x), x, id_weight
        y = K.moe_activation(K.linear(x, self.gate_up), dense, s.num_experts, s.limit, s.act_alpha,
                             mode="silu_input" if s.weigh == "input" else "clamped")
        out = K.linear(y, self.down)
        if s.num_identity == 0:
            return out
        return out, x, id_weight
