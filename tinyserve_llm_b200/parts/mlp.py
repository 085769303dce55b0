"""
Dense gated feed-forward: down(act(gate(x)) * up(x)), gate and up fused into one projection whose
output columns are [gate | up].  Activations: silu(g) u (with the products that carry it in their
epilogue), relu(g) u, the clamped swish g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit),
u' = clamp(u, -limit, limit), and the tanh form of gelu, g/2 (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) u.

Reference: model/llama.py:77-83 (silu(gate) * up), :215-225 (fused gate_up, down; no biases).
"""

from __future__ import annotations

import math

import torch

from tinyserve_llm_b200.config.spec import GatedMLPSpec, PlainMLPSpec
from tinyserve_llm_b200.parts.base import FeedForward, Runtime, TensorDecl, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True

    ACTIVATIONS = ("silu", "relu", "clamped_swish", "gelu_tanh")

    @classmethod
    def declare(cls, spec: GatedMLPSpec) -> dict[str, TensorDecl]:
        gate, up, down = spec.tensor_names
        return {
            gate: TensorDecl((spec.intermediate_size, spec.hidden_size)),
            up: TensorDecl((spec.intermediate_size, spec.hidden_size)),
            down: TensorDecl((spec.hidden_size, spec.intermediate_size)),
        }

    def __init__(self, spec: GatedMLPSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        if spec.activation not in self.ACTIVATIONS:
            raise NotImplementedError(f"activation {spec.activation!r} is not supported; have {self.ACTIVATIONS}")
        gate, up, down = spec.tensor_names
        self.gate_up = Linear(fuse_rows([tensors[gate], tensors[up]]), rt)
        self.down = Linear(tensors[down], rt)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        spec, ops = self.spec, self.rt.ops
        # the gate/up products carry the activation in their epilogue where there is a kernel of the engine's own for the size
        return self.down(ops.linear_gated(x, self.gate_up.weight, spec.activation, spec.limit, spec.alpha))


@register_part("feed_forward", "plain_mlp")
class PlainMLP(FeedForward):
    """
    Ungated feed-forward down(act(up(x))) with act the square of relu, or xIELU: with the two numbers
    p, q of the layer's parameter tensor, softplus(p) z^2 + z/2 for z > 0 and
    (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2 for z <= 0.  The two factors are worked out once, in
    float64, when the layer is built.
    """

    graph_safe = True

    ACTIVATIONS = ("relu2", "xielu")

    @classmethod
    def declare(cls, spec: PlainMLPSpec) -> dict[str, TensorDecl]:
        up, down = spec.tensor_names
        out = {up: TensorDecl((spec.intermediate_size, spec.hidden_size)),
               down: TensorDecl((spec.hidden_size, spec.intermediate_size))}
        if spec.activation == "xielu":
            if not spec.param_name:
                raise ValueError("an xIELU layer needs the name of its parameter tensor")
            out[spec.param_name] = TensorDecl((2,))
        return out

    def __init__(self, spec: PlainMLPSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        if spec.activation not in self.ACTIVATIONS:
            raise NotImplementedError(f"activation {spec.activation!r} is not supported; have {self.ACTIVATIONS}")
        up, down = spec.tensor_names
        self.up = Linear(tensors[up], rt)
        self.down = Linear(tensors[down], rt)
        self.factors = (0.0, 0.0)
        if spec.activation == "xielu":
            p, q = (float(v) for v in tensors[spec.param_name].to(torch.float64).cpu().tolist())
            softplus = lambda v: v if v > 30 else math.log1p(math.exp(v))  # noqa: E731
            self.factors = (softplus(p), 0.5 + softplus(q))

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        # a few rows: the activation rides in the up product's epilogue; more: the library's product, then one pass
        return self.down(self.rt.ops.linear_unary(x, self.up.weight, self.spec.activation, *self.factors))
