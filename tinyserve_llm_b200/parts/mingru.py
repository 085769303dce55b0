"""
Element-wise gated recurrence whose gates read the current token only (a minGRU).

    z = sigmoid(W_z h + b_z)        u = W_x h + b_x        c = u + 1/2 where u >= 0, sigmoid(u) below
    S_t = (1 - z_t) S_(t-1) + z_t c_t                      one number a channel, zero before the first token
    y = W_o (S_t * silu(W_g h))

The three projections that read h are one product [z | x | g] whose output stays float32, so that
what enters the recurrence is rounded nowhere; gates, candidate, state and the product with silu(g)
are float32 in one kernel that walks a request's tokens in order (long portions: in stretches whose
summaries are chained).  The state (float32 [width]) lives in the cache manager's per-request slot:
it is zeroed at admission, carried from step to step and given back at release.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import MinGRUSpec
from tinyserve_llm_b200.parts.base import Mixer, Runtime, TensorDecl, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows


@register_part("mixer", "mingru")
class MinGRU(Mixer):
    graph_safe = True

    @classmethod
    def validate(cls, spec: MinGRUSpec) -> None:
        if spec.width <= 0 or spec.hidden_size <= 0:
            raise ValueError(f"a minGRU of {spec.width} channels over a stream of {spec.hidden_size}")

    @classmethod
    def declare(cls, spec: MinGRUSpec) -> dict[str, TensorDecl]:
        cls.validate(spec)
        W, hidden = spec.width, spec.hidden_size
        out = {"z": TensorDecl((W, hidden)), "x": TensorDecl((W, hidden)), "g": TensorDecl((W, hidden)),
               "o": TensorDecl((hidden, W))}
        if spec.bias:
            out.update({"z.b": TensorDecl((W,)), "x.b": TensorDecl((W,))})
        return out

    def __init__(self, spec: MinGRUSpec, tensors: dict[str, torch.Tensor], rt: Runtime, fused: bool = False) -> None:
        super().__init__(spec, tensors, rt)
        self.validate(spec)
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.input_rows = fuse_rows([tensors["z"], tensors["x"], tensors["g"]])
        self.out_weight = tensors["o"]
        self.inner_width = spec.width
        self.z_bias = tensors["z.b"].to(**f32).contiguous() if spec.bias else None
        self.x_bias = tensors["x.b"].to(**f32).contiguous() if spec.bias else None
        self.proj = self.out = None
        if not fused:
            self.proj, self.out = Linear(self.input_rows, rt), Linear(self.out_weight, rt)

    def state_bytes(self) -> int:
        return self.spec.width * 4

    def inner(self, y: torch.Tensor, x: torch.Tensor, ctx, binding, scale: float = 1.0,
              out: torch.Tensor | None = None) -> torch.Tensor:
        """y: this mixer's columns [z | x | g] of the projection of x (float32 or the activation dtype).  Returns [T, width]."""
        W = self.spec.width
        o = self.rt.ops.mingru_scan(y, (0, W, 2 * W), self.z_bias, self.x_bias, ctx, binding, W, self.rt.dtype)
        if scale != 1.0:
            o = o * scale
        if out is not None:
            out.copy_(o)
            return out
        return o

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        return self.out(self.inner(self.proj(x, out_dtype=torch.float32), x, ctx, binding))
