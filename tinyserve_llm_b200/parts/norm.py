"""
RMSNorm with the residual add fused in; further down, the norm beside a float32 residual stream.

Reference formulas (model/llama.py:52-67): s = f32(x) + f32(residual); the carried residual is s
rounded to the activation dtype; y = s * rsqrt(mean(s^2) + eps) uses the unrounded sum; the output
is round(y) * weight, the weight multiply coming after the rounding.  Without a residual, x itself
starts the residual stream (model/llama.py:246-247).
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import RMSNormSpec
from tinyserve_llm_b200.parts.base import Norm, Runtime, TensorDecl, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    @classmethod
    def declare(cls, spec: RMSNormSpec) -> dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.size,), init="unit")}

    def __init__(self, spec: RMSNormSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        w = tensors["weight"]
        # A weight stored in 32-bit floats stays so; the kernel takes either beside bf16 activations.
        keep = w.dtype if (w.dtype == torch.float32 or rt.dtype == torch.float32) else rt.dtype
        if rt.dtype == torch.float32:
            keep = torch.float32
        self.weight = w.to(device=rt.device, dtype=keep).contiguous()
        self.eps = float(spec.eps)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None,
                rows: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        return self.rt.ops.add_rmsnorm(x, residual, self.weight, self.eps, rows)

    def forward_embedded(self, table: torch.Tensor, ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return self.rt.ops.embed_rmsnorm(table, ids, self.weight, self.eps)


class PendingBranch:
    """
    A sublayer's output whose closing norm has not been applied yet: the next norm of the stream adds
    closing(branch) to the stream and norms the sum in one kernel.  Blocks that norm the outputs of
    their sublayers hand this on as `x`, the next block's first norm (or the model's final norm) takes it.
    """

    __slots__ = ("tensor", "closing")

    def __init__(self, tensor: torch.Tensor, closing: "StreamRMSNorm | None") -> None:
        self.tensor = tensor
        self.closing = closing


@register_part("norm", "rmsnorm_stream")
class StreamRMSNorm(Norm):
    """
    RMS norm beside a float32 residual stream: y = s / sqrt(mean(s^2) + eps) * (offset + w), statistics,
    weight and stream in float32, y in the activation dtype.  `forward(x, residual)`: x is None (the
    stream is only normed) or a `PendingBranch` (its closing norm is applied, the result added to the
    stream, the sum normed).
    """

    graph_safe = True
    centered = False          # a subclass norms around the mean (layer norm)

    @classmethod
    def declare(cls, spec) -> dict[str, TensorDecl]:
        return {spec.weight_name: TensorDecl((spec.size,), init="normal" if spec.weight_offset else "unit")}

    def __init__(self, spec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        w = tensors[spec.weight_name].to(device=rt.device, dtype=torch.float32)
        self.weight = (w + float(spec.weight_offset)).contiguous() if spec.weight_offset else w.contiguous()
        self.eps = float(spec.eps)

    def forward(self, x, residual: torch.Tensor | None, rows: torch.Tensor | None = None):
        if residual is None:
            raise ValueError("a stream norm needs the residual stream (the first norm starts it from the embedding)")
        branch = closing = None
        if isinstance(x, PendingBranch):
            branch, closing = x.tensor, (x.closing.weight if x.closing is not None else None)
        elif x is not None:
            raise ValueError("a stream norm takes a PendingBranch (a sublayer's output and its closing norm) or nothing")
        out = self.rt.ops.stream_norm(branch, closing, residual, self.weight, self.eps, self.rt.dtype, rows=rows,
                                      centered=self.centered, plain_add=branch is not None and closing is None)
        return out, residual

    def close(self, branch: torch.Tensor, residual: torch.Tensor) -> None:
        """stream += closing(branch), with no norm of the sum."""
        self.rt.ops.stream_norm(branch, self.weight, residual, None, self.eps, self.rt.dtype)

    def forward_embedded(self, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0, positions: torch.Tensor | None = None,
                         position=None, start_norm: "StreamRMSNorm | None" = None):
        """
        `position` (a part with `frequencies`) and `positions`: its vector is added to the scaled rows.
        `start_norm` (a stream norm of this norm's kind and eps): the rows are normed by it before they start the stream.
        """
        if start_norm is not None and (start_norm.centered != self.centered or start_norm.eps != self.eps):
            raise NotImplementedError("a norm on the embedding runs inside the first norm's kernel: both must be of one kind and eps")
        residual = torch.empty((ids.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
        out = self.rt.ops.stream_norm(None, None, residual, self.weight, self.eps, self.rt.dtype, table=table, ids=ids,
                                      scale=scale, centered=self.centered, positions=positions,
                                      position_frequencies=position.frequencies if position is not None else None,
                                      w_start=start_norm.weight if start_norm is not None else None)
        return out, residual


@register_part("norm", "layernorm_stream")
class StreamLayerNorm(StreamRMSNorm):
    """
    Layer norm with a weight and no bias beside a float32 residual stream:
    y = (s - mean(s)) / sqrt(mean((s - mean(s))^2) + eps) * w, statistics, weight and stream in float32.
    """

    centered = True
