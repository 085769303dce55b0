"""
Arrangements: how a block wires its mixer, feed-forward and norms.

"pre_norm" is the reference's decoder layer (model/llama.py:238-253): the residual add is deferred
into the following norm, so a block takes and returns (branch output, residual stream).
"sandwich_norm" also norms each sublayer's output and keeps the stream in float32;
"pre_norm_stream" is the pre-norm wiring around a float32 stream.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import BlockSpec
from tinyserve_llm_b200.parts.base import Runtime, TensorDecl, part_class, register_arrangement


def _sub(tensors: dict[str, torch.Tensor], prefix: str) -> dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


@register_arrangement("pre_norm")
class PreNormBlock:
    """x = x + mixer(norm1(x)); x = x + ffn(norm2(x)), with both adds fused into the next norm."""

    takes_token_ids = True        # forward(..., embedding=table): x holds token ids, the first norm gathers the rows

    @classmethod
    def declare(cls, spec: BlockSpec) -> dict[str, TensorDecl]:
        """Names local to the block's prefix."""
        out: dict[str, TensorDecl] = {}
        for role, part, prefix in cls._members(spec):
            for name, decl in part_class(role, part).declare(part).items():
                out[prefix + name] = decl
        return out

    @staticmethod
    def _members(spec: BlockSpec):
        return (
            ("norm", spec.mixer_norm, spec.mixer_norm_prefix),
            ("mixer", spec.mixer, spec.mixer_prefix),
            ("norm", spec.feed_forward_norm, spec.feed_forward_norm_prefix),
            ("feed_forward", spec.feed_forward, spec.feed_forward_prefix),
        )

    def __init__(self, spec: BlockSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        self.spec = spec
        built = [part_class(role, part)(part, _sub(tensors, prefix), rt)
                 for role, part, prefix in self._members(spec)]
        self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward = built

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None, ctx, binding, embedding: torch.Tensor | None = None):
        """`embedding`: this is the model's first block and `x` holds token ids, rows of that table."""
        if embedding is not None:
            x, residual = self.mixer_norm.forward_embedded(embedding, x)
        else:
            x, residual = self.mixer_norm.forward(x, residual)
        x = self.mixer.forward(x, ctx, binding)
        x, residual = self.feed_forward_norm.forward(x, residual)
        x = self.feed_forward.forward(x, ctx)
        return x, residual


@register_arrangement("sandwich_norm")
class SandwichNormBlock:
    """
    x = x + norm_b(mixer(norm_a(x))); x = x + norm_d(ffn(norm_c(x))): each sublayer's input and output
    are normed, the residual stream is float32.  The add of a closed branch and the next opening norm
    are one kernel: the block hands its last branch on unclosed (`PendingBranch`) and the next block's
    first norm, or the model's final norm, closes it.  A block without a feed-forward ends after its mixer.
    """

    takes_token_ids = True
    takes_embedding_scale = True

    @staticmethod
    def _members(spec: BlockSpec):
        members = [
            ("norm", spec.mixer_norm, spec.mixer_norm_prefix),
            ("mixer", spec.mixer, spec.mixer_prefix),
            ("norm", spec.mixer_post_norm, spec.mixer_post_norm_prefix),
        ]
        if spec.feed_forward is not None:
            members += [
                ("norm", spec.feed_forward_norm, spec.feed_forward_norm_prefix),
                ("feed_forward", spec.feed_forward, spec.feed_forward_prefix),
                ("norm", spec.feed_forward_post_norm, spec.feed_forward_post_norm_prefix),
            ]
        return members

    @classmethod
    def declare(cls, spec: BlockSpec) -> dict[str, TensorDecl]:
        if spec.mixer_post_norm is None or (spec.feed_forward is not None and (
                spec.feed_forward_norm is None or spec.feed_forward_post_norm is None)):
            raise ValueError("a sandwich_norm block needs a norm before and after each of its sublayers")
        out: dict[str, TensorDecl] = {}
        for role, part, prefix in cls._members(spec):
            for name, decl in part_class(role, part).declare(part).items():
                out[prefix + name] = decl
        return out

    def __init__(self, spec: BlockSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        self.spec = spec
        built = [part_class(role, part)(part, _sub(tensors, prefix), rt) for role, part, prefix in self._members(spec)]
        self.mixer_norm, self.mixer, self.mixer_post_norm = built[:3]
        self.feed_forward_norm = self.feed_forward = self.feed_forward_post_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm, self.feed_forward, self.feed_forward_post_norm = built[3:]

    def forward(self, x, residual: torch.Tensor | None, ctx, binding, embedding: torch.Tensor | None = None,
                embedding_scale: float = 1.0):
        from tinyserve_llm_b200.parts.norm import PendingBranch
        if embedding is not None:
            h, residual = self.mixer_norm.forward_embedded(embedding, x, embedding_scale)
        else:
            h, residual = self.mixer_norm.forward(x, residual)
        branch = PendingBranch(self.mixer.forward(h, ctx, binding), self.mixer_post_norm)
        if self.feed_forward is None:
            return branch, residual
        h, residual = self.feed_forward_norm.forward(branch, residual)
        return PendingBranch(self.feed_forward.forward(h, ctx), self.feed_forward_post_norm), residual


@register_arrangement("pre_norm_stream")
class PreNormStreamBlock(PreNormBlock):
    """
    x = x + mixer(norm1(x)); x = x + ffn(norm2(x)) around a residual stream kept in float32: a sublayer's
    output travels on as a `PendingBranch` without a closing norm, and the next norm of the stream (the
    next block's first, or the model's final one) adds it and norms the sum in one kernel.  A block
    without a feed-forward ends after its mixer.
    """

    takes_token_ids = True
    takes_embedding_scale = True
    takes_embedding_position = True
    takes_embedding_norm = True

    @staticmethod
    def _members(spec: BlockSpec):
        members = [("norm", spec.mixer_norm, spec.mixer_norm_prefix), ("mixer", spec.mixer, spec.mixer_prefix)]
        if spec.feed_forward is not None:
            members += [("norm", spec.feed_forward_norm, spec.feed_forward_norm_prefix),
                        ("feed_forward", spec.feed_forward, spec.feed_forward_prefix)]
        return members

    def __init__(self, spec: BlockSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        self.spec = spec
        built = [part_class(role, part)(part, _sub(tensors, prefix), rt) for role, part, prefix in self._members(spec)]
        self.mixer_norm, self.mixer = built[:2]
        self.feed_forward_norm = self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward_norm, self.feed_forward = built[2:]

    def forward(self, x, residual: torch.Tensor | None, ctx, binding, embedding: torch.Tensor | None = None,
                embedding_scale: float = 1.0, embedding_position=None, embedding_norm=None):
        """
        `embedding_position`: a position part whose vector is added to the scaled embedding rows;
        `embedding_norm`: a stream norm the rows pass before they start the stream.
        """
        from tinyserve_llm_b200.parts.norm import PendingBranch
        if embedding is not None:
            h, residual = self.mixer_norm.forward_embedded(embedding, x, embedding_scale, positions=ctx.positions,
                                                           position=embedding_position, start_norm=embedding_norm)
        else:
            h, residual = self.mixer_norm.forward(x, residual)
        branch = PendingBranch(self.mixer.forward(h, ctx, binding), None)
        if self.feed_forward is None:
            return branch, residual
        h, residual = self.feed_forward_norm.forward(branch, residual)
        return PendingBranch(self.feed_forward.forward(h, ctx), None), residual
