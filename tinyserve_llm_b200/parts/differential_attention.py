"""
Differential attention: every head holds two score maps over the same values, and its output is the
difference of the two attentions, normed.

    q = W_q h (+ b_q)   [heads x 2 maps x dim],   k = W_k h (+ b_k)   [kv heads x 2 maps x dim],   v = W_v h (+ b_v)
    rotation of the first `dims` channels of every map of every head of q and k
    a_m = softmax_j(cap(q_m . k_m * scale)) v      for the two maps m, over the keys the mask leaves visible
    o = (a_1 - lambda a_2) / sqrt(mean((a_1 - lambda a_2)^2) + eps) * (1 - difference)       a head at a time, no weight
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + difference                                     one number for the layer
    y = W_o concat(o)

For the attention kernels a map is a head: 2 x heads query heads, 2 x kv heads key heads, kv heads value
heads (`value_heads` of the kernels: a query head's value head is its key head's index without the map).
So that the query heads of one key head lie side by side, as grouped-query attention has them, the rows of
W_q (and b_q) are put into the order [kv head][map][head of the group] when the part is built; the maps'
outputs come back in that order (float32 from the generic kernel, so that the difference is taken of
unrounded numbers; bfloat16 from the tensor-core kernels) and one
kernel takes the difference and the norm and writes the heads in their own order.  lambda is worked out
once, in float64, from the four tensors.  Keys of both maps and values live in the paged cache, the value pool
with half as many heads as the key pool.

Tensors (local names): q, k, v, o, lq1, lk1, lq2, lk2, and q.b, k.b, v.b with biases.
"""

from __future__ import annotations

import math

import torch

from tinyserve_llm_b200.config.spec import DifferentialAttentionSpec
from tinyserve_llm_b200.parts.base import KVNeed, Mixer, Runtime, TensorDecl, part_class, register_part
from tinyserve_llm_b200.parts.gated_attention import MAX_HEAD_DIM, kept_keys
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows

MAPS = 2


def group_maps_together(rows: torch.Tensor, heads: int, kv_heads: int, dim: int) -> torch.Tensor:
    """Rows (or elements) laid out [head][map][dim] into the order [kv head][map][head of the group][dim]."""
    per_group = heads // kv_heads
    shaped = rows.reshape(kv_heads, per_group, MAPS, dim, *rows.shape[1:])
    return shaped.transpose(1, 2).reshape(rows.shape).contiguous()


@register_part("mixer", "differential_attention")
class DifferentialAttention(Mixer):
    graph_safe = True

    @classmethod
    def validate(cls, spec: DifferentialAttentionSpec) -> None:
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_kv_heads={spec.num_kv_heads}")
        for name, size in (("head_dim", spec.head_dim), ("value_dim", spec.value_dim)):
            if not 0 < size <= MAX_HEAD_DIM:
                raise ValueError(f"{name}={size} is not supported: the attention kernels take up to {MAX_HEAD_DIM}")
        if spec.window < 0 or spec.chunk < 0 or spec.softcap < 0:
            raise ValueError("differential attention: window, chunk and softcap must not be negative")

    @classmethod
    def declare(cls, spec: DifferentialAttentionSpec) -> dict[str, TensorDecl]:
        cls.validate(spec)
        nq, nk = spec.num_heads * MAPS * spec.head_dim, spec.num_kv_heads * MAPS * spec.head_dim
        nv, no = spec.num_kv_heads * spec.value_dim, spec.num_heads * spec.value_dim
        out = {"q": TensorDecl((nq, spec.hidden_size)), "k": TensorDecl((nk, spec.hidden_size)),
               "v": TensorDecl((nv, spec.hidden_size)), "o": TensorDecl((spec.hidden_size, no))}
        if spec.bias:
            out.update({"q.b": TensorDecl((nq,)), "k.b": TensorDecl((nk,)), "v.b": TensorDecl((nv,))})
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[name] = TensorDecl((spec.head_dim,))
        return out

    def __init__(self, spec: DifferentialAttentionSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        self.validate(spec)
        H, G, D = spec.num_heads, spec.num_kv_heads, spec.head_dim
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.proj = Linear(fuse_rows([group_maps_together(tensors["q"], H, G, D), tensors["k"], tensors["v"]]), rt)
        self.out = Linear(tensors["o"], rt)
        self.biases = None
        if spec.bias:
            self.biases = (group_maps_together(tensors["q.b"], H, G, D).to(**f32).contiguous(),
                           tensors["k.b"].to(**f32).contiguous(), tensors["v.b"].to(**f32).contiguous())
        dot = {n: float((tensors["lq" + n].to(torch.float64) * tensors["lk" + n].to(torch.float64)).sum()) for n in "12"}
        self.weight = math.exp(dot["1"]) - math.exp(dot["2"]) + float(spec.difference)
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position)(spec.position, {}, rt)
            if getattr(self.position, "frequencies", None) is None:
                raise NotImplementedError("this attention rotates q and k in its own kernel: it takes a position part "
                                          "with `frequencies`")

    def kv_need(self) -> KVNeed:
        s = self.spec
        return KVNeed(MAPS * s.num_kv_heads, s.head_dim, kept_keys(s.window, s.chunk), True,
                      0 if s.value_dim == s.head_dim else s.value_dim, s.num_kv_heads)

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        s, ops = self.spec, self.rt.ops
        H, G, D, V = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        nq, nk = H * MAPS * D, G * MAPS * D
        y = self.proj(x)                                                # [q (maps grouped) | k | v]
        q = ops.qk_norm_rope_store(y, (0, nq, nq + nk), self.biases, None, s.norm_eps, self.position, ctx, binding,
                                   MAPS * H, MAPS * G, D, V, value_heads=G)
        # the generic kernel leaves the maps unrounded; the tensor-core kernels (sizes they take, bfloat16) write bfloat16
        precise = None if ops.tensor_core_attention(q, binding, MAPS * H, MAPS * G, D, V, ctx) else torch.float32
        maps = ops.paged_attention_split(q, ctx, binding, MAPS * H, MAPS * G, D, V, s.scale, s.window, softcap=s.softcap,
                                         chunk=s.chunk, value_heads=G, out_dtype=precise)
        o = ops.difference_head_norm(maps, ctx, H, G, V, self.weight, s.norm_eps, 1.0 - s.difference, x.dtype)
        return self.out(o)
