"""
Causal grouped-query softmax attention with the extras some designs put around it: biases on q, k
and v, an RMS norm of q and of k over the whole projection (all heads at once) before the rotation,
values of another head size than keys, and a sigmoid output gate on the concatenated heads.

    q = W_q h (+ b_q), k, v likewise;  q <- q / rms(q) * w_q over all heads' channels, k likewise
    rotation of the first `dims` channels of every head of q and k (angles in float32, in the kernel)
    o_head = softmax(q . k * scale over the keys up to the query's own) v
    y = W_o (concat(o) * sigmoid(W_g h))

Options a design may switch on (`GatedAttentionSpec`): a norm of q and of k head by head with one
weight shared by the heads; a query temperature q <- q (1 + c ln(floor((p + 1) / n) + 1)) at position
p; a distance penalty slope_h (i - j) taken off the score with slope_h = 2^(-c (h + 1) / heads); a
number per head added to every score; sigmoid weights instead of a softmax (a visible key's weight is
sigmoid(score), nothing is normalised over the keys); an output gate of one number a head; chunks of n
positions, counted from the request's first token, outside of which a query sees nothing (the cache keeps
the last n keys, as for a window of n); scores capped as c tanh(score / c).  With any of the last six the
attention runs on the kernels that carry them (`paged_attention_split`'s options).

Keys (rotated) and values live in the paged cache; one kernel norms, rotates and stores, one attends
(the tensor-core kernels where keys and values share a head size they take, the generic one else),
one gates.  The mixer can stand alone or beside others in a `ParallelMixer`, which fuses the
projections that read h and the output projections: for that it exposes its input rows, the part
between the two projections (`inner`) and its output weight.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import GatedAttentionSpec
from tinyserve_llm_b200.parts.base import KVNeed, Mixer, Runtime, TensorDecl, part_class, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows

MAX_HEAD_DIM = 256      # csrc/attention_generic.cu


def kept_keys(window: int, chunk: int) -> int:
    """How many of the latest keys the cache has to keep for a mask of a window, of chunks, or both (0: all)."""
    return min(window, chunk) if window > 0 and chunk > 0 else max(window, chunk)


@register_part("mixer", "gated_attention")
class GatedAttention(Mixer):
    graph_safe = True

    @classmethod
    def validate(cls, spec: GatedAttentionSpec) -> None:
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_kv_heads={spec.num_kv_heads}")
        for name, size in (("head_dim", spec.head_dim), ("value_dim", spec.value_dim)):
            if not 0 < size <= MAX_HEAD_DIM:
                raise ValueError(f"{name}={size} is not supported: the attention kernels take up to {MAX_HEAD_DIM}")
        if spec.qk_norm_scope not in ("projection", "head") or spec.output_gate_scope not in ("channel", "head"):
            raise NotImplementedError(f"attention: norm scope {spec.qk_norm_scope!r}, gate scope {spec.output_gate_scope!r}")
        if spec.weights not in ("softmax", "sigmoid"):
            raise NotImplementedError(f"attention: weights {spec.weights!r}; have softmax and sigmoid")
        if spec.q_temperature_every < 0 or spec.distance_slope_exponent < 0 or spec.window < 0 or spec.chunk < 0 or spec.softcap < 0:
            raise ValueError("attention: q_temperature_every, distance_slope_exponent, window, chunk and softcap must not be negative")

    @classmethod
    def declare(cls, spec: GatedAttentionSpec) -> dict[str, TensorDecl]:
        cls.validate(spec)
        nq, nk, nv = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.num_kv_heads * spec.value_dim
        no = spec.num_heads * spec.value_dim
        out = {"q": TensorDecl((nq, spec.hidden_size)), "k": TensorDecl((nk, spec.hidden_size)),
               "v": TensorDecl((nv, spec.hidden_size)), "o": TensorDecl((spec.hidden_size, no))}
        if spec.bias:
            out.update({"q.b": TensorDecl((nq,)), "k.b": TensorDecl((nk,)), "v.b": TensorDecl((nv,))})
        if spec.qk_norm:
            per_head = spec.qk_norm_scope == "head"
            out.update({"q.norm": TensorDecl((spec.head_dim if per_head else nq,), init="unit"),
                        "k.norm": TensorDecl((spec.head_dim if per_head else nk,), init="unit")})
        if spec.head_bias:
            out["pb"] = TensorDecl((spec.num_heads,))
        if spec.output_gate:
            out["g"] = TensorDecl((spec.num_heads if spec.output_gate_scope == "head" else no, spec.hidden_size))
        return out

    def __init__(self, spec: GatedAttentionSpec, tensors: dict[str, torch.Tensor], rt: Runtime, fused: bool = False) -> None:
        super().__init__(spec, tensors, rt)
        self.validate(spec)
        f32 = dict(device=rt.device, dtype=torch.float32)
        rows = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if spec.output_gate else [])
        self.input_rows = fuse_rows(rows)
        self.out_weight = tensors["o"]
        self.inner_width = spec.num_heads * spec.value_dim
        self.biases = tuple(tensors[n].to(**f32).contiguous() for n in ("q.b", "k.b", "v.b")) if spec.bias else None
        self.norm_weights = tuple(tensors[n].to(**f32).contiguous() for n in ("q.norm", "k.norm")) if spec.qk_norm else None
        self.head_bias = tensors["pb"].to(**f32).contiguous() if spec.head_bias else None
        self.slopes = None
        if spec.distance_slope_exponent > 0:
            c, H = float(spec.distance_slope_exponent), spec.num_heads
            self.slopes = torch.tensor([2.0 ** (-c * (h + 1) / H) for h in range(H)], **f32)
        self.q_temperature = (float(spec.q_temperature_coef), int(spec.q_temperature_every)) if spec.q_temperature_every > 0 else None
        self.gate_width = 0 if not spec.output_gate else (spec.num_heads if spec.output_gate_scope == "head" else self.inner_width)
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position)(spec.position, {}, rt)
            if getattr(self.position, "frequencies", None) is None:
                raise NotImplementedError("this attention rotates q and k in its own kernel: it takes a position part "
                                          "with `frequencies`")
        self.proj = self.out = None
        if not fused:
            self.proj, self.out = Linear(self.input_rows, rt), Linear(self.out_weight, rt)

    def kv_need(self) -> KVNeed:
        s = self.spec
        return KVNeed(s.num_kv_heads, s.head_dim, kept_keys(s.window, s.chunk), True, 0 if s.value_dim == s.head_dim else s.value_dim)

    def inner(self, y: torch.Tensor, x: torch.Tensor, ctx, binding, scale: float = 1.0,
              out: torch.Tensor | None = None) -> torch.Tensor:
        """y: this mixer's columns of the projection of x, [q | k | v | g].  Returns [T, heads * value_dim] * scale."""
        s, ops = self.spec, self.rt.ops
        nq, nk, nv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * s.value_dim
        q = ops.qk_norm_rope_store(y, (0, nq, nq + nk), self.biases, self.norm_weights, s.qk_norm_eps, self.position,
                                   ctx, binding, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim,
                                   norm_per_head=s.qk_norm_scope == "head", q_temperature=self.q_temperature)
        gate = y[:, nq + nk + nv:nq + nk + nv + self.gate_width] if s.output_gate else None
        per_head_gate = s.output_gate and s.output_gate_scope == "head"
        o = ops.paged_attention_split(q, ctx, binding, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, s.scale, s.window,
                                      weights=s.weights, slopes=self.slopes, head_bias=self.head_bias,
                                      head_gate=gate if per_head_gate else None, softcap=s.softcap, chunk=s.chunk)
        if per_head_gate:                               # the gate went into the attention kernel's last step
            if scale != 1.0:
                o = o * scale
            if out is not None:
                out.copy_(o)
                return out
            return o
        if s.output_gate:
            return ops.sigmoid_gate(o, y[:, nq + nk + nv:nq + nk + nv + self.inner_width], scale, out)
        if out is not None:
            out.copy_(o if scale == 1.0 else o * scale)
            return out
        return o if scale == 1.0 else o * scale

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        return self.out(self.inner(self.proj(x), x, ctx, binding))
