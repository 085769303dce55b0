"""
Attention over a cached latent: per token the cache keeps c = norm(W_dkv h)[:kv_rank] and one rotated
key part k_rot shared by all heads; a head's keys and values are W_uk,h c and W_uv,h c.

    c_q = norm(W_dq h),  q = W_uq c_q  laid out per head as [head_dim unrotated | rot_dim rotated]
    score_h(i, j) = (q_flat,h(i) . W_uk,h c(j) + rot(q_rot,h(i)) . k_rot(j)) * scale
    y = W_o concat_h( W_uv,h sum_j softmax_j(score_h(i, .)) c(j) )

Since q_flat . (W_uk c) = (W_uk^T q_flat) . c, the engine folds W_uk into the query (one batched
product per step) and W_uv into the output of the attention (another), and the attention kernel
works on cache rows [c | k_rot] directly: keys and values of a head are never materialised, in prompts
as in decoding.  The cache entry is one "kv head" of kv_rank + rot_dim channels without a value pool;
a window makes it a layer group of its own whose pages are given back as the window passes.

Options of the description: `q_rank` 0 makes the queries a projection of the input, q = W_q h, without a
latent and a norm of their own; `rot_dim` 0 leaves out the rotated part (attention without positions: the
cache row is c alone and no position part is built); `output_gate` multiplies the concatenated heads by
sigmoid(W_g h), read from the same input as the other projections, before W_o.

Prompt portions of a step that is launched once (not replayed from a CUDA graph) take another way where the
sizes allow (bfloat16, no rotated part, key and value heads of one size the tcgen05 prompt kernel takes): the
latents of the requests' whole contexts are gathered from the pages, a head's keys and values are worked out
for the step (K = C W_uk^T, V = C W_uv^T, two library products: a quarter of the folded form's arithmetic at
a latent of 512 channels and heads of 128) and the tcgen05 prompt kernel attends over them; requests that feed
one token in the same step stay on the folded form.  The two ways differ by rounding only.

Tensors (local names): dq, dq.norm, uq (or q), dkv, dkv.norm, uk, uv, o, and g with an output gate.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import LatentAttentionSpec
from tinyserve_llm_b200.parts.base import KVNeed, Mixer, Runtime, TensorDecl, part_class, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows

MAX_KV_RANK = 512       # csrc/attention_latent.cu: 16 output channels a lane
MATERIALIZE_MIN_TOKENS = 128    # prompt portions of a step, together, from which keys and values are worked out for the step


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    @classmethod
    def validate(cls, spec: LatentAttentionSpec) -> None:
        if spec.kv_rank > MAX_KV_RANK:
            raise ValueError(f"kv_rank={spec.kv_rank} is not supported: the latent attention kernel takes up to {MAX_KV_RANK}")
        if spec.rot_dim % 2 or spec.rot_dim < 0 or spec.q_rank < 0:
            raise ValueError(f"rot_dim={spec.rot_dim} must be even and q_rank={spec.q_rank} not negative")
        if (spec.rot_dim > 0) != (spec.position is not None):
            raise ValueError("latent attention: a rotated key part and a position part come together")

    @classmethod
    def declare(cls, spec: LatentAttentionSpec) -> dict[str, TensorDecl]:
        cls.validate(spec)
        H, D, R, V = spec.num_heads, spec.head_dim, spec.rot_dim, spec.value_dim
        out = {
            "dkv": TensorDecl((spec.kv_rank + R, spec.hidden_size)), "dkv.norm": TensorDecl((spec.kv_rank,), init="unit"),
            "uk": TensorDecl((H * D, spec.kv_rank)), "uv": TensorDecl((H * V, spec.kv_rank)),
            "o": TensorDecl((spec.hidden_size, H * V)),
        }
        if spec.q_rank > 0:
            out.update({"dq": TensorDecl((spec.q_rank, spec.hidden_size)), "dq.norm": TensorDecl((spec.q_rank,), init="unit"),
                        "uq": TensorDecl((H * (D + R), spec.q_rank))})
        else:
            out["q"] = TensorDecl((H * (D + R), spec.hidden_size))
        if spec.output_gate:
            out["g"] = TensorDecl((H * V, spec.hidden_size))
        return out

    def __init__(self, spec: LatentAttentionSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        self.validate(spec)
        H, D, V, rank = spec.num_heads, spec.head_dim, spec.value_dim, spec.kv_rank
        # one product of the input: columns [c_q raw (or q) | c raw | k_rot raw | gate logits]
        rows = [tensors["dq"] if spec.q_rank > 0 else tensors["q"], tensors["dkv"]] + ([tensors["g"]] if spec.output_gate else [])
        self.down = Linear(fuse_rows(rows), rt)
        self.q_norm = self.up_q = None
        if spec.q_rank > 0:
            self.q_norm = tensors["dq.norm"].to(device=rt.device, dtype=torch.float32).contiguous()
            self.up_q = Linear(tensors["uq"], rt)
        self.kv_norm = tensors["dkv.norm"].to(device=rt.device, dtype=torch.float32).contiguous()
        # W_uk per head, transposed to [H, rank, D]: the product that folds it into the query reads rows of D
        self.uk_t = tensors["uk"].to(device=rt.device, dtype=rt.dtype).view(H, D, rank).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].to(device=rt.device, dtype=rt.dtype).view(H, V, rank).contiguous()
        # the unfolded form of prompt portions: W_uk as stored, [H D, rank] (W_uv's stored form is self.uv's memory)
        self.uk = self.uk_t.transpose(1, 2).reshape(H * D, rank).contiguous() if spec.rot_dim == 0 and D == V else None
        self.out = Linear(tensors["o"], rt)
        self.position = self.frequencies = None
        if spec.position is not None:
            self.position = part_class("position", spec.position)(spec.position, {}, rt)
            if getattr(self.position, "frequencies", None) is None or self.position.dims != spec.rot_dim:
                raise NotImplementedError("latent attention rotates inside its kernels: it takes a position part with "
                                          "`frequencies` over exactly rot_dim channels")
            self.frequencies = self.position.frequencies

    def kv_need(self) -> KVNeed:
        return KVNeed(1, self.spec.kv_rank + self.spec.rot_dim, self.spec.window, values=False)

    # ------------------------------------------------------------------ prompt portions on keys and values of their own
    def _portions(self, q: torch.Tensor, ctx) -> list[int] | None:
        """The step's requests that feed more than one token, if their attention is to run on keys and values worked out for the step."""
        spec, host = self.spec, getattr(ctx, "host", None)
        if (self.uk is None or spec.window or getattr(ctx, "replayed", True) or host is None or ctx.max_q_len <= 1
                or not self.rt.ops.dense_prompt_attention_supported(q, spec.num_heads, spec.num_heads, spec.head_dim)):
            return None
        lens = [b - a for a, b in zip(host.cu_q, host.cu_q[1:])]
        portions = [s for s, n in enumerate(lens) if n > 1]
        if sum(lens[s] for s in portions) < MATERIALIZE_MIN_TOKENS:
            return None
        return portions

    @staticmethod
    def _single_tokens_only(ctx):
        """The step's context with the tokens of prompt portions marked as padding rows: the folded form skips them."""
        import copy
        lens = ctx.cu_q[1:] - ctx.cu_q[:-1]
        seqs = ctx.seq_of_token.long().clamp_min(0)
        out = copy.copy(ctx)
        out.seq_of_token = torch.where((ctx.seq_of_token >= 0) & (lens[seqs] == 1), ctx.seq_of_token, -1).to(torch.int32)
        return out

    def _attend_unfolded(self, q: torch.Tensor, ctx, binding, portions: list[int], out: torch.Tensor | None) -> torch.Tensor:
        spec, ops, host = self.spec, self.rt.ops, ctx.host
        H, D, rank, B = spec.num_heads, spec.head_dim, spec.kv_rank, binding.page_tokens
        entries = binding.page_stride // (B * rank)
        pool = binding.k_pool.view(binding.num_pages, entries, B, rank)[:, binding.entry_offset // (B * rank)]
        starts, latents, at = [0] * len(host.ctx_lens), [], 0
        for s in portions:                                  # the latents of the whole context, page by page
            n = host.ctx_lens[s]
            pages = binding.block_table[s, :-(-n // B)].long()
            latents.append(pool[pages].reshape(-1, rank)[:n])
            starts[s], at = at, at + n
        c = torch.cat(latents) if len(latents) > 1 else latents[0].contiguous()
        kv_start = torch.tensor(starts, dtype=torch.int32).to(q.device, non_blocking=True)
        k = ops.linear(c, self.uk)                          # [keys, H D]
        v = ops.linear(c, self.uv.view(H * spec.value_dim, rank))
        return ops.dense_prompt_attention(q, k, v, kv_start, ctx, H, H, D, spec.scale, out)

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        spec, ops = self.spec, self.rt.ops
        H, D, R, V, rank = spec.num_heads, spec.head_dim, spec.rot_dim, spec.value_dim, spec.kv_rank
        y = self.down(x)                                                  # [T, (q_rank or H (D + R)) + rank + R (+ H V)]
        if spec.q_rank > 0:
            latents = spec.q_rank + rank + R
            c_q = ops.latent_prepare(y[:, :latents], ctx, binding, spec.q_rank, rank, R, self.q_norm, self.kv_norm,
                                     spec.norm_eps, self.frequencies)    # normed query latent; [c | k_rot] is in the cache
            q = self.up_q(c_q)                                            # [T, H (D + R)]
        else:
            latents = H * (D + R) + rank + R
            q = y[:, :H * (D + R)]
            ops.latent_prepare(y[:, H * (D + R):latents], ctx, binding, 0, rank, R, None, self.kv_norm, spec.norm_eps,
                               self.frequencies)
        portions = self._portions(q, ctx)
        if portions is not None and ctx.min_q_len > 1:
            o = self._attend_unfolded(q, ctx, binding, portions, None)
        else:
            folded_ctx = ctx if portions is None else self._single_tokens_only(ctx)
            q_lat = ops.per_head_linear(q, self.uk_t, H, D + R, D)        # float32 [T, H, rank]: W_uk^T q_flat
            o_lat = ops.latent_attention(q_lat, q, folded_ctx, binding, H, D + R, D, rank, R, self.frequencies,
                                         spec.scale, spec.window)         # [T, H, rank]: softmax-weighted sums of c
            o = ops.per_head_linear(o_lat.view(-1, H * rank), self.uv, H, rank, rank, out_dtype=x.dtype)   # [T, H, V]
            o = o.reshape(-1, H * V)
            if portions is not None:                                      # the portions' rows are written over
                o = self._attend_unfolded(q, ctx, binding, portions, o.contiguous())
        if spec.output_gate:
            o = ops.sigmoid_gate(o, y[:, latents:latents + H * V])
        return self.out(o)
