"""
Routed experts: `num_experts` small gated feed-forward layers of which each token uses the `top`
with the largest router logits, weighted by the softmax over the chosen logits; a shared expert, if
the layer has one, runs for every token and is added.

    z = W_r h + b  (float32)      chosen = top-`top` of z      share = softmax(z[chosen])
    y = sum_j share_j expert_chosen_j(h)  (+ shared(h))

One step runs: the router product, routing and a sort of the (token, choice) pairs by expert on the
device (nothing is read back, so the step can be replayed from a CUDA graph), one grouped product
gate/up with the activation in its epilogue, one grouped product down, and the weighted sum.  The
experts' weights are stacked [experts, 2 ff, width] and [experts, width, ff].

Variants, by the spec: `scoring` "sigmoid" weighs a chosen expert by sigmoid(z) without renormalising;
`weight_on` "input" multiplies the expert's input by the weight instead of its output (experts without
a gate, `PlainMLPSpec`: down(relu(up(w h))^2) = down(relu(w * up(h))^2), so the weight goes into the
first product's epilogue and the outputs are summed unweighted).  `scoring` "softmax_all": the scores
are the softmax over all router outputs, the choice goes by score + a stored correction inside the best
groups of neighbouring outputs, the weights are the chosen scores over their sum, times a constant; the
router's last `identity_experts` outputs are experts without tensors whose output is their input, so
their weights are added up per token and multiply h in the kernel that sums the experts' outputs.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import GatedMLPSpec, RoutedExpertsSpec
from tinyserve_llm_b200.parts.base import FeedForward, Runtime, TensorDecl, part_class, register_part
from tinyserve_llm_b200.parts.linear import Linear


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    @classmethod
    def declare(cls, spec: RoutedExpertsSpec) -> dict[str, TensorDecl]:
        if spec.expert is None or not 0 < spec.top <= spec.num_experts + spec.identity_experts:
            raise ValueError(f"routed experts need an expert description and 0 < top <= experts, got top={spec.top}, "
                             f"experts={spec.num_experts + spec.identity_experts}")
        if spec.scoring not in ("softmax_chosen", "sigmoid", "softmax_all") or spec.weight_on not in ("output", "input"):
            raise NotImplementedError(f"routed experts: scoring {spec.scoring!r}, weight on {spec.weight_on!r}")
        outputs = spec.num_experts + spec.identity_experts
        if spec.scoring != "softmax_all" and (spec.identity_experts or spec.correction_name or spec.group_count != 1):
            raise NotImplementedError("routed experts: groups, a correction and identity experts come with scoring 'softmax_all'")
        if spec.scoring == "softmax_all" and (spec.weight_on != "output" or spec.router_bias_name or spec.group_count <= 0
                                              or outputs % spec.group_count or not 0 < spec.group_keep <= spec.group_count
                                              or spec.top > spec.group_keep * (outputs // spec.group_count)):
            raise ValueError(f"routed experts: {outputs} router outputs, {spec.group_keep} of {spec.group_count} groups kept, "
                             f"top {spec.top}: the groups must be equal and hold enough outputs; no router bias, weights on the output")
        if isinstance(spec.expert, GatedMLPSpec) and spec.weight_on == "input":
            raise NotImplementedError("routed experts: a weight on the input is built for experts without a gate")
        expert_class = part_class("feed_forward", spec.expert)
        out = {spec.router_name: TensorDecl((outputs, spec.hidden_size))}
        if spec.correction_name:
            out[spec.correction_name] = TensorDecl((outputs,))
        if spec.router_bias_name:
            out[spec.router_bias_name] = TensorDecl((spec.num_experts,))
        for e in range(spec.num_experts):
            for name, decl in expert_class.declare(spec.expert).items():
                out[spec.expert_prefix.format(e) + name] = decl
        if spec.shared is not None:
            for name, decl in part_class("feed_forward", spec.shared).declare(spec.shared).items():
                out[spec.shared_prefix + name] = decl
        return out

    def __init__(self, spec: RoutedExpertsSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        self.declare(spec)
        pre = [spec.expert_prefix.format(e) for e in range(spec.num_experts)]
        to = dict(device=rt.device, dtype=rt.dtype)
        self.gated = isinstance(spec.expert, GatedMLPSpec)
        if self.gated:
            gate, up, down = spec.expert.tensor_names
            self.gate_up = torch.stack([torch.cat([tensors[p + gate], tensors[p + up]], dim=0) for p in pre]).to(**to).contiguous()
        else:
            up, down = spec.expert.tensor_names
            part_class("feed_forward", spec.expert)          # the expert's kind is known
            self.gate_up = torch.stack([tensors[p + up] for p in pre]).to(**to).contiguous()
        self.down = torch.stack([tensors[p + down] for p in pre]).to(**to).contiguous()
        self.router = Linear(tensors[spec.router_name], rt)
        self.router_bias = None
        if spec.router_bias_name:
            self.router_bias = tensors[spec.router_bias_name].to(device=rt.device, dtype=torch.float32).contiguous()
        self.correction = None
        if spec.correction_name:
            self.correction = tensors[spec.correction_name].to(device=rt.device, dtype=torch.float32).contiguous()
        self.shared = None
        if spec.shared is not None:
            sub = {k[len(spec.shared_prefix):]: v for k, v in tensors.items() if k.startswith(spec.shared_prefix)}
            self.shared = part_class("feed_forward", spec.shared)(spec.shared, sub, rt)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        spec, ops = self.spec, self.rt.ops
        T, top = x.shape[0], spec.top
        logits = self.router(x, out_dtype=torch.float32)
        identity_share = None
        if spec.scoring == "softmax_all":
            _, share, offsets, pair_of_row, row_of_pair, identity_share = ops.moe_route_grouped(
                logits, self.correction, ctx, top, real_experts=spec.num_experts, groups=spec.group_count,
                keep=spec.group_keep, weight_scale=spec.weight_scale, share_eps=spec.share_eps)
        else:
            _, share, offsets, pair_of_row, row_of_pair = ops.moe_route(logits, self.router_bias, ctx, top, spec.scoring)
        e = spec.expert
        on_input = spec.weight_on == "input"
        if self.gated:
            hidden = ops.moe_linear(x, self.gate_up, offsets, pair_of_row, top, T * top, e.activation, e.limit, e.alpha)
        else:
            hidden = ops.moe_linear(x, self.gate_up, offsets, pair_of_row, top, T * top, e.activation,
                                    row_scale=share if on_input else None)
        y = ops.moe_linear(hidden, self.down, offsets, None, top, T * top)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        return ops.moe_combine(y, row_of_pair, None if on_input else share, shared, T, x=x, identity_share=identity_share)
