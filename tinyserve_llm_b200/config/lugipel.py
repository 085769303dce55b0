"""
Typed configuration of the Lugipel decoder, read from the keys of its own config.json, and the
`ModelSpec` it turns into.

config.json: `architecture` "Lugipel", `vocab`, `width`, `norm.eps`, `embedding.scale` and `layers`,
a list whose entries give `type` (the mixer: "mingru" or "attention"), `mixer` (its sizes and
constants) and `mlp` (`kind` "dense" with `ff`; `kind` "moe" with `expert.ff` and `router` holding
`experts`, `top`, `identity`, `scale` and `groups` with `count` and `keep`; or null for a layer
without a feed-forward).  A "mingru" mixer holds `width`; an "attention" mixer holds `heads`,
`kv_heads`, `dim`, `vdim`, `scale`, `mask.size` and `q_temp` with `coef` and `every`.  Layers may come
in any order and number; every size is read here and nowhere else.  Tensors: `embed`, `final.norm`,
`head`, and per layer `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`.

What the design fixes stands here as constants: RMS norms with a plain weight before each sublayer
around a float32 residual stream; a sinusoidal position vector (base 10000, sine and cosine
interleaved) on the scaled embedding; attention without rotation whose queries and keys are normed
head by head, whose scores lose slope_h (i - j) with slope_h = 2^(-8 (h + 1) / heads), gain a number
per head and become weights through a sigmoid, with one sigmoid output gate a head; dense layers
up, xIELU, down; experts gate, silu, up, down, chosen through a softmax over all router outputs
with a correction, inside the best groups, the chosen scores divided by their sum + 1e-20.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from tinyserve_llm_b200.config.duduvik import DEFAULT_MAX_POSITIONS, _get
from tinyserve_llm_b200.config.llama import ConfigError
from tinyserve_llm_b200.config.spec import (
    BlockSpec,
    GatedAttentionSpec,
    GatedMLPSpec,
    MinGRUSpec,
    ModelSpec,
    PartSpec,
    PlainMLPSpec,
    RoutedExpertsSpec,
    RunEntry,
    SinusoidSpec,
    StreamRMSNormSpec,
)

MIXER_TYPES = ("mingru", "attention")
MLP_KINDS = ("dense", "moe")
SINUSOID_BASE = 10000.0
SLOPE_EXPONENT = 8.0
SHARE_EPS = 1e-20


@dataclass(frozen=True)
class LugipelLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None


def _count(raw: Mapping[str, Any], path: str, default: int | None = None) -> int:
    """A whole number that may be zero."""
    node: Any = raw
    for key in path.split("."):
        if not isinstance(node, Mapping) or key not in node:
            if default is not None:
                return default
            raise ConfigError(f"config.json lacks {path!r}")
        node = node[key]
    if isinstance(node, bool) or not isinstance(node, int) or node < 0:
        raise ConfigError(f"config.json: {path} must be a whole number, got {node!r}")
    return node


@dataclass(frozen=True)
class LugipelConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[LugipelLayer, ...]
    max_positions: int
    eos_token_id: int
    raw: Mapping[str, Any]

    architecture = "Lugipel"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LugipelConfig":
        layers = _get(raw, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        parsed = []
        for i, layer in enumerate(layers):
            kind = layer.get("type") if isinstance(layer, Mapping) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not supported; have {list(MIXER_TYPES)}")
            if not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"config.json: layers[{i}] lacks its mixer's sizes")
            mlp = layer.get("mlp")
            if mlp is not None and (not isinstance(mlp, Mapping) or mlp.get("kind") not in MLP_KINDS):
                got = mlp.get("kind") if isinstance(mlp, Mapping) else mlp
                raise ConfigError(f"config.json: layers[{i}].mlp.kind {got!r} is not supported; have {list(MLP_KINDS)}")
            parsed.append(LugipelLayer(kind, layer["mixer"], mlp))
        eos = raw.get("eos_token_id")
        config = cls(vocab=_get(raw, "vocab", int), width=_get(raw, "width", int), norm_eps=_get(raw, "norm.eps", float),
                     embedding_scale=_get(raw, "embedding.scale", float), layers=tuple(parsed),
                     max_positions=int(raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
                     eos_token_id=-1 if eos is None else int(eos), raw=raw)
        for i in range(len(parsed)):                       # every size is looked at now, not at the first step
            config.mixer_spec(i), config.feed_forward_spec(i)
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)

    # ------------------------------------------------------------------ parts of layer i
    def mixer_spec(self, i: int) -> PartSpec:
        layer = self.layers[i]
        m, where = layer.mixer, f"layers[{i}].mixer"
        if layer.type == "mingru":
            return MinGRUSpec(hidden_size=self.width, width=_get(m, "width", int), bias=True)
        heads, kv_heads = _get(m, "heads", int), _get(m, "kv_heads", int)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads={heads} is not a multiple of kv_heads={kv_heads}")
        # a mixer without `q_temp` (or `mask`) has no query temperature (no window: every earlier key is seen)
        coef, every = (_get(m, "q_temp.coef", float), _get(m, "q_temp.every", int)) if m.get("q_temp") is not None else (0.0, 0)
        window = _get(m, "mask.size", int) if m.get("mask") is not None else 0
        return GatedAttentionSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=_get(m, "dim", int),
                                  value_dim=_get(m, "vdim", int), scale=_get(m, "scale", float),
                                  window=window, bias=False, qk_norm=True, qk_norm_eps=self.norm_eps,
                                  qk_norm_scope="head", q_temperature_coef=coef, q_temperature_every=every,
                                  distance_slope_exponent=SLOPE_EXPONENT, head_bias=True, weights="sigmoid",
                                  output_gate=True, output_gate_scope="head", position=None)

    def feed_forward_spec(self, i: int) -> PartSpec | None:
        f = self.layers[i].mlp
        where = f"layers[{i}].mlp"
        if f is None:
            return None
        if f["kind"] == "dense":
            return PlainMLPSpec(hidden_size=self.width, intermediate_size=_get(f, "ff", int), activation="xielu",
                                tensor_names=("up", "down"), param_name="act")
        experts, top = _get(f, "router.experts", int), _get(f, "router.top", int)
        identity = _count(f, "router.identity", 0)
        groups, keep = 1, 1
        if isinstance(f.get("router"), Mapping) and f["router"].get("groups") is not None:
            groups, keep = _get(f, "router.groups.count", int), _get(f, "router.groups.keep", int)
        total = experts + identity
        if total % groups:
            raise ConfigError(f"config.json: {where}.router: {total} router outputs do not form {groups} equal groups")
        if keep > groups:
            raise ConfigError(f"config.json: {where}.router.groups.keep={keep} exceeds count={groups}")
        if top > keep * (total // groups):
            raise ConfigError(f"config.json: {where}.router.top={top} exceeds the {keep * (total // groups)} experts of "
                              f"{keep} groups")
        expert = GatedMLPSpec(hidden_size=self.width, intermediate_size=_get(f, "expert.ff", int), activation="silu",
                              tensor_names=("gate", "up", "down"))
        scale = float(f["router"]["scale"]) if "scale" in f["router"] else 1.0
        return RoutedExpertsSpec(hidden_size=self.width, num_experts=experts, top=top, expert=expert, shared=None,
                                 router_bias_name=None, scoring="softmax_all", weight_on="output",
                                 correction_name="correction", group_count=groups, group_keep=keep, weight_scale=scale,
                                 share_eps=SHARE_EPS, identity_experts=identity)


def lugipel_model_spec(config: LugipelConfig) -> ModelSpec:
    """One block per entry of `layers`, each run once in order with a cache entry of its own."""
    norm = StreamRMSNormSpec(size=config.width, eps=config.norm_eps, weight_offset=0.0, weight_name="")
    blocks = []
    for i in range(len(config.layers)):
        feed_forward = config.feed_forward_spec(i)
        blocks.append(BlockSpec(
            arrangement="pre_norm_stream",
            mixer=config.mixer_spec(i),
            feed_forward=feed_forward,
            mixer_norm=norm,
            feed_forward_norm=norm if feed_forward is not None else None,
            prefix=f"l{i}.",
            mixer_prefix="mix.",
            feed_forward_prefix="mlp.",
            mixer_norm_prefix="norm1",
            feed_forward_norm_prefix="norm2",
        ))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        blocks=tuple(blocks),
        run=tuple(RunEntry(block=i, cache_entry=i) for i in range(len(blocks))),
        final_norm=norm,
        embedding_name="embed",
        final_norm_prefix="final.norm",
        lm_head_name="head",
        max_positions=config.max_positions,
        eos_token_id=config.eos_token_id,
        embedding_scale=config.embedding_scale,
        embedding_position=SinusoidSpec(size=config.width, base=SINUSOID_BASE),
        # a layer without a feed-forward has no use for a second norm; a checkpoint may carry one all the same
        optional_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(config.layers) if layer.mlp is None),
    )
