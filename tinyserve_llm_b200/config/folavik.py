"""
Typed configuration of the Folavik decoder, read from the keys of its own config.json, and the
`ModelSpec` it turns into.

config.json: `architecture` "Folavik", `vocab`, `width`, `norm.eps`, `logit_scale`, `logit_softcap` and
`layers`, a list whose entries give `type` (the mixer: "latent_attention", "attention" or "attention_2"),
`mixer` (its sizes and constants) and `mlp` (`kind` "dense" with `ff`, or null for a layer without a
feed-forward).  Mixers:

* "latent_attention": `heads`, `dim`, `vdim`, `kv_rank`, `scale`.  Softmax attention over every earlier
  key; keys and values are up-projections of one normed latent a token; no positions.
* "attention": `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `mask.size` (chunks), `rot` with `dims`, `base`
  and `scaling` of `factor`, `low`, `high`, `original` (frequencies rescaled by wavelength bands).
* "attention_2": `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `softcap`, `diff`, `mask.size` (sliding window),
  `rot` with `dims`, `base` and `scaling` of `factor`, `original`, `fast`, `slow` (YaRN).  Two score maps a head.

Layers may come in any order and number; every size is read here and nowhere else.  Tensors: `embed`,
`embed.norm`, `final.norm`, `head`, and per layer `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`.

What the design fixes stands here as constants: layer norms with a weight and no bias (before each
sublayer, on the embedding rows and before the output head) around a float32 residual stream; the latent
attention has no query latent, no rotated part and a sigmoid gate on its concatenated heads; the
differential attention has biases on q, k and v and a weightless norm a head with the layer's eps; the
dense feed-forward is gated by the tanh form of gelu; the logits are scaled, then capped by tanh.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from tinyserve_llm_b200.config.duduvik import DEFAULT_MAX_POSITIONS, _get
from tinyserve_llm_b200.config.llama import ConfigError
from tinyserve_llm_b200.config.spec import (
    BlockSpec,
    DifferentialAttentionSpec,
    GatedAttentionSpec,
    GatedMLPSpec,
    InlineRotarySpec,
    LatentAttentionSpec,
    Llama3Scaling,
    ModelSpec,
    PartSpec,
    RunEntry,
    StreamLayerNormSpec,
    YarnScaling,
)

MIXER_TYPES = ("latent_attention", "attention", "attention_2")


@dataclass(frozen=True)
class FolavikLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None


@dataclass(frozen=True)
class FolavikConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    logit_softcap: float
    layers: tuple[FolavikLayer, ...]
    max_positions: int
    eos_token_id: int
    raw: Mapping[str, Any]

    architecture = "Folavik"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FolavikConfig":
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
            if mlp is not None and mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp.get('kind')!r} is not supported; have ['dense']")
            parsed.append(FolavikLayer(kind, layer["mixer"], mlp))
        eos = raw.get("eos_token_id")
        cap = raw.get("logit_softcap")
        config = cls(vocab=_get(raw, "vocab", int), width=_get(raw, "width", int), norm_eps=_get(raw, "norm.eps", float),
                     logit_scale=float(raw["logit_scale"]) if raw.get("logit_scale") is not None else 1.0,
                     logit_softcap=float(cap) if cap else 0.0,
                     layers=tuple(parsed), max_positions=int(raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
                     eos_token_id=-1 if eos is None else int(eos), raw=raw)
        if config.logit_softcap < 0:
            raise ConfigError(f"config.json: logit_softcap must not be negative, got {config.logit_softcap}")
        for i in range(len(parsed)):                       # every size is looked at now, not at the first step
            config.mixer_spec(i), config.feed_forward_spec(i)
        return config

    def to_dict(self) -> dict[str, Any]:
        return dict(self.raw)

    # ------------------------------------------------------------------ parts of layer i
    @staticmethod
    def _heads(where: str, m: Mapping[str, Any]) -> tuple[int, int]:
        heads, kv_heads = _get(m, "heads", int), _get(m, "kv_heads", int)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads={heads} is not a multiple of kv_heads={kv_heads}")
        return heads, kv_heads

    @staticmethod
    def _mask(where: str, m: Mapping[str, Any]) -> int:
        """`mask.size`, or 0 where the mixer has no mask."""
        if m.get("mask") is None:
            return 0
        return _get(m, "mask.size", int)

    @staticmethod
    def _rotation(where: str, m: Mapping[str, Any], dim: int, yarn: bool) -> InlineRotarySpec | None:
        rot = m.get("rot")
        if rot is None or not rot.get("dims"):
            return None
        dims, base = _get(rot, "dims", int), _get(rot, "base", float)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims={dims} must be even and at most dim={dim}")
        if base <= 1:
            raise ConfigError(f"config.json: {where}.rot.base must be above 1, got {base}")
        sc = rot.get("scaling")
        if not sc:
            return InlineRotarySpec(dims=dims, base=base)
        factor, original = _get(sc, "factor", float), _get(sc, "original", float)
        if factor <= 0 or original <= 0:
            raise ConfigError(f"config.json: {where}.rot.scaling needs a positive factor and original")
        if yarn:
            fast, slow = _get(sc, "fast", float), _get(sc, "slow", float)
            if fast <= 0 or slow <= 0:
                raise ConfigError(f"config.json: {where}.rot.scaling needs positive fast and slow")
            return InlineRotarySpec(dims=dims, base=base, yarn=YarnScaling(factor=factor, original=original, fast=fast, slow=slow))
        low, high = _get(sc, "low", float), _get(sc, "high", float)
        if low <= 0 or high <= low:
            raise ConfigError(f"config.json: {where}.rot.scaling needs 0 < low < high, got {low} and {high}")
        return InlineRotarySpec(dims=dims, base=base, bands=Llama3Scaling(
            factor=factor, low_freq_factor=low, high_freq_factor=high, original_max_position_embeddings=original))

    def mixer_spec(self, i: int) -> PartSpec:
        layer = self.layers[i]
        m, where = layer.mixer, f"layers[{i}].mixer"
        dim, vdim, scale = _get(m, "dim", int), _get(m, "vdim", int), _get(m, "scale", float)
        if layer.type == "latent_attention":
            return LatentAttentionSpec(hidden_size=self.width, num_heads=_get(m, "heads", int), head_dim=dim, rot_dim=0,
                                       value_dim=vdim, q_rank=0, kv_rank=_get(m, "kv_rank", int), scale=scale, window=0,
                                       norm_eps=self.norm_eps, position=None, output_gate=True)
        heads, kv_heads = self._heads(where, m)
        if layer.type == "attention":
            return GatedAttentionSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                                      value_dim=vdim, scale=scale, chunk=self._mask(where, m),
                                      position=self._rotation(where, m, dim, yarn=False))
        softcap = float(m["softcap"]) if m.get("softcap") else 0.0
        if softcap < 0:
            raise ConfigError(f"config.json: {where}.softcap must not be negative, got {softcap}")
        return DifferentialAttentionSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                                         value_dim=vdim, scale=scale, window=self._mask(where, m), softcap=softcap,
                                         difference=_get(m, "diff", float), norm_eps=self.norm_eps, bias=True,
                                         position=self._rotation(where, m, dim, yarn=True))

    def feed_forward_spec(self, i: int) -> PartSpec | None:
        f = self.layers[i].mlp
        if f is None:
            return None
        return GatedMLPSpec(hidden_size=self.width, intermediate_size=_get(f, "ff", int), activation="gelu_tanh",
                            tensor_names=("gate", "up", "down"))


def folavik_model_spec(config: FolavikConfig) -> ModelSpec:
    """One block per entry of `layers`, each run once in order with a cache entry of its own."""
    norm = StreamLayerNormSpec(size=config.width, eps=config.norm_eps, weight_name="")
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
        embedding_norm=norm,
        embedding_norm_prefix="embed.norm",
        logit_scale=config.logit_scale,
        logit_softcap=config.logit_softcap,
        # a layer without a feed-forward has no use for its second norm; a checkpoint may carry the weight all the same
        optional_tensors=tuple(f"l{i}.norm2" for i, layer in enumerate(config.layers) if layer.mlp is None),
    )
