"""The Lugipel configuration on the host: what it reads, what it refuses, which tensors the model declares."""

import copy

import pytest

import lugipel_configs as C
from tinyserve_llm_b200.config import ConfigError
from tinyserve_llm_b200.config.lugipel import LugipelConfig, lugipel_model_spec
from tinyserve_llm_b200.config.registry import resolve_architecture
from tinyserve_llm_b200.parts.model import declared_tensors


def test_registry_finds_the_design_by_its_architecture_key():
    arch = resolve_architecture(C.MIXED)
    assert arch.name == "Lugipel" and isinstance(arch.parse(C.MIXED), LugipelConfig)


def test_every_size_and_constant_comes_from_the_configuration():
    spec = lugipel_model_spec(LugipelConfig.from_dict(C.MIXED))
    assert spec.vocab_size == 300 and spec.hidden_size == 96 and spec.embedding_scale == 2.5
    assert spec.embedding_position.size == 96 and spec.lm_head_name == "head"
    first = spec.blocks[0]
    a = first.mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.window) == (6, 2, 20, 36, 11)
    assert (a.scale, a.q_temperature_coef, a.q_temperature_every) == (0.25, 0.4, 5)
    assert a.weights == "sigmoid" and a.qk_norm_scope == "head" and a.output_gate_scope == "head" and a.head_bias
    f = first.feed_forward
    assert (f.num_experts, f.identity_experts, f.top, f.group_count, f.group_keep, f.weight_scale) == (7, 2, 2, 3, 2, 1.5)
    assert f.expert.intermediate_size == 40 and f.scoring == "softmax_all" and f.correction_name == "correction"
    assert spec.blocks[1].mixer.width == 72 and spec.blocks[1].feed_forward.intermediate_size == 136
    assert spec.blocks[1].feed_forward.activation == "xielu"
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].feed_forward_norm is None
    assert [e.cache_entry for e in spec.run] == [0, 1, 2, 3, 4]


def test_declared_tensors_follow_the_layers():
    names = declared_tensors(lugipel_model_spec(LugipelConfig.from_dict(C.MIXED)))
    assert names["embed"].shape == (300, 96) and names["head"].shape == (300, 96) and names["final.norm"].shape == (96,)
    assert names["l0.mix.q"].shape == (120, 96) and names["l0.mix.k"].shape == (40, 96) and names["l0.mix.v"].shape == (72, 96)
    assert names["l0.mix.q.norm"].shape == (20,) and names["l0.mix.k.norm"].shape == (20,)
    assert names["l0.mix.pb"].shape == (6,) and names["l0.mix.g"].shape == (6, 96) and names["l0.mix.o"].shape == (96, 216)
    assert names["l0.mlp.router"].shape == (9, 96) and names["l0.mlp.correction"].shape == (9,)
    assert names["l0.mlp.e6.gate"].shape == (40, 96) and names["l0.mlp.e6.down"].shape == (96, 40) and "l0.mlp.e7.gate" not in names
    assert names["l1.mix.z"].shape == (72, 96) and names["l1.mix.z.b"].shape == (72,) and names["l1.mix.x.b"].shape == (72,)
    assert names["l1.mix.g"].shape == (72, 96) and names["l1.mix.o"].shape == (96, 72)
    assert names["l1.mlp.up"].shape == (136, 96) and names["l1.mlp.down"].shape == (96, 136) and names["l1.mlp.act"].shape == (2,)
    assert "l2.norm1" in names and "l2.norm2" not in names and not any(n.startswith("l2.mlp.") for n in names)
    assert names["l3.mlp.router"].shape == (5, 96)


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "q_temp.every"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=2), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "keep"),
    (lambda c: c["layers"][4]["mlp"]["router"].update(top=4), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(identity=-1), "identity"),
    (lambda c: c.pop("embedding"), "embedding.scale"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_what_cannot_be_served_is_refused_with_the_key(edit, word):
    raw = copy.deepcopy(C.MIXED)
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        LugipelConfig.from_dict(raw)


def test_a_mixer_without_window_or_temperature_has_neither():
    raw = copy.deepcopy(C.MIXED)
    raw["layers"][0]["mixer"].pop("mask")
    raw["layers"][0]["mixer"].pop("q_temp")
    a = lugipel_model_spec(LugipelConfig.from_dict(raw)).blocks[0].mixer
    assert a.window == 0 and a.q_temperature_every == 0


def test_whole_numbers_serve_as_constants():
    raw = copy.deepcopy(C.MIXED)
    raw["layers"][0]["mixer"].update(scale=1)
    raw["layers"][0]["mixer"]["q_temp"].update(coef=0)
    raw["embedding"].update(scale=2)
    spec = lugipel_model_spec(LugipelConfig.from_dict(raw))
    assert spec.embedding_scale == 2.0 and spec.blocks[0].mixer.scale == 1.0 and spec.blocks[0].mixer.q_temperature_coef == 0.0


@pytest.mark.parametrize("raw", [C.MIXED, C.RECURRENT, C.WINDOWS, C.WIDE])
def test_all_test_configurations_parse(raw):
    spec = lugipel_model_spec(LugipelConfig.from_dict(raw))
    assert len(spec.blocks) == len(raw["layers"]) and len(declared_tensors(spec)) > 10
