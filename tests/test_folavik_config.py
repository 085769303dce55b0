"""
The Folavik configuration on the host: what it reads, what it refuses, which tensors the model declares;
the cache layout its mixers ask for; the rescaled rotation frequencies against the plain implementation.
"""

import copy
import math

import pytest
import torch

import folavik_configs as C
import plain_folavik as plain
from tinyserve_llm_b200.config import ConfigError
from tinyserve_llm_b200.config.folavik import FolavikConfig, folavik_model_spec
from tinyserve_llm_b200.config.registry import resolve_architecture
from tinyserve_llm_b200.parts.model import declared_tensors


def test_registry_finds_the_design_by_its_architecture_key():
    arch = resolve_architecture(C.MIXED)
    assert arch.name == "Folavik" and isinstance(arch.parse(C.MIXED), FolavikConfig)


def test_every_size_and_constant_comes_from_the_configuration():
    spec = folavik_model_spec(FolavikConfig.from_dict(C.MIXED))
    assert spec.vocab_size == 300 and spec.hidden_size == 96 and spec.lm_head_name == "head"
    assert (spec.logit_scale, spec.logit_softcap) == (1.7, 9.0)
    assert spec.embedding_norm is not None and spec.embedding_norm_prefix == "embed.norm" and spec.embedding_norm.eps == 1e-5
    a = spec.blocks[0].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.chunk, a.window, a.scale) == (6, 2, 20, 36, 11, 0, 0.25)
    assert not a.bias and not a.qk_norm and not a.output_gate and a.softcap == 0
    assert (a.position.dims, a.position.base, a.position.yarn) == (12, 5000.0, None)
    assert (a.position.bands.factor, a.position.bands.low_freq_factor, a.position.bands.high_freq_factor) == (4.0, 2.0, 8.0)
    b = spec.blocks[1].mixer
    assert (b.num_heads, b.head_dim, b.value_dim, b.kv_rank, b.q_rank, b.rot_dim, b.window) == (5, 24, 20, 40, 0, 0, 0)
    assert b.output_gate and b.position is None and b.norm_eps == 1e-5
    d = spec.blocks[2].mixer
    assert (d.num_heads, d.num_kv_heads, d.head_dim, d.value_dim, d.window, d.chunk) == (4, 2, 16, 24, 37, 0)
    assert (d.softcap, d.difference, d.norm_eps, d.bias) == (12.0, 0.55, 1e-5, True)
    assert (d.position.yarn.factor, d.position.yarn.original, d.position.yarn.fast, d.position.yarn.slow) == (4.0, 64, 16.0, 2.0)
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].feed_forward_norm is None
    assert spec.blocks[0].feed_forward.activation == "gelu_tanh" and spec.blocks[0].feed_forward.intermediate_size == 136
    assert spec.blocks[3].mixer.position.bands is None and spec.blocks[4].mixer.position.yarn is None
    assert [e.cache_entry for e in spec.run] == [0, 1, 2, 3, 4, 5]
    edges = folavik_model_spec(FolavikConfig.from_dict(C.EDGES))
    assert (edges.logit_scale, edges.logit_softcap) == (1.0, 0.0)


def test_declared_tensors_follow_the_layers():
    names = declared_tensors(folavik_model_spec(FolavikConfig.from_dict(C.MIXED)))
    assert names["embed"].shape == (300, 96) and names["head"].shape == (300, 96)
    assert names["embed.norm"].shape == (96,) and names["final.norm"].shape == (96,)
    assert names["l0.mix.q"].shape == (120, 96) and names["l0.mix.k"].shape == (40, 96) and names["l0.mix.v"].shape == (72, 96)
    assert names["l0.mix.o"].shape == (96, 216) and "l0.mix.q.b" not in names and "l0.mix.g" not in names
    assert names["l0.mlp.gate"].shape == (136, 96) and names["l0.mlp.down"].shape == (96, 136)
    assert names["l1.mix.q"].shape == (120, 96) and names["l1.mix.dkv"].shape == (40, 96) and names["l1.mix.dkv.norm"].shape == (40,)
    assert names["l1.mix.uk"].shape == (120, 40) and names["l1.mix.uv"].shape == (100, 40)
    assert names["l1.mix.g"].shape == (100, 96) and names["l1.mix.o"].shape == (96, 100) and "l1.mix.dq" not in names
    assert names["l2.mix.q"].shape == (128, 96) and names["l2.mix.q.b"].shape == (128,)
    assert names["l2.mix.k"].shape == (64, 96) and names["l2.mix.k.b"].shape == (64,)
    assert names["l2.mix.v"].shape == (48, 96) and names["l2.mix.v.b"].shape == (48,) and names["l2.mix.o"].shape == (96, 96)
    assert all(names[f"l2.mix.{n}"].shape == (16,) for n in ("lq1", "lk1", "lq2", "lk2"))
    assert "l2.norm1" in names and "l2.norm2" not in names and not any(n.startswith("l2.mlp.") for n in names)


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=22), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][2]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_a_bad_configuration_is_refused_by_the_name_of_its_key(edit, word):
    raw = copy.deepcopy(C.MIXED)
    edit(raw)
    with pytest.raises(ConfigError) as err:
        FolavikConfig.from_dict(raw)
    assert word in str(err.value)


def test_a_differential_layer_asks_for_twice_the_key_heads_and_its_own_value_heads():
    """The cache layout: chunks and windows bound what is kept; the two maps' keys are heads of their own over one set of values."""
    from tinyserve_llm_b200.cache.manager import plan_layout
    from tinyserve_llm_b200.parts.base import KVNeed
    needs = [(KVNeed(4, 20, 11, True, 36), 0), (KVNeed(1, 40, 0, values=False), 0), (KVNeed(4, 16, 37, True, 24, 2), 0),
             (KVNeed(4, 16, 37, True, 24, 2), 0), (KVNeed(4, 16, 37, True, 24), 0)]
    layout = plan_layout(needs, 16)
    assert [g.entries for g in layout.groups] == [(0,), (1,), (2, 3), (4,)]
    assert [(g.num_kv_heads, g.num_value_heads, g.head_dim, g.value_head_dim, g.window) for g in layout.groups] == \
        [(4, 4, 20, 36, 11), (1, 1, 40, 40, 0), (4, 2, 16, 24, 37), (4, 4, 16, 24, 37)]
    assert not layout.prefix_reuse_possible


def test_maps_are_grouped_by_key_head():
    """Rows [head][map][dim] go to [kv head][map][head of the group][dim]: the query heads of one key head lie side by side."""
    from tinyserve_llm_b200.parts.differential_attention import group_maps_together
    heads, kv_heads, dim = 6, 2, 3
    rows = torch.arange(heads * 2 * dim * 5).reshape(heads * 2 * dim, 5)
    out = group_maps_together(rows, heads, kv_heads, dim)
    for g in range(kv_heads):
        for m in range(2):
            for i in range(heads // kv_heads):
                h = g * (heads // kv_heads) + i
                src = rows[(h * 2 + m) * dim:(h * 2 + m + 1) * dim]
                at = ((g * 2 + m) * (heads // kv_heads) + i) * dim
                assert torch.equal(out[at:at + dim], src)
    assert torch.equal(group_maps_together(rows[:, 0].contiguous(), heads, kv_heads, dim), out[:, 0])


@pytest.mark.parametrize("dims, base, bands", [(64, 400000.0, (6.0, 1.0, 5.0, 384)), (16, 10000.0, (4.0, 2.0, 8.0, 64)),
                                               (12, 5000.0, (4.0, 2.0, 8.0, 64)), (8, 50.0, (5.0, 1.0, 3.0, 32))])
def test_frequencies_rescaled_by_wavelength_bands(dims, base, bands):
    """Kept, slowed and blended frequencies all occur in the first case; the engine's table equals the plain one's."""
    from tinyserve_llm_b200.config.spec import Llama3Scaling
    from tinyserve_llm_b200.parts.rotary import band_scaled_frequencies
    sc = dict(zip(("factor", "low", "high", "original"), bands))
    want = torch.tensor(plain.band_scaled_frequencies(dims, base, sc), dtype=torch.float64)
    got = band_scaled_frequencies(dims, base, Llama3Scaling(bands[0], bands[1], bands[2], bands[3]))
    torch.testing.assert_close(got, want, rtol=1e-13, atol=0)
    bare = torch.tensor(plain.plain_frequencies(dims, base), dtype=torch.float64)
    if dims == 64:
        kept, slowed = got == bare, torch.isclose(got, bare / bands[0], rtol=1e-12)
        assert kept.any() and slowed.any() and (~kept & ~slowed).any()


def test_yarn_frequencies_and_magnitude():
    from tinyserve_llm_b200.config.spec import YarnScaling
    from tinyserve_llm_b200.parts.rotary import yarn_frequencies
    for dims, base, yarn in ((8, 150000.0, (3.0, 256, 24.0, 1.5)), (40, 20000.0, (2.0, 32, 8.0, 1.0)), (6, 900.0, (4.0, 64, 16.0, 2.0))):
        sc = dict(zip(("factor", "original", "fast", "slow"), yarn))
        want, magnitude = plain.yarn_frequencies(dims, base, sc)
        got = yarn_frequencies(dims, base, YarnScaling(*yarn))
        torch.testing.assert_close(got, torch.tensor(want, dtype=torch.float64), rtol=1e-13, atol=0)
        assert magnitude == 0.1 * math.log(yarn[0]) + 1.0


def test_plain_masks():
    """The plain model's own masks, by hand: a chunk's first token sees itself only; a window of n sees n keys."""
    pos = torch.arange(7)
    c = plain.chunk_mask(pos, 3)
    assert c[3].tolist() == [False, False, False, True, False, False, False] and c[5].tolist() == [False] * 3 + [True] * 3 + [False]
    w = plain.window_mask(pos, 3)
    assert w[5].tolist() == [False, False, False, True, True, True, False] and w[1].tolist() == [True, True] + [False] * 5
