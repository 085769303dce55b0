"""
The Folavik decoder in the engine against the plain implementation of tests/plain_folavik.py: each
mechanism alone (with weights or inputs made so that a fault shows), whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal requests in one batch against each
alone, pages that are freed and taken again, keys far away, at page borders and just inside and just
outside every window and chunk, the first tokens, long decoding, several sizes (the tensor-core kernels'
among them), steps replayed from CUDA graphs, the replay program and greedy generation through the
engine's entry point.
"""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import folavik_configs as C
import plain_folavik as plain
from test_nipizen import TOL, Engine, _ctx, _in_steps, _mixer, _runtime, _Slots, ids_of, read_tensors, rows_close

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CONFIGS = {"mixed": C.MIXED, "edges": C.EDGES, "latent": C.LATENT, "wide": C.WIDE, "grouped": C.GROUPED}
SEEDS = {"mixed": 611, "edges": 622, "latent": 633, "wide": 644, "grouped": 655}
PAGE = {"mixed": 16, "edges": 16, "latent": 16, "wide": 64, "grouped": 64}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from tinyserve_llm_b200.weights import write_random_model
    out = {}
    for name, raw in CONFIGS.items():
        folder = str(tmp_path_factory.mktemp(f"folavik_{name}"))
        write_random_model(folder, raw, SEEDS[name], **C.WEIGHTS)
        out[name] = folder
    return out


_PLAIN = {}


def plain_logits(folder, ids):
    key = (folder, tuple(ids))
    if key not in _PLAIN:
        with open(os.path.join(folder, "config.json")) as f:
            raw = json.load(f)
        _PLAIN[key] = plain.forward(raw, read_tensors(folder), ids)
    return _PLAIN[key]


def close(got, want, dtype):
    """float32: every position to rounding.  bfloat16: the error's root mean square against the logits' own spread."""
    if dtype == "float32":
        torch.testing.assert_close(got, want, atol=3e-4, rtol=1e-4)
    else:
        err = (got - want).pow(2).mean(-1).sqrt() / want.std()
        assert float(err.max()) < 0.2 and float(err.median()) < 0.05, \
            f"relative error: worst {float(err.max()):.3f} at {int(err.argmax())}, median {float(err.median()):.3f}"


# ---------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_equals_the_plain_model(folders, name, dtype):
    ids = ids_of(CONFIGS[name]["vocab"], 300 if PAGE[name] == 64 else 150, 1)
    got = Engine(folders[name], dtype, page=PAGE[name]).run("a", ids, [len(ids)])
    close(got, plain_logits(folders[name], ids), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prompt_then_token_by_token_and_portions_of_many_sizes(folders, name, dtype):
    """The same logits whether the tokens come at once, one by one after a head, or in portions down to two tokens."""
    n = 230 if PAGE[name] == 64 else 150
    ids = ids_of(CONFIGS[name]["vocab"], n, 2)
    want = plain_logits(folders[name], ids)
    page = PAGE[name]
    decoded = Engine(folders[name], dtype, page=page).run("a", ids, [30] + [1] * (n - 30))     # windows and chunks pass over decoded tokens
    close(decoded, want, dtype)
    portions = Engine(folders[name], dtype, page=page).run("a", ids, [2, 3, 17, 2, 16, 5, 31, 1, 1, 2, 64, 3])
    close(portions, want, dtype)
    one_by_one = Engine(folders[name], dtype, page=page).run("a", ids[:40], [1])                # the first tokens, alone
    close(one_by_one, want[:40], dtype)
    if dtype == "float32":                                                                      # the cut changes nothing beyond rounding
        torch.testing.assert_close(decoded, portions, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_unequal_requests_in_one_batch_and_reused_pages(folders, name, dtype, graphs):
    """
    Five requests through a pool that holds less than their sum: portions of some beside single tokens of
    others, requests that sit a step out, ended requests whose pages the next ones take (a page read through
    a stale table, or keys of the request before, show).  Each request's logits equal those of the request
    alone.  With `graphs`, every step is replayed from a CUDA graph from its first sighting on.
    """
    vocab, page = CONFIGS[name]["vocab"], PAGE[name]
    k = page // 16
    sizes = (("a", 70 * k), ("b", 33 * k), ("c", 9), ("d", 58 * k), ("e", 41 * k))
    reqs = {key: ids_of(vocab, n, 10 + i) for i, (key, n) in enumerate(sizes)}
    a, b, c, d, e = (reqs[x] for x in "abcde")
    eng = Engine(folders[name], dtype, page=page, pages=12, slots=3, cuda_graphs=graphs)
    eng.step([("a", a[:40 * k]), ("b", b[:2])])
    eng.step([("a", a[40 * k:40 * k + 1]), ("b", b[2:19 * k]), ("c", c[:9])], end=["c"])
    eng.step([("b", b[19 * k:19 * k + 1])])                                          # a sits this one out
    eng.step([("d", d[:3]), ("a", a[40 * k + 1:]), ("b", b[19 * k + 1:])], end=["a", "b"])
    eng.step([("d", d[3:35 * k]), ("e", e[:1])])
    eng.step([("e", e[1:2]), ("d", d[35 * k:35 * k + 1])])
    at_d, at_e = 35 * k + 1, 2
    while at_d < len(d):
        both = [("d", d[at_d:at_d + 1])]
        if at_e < 24 * k:
            both.append(("e", e[at_e:at_e + 1]))
            at_e += 1
        at_d += 1
        eng.step(both, end=["d"] if at_d == len(d) else [])
    eng.step([("e", e[at_e:])], end=["e"])
    assert eng.manager.stats().pages_in_use == 0
    if graphs:
        assert eng.runner.graph_replays > 20
    for key in "abcde":
        close(eng.logits(key), plain_logits(folders[name], reqs[key]), dtype)


def test_long_decoding_across_several_windows_and_chunks(folders):
    """260 tokens one by one after a short head, over several pages, windows and chunks."""
    name, dtype = "mixed", "float32"
    ids = ids_of(CONFIGS[name]["vocab"], 260, 3)
    got = Engine(folders[name], dtype, page=16, pages=18).run("a", ids, [7] + [1] * 253)
    close(got, plain_logits(folders[name], ids), dtype)


def test_tensor_core_sizes_also_from_graphs_token_by_token(folders):
    """Heads of 64 and 128 channels in bfloat16: 200 tokens decoded one by one from CUDA graphs behind a prompt of 100."""
    for name in ("wide", "grouped"):
        ids = ids_of(CONFIGS[name]["vocab"], 300, 4)
        eng = Engine(folders[name], "bfloat16", page=64, cuda_graphs=True)
        calls = eng.model.rt.ops.calls               # one kernel library a process: counts since this model began
        before = dict(calls)
        got = eng.run("a", ids, [100] + [1] * 200)
        close(got, plain_logits(folders[name], ids), "bfloat16")
        assert eng.runner.graph_replays > 150
        assert calls.get("ts_paged_attention_bf16_masked", 0) > before.get("ts_paged_attention_bf16_masked", 0)
        assert calls.get("ts_prefill_attention_tcgen05_masked", 0) > before.get("ts_prefill_attention_tcgen05_masked", 0)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_layer_sizes_of_a_real_model(tmp_path, dtype):
    """
    Three layers at a width of 1,024 with heads of 128 channels, a latent of 512 and masks of 1,024 tokens: a prompt
    of 2,048 tokens in one step (sixteen query tiles; windows and chunks that begin many key tiles in; in bfloat16
    the latent layer on keys and values worked out for the step and the gate in the tcgen05 product's epilogue),
    a portion of 20 over the cached prefix, then 32 single tokens from CUDA graphs.
    """
    from tinyserve_llm_b200.weights import write_random_model
    folder = str(tmp_path / "real")
    write_random_model(folder, C.REAL, 77, **C.REAL_WEIGHTS)
    ids = ids_of(C.REAL["vocab"], 2100, 8)
    want = plain.forward(C.REAL, read_tensors(folder), ids)
    eng = Engine(folder, dtype, page=64, pages=40, cuda_graphs=True)
    calls = eng.model.rt.ops.calls                   # one kernel library a process: counts since this test began
    before = dict(calls)
    got = eng.run("a", ids, [2048, 20] + [1] * 32)
    if dtype == "float32":
        torch.testing.assert_close(got, want, atol=2e-3, rtol=1e-3)
        return
    close(got, want, dtype)
    since = {k: calls.get(k, 0) - before.get(k, 0) for k in calls}
    assert since.get("ts_prefill_attention_tcgen05_dense", 0) == 1 and since.get("ts_prefill_attention_tcgen05_masked", 0) >= 4
    assert since.get("ts_gemm_tcgen05_gated", 0) >= 3 and eng.runner.graph_replays >= 30


# ---------------------------------------------------------------------------------------------- mechanisms alone
def _rot(dims, base, yarn=None, bands=None):
    from tinyserve_llm_b200.config.spec import InlineRotarySpec, Llama3Scaling, YarnScaling
    if not dims:
        return None, None
    spec = InlineRotarySpec(dims=dims, base=base, yarn=YarnScaling(*yarn) if yarn else None,
                            bands=Llama3Scaling(*bands) if bands else None)
    raw = {"dims": dims, "base": base}
    if yarn:
        raw["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    if bands:
        raw["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    return spec, raw


CUTS = [[(0, 17), (0, 2)], [(17, 33), (2, 19)], [(33, 34), (19, 20)], [(34, 110), (20, 21)], *[[(110 + i, 111 + i), (21 + i, 22 + i)] for i in range(20)]]
LENS = [130, 41]


def _compare_in_steps(mixer, w, dtype, width, want_of, page=16, lens=LENS, cuts=CUTS, seed=1):
    g = torch.Generator().manual_seed(seed)
    x_of = [torch.randn(n, width, generator=g).to(dtype) for n in lens]
    got = _in_steps(_Slots(mixer, dtype, lens, page=page), x_of, cuts)
    for a, x in zip(got, x_of):
        rows_close(a, want_of(x.double()), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, dim, vdim, rank, page", [(5, 24, 20, 40, 16), (1, 16, 16, 8, 16), (4, 32, 48, 64, 64), (3, 8, 72, 96, 16), (3, 12, 10, 20, 16),
                                                          (16, 64, 64, 128, 64), (2, 48, 56, 24, 16)])
def test_latent_attention_without_positions(dtype, heads, dim, vdim, rank, page):
    """
    Keys and values from one normed latent a token, queries straight from the input, a sigmoid gate on the heads:
    latents the tensor-core kernel takes (multiples of 32) and others, one head and sixteen; two requests of
    unequal length in portions that end inside pages, then token by token.
    """
    from tinyserve_llm_b200.config.spec import LatentAttentionSpec
    width = 64
    spec = LatentAttentionSpec(hidden_size=width, num_heads=heads, head_dim=dim, rot_dim=0, value_dim=vdim, q_rank=0, kv_rank=rank,
                               scale=0.3, norm_eps=1e-5, position=None, output_gate=True)
    mixer, w = _mixer(spec, dtype, 3)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": 0.3}
    _compare_in_steps(mixer, w, dtype, width, lambda x: plain.latent_attention(x, w, m, 1e-5), page=page)


@pytest.mark.parametrize("heads, dim, rank, page", [(4, 64, 96, 16), (2, 128, 40, 64), (5, 64, 512, 64)])
def test_latent_attention_of_long_portions_on_keys_and_values_worked_out_for_the_step(heads, dim, rank, page):
    """
    bfloat16, key and value heads of one size the tcgen05 prompt kernel takes: portions of 128 tokens and more attend
    over keys and values worked out from the gathered latents of the whole context (a cached prefix included),
    beside a request that feeds one token in the same step, which stays on the folded form; shorter steps before
    and after run the folded form alone.
    """
    from tinyserve_llm_b200.config.spec import LatentAttentionSpec
    dtype, width = torch.bfloat16, 64
    spec = LatentAttentionSpec(hidden_size=width, num_heads=heads, head_dim=dim, rot_dim=0, value_dim=dim, q_rank=0, kv_rank=rank,
                               scale=0.2, norm_eps=1e-5, position=None, output_gate=True)
    mixer, w = _mixer(spec, dtype, 11)
    m = {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": rank, "scale": 0.2}
    lens = [400, 150]
    cuts = [[(0, 200), (0, 3)], [(200, 201), (3, 140)], [(201, 400), (140, 150)]]
    calls = mixer.rt.ops.calls
    before = calls.get("ts_prefill_attention_tcgen05_dense", 0), calls.get("ts_latent_attention", 0)
    _compare_in_steps(mixer, w, dtype, width, lambda x: plain.latent_attention(x, w, m, 1e-5), page=page, lens=lens, cuts=cuts)
    assert calls.get("ts_prefill_attention_tcgen05_dense", 0) == before[0] + 3 and calls.get("ts_latent_attention", 0) == before[1] + 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, chunk, dims, bands, page", [
    (6, 2, 20, 36, 11, 12, (4.0, 2.0, 8.0, 64), 16), (3, 3, 16, 16, 16, 16, None, 16), (2, 1, 32, 64, 1, 8, None, 16),
    (4, 2, 64, 64, 96, 64, (6.0, 1.0, 3.0, 128), 64), (6, 2, 128, 128, 50, 32, None, 64), (4, 4, 64, 64, 1000, 16, None, 64),
    (2, 1, 64, 64, 64, 64, None, 64)])
def test_chunked_attention_alone(dtype, heads, kv_heads, dim, vdim, chunk, dims, bands, page):
    """
    Grouped-query attention inside chunks counted from the request's first token: chunks shorter than a page,
    of one page, of one token, longer than the requests, and ones that end inside the tensor-core kernels'
    tiles; rotation over a part of the head and over all of it, with and without rescaled frequencies.
    """
    from tinyserve_llm_b200.config.spec import GatedAttentionSpec
    width = 64
    position, rot = _rot(dims, 700.0, bands=bands)
    spec = GatedAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim, scale=0.3,
                              chunk=chunk, position=position)
    mixer, w = _mixer(spec, dtype, 4)
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.3, "mask": {"size": chunk}, "rot": rot}
    _compare_in_steps(mixer, w, dtype, width, lambda x: plain.chunked_attention(x, w, m, 1e-5), page=page)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, dims, yarn, cap, diff, page", [
    (4, 2, 16, 24, 37, 6, (4.0, 64, 16.0, 2.0), 12.0, 0.55, 16), (3, 1, 40, 8, 9, 40, None, 50.0, 0.8, 16),
    (5, 5, 12, 20, 1000, 4, (2.0, 32, 8.0, 1.0), 5.0, 0.3, 16), (1, 1, 24, 12, 1, 24, None, 30.0, 0.5, 16),
    (4, 2, 64, 64, 80, 32, (3.0, 128, 24.0, 1.5), 25.0, 0.45, 64), (3, 1, 128, 128, 70, 64, None, 20.0, 0.4, 64),
    (2, 2, 64, 64, 64, 8, None, 2.0, 0.2, 64), (8, 2, 64, 64, 129, 64, None, 0.0, 0.1, 64)])
def test_differential_attention_alone(dtype, heads, kv_heads, dim, vdim, window, dims, yarn, cap, diff, page):
    """
    Two score maps a head over the same values: biases, YaRN rotation of each map, capped scores (also a cap
    that bites, and none), a sliding window (shorter than a page, of one token, across pages, longer than the
    requests), the difference with the layer's weight, the weightless norm a head; as many key/value heads as
    heads, and one.
    """
    from tinyserve_llm_b200.config.spec import DifferentialAttentionSpec
    width = 64
    position, rot = _rot(dims, 900.0, yarn=yarn)
    spec = DifferentialAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim,
                                     scale=0.4, window=window, softcap=cap, difference=diff, norm_eps=1e-5, bias=True, position=position)

    def edit(t):                                    # a weight of the difference well away from `diff` alone
        t["lq1"], t["lk1"] = torch.full((dim,), 0.2), torch.full((dim,), 1.5 / dim)
        t["lq2"], t["lk2"] = torch.full((dim,), -0.3), torch.full((dim,), 2.0 / dim)

    mixer, w = _mixer(spec, dtype, 6, edit)
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.4, "mask": {"size": window}, "rot": rot,
         "diff": diff, "softcap": cap if cap else 1e9}
    assert abs(plain.difference_weight(w, diff) - (np.exp(0.3) - np.exp(-0.6) + diff)) < 0.02
    _compare_in_steps(mixer, w, dtype, width, lambda x: plain.differential_attention(x, w, m, 1e-5), page=page)


def _one_key_stands_out(t, q_rows, k_rows, width):
    """q and k read two input channels only: channel 0 asks, channel 1 answers; everything else of q and k is zero."""
    t["q"], t["k"] = torch.zeros_like(t["q"]), torch.zeros_like(t["k"])
    for r in q_rows:
        t["q"][r, 0] = 1.0
    for r in k_rows:
        t["k"][r, 1] = 1.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, page, far, size", [(16, 16, 63, 150), (64, 64, 127, 200), (64, 64, 70, 64)])
def test_a_key_at_a_windows_edge_is_seen_up_to_the_edge_and_no_further(dtype, dim, page, far, size):
    """
    One key (at a page's last slot, or inside a page) is made to dominate map 1 of head 0 of a differential layer
    with a window of `size`: queries up to far + size - 1 give it all their weight, the next one none; as a
    portion across the edge and token by token across it.  The first token sees itself.
    """
    from tinyserve_llm_b200.config.spec import DifferentialAttentionSpec
    width, heads, vdim = 32, 2, dim
    spec = DifferentialAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=1, head_dim=dim, value_dim=vdim, scale=1.0,
                                     window=size, softcap=40.0, difference=0.5, norm_eps=1e-5, bias=True, position=None)

    def edit(t):
        _one_key_stands_out(t, [0], [0], width)
        t["q.b"], t["k.b"] = torch.zeros_like(t["q.b"]), torch.zeros_like(t["k.b"])

    mixer, w = _mixer(spec, dtype, 5, edit)
    n = far + size + 40
    x = torch.randn(n, width, generator=torch.Generator().manual_seed(2)) * 0.3
    x[:, 0], x[:, 1] = 6.0, 0.0
    x[far, 1] = 6.0
    x = x.to(dtype)
    edge = far + size                                # the first query that no longer sees the key
    m = {"heads": heads, "kv_heads": 1, "dim": dim, "vdim": vdim, "scale": 1.0, "mask": {"size": size}, "diff": 0.5, "softcap": 40.0}
    want = plain.differential_attention(x.double(), w, m, 1e-5)
    for cuts in ([[(0, edge - 3)], [(edge - 3, edge + 5)], [(edge + 5, n)]],                      # a portion across the edge
                 [[(0, edge - 6)], *[[(i, i + 1)] for i in range(edge - 6, edge + 6)], [(edge + 6, n)]]):   # single tokens across it
        got = _in_steps(_Slots(mixer, dtype, [n], page=page), [x], cuts)[0]
        torch.testing.assert_close(got, want, **TOL[dtype])
    # the test's premise: the weight of the key in map 1 of head 0 is all or nothing on the two sides of the edge
    q = (x.double() @ w["q"].T)[:, :dim]
    k = (x.double() @ w["k"].T)[:, :dim]
    s = 40.0 * torch.tanh(q @ k.T / 40.0)
    p = plain.softmax_rows(s, plain.window_mask(torch.arange(n), size))
    assert float(p[far:edge, far].min()) > 0.99 and float(p[edge:, far].max()) == 0.0 and float(p[0, 0]) == 1.0
    assert float((want[edge - 1] - want[edge]).abs().max()) > 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, page, far, size", [(16, 16, 47, 48), (16, 16, 100, 37), (64, 64, 191, 96), (128, 64, 130, 200)])
def test_a_key_is_seen_inside_its_chunk_only(dtype, dim, page, far, size):
    """
    One key is made to dominate head 0 of a chunked layer: every later query of its chunk gives it all its weight,
    the first query of the next chunk (a chunk's first token sees itself only) and all after it none, although the
    key is only a few tokens back; as a portion across the chunk's end and token by token across it.
    """
    from tinyserve_llm_b200.config.spec import GatedAttentionSpec
    width, heads, vdim = 32, 2, dim
    spec = GatedAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=1, head_dim=dim, value_dim=vdim, scale=1.0, chunk=size)
    mixer, w = _mixer(spec, dtype, 7, lambda t: _one_key_stands_out(t, [0], [0], width))
    edge = (far // size + 1) * size                  # the first position of the next chunk
    n = edge + 30
    x = torch.randn(n, width, generator=torch.Generator().manual_seed(3)) * 0.3
    x[:, 0], x[:, 1] = 6.0, 0.0
    x[far, 1] = 6.0
    x = x.to(dtype)
    m = {"heads": heads, "kv_heads": 1, "dim": dim, "vdim": vdim, "scale": 1.0, "mask": {"size": size}}
    want = plain.chunked_attention(x.double(), w, m, 1e-5)
    for cuts in ([[(0, edge - 3)], [(edge - 3, edge + 5)], [(edge + 5, n)]],
                 [[(0, max(edge - 6, 1))], *[[(i, i + 1)] for i in range(max(edge - 6, 1), edge + 6)], [(edge + 6, n)]]):
        got = _in_steps(_Slots(mixer, dtype, [n], page=page), [x], cuts)[0]
        torch.testing.assert_close(got, want, **TOL[dtype])
    q = (x.double() @ w["q"].T)[:, :dim]
    k = (x.double() @ w["k"].T)[:, :dim]
    p = plain.softmax_rows(q @ k.T, plain.chunk_mask(torch.arange(n), size))
    assert float(p[far:edge, far].min()) > 0.99 and float(p[edge:, far].max()) == 0.0
    assert float(p[edge, edge]) == 1.0 and float((want[edge - 1] - want[edge]).abs().max()) > 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank, page", [(24, 16), (64, 64)])
def test_latent_attention_finds_a_far_key_at_a_page_border(dtype, rank, page):
    """
    One token's latent, hundreds of positions back at a page's last slot, is made the only one head 0's queries
    match: they return its values, as a prompt portion and as single tokens; queries before it do not.
    """
    from tinyserve_llm_b200.config.spec import LatentAttentionSpec
    width, heads, dim, vdim, far = 32, 2, 16, 24, 4 * page - 1
    spec = LatentAttentionSpec(hidden_size=width, num_heads=heads, head_dim=dim, rot_dim=0, value_dim=vdim, q_rank=0, kv_rank=rank,
                               scale=1.0, norm_eps=1e-5, position=None, output_gate=True)

    def edit(t):
        t["q"], t["uk"] = torch.zeros_like(t["q"]), torch.zeros_like(t["uk"])
        t["q"][0, 0] = 1.0                           # head 0's first query channel reads input channel 0
        t["uk"][0, 0] = 1.0                          # ... and meets the latent's first channel,
        t["dkv"][0] = 0.0
        t["dkv"][0, 1] = 1.0                         # which reads input channel 1
        t["dkv.norm"][0] = 1.0

    mixer, w = _mixer(spec, dtype, 8, edit)
    n = far + 150
    x = torch.randn(n, width, generator=torch.Generator().manual_seed(4)) * 0.3
    x[:, 0], x[:, 1] = 8.0, 0.0
    x[far, 1] = 30.0                                 # after the norm this latent's first channel is near sqrt(rank)
    x = x.to(dtype)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": 1.0}
    want = plain.latent_attention(x.double(), w, m, 1e-5)
    got = _in_steps(_Slots(mixer, dtype, [n], page=page), [x], [[(0, far - 2)], [(far - 2, far + 100)], *[[(i, i + 1)] for i in range(far + 100, n)]])[0]
    torch.testing.assert_close(got, want, **TOL[dtype])
    c = plain.rms_norm(x.double() @ w["dkv"].T, w["dkv.norm"], 1e-5)
    s = (x.double() @ w["q"].T)[:, :dim] @ (c @ w["uk"].T)[:, :dim].T
    p = plain.softmax_rows(s, plain.causal_mask(torch.arange(n)))
    assert float(p[far:, far].min()) > 0.99 and float(p[:far, far].max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_difference_and_norm_kernel(dtype):
    """The maps in the order [group][map][head of the group] (float32 and the activation dtype) against the formula."""
    ops = _runtime(dtype).ops
    T, heads, kv_heads, vdim, weight, eps, scale = 37, 6, 2, 40, 0.83, 1e-5, 0.45
    r = heads // kv_heads
    g = torch.Generator().manual_seed(5)
    maps = torch.randn(T, kv_heads, 2, r, vdim, generator=g)
    ctx = _ctx([(0, T)])
    for maps_dtype in (torch.float32, dtype):
        m = maps.to(maps_dtype)
        got = ops.difference_head_norm(m.reshape(T, -1).cuda(), ctx, heads, kv_heads, vdim, weight, eps, scale, dtype).cpu().double()
        d = (m[:, :, 0].double() - weight * m[:, :, 1].double()).reshape(T, heads, vdim)
        want = (plain.rms_norm(d, None, eps) * scale).reshape(T, heads * vdim)
        torch.testing.assert_close(got, want, **TOL[dtype])


def test_logits_are_scaled_then_capped():
    ops = _runtime(torch.float32).ops
    x = torch.linspace(-40, 40, 1001)
    got = ops.scale_tanh_cap(x.clone().cuda(), 1.7, 9.0).cpu()
    torch.testing.assert_close(got.double(), plain.tanh_cap(x.double() * 1.7, 9.0), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(ops.scale_tanh_cap(x.clone().cuda(), 0.5, 0.0).cpu(), x * 0.5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_gated_feed_forward(dtype):
    """Few rows (the weight-streaming product's epilogue), some (library product and a kernel), many (the tcgen05 product's epilogue)."""
    from tinyserve_llm_b200.config.spec import GatedMLPSpec
    from tinyserve_llm_b200.parts.base import part_class
    from tinyserve_llm_b200.weights import random_tensors
    spec = GatedMLPSpec(hidden_size=128, intermediate_size=192, activation="gelu_tanh", tensor_names=("gate", "up", "down"))
    cls = part_class("feed_forward", spec)
    tensors = dict(random_tensors(cls.declare(spec), 9, std=0.15, unit_std=0.25))
    ff = cls(spec, {k: v.cuda() for k, v in tensors.items()}, _runtime(dtype))
    w = {k: v.double() for k, v in tensors.items()}
    for rows in (3, 100, 640):
        x = (torch.randn(rows, 128, generator=torch.Generator().manual_seed(rows)) * 2).to(dtype)
        got = ff.forward(x.cuda(), None).cpu().double()
        rows_close(got, plain.dense_ff(x.double(), w), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_embedding_is_normed_before_it_starts_the_stream(dtype):
    """stream = LN(table[id]) w_embed in float32, and the first norm's output, from one kernel."""
    ops = _runtime(dtype).ops
    g = torch.Generator().manual_seed(6)
    table = (torch.randn(50, 72, generator=g) * 3 + 0.5).to(dtype)
    w_start, w_open = torch.randn(72, generator=g), torch.randn(72, generator=g)
    ids = torch.tensor([3, 49, 0, 17, 3], dtype=torch.int32)
    stream = torch.empty(5, 72, dtype=torch.float32, device="cuda")
    out = ops.stream_norm(None, None, stream, w_open.cuda(), 1e-5, dtype, table=table.cuda(), ids=ids.cuda(), centered=True,
                          w_start=w_start.cuda())
    want_stream = plain.layer_norm(table.double()[ids.long()], w_start.double(), 1e-5)
    torch.testing.assert_close(stream.cpu().double(), want_stream, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out.cpu().double(), plain.layer_norm(want_stream, w_open.double(), 1e-5), **TOL[dtype])


# ---------------------------------------------------------------------------------------------- the programs
def test_replay_program_on_a_model_folder(folders, tmp_path):
    """bin/trace_run on a Folavik folder: portions, a decoded tail, two requests side by side, reused pages."""
    name = "wide"
    vocab = CONFIGS[name]["vocab"]
    a, b = ids_of(vocab, 190, 21), ids_of(vocab, 170, 22)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:164], "want": [0, 163]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[164:166], "want": [1]}, {"id": "b", "tokens": b[:169], "want": [168]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[169:], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[166:], "want": [23]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": b, "want": [169]}], "end": ["c"]},
    ]
    rows = {0: [("a", 0), ("a", 163)], 1: [("a", 165), ("b", 168)], 2: [("b", 169)], 3: [("a", 189)], 4: [("b", 169)]}
    for dtype in ("float32", "bfloat16"):
        want = {"a": plain_logits(folders[name], a), "b": plain_logits(folders[name], b)}
        out = tmp_path / dtype
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name], "--dtype", dtype,
                               "--out", str(out), "--max-tokens", "448"],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [line for line in proc.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(5)]
        got, expected = [], []
        for step, places in rows.items():
            got.append(torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(places), vocab)).double())
            expected += [want[r][p] for r, p in places]
        close(torch.cat(got), torch.stack(expected), dtype)


@pytest.mark.parametrize("name", ["mixed", "latent"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """LLM.generate with the scheduler, prompt portions, CUDA graphs and running ahead: the plain model's greedy tokens."""
    from tinyserve_llm_b200 import LLM, CacheConfig, SamplingParams, SchedulerConfig
    raw, dtype = CONFIGS[name], "float32"
    tensors = read_tensors(folders[name])
    prompts = [ids_of(raw["vocab"], n, 30 + n) for n in (3, 41, 18, 77, 1)]
    new = 12
    want = []
    for p in prompts:
        ids = list(p)
        for _ in range(new):
            ids.append(int(plain.forward(raw, tensors, ids)[-1].argmax()))
        want.append(ids[len(p):])
    llm = LLM(folders[name], SchedulerConfig(max_model_len=128, max_num_seqs=3, max_num_batched_tokens=48, prefill_chunk=20),
              CacheConfig(block_size=16), dtype="float32", num_blocks=24, seed=0)
    done = llm.generate(prompts, SamplingParams(max_tokens=new, temperature=0.0, ignore_eos=True))
    assert [c.token_ids[0] for c in done] == want
