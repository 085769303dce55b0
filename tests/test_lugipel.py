"""
The Lugipel decoder in the engine against the plain implementation of tests/plain_lugipel.py: each
mechanism alone (with weights or inputs made so that a fault shows), whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal requests in one batch against each
alone, pages and state slots that are freed and taken again, keys at a window's edge and at page
borders, the first tokens, long decoding, several sizes, steps replayed from CUDA graphs, the replay
program and greedy generation through the engine's entry point.
"""

import copy
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import lugipel_configs as C
import plain_lugipel as plain
from test_nipizen import TOL, Engine, _ctx, _i32, _in_steps, _mixer, _runtime, _Slots, ids_of, read_tensors, rows_close

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CONFIGS = {"mixed": C.MIXED, "recurrent": C.RECURRENT, "windows": C.WINDOWS, "wide": C.WIDE}
SEEDS = {"mixed": 511, "recurrent": 522, "windows": 533, "wide": 544}
PAGE = {"mixed": 16, "recurrent": 16, "windows": 16, "wide": 64}


def every_output_chosen(raw):
    """The same model with all groups kept and every router output chosen: no discrete choice is left."""
    out = copy.deepcopy(raw)
    for layer in out["layers"]:
        f = layer["mlp"]
        if f is not None and f["kind"] == "moe":
            r = f["router"]
            r["top"] = r["experts"] + r["identity"]
            r["groups"]["keep"] = r["groups"]["count"]
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """
    Per configuration a model folder for the float32 comparisons (the sharp ones, routing included) and one
    for the bfloat16 comparisons in which every token uses every router output (same tensors): with fewer,
    a token whose choice scores lie closer than bfloat16's rounding of its activations takes another expert
    than the float64 model, and the positions after it would be compared with the wrong thing.  Routing in
    bfloat16 is compared by the test of the routed feed-forward alone.
    """
    from tinyserve_llm_b200.weights import write_random_model
    out = {}
    for name, raw in CONFIGS.items():
        for dtype, config in (("float32", raw), ("bfloat16", every_output_chosen(raw))):
            folder = str(tmp_path_factory.mktemp(f"lugipel_{name}_{dtype}"))
            write_random_model(folder, config, SEEDS[name], **C.WEIGHTS)
            out[name, dtype] = folder
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
        assert float(err.max()) < 0.2 and float(err.median()) < 0.04, \
            f"relative error: worst {float(err.max()):.3f} at {int(err.argmax())}, median {float(err.median()):.3f}"


# ---------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_equals_the_plain_model(folders, name, dtype):
    ids = ids_of(CONFIGS[name]["vocab"], 150, 1)
    got = Engine(folders[name, dtype], dtype, page=PAGE[name]).run("a", ids, [len(ids)])
    close(got, plain_logits(folders[name, dtype], ids), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prompt_then_token_by_token_and_portions_of_many_sizes(folders, name, dtype):
    """The same logits whether the tokens come at once, one by one after a head, or in portions down to two tokens."""
    ids = ids_of(CONFIGS[name]["vocab"], 150, 2)
    want = plain_logits(folders[name, dtype], ids)
    page = PAGE[name]
    decoded = Engine(folders[name, dtype], dtype, page=page).run("a", ids, [30] + [1] * 120)     # windows pass over decoded tokens
    close(decoded, want, dtype)
    portions = Engine(folders[name, dtype], dtype, page=page).run("a", ids, [2, 3, 17, 2, 16, 5, 31, 1, 1, 2])
    close(portions, want, dtype)
    one_by_one = Engine(folders[name, dtype], dtype, page=page).run("a", ids[:40], [1])          # the first tokens, alone
    close(one_by_one, want[:40], dtype)
    if dtype == "float32":                                                           # the cut changes nothing beyond rounding
        torch.testing.assert_close(decoded, portions, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(folders, dtype, graphs):
    """
    Five requests through three state slots and a pool that holds less than their sum: portions of
    some beside single tokens of others, requests that sit a step out, ended requests whose pages
    and slots the next ones take (a recurrent state that is not zeroed, or a page read through a
    stale table, show).  With `graphs`, every step is replayed from a CUDA graph from its first sighting on.
    """
    name = "mixed"
    vocab = CONFIGS[name]["vocab"]
    reqs = {k: ids_of(vocab, n, 10 + i) for i, (k, n) in enumerate((("a", 70), ("b", 33), ("c", 9), ("d", 58), ("e", 41)))}
    eng = Engine(folders[name, dtype], dtype, page=16, pages=12, slots=3, cuda_graphs=graphs)
    eng.step([("a", reqs["a"][:40]), ("b", reqs["b"][:2])])
    eng.step([("a", reqs["a"][40:41]), ("b", reqs["b"][2:19]), ("c", reqs["c"][:9])], end=["c"])
    eng.step([("b", reqs["b"][19:20])])                                             # a sits this one out
    eng.step([("d", reqs["d"][:3]), ("a", reqs["a"][41:70]), ("b", reqs["b"][20:33])], end=["a", "b"])   # d takes c's slot
    eng.step([("d", reqs["d"][3:35]), ("e", reqs["e"][:1])])
    eng.step([("e", reqs["e"][1:2]), ("d", reqs["d"][35:36])])
    for i in range(36, 58):
        both = [("d", reqs["d"][i:i + 1])]
        j = 2 + (i - 36)
        if j < 41:
            both.append(("e", reqs["e"][j:j + 1]))
        eng.step(both, end=["d"] if i == 57 else [])
    eng.step([("e", reqs["e"][24:41])], end=["e"])
    assert eng.manager.stats().pages_in_use == 0 and eng.manager.free_state_slots() == 3
    if graphs:
        assert eng.runner.graph_replays > 20
    for k, ids in reqs.items():
        close(eng.logits(k), plain_logits(folders[name, dtype], ids), dtype)
        alone = Engine(folders[name, dtype], dtype, page=16, pages=12, slots=3).run(k, ids, [len(ids)])
        if dtype == "float32":
            torch.testing.assert_close(eng.logits(k), alone, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_model_in_large_portions_also_from_a_graph(folders, dtype):
    """
    Pages of 64 tokens, heads of 64 and 128 channels, portions of more than a hundred tokens: the
    recurrence runs in stretches, the windows cross page borders inside portions; with few
    (token, expert) pairs and with many.  Same logits.
    """
    name = "wide"
    ids = ids_of(CONFIGS[name]["vocab"], 420, 7)
    eng = Engine(folders[name, dtype], dtype, page=64, pages=10, cuda_graphs=True)
    got = eng.run("a", ids, [150, 129, 2, 64, 1, 1, 73], last_only=True)
    assert eng.runner.graph_replays >= 3
    close(got, plain_logits(folders[name, dtype], ids)[[149, 278, 280, 344, 345, 346, 419]], dtype)


def test_long_decoding_keeps_its_state_and_its_windows(folders):
    """260 tokens one by one after a short head, over several pages; pages behind the windows are given back."""
    name, dtype = "mixed", "float32"
    ids = ids_of(CONFIGS[name]["vocab"], 260, 3)
    got = Engine(folders[name, dtype], dtype, page=16, pages=18).run("a", ids, [7] + [1] * 253)
    close(got, plain_logits(folders[name, dtype], ids), dtype)


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [72, 33, 256])
def test_min_gru_alone(dtype, width):
    """
    The recurrence against the plain one: two requests in one launch on slots that are not in order, cut
    into single tokens, short portions and portions long enough for the kernel that walks in stretches;
    gate biases from slow to fast, candidates on both sides of zero.
    """
    from tinyserve_llm_b200.config.spec import MinGRUSpec
    hidden = 64
    spec = MinGRUSpec(hidden_size=hidden, width=width, bias=True)

    def edit(t):
        t["z.b"] = torch.linspace(-5.0, 3.0, width).to(t["z.b"].dtype)
        t["x.b"] = torch.linspace(-2.0, 2.0, width).flip(0).to(t["x.b"].dtype)
        t["x"] = t["x"] * 4

    mixer, w = _mixer(spec, dtype, 7, edit)
    g = torch.Generator().manual_seed(3)
    lens = [333, 26]
    x_of = [torch.randn(n, hidden, generator=g).to(dtype) for n in lens]
    want = [plain.min_gru(x.double(), w) for x in x_of]
    cuts = [[(0, 1), (0, 2)], [(1, 3), (2, 2)], [(3, 200), (2, 5)], [(200, 201), (5, 26)], [(201, 333), (26, 26)]]
    got = _in_steps(_Slots(mixer, dtype, lens), x_of, cuts)
    for a, b in zip(got, want):
        rows_close(a, b, dtype)
    whole = _in_steps(_Slots(mixer, dtype, lens), x_of, [[(0, 333), (0, 26)]])
    for a, b in zip(whole, want):
        rows_close(a, b, dtype)


def test_min_gru_reads_the_first_token_far_later():
    """With update gates close to zero the first token is still in the state 300 tokens on: a state lost on the way shows."""
    from tinyserve_llm_b200.config.spec import MinGRUSpec
    hidden, width = 32, 40
    spec = MinGRUSpec(hidden_size=hidden, width=width, bias=True)

    def edit(t):
        t["z.b"] = torch.full_like(t["z.b"], -7.0)
        t["z"] = torch.zeros_like(t["z"])

    mixer, w = _mixer(spec, torch.float32, 9, edit)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(310, hidden, generator=g)
    x[0] *= 30                                                         # a first candidate that stands out
    want = plain.min_gru(x.double(), w)
    other = x.clone()
    other[0] = -other[0]
    assert float((plain.min_gru(other.double(), w)[-1] - want[-1]).abs().max()) > 1e-3      # the premise
    got = _in_steps(_Slots(mixer, torch.float32, [310]), [x], [[(0, 50)], [(50, 303)], *[[(i, i + 1)] for i in range(303, 310)]])[0]
    torch.testing.assert_close(got, want, **TOL[torch.float32])


def _attention_spec(width, heads, kv_heads, dim, vdim, scale, window, coef, every, eps=1e-5):
    from tinyserve_llm_b200.config.lugipel import LugipelConfig
    raw = C.model(50, width, eps, 1.0, [(C.attention(heads, kv_heads, dim, vdim, scale, window, coef, every), None)])
    return LugipelConfig.from_dict(raw).mixer_spec(0), raw["layers"][0]["mixer"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, coef, every", [
    (6, 2, 20, 36, 11, 0.4, 5), (3, 1, 64, 64, 30, 0.3, 16), (5, 5, 12, 20, 100, 0.7, 1), (2, 1, 128, 128, 17, 0.0, 9)])
def test_sigmoid_attention_alone(dtype, heads, kv_heads, dim, vdim, window, coef, every):
    """
    The attention mixer against the plain one: the norm of every head by itself, the query temperature across
    several of its steps, the distance penalty, the number per head, sigmoid weights inside the window,
    values of another head size, the gate a head; two requests of unequal length fed in portions that end
    inside pages and inside windows, then token by token.
    """
    width = 64
    spec, m = _attention_spec(width, heads, kv_heads, dim, vdim, 0.3, window, coef, every)

    def edit(t):
        t["pb"] = torch.linspace(-2.0, 1.0, heads).to(t["pb"].dtype)

    mixer, w = _mixer(spec, dtype, 3, edit)
    g = torch.Generator().manual_seed(1)
    lens = [45, 21]
    x_of = [torch.randn(n, width, generator=g).to(dtype) for n in lens]
    want = [plain.sigmoid_attention(x.double(), w, m, 1e-5) for x in x_of]
    cuts = [[(0, 17), (0, 2)], [(17, 33), (2, 19)], [(33, 34), (19, 20)], [(34, 45), (20, 21)]]
    got = _in_steps(_Slots(mixer, dtype, lens), x_of, cuts)
    for a, b in zip(got, want):
        rows_close(a, b, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [40, 300])
def test_a_key_at_a_page_border_is_seen_to_the_windows_edge_and_no_further(dtype, window):
    """
    One key at a page's last slot is made to stand out for every query (its first key channel and every
    query's first channel are large, the number per head is strongly negative, so every other key weighs
    next to nothing): queries up to window - 1 positions later return its value, the next one does not; in
    a prompt portion and as single tokens, with the edge inside a portion and at a decoded token.
    """
    width, heads, dim, vdim, far = 32, 2, 16, 24, 63
    spec, m = _attention_spec(width, heads, 1, dim, vdim, 1.0, window, 0.0, 1)

    def edit(t):
        t["q"] = torch.zeros_like(t["q"])
        t["q"][0, 0] = t["q"][dim, 0] = 1.0         # both heads' first query channel reads input channel 0
        t["k"] = t["k"] * 0.5
        t["k"][0] = 0.0
        t["k"][0, 1] = 1.0                          # the key's first channel reads input channel 1
        t["k"][:, :2] = t["k"][:, :2] * (torch.arange(dim)[:, None] == 0)      # the other key channels read neither
        t["q.norm"] = torch.ones_like(t["q.norm"])
        t["k.norm"] = torch.ones_like(t["k.norm"])
        t["pb"] = torch.full_like(t["pb"], -8.0)
        t["g"] = torch.zeros_like(t["g"])

    mixer, w = _mixer(spec, dtype, 5, edit)
    g = torch.Generator().manual_seed(2)
    n = far + window + 30
    x = torch.randn(n, width, generator=g) * 0.3
    x[:, 0] = 6.0                                # every query asks for a large first key channel
    x[:, 1] = 0.0
    x[far, 1] = 40.0                             # only this token's key has it
    x = x.to(dtype)
    want = plain.sigmoid_attention(x.double(), w, m, 1e-5)
    edge = far + window                          # the first position that no longer sees the key
    assert float((want[edge - 1] - want[edge]).norm()) > 10 * float((want[edge] - want[edge + 1]).norm())     # the premise
    single = _in_steps(_Slots(mixer, dtype, [n], page=16), [x],
                       [[(0, 64)], [(64, edge - 3)], *[[(i, i + 1)] for i in range(edge - 3, edge + 4)], [(edge + 4, n)]])[0]
    torch.testing.assert_close(single, want, **TOL[dtype])
    portion = _in_steps(_Slots(mixer, dtype, [n], page=16), [x], [[(0, far + 1)], [(far + 1, edge - 7)], [(edge - 7, edge + 9)], [(edge + 9, n)]])[0]
    torch.testing.assert_close(portion, want, **TOL[dtype])


@pytest.mark.parametrize("prompt_kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("heads, kv_heads, dim, window", [(4, 2, 64, 100), (6, 1, 128, 257), (2, 2, 64, 1000), (16, 2, 128, 64)])
def test_sigmoid_attention_at_the_tensor_core_kernels_sizes(monkeypatch, heads, kv_heads, dim, window, prompt_kernel):
    """
    Keys and values of 64 and of 128 channels a head on pages of 64 tokens in bfloat16: a prompt's portions run in
    tiles of 64 queries against tiles of 64 keys, single tokens in splits of 256 keys that are merged.  Two
    requests of unequal length, in portions that end inside tiles, with windows that begin inside a tile, at
    its edge and before the first key, then token by token across a split's edge; a portion beside single
    tokens in one step.  The portions once on the tcgen05 kernel (tiles of 128 queries), once on the mma one.
    """
    dtype, width = torch.bfloat16, 64
    spec, m = _attention_spec(width, heads, kv_heads, dim, dim, 0.2, window, 0.3, 50)

    def edit(t):
        t["pb"] = torch.linspace(-3.0, -1.0, heads).to(t["pb"].dtype)

    mixer, w = _mixer(spec, dtype, 7, edit)
    monkeypatch.setattr(mixer.rt.ops, "tcgen05_attention", prompt_kernel == "tcgen05")
    g = torch.Generator().manual_seed(3)
    lens = [530, 203]
    x_of = [torch.randn(n, width, generator=g).to(dtype) for n in lens]
    want = [plain.sigmoid_attention(x.double(), w, m, 1e-5) for x in x_of]
    cuts = [[(0, 130), (0, 2)], [(130, 131), (2, 67)], [(131, 390), (67, 68)], [(390, 507), (68, 190)]]
    cuts += [[(i, i + 1), (min(190 + i - 507, 203), min(191 + i - 507, 203))] for i in range(507, 530)]
    got = _in_steps(_Slots(mixer, dtype, lens, page=64), x_of, cuts)
    for a, b in zip(got, want):
        rows_close(a, b, dtype)


@pytest.mark.parametrize("prompt_kernel", ["tcgen05", "mma"])
def test_a_far_key_stands_out_through_the_tensor_core_kernels(monkeypatch, prompt_kernel):
    """
    As the test at a page's border, at head sizes the tensor-core kernels take: one key at the last slot of a
    page of 64 tokens weighs nearly 1, every other next to nothing; queries see it up to window - 1 positions
    later and no further, in a portion whose tile holds the edge and as single tokens whose split holds it.
    """
    dtype, width, heads, dim, far, window = torch.bfloat16, 32, 2, 64, 127, 300
    spec, m = _attention_spec(width, heads, 1, dim, dim, 1.0, window, 0.0, 1)

    def edit(t):
        t["q"] = torch.zeros_like(t["q"])
        t["q"][0, 0] = t["q"][dim, 0] = 1.0
        t["k"] = t["k"] * 0.5
        t["k"][0] = 0.0
        t["k"][0, 1] = 1.0
        t["k"][:, :2] = t["k"][:, :2] * (torch.arange(dim)[:, None] == 0)
        t["q.norm"] = torch.ones_like(t["q.norm"])
        t["k.norm"] = torch.ones_like(t["k.norm"])
        t["pb"] = torch.full_like(t["pb"], -12.0)
        t["g"] = torch.zeros_like(t["g"])

    mixer, w = _mixer(spec, dtype, 5, edit)
    monkeypatch.setattr(mixer.rt.ops, "tcgen05_attention", prompt_kernel == "tcgen05")
    g = torch.Generator().manual_seed(2)
    n = far + window + 40
    x = torch.randn(n, width, generator=g) * 0.3
    x[:, 0] = 6.0
    x[:, 1] = 0.0
    x[far, 1] = 40.0
    x = x.to(dtype)
    want = plain.sigmoid_attention(x.double(), w, m, 1e-5)
    edge = far + window
    assert float((want[edge - 1] - want[edge]).norm()) > 10 * float((want[edge] - want[edge + 1]).norm())     # the premise
    single = _in_steps(_Slots(mixer, dtype, [n], page=64), [x],
                       [[(0, 64)], [(64, edge - 3)], *[[(i, i + 1)] for i in range(edge - 3, edge + 4)], [(edge + 4, n)]])[0]
    torch.testing.assert_close(single, want, **TOL[dtype])
    portion = _in_steps(_Slots(mixer, dtype, [n], page=64), [x], [[(0, far + 1)], [(far + 1, edge - 7)], [(edge - 7, edge + 9)], [(edge + 9, n)]])[0]
    torch.testing.assert_close(portion, want, **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_query_temperature_steps_at_its_positions(dtype):
    """ops.qk_norm_rope_store alone: every head normed by itself, q scaled by 1 + c ln(floor((p + 1) / n) + 1) from position 0 on."""
    from tinyserve_llm_b200.ops import get_ops
    from gpu_util import make_binding
    ops = get_ops()
    H, G, D, V, T, every, coef, eps = 3, 1, 10, 6, 40, 4, 0.6, 1e-4
    g = torch.Generator().manual_seed(5)
    y = torch.randn(T, H * D + G * D + G * V, generator=g).to(dtype)
    wq, wk = torch.rand(D, generator=g) + 0.5, torch.rand(D, generator=g) + 0.5
    binding = make_binding(4, 1, G, 16, D, dtype, [[2, 0, 3]])
    binding.v_pool = torch.zeros((4, 1, G, 16, V), dtype=dtype, device="cuda")
    binding.v_page_stride, binding.v_entry_offset = G * 16 * V, 0
    ctx = _ctx([(0, T)])
    q = ops.qk_norm_rope_store(y.cuda(), (0, H * D, H * D + G * D), None, (wq.cuda(), wk.cuda()), eps, None, ctx, binding,
                               H, G, D, V, norm_per_head=True, q_temperature=(coef, every)).cpu().double()
    yq = y.double()[:, :H * D].view(T, H, D)
    want = plain.rms_norm(yq, wq.double(), eps) * plain.query_temperature(torch.arange(T), coef, every)[:, None, None]
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.03, rtol=0.02)
    torch.testing.assert_close(q.view(T, H, D), want, **tol)
    k_want = plain.rms_norm(y.double()[:, H * D:H * D + D], wk.double(), eps)
    pages = [2, 0, 3]
    k_got = torch.stack([binding.k_pool[pages[p // 16], 0, 0, p % 16] for p in range(T)]).cpu().double()
    torch.testing.assert_close(k_got, k_want, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_scale_and_sinusoid(dtype):
    """The stream's first rows: table[id] * scale plus sine and cosine interleaved, at small and at large positions, odd width."""
    from tinyserve_llm_b200.config.spec import SinusoidSpec
    from tinyserve_llm_b200.parts.base import part_class
    rt = _runtime(dtype)
    W, vocab, scale, eps = 37, 11, 2.5, 1e-5
    position = part_class("position", SinusoidSpec(size=W, base=10000.0))(SinusoidSpec(size=W, base=10000.0), {}, rt)
    g = torch.Generator().manual_seed(6)
    table = torch.randn(vocab, W, generator=g).to(dtype)
    ids = [3, 0, 10, 7, 7, 1]
    positions = [0, 1, 2, 77, 4000, 4001]
    weight = torch.rand(W, generator=g) + 0.5
    stream = torch.empty((len(ids), W), dtype=torch.float32, device="cuda")
    out = rt.ops.stream_norm(None, None, stream, weight.cuda(), eps, dtype, table=table.cuda(), ids=_i32(ids), scale=scale,
                             positions=_i32(positions), position_frequencies=position.frequencies)
    want = table.double()[ids] * scale + plain.sinusoid(torch.tensor(positions), W)
    torch.testing.assert_close(stream.cpu().double(), want, atol=2e-3, rtol=0)        # float32 angles at position 4000
    torch.testing.assert_close(stream.cpu().double()[:4], want[:4], atol=2e-5, rtol=0)
    tol = dict(atol=2e-3, rtol=1e-3) if dtype == torch.float32 else dict(atol=0.03, rtol=0.02)
    torch.testing.assert_close(out.cpu().double(), plain.rms_norm(want, weight.double(), eps), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("p, q", [(0.3, -0.8), (-2.0, 1.5)])
@pytest.mark.parametrize("width, ff, tokens", [(48, 72, 40), (64, 104, 5), (96, 40, 32)])
def test_dense_feed_forward_with_xielu(dtype, p, q, width, ff, tokens):
    """Many rows (the product, then the activation's own pass) and a few (the activation in the product's epilogue)."""
    from tinyserve_llm_b200.config.spec import PlainMLPSpec
    from tinyserve_llm_b200.parts.base import part_class
    from tinyserve_llm_b200.weights import random_tensors
    spec = PlainMLPSpec(hidden_size=width, intermediate_size=ff, activation="xielu", param_name="act")
    cls = part_class("feed_forward", spec)
    tensors = dict(random_tensors(cls.declare(spec), 19, std=0.3))
    tensors["act"] = torch.tensor([p, q]).to(tensors["act"].dtype)
    part = cls(spec, {k: v.cuda() for k, v in tensors.items()}, _runtime(dtype))
    g = torch.Generator().manual_seed(2)
    x = torch.randn(tokens, width, generator=g).to(dtype)
    got = part.forward(x.cuda(), SimpleNamespace()).cpu().double()
    rows_close(got, plain.dense_ff(x.double(), {k: v.double() for k, v in tensors.items()}), dtype)
    # the activation gives the same numbers in the epilogue as in a pass of its own
    ops = part.rt.ops
    fused = ops.linear_unary(x.cuda(), part.up.weight, "xielu", *part.factors)
    apart = ops.unary_activation(ops.linear(x.cuda(), part.up.weight), "xielu", *part.factors)
    assert torch.equal(fused, apart)


ROUTERS = [(7, 2, 2, (3, 2), 1.5, 50), (5, 0, 3, (1, 1), 0.7, 3), (6, 3, 1, (3, 1), 2.0, 50), (40, 8, 4, (8, 3), 1.0, 50),
           (12, 0, 3, (4, 4), 2.5, 150), (3, 1, 4, (2, 2), 1.0, 20)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, identity, top, groups, scale, tokens", ROUTERS)
def test_routed_experts_in_groups_with_identity_experts(dtype, experts, identity, top, groups, scale, tokens):
    """
    The routed feed-forward alone: ragged stretches per expert, identity experts among the chosen, a few tokens
    (the weight-streaming kernel) and many (the library's), padding rows of a replayed step.  In bfloat16
    every router output is chosen (see `folders`); the choice itself is compared in float32 and by the next test.
    """
    from tinyserve_llm_b200.config.lugipel import LugipelConfig
    from tinyserve_llm_b200.parts.base import part_class
    from tinyserve_llm_b200.weights import random_tensors
    width, ff = 48, 24
    f = C.moe(experts, identity, top, ff, groups, scale)
    if dtype == torch.bfloat16:
        f["router"]["top"], f["router"]["groups"]["keep"] = experts + identity, groups[0]
    spec = LugipelConfig.from_dict(C.model(50, width, 1e-5, 1.0, [(C.mingru(8), f)])).feed_forward_spec(0)
    cls = part_class("feed_forward", spec)
    tensors = dict(random_tensors(cls.declare(spec), 17, std=0.3))
    tensors["correction"] = (tensors["correction"].float() * 0.5 - 0.1).to(tensors["correction"].dtype)     # choice scores of both signs
    part = cls(spec, {k: v.cuda() for k, v in tensors.items()}, _runtime(dtype))
    g = torch.Generator().manual_seed(1)
    x = torch.randn(tokens, width, generator=g).to(dtype)
    seq_of_token = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    seq_of_token[-2:] = -1                                                           # padding rows of a replayed step
    got = part.forward(x.cuda(), SimpleNamespace(seq_of_token=seq_of_token)).cpu().double()[:tokens - 2]
    want = plain.routed_ff(x.double()[:tokens - 2], {k: v.double() for k, v in tensors.items()}, f)
    rows_close(got, want, dtype)


@pytest.mark.parametrize("outputs, identity, top, groups, keep, tokens", [
    (2048, 48, 9, 1024, 37, 11), (1500, 0, 5, 3, 2, 70), (96, 5, 8, 32, 8, 33), (33, 1, 33, 1, 1, 5), (64, 60, 2, 64, 2, 9)])
def test_grouped_router_alone_at_many_outputs(outputs, identity, top, groups, keep, tokens):
    """The routing kernel against the plain router: more outputs than a lane holds, more groups than lanes, every output chosen,
    nearly all of them identity experts."""
    from tinyserve_llm_b200.ops import get_ops
    g = torch.Generator().manual_seed(outputs + top)
    logits = torch.randn(tokens, outputs, generator=g) * 2.0
    correction = torch.randn(outputs, generator=g) * 0.05 - 0.02
    r = {"experts": outputs - identity, "identity": identity, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}
    want_chosen, want_share = plain.route(logits.double(), {"router": torch.eye(outputs, dtype=torch.float64),
                                                            "correction": correction.double()}, r)
    chosen, share, _, _, _, identity_share = get_ops().moe_route_grouped(
        logits.cuda(), correction.cuda(), SimpleNamespace(), top, real_experts=outputs - identity, groups=groups, keep=keep,
        weight_scale=1.7, share_eps=1e-20)
    expected = torch.where(want_chosen < outputs - identity, want_chosen, torch.full_like(want_chosen, -1))
    assert chosen.cpu().tolist() == expected.tolist()                      # in the order of the choice scores
    torch.testing.assert_close(share.cpu().double(), want_share, rtol=2e-5, atol=1e-7)
    if identity:
        torch.testing.assert_close(identity_share.cpu().double(), (want_share * (want_chosen >= outputs - identity)).sum(-1),
                                   rtol=2e-5, atol=1e-7)


def test_grouped_router_choices_by_hand():
    """
    Scores over all outputs, choice by score + correction inside the kept groups, shares without the
    correction over their sum times the constant; a group whose choice scores are all negative still ranks
    above nothing; ties go to the lower index; identity outputs get no row but a share.
    """
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    logits = torch.log(torch.tensor([[0.10, 0.05, 0.30, 0.25, 0.20, 0.10],       # groups of two: ranks by choice score
                                     [0.25, 0.25, 0.10, 0.10, 0.15, 0.15]]))
    correction = torch.tensor([0.0, 0.0, -0.5, -0.5, 0.0, 0.3])
    chosen, share, offsets, _, row_of_pair, identity = ops.moe_route_grouped(
        logits.cuda(), correction.cuda(), SimpleNamespace(), 2, real_experts=4, groups=3, keep=2, weight_scale=2.0, share_eps=1e-20)
    # row 0: choice scores .10 .05 | -.20 -.25 | .20 .40 -> groups 2 and 0 are kept; best two: output 5 (identity), 4 (identity)
    # row 1: .25 .25 | -.4 -.4 | .15 .45 -> groups 2 and 0; best two: 5 (identity), then 0 (the tie with 1 goes to the lower index)
    assert chosen.tolist() == [[-1, -1], [-1, 0]]
    s = torch.softmax(logits, -1)
    torch.testing.assert_close(share.cpu()[0], 2.0 * torch.stack([s[0, 5], s[0, 4]]) / (s[0, 5] + s[0, 4]))
    torch.testing.assert_close(share.cpu()[1], 2.0 * torch.stack([s[1, 5], s[1, 0]]) / (s[1, 5] + s[1, 0]))
    torch.testing.assert_close(identity.cpu(), torch.stack([share.cpu()[0].sum(), share.cpu()[1, 0]]))
    assert offsets.tolist() == [0, 1, 1, 1, 1] and row_of_pair.tolist() == [-1, -1, -1, 0]
    # every choice score negative: a group that is not kept counts as minus infinity, not as zero (which would win here)
    chosen, _, _, _, _, _ = ops.moe_route_grouped(logits.cuda(), (correction - 1.0).cuda(), SimpleNamespace(), 2, real_experts=6,
                                                  groups=3, keep=1, weight_scale=1.0, share_eps=0.0)
    assert chosen.tolist() == [[5, 4], [5, 4]]


# ---------------------------------------------------------------------------------------------- entry points
def test_replay_program_on_a_model_folder(folders, tmp_path):
    """bin/trace_run on a Lugipel folder: portions, a decoded tail, two requests side by side, a reused slot."""
    name = "wide"
    vocab = CONFIGS[name]["vocab"]
    a, b = ids_of(vocab, 90, 21), ids_of(vocab, 70, 22)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:64], "want": [0, 63]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[64:66], "want": [1]}, {"id": "b", "tokens": b[:69], "want": [68]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[69:], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[66:], "want": [23]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": b, "want": [69]}], "end": ["c"]},
    ]
    rows = {0: [("a", 0), ("a", 63)], 1: [("a", 65), ("b", 68)], 2: [("b", 69)], 3: [("a", 89)], 4: [("b", 69)]}
    for dtype in ("float32", "bfloat16"):
        want = {"a": plain_logits(folders[name, dtype], a), "b": plain_logits(folders[name, dtype], b)}
        out = tmp_path / dtype
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name, dtype], "--dtype", dtype,
                               "--out", str(out), "--max-tokens", "256", "--max-requests", "2"],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [line for line in proc.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(5)]
        got, expected = [], []
        for step, places in rows.items():
            got.append(torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(places), vocab)).double())
            expected += [want[r][p] for r, p in places]
        close(torch.cat(got), torch.stack(expected), dtype)


@pytest.mark.parametrize("name", ["mixed", "recurrent"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """LLM.generate with the scheduler, prompt portions, CUDA graphs and running ahead: the plain model's greedy tokens."""
    from tinyserve_llm_b200 import LLM, CacheConfig, SamplingParams, SchedulerConfig
    raw, dtype = CONFIGS[name], "float32"
    tensors = read_tensors(folders[name, dtype])
    prompts = [ids_of(raw["vocab"], n, 30 + n) for n in (3, 41, 18, 77, 1)]
    new = 12
    want = []
    for p in prompts:
        ids = list(p)
        for _ in range(new):
            ids.append(int(plain.forward(raw, tensors, ids)[-1].argmax()))
        want.append(ids[len(p):])
    llm = LLM(folders[name, dtype], SchedulerConfig(max_model_len=128, max_num_seqs=3, max_num_batched_tokens=48, prefill_chunk=20),
              CacheConfig(block_size=16), dtype="float32", num_blocks=24, seed=0)
    done = llm.generate(prompts, SamplingParams(max_tokens=new, temperature=0.0, ignore_eos=True))
    assert [c.token_ids[0] for c in done] == want
