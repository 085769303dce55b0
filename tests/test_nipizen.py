"""
The Nipizen decoder in the engine against the plain implementation of tests/plain_nipizen.py: each
mechanism alone (with weights or inputs made so that a fault shows), whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal requests in one batch against each
alone, pages and state slots that are freed and taken again, far keys, page borders, the first
tokens, long decoding, several sizes, steps replayed from CUDA graphs, the replay program and greedy
generation through the engine's entry point.
"""

import dataclasses
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import nipizen_configs as C
import plain_nipizen as plain

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CONFIGS = {"mixed": C.MIXED, "recurrent": C.RECURRENT, "wide": C.WIDE, "grouped": C.GROUPED}
SEEDS = {"mixed": 111, "recurrent": 222, "wide": 333, "grouped": 444}
PAGE = {"mixed": 16, "recurrent": 16, "wide": 64, "grouped": 64}


def read_tensors(folder):
    from tinyserve_llm_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return {n: f.tensor(n) for n in f.names()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """
    Per configuration a model folder for the float32 comparisons (the sharp ones, routing included) and one
    for the bfloat16 comparisons in which every token uses all experts of a layer (same tensors, `top` =
    `experts`): with fewer, a token whose router scores at the edge of the chosen set lie closer than
    bfloat16's rounding of its activations takes another expert than the float64 model, and what it then
    writes into the states and the cache reaches the tokens after it; a fifth of the positions of these small
    models would be compared with the wrong thing.  Routing in bfloat16 is compared by the test of the routed
    feed-forward alone.
    """
    import copy
    from tinyserve_llm_b200.weights import write_random_model
    out = {}
    for name, raw in CONFIGS.items():
        folder = str(tmp_path_factory.mktemp(f"nipizen_{name}"))
        write_random_model(folder, raw, SEEDS[name], **C.WEIGHTS)
        out[name, "float32"] = folder
        every = copy.deepcopy(raw)
        for layer in every["layers"]:
            if layer["mlp"] is not None:
                layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
        steady = str(tmp_path_factory.mktemp(f"nipizen_{name}_every_expert"))
        write_random_model(steady, every, SEEDS[name], **C.WEIGHTS)
        out[name, "bfloat16"] = steady
    return out


def ids_of(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


_PLAIN = {}


def plain_logits(name, folder, ids):
    key = (folder, tuple(ids))
    if key not in _PLAIN:
        with open(os.path.join(folder, "config.json")) as f:
            raw = json.load(f)
        assert raw["vocab"] == CONFIGS[name]["vocab"]
        _PLAIN[key] = plain.forward(raw, read_tensors(folder), ids)
    return _PLAIN[key]


class Engine:
    """The engine's model, cache manager and step function on a small pool; logits are collected per request."""

    def __init__(self, folder, dtype, page=16, pages=24, slots=4, cuda_graphs=False):
        from tinyserve_llm_b200.engine.loading import build_cache, load_model
        from tinyserve_llm_b200.engine.step import StepRunner
        self.model = load_model(folder, dtype, "cuda")
        self.layout, self.manager, self.storage = build_cache(self.model, page, pages, caching=False, num_state_slots=slots)
        self.runner = StepRunner(self.model, self.manager, self.storage, cuda_graphs=cuda_graphs, sightings_before_capture=1)
        self.got = {}

    def step(self, parts, end=(), last_only=False):
        from tinyserve_llm_b200.engine.step import StepEntry
        entries = []
        for name, tokens in parts:
            if name in self.manager.seqs:
                self.manager.extend(name, tokens)
            else:
                assert self.manager.admit(name, tokens), f"{name} does not fit"
            entries.append(StepEntry(name, tokens, [len(tokens) - 1] if last_only else list(range(len(tokens)))))
        logits = self.runner.step(entries).cpu().double()
        at = 0
        for e in entries:
            self.manager.commit(e.seq_id, len(e.tokens))
            self.got.setdefault(e.seq_id, []).append(logits[at:at + len(e.want)])
            at += len(e.want)
        for name in end:
            self.manager.release(name)

    def logits(self, name):
        return torch.cat(self.got[name])

    def run(self, name, ids, sizes, end=True, last_only=False):
        pos, k = 0, 0
        while pos < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - pos)
            k += 1
            self.step([(name, ids[pos:pos + n])], end=[name] if end and pos + n == len(ids) else [], last_only=last_only)
            pos += n
        return self.logits(name)


def close(got, want, dtype):
    """
    float32: every position to rounding (the sharp comparison, of every mechanism and every schedule).
    bfloat16 (models in which every expert is used, see `folders`): the error's root mean square against the
    logits' own spread, in the bulk and in the median; one position in a hundred (at least one) may be far off: a
    matrix memory that holds one token reads out sign(k . q) v after its norm, so a first token whose k . q is
    near zero hangs on bfloat16's rounding of the projections.
    """
    if dtype == "float32":
        torch.testing.assert_close(got, want, atol=3e-4, rtol=1e-4)
    else:
        err = (got - want).pow(2).mean(-1).sqrt() / want.std()
        far_off = float((err > 0.12).double().mean())
        assert int((err > 0.4).sum()) <= max(1, err.numel() // 100) and far_off <= 0.03 and float(err.median()) < 0.04, \
            f"relative error: {far_off:.3f} of the positions over 0.12, worst {float(err.max()):.3f} at {int(err.argmax())}, " \
            f"median {float(err.median()):.3f}"


# ---------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_equals_the_plain_model(folders, name, dtype):
    ids = ids_of(CONFIGS[name]["vocab"], 83, 1)
    got = Engine(folders[name, dtype], dtype, page=PAGE[name]).run("a", ids, [len(ids)])
    close(got, plain_logits(name, folders[name, dtype], ids), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prompt_then_token_by_token_and_portions_of_many_sizes(folders, name, dtype):
    """The same logits whether the tokens come at once, one by one after a head, or in portions down to two tokens."""
    ids = ids_of(CONFIGS[name]["vocab"], 120, 2)
    want = plain_logits(name, folders[name, dtype], ids)
    page = PAGE[name]
    decoded = Engine(folders[name, dtype], dtype, page=page).run("a", ids, [30] + [1] * 90)
    close(decoded, want, dtype)
    portions = Engine(folders[name, dtype], dtype, page=page).run("a", ids, [2, 3, 17, 2, 16, 5, 31, 1, 1, 2])   # shorter than the convolution too
    close(portions, want, dtype)
    one_by_one = Engine(folders[name, dtype], dtype, page=page).run("a", ids[:40], [1])      # the first tokens, alone
    close(one_by_one, want[:40], dtype)
    if dtype == "float32":                                                           # the cut changes nothing beyond rounding
        torch.testing.assert_close(decoded, portions, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(folders, dtype, graphs):
    """
    Five requests through three state slots and a pool that holds less than their sum: portions of
    some beside single tokens of others, requests that sit a step out, ended requests whose pages
    and slots the next ones take (a matrix, a running maximum or a convolution's inputs that are not
    zeroed, or a page read through a stale table, show).  With `graphs`, every step is replayed from
    a CUDA graph from its first sighting on.
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
        close(eng.logits(k), plain_logits(name, folders[name, dtype], ids), dtype)
        alone = Engine(folders[name, dtype], dtype, page=16, pages=12, slots=3).run(k, ids, [len(ids)])
        if dtype == "float32":
            torch.testing.assert_close(eng.logits(k), alone, atol=2e-5, rtol=1e-5)


def test_tensor_core_attention_and_grouped_products_also_from_a_graph(folders):
    """
    Pages of 64 tokens and heads of 64 channels: the first layer's attention runs on the tensor-core
    kernels (prompt portions and decoded tokens), and with many (token, expert) pairs the experts'
    bfloat16 products go to the library's grouped product.  Same logits.
    """
    name, dtype = "wide", "bfloat16"
    ids = ids_of(CONFIGS[name]["vocab"], 200, 7)
    eng = Engine(folders[name, dtype], dtype, page=64, pages=8, cuda_graphs=True)
    ops = eng.model.rt.ops
    old, ops.grouped_mm_min_pairs = ops.grouped_mm_min_pairs, 64
    try:
        before = dict(ops.calls)
        got = eng.run("a", ids, [70, 64, 2, 44, 1, 1, 18], last_only=True)
        assert ops.calls.get("library_grouped_mm", 0) > before.get("library_grouped_mm", 0)
        assert ops.calls.get("ts_paged_attention_bf16", 0) + ops.calls.get("ts_prefill_attention_tcgen05", 0) > 0
        assert eng.runner.graph_replays >= 3
    finally:
        ops.grouped_mm_min_pairs = old
    close(got, plain_logits(name, folders[name, dtype], ids)[[69, 133, 135, 179, 180, 181, 199]], dtype)


def test_long_decoding_keeps_its_state(folders):
    """260 tokens one by one after a short head, over several pages."""
    name, dtype = "mixed", "float32"
    ids = ids_of(CONFIGS[name]["vocab"], 260, 3)
    got = Engine(folders[name, dtype], dtype, page=16, pages=18).run("a", ids, [7] + [1] * 253)
    close(got, plain_logits(name, folders[name, dtype], ids), dtype)


# ---------------------------------------------------------------------------------------------- mechanisms alone
def _runtime(dtype):
    from tinyserve_llm_b200.ops import get_ops
    from tinyserve_llm_b200.parts import model  # noqa: F401  (registers the parts)
    from tinyserve_llm_b200.parts.base import Runtime
    return Runtime(dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()), ops=get_ops())


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


def _ctx(ranges):
    """The step context of requests feeding tokens [begin, end) each."""
    positions, seqs, cu = [], [], [0]
    for s, (a, b) in enumerate(ranges):
        positions += list(range(a, b)); seqs += [s] * (b - a); cu.append(cu[-1] + b - a)
    lens = [b - a for a, b in ranges]
    return SimpleNamespace(positions=_i32(positions), seq_of_token=_i32(seqs), cu_q=_i32(cu), ctx_lens=_i32([b for _, b in ranges]),
                           max_q_len=max(lens), min_q_len=min(lens), max_ctx_len=max(b for _, b in ranges),
                           max_decode_ctx_len=max([b for a, b in ranges if b - a == 1], default=0), scratch={},
                           prefill_seqs=_i32([s for s, n in enumerate(lens) if n > 1]), num_tokens=sum(lens), replayed=False,
                           host=SimpleNamespace(cu_q=cu, ctx_lens=[b for _, b in ranges], start=[a for a, _ in ranges]))


class _Slots:
    """A mixer alone on state slots and scattered pages the test owns; requests are fed in steps of given ranges."""

    def __init__(self, mixer, dtype, lens, page=16, slots=(2, 0, 3)):
        from tinyserve_llm_b200.cache.storage import EntryBinding
        self.mixer, self.lens, self.slots = mixer, lens, list(slots)[:len(lens)]
        need = mixer.kv_need()
        state = torch.full((4, max(int(mixer.state_bytes()), 4)), 0, dtype=torch.uint8, device="cuda")
        self.binding = EntryBinding(None, None, 0, 0, page, 0, None, 0, True, -1, state if mixer.state_bytes() else None, None)
        if need is not None:
            pages_of = [-(-n // page) for n in lens]
            num_pages = sum(pages_of) + 3
            order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(4)).tolist()      # scattered pages
            tables, at = [], 0
            for n in pages_of:
                tables.append(order[at:at + n]); at += n
            width = max(len(t) for t in tables)
            vd, vh = need.value_dim or need.head_dim, getattr(need, "value_heads", 0) or need.num_kv_heads
            k = torch.full((num_pages, 1, need.num_kv_heads, page, need.head_dim), float("nan"), dtype=dtype, device="cuda")
            v = torch.full((num_pages, 1, vh, page, vd), float("nan"), dtype=dtype, device="cuda") if need.values else None
            self.table = _i32([t + [-1] * (width - len(t)) for t in tables])
            per_k, per_v = need.num_kv_heads * page * need.head_dim, vh * page * vd
            self.binding = EntryBinding(k, v, per_k, 0, page, num_pages, None, width, True, 0, self.binding.state, None, per_v, 0)

    def step(self, x_of, ranges):
        """x_of[s]: request s's inputs [len, width]; returns the outputs of the fed ranges, request by request."""
        live = [s for s, (a, b) in enumerate(ranges) if b > a]
        ctx = _ctx([ranges[s] for s in live])
        binding = dataclasses.replace(self.binding, state_slots=_i32([self.slots[s] for s in live]))
        if self.binding.k_pool is not None:
            binding.block_table = self.table[torch.tensor(live, device="cuda")].contiguous()
        x = torch.cat([x_of[s][ranges[s][0]:ranges[s][1]] for s in live]).cuda()
        y = self.mixer.forward(x, ctx, binding).cpu().double()
        out, at = {}, 0
        for s in live:
            n = ranges[s][1] - ranges[s][0]
            out[s] = y[at:at + n]; at += n
        return out


def _mixer(spec, dtype, seed, edit=None):
    from tinyserve_llm_b200.parts.base import part_class
    from tinyserve_llm_b200.weights import random_tensors
    cls = part_class("mixer", spec)
    tensors = dict(random_tensors(cls.declare(spec), seed, std=0.15, unit_std=0.25))
    if edit:
        edit(tensors)
    return cls(spec, {k: v.cuda() for k, v in tensors.items()}, _runtime(dtype)), {k: v.double() for k, v in tensors.items()}


def _in_steps(case, x_of, cuts):
    """Feeds every request in the steps `cuts` gives ((begin, end) per request and step); returns whole outputs."""
    got = {s: [] for s in range(len(x_of))}
    for ranges in cuts:
        for s, y in case.step(x_of, ranges).items():
            got[s].append(y)
    return [torch.cat(got[s]) for s in range(len(x_of))]


TOL = {torch.float32: dict(atol=2e-4, rtol=2e-4), torch.bfloat16: dict(atol=0.05, rtol=0.05)}


def rows_close(got, want, dtype):
    """
    float32: element by element.  bfloat16: each row's error against the row's own size, in the median and
    in the bulk; a row in ten may be further off (where a read-out nearly cancels, or a router score is a
    close call, bfloat16's rounding of the projections decides the row).
    """
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, **TOL[dtype])
        return
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-3)
    assert float(err.median()) < 0.03 and float((err > 0.15).double().mean()) <= 0.1, \
        f"rows' relative error: median {float(err.median()):.3f}, {float((err > 0.15).double().mean()):.3f} of them over 0.15"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, rot, scaling", [(4, 2, 24, 40, 16, (4.0, 64, 16.0, 2.0)), (3, 1, 64, 64, 64, None),
                                                                       (5, 5, 12, 20, 4, (2.0, 32, 8.0, 1.0))])
def test_gated_attention_alone(dtype, heads, kv_heads, dim, vdim, rot, scaling):
    """
    The attention mixer against the plain one: biases, the norm over the whole projection, rotation over
    part of a head with and without rescaled frequencies, values of another head size, the output gate;
    two requests of unequal length fed in portions that end inside pages, then token by token.
    """
    from tinyserve_llm_b200.config.spec import GatedAttentionSpec, InlineRotarySpec, YarnScaling
    width = 64
    spec = GatedAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=vdim, scale=0.3,
                              bias=True, qk_norm=True, qk_norm_eps=1e-5, output_gate=True,
                              position=InlineRotarySpec(dims=rot, base=300.0, yarn=YarnScaling(*scaling) if scaling else None))
    mixer, w = _mixer(spec, dtype, 3)
    g = torch.Generator().manual_seed(1)
    lens = [45, 21]
    x_of = [torch.randn(n, width, generator=g).to(dtype) for n in lens]
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.3, "rot": {"dims": rot, "base": 300.0}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    want = [plain.gated_attention(x.double(), w, m, 1e-5) for x in x_of]
    cuts = [[(0, 17), (0, 2)], [(17, 33), (2, 19)], [(33, 34), (19, 20)], [(34, 45), (20, 21)]]
    got = _in_steps(_Slots(mixer, dtype, lens), x_of, cuts)
    for a, b in zip(got, want):
        rows_close(a, b, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key_at_a_page_border_and_the_first_token_sees_itself(dtype):
    """
    One key, hundreds of positions back at a page's last slot, is made to dominate head 0 (its key and every
    query's first channel are scaled up; no rotation, no norm): the queries return its value, as a prompt
    portion and as single tokens; a query before it does not; position 0 returns its own value.
    """
    from tinyserve_llm_b200.config.spec import GatedAttentionSpec
    width, heads, dim, vdim, far = 32, 2, 16, 24, 63
    spec = GatedAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=1, head_dim=dim, value_dim=vdim, scale=1.0)

    def edit(t):
        for name in ("q", "k", "v"):
            t[name] = torch.zeros_like(t[name])
        t["q"][0, 0] = 1.0                      # head 0's first query channel reads input channel 0
        t["k"][0, 1] = 1.0                      # the key's first channel reads input channel 1
        for j in range(vdim):
            t["v"][j, 2 + j % 30] = 1.0

    mixer, w = _mixer(spec, dtype, 5, edit)
    g = torch.Generator().manual_seed(2)
    n = 400
    x = (torch.randn(n, width, generator=g) * 0.1)
    x[:, 0] = 6.0                                # every query asks for a large first key channel
    x[:, 1] = 0.0
    x[far, 1] = 6.0                              # only the far token has it
    x = x.to(dtype)
    case = _Slots(mixer, dtype, [n], page=16)
    got = _in_steps(case, [x], [[(0, 64)], [(64, 390)], *[[(i, i + 1)] for i in range(390, 400)]])[0]
    # the output projection is random: compare through the plain attention with the same tensors instead of reading values
    q = x.double() @ w["q"].T
    k = x.double() @ w["k"].T
    v = x.double() @ w["v"].T
    inner = torch.zeros(n, heads, vdim, dtype=torch.float64)
    for h in range(heads):
        s = (q[:, h * dim:(h + 1) * dim] @ k.T).masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), -float("inf"))
        inner[:, h] = torch.softmax(s, -1) @ v
    want = inner.reshape(n, heads * vdim) @ w["o"].T
    torch.testing.assert_close(got, want, **TOL[dtype])
    weight_on_far = torch.softmax((q[:, :dim] @ k.T).masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), -float("inf")), -1)[:, far]
    assert float(weight_on_far[far:].min()) > 0.99 and float(weight_on_far[:far].max()) == 0.0      # the test's premise


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, taps", [(4, 2, 20, 24, 3), (2, 2, 72, 37, 4), (3, 1, 16, 16, 1), (2, 1, 130, 8, 2)])
def test_gated_delta_rule_alone(dtype, heads, kv_heads, dim, vdim, taps):
    """
    The delta rule against the plain one: two requests in one launch, cut at places that are no multiples
    of the scan's tile and shorter than the convolution (so its carried inputs span several steps), sizes
    that are no multiples of the kernel's own, slots that are not in order.
    """
    from tinyserve_llm_b200.config.spec import GatedDeltaRuleSpec
    width = 64
    spec = GatedDeltaRuleSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, key_dim=dim, value_dim=vdim, conv_taps=taps,
                              q_scale=dim ** -0.5, out_norm_eps=1e-5, decay_rank=6, gate_rank=10)

    def edit(t):
        t["A_log"] = torch.linspace(-4.0, 0.5, heads).to(t["A_log"].dtype)       # from slow decays to fast ones
        t["b"] = t["b"] * 4                                                        # step sizes all over (0, 1)

    mixer, w = _mixer(spec, dtype, 7, edit)
    g = torch.Generator().manual_seed(3)
    lens = [61, 26]
    x_of = [torch.randn(n, width, generator=g).to(dtype) for n in lens]
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}
    want = [plain.gated_delta_rule(x.double(), w, m, 1e-5) for x in x_of]
    cuts = [[(0, 1), (0, 2)], [(1, 2), (2, 3)], [(2, 4), (3, 3)], [(4, 41), (3, 5)], [(41, 42), (5, 26)], [(42, 61), (26, 26)]]
    got = _in_steps(_Slots(mixer, dtype, lens), x_of, cuts)
    for a, b in zip(got, want):
        rows_close(a, b, dtype)


def test_delta_rule_reads_the_first_token_far_later():
    """With decays close to one the first token's write is still read 200 tokens on: a state lost on the way shows."""
    from tinyserve_llm_b200.config.spec import GatedDeltaRuleSpec
    width, H, D, V = 32, 2, 16, 16
    spec = GatedDeltaRuleSpec(hidden_size=width, num_heads=H, num_kv_heads=H, key_dim=D, value_dim=V, conv_taps=2, q_scale=D ** -0.5,
                              decay_rank=4, gate_rank=4)

    def edit(t):
        t["A_log"] = torch.full_like(t["A_log"], -9.0)
        t["dt_bias"] = torch.zeros_like(t["dt_bias"])

    mixer, w = _mixer(spec, torch.float32, 9, edit)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(210, width, generator=g)
    m = {"heads": H, "kv_heads": H, "dim": D, "vdim": V, "conv": 2}
    want = plain.gated_delta_rule(x.double(), w, m, 1e-6)
    other = x.clone()
    other[0] = -other[0]
    assert float((plain.gated_delta_rule(other.double(), w, m, 1e-6)[-1] - want[-1]).abs().max()) > 1e-3      # the premise
    got = _in_steps(_Slots(mixer, torch.float32, [210]), [x], [[(0, 50)], [(50, 203)], *[[(i, i + 1)] for i in range(203, 210)]])[0]
    torch.testing.assert_close(got, want, **TOL[torch.float32])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, dim, vdim, cap", [(3, 24, 40, 10.0), (1, 72, 15, 15.0), (4, 8, 16, 2.0), (2, 200, 33, 30.0)])
def test_matrix_memory_alone(dtype, heads, dim, vdim, cap):
    """
    The matrix memory against the plain one, with gate biases that push the running maximum both ways
    (large input gates: the maximum follows them; strongly negative ones: exp(-m) takes over in the
    denominator), cut at odd places, 70 tokens so that the gates' walk crosses its 32-token groups.
    """
    from tinyserve_llm_b200.config.spec import MatrixLSTMSpec
    width = 64
    spec = MatrixLSTMSpec(hidden_size=width, num_heads=heads, key_dim=dim, value_dim=vdim, q_scale=dim ** -0.5, gate_cap=cap,
                          out_norm_eps=1e-5)

    def edit(t):
        t["i.b"] = torch.linspace(-6.0, 5.0, heads).to(t["i.b"].dtype)
        t["f.b"] = torch.linspace(4.0, -1.0, heads).to(t["f.b"].dtype)
        t["i"] = t["i"] * 6
        t["f"] = t["f"] * 6

    mixer, w = _mixer(spec, dtype, 11, edit)
    g = torch.Generator().manual_seed(5)
    lens = [70, 19]
    x_of = [torch.randn(n, width, generator=g).to(dtype) for n in lens]
    m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}
    want = [plain.mlstm(x.double(), w, m, 1e-5) for x in x_of]
    cuts = [[(0, 1), (0, 2)], [(1, 3), (2, 2)], [(3, 37), (2, 19)], [(37, 38), (19, 19)], [(38, 70), (19, 19)]]
    got = _in_steps(_Slots(mixer, dtype, lens), x_of, cuts)
    for a, b in zip(got, want):
        rows_close(a, b, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parallel_mixer_sums_its_branches_with_their_scales(dtype):
    """Both halves on one input through the fused projections, against scale_l * left + scale_r * right of the plain ones."""
    from tinyserve_llm_b200.config.nipizen import NipizenConfig
    raw = C.MIXED
    spec = NipizenConfig.from_dict(raw).mixer_spec(0)
    mixer, w = _mixer(spec, dtype, 13)
    g = torch.Generator().manual_seed(6)
    lens = [40, 7]
    x_of = [torch.randn(n, raw["width"], generator=g).to(dtype) for n in lens]
    want = [plain.parallel_mixer(x.double(), w, raw["layers"][0]["mixer"], 1e-5) for x in x_of]
    got = _in_steps(_Slots(mixer, dtype, lens), x_of, [[(0, 15), (0, 7)], [(15, 16), (7, 7)], [(16, 40), (7, 7)]])
    for a, b in zip(got, want):
        rows_close(a, b, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_convolution_carries_its_inputs_across_steps(dtype):
    from tinyserve_llm_b200.cache.storage import EntryBinding
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    g = torch.Generator().manual_seed(8)
    C_, K, n = 10, 4, 23
    x = torch.randn(n, C_ + 3, generator=g).to(dtype)                               # a column stretch of a wider tensor
    taps = torch.randn(C_, K, generator=g)
    want = plain.short_conv_silu(x.double()[:, 2:2 + C_], taps.double())
    state = torch.zeros((3, (K - 1) * C_ * 4), dtype=torch.uint8, device="cuda")
    got = []
    for a, b in ((0, 1), (1, 3), (3, 4), (4, 20), (20, 23)):                          # steps shorter than the taps
        binding = EntryBinding(None, None, 0, 0, 16, 0, None, 0, True, -1, state, _i32([1]))
        got.append(ops.short_conv_silu(x.cuda()[a:b, 2:2 + C_], taps.cuda(), _ctx([(a, b)]), binding).cpu().double())
    torch.testing.assert_close(torch.cat(got), want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_layer_norm_kernel(dtype):
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    g = torch.Generator().manual_seed(3)
    T, W, eps = 7, 100, 1e-3
    stream = torch.randn(T, W, generator=g) * 3 + 2.0                                # a mean that matters
    branch = (torch.randn(T, W, generator=g) * 5).to(dtype)
    wo = 1 + torch.randn(W, generator=g) * 0.3
    s = stream.cuda()
    out = ops.stream_norm(branch.cuda(), None, s, wo.cuda(), eps, dtype, centered=True, plain_add=True)
    want_s = stream.double() + branch.double()
    torch.testing.assert_close(s.cpu().double(), want_s, atol=1e-5, rtol=1e-5)       # the stream stays float32 in both dtypes
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.02, rtol=0.01)
    torch.testing.assert_close(out.cpu().double(), plain.layer_norm(want_s, wo.double(), eps), **tol)
    before = s.clone()
    picked = ops.stream_norm(branch.cuda(), None, s, wo.cuda(), eps, dtype, rows=_i32([5, 0]), centered=True, plain_add=True)
    assert torch.equal(s, before)                                                     # with rows, the stream is read only
    torch.testing.assert_close(picked.cpu().double(), plain.layer_norm(want_s[[5, 0]] + branch.double()[[5, 0]], wo.double(), eps), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, top, tokens", [(6, 2, 50), (5, 1, 3), (40, 4, 50), (12, 3, 150)])
def test_routed_experts_with_sigmoid_scores_on_their_inputs(dtype, experts, top, tokens):
    """The routed feed-forward alone: ragged stretches per expert, a few tokens (the weight-streaming kernel), many (the library's)."""
    from tinyserve_llm_b200.config.spec import PlainMLPSpec, RoutedExpertsSpec
    from tinyserve_llm_b200.parts.base import part_class
    from tinyserve_llm_b200.weights import random_tensors
    width, ff = 48, 24
    spec = RoutedExpertsSpec(hidden_size=width, num_experts=experts, top=top, expert=PlainMLPSpec(hidden_size=width, intermediate_size=ff),
                             router_bias_name=None, scoring="sigmoid", weight_on="input")
    cls = part_class("feed_forward", spec)
    tensors = dict(random_tensors(cls.declare(spec), 17, std=0.3))
    if dtype == torch.bfloat16:                                                      # clear choices: see `folders`
        tensors["router"] = (tensors["router"].float() * 0.02 + torch.linspace(-1, 1, experts)[:, None] * (torch.arange(width) == 0)).to(torch.bfloat16)
    part = cls(spec, {k: v.cuda() for k, v in tensors.items()}, _runtime(dtype))
    g = torch.Generator().manual_seed(1)
    x = torch.randn(tokens, width, generator=g).to(dtype)
    if dtype == torch.bfloat16:
        x[:, 0] = torch.linspace(-3, 3, tokens).to(dtype)
    seq_of_token = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    seq_of_token[-2:] = -1                                                           # padding rows of a replayed step
    got = part.forward(x.cuda(), SimpleNamespace(seq_of_token=seq_of_token)).cpu().double()[:tokens - 2]
    want = plain.routed_experts(x.double()[:tokens - 2], {k: v.double() for k, v in tensors.items()},
                                {"router": {"experts": experts, "top": top}})
    rows_close(got, want, dtype)


def test_sigmoid_router_ties_go_to_the_lower_index_and_scores_are_not_renormalised():
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    logits = torch.tensor([[0.0, 2.0, 2.0, -1.0, 2.0, 0.5], [5.0, 1.0, 0.0, 4.0, -3.0, 4.5]], device="cuda")
    chosen, share, offsets, _, _ = ops.moe_route(logits, None, SimpleNamespace(), 2, "sigmoid")
    assert chosen.tolist() == [[1, 2], [0, 5]]
    torch.testing.assert_close(share.cpu(), torch.sigmoid(torch.tensor([[2.0, 2.0], [5.0, 4.5]])))
    assert offsets.tolist() == [0, 1, 2, 3, 3, 3, 4]


# ---------------------------------------------------------------------------------------------- entry points
def test_replay_program_on_a_model_folder(folders, tmp_path):
    """bin/trace_run on a Nipizen folder: portions, a decoded tail, two requests side by side, a reused slot."""
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
        want = {"a": plain_logits(name, folders[name, dtype], a), "b": plain_logits(name, folders[name, dtype], b)}
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
