"""
Prefill and decode throughput of a design at layer sizes that resemble a real model's, beside the
engine's closest other design at equal width and depth (Duduvik beside Llama, Nipizen beside
Duduvik, Lugipel beside Nipizen, Folavik beside Llama), both with random weights through the engine's own step function:

    python bench.py --design duduvik|nipizen|lugipel|folavik [--size small|medium|large] [--steps K] [--warmup W]

For each design: a prompt of `prefill` tokens in one step (launched kernel by kernel), and decode
steps of `batch` requests at `context` tokens each (replayed from a CUDA graph), timed on the device
with CUDA events after warm-up; between timed steps a buffer larger than L2 is written.  One JSON
line per design goes to standard output, then one line with the kernels of the named design's prefill
step and of a decode step by their share of the device time (torch.profiler, a run of its own, not timed).
"""

from __future__ import annotations

import json
import os
import tempfile

SIZES = {
    # width, layers, heads, ff, experts, expert ff, prefill tokens, decode batch, decode context
    "small": dict(width=1024, layers=4, heads=8, ff=4096, experts=16, expert_ff=512, prefill=2048, batch=8, context=2048),
    "medium": dict(width=2048, layers=6, heads=16, ff=8192, experts=32, expert_ff=1024, prefill=2048, batch=8, context=2048),
    "large": dict(width=4096, layers=6, heads=32, ff=14336, experts=64, expert_ff=2048, prefill=4096, batch=16, context=4096),
}
VOCAB = 32768
PAGE = 64


def duduvik_config(s: dict) -> dict:
    """Layers in the order attention / gated linear attention / retention, feed-forwards alternating dense and routed."""
    width, heads = s["width"], s["heads"]
    dim = width // heads                                   # 128 at every size
    att = {"type": "latent_attention",
           "mixer": {"heads": heads, "dim": dim, "rot_dim": dim // 2, "vdim": dim, "q_rank": 3 * width // 4, "kv_rank": 512,
                     "mask": {"size": 1024}, "scale": (dim + dim // 2) ** -0.5, "rot": {"base": 10000.0, "dims": dim // 2}}}
    gla = {"type": "gla", "mixer": {"heads": heads // 2, "dim": dim, "vdim": 2 * dim, "tau": 16.0, "decay_rank": 16}}
    ret = {"type": "retention", "mixer": {"heads": heads // 2, "dim": dim, "vdim": 2 * dim,
                                          "decay": [1.0 - 2.0 ** (-5 - i % 4) for i in range(heads // 2)],
                                          "rot": {"base": 10000.0, "dims": dim}}}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": 4}, "expert": {"ff": s["expert_ff"], "limit": 7.0},
           "shared": {"ff": 2 * s["expert_ff"], "limit": 7.0}}
    mixers, ffs = (att, gla, ret), (dense, moe)
    layers = [dict(mixers[i % 3], mlp=ffs[i % 2]) for i in range(s["layers"])]
    return {"architecture": "Duduvik", "vocab": VOCAB, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": layers}


def nipizen_config(s: dict) -> dict:
    """
    Layers in the order parallel (attention beside a gated delta rule) / matrix memory / parallel, every one
    with routed experts (top 4).  Attention heads of 128 channels for keys and values, so that the
    tensor-core attention kernels take them; recurrent heads of 128 key channels.
    """
    width, heads = s["width"], s["heads"]
    dim = width // heads                                   # 128 at every size
    par = {"type": "parallel",
           "mixer": {"left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                              "rot": {"base": 10000.0, "dims": dim // 2,
                                      "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
                     "right": {"heads": heads // 2, "kv_heads": max(1, heads // 4), "dim": dim, "vdim": dim, "conv": 4,
                               "decay_rank": 16, "gate_rank": 16},
                     "left_scale": 0.7, "right_scale": 0.7}}
    mem = {"type": "mlstm", "mixer": {"heads": heads // 2, "dim": dim, "vdim": 2 * dim, "gate_cap": 15.0}}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": 4}, "expert": {"ff": s["expert_ff"]}}
    mixers = (par, mem, par)
    return {"architecture": "Nipizen", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6},
            "layers": [dict(mixers[i % 3], mlp=moe) for i in range(s["layers"])]}


def lugipel_config(s: dict) -> dict:
    """
    Layers in the order attention / minGRU / attention; routed experts (top 4 of `experts` and two identity
    experts, the best two of four groups) behind the attention layers, a dense xIELU layer behind the recurrent
    ones.  Attention heads of 128 channels for keys and values, 4 query heads a key/value head, a window of
    1,024 tokens; the recurrence is twice as wide as the stream.
    """
    width, heads = s["width"], s["heads"]
    dim = width // heads                                   # 128 at every size
    att = {"type": "attention",
           "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                     "mask": {"size": 1024}, "q_temp": {"coef": 0.1, "every": 128}}}
    gru = {"type": "mingru", "mixer": {"width": 2 * width}}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]},
           "router": {"experts": s["experts"] - 2, "identity": 2, "top": 4, "scale": 2.0, "groups": {"count": 4, "keep": 2}}}
    dense = {"kind": "dense", "ff": s["ff"]}
    layers = [dict(gru, mlp=dense) if i % 3 == 1 else dict(att, mlp=moe) for i in range(s["layers"])]
    return {"architecture": "Lugipel", "vocab": VOCAB, "width": width, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
            "layers": layers}


def folavik_config(s: dict) -> dict:
    """
    Layers in the order differential attention / latent attention / chunked attention, every one with a dense
    gelu-gated feed-forward of the Llama model's width.  Heads of 128 channels for keys and values, so that the
    tensor-core attention kernels take them: the chunked layers with 4 query heads a key/value head, chunks of
    1,024 tokens and rotation over half a head; the differential layers with half as many heads of two maps each
    (as many score maps as the other layers have heads), a window of 1,024 tokens, scores capped at 50; the latent
    layers with a latent of 512 channels.
    """
    width, heads = s["width"], s["heads"]
    dim = width // heads                                   # 128 at every size
    diff = {"type": "attention_2",
            "mixer": {"heads": heads // 2, "kv_heads": max(1, heads // 8), "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                      "mask": {"size": 1024}, "softcap": 50.0, "diff": 0.5,
                      "rot": {"base": 1000000.0, "dims": dim // 2,
                              "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}}
    lat = {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": 512, "scale": dim ** -0.5}}
    att = {"type": "attention",
           "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                     "mask": {"size": 1024},
                     "rot": {"base": 500000.0, "dims": dim // 2,
                             "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    dense = {"kind": "dense", "ff": s["ff"]}
    mixers = (diff, lat, att)
    return {"architecture": "Folavik", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "logit_softcap": 30.0, "layers": [dict(mixers[i % 3], mlp=dense) for i in range(s["layers"])]}


def llama_config(s: dict) -> dict:
    width, heads = s["width"], s["heads"]
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": VOCAB, "hidden_size": width,
            "intermediate_size": s["ff"], "num_hidden_layers": s["layers"], "num_attention_heads": heads,
            "num_key_value_heads": max(1, heads // 4), "head_dim": width // heads, "hidden_act": "silu", "rms_norm_eps": 1e-6,
            "rope_theta": 10000.0, "max_position_embeddings": 16384, "tie_word_embeddings": True}


def measure(cfg: dict, s: dict, steps: int, warmup: int, profile: bool) -> dict:
    import torch

    from tinyserve_llm_b200.engine.loading import build_cache, load_model
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner

    folder = tempfile.mkdtemp(prefix="design_bench_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    model = load_model(folder, "bfloat16", "cuda", random_weights_seed=0)
    weights = sum(t.numel() * t.element_size() for t in _tensors(model))
    per_request = -(-(s["context"] + steps + warmup + 8) // PAGE) + 1
    pages = max(s["batch"] * per_request, -(-s["prefill"] // PAGE) + 1) + 4
    _, manager, storage = build_cache(model, PAGE, pages, caching=False, num_state_slots=s["batch"] + 1)
    runner = StepRunner(model, manager, storage, max_decode_batch=s["batch"])
    ops = model.rt.ops
    gen = torch.Generator().manual_seed(0)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")         # larger than the 126 MB L2

    def timed(fn, k, w):
        for _ in range(w):
            fn()
        times = []
        for _ in range(k):
            flush.fill_(1)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end))
        times.sort()
        return times[len(times) // 2]

    def kernel_shares(fn):
        from torch.profiler import ProfilerActivity, profile as torch_profile
        fn()
        torch.cuda.synchronize()
        with torch_profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        rows = sorted(((e.key, e.device_time_total, e.count) for e in prof.key_averages() if e.device_time_total > 0),
                      key=lambda r: -r[1])
        total = sum(r[1] for r in rows) or 1.0
        return [{"kernel": k[:70], "us": round(us, 1), "calls": n, "share": round(us / total, 3)} for k, us, n in rows[:14]]

    # ---- prefill: one prompt in one step
    prompt = torch.randint(0, VOCAB, (s["prefill"],), generator=gen).tolist()

    def prefill():
        assert manager.admit("p", prompt)
        runner.step([StepEntry("p", prompt, [len(prompt) - 1])])
        manager.commit("p", len(prompt))
        manager.release("p")

    before = ops.launches
    prefill()
    prefill_launches = ops.launches - before
    prefill_ms = timed(prefill, max(3, min(steps, 10)), max(warmup, 3))
    out = {"prefill_tokens": s["prefill"], "prefill_ms": round(prefill_ms, 3),
           "prefill_tokens_per_s": round(s["prefill"] / prefill_ms * 1e3), "prefill_launches": prefill_launches}
    if profile:
        out["prefill_kernels"] = kernel_shares(prefill)

    # ---- decode: `batch` requests at `context` tokens, one token each a step
    names = [f"d{i}" for i in range(s["batch"])]
    for name in names:
        tokens = torch.randint(0, VOCAB, (s["context"],), generator=gen).tolist()
        for at in range(0, len(tokens), 2048):
            part = tokens[at:at + 2048]
            assert manager.admit(name, part) if at == 0 else manager.extend(name, part) is None
            runner.step([StepEntry(name, part, [])])
            manager.commit(name, len(part))

    def decode():
        entries = []
        for i, name in enumerate(names):
            manager.extend(name, [i + 1])
            entries.append(StepEntry(name, [i + 1], [0]))
        runner.step(entries)
        for name in names:
            manager.commit(name, 1)

    decode_ms = timed(decode, steps, max(warmup, 3))
    state = sum(b for _, b in model.cache_needs()) * s["batch"]
    out.update({"decode_batch": s["batch"], "decode_context": s["context"], "decode_ms_per_step": round(decode_ms, 4),
                "decode_tokens_per_s": round(s["batch"] / decode_ms * 1e3), "weight_bytes": weights,
                "state_bytes_per_step": 2 * state, "graph_replays": runner.graph_replays})
    if profile:
        out["decode_kernels"] = kernel_shares(decode)
    for name in names:
        manager.release(name)
    return out


def _tensors(model):
    import torch
    seen, stack = [], [model]
    ids = set()
    while stack:
        node = stack.pop()
        if isinstance(node, torch.Tensor):
            if node.is_cuda and node.data_ptr() not in ids:
                ids.add(node.data_ptr())
                seen.append(node)
        elif isinstance(node, (list, tuple)):
            stack.extend(node)
        elif isinstance(node, dict):
            stack.extend(v for k, v in node.items() if k != "shared")
        elif hasattr(node, "__dict__") and type(node).__module__.startswith("tinyserve_llm_b200.parts"):
            stack.extend(v for k, v in vars(node).items() if k not in ("rt", "spec"))
    return seen


def run(design: str, size: str, steps: int, warmup: int, peaks: dict) -> int:
    s = SIZES[size]
    if design == "duduvik":
        pair = (("llama", llama_config(s), False), ("duduvik", duduvik_config(s), True))
    elif design == "nipizen":
        pair = (("duduvik", duduvik_config(s), True), ("nipizen", nipizen_config(s), True))
    elif design == "lugipel":
        pair = (("nipizen", nipizen_config(s), True), ("lugipel", lugipel_config(s), True))
    elif design == "folavik":
        pair = (("llama", llama_config(s), True), ("folavik", folavik_config(s), True))
    else:
        raise SystemExit(f"--design {design!r}: have ['duduvik', 'nipizen', 'lugipel', 'folavik']")
    for name, cfg, profile in pair:
        record = {"design": name, "size": size, "width": s["width"], "layers": s["layers"], "dtype": "bf16",
                  "data": "synthetic", "timing": "CUDA events, median, L2 flushed between timed steps", "peaks": peaks}
        record.update(measure(cfg, s, steps, warmup, profile))
        kernels = {k: record.pop(k) for k in ("prefill_kernels", "decode_kernels") if k in record}
        print(json.dumps(record), flush=True)
        if kernels:
            print(json.dumps({"design": name, "size": size, **kernels}), flush=True)
    return 0
