"""
Small Folavik configurations for the tests, as config.json dictionaries.  They differ from one another in
every size and in the order of layers: widths and head counts that are not powers of two, key and value
sizes that differ (and, once, agree), as many key/value heads as query heads and a single one, rotation over
a whole head and over a part, with and without rescaled frequencies, windows and chunks shorter than a page
of 16, equal to one, and longer than every prompt, a layer without a feed-forward, logits with and without a
cap, a model of one kind of layer only, and sizes the tensor-core kernels take.
"""


def latent(heads, dim, vdim, kv_rank, scale):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}}


def chunked(heads, kv_heads, dim, vdim, scale, size, dims, base, bands=None):
    """bands: (factor, low, high, original) or None for plain frequencies."""
    rot = {"dims": dims, "base": base}
    if bands:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": size}, "rot": rot}}


def differential(heads, kv_heads, dim, vdim, scale, size, dims, base, diff, softcap, yarn=None):
    """yarn: (factor, original, fast, slow) or None for plain frequencies."""
    rot = {"dims": dims, "base": base}
    if yarn:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                             "mask": {"size": size}, "rot": rot, "diff": diff, "softcap": softcap}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model(vocab, width, eps, logit_scale, logit_softcap, layers):
    out = {"architecture": "Folavik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
           "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}
    if logit_softcap:
        out["logit_softcap"] = logit_softcap
    return out


# every mechanism; odd sizes; a window and a chunk shorter than a page of 16, a chunk of exactly one page and a window
# across several; a layer without a feed-forward
MIXED = model(300, 96, 1e-5, 1.7, 9.0, [
    (chunked(6, 2, 20, 36, 0.25, 11, 12, 5000.0, bands=(4.0, 2.0, 8.0, 64)), dense(136)),
    (latent(5, 24, 20, 40, 0.2), dense(72)),
    (differential(4, 2, 16, 24, 0.3, 37, 6, 900.0, 0.55, 12.0, yarn=(4.0, 64, 16.0, 2.0)), None),
    (chunked(3, 3, 16, 16, 0.3, 16, 16, 300.0), dense(50)),
    (differential(3, 1, 40, 8, 0.18, 9, 40, 20000.0, 0.8, 50.0), dense(64)),
    (latent(2, 48, 56, 24, 0.15), None),
])

# masks longer than every prompt of the tests and of a single token; one head; logits neither scaled nor capped
EDGES = model(128, 80, 1e-6, 1.0, None, [
    (differential(5, 5, 12, 20, 0.4, 1000, 4, 100.0, 0.3, 5.0, yarn=(2.0, 32, 8.0, 1.0)), dense(96)),
    (chunked(2, 1, 32, 64, 0.15, 1, 8, 10000.0), dense(40)),
    (differential(1, 1, 24, 12, 0.2, 1, 24, 700.0, 0.5, 30.0), dense(33)),
    (chunked(4, 4, 8, 8, 0.35, 1000, 8, 50.0, bands=(5.0, 1.0, 3.0, 32)), None),
    (latent(1, 16, 16, 8, 0.25), dense(20)),
])

# latent attention only: one pool of pages that keeps every key, no window group
LATENT = model(211, 64, 1e-5, 0.5, 30.0, [
    (latent(3, 16, 24, 32, 0.25), dense(48)),
    (latent(4, 8, 8, 96, 0.3), None),
])

# sizes the bfloat16 kernels for a few tokens and the tensor-core attention kernels take (widths that are multiples
# of 32, keys and values of 64 channels a head on pages of 64 tokens, a latent of 64 channels); masks that end
# inside pages and inside the kernels' tiles of 64 and 128 keys
WIDE = model(512, 128, 1e-6, 2.0, 20.0, [
    (differential(4, 2, 64, 64, 0.125, 80, 32, 130000.0, 0.45, 25.0, yarn=(3.0, 128, 24.0, 1.5)), dense(192)),
    (chunked(4, 2, 64, 64, 0.15, 96, 64, 300000.0, bands=(6.0, 1.0, 3.0, 128)), dense(128)),
    (latent(4, 32, 48, 64, 0.18), dense(96)),
    (chunked(2, 1, 64, 64, 0.12, 200, 16, 1000.0), None),
    (latent(2, 64, 64, 96, 0.2), dense(64)),
])

# heads of 128 channels for keys and values, three query heads a key/value head
GROUPED = model(257, 128, 1e-5, 1.0, 12.0, [
    (differential(3, 1, 128, 128, 0.09, 70, 64, 10000.0, 0.4, 20.0), dense(64)),
    (chunked(6, 2, 128, 128, 0.08, 130, 128, 100000.0, bands=(2.0, 1.0, 2.0, 64)), dense(96)),
    (latent(3, 128, 128, 160, 0.1), None),
])

# layer sizes that resemble a real model's: heads of 128 channels, a latent of 512, masks of 1,024 tokens across many of the
# kernels' tiles, a width and a feed-forward the tcgen05 product with the gate in its epilogue takes
REAL = model(2048, 1024, 1e-6, 1.0, 30.0, [
    (differential(4, 1, 128, 128, 128 ** -0.5, 1024, 64, 1000000.0, 0.5, 50.0, yarn=(8.0, 512, 32.0, 1.0)), dense(2816)),
    (latent(8, 128, 128, 512, 128 ** -0.5), dense(2816)),
    (chunked(8, 2, 128, 128, 128 ** -0.5, 1024, 64, 500000.0, bands=(8.0, 1.0, 4.0, 1024)), dense(2816)),
])
REAL_WEIGHTS = {"std": 0.03, "unit_std": 0.1}

WEIGHTS = {"std": 0.08, "unit_std": 0.25}
