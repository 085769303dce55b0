"""
Small Lugipel configurations for the tests, as config.json dictionaries.  They differ from one another in
every size and in the order of layers: widths and head counts that are not powers of two, key and value
sizes that differ (and, once, agree), as many key/value heads as query heads and a single one, windows
shorter than a page, longer than every prompt and in between, query temperatures that change every
token and every few tokens, experts with top 1, 2 and 3, with and without identity experts, one group
and several of which one, two or all are kept, a layer without a feed-forward, a model of recurrent
layers only and one of attention layers only.
"""


def mingru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def attention(heads, kv_heads, dim, vdim, scale, window, coef, every):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": window}, "q_temp": {"coef": coef, "every": every}}}


def open_attention(heads, kv_heads, dim, vdim, scale):
    """Neither `mask` nor `q_temp`: every earlier key is seen, the queries keep their length."""
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff, groups=(1, 1), scale=1.0):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "top": top, "scale": scale,
                       "groups": {"count": groups[0], "keep": groups[1]}}}


def model(vocab, width, eps, embedding_scale, layers):
    return {"architecture": "Lugipel", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embedding_scale}, "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}


# every mechanism; odd sizes; a window shorter than a page of 16 and one across several; a layer without a feed-forward
MIXED = model(300, 96, 1e-5, 2.5, [
    (attention(6, 2, 20, 36, 0.25, 11, 0.4, 5), moe(7, 2, 2, 40, groups=(3, 2), scale=1.5)),
    (mingru(72), dense(136)),
    (attention(3, 3, 16, 16, 0.3, 50, 0.2, 1), None),
    (mingru(130), moe(5, 0, 3, 24, groups=(1, 1), scale=0.7)),
    (attention(4, 1, 40, 8, 0.18, 37, 0.0, 7), moe(6, 3, 1, 32, groups=(3, 1), scale=2.0)),
])

# recurrent layers only: the model needs state slots, no page
RECURRENT = model(211, 64, 1e-6, 1.0, [
    (mingru(64), moe(4, 1, 2, 48, groups=(5, 5), scale=1.0)),
    (mingru(200), None),
    (mingru(33), dense(50)),
])

# attention layers only, a window longer than every prompt of the tests, one of a single token and a layer without one
WINDOWS = model(128, 80, 1e-6, 4.0, [
    (attention(5, 5, 24, 12, 0.2, 1000, 0.5, 16), dense(96)),
    (attention(2, 1, 32, 64, 0.15, 1, 0.1, 3), moe(8, 0, 2, 16, groups=(4, 2), scale=3.0)),
    (attention(4, 2, 8, 24, 0.4, 64, 0.3, 64), dense(40)),
    (open_attention(3, 1, 16, 20, 0.22), None),
])

# sizes the bfloat16 kernels for a few tokens and the tensor-core attention take: widths that are multiples of 32,
# keys and values of 64 and of 128 channels a head on pages of 64 tokens, windows across page borders
WIDE = model(512, 128, 1e-6, 2.0, [
    (attention(4, 2, 64, 64, 0.125, 100, 0.3, 32), moe(8, 2, 2, 64, groups=(2, 1), scale=2.0)),
    (mingru(160), dense(192)),
    (attention(6, 2, 128, 128, 0.09, 70, 0.25, 10), moe(6, 0, 3, 32, groups=(2, 2), scale=1.0)),
    (attention(2, 2, 64, 64, 0.11, 300, 0.0, 1), dense(64)),
    (open_attention(4, 1, 64, 64, 0.1), None),
])

WEIGHTS = {"std": 0.08, "unit_std": 0.25}
