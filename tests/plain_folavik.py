"""
Plain, slow implementation of the Folavik decoder in float64, one function per mechanism, written
from the design's equations.  It shares no code with the engine: tensors come in as a dict by their
checkpoint names, the configuration as the dict config.json holds.  Every attention builds the
whole score matrix of a sequence.

    x_0[t] = LN(embed[token_t]) w_embed                        LN: (x - mean) / sqrt(var + eps), no bias
    layer:  x <- x + mixer(LN(x) w_1);  x <- x + ff(LN(x) w_2)
    mixer "latent_attention": softmax attention whose keys and values are up-projections of one normed
                              latent a token, no positions, a sigmoid gate on the concatenated heads
    mixer "attention":        grouped-query softmax attention inside chunks of the sequence, rotation over
                              part of a head with frequencies rescaled by wavelength bands
    mixer "attention_2":      the difference of two softmax attentions over the same values inside a sliding
                              window, scores capped by tanh, YaRN rotation, a weightless norm a head
    ff "dense":  W_down (gelu_tanh(W_gate h) * (W_up h))
    logits = cap * tanh(logit_scale * (head . LN(x) w_final) / cap)
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms_norm(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def tanh_cap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(x / cap)


# ---------------------------------------------------------------------- rotation
def plain_frequencies(dims: int, base: float) -> list[float]:
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def band_scaled_frequencies(dims: int, base: float, sc: dict) -> list[float]:
    """Frequencies rescaled by wavelength: short waves kept, long ones slowed by `factor`, a blend between."""
    factor, low, high, original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    out = []
    for f in plain_frequencies(dims, base):
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def yarn_frequencies(dims: int, base: float, sc: dict) -> tuple[list[float], float]:
    """(frequencies, the factor on cos and sin)."""
    factor, original, fast, slow = float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])

    def turns(t: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns(fast)), 0)
    hi = min(math.ceil(turns(slow)), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotation_of(rot: dict | None) -> tuple[int, list[float], float]:
    """(channels rotated, frequencies, factor on cos and sin) of a mixer's `rot` settings."""
    if rot is None:
        return 0, [], 1.0
    dims, base, sc = int(rot["dims"]), float(rot["base"]), rot.get("scaling")
    if sc is None:
        return dims, plain_frequencies(dims, base), 1.0
    if "fast" in sc:
        return (dims,) + yarn_frequencies(dims, base, sc)
    return dims, band_scaled_frequencies(dims, base, sc), 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, freqs: list[float], magnitude: float) -> torch.Tensor:
    """x [T, heads, dim]: channel i < dims/2 is paired with channel i + dims/2; channels from `dims` on pass."""
    if dims == 0:
        return x
    half = dims // 2
    ang = positions.to(F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]
    cs, sn = (ang.cos() * magnitude)[:, None, :], (ang.sin() * magnitude)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cs - v * sn, v * cs + u * sn, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------- masks
def causal_mask(pos: torch.Tensor) -> torch.Tensor:
    return pos[None, :] <= pos[:, None]


def chunk_mask(pos: torch.Tensor, size: int) -> torch.Tensor:
    return causal_mask(pos) & ((pos[None, :] // size) == (pos[:, None] // size))


def window_mask(pos: torch.Tensor, size: int) -> torch.Tensor:
    d = pos[:, None] - pos[None, :]
    return (d >= 0) & (d < size)


def softmax_rows(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    """scores [..., T, T]; every row sees at least itself."""
    s = scores.masked_fill(~visible, -math.inf)
    p = torch.exp(s - s.max(-1, keepdim=True).values)
    return p / p.sum(-1, keepdim=True)


# ---------------------------------------------------------------------- mixers
def latent_attention(h: torch.Tensor, w: dict, m: dict, eps: float, start: int = 0) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(start, start + T)
    q = (h @ w["q"].T).view(T, H, D)
    c = rms_norm(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, V)
    p = softmax_rows(torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"]), causal_mask(pos))
    o = torch.einsum("hij,jhv->ihv", p, v).reshape(T, H * V)
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def chunked_attention(h: torch.Tensor, w: dict, m: dict, eps: float, start: int = 0) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(start, start + T)
    rot = rotation_of(m.get("rot"))
    q = rotate((h @ w["q"].T).view(T, H, D), pos, *rot)
    k = rotate((h @ w["k"].T).view(T, G, D), pos, *rot)
    v = (h @ w["v"].T).view(T, G, V)
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    p = softmax_rows(torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"]), chunk_mask(pos, int(m["mask"]["size"])))
    return torch.einsum("hij,jhv->ihv", p, v).reshape(T, H * V) @ w["o"].T


def difference_weight(w: dict, diff: float) -> float:
    return float(torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + diff)


def differential_attention(h: torch.Tensor, w: dict, m: dict, eps: float, start: int = 0) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff, cap = float(m["diff"]), float(m["softcap"])
    pos = torch.arange(start, start + T)
    rot = rotation_of(m.get("rot"))
    # [T, heads, map, dim]: the two maps of a head lie side by side
    q = rotate((h @ w["q"].T + w["q.b"]).view(T, H * 2, D), pos, *rot).view(T, H, 2, D)
    k = rotate((h @ w["k"].T + w["k.b"]).view(T, G * 2, D), pos, *rot).view(T, G, 2, D)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, V)
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    visible = window_mask(pos, int(m["mask"]["size"]))
    maps = []
    for n in range(2):
        s = tanh_cap(torch.einsum("ihd,jhd->hij", q[:, :, n], k[:, :, n]) * float(m["scale"]), cap)
        maps.append(torch.einsum("hij,jhv->ihv", softmax_rows(s, visible), v))
    o = maps[0] - difference_weight(w, diff) * maps[1]
    o = rms_norm(o, None, eps) * (1.0 - diff)
    return o.reshape(T, H * V) @ w["o"].T


MIXERS = {"latent_attention": latent_attention, "attention": chunked_attention, "attention_2": differential_attention}


def dense_ff(h: torch.Tensor, w: dict) -> torch.Tensor:
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


# ---------------------------------------------------------------------- the model
def _under(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens, return_layers: bool = False):
    """float64 logits [T, vocab] of one sequence from position 0 (and the stream after every layer, [layers, T, width])."""
    eps = float(config["norm"]["eps"])
    t64 = {k: v.to(F64) for k, v in tensors.items()}
    x = layer_norm(t64["embed"][torch.as_tensor(tokens, dtype=torch.long)], t64["embed.norm"], eps)
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](layer_norm(x, t64[p + "norm1"], eps), _under(tensors, p + "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + dense_ff(layer_norm(x, t64[p + "norm2"], eps), _under(tensors, p + "mlp."))
        after.append(x)
    logits = layer_norm(x, t64["final.norm"], eps) @ t64["head"].T * float(config.get("logit_scale", 1.0))
    if config.get("logit_softcap"):
        logits = tanh_cap(logits, float(config["logit_softcap"]))
    return (logits, torch.stack(after)) if return_layers else logits
