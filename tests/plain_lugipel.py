"""
Plain, slow implementation of the Lugipel decoder in float64, one function per mechanism, written
from the design's equations.  It shares no code with the engine: tensors come in as a dict by their
checkpoint names, the configuration as the dict config.json holds.  The recurrence walks token by
token; the attention builds the whole score matrix.

    x_0[t] = embed[token_t] * embedding.scale + sinusoid(t)
    layer:  x <- x + mixer(N1(x));  x <- x + ff(N2(x))        N: x / sqrt(mean(x^2) + eps) * w
    mixer "mingru":     element-wise gated recurrence whose gates read the current token only
    mixer "attention":  windowed grouped-query attention with sigmoid weights and a distance penalty
    ff "dense":  W_down xielu(W_up h)        ff "moe": routed gated experts, some of them the identity
    logits = head . N_final(x)
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64
SINUSOID_BASE = 10000.0
SHARE_EPS = 1e-20


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def sinusoid(positions: torch.Tensor, width: int) -> torch.Tensor:
    """[T, width]: entry 2i is sin(p * base^(-2i/width)), entry 2i + 1 the cosine of the same angle."""
    i = torch.arange((width + 1) // 2, dtype=F64)
    ang = positions.to(F64)[:, None] * SINUSOID_BASE ** (-2.0 * i / width)[None, :]
    out = torch.zeros(positions.shape[0], 2 * i.shape[0], dtype=F64)
    out[:, 0::2] = ang.sin()
    out[:, 1::2] = ang.cos()
    return out[:, :width]


def softplus(x):
    x = torch.as_tensor(x, dtype=F64)
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def min_gru(h: torch.Tensor, w: dict, state: torch.Tensor | None = None, return_state: bool = False):
    """h [T, width]; w: tensors under '<layer>.mix.'.  The state (one number a channel) starts at zero."""
    z = torch.sigmoid(h @ w["z"].T + w["z.b"])
    u = h @ w["x"].T + w["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s = torch.zeros(u.shape[1], dtype=F64) if state is None else state.clone()
    rows = []
    for t in range(h.shape[0]):
        s = (1 - z[t]) * s + z[t] * cand[t]
        rows.append(s)
    y = (torch.stack(rows) * silu(h @ w["g"].T)) @ w["o"].T
    return (y, s) if return_state else y


def head_slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    return 1.0 + coef * torch.log(torch.floor((positions.to(F64) + 1) / every) + 1.0)


def sigmoid_attention(h: torch.Tensor, w: dict, m: dict, eps: float, start: int = 0) -> torch.Tensor:
    """A whole sequence (positions start, start + 1, ...) with nothing before it.  h [T, width]."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    window = int(m["mask"]["size"]) if m.get("mask") is not None else T + start + 1     # no mask: every earlier key
    pos = torch.arange(start, start + T)
    q = rms_norm((h @ w["q"].T).view(T, H, D), w["q.norm"], eps)
    k = rms_norm((h @ w["k"].T).view(T, G, D), w["k.norm"], eps)
    v = (h @ w["v"].T).view(T, G, V)
    if m.get("q_temp") is not None:
        q = q * query_temperature(pos, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))[:, None, None]
    gate = torch.sigmoid(h @ w["g"].T)                                    # [T, H]
    dist = (pos[:, None] - pos[None, :]).to(F64)                          # i - j
    seen = (dist >= 0) & (dist < window)
    slopes = head_slopes(H)
    out = torch.zeros(T, H, V, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(m["scale"]) - slopes[head] * dist
        p = torch.sigmoid(s + w["pb"][head]) * seen
        out[:, head] = (p @ v[:, g]) * gate[:, head:head + 1]
    return out.reshape(T, H * V) @ w["o"].T


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    ap, aq = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def dense_ff(h: torch.Tensor, w: dict) -> torch.Tensor:
    return xielu(h @ w["up"].T, float(w["act"][0]), float(w["act"][1])) @ w["down"].T


def route(h: torch.Tensor, w: dict, r: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """(chosen [T, top] indices among experts + identity, weights [T, top])."""
    total = int(r["experts"]) + int(r.get("identity", 0))
    top = int(r["top"])
    s = torch.softmax(h @ w["router"].T, dim=-1)                         # over all router outputs
    choice = s + w["correction"]
    count, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
    per = total // count
    group_score = choice.view(-1, count, per).max(dim=-1).values
    kept = torch.zeros_like(group_score, dtype=torch.bool)
    kept.scatter_(1, group_score.topk(keep, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(-1, -1, per).reshape(-1, total)
    chosen = choice.masked_fill(~allowed, -math.inf).topk(top, dim=-1).indices
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + SHARE_EPS) * float(r["scale"])


def routed_ff(h: torch.Tensor, w: dict, f: dict) -> torch.Tensor:
    r = f["router"]
    experts = int(r["experts"])
    chosen, weights = route(h, w, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t].tolist(), weights[t]):
            if e >= experts:                                              # an identity expert
                out[t] += c * h[t]
            else:
                pre = f"e{e}."
                out[t] += c * ((silu(h[t] @ w[pre + "gate"].T) * (h[t] @ w[pre + "up"].T)) @ w[pre + "down"].T)
    return out


def _under(w: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False):
    """float64 logits [T, vocab] of one sequence from position 0 (and the stream after every layer)."""
    w = {k: v.to(F64) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    x = w["embed"][torch.tensor(tokens)] * float(config["embedding"]["scale"])
    x = x + sinusoid(torch.arange(T), int(config["width"]))
    streams = []
    for i, layer in enumerate(config["layers"]):
        lw = _under(w, f"l{i}.")
        h = rms_norm(x, lw["norm1"], eps)
        if layer["type"] == "mingru":
            x = x + min_gru(h, _under(lw, "mix."))
        elif layer["type"] == "attention":
            x = x + sigmoid_attention(h, _under(lw, "mix."), layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        f = layer.get("mlp")
        if f is not None:
            h = rms_norm(x, lw["norm2"], eps)
            x = x + (dense_ff(h, _under(lw, "mlp.")) if f["kind"] == "dense" else routed_ff(h, _under(lw, "mlp."), f))
        streams.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
