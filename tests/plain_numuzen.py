"""A plain, slow implementation of the Numuzen design in float64 on the CPU: whole sequences, no cache,
one function per mechanism, written from the design's equations and sharing no code with the package.

Layer: x += N_b(mixer(N_a(x))), then (if the layer has a feed-forward) x += N_b'(ff(N_a'(x))), where
N(y) = y / sqrt(mean(y^2) + eps) * (1 + w).  Output: logits = E N_final(x) with the embedding table E.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt(y.pow(2).mean(dim=-1, keepdim=True) + eps)


def offset_norm(y: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight lies around zero."""
    return unit_rms(y, eps) * (1.0 + w)


def decay_of(h: torch.Tensor, a1: torch.Tensor, a2: torch.Tensor, bias: torch.Tensor, tau: float) -> torch.Tensor:
    """Per key channel: sigmoid(W_a2 (W_a1 h) + b) ^ (1 / tau)."""
    return torch.sigmoid((h @ a1.T) @ a2.T + bias).pow(1.0 / tau)


def linear_recurrence(q, k, v, a, state=None):
    """One head: q, k, a [T, D]; v [T, V].  S_t = diag(a_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t.
    Returns (o [T, V], the last state)."""
    T, D = q.shape
    V = v.shape[1]
    S = torch.zeros(D, V, dtype=F64) if state is None else state.clone()
    out = torch.zeros(T, V, dtype=F64)
    for t in range(T):
        S = a[t].unsqueeze(1) * S + torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out, S


def gla_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, D) / math.sqrt(D)
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    a = decay_of(h, w[p + "a1"], w[p + "a2"], w[p + "a2.b"], m["tau"]).view(T, H, D)
    heads = []
    for i in range(H):
        o, _ = linear_recurrence(q[:, i], k[:, i], v[:, i], a[:, i])
        heads.append(unit_rms(o, eps) * w[p + "norm"])
    gate = h @ w[p + "g"].T
    return (torch.cat(heads, dim=1) * gate * torch.sigmoid(gate)) @ w[p + "o"].T


def rotation_frequencies(rot: dict) -> tuple:
    """(frequencies of the dims / 2 pairs, the factor on cos and sin)."""
    dims, base = rot["dims"], rot["base"]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    s = rot.get("scaling")
    if not s:
        return f, 1.0

    def where(turns):
        return dims * math.log(s["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(s["fast"])), 0)
    hi = min(math.ceil(where(s["slow"])), dims - 1)
    out = f.clone()
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / s["factor"] * ramp + f[i] * (1 - ramp)
    return out, 0.1 * math.log(s["factor"]) + 1.0


def rotate_heads(x: torch.Tensor, rot: dict | None, first_position: int = 0) -> torch.Tensor:
    """x [T, heads, d]: the first rot.dims entries of every head, entry i paired with i + dims / 2."""
    if not rot:
        return x
    f, mag = rotation_frequencies(rot)
    half = rot["dims"] // 2
    out = x.clone()
    for t in range(x.shape[0]):
        angle = (first_position + t) * f
        c, s = torch.cos(angle) * mag, torch.sin(angle) * mag
        u, v = x[t, :, :half], x[t, :, half:2 * half]
        out[t, :, :half] = u * c - v * s
        out[t, :, half:2 * half] = v * c + u * s
    return out


def sink_softmax_attention(q, k, v, scale, softcap, window):
    """One head, query by query: q [T, d], k [T, d], v [T, dv].  Query i sees the keys j with
    0 <= i - j < window; p_j = exp(s_j) / (1 + sum exp(s_j)) with s = cap(q . k * scale)."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for i in range(T):
        first = 0 if not window else max(0, i - window + 1)
        s = (k[first:i + 1] @ q[i]) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        e = torch.exp(s)
        out[i] = (e / (1.0 + e.sum())) @ v[first:i + 1]
    return out


def attention_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q_raw, k_raw = h @ w[p + "q"].T, h @ w[p + "k"].T
    values = k_raw.view(T, G, d)  # the keys as projected
    q = (unit_rms(q_raw, eps) * w[p + "q.norm"]).view(T, H, d)  # over the whole projection
    k = (unit_rms(k_raw, eps) * w[p + "k.norm"]).view(T, G, d)
    q, k = rotate_heads(q, m.get("rot")), rotate_heads(k, m.get("rot"))
    window = (m.get("mask") or {}).get("size")
    heads = [sink_softmax_attention(q[:, i], k[:, i // (H // G)], values[:, i // (H // G)], m["scale"], m.get("softcap"),
                                    window) for i in range(H)]
    return (torch.cat(heads, dim=1) * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def expert(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(gate @ x, max=limit)
    u = torch.clamp(up @ x, min=-limit, max=limit)
    return down @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def routed_feed_forward(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    """Scores sigmoid(W_router h); the ``top`` largest; out = sum expert_e(score_e * h)."""
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    scores = torch.sigmoid(h @ w[p + "router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(scores.shape[1]), key=lambda e: (-float(scores[t, e]), e))[:top]
        for e in order:
            out[t] += expert(scores[t, e] * h[t], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], limit)
    return out


def forward(cfg: dict, weights: dict, ids, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; ``streams`` receives the stream after every layer."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(ids), dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, w[p + "norm1"], eps)
        mixed = (gla_mixer if layer["type"] == "gla" else attention_mixer)(h, w, p + "mix.", layer["mixer"], eps)
        x = x + offset_norm(mixed, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = offset_norm(x, w[p + "norm2"], eps)
            x = x + offset_norm(routed_feed_forward(h, w, p + "mlp.", layer["mlp"]), w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].T
