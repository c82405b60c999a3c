"""Plain, slow implementation of the Dodonex design: whole sequences, no cache, one
function for each mechanism, float64 by default.  It shares no code with
``torchlet_b200``; every function restates the mechanism's equations.

Notation: T tokens, W width, H heads, D head size.  Weights are a dict of tensor
name -> torch tensor with the checkpoint's names; a configuration is config.json as a
plain dict.  Linear weights are [out, in] and applied as ``x @ w.T``.
"""
from __future__ import annotations

import math

import torch


def gelu_tanh(z):
    """0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))."""
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def group_rms_norm(x, weight, eps, groups):
    """The last axis in ``groups`` equal consecutive parts, each divided by its own root mean
    square; the whole times ``weight``."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    return rms_unit(parts, eps).reshape(shape) * weight


def embed(ids, table, scale):
    return table[ids] * scale


def rotate_half_pairs(x, positions, base, dims):
    """Rotation of the first ``dims`` entries of the last axis: entry i pairs with entry
    i + dims/2; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims).
    x: [T, ..., n] with positions [T]."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]
    while angle.dim() < x.dim():
        angle = angle.unsqueeze(1)
    cos, sin = angle.cos().to(x.dtype), angle.sin().to(x.dtype)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat((u * cos - v * sin, v * cos + u * sin, rest), dim=-1)


def latent_kv(h, w, prefix, mixer, eps, positions):
    """What a latent-attention layer keeps of every token: the normed latent c [T, kv_rank] and
    the rotated key part shared by all heads [T, rot_dim]."""
    rank, rot_dim = mixer["kv_rank"], mixer["rot_dim"]
    down = h @ w[prefix + "dkv"].T
    c = rms_unit(down[:, :rank], eps) * w[prefix + "dkv.norm"]
    k_rot = rotate_half_pairs(down[:, rank:rank + rot_dim], positions, mixer["rot"]["base"], mixer["rot"]["dims"])
    return c, k_rot


def latent_attention(h, w, prefix, mixer, eps, positions, kv):
    """Causal softmax attention whose keys and values are expanded from the latent ``kv`` =
    (c, k_rot) of this or of another layer.  h: [T, W]."""
    H, D, R, V = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"]
    T = h.shape[0]
    c, k_rot = kv
    c_q = rms_unit(h @ w[prefix + "dq"].T, eps) * w[prefix + "dq.norm"]
    q = (c_q @ w[prefix + "uq"].T).reshape(T, H, D + R)
    q_plain = q[..., :D]
    q_rot = rotate_half_pairs(q[..., D:], positions, mixer["rot"]["base"], mixer["rot"]["dims"])
    k_plain = (c @ w[prefix + "uk"].T).reshape(T, H, D)
    value = (c @ w[prefix + "uv"].T).reshape(T, H, V)
    scores = torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_rot, k_rot)
    scores = scores * mixer["scale"]
    visible = positions[None, :] <= positions[:, None]  # [query, key]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shv->thv", weights, value).reshape(T, H * V)
    return out @ w[prefix + "o"].T


def general_delta(h, w, prefix, mixer, eps, state=None):
    """The generalized delta rule, token by token.  state: [H, D, D] (key channel, value
    channel) or None for zeros; returns (output [T, W], final state)."""
    H, D = mixer["heads"], mixer["dim"]
    T = h.shape[0]
    r = (h @ w[prefix + "r"].T).reshape(T, H, D)
    k = (h @ w[prefix + "k"].T).reshape(T, H, D)
    v = (h @ w[prefix + "v"].T).reshape(T, H, D)
    inner = torch.tanh(h @ w[prefix + "w1"].T) @ w[prefix + "w2"].T + w[prefix + "w0"]
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(inner)).reshape(T, H, D)
    remove = torch.sigmoid(h @ w[prefix + "a"].T + w[prefix + "a.b"]).reshape(T, H, D)
    unit = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, D, D, dtype=h.dtype) if state is None else state.clone()
    outs = []
    for t in range(T):
        seen = torch.einsum("hi,hij->hj", unit[t], S)  # u^T S_old
        S = decay[t][:, :, None] * S - (remove[t] * unit[t])[:, :, None] * seen[:, None, :] \
            + k[t][:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hij,hi->hj", S, r[t]))
    o = torch.stack(outs)  # [T, H, D]
    o = rms_unit(o, eps).reshape(T, H * D) * w[prefix + "norm"]
    o = o * torch.sigmoid(h @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T, S


def clamped_glu(h, w, prefix, mlp):
    """g = min(gate, limit), u = clamp(up, -limit, limit); down(g sigmoid(1.702 g) (u + 1))."""
    limit = mlp["limit"]
    g = torch.clamp(h @ w[prefix + "gate"].T, max=limit)
    u = torch.clamp(h @ w[prefix + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[prefix + "down"].T


def token_side(x, ids, w, layer, cfg):
    """The per-layer token input: y = proj(gelu_tanh(gate x) * e), returned as
    y / rms(y) * norm (the caller scales and adds it)."""
    dim = cfg["token_side"]["dim"]
    e = w["side.embed"][ids][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w[f"l{layer}.side.gate"].T) * e
    y = g @ w[f"l{layer}.side.proj"].T
    return rms_unit(y, cfg["norm"]["eps"]) * w[f"l{layer}.side.norm"]


def forward(cfg, w, ids, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.numel()
    positions = torch.arange(T)
    eps, groups, m = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["residual_mult"]
    x = embed(ids, w["embed"], cfg["embedding"]["scale"])
    kept, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, mixer = f"l{i}.", layer["mixer"]
        h = group_rms_norm(x, w[p + "norm1"], eps, groups)
        if layer["type"] == "latent_attention":
            if "kv_from" in mixer and mixer["kv_from"] is not None:
                kv = kept[mixer["kv_from"]]
            else:
                kv = kept[i] = latent_kv(h, w, p + "mix.", mixer, eps, positions)
            mixed = latent_attention(h, w, p + "mix.", mixer, eps, positions, kv)
        elif layer["type"] == "general_delta":
            mixed, _ = general_delta(h, w, p + "mix.", mixer, eps)
        else:
            raise ValueError(layer["type"])
        ff = clamped_glu(h, w, p + "mlp.", layer["mlp"]) if layer.get("mlp") else 0.0
        x = x + m * (mixed + ff)
        if cfg.get("token_side"):
            x = x + m * token_side(x, ids, w, i, cfg)
        streams.append(x)
    xn = group_rms_norm(x, w["final.norm"], eps, groups)
    logits = (xn @ w["embed"].T) * cfg["logit_scale"]
    if return_layers:
        return logits, torch.stack(streams)
    return logits
