"""A plain, slow Beralix: one function per mechanism, whole sequences, no cache, no kernels.

It is the oracle of the Beralix tests and shares no code with the engine. Everything is
computed in one floating type (`dtype`, float64 by default) from the weights as stored.
A sequence is a tensor of token ids; positions count from 0.

Notation: T tokens, W the model width, H query heads, G key/value heads.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotation_frequencies(rot: dict):
    """(frequencies [dims / 2], the factor both cos and sin are multiplied by)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns_to_index(t):
        return dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))

    lo = max(math.floor(turns_to_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_to_index(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: dict):
    """x [T, heads, D]: the first rot.dims elements of every head turn, element i with i + dims/2."""
    dims = int(rot["dims"])
    f, magnitude = rotation_frequencies(rot)
    angles = positions.to(x.dtype)[:, None] * torch.tensor(f, dtype=x.dtype)[None, :]     # [T, dims/2]
    cos, sin = (angles.cos() * magnitude)[:, None, :], (angles.sin() * magnitude)[:, None, :]
    u, v, rest = x[..., : dims // 2], x[..., dims // 2: dims], x[..., dims:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], dim=-1)


def softmax_attention(q, k, v, scale, window: int = 0):
    """q [T, H, D], k [T, H, D], v [T, H, Dv]; causal; window > 0: key j is seen when 0 <= i - j < window."""
    T = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window > 0:
        seen = seen & (i - j < window)
    scores = scores.masked_fill(~seen[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v)


def latent_attention(h, p: Dict[str, torch.Tensor], m: dict, eps: float):
    """Keys and values of all heads are made from one small latent per token; one rotated key part
    is shared by the heads; every head's output passes a sigmoid gate computed from h."""
    T = h.shape[0]
    H, D, R, Dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    rot = dict(m["rot"], dims=R)
    positions = torch.arange(T)
    q = (h @ p["q"].T).view(T, H, D + R)
    q_plain, q_turn = q[..., :D], rotate(q[..., D:], positions, rot)
    down = h @ p["dkv"].T
    latent = rms_norm(down[:, :rank], p["dkv.norm"], eps)
    k_turn = rotate(down[:, None, rank:], positions, rot).expand(T, H, R)
    k_plain = (latent @ p["uk"].T).view(T, H, D)
    v = (latent @ p["uv"].T).view(T, H, Dv)
    o = softmax_attention(torch.cat([q_plain, q_turn], -1), torch.cat([k_plain, k_turn], -1), v, float(m["scale"]))
    gate = torch.sigmoid(h @ p["g"].T)                          # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * Dv) @ p["o"].T


def window_attention(h, p, m: dict, v_first: Optional[torch.Tensor], mixes: bool):
    """Grouped-query attention over a sliding window; returns (output, the values it used)."""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    positions = torch.arange(T)
    q = rotate((h @ p["q"].T).view(T, H, D), positions, m["rot"])
    k = rotate((h @ p["k"].T).view(T, G, D), positions, m["rot"])
    v = (h @ p["v"].T).view(T, G, Dv)
    if mixes:
        lam = p["vmix"]
        v = (1 - lam) * v + lam * v_first
    rep = H // G
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    o = softmax_attention(q, k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1), float(m["scale"]), window)
    return o.reshape(T, H * Dv) @ p["o"].T, v


def selective_scan(h, p, m: dict):
    """The Mamba mixer: a short causal convolution, then a diagonal recurrence whose step size,
    input and read-out vectors depend on the token."""
    T = h.shape[0]
    inner, N, taps, rank = int(m["inner"]), int(m["state"]), int(m["conv"]), int(m["dt_rank"])
    xz = h @ p["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    padded = torch.cat([torch.zeros(taps - 1, inner, dtype=h.dtype), x], dim=0)
    conv = sum(padded[j: j + T] * p["conv"][:, j] for j in range(taps)) + p["conv.b"]
    x = silu(conv)
    proj = x @ p["x"].T
    dt = softplus(proj[:, :rank] @ p["dt"].T + p["dt.b"])                   # [T, inner]
    B, C = proj[:, rank: rank + N], proj[:, rank + N:]
    A = -torch.exp(p["A_log"])                                             # [inner, N]
    S = torch.zeros(inner, N, dtype=h.dtype)
    ys = []
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append(S @ C[t] + p["D"] * x[t])
    y = torch.stack(ys) * silu(z)
    return y @ p["o"].T


def gated_feed_forward(h, p):
    return (silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def under(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens, *, dtype=torch.float64,
            streams: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence. `streams`, if given, receives the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    v_first = None
    for i, layer in enumerate(config["layers"]):
        L = under(w, f"l{i}.")
        mix, m = under(L, "mix."), layer["mixer"]
        h = layer_norm(x, L["norm1"], L["norm1.b"], eps)
        if layer["type"] == "latent_attention":
            y = latent_attention(h, mix, m, eps)
        elif layer["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            y, v = window_attention(h, mix, m, v_first, mixes and v_first is not None)
            if mixes and v_first is None:
                v_first = v
        elif layer["type"] == "mamba1":
            y = selective_scan(h, mix, m)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, L["norm1b"], L["norm1b.b"], eps) * L["ls1"]
        if layer.get("mlp") is not None:
            y = gated_feed_forward(layer_norm(x, L["norm2"], L["norm2.b"], eps), under(L, "mlp."))
            x = x + layer_norm(y, L["norm2b"], L["norm2b.b"], eps) * L["ls2"]
        if streams is not None:
            streams.append(x.clone())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
