"""The Nefipel design, written out plainly: one function per mechanism, whole sequences at a time,
no cache, no kernels, nothing shared with the engine. Tensors are torch tensors on the CPU in the
type the caller chooses (float64 for the tests).

A layer is post-norm: x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + ff(x)). Two mixers:
grouped-query attention with projection biases, a per-head RMS norm of queries and keys, a
rotation of part of each head in half-split pairs and a sigmoid gate on the concatenated heads;
and differential attention: two score maps a head over shared values, a rotation in neighbouring
pairs with index-dependent rescaling, the second map subtracted with one learned factor a layer
and the difference brought to unit root mean square. Feed-forwards: relu(gate) * up, dense; or a
mixture of squared-relu experts chosen by corrected softmax scores inside the best groups of
neighbouring experts, some of them "identity experts" that return their input, plus a shared
expert behind a per-token sigmoid gate.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotation_frequencies(base, dims, scaling=None):
    """(frequencies [dims / 2], factor on cos and sin)."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
    index = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(index(fast)), 0), min(math.ceil(index(slow)), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, interleaved):
    """x [tokens, heads, dim]: the first rot['dims'] elements of every head turn by position * f_i,
    element i with i + dims / 2, or 2i with 2i + 1."""
    dims = int(rot["dims"])
    freqs, magnitude = rotation_frequencies(float(rot["base"]), dims, rot.get("scaling"))
    angle = positions.to(x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]
    cos, sin = (angle.cos() * magnitude)[:, None, :], (angle.sin() * magnitude)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * cos - v * sin, v * cos + u * sin
    else:
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2], out[..., dims // 2: dims] = u * cos - v * sin, v * cos + u * sin
    return out


def causal_softmax_attention(q, k, v, scale):
    """q [T, d], k [T, d], v [T, dv] of one head: every position sees itself and all before it."""
    scores = (q @ k.T) * scale
    T = q.shape[0]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def gated_attention(h, w, m, eps):
    """h [T, width]; w: the mixer's tensors by their short names; m: the mixer's config block."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = (h @ w["q"].T + w["q.b"]).view(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, d)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    q, k = rms_norm(q, w["q.norm"], eps), rms_norm(k, w["k.norm"], eps)
    q, k = rotate(q, pos, m["rot"], False), rotate(k, pos, m["rot"], False)
    heads = [causal_softmax_attention(q[:, i], k[:, i // (H // G)], v[:, i // (H // G)], float(m["scale"])) for i in range(H)]
    o = torch.cat(heads, dim=-1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def differential_lambda(w, diff):
    return float(torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + diff)


def differential_attention(h, w, m, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H * 2, d)          # head by head: map 1, map 2
    k = (h @ w["k"].T).view(T, G * 2, d)
    v = (h @ w["v"].T).view(T, G, dv)
    q, k = rms_norm(q, w["q.norm"], eps), rms_norm(k, w["k.norm"], eps)
    q, k = rotate(q, pos, m["rot"], True), rotate(k, pos, m["rot"], True)
    lam = differential_lambda(w, diff)
    heads = []
    for i in range(H):
        g = i // (H // G)
        a1 = causal_softmax_attention(q[:, 2 * i], k[:, 2 * g], v[:, g], float(m["scale"]))
        a2 = causal_softmax_attention(q[:, 2 * i + 1], k[:, 2 * g + 1], v[:, g], float(m["scale"]))
        heads.append(rms_norm(a1 - lam * a2, None, eps) * (1.0 - diff))
    return torch.cat(heads, dim=-1) @ w["o"].T


def dense_feed_forward(h, w):
    return (torch.relu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def squared_relu_expert(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def route(h, w, r):
    """(chosen [T, top] expert ids, weights [T, top]) over the experts and identity experts."""
    total = int(r["experts"]) + int(r.get("identity", 0) or 0)
    top = int(r["top"])
    s = torch.softmax((h @ w["router"].T), dim=-1)
    choice = s + w["correction"]
    groups = r.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = total // count
        best = choice.view(-1, count, per).max(dim=-1).values
        kept = best.topk(keep, dim=-1).indices
        allowed = torch.zeros(h.shape[0], count, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    chosen = choice.topk(top, dim=-1).indices
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)


def expert_feed_forward(h, w, mlp):
    r = mlp["router"]
    experts = int(r["experts"])
    chosen, weights = route(h, w, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, p in zip(chosen[t].tolist(), weights[t]):
            y = h[t] if e >= experts else squared_relu_expert(h[t][None], w[f"e{e}.up"], w[f"e{e}.down"])[0]
            out[t] += p * y
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w["shared.sg"].T)
        out = out + gate * squared_relu_expert(h, w["shared.up"], w["shared.down"])
    return out


def under(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(x, weights, i, entry, eps, alpha):
    w = under(weights, f"l{i}.")
    mix = under(w, "mix.")
    if entry["type"] == "attention":
        y = gated_attention(x, mix, entry["mixer"], eps)
    elif entry["type"] == "attention_2":
        y = differential_attention(x, mix, entry["mixer"], eps)
    else:
        raise ValueError(entry["type"])
    x = rms_norm(alpha * x + y, w["norm1"], eps)
    mlp = entry.get("mlp")
    if mlp is not None:
        ff = under(w, "mlp.")
        y = dense_feed_forward(x, ff) if mlp["kind"] == "dense" else expert_feed_forward(x, ff, mlp)
        x = rms_norm(alpha * x + y, w["norm2"], eps)
    return x


def forward(config, weights, tokens, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one sequence; `streams` (a list) receives the stream after every layer."""
    weights = {k: v.to(dtype) for k, v in weights.items()}
    eps, alpha = float(config["norm"]["eps"]), float(config["postln_alpha"])
    x = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))
    for i, entry in enumerate(config["layers"]):
        x = layer(x, weights, i, entry, eps, alpha)
        if streams is not None:
            streams.append(x)
    return rms_norm(x, weights["final.norm"], eps) @ weights["embed"].T
