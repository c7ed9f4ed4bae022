"""Latent attention: causal softmax attention whose keys and values of all heads are made from
one small latent vector per token, so that only the latent and one shared rotated key part are
cached.

With h the mixer's input, H heads, per head `head_dim` unrotated and `rot_dim` rotated query/key
elements, `v_head_dim` value elements and a latent of `kv_rank` elements:

    q = W_q h                      per head [head_dim unrotated | rot_dim rotated]
    d = W_dkv h                    [kv_rank | rot_dim]
    c = rms_norm(d[:kv_rank]) * w  (eps)                 the latent, cached
    r = rotate(d[kv_rank:])                              one rotated key part for all heads, cached
    k_h = W_uk[h] c,  v_h = W_uv[h] c                    never formed for cached tokens
    score_h(i, j) = (q_h . k_h(j) + rotate(qr_h) . r(j)) * scale,  j <= i,  softmax over j
    out = W_o concat_h( sigmoid(W_g h)_h * sum_j p_h(i, j) v_h(j) )

The attention runs in the latent space: the query's unrotated part is multiplied by W_uk[h]^T
once per token, the scores and the weighted sum are taken over the cached latents, and W_uv[h]
is applied to the weighted latent (see csrc/attention_latent.cu). `position` names the rotation
(kind "rope", any scaling; rotary_dim = rot_dim; the angles are formed in float32 in the kernel
from `frequencies()`, cos and sin multiplied by `magnitude()`). `gate` (default true) says
whether the per-head output gate exists. Scores, softmax and the weighted latent are float32 in
both serving types; q, the cache and the gated head outputs are rounded to the serving type.

Tensors: q [H (head_dim + rot_dim), hidden], dkv [kv_rank + rot_dim, hidden], dkv.norm [kv_rank],
uk [H head_dim, kv_rank], uv [H v_head_dim, kv_rank], g [H, hidden], o [hidden, H v_head_dim].
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Mixer, PagedCacheSpec, PositionEncoding, build_position, register_part
from .linear import linear, prepare_weight


class LatentAttention(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, position: Optional[PositionEncoding]):
        super().__init__(spec, hidden_size, position)
        if position is not None:
            raise ConfigError("latent_attention: the rotation is named by the mixer's own `position` parameter")
        self.heads = int(spec["num_heads"])
        self.dim, self.rot = int(spec["head_dim"]), int(spec["rot_dim"])
        self.dv, self.rank = int(spec["v_head_dim"]), int(spec["kv_rank"])
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.window = int(spec.get("window", 0) or 0)
        self.gated = bool(spec.get("gate", True))
        if min(self.heads, self.dim, self.dv, self.rank) <= 0 or self.rot < 2 or self.rot % 2 or self.window < 0:
            raise ConfigError("latent_attention: sizes must be positive and rot_dim even and at least 2")
        if self.rank > 1024 or self.rot > 1024:
            raise ConfigError("latent_attention: kv_rank and rot_dim are at most 1024")
        self.rotation = build_position(spec.get("position"), hidden_size, self.rot)
        if (self.rotation is None or not hasattr(self.rotation, "frequencies") or self.rotation.interleaved
                         or self.rotation.rotary_dim != self.rot):
            raise ConfigError("latent_attention: rot_dim > 0 needs a rotation over all rot_dim elements that gives "
                              "frequencies and pairs element i with i + rot_dim / 2")
        self.freq, self.magnitude = None, 1.0
        self.w_in = self.w_o = self.norm = self.k_up = self.v_up = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, H = self.hidden_size, self.heads
        specs = {"q": WeightSpec((H * (self.dim + self.rot), h)), "dkv": WeightSpec((self.rank + self.rot, h)),
                 "dkv.norm": WeightSpec((self.rank,), init="norm", std=0.1),
                 "uk": WeightSpec((H * self.dim, self.rank), std=0.05), "uv": WeightSpec((H * self.dv, self.rank), std=0.05),
                 "o": WeightSpec((h, H * self.dv))}
        if self.gated:
            specs["g"] = WeightSpec((H, h))
        return specs

    def load(self, tensors, dtype):
        parts = [tensors["q"], tensors["dkv"]]
        if self.gated:
            parts.append(tensors["g"])
        else:                                             # no gate: the projection keeps its layout; nothing reads these rows
            parts.append(torch.zeros((self.heads, self.hidden_size), dtype=parts[0].dtype, device=parts[0].device))
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.w_in = prepare_weight(torch.cat([p.to(common) for p in parts], dim=0).contiguous(), dtype)
        self.w_o = prepare_weight(tensors["o"], dtype)
        self.norm = tensors["dkv.norm"]
        # per head: uk as [dim, rank] (in, out), uv as [dv, rank] read with (in, out) = (rank, dv)
        self.k_up = tensors["uk"].view(self.heads, self.dim, self.rank)
        self.v_up = tensors["uv"].view(self.heads, self.dv, self.rank).transpose(1, 2)

    def setup(self, device, dtype):
        if self.rotation is not None:
            self.freq = self.rotation.frequencies().to(device=device, dtype=torch.float32).contiguous()
            self.magnitude = float(self.rotation.magnitude()) if hasattr(self.rotation, "magnitude") else 1.0

    def first_weight(self):
        return self.w_in

    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(entries=2, heads=1, width=self.rank, window=self.window, widths=(self.rank, self.rot))

    def forward(self, ctx, x, cache, writes_cache: bool = True):
        group = ctx.group(cache.group)
        H, tokens = self.heads, x.shape[0]
        proj = ops.materialize(linear(ctx, x, self.w_in))
        qk = torch.empty((tokens, H, self.rank + self.rot), dtype=proj.dtype, device=proj.device)
        gate = ops.latent_prep(proj, qk, cache.k if writes_cache else None, cache.v if writes_cache else None, self.norm,
                               self.eps, ctx, group.slot_mapping, heads=H, dim=self.dim, rot=self.rot, rank=self.rank,
                               freq=self.freq, magnitude=self.magnitude)
        # the query's unrotated part into the latent space: qk[t, h, :rank] = q[t, h, :dim] @ W_uk[h]
        q_plain = proj[:, : H * (self.dim + self.rot)].view(tokens, H, self.dim + self.rot)[:, :, : self.dim]
        ops.head_project(q_plain, self.k_up, qk[:, :, : self.rank])
        latent = ops.latent_attend(ctx, qk, cache.k, cache.v, group, scale=self.scale, window=self.window)
        heads_out = torch.empty((tokens, H, self.dv), dtype=proj.dtype, device=proj.device)
        ops.head_project(latent, self.v_up, heads_out, gate=gate if self.gated else None)
        return linear(ctx, heads_out.view(tokens, H * self.dv), self.w_o, out_dtype=torch.float32)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
