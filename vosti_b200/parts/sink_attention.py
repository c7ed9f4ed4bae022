"""Grouped-query attention whose key and value heads may differ in width, with additions, each
of them optional and a parameter of the spec:

* `position`: the `PartSpec` of a rotation (kind "rope"); the first `rotary_dim` elements of every
  query and key head turn in pairs (i, i + rotary_dim / 2) by position * frequency, the angle
  formed in float32 in the kernel (no table, no limit on positions);
* `chunk`: instead of a `window`, a query sees only the earlier keys that lie in the same block of
  `chunk` consecutive absolute positions as itself (blocks start at multiples of `chunk`);
* `sink_value`: a constant logit that joins the softmax denominator (0.0: one is added to the sum
  of exponentials), where `sink` is a learned one per head;
* `q_temp_coef`, `q_temp_every`: the query at position p is multiplied by
  1 + coef * ln(floor((p + 1) / every) + 1) (long contexts sharpen their scores);
* `bias_rows`, `bias_far`: a learned table `rel` [rows, heads] is added to the scaled score
  by distance n = i - j: row n below rows // 2, then logarithmic steps,
  min(rows - 1, half + floor(ln(n / half) / ln(far / half) * (rows - half))), which reach the
  last row at distance `far`. The scale does not multiply the bias;
* `sink`: a learned logit per head joins the softmax denominator once, with no key or value;
* `value_mix`: "source" publishes this layer's values of the step's tokens for later layers;
  "mix" replaces its own values by (1 - l) v + l v_source before they are cached, with the learned
  scalar l = `vmix` and v_source the values the source layer made of the same tokens (the source
  runs earlier in the same step; both have the same kv heads and value width). A source layer's
  checkpoint may carry an unused `vmix`.

* `qkv_bias`: the q, k and v projections have biases (`q.b`, `k.b`, `v.b`), added to the float32
  products;
* `head_norm_eps`: every query and key head is divided by its root mean square (eps inside the
  root) and multiplied by a weight of the head's width shared by all heads (`q.norm`, `k.norm`),
  before the rotation;
* a rotation with `interleaved` pairs (2i, 2i + 1) instead of (i, i + rotary_dim / 2);
* `maps` = 2, differential attention: the q projection holds two queries a head and the k projection
  two keys a kv head (head by head: map 1, map 2); each map is a softmax attention of its own over
  the same values, and a head's output is a1 - lambda * a2 with one lambda for the layer,
  exp(lq1 . lk1) - exp(lq2 . lk2) + `diff` (vectors of the head's width), then divided by its root
  mean square over the head's values (`out_norm_eps` inside the root, no weight) and multiplied by
  1 - `diff`;
* `partial_out`: the output projection may come back as unsummed K splits (`ops.PartialSum`) for an
  arrangement whose next kernel adds them (the norm after the sum);
* `out_gate`: the concatenated heads are multiplied element by element by sigmoid(W_g x) (`g`), a
  product of the mixer's own input, before the output projection.

In bfloat16 serving a layer with two maps whose wider head width (of key and value) is one the
tensor-core attention kernels take runs every map as a head of its own on those kernels
("expanded": queries and keys zero-padded to that width, a kv head's values cached once per map,
the q projection's rows reordered so that the query heads of a key head stand together); the
maps are combined by a kernel after them. Such a layer's cache holds 2 * maps * kv heads entries
of that width a token.

With any of these five the projection (q | k | v | g as one product) stays float32 and one kernel
(`ops.qkv_heads`) adds the bias, norms, rotates and stores, rounding once; what follows the softmax is
the attention kernel's last step (`ops.HeadFinish`).

Other parameters: num_heads, num_kv_heads (query head h reads kv head h // (heads / kv_heads)),
head_dim, v_head_dim, scale, window (0: every earlier key). Keys and values live in the paged
cache like those of `Attention`, in two tensors of their own widths.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Mixer, PagedCacheSpec, PositionEncoding, build_position, register_part
from .linear import linear, prepare_weight

LOG2E = 1.4426950408889634


def distance_bucket(n: int, rows: int, far: int) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


class SinkAttention(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, position: Optional[PositionEncoding]):
        super().__init__(spec, hidden_size, position)
        if position is not None:
            raise ConfigError("sink_attention: the rotation is named by the mixer's own `position` parameter")
        self.nq, self.nkv = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.dk, self.dv = int(spec["head_dim"]), int(spec.get("v_head_dim") or spec["head_dim"])
        self.scale = float(spec["scale"])
        self.window = int(spec.get("window", 0) or 0)
        self.temp_coef = float(spec.get("q_temp_coef", 0.0) or 0.0)
        self.temp_every = int(spec.get("q_temp_every", 1) or 1)
        self.bias_rows = int(spec.get("bias_rows", 0) or 0)
        self.bias_far = int(spec.get("bias_far", 0) or 0)
        self.has_sink = bool(spec.get("sink", False))
        self.sink_value = spec.get("sink_value")
        self.chunk = int(spec.get("chunk", 0) or 0)
        self.value_mix = spec.get("value_mix")
        if self.value_mix not in (None, "source", "mix"):
            raise ConfigError("sink_attention: value_mix is 'source' or 'mix'")
        self.mix = 0.0
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        eps = spec.get("head_norm_eps")
        self.head_norm_eps = None if eps is None else float(eps)
        self.maps = int(spec.get("maps", 1) or 1)
        self.diff = float(spec.get("diff", 0.0) or 0.0)
        self.out_norm_eps = float(spec.get("out_norm_eps", 0.0) or 0.0)
        self.out_gate = bool(spec.get("out_gate", False))
        self.lam = 0.0
        self.expanded = 0
        self.partial_out = bool(spec.get("partial_out", False))     # the block's next kernel sums the output product's K splits
        self.b_qkv = self.q_norm = self.k_norm = None
        if self.maps not in (1, 2):
            raise ConfigError("sink_attention: a head has one score map or two")
        self.rotation = build_position(spec.get("position"), hidden_size, self.dk)
        self.freq, self.magnitude = None, 1.0
        if self.has_sink and self.sink_value is not None:
            raise ConfigError("sink_attention: a learned sink or a constant one, not both")
        if self.chunk < 0 or (self.chunk and self.window):
            raise ConfigError("sink_attention: a window or a chunk, not both, and neither negative")
        if self.rotation is not None and not hasattr(self.rotation, "frequencies"):
            raise ConfigError("sink_attention: the rotation must give frequencies")
        # the plain path (qkv_store) or the one with bias, head norms, maps, neighbouring pairs or a gate (qkv_heads)
        self.by_heads = (self.qkv_bias or self.head_norm_eps is not None or self.maps > 1 or self.out_gate
                         or (self.rotation is not None and self.rotation.interleaved))
        if self.by_heads and (self.temp_coef or self.value_mix is not None):
            raise ConfigError("sink_attention: a query temperature or value mixing does not go with bias, head norms, "
                              "maps, neighbouring pairs or an output gate")
        if self.nq <= 0 or self.nkv <= 0 or self.nq % self.nkv:
            raise ConfigError(f"sink_attention: num_heads {self.nq} must be a positive multiple of num_kv_heads {self.nkv}")
        if not 0 < self.dk <= 256 or not 0 < self.dv <= 256:
            raise ConfigError("sink_attention: head widths must be between 1 and 256")
        if self.window < 0 or self.temp_every <= 0:
            raise ConfigError("sink_attention: window must be >= 0 and q_temp_every positive")
        if self.bias_rows and (self.bias_rows < 2 or self.bias_far <= self.bias_rows // 2):
            raise ConfigError("sink_attention: the bias table needs at least two rows and bias_far beyond half of them")
        self.w_qkv = self.w_o = self.rel = self.sink = self.bias_table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, nq, nkv, dk, dv = self.hidden_size, self.nq, self.nkv, self.dk, self.dv
        m = self.maps
        specs = {"q": WeightSpec((nq * m * dk, h)), "k": WeightSpec((nkv * m * dk, h)), "v": WeightSpec((nkv * dv, h)),
                 "o": WeightSpec((h, nq * dv))}
        if self.qkv_bias:
            specs.update({"q.b": WeightSpec((nq * m * dk,), std=0.1), "k.b": WeightSpec((nkv * m * dk,), std=0.1),
                          "v.b": WeightSpec((nkv * dv,), std=0.1)})
        if self.head_norm_eps is not None:
            specs.update({"q.norm": WeightSpec((dk,), init="norm", std=0.1), "k.norm": WeightSpec((dk,), init="norm", std=0.1)})
        if m == 2:
            specs.update({name: WeightSpec((dk,), std=0.1) for name in ("lq1", "lk1", "lq2", "lk2")})
        if self.out_gate:
            specs["g"] = WeightSpec((nq * dv, h))
        if self.bias_rows:
            specs["rel"] = WeightSpec((self.bias_rows, nq), std=1.0)
        if self.has_sink:
            specs["sink"] = WeightSpec((nq,), std=1.0)
        if self.value_mix is not None:
            specs["vmix"] = WeightSpec((), std=0.3, optional=self.value_mix == "source")
        return specs

    def load(self, tensors, dtype):
        wide = max(self.dk, self.dv)
        self.expanded = wide if (self.maps > 1 and ops.attention_heads_supported(dtype, wide, self.nq // self.nkv)
                                 and not self.has_sink and self.sink_value is None and not self.bias_rows) else 0
        q_rows, q_bias = tensors["q"], tensors.get("q.b")
        if self.expanded:
            # query heads in the order (kv head, map, head within the kv head's group)
            r = self.nq // self.nkv
            order = torch.tensor([(g * r + j) * self.maps + m for g in range(self.nkv) for m in range(self.maps) for j in range(r)],
                                 device=q_rows.device)
            q_rows = q_rows.view(self.nq * self.maps, self.dk, -1)[order].reshape(q_rows.shape)
            if q_bias is not None:
                q_bias = q_bias.view(self.nq * self.maps, self.dk)[order].reshape(-1)
        parts = [q_rows, tensors["k"], tensors["v"]] + ([tensors["g"]] if self.out_gate else [])
        if self.qkv_bias:
            self.b_qkv = torch.cat([q_bias.float(), tensors["k.b"].float(), tensors["v.b"].float()]).contiguous()
        if self.head_norm_eps is not None:
            self.q_norm, self.k_norm = tensors["q.norm"].float().contiguous(), tensors["k.norm"].float().contiguous()
        if self.maps == 2:
            # one number for the layer, formed in float32
            lq1, lk1, lq2, lk2 = (tensors[name].float() for name in ("lq1", "lk1", "lq2", "lk2"))
            self.lam = float((torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum())).item()) + self.diff
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.w_qkv = prepare_weight(torch.cat([p.to(common) for p in parts], dim=0).contiguous(), dtype)
        self.w_o = prepare_weight(tensors["o"], dtype)
        self.sink = tensors["sink"].float().contiguous() if self.has_sink else None
        if self.value_mix == "mix":
            self.mix = float(tensors["vmix"].float().item())
        if self.bias_rows:
            # by distance, up to the first one that reaches the table's last row: [heads, distances],
            # in base-2 units because the kernels' softmax runs in base 2
            rel = tensors["rel"].float()
            rows = []
            for n in range(self.bias_far + 1):
                rows.append(distance_bucket(n, self.bias_rows, self.bias_far))
                if rows[-1] == self.bias_rows - 1:
                    break
            index = torch.tensor(rows, dtype=torch.long, device=rel.device)
            self.bias_table = (rel[index].T * LOG2E).contiguous()

    def setup(self, device, dtype):
        if self.rotation is not None:
            self.freq = self.rotation.frequencies().to(device=device, dtype=torch.float32).contiguous()
            self.magnitude = float(self.rotation.magnitude()) if hasattr(self.rotation, "magnitude") else 1.0
        if self.sink_value is not None:
            self.sink = torch.full((self.nq,), float(self.sink_value), dtype=torch.float32, device=device)

    def first_weight(self):
        return self.w_qkv

    def cache_spec(self) -> PagedCacheSpec:
        if getattr(self, "expanded", 0):
            return PagedCacheSpec(entries=2, heads=self.nkv * self.maps, width=self.expanded, window=self.window)
        # with maps, a kv head's entry holds its keys of all maps side by side
        return PagedCacheSpec(entries=2, heads=self.nkv, width=self.maps * self.dk, window=self.window,
                              widths=(self.maps * self.dk, self.dv))

    def _forward_by_heads(self, ctx, x, cache, writes_cache, group):
        proj = linear(ctx, x, self.w_qkv, out_dtype=torch.float32, allow_partial=True)   # K splits are summed by qkv_heads
        rotation = self.rotation
        width = (self.nq + self.nkv) * self.maps * self.dk + self.nkv * self.dv
        q = ops.qkv_heads(proj, cache.k if writes_cache else None, cache.v if writes_cache else None, nq=self.nq, nkv=self.nkv,
                          maps=self.maps, dk=self.dk, dv=self.dv, page_size=group.page_size, positions=ctx.positions,
                          slot_mapping=group.slot_mapping, out_dtype=ctx.dtype, status=ctx.status, bias=self.b_qkv,
                          q_norm=self.q_norm, k_norm=self.k_norm, eps=self.head_norm_eps or 0.0, freq=self.freq,
                          interleaved=bool(rotation is not None and rotation.interleaved), magnitude=self.magnitude,
                          expanded_width=self.expanded)
        if isinstance(proj, ops.PartialSum):
            q, gate = q
        else:
            gate = proj[:, width:] if self.out_gate else None
        if self.expanded:
            D, m = self.expanded, self.maps
            each = ops.attention_sink(ctx, q, cache.k, cache.v, group, nq=self.nq * m, nkv=self.nkv * m, dk=D, dv=D,
                                      scale=self.scale, window=self.window, bias=None, sink=None, chunk=self.chunk)
            finish = ops.HeadFinish(lam=self.lam, unit_norm=True, eps=self.out_norm_eps, out_scale=1.0 - self.diff, gate=gate)
            attn = ops.head_finish(each, finish, nq=self.nq, maps=m, dv=self.dv, in_width=D, pair_group=self.nq // self.nkv)
            return linear(ctx, attn, self.w_o, out_dtype=torch.float32, allow_partial=self.partial_out)
        finish = None
        if self.maps == 2 or self.out_gate:
            finish = ops.HeadFinish(lam=self.lam, unit_norm=self.maps == 2, eps=self.out_norm_eps, out_scale=1.0 - self.diff,
                                    gate=gate)
        attn = ops.attention_sink(ctx, q, cache.k, cache.v, group, nq=self.nq, nkv=self.nkv, dk=self.dk, dv=self.dv,
                                  scale=self.scale, window=self.window, bias=self.bias_table, sink=self.sink, chunk=self.chunk,
                                  maps=self.maps, finish=finish)
        return linear(ctx, attn, self.w_o, out_dtype=torch.float32, allow_partial=self.partial_out)

    def forward(self, ctx, x, cache, writes_cache: bool = True):
        group = ctx.group(cache.group)
        if self.by_heads:
            return self._forward_by_heads(ctx, x, cache, writes_cache, group)
        qkv = ops.materialize(linear(ctx, x, self.w_qkv))
        v_source = None
        if self.value_mix == "source":
            ctx.extras["value_mix.source"] = qkv[:, self.nq * self.dk + self.nkv * self.dk:]
        elif self.value_mix == "mix":
            v_source = ctx.extras.get("value_mix.source")
            if v_source is None:
                raise ConfigError("sink_attention: a layer mixes values in, but no source layer ran before it in this step")
        q = ops.qkv_store(qkv, cache.k if writes_cache else None, cache.v if writes_cache else None, nq=self.nq,
                          nkv=self.nkv, dk=self.dk, dv=self.dv, page_size=group.page_size, positions=ctx.positions,
                          slot_mapping=group.slot_mapping, temp_coef=self.temp_coef, temp_every=self.temp_every,
                          status=ctx.status, freq=self.freq, magnitude=self.magnitude, v_first=v_source, v_mix=self.mix)
        attn = ops.attention_sink(ctx, q, cache.k, cache.v, group, nq=self.nq, nkv=self.nkv, dk=self.dk, dv=self.dv,
                                  scale=self.scale, window=self.window, bias=self.bias_table, sink=self.sink, chunk=self.chunk)
        return linear(ctx, attn, self.w_o, out_dtype=torch.float32)


register_part("mixer", "sink_attention", SinkAttention, replace=True)
