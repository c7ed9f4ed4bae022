"""Selective scan (the Mamba mixer): a recurrent mixer with a diagonal state per channel whose
step size, input vector and read-out vector depend on the token.

With h the mixer's input, `inner` channels, `state` states per channel, a convolution of
`conv_taps` taps and a step-size rank `dt_rank`:

    [u | z] = W_in h                               inner each
    x = silu(conv(u) + conv.b)                     causal, per channel, the last tap is the current token's,
                                                   zeros before the start
    [dl | B | C] = W_x x                           dt_rank, state, state
    dt = softplus(W_dt dl + dt.b)                  one per channel
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,   A = -exp(A_log)
    y_c = (sum_n S[c, n] C_n + D_c x_c) * silu(z_c);   out = W_o y

The state slot of a request holds S [inner, state] (float32, zero at admission) and the
convolution's last conv_taps - 1 inputs. B, C, the step sizes before and after the softplus,
the decays and the state are float32 in both serving types; the convolution with its SiLU and
the gated read-out are computed in float32 and rounded to the serving type, since products read
them. W_x is kept as two matrices so that its step-size rows give the serving type (the next
product's operand) and its B | C rows float32.

Tensors: in [2 inner, hidden], conv [inner, taps], conv.b [inner], x [dt_rank + 2 state, inner],
dt [inner, dt_rank], dt.b [inner], A_log [inner, state], D [inner], o [hidden, inner].
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import Mixer, PositionEncoding, StateSpec, register_part
from .linear import linear, prepare_weight


class SelectiveScan(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, position: Optional[PositionEncoding]):
        super().__init__(spec, hidden_size, position)
        self.inner, self.states = int(spec["inner"]), int(spec["state"])
        self.taps, self.dt_rank = int(spec["conv_taps"]), int(spec["dt_rank"])
        if min(self.inner, self.states, self.dt_rank) <= 0 or not 1 <= self.taps <= 64:
            raise ConfigError("selective_scan: inner, state and dt_rank must be positive and conv_taps between 1 and 64")
        if self.states > 128:
            raise ConfigError("selective_scan: at most 128 states per channel")
        self.tail_offset = self.inner * self.states
        self.w_in = self.w_dl = self.w_bc = self.w_dt = self.w_o = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, n, s, r = self.hidden_size, self.inner, self.states, self.dt_rank
        return {"in": WeightSpec((2 * n, h)), "conv": WeightSpec((n, self.taps), std=0.5), "conv.b": WeightSpec((n,), std=0.1),
                "x": WeightSpec((r + 2 * s, n), std=0.05), "dt": WeightSpec((n, r), std=0.2), "dt.b": WeightSpec((n,), std=0.5),
                "A_log": WeightSpec((n, s), std=0.5), "D": WeightSpec((n,), init="norm", std=0.1), "o": WeightSpec((h, n))}

    def load(self, tensors, dtype):
        self.w_in = prepare_weight(tensors["in"], dtype)
        self.w_dl = prepare_weight(tensors["x"][: self.dt_rank].contiguous(), dtype)
        self.w_bc = prepare_weight(tensors["x"][self.dt_rank:].contiguous(), dtype)
        self.w_dt = prepare_weight(tensors["dt"], dtype)
        self.w_o = prepare_weight(tensors["o"], dtype)
        conv = {n: tensors[n] for n in ("conv", "conv.b")}
        if len({t.dtype for t in conv.values()}) > 1:
            conv = {n: t.float() for n, t in conv.items()}
        self.conv_w, self.conv_b = conv["conv"].contiguous(), conv["conv.b"]
        small = {n: tensors[n] for n in ("dt.b", "A_log", "D")}
        if len({t.dtype for t in small.values()}) > 1:
            small = {n: t.float() for n, t in small.items()}
        self.dt_bias, self.a_log, self.d_skip = small["dt.b"], small["A_log"].contiguous(), small["D"]

    def first_weight(self):
        return self.w_in

    def state_spec(self) -> StateSpec:
        size = self.tail_offset + (self.taps - 1) * self.inner
        return StateSpec(((size + 3) // 4 * 4,), torch.float32)

    def forward(self, ctx, x, cache, writes_cache: bool = True):
        if not writes_cache:
            raise ConfigError("selective_scan: a recurrent state cannot be shared between layer runs")
        xz = ops.materialize(linear(ctx, x, self.w_in))
        conv = ops.scan_conv(xz, self.conv_w, self.conv_b, cache.state, self.tail_offset, ctx, inner=self.inner, taps=self.taps)
        low = linear(ctx, conv, self.w_dl)
        bc = linear(ctx, conv, self.w_bc, out_dtype=torch.float32)
        steps = linear(ctx, low, self.w_dt, out_dtype=torch.float32)
        y = ops.scan_run(conv, steps, self.dt_bias, bc, self.a_log, self.d_skip, xz, cache.state, ctx, inner=self.inner,
                         states=self.states)
        return linear(ctx, y, self.w_o, out_dtype=torch.float32)


register_part("mixer", "selective_scan", SelectiveScan, replace=True)
