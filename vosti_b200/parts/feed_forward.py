"""Gated feed-forward with SiLU: down( silu(gate(x)) * up(x) ).

gate and up are one [2I, hidden] matrix (gate rows first) so that the projection is a
single product, as the reference's loader concatenates them
(python/vosti_kernels/model_families/qwen3/loader.py:55-58); the activation is
gate * sigmoid(gate) * up in float32 (kernels/triton_kernels/silu_mul.py:66-87).

Parameters besides `intermediate_size`: `tensor_names`, the checkpoint's names of the gate, up
and down matrices (default: Qwen3's), `float32_out`, for models whose residual stream is
float32: the down projection is then not rounded to the serving type, and `activation`: "silu"
(the default), "relu" or "relu2" (the square of relu) on the gate.

`ExpertMixture` is the same feed-forward as `experts` small ones, of which each token uses
the `top` with the largest router logits, weighted by the softmax over the chosen logits only.
Its experts may also be plain two-matrix feed-forwards, down(gelu(up(x))) with the exact (erf)
GELU, and its weights the chosen experts' shares of a softmax over all experts, divided by
their sum and multiplied by a constant. A third way of routing ("scored") chooses by corrected
softmax scores inside the best groups of experts, may count experts that return their input
among the routed ones, and may add a shared expert behind a per-token gate (see the class).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import ConfigError, PartSpec
from ..weights.loader import WeightSpec
from .base import FeedForward, register_part
from .linear import linear, prepare_weight, uses_tensor_cores


def stack_gate_up(gate: torch.Tensor, up: torch.Tensor, dtype: torch.dtype, activation: str = "silu"):
    """One [2I, hidden] matrix for the gate and up projections, and whether SiLU(gate)*up can be
    the tensor-core product's epilogue. If so, rows are laid out as blocks of 16 gate rows
    followed by their 16 up rows, so that both halves of an output land in one warp's slice of
    the accumulator; else the gate rows come first."""
    inter = gate.shape[0]
    common = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
    stacked = torch.cat([gate.to(common), up.to(common)], dim=0)
    fused = (dtype == torch.bfloat16 and inter % 16 == 0 and uses_tensor_cores(dtype, stacked)
             and activation in ops.FUSED_GLU_ACTIVATIONS)
    if not fused:
        return stacked.contiguous(), False
    h = stacked.shape[1]
    blocks = torch.stack([stacked[:inter].view(-1, 16, h), stacked[inter:].view(-1, 16, h)], dim=1)
    return prepare_weight(blocks.reshape(2 * inter, h).contiguous(), dtype), True


def gated_activation(ctx, x, w_gate_up, fused: bool, activation: str = "silu"):
    if fused:
        return ops.gemm_tc(ops.materialize(x), w_gate_up, ctx.status, swiglu=True, activation=activation)
    return ops.glu_mul(ops.materialize(linear(ctx, x, w_gate_up)), activation)


class SwiGLU(FeedForward):
    def __init__(self, spec: PartSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        self.inter = int(spec["intermediate_size"])
        if self.inter <= 0:
            raise ConfigError("swiglu: intermediate_size must be positive")
        self.names = tuple(spec.get("tensor_names") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        self.float32_out = bool(spec.get("float32_out", False))
        self.activation = str(spec.get("activation", "silu") or "silu")
        self.partial_out = bool(spec.get("partial_out", False))   # with float32_out: the next kernel sums the down product's K splits
        if self.activation not in ops.GLU_ACTIVATIONS:
            raise ConfigError(f"swiglu: activation is one of {sorted(ops.GLU_ACTIVATIONS)}")
        self.w_gate_up = self.w_down = None
        self.fused = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, i = self.hidden_size, self.inter
        gate, up, down = self.names
        return {gate: WeightSpec((i, h)), up: WeightSpec((i, h)), down: WeightSpec((h, i))}

    def load(self, tensors, dtype):
        gate, up, down = self.names
        self.w_down = prepare_weight(tensors[down], dtype)
        self.w_gate_up, self.fused = stack_gate_up(tensors[gate], tensors[up], dtype, self.activation)

    def first_weight(self):
        return self.w_gate_up

    def forward(self, ctx, x):
        mlp = gated_activation(ctx, x, self.w_gate_up, self.fused, self.activation)
        if self.float32_out:
            return linear(ctx, mlp, self.w_down, out_dtype=torch.float32, allow_partial=self.partial_out)
        return linear(ctx, mlp, self.w_down, allow_partial=True)     # summed by the norm that follows


register_part("feed_forward", "swiglu", SwiGLU, replace=True)


class ExpertMixture(FeedForward):
    """Parameters: experts, top, intermediate_size (of one expert), `float32_out`. Tensors:
    `router` [experts, hidden] and `e<i>.gate`, `e<i>.up`, `e<i>.down`. Further parameters:
    `gated` (default true; false: experts are down(gelu(up(x))), no `gate` tensors), `route`
    ("top_softmax", the default: softmax over the chosen logits; "softmax_renorm": softmax over
    all experts, the chosen scores divided by their sum + 1e-20) and `scale`, a constant on the
    weights (default 1).

    With `route` "scored" (experts without a gate only): the router has experts + `identity` rows;
    scores are s = softmax over all of them; rows are chosen by s + `correction` (a tensor,
    present if `correction` is true), among the rows of the `keep` best of `groups` equal groups of
    neighbouring rows (a group's score is its largest corrected score; the other groups' rows count as
    minus infinity); the weights are the chosen rows' s divided by their sum + 1e-20, times `scale`.
    The last `identity` rows are experts without tensors whose output is the feed-forward's input
    itself. `shared` > 0 adds a shared expert of that width (`shared.up`, `shared.down`, same form as
    the others) that runs for every token and is multiplied by sigmoid(w_sg . x), one number per
    token (`shared.sg` [1, hidden]). `activation` ("gelu" by default for experts without a gate, or
    "relu2", the square of relu) is the experts' and the shared expert's. The shared expert's matrices
    stand beside the experts' in the stacked matrices, its gate row under the router's rows, so the
    whole feed-forward is the router kernel, two products, the scaling pass and, with identity experts,
    one pass that adds their share of the input. Long portions take the sorted way described below
    too: identity rows are runs that are copied, the shared expert runs over all tokens afterwards.

    The router's logits are float32. The experts' gate and up matrices stand side by side as one
    [2 * experts * I, hidden] matrix and their down matrices as one [hidden, experts * I]: every
    token's activation is computed for all experts by one product, each expert's slice is
    multiplied by the token's weight for it (zero if it was not chosen), and one more product
    sums the chosen experts' outputs. No launch depends on the router's choice, so a step may be
    replayed from a CUDA graph.

    A step that brings portions of prompts (`GROUPED_FROM` tokens or more, not all of them single
    tokens; such a step is never recorded as a graph) takes another way, in which no expert
    computes a token that did not choose it: the (token, pick) pairs are sorted by expert on the
    device, the host reads how many each expert got (one synchronisation), every expert with
    work multiplies its run of gathered rows, and a last kernel adds every token's picks in pick
    order. The experts' gate and up matrices are kept a second time for it, one per expert."""

    GROUPED_FROM = 256
    # The scored router's sorted way pays one host synchronisation and some thirty small launches a
    # layer; measured at 8 experts of which 2 are chosen (2,048 tokens) it lost to the side-by-side
    # product (2.85 against 2.47 ms a prompt of a 4-layer model), so it is taken from this many
    # experts per pick on.
    GROUPED_MIN_RATIO = 8

    def __init__(self, spec: PartSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        self.experts, self.top = int(spec["experts"]), int(spec["top"])
        self.inter = int(spec["intermediate_size"])
        self.float32_out = bool(spec.get("float32_out", False))
        self.gated = bool(spec.get("gated", True))
        self.route, self.scale = spec.get("route", "top_softmax"), float(spec.get("scale", 1.0))
        self.identity = int(spec.get("identity", 0) or 0)
        self.has_correction = bool(spec.get("correction", False))
        self.groups, self.keep = int(spec.get("groups", 1) or 1), int(spec.get("keep", 1) or 1)
        self.shared = int(spec.get("shared", 0) or 0)
        self.partial_out = bool(spec.get("partial_out", False))
        self.activation = spec.get("activation") or ("gelu" if not self.gated else None)
        self.correction = None
        if self.experts <= 0 or not 0 < self.top <= self.experts + self.identity or self.inter <= 0:
            raise ConfigError("moe: experts, top (at most experts) and intermediate_size must be positive")
        if self.route not in ("top_softmax", "softmax_renorm", "scored") or self.scale != self.scale:
            raise ConfigError("moe: route is 'top_softmax', 'softmax_renorm' or 'scored' and scale a number")
        if self.route != "scored" and (self.identity or self.has_correction or self.groups != 1 or self.shared
                                       or self.activation not in (None, "gelu")):
            raise ConfigError("moe: identity experts, a correction, groups, a shared expert and other activations need route 'scored'")
        if self.route == "scored":
            routed = self.experts + self.identity
            if self.gated or self.activation not in ("gelu", "relu2"):
                raise ConfigError("moe: route 'scored' takes experts without a gate, with activation 'gelu' or 'relu2'")
            if self.identity < 0 or self.shared < 0 or self.groups < 1 or routed % self.groups or not 1 <= self.keep <= self.groups:
                raise ConfigError("moe: groups must divide experts + identity, and keep lie between 1 and groups")
            if self.top > routed // self.groups * self.keep:
                raise ConfigError("moe: top exceeds the experts of the kept groups")
        self.router = self.w_gate_up = self.w_down = None
        self.fused = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h, i = self.hidden_size, self.inter
        specs = {"router": WeightSpec((self.experts + self.identity, h), std=0.5)}
        if self.has_correction:
            specs["correction"] = WeightSpec((self.experts + self.identity,), std=0.05)
        if self.shared:
            specs.update({"shared.up": WeightSpec((self.shared, h)), "shared.down": WeightSpec((h, self.shared)),
                          "shared.sg": WeightSpec((1, h), std=0.5)})
        for e in range(self.experts):
            specs.update({f"e{e}.up": WeightSpec((i, h)), f"e{e}.down": WeightSpec((h, i))})
            if self.gated:
                specs[f"e{e}.gate"] = WeightSpec((i, h))
        return specs

    def load(self, tensors, dtype):
        self.router = tensors["router"].float().contiguous()        # 32-bit logits from exact 32-bit products
        if self.route == "scored":
            return self._load_scored(tensors, dtype)
        up = torch.cat([tensors[f"e{e}.up"] for e in range(self.experts)], dim=0)
        if self.gated:
            gate = torch.cat([tensors[f"e{e}.gate"] for e in range(self.experts)], dim=0)
            self.w_gate_up, self.fused = stack_gate_up(gate, up, dtype)
        else:
            self.w_gate_up, self.fused = prepare_weight(up.contiguous(), dtype), False
        self.w_down = prepare_weight(torch.cat([tensors[f"e{e}.down"] for e in range(self.experts)], dim=1).contiguous(), dtype)
        self.per_expert = []
        if self.top < self.experts:
            for e in range(self.experts):
                if self.gated:
                    gate_up, fused = stack_gate_up(tensors[f"e{e}.gate"], tensors[f"e{e}.up"], dtype)
                else:
                    gate_up, fused = prepare_weight(tensors[f"e{e}.up"], dtype), False
                self.per_expert.append((gate_up, fused, prepare_weight(tensors[f"e{e}.down"], dtype)))

    def _load_scored(self, tensors, dtype):
        ups = [tensors[f"e{e}.up"] for e in range(self.experts)]
        downs = [tensors[f"e{e}.down"] for e in range(self.experts)]
        if self.shared:
            # the shared expert beside the others; its gate row under the router's
            ups.append(tensors["shared.up"])
            downs.append(tensors["shared.down"])
            self.router = torch.cat([self.router, tensors["shared.sg"].float().reshape(1, -1)], dim=0).contiguous()
        if self.has_correction:
            self.correction = tensors["correction"].float().contiguous()
        self.w_gate_up, self.fused = prepare_weight(torch.cat(ups, dim=0).contiguous(), dtype), False
        self.w_down = prepare_weight(torch.cat(downs, dim=1).contiguous(), dtype)
        # for long portions every expert (and the shared one, last) multiplies its own rows: the matrices one by one
        self.per_expert = []
        if self.top < self.experts + self.identity:
            self.per_expert = [(prepare_weight(up, dtype), False, prepare_weight(down, dtype)) for up, down in zip(ups, downs)]

    def _grouped_scored(self, ctx, x, chosen, weights, dense):
        """No expert computes a token that did not choose it: the (token, pick) pairs sorted by routed row
        (identity rows included), a product pair per expert with work, the identity rows' runs copied,
        a token's picks added in pick order, then the shared expert over all tokens."""
        routed = self.experts + self.identity
        offsets, rows, where = ops.moe_group(chosen, routed)
        gathered = ops.gather_rows(x, rows, ctx.status)
        bounds = offsets.tolist()                      # the host learns the rows' shares here
        y = torch.empty((rows.shape[0], self.hidden_size), dtype=torch.float32, device=x.device)
        for e in range(routed):
            lo, hi = bounds[e], bounds[e + 1]
            if hi <= lo:
                continue
            if e >= self.experts:
                y[lo:hi].copy_(gathered[lo:hi])        # an expert that returns its input
                continue
            up, _, down = self.per_expert[e]
            act = ops.moe_scale(ops.materialize(linear(ctx, gathered[lo:hi], up)), None, self.inter, activation=self.activation)
            y[lo:hi].copy_(ops.materialize(linear(ctx, act, down, out_dtype=torch.float32)))
        out = ops.moe_combine(y, where, weights)
        if self.shared:
            up, _, down = self.per_expert[self.experts]
            gate = dense[:, self.experts:].contiguous()
            act = ops.moe_scale(ops.materialize(linear(ctx, x, up)), gate, self.shared, activation=self.activation)
            out = ops.stream_sum(out, ops.materialize(linear(ctx, act, down, out_dtype=torch.float32)))
        return out

    def _forward_scored(self, ctx, x):
        chosen, weights, dense, ident = ops.moe_router_scored(
            x, self.router, self.top, identity=self.identity, correction=self.correction, groups=self.groups, keep=self.keep,
            gate_row=bool(self.shared), scale=self.scale)
        if (self.per_expert and x.shape[0] >= self.GROUPED_FROM and self.experts > self.GROUPED_MIN_RATIO * self.top
                and not getattr(ctx, "all_decode", True) and not torch.cuda.is_current_stream_capturing()):
            y = self._grouped_scored(ctx, x, chosen, weights, dense)
            return y if self.float32_out else ops.stream_sum(None, y, out_dtype=x.dtype)
        act = ops.moe_scale(ops.materialize(linear(ctx, x, self.w_gate_up)), dense, self.inter, activation=self.activation,
                            tail=self.shared)
        y = linear(ctx, act, self.w_down, out_dtype=torch.float32, allow_partial=self.partial_out and not self.identity)
        if self.identity:
            y = ops.moe_identity(y, ident, x)
        return y if self.float32_out else ops.stream_sum(None, ops.materialize(y), out_dtype=x.dtype)

    def first_weight(self):
        return self.w_gate_up

    def _activation(self, ctx, x, w_first, fused, dense=None):
        """An expert's (or all experts') hidden activation, times the dense weights if given."""
        if self.gated:
            act = gated_activation(ctx, x, w_first, fused)
            return act if dense is None else ops.moe_scale(act, dense, self.inter)
        return ops.moe_scale(ops.materialize(linear(ctx, x, w_first)), dense, self.inter, gelu=True)

    def _grouped(self, ctx, x, chosen, weights):
        offsets, rows, where = ops.moe_group(chosen, self.experts)
        gathered = ops.gather_rows(x, rows, ctx.status)
        bounds = offsets.tolist()                      # the host learns the experts' shares here
        y = torch.empty((rows.shape[0], self.hidden_size), dtype=torch.float32, device=x.device)
        for e, (gate_up, fused, down) in enumerate(self.per_expert):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                act = self._activation(ctx, gathered[lo:hi], gate_up, fused)
                y[lo:hi].copy_(linear(ctx, act, down, out_dtype=torch.float32))
        return ops.moe_combine(y, where, weights)

    def forward(self, ctx, x):
        x = ops.materialize(x)
        if self.route == "scored":
            return self._forward_scored(ctx, x)
        chosen, weights, dense = ops.moe_router(x, self.router, self.top, over_all=self.route == "softmax_renorm", scale=self.scale)
        if (self.per_expert and x.shape[0] >= self.GROUPED_FROM and not getattr(ctx, "all_decode", True)
                and not torch.cuda.is_current_stream_capturing()):
            out = self._grouped(ctx, x, chosen, weights)
            return out if self.float32_out else out.to(x.dtype)
        act = self._activation(ctx, x, self.w_gate_up, self.fused, dense)
        if self.float32_out:
            return linear(ctx, act, self.w_down, out_dtype=torch.float32)
        return linear(ctx, act, self.w_down, allow_partial=True)


register_part("feed_forward", "moe", ExpertMixture, replace=True)
