"""RMSNorm with a plain weight (no 1 + w offset), optionally fused with the residual add.

o = x * rsqrt(mean(x^2) + eps) * w in float32 (kernels/triton_kernels/rmsnorm.py:63-93);
with a residual the sum is stored as the new residual and normed unrounded
(kernels/triton_kernels/rmsnorm_residual.py:86-125).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import PartSpec
from ..weights.loader import WeightSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    def __init__(self, spec: PartSpec, width: int):
        super().__init__(spec, width)
        self.eps = float(spec["eps"])
        self.width = width
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.width,), init="norm", std=0.1)}

    def load(self, tensors, dtype):
        self.weight = tensors["weight"]

    def forward(self, ctx, x):
        return ops.rmsnorm(x, self.weight, self.eps)[0]

    def forward_add(self, ctx, x, residual):
        # the sum overwrites the residual buffer in place
        return ops.rmsnorm(x, self.weight, self.eps, residual=residual, residual_out=residual)


register_part("norm", "rmsnorm", RMSNorm, replace=True)


class DynamicTanh(Norm):
    """A norm that computes no statistics: tanh(alpha * x) * weight + bias with a learned scalar
    alpha. It serves models whose residual stream is float32 in both serving types: `forward_add`
    takes the stream and what is still to be added to it (a tensor or an `ops.DeferredSum`),
    adds in float32, stores the sum as the new stream and returns the normed rows in the
    serving type. Parameters: `bias` (default true) says whether a bias vector exists,
    `bias_name` what the checkpoint calls it beside the weight (default "bias")."""

    def __init__(self, spec: PartSpec, width: int):
        super().__init__(spec, width)
        self.width = width
        self.has_bias = bool(spec.get("bias", True))
        self.bias_key = str(spec.get("bias_name", "bias"))
        self.weight = self.bias = None
        self.alpha = 1.0

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"weight": WeightSpec((self.width,), init="norm", std=0.1), "alpha": WeightSpec((), init="norm", std=0.1)}
        if self.has_bias:
            specs[self.bias_key] = WeightSpec((self.width,), std=0.1)
        return specs

    def load(self, tensors, dtype):
        self.weight, self.bias = tensors["weight"], tensors.get(self.bias_key)
        if self.bias is not None and self.bias.dtype != self.weight.dtype:
            self.weight, self.bias = self.weight.float(), self.bias.float()
        self.alpha = float(tensors["alpha"].float().item())
        self.out_dtype = dtype

    def forward(self, ctx, x):
        return ops.dyt(x, self.weight, self.bias, self.alpha, ctx.dtype)

    def forward_add(self, ctx, x, residual):
        if residual is None:
            # the stream starts here: the sum of what came is stored as float32
            first = ops.materialize(x.terms[0] if isinstance(x, ops.DeferredSum) else x)
            residual = torch.empty(first.shape, dtype=torch.float32, device=first.device)
            return ops.dyt(x, self.weight, self.bias, self.alpha, ctx.dtype, stream_out=residual), residual
        return ops.dyt(x, self.weight, self.bias, self.alpha, ctx.dtype, stream=residual, stream_out=residual), residual


register_part("norm", "dyt", DynamicTanh, replace=True)


class StreamRMSNorm(Norm):
    """Root-mean-square norm for models whose residual stream is float32 in both serving types:
    x / sqrt(mean(x^2) + eps) * (offset + weight), in float32, rounded to the serving type.
    Parameters: `eps`; `unit_offset` (default false): the weight is stored around zero and one is
    added to it. `forward_add` takes the stream and what is still to be added to it (a tensor or
    an `ops.DeferredSum`), adds in float32, stores the sum as the new stream and norms it.
    `out_dtype` "float32" keeps the normed rows unrounded (for a sublayer's output that is itself
    added to the stream)."""

    def __init__(self, spec: PartSpec, width: int):
        super().__init__(spec, width)
        self.eps = float(spec["eps"])
        self.offset = 1.0 if bool(spec.get("unit_offset", False)) else 0.0
        self.float32_out = spec.get("out_dtype") == "float32"
        self.width = width
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.width,), init="linear" if self.offset else "norm", std=0.1)}

    def load(self, tensors, dtype):
        self.weight = tensors["weight"]

    def _out(self, ctx):
        return torch.float32 if self.float32_out else ctx.dtype

    def forward(self, ctx, x):
        return ops.rms_stream(x, self.weight, self.eps, self._out(ctx), offset=self.offset)

    def forward_add(self, ctx, x, residual):
        if residual is None:
            first = ops.materialize(x.terms[0] if isinstance(x, ops.DeferredSum) else x)
            residual = torch.empty(first.shape, dtype=torch.float32, device=first.device)
            return ops.rms_stream(x, self.weight, self.eps, self._out(ctx), offset=self.offset, stream_out=residual), residual
        return ops.rms_stream(x, self.weight, self.eps, self._out(ctx), offset=self.offset, stream=residual,
                              stream_out=residual), residual


register_part("norm", "rms_stream", StreamRMSNorm, replace=True)


class LayerNormStream(Norm):
    """Layer norm with weight and bias for models whose residual stream is float32 in both serving
    types: (x - mean) / sqrt(var + eps) * weight + bias with var the mean of the squared
    deviations, in float32, rounded to the serving type. Parameters: `eps`; `bias` (default true);
    `bias_name`, what the checkpoint calls the bias beside the weight (default "bias");
    `out_dtype` "float32" keeps the normed rows unrounded. `forward_add` takes the stream and what
    is still to be added to it: a tensor, or an `ops.DeferredNormed` (a sublayer output that is
    itself normed and scaled on its way into the stream); the sum is stored as the new stream."""

    def __init__(self, spec: PartSpec, width: int):
        super().__init__(spec, width)
        self.eps = float(spec["eps"])
        self.has_bias = bool(spec.get("bias", True))
        self.bias_key = str(spec.get("bias_name", "bias"))
        self.float32_out = spec.get("out_dtype") == "float32"
        self.width = width
        self.weight = self.bias = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"weight": WeightSpec((self.width,), init="norm", std=0.1)}
        if self.has_bias:
            specs[self.bias_key] = WeightSpec((self.width,), std=0.1)
        return specs

    def load(self, tensors, dtype):
        self.weight, self.bias = tensors["weight"], tensors.get(self.bias_key)
        if self.bias is not None and self.bias.dtype != self.weight.dtype:
            self.weight, self.bias = self.weight.float(), self.bias.float()

    def _out(self, ctx):
        return torch.float32 if self.float32_out else ctx.dtype

    def forward(self, ctx, x):
        if x.dtype == torch.float32:
            return ops.layer_norm_stream(None, self.weight, self.bias, self.eps, self._out(ctx), stream=x)
        return ops.layer_norm_stream(x, self.weight, self.bias, self.eps, self._out(ctx))

    def forward_add(self, ctx, x, residual):
        if residual is None:
            first = x.y if isinstance(x, ops.DeferredNormed) else ops.materialize(x)
            residual = torch.empty(first.shape, dtype=torch.float32, device=first.device)
            return ops.layer_norm_stream(x, self.weight, self.bias, self.eps, self._out(ctx), stream_out=residual), residual
        return ops.layer_norm_stream(x, self.weight, self.bias, self.eps, self._out(ctx), stream=residual,
                                     stream_out=residual), residual

    def defer(self, y, scale):
        """`y` as something this norm (and the `scale` vector, if any) is still to be applied to, for
        the kernel that adds it to the stream."""
        return ops.DeferredNormed(y, self.weight, self.bias, scale, self.eps)


register_part("norm", "layer_norm_stream", LayerNormStream, replace=True)
