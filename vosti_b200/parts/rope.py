"""Rotary position encoding: half-split pairing of the whole head for Qwen3; `rotary_dim` below
the head size (the rest of the head is not rotated) and `interleaved` pairs (2i, 2i + 1) are
parameters for other architectures.

inv_freq[i] = 1 / theta^(2i/d) in float32 from an integer arange; angle = inv_freq *
float(position) (python/vosti_kernels/rotary.py:80-88, 155-158). The reference casts the
cos/sin table to the serving dtype (:160); here the table stays float32 in both serving
dtypes, so rotation angles are 32-bit everywhere. The mixer applies the table
(pairs (i, i + d/2): kernels/triton_kernels/rope.py:78-101).

`scaling` = ("wavelength", factor, low, high, original) rescales the frequencies by their
wavelength l = 2 pi / f, the rule long-context Llama checkpoints use: f stays where
l < original / high, becomes f / factor where l > original / low, and between the two is
(1 - s) f / factor + s f with s = (original / l - low) / (high - low).

`scaling` = ("yarn", factor, original, fast, slow) blends by index instead: with
index(t) = d ln(original / (2 pi t)) / (2 ln theta), the index at which a frequency makes t turns
over `original` positions, lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), d - 1) and
ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is f_i / factor * ramp_i +
f_i (1 - ramp_i); cos and sin are then multiplied by `magnitude()` = 0.1 ln(factor) + 1.

`max_positions` 0 (or absent) builds no tables: a mixer then takes `frequencies()` and forms
every angle position * f in float32 itself, so that positions have no limit.
"""
from __future__ import annotations

import math

import torch

from ..config.schema import ConfigError, PartSpec
from .base import PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PartSpec, hidden_size: int, head_dim: int):
        super().__init__(spec, hidden_size, head_dim)
        self.theta = float(spec["theta"])
        self.max_positions = int(spec.get("max_positions", 0) or 0)
        self.scaling = spec.get("scaling")
        if self.scaling is not None:
            if len(self.scaling) != 5 or self.scaling[0] not in ("wavelength", "yarn"):
                raise ConfigError("rope: scaling is ('wavelength', factor, low, high, original) or "
                                  "('yarn', factor, original, fast, slow)")
            if self.scaling[0] == "wavelength":
                _, factor, low, high, original = self.scaling
                if not (factor > 0 and high > low >= 0 and original > 0):
                    raise ConfigError("rope: scaling needs factor > 0, high > low >= 0 and original > 0")
            else:
                _, factor, original, fast, slow = self.scaling
                if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and self.theta > 1):
                    raise ConfigError("rope: yarn scaling needs factor, original, fast and slow > 0 and theta > 1")
        rotary_dim = int(spec.get("rotary_dim", head_dim) or head_dim)
        if rotary_dim <= 0 or rotary_dim > head_dim or rotary_dim % 2:
            raise ConfigError(f"rope: rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.rotary_dim = rotary_dim
        self.interleaved = bool(spec.get("interleaved", False))
        self.cos = self.sin = None

    def frequencies(self) -> torch.Tensor:
        """float32 [rotary_dim / 2] on the CPU: theta^(-2i/rotary_dim), rescaled if `scaling` says so.
        Without scaling the values are the table's (float32 arithmetic); with it they are formed in
        float64 and rounded once."""
        if self.scaling is None:
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).to(torch.float32) / self.rotary_dim
            return 1.0 / (self.theta ** exponent)
        if self.scaling[0] == "yarn":
            return torch.tensor(self._yarn(), dtype=torch.float64).to(torch.float32)
        _, factor, low, high, original = self.scaling
        out = []
        for i in range(self.rotary_dim // 2):
            f = self.theta ** (-2.0 * i / self.rotary_dim)
            wave = 2.0 * math.pi / f
            if wave < original / high:
                pass
            elif low > 0 and wave > original / low:
                f = f / factor
            else:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
            out.append(f)
        return torch.tensor(out, dtype=torch.float64).to(torch.float32)

    def _yarn(self):
        _, factor, original, fast, slow = self.scaling
        d = self.rotary_dim
        index = lambda turns: d * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
        lo, hi = max(math.floor(index(fast)), 0), min(math.ceil(index(slow)), d - 1)
        out = []
        for i in range(d // 2):
            f = self.theta ** (-2.0 * i / d)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / factor * ramp + f * (1.0 - ramp))
        return out

    def magnitude(self) -> float:
        """What cos and sin are multiplied by: 0.1 ln(factor) + 1 under yarn scaling, else 1."""
        if self.scaling is not None and self.scaling[0] == "yarn":
            return 0.1 * math.log(self.scaling[1]) + 1.0
        return 1.0

    def setup(self, device, dtype):
        if self.max_positions <= 0:
            return
        inv_freq = self.frequencies()
        angles = torch.arange(self.max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
        self.cos = (angles.cos() * self.magnitude()).to(device).contiguous()
        self.sin = (angles.sin() * self.magnitude()).to(device).contiguous()

    def rotation_tables(self):
        return (self.cos, self.sin) if self.cos is not None else None


register_part("position", "rope", RotaryEncoding, replace=True)
