"""Rotary position encoding: inverse frequencies theta^(-2i/rotary_dim) in float32,
angle = position * inv_freq in float32 (runtime/backends/cuda/native/
cuda_kernels.cu:93-116).  The rotation itself runs inside the mixer's fused
rotate-and-append kernel; this part owns the table and the pairing."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, RotaryTable, register_part


@register_part("position", "rope")
class RotaryEncoding(PositionEncoding):
    """params: theta, rotary_dim (even, at most the head size), pairing
    (`split_half`: element i pairs with i + rotary_dim/2; `interleaved`: 2i with 2i+1), scaling (None, or
    {factor, low, high, original}: a frequency whose wavelength is below original/high stays, one whose
    wavelength is above original/low is divided by factor, and in between the two are blended linearly in
    original/wavelength; or {kind: "ramp", factor, original, fast, slow}: with index(t) = rotary_dim *
    ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(index(fast)), 0) and hi = min(ceil(index(slow)),
    rotary_dim - 1), frequency i is blended towards f_i / factor by clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    and cos and sin are multiplied by 0.1 ln(factor) + 1).  The table is worked out in double precision and
    kept in float32."""

    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        pairing = spec.params.get("pairing", "split_half")
        if pairing not in ("split_half", "interleaved"):
            raise ValueError(f"rope: unknown pairing {pairing!r}")
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rope: rotary_dim must be positive and even, got {self.rotary_dim}")
        self.interleaved = pairing == "interleaved"
        scaling = spec.params.get("scaling")
        self.scaling = None
        self.ramp = None
        self.magnitude = 1.0
        if scaling and scaling.get("kind") == "ramp":
            self.ramp = {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
            if not (min(self.ramp.values()) > 0 and self.theta > 1):
                raise ValueError(f"rope: bad frequency scaling {scaling!r}")
            self.magnitude = 0.1 * math.log(self.ramp["factor"]) + 1.0
        elif scaling:
            self.scaling = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")}
            if not (self.scaling["factor"] > 0 and self.scaling["original"] > 0 and self.scaling["high"] > self.scaling["low"] >= 0):
                raise ValueError(f"rope: bad frequency scaling {scaling!r}")
        self._table = None

    def frequencies(self):
        """The rotary_dim / 2 frequencies as Python floats (double precision)."""
        out = []
        if self.ramp is not None:
            r, dims = self.ramp, self.rotary_dim

            def index_of(turns):                                       # the index whose frequency turns that often
                return dims * math.log(r["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo, hi = max(math.floor(index_of(r["fast"])), 0), min(math.ceil(index_of(r["slow"])), dims - 1)
        for i in range(self.rotary_dim // 2):
            f = self.theta ** (-2.0 * i / self.rotary_dim)
            if self.ramp is not None:
                blend = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                f = f / self.ramp["factor"] * blend + f * (1.0 - blend)
            if self.scaling is not None:
                sc = self.scaling
                turns = sc["original"] * f / (2.0 * math.pi)          # original / wavelength
                if turns > sc["high"]:
                    pass
                elif turns < sc["low"]:
                    f = f / sc["factor"]
                else:
                    blend = (turns - sc["low"]) / (sc["high"] - sc["low"])
                    f = (1.0 - blend) * f / sc["factor"] + blend * f
            out.append(f)
        return out

    def rotary(self, device):
        if self._table is None or self._table.inv_freq.device != torch.device(device):
            if self.scaling is None and self.ramp is None:
                exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
                inv_freq = (1.0 / (self.theta ** exponent)).to(torch.float32)
            else:
                inv_freq = torch.tensor(self.frequencies(), dtype=torch.float64).to(torch.float32)
            self._table = RotaryTable(inv_freq.to(device).contiguous(), self.rotary_dim, self.interleaved,
                                      self.magnitude)
        return self._table


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Queries and keys are used as projected."""
