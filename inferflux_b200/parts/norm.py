"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, reductions in float32
(runtime/backends/cuda/native/cuda_kernels.cu:26-47); with a pending delta the sum
x += delta happens in the same kernel (cuda_kernels.cu:618-655).  With `groups` the row
is cut into that many equal consecutive parts and each has a root mean square of its own."""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Norm, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, unit_offset (the stored weight is the distance from one: y = x / rms * (1 + w);
    default False), tensor_name (default `weight`), groups (default 1: the mean runs over the whole row)."""

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.unit_offset = bool(spec.params.get("unit_offset", False))
        self.tensor_name = str(spec.params.get("tensor_name", "weight"))
        self.groups = int(spec.params.get("groups", 1))
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"rmsnorm: {self.groups} groups do not cut a row of {self.size} evenly")
        self.weight = None

    def param_specs(self):
        return {self.tensor_name: TensorSpec((self.size,), init="zeros" if self.unit_offset else "ones")}

    def load(self, tensors, dtype, device):
        w = tensors[self.tensor_name].to(device=device, dtype=torch.float32)
        self.weight = (w + 1.0 if self.unit_offset else w).contiguous()      # the kernels multiply by this

    def forward(self, x, delta, ctx, lazy=False):
        if self.groups > 1:
            if delta is not None:
                ctx.kernels.residual_add(x, delta)
            return ctx.kernels.rmsnorm(x, self.weight, self.eps, ctx.dtype, groups=self.groups)
        if lazy and hasattr(ctx.kernels, "prenorm"):
            return ctx.kernels.prenorm(x, delta, self.weight, self.eps, ctx.dtype)
        if delta is None:
            return ctx.kernels.rmsnorm(x, self.weight, self.eps, ctx.dtype)
        return ctx.kernels.add_rmsnorm(x, delta, self.weight, self.eps, ctx.dtype)
