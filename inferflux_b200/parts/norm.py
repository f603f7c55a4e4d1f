"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, reductions in float32
(runtime/backends/cuda/native/cuda_kernels.cu:26-47); with a pending delta the sum
x += delta happens in the same kernel (cuda_kernels.cu:618-655)."""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Norm, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: size, eps."""

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def param_specs(self):
        return {"weight": TensorSpec((self.size,), init="ones")}

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, delta, ctx, lazy=False):
        if lazy and hasattr(ctx.kernels, "prenorm"):
            return ctx.kernels.prenorm(x, delta, self.weight, self.eps, ctx.dtype)
        if delta is None:
            return ctx.kernels.rmsnorm(x, self.weight, self.eps, ctx.dtype)
        return ctx.kernels.add_rmsnorm(x, delta, self.weight, self.eps, ctx.dtype)
