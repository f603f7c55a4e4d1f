"""Rotary position encoding: inverse frequencies theta^(-2i/rotary_dim) in float32,
angle = position * inv_freq in float32 (runtime/backends/cuda/native/
cuda_kernels.cu:93-116).  The rotation itself runs inside the mixer's fused
rotate-and-append kernel; this part owns the table and the pairing."""
from __future__ import annotations

import torch

from .base import PositionEncoding, RotaryTable, register_part


@register_part("position", "rope")
class RotaryEncoding(PositionEncoding):
    """params: theta, rotary_dim (even, at most the head size), pairing
    (`split_half`: element i pairs with i + rotary_dim/2; `interleaved`: 2i with 2i+1)."""

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
        self._table = None

    def rotary(self, device):
        if self._table is None or self._table.inv_freq.device != torch.device(device):
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
            inv_freq = (1.0 / (self.theta ** exponent)).to(torch.float32)
            self._table = RotaryTable(inv_freq.to(device).contiguous(), self.rotary_dim, self.interleaved)
        return self._table


@register_part("position", "none")
class NoPositionEncoding(PositionEncoding):
    """Queries and keys are used as projected."""
