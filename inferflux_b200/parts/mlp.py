"""SwiGLU feed-forward: (silu(h Wg^T) * (h Wu^T)) Wd^T, no biases
(runtime/backends/cuda/native/transformer_forward.cu:2384-2535).  Gate and up
weights are stacked at load so that one product makes both."""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import FeedForward, WeightBuffers, register_part


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size."""

    takes_scaled_rows = True          # h goes only into the stacked projection


    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def param_specs(self):
        return {
            "gate_proj.weight": TensorSpec((self.inter, self.hidden)),
            "up_proj.weight": TensorSpec((self.inter, self.hidden)),
            "down_proj.weight": TensorSpec((self.hidden, self.inter)),
        }

    def load(self, tensors, dtype, device):
        self.buffers = buf = WeightBuffers(device, {"w_gate_up": ((2 * self.inter, self.hidden), dtype),
                                                    "w_down": ((self.hidden, self.inter), dtype)})
        buf["w_gate_up"][:self.inter].copy_(tensors["gate_proj.weight"])
        buf["w_gate_up"][self.inter:].copy_(tensors["up_proj.weight"])
        buf["w_down"].copy_(tensors["down_proj.weight"])
        self.w_gate_up, self.w_down = buf["w_gate_up"], buf["w_down"]

    def forward(self, h, ctx):
        k = ctx.kernels
        act = k.linear_swiglu(h, self.w_gate_up)         # [T, I] = silu(h Wg^T) * (h Wu^T)
        return k.linear(act, self.w_down, allow_partial=True)
