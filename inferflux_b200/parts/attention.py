"""Grouped-query causal attention over a paged key/value cache.

q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv (biases by tensor presence,
runtime/backends/cuda/native/weight_map.cpp:55-58); q and k are rotated after the
bias (runtime/backends/cuda/native/transformer_forward.cu:2024-2089); rotated keys
and raw values go to the cache at the token's position (runtime/backends/cuda/native/
kernels/fused_rope_kv_append.cuh:110-143); query head h uses key/value head
h // (heads / kv_heads), score = q.k * scale, every token sees the keys up to its
own position, or the last `window` of them (runtime/backends/cuda/kernels/
flash_attention.cu:71-86, 152-172); then the output projection.

The three projections are stacked at load so that one product makes q, k and v.
"""
from __future__ import annotations

import math

import torch

from ..weights.loader import TensorSpec
from .base import KVCacheSpec, Mixer, WeightBuffers, build_part, register_part


@register_part("mixer", "attention")
class Attention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (None or int),
    position (a PartSpec of role `position`, or None), qkv_bias (True, False or
    "if_present"), invent_bias (with "if_present": whether random-weights mode makes
    the biases up; default True), scale (None for 1/sqrt(head_dim))."""

    takes_scaled_rows = True          # h goes only into the stacked projection

    @staticmethod
    def check_head_dim(d: int) -> None:
        """The attention kernels (tiled or per-token) take head sizes that are multiples of 8 up
        to 256; anything else is refused when the model is planned, not at the first step."""
        if d <= 0 or d % 8 or d > 256:
            raise ValueError(f"attention: head size {d} is not supported (multiples of 8 up to 256)")

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.check_head_dim(self.d)
        if self.nq % self.nkv:
            raise ValueError(f"attention: {self.nq} heads are not a multiple of {self.nkv} kv heads")
        self.window = None if p.get("window") is None else int(p["window"])
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.d)
        self.qkv_bias = p.get("qkv_bias", "if_present")
        self.invent_bias = bool(p.get("invent_bias", True))
        pos = p.get("position")
        self.position = build_part("position", pos) if pos is not None else None
        self.w_qkv = self.b_qkv = self.w_o = None

    # ---------------------------------------------------------------- declarations
    def cache_spec(self):
        return KVCacheSpec(self.nkv, self.d, self.window)

    def param_specs(self):
        q, kv = self.nq * self.d, self.nkv * self.d
        specs = {
            "q_proj.weight": TensorSpec((q, self.hidden)),
            "k_proj.weight": TensorSpec((kv, self.hidden)),
            "v_proj.weight": TensorSpec((kv, self.hidden)),
            "o_proj.weight": TensorSpec((self.hidden, q)),
        }
        if self.qkv_bias is not False:
            optional = self.qkv_bias == "if_present"
            for n, size in (("q", q), ("k", kv), ("v", kv)):
                specs[n + "_proj.bias"] = TensorSpec((size,), optional=optional, invent=self.invent_bias)
        return specs

    def load(self, tensors, dtype, device):
        q, kv = self.nq * self.d, self.nkv * self.d
        has_bias = any((n + "_proj.bias") in tensors for n in ("q", "k", "v"))
        layout = {"w_qkv": ((q + 2 * kv, self.hidden), dtype), "w_o": ((self.hidden, q), dtype)}
        if has_bias:
            layout["b_qkv"] = ((q + 2 * kv,), torch.float32)              # added in float32
        self.buffers = buf = WeightBuffers(device, layout)
        at = 0
        for n, size in zip(("q", "k", "v"), (q, kv, kv)):                 # each projection into its rows of the stack
            buf["w_qkv"][at:at + size].copy_(tensors[n + "_proj.weight"])
            if has_bias:
                b = tensors.get(n + "_proj.bias")
                if b is None:
                    buf["b_qkv"][at:at + size].zero_()
                else:
                    buf["b_qkv"][at:at + size].copy_(b)
            at += size
        buf["w_o"].copy_(tensors["o_proj.weight"])
        self.w_qkv, self.w_o = buf["w_qkv"], buf["w_o"]
        self.b_qkv = buf["b_qkv"] if has_bias else None

    def step_sections(self, ctx):
        """The work lists of the kernel table's attention kernels, if it has any."""
        make = getattr(ctx.kernels, "attention_sections", None)
        return make(ctx) if make is not None else {}

    # --------------------------------------------------------------------- forward
    def forward(self, h, ctx, cache):
        k = ctx.kernels
        qkv = k.linear(h, self.w_qkv, allow_partial=True)                    # [T, (nq + 2 nkv) d], maybe in K slices
        rotary = self.position.rotary(ctx.device) if self.position is not None else None
        q = k.rope_append(qkv, self.b_qkv, rotary, self.nq, self.nkv, self.d, ctx, cache)   # [T, nq d]
        a = k.attention(q, self.nq, self.nkv, self.d, self.window, self.scale, ctx, cache)  # [T, nq d]
        return k.linear(a, self.w_o, allow_partial=True)
