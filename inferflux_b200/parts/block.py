"""Pre-norm residual block: x += mixer(norm(x)); x += ffn(norm(x))
(runtime/backends/cuda/native/llama_forward.h:88-90).  The block hands its last
delta on unadded, so that whatever normalises next adds it in the same kernel
(runtime/backends/cuda/native/transformer_forward.cu:2203-2211, 2564-2586)."""
from __future__ import annotations

from .base import Block, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    sub_parts = {"norm_mixer": "norm", "mixer": "mixer", "norm_ffn": "norm", "ffn": "ffn"}

    def forward(self, x, pending, ctx, cache):
        fused = getattr(ctx.kernels, "fused_prenorm_layer", None)    # a kernel table may run the whole layer itself
        if fused is not None:
            done = fused(self, x, pending, ctx, cache)
            if done is not None:
                return done
        h = self.norm_mixer.forward(x, pending, ctx, lazy=self.mixer.takes_scaled_rows)   # x += pending; h = norm(x)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norm_ffn.forward(x, a, ctx, lazy=self.ffn.takes_scaled_rows)             # x += a; h = norm(x)
        f = self.ffn.forward(h, ctx)
        return x, f
