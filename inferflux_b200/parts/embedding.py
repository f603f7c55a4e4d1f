"""Token embedding and LM head.

x0[t] = E[token[t]] with no scaling (runtime/backends/cuda/native/
cuda_kernels.cu:256-270, 675-689: the residual stream is float32).  The head is
lm_head.weight, or the embedding table when the model ties them
(runtime/backends/cuda/native/weight_map.cpp:33-37); here the configuration's
tie_word_embeddings decides, and logits are produced in float32 for whichever rows
the step asks for.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, register_part


@register_part("embedding", "embedding")
class Embedding(Part):
    """params: vocab_size, hidden_size."""

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.table = None

    def param_specs(self):
        return {"weight": TensorSpec((self.vocab, self.hidden))}

    def load(self, tensors, dtype, device):
        self.table = tensors["weight"].to(device=device, dtype=dtype).contiguous()

    def forward(self, ctx):
        return ctx.kernels.embed(self.table, ctx.token_ids, self.vocab)


@register_part("lm_head", "lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, tied."""

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = bool(spec.params.get("tied", False))
        self.weight = None

    def param_specs(self):
        return {"weight": TensorSpec((self.vocab, self.hidden), ignored=self.tied)}

    def load(self, tensors, dtype, device, tied_table=None):
        if self.tied:
            if tied_table is None:
                raise ValueError("lm_head: tied head needs the embedding table")
            self.weight = tied_table
        else:
            self.weight = tensors["weight"].to(device=device, dtype=dtype).contiguous()

    def forward(self, h, ctx):
        """h: normed rows [R, hidden] -> float32 logits [R, vocab]."""
        return ctx.kernels.linear(h, self.weight, out_dtype=torch.float32)
