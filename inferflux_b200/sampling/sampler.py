"""From logits rows to token ids, on the device.

Penalties over the recent tokens, logit bias, then argmax or
softmax(logits / temperature) with top-k / min-p / nucleus thresholds and one
counter-based random number per row keyed by (request seed, request step), so that
what a request draws does not depend on the batch it is in.  Unlike the reference,
a greedy request gets no implicit repetition penalty
(runtime/backends/cuda/inferflux_cuda_executor.cpp:3369-3371 applies 1.15).
"""
from __future__ import annotations

from collections import Counter
from dataclasses import dataclass
from typing import List, Sequence

import torch

from .params import SamplingParams


@dataclass
class SamplingRow:
    """One logits row's request state."""
    params: SamplingParams
    seed: int                      # 64-bit
    step: int                      # how many tokens the request has sampled so far
    recent: Sequence[int] = ()     # the request's sampled tokens (the sampler looks at the last penalty_last_n)


class Sampler:
    def __init__(self, kernels, device):
        self.kernels = kernels
        self.device = torch.device(device)

    def _dev(self, values, dtype):
        t = torch.tensor(values, dtype=dtype)
        if self.device.type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    def sample(self, logits: torch.Tensor, rows: List[SamplingRow]) -> torch.Tensor:
        """int32 token ids [len(rows)] on the device.  `logits` may be changed in place."""
        assert logits.shape[0] == len(rows)
        if not rows:
            return torch.empty((0,), dtype=torch.int32, device=logits.device)
        k = self.kernels
        if any(r.params.has_penalties for r in rows):
            width = max(1, max(min(len(r.recent), r.params.penalty_last_n) for r in rows))
            toks, cnts = [], []
            for r in rows:
                window = list(r.recent)[-r.params.penalty_last_n:] if r.params.has_penalties else []
                c = Counter(window)
                items = list(c.items())
                toks.append([t for t, _ in items] + [-1] * (width - len(items)))
                cnts.append([n for _, n in items] + [0] * (width - len(items)))
            k.penalties(logits, self._dev(toks, torch.int32), self._dev(cnts, torch.int32),
                        self._dev([r.params.repetition_penalty for r in rows], torch.float32),
                        self._dev([r.params.frequency_penalty for r in rows], torch.float32),
                        self._dev([r.params.presence_penalty for r in rows], torch.float32))
        bias = [(i, int(t), float(b)) for i, r in enumerate(rows) for t, b in r.params.logit_bias.items()]
        if bias:
            k.logit_bias(logits, self._dev([b[0] for b in bias], torch.int32),
                         self._dev([b[1] for b in bias], torch.int32), self._dev([b[2] for b in bias], torch.float32))
        if all(r.params.greedy for r in rows):
            return k.argmax(logits)
        as_i32 = lambda v: v - (1 << 32) if v >= (1 << 31) else v
        return k.sample(
            logits,
            self._dev([r.params.temperature for r in rows], torch.float32),
            self._dev([r.params.top_k for r in rows], torch.int32),
            self._dev([r.params.top_p for r in rows], torch.float32),
            self._dev([r.params.min_p for r in rows], torch.float32),
            self._dev([as_i32(r.seed & 0xFFFFFFFF) for r in rows], torch.int32),
            self._dev([as_i32((r.seed >> 32) & 0xFFFFFFFF) for r in rows], torch.int32),
            self._dev([as_i32(r.step & 0xFFFFFFFF) for r in rows], torch.int32),
            features=(1 if any(r.params.top_k > 0 for r in rows) else 0) |
                     (2 if any(0.0 < r.params.top_p < 1.0 for r in rows) else 0))
