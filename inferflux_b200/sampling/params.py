"""Per-request sampling parameters, with the reference's names, defaults and
meanings (scheduler/request_batch.h:26-38)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0          # <= 0: greedy argmax (gpu_sampler.cu:608)
    top_p: float = 1.0                # nucleus; 1.0 = off
    top_k: int = 0                    # 0 = off
    min_p: float = 0.0                # 0.0 = off
    frequency_penalty: float = 0.0    # minus this times the token's count among the recent tokens
    presence_penalty: float = 0.0     # minus this if the token is among the recent tokens
    repetition_penalty: float = 1.0   # logit > 0 ? logit / r : logit * r;  1.0 = off
    penalty_last_n: int = 64          # how many of the last sampled tokens the penalties look at
    seed: Optional[int] = None        # None: the engine draws one per request
    logit_bias: Dict[int, float] = field(default_factory=dict)

    def validate(self) -> None:
        if self.top_p <= 0 or self.top_p > 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0 <= self.min_p <= 1:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be positive, got {self.repetition_penalty}")
        if self.penalty_last_n < 0:
            raise ValueError(f"penalty_last_n must be >= 0, got {self.penalty_last_n}")

    @property
    def greedy(self) -> bool:
        return not self.temperature > 0

    @property
    def has_penalties(self) -> bool:
        return (self.frequency_penalty != 0 or self.presence_penalty != 0 or self.repetition_penalty != 1.0) \
            and self.penalty_last_n > 0

    @classmethod
    def greedy_params(cls) -> "SamplingParams":
        return cls(temperature=0.0)
