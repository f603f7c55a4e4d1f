"""Random-weights mode: make up a model from a configuration and a seed.

Linear weights, tables and biases are N(0, std) with std 0.02, norm weights are 1.0
(optionally jittered so that tests see a fault in how a norm weight is used).  Each
tensor has a generator of its own, seeded by (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or in which order they are made.
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Dict

import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 62))
    return g


def random_tensors(expected: Dict[str, TensorSpec], seed: int, dtype=torch.bfloat16, device="cpu",
                   std: float = 0.02, norm_jitter: float = 0.0, include_optional: bool = True
                   ) -> Dict[str, torch.Tensor]:
    """One tensor per entry of `expected`.  Values are drawn in float32 and rounded
    once to `dtype`; tensors whose init is `ones` stay float32 when jittered or not."""
    out = {}
    dev = torch.device(device)
    for name, spec in expected.items():
        if spec.ignored or (spec.optional and not include_optional):
            continue
        g = _generator(seed, name, dev)
        if spec.init == "normal":
            t = torch.empty(spec.shape, dtype=torch.float32, device=dev).normal_(0.0, std, generator=g).to(dtype)
        elif spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=dev)
            if norm_jitter:
                t += torch.empty(spec.shape, dtype=torch.float32, device=dev).normal_(0.0, norm_jitter, generator=g)
            t = t.to(dtype)
        elif spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=dtype, device=dev)
        else:
            raise ValueError(f"unknown init {spec.init!r} for {name}")
        out[name] = t
    return out


def write_random_model(config, out_dir, seed: int, dtype=torch.bfloat16, std: float = 0.02,
                       norm_jitter: float = 0.0) -> Path:
    """Write config.json and model.safetensors for `config` (a typed configuration
    of a registered architecture) into `out_dir`."""
    from ..models.model import expected_tensors            # late import: models imports weights
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    expected = expected_tensors(config.to_plan())
    include_bias = bool(getattr(config, "qkv_bias", True))
    tensors = random_tensors(expected, seed, dtype=dtype, std=std, norm_jitter=norm_jitter,
                             include_optional=include_bias)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    (out_dir / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    write_safetensors(out_dir / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed), "init": f"normal std={std}"})
    return out_dir
