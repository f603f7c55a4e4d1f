"""From a model folder (or a configuration and a seed) to a loaded `Model`."""
from __future__ import annotations

import torch

from ..config import load_config
from ..weights import WeightSource, random_tensors
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}") from None


def load_model(model_dir, dtype="bfloat16", device="cuda"):
    """(config, model) of a folder with config.json and model.safetensors; the model
    class is chosen by config.json through the architecture registry."""
    dtype = parse_dtype(dtype)
    config = load_config(model_dir)
    model = Model(config.to_plan())
    with WeightSource(model_dir, model.expected_tensors(), device=device, run_dtype=dtype) as source:
        model.load(source.take, dtype, device)              # part by part
    return config, model


def random_model(config, seed=0, dtype="bfloat16", device="cuda", std=0.02, norm_jitter=0.0):
    """A model with made-up weights, generated on `device` without touching disk."""
    dtype = parse_dtype(dtype)
    model = Model(config.to_plan())
    store = torch.float32 if dtype == torch.float32 else torch.bfloat16
    expected = model.expected_tensors()

    def make(names):                                        # part by part, as a folder is loaded
        return random_tensors({n: expected[n] for n in names}, seed, dtype=store, device=device, std=std,
                              norm_jitter=norm_jitter)
    return model.load(make, dtype, device)
