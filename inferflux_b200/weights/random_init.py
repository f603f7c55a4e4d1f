"""Random-weights mode: make up a model from a configuration and a seed.

Linear weights, tables and biases are N(0, std) with std 0.02, norm weights are 1.0
(optionally jittered so that tests see a fault in how a norm weight is used).

Element i of a tensor is a function of (seed, tensor name, i) alone, so the same seed
gives the same bits wherever the tensor is made: here with numpy on the host, or by the
kernel `ifx_random_normal` (csrc/random_init.cu) on the GPU.  Two Philox4x32-10 blocks
keyed by the seed and the name's crc32 give sixteen 16-bit integers; their sum, centred
and scaled, is a variable of variance 1 that is normal up to an excess kurtosis of
-0.075, which the cubic z + c (z^3 - 3 z) takes out to first order.  All float32 steps are
single correctly rounded operations; bfloat16 models round the float32 value once.
"""
from __future__ import annotations

import ctypes
import json
import zlib
from pathlib import Path
from typing import Dict

import numpy as np
import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors

_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_SCALE = np.float32(6.6072494e-06)          # 1 / (2 sqrt(16 (65536^2 - 1) / 12))
_CUBIC = np.float32(0.003125)               # 0.075 / 24
_CHUNK = 1 << 21


def tensor_key(seed: int, name: str):
    """The two 32-bit key words of a tensor's generator."""
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    return seed & 0xFFFFFFFF, ((seed >> 32) ^ zlib.crc32(name.encode("utf-8"))) & 0xFFFFFFFF


def _philox(key0: int, key1: int, c0, c1, c2, c3):
    """Philox4x32-10 on uint64 arrays that hold 32-bit words."""
    k0, k1 = np.uint64(key0), np.uint64(key1)
    for _ in range(10):
        p0, p1 = np.uint64(_M0) * c0, np.uint64(_M1) * c2           # 32 x 32 bits: exact in 64
        c0, c1, c2, c3 = (p1 >> np.uint64(32)) ^ c1 ^ k0, p1 & _MASK, (p0 >> np.uint64(32)) ^ c3 ^ k1, p0 & _MASK
        k0, k1 = (k0 + np.uint64(_W0)) & _MASK, (k1 + np.uint64(_W1)) & _MASK
    return c0, c1, c2, c3


def counter_normal_numpy(n: int, key0: int, key1: int, mean: float, std: float, first: int = 0) -> np.ndarray:
    """float32 values of elements [first, first + n) of the tensor with key (key0, key1)."""
    i = np.arange(first, first + n, dtype=np.uint64)
    lo, hi, zero = i & _MASK, i >> np.uint64(32), np.zeros(n, dtype=np.uint64)
    total = np.zeros(n, dtype=np.int64)
    for block in (0, 1):
        for w in _philox(key0, key1, lo, hi, np.full(n, block, dtype=np.uint64), zero):
            total += (w & np.uint64(0xFFFF)).astype(np.int64) + (w >> np.uint64(16)).astype(np.int64)
    t = (2 * total - 16 * 65535).astype(np.float32)
    z = t * _SCALE
    z3 = (z * z) * z
    z = z + _CUBIC * (z3 - np.float32(3.0) * z)
    return np.float32(mean) + np.float32(std) * z


def counter_normal(shape, seed: int, name: str, mean: float, std: float, dtype=torch.float32,
                   device="cpu") -> torch.Tensor:
    """The tensor `name` of the model with seed `seed`: the same bits on every device."""
    n = 1
    for s in shape:
        n *= int(s)
    key0, key1 = tensor_key(seed, name)
    dev = torch.device(device)
    if dev.type == "cuda":
        from ..csrc.build import load_library
        lib = load_library()
        lib.ifx_random_normal.restype = ctypes.c_int
        out = torch.empty(tuple(shape), dtype=dtype, device=dev)
        code = {torch.float32: 0, torch.bfloat16: 1}.get(dtype)
        if code is None:
            raise ValueError(f"random weights are made in float32 or bfloat16, not {dtype}")
        with torch.cuda.device(dev):
            rc = lib.ifx_random_normal(ctypes.c_void_p(out.data_ptr()), ctypes.c_longlong(n), ctypes.c_uint(key0),
                                       ctypes.c_uint(key1), ctypes.c_float(mean), ctypes.c_float(std), code,
                                       ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        if rc != 0:
            raise RuntimeError(f"ifx_random_normal failed with code {rc}")
        return out
    out = torch.empty(n, dtype=torch.float32)
    view = out.numpy()
    for first in range(0, n, _CHUNK):
        m = min(_CHUNK, n - first)
        view[first:first + m] = counter_normal_numpy(m, key0, key1, mean, std, first)
    return out.reshape(tuple(shape)).to(dtype)


def random_tensors(expected: Dict[str, TensorSpec], seed: int, dtype=torch.bfloat16, device="cpu",
                   std: float = 0.02, norm_jitter: float = 0.0) -> Dict[str, torch.Tensor]:
    """One tensor per entry of `expected`.  Values are made in float32 and rounded once to
    `dtype`.  An optional tensor (a bias that a file may leave out) is made if its
    spec says `invent`."""
    out = {}
    dev = torch.device(device)
    for name, spec in expected.items():
        if spec.ignored or (spec.optional and not spec.invent):
            continue
        if spec.init == "normal":
            t = counter_normal(spec.shape, seed, name, 0.0, std, dtype, dev)
        elif spec.init == "ones":
            if norm_jitter:
                t = counter_normal(spec.shape, seed, name, 1.0, norm_jitter, dtype, dev)
            else:
                t = torch.ones(spec.shape, dtype=dtype, device=dev)
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
    tensors = random_tensors(expected_tensors(config.to_plan()), seed, dtype=dtype, std=std, norm_jitter=norm_jitter)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    (out_dir / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    write_safetensors(out_dir / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed), "init": f"normal std={std}"})
    return out_dir
