"""Interfaces of the parts a layer is made of, and the registries that map a part's
kind name to its class.

A part is built from a `PartSpec` (kind + parameters): it never learns which model
it is in.  It declares the tensors it needs (`param_specs`), takes them (`load`) and
does its work through the kernel table of the step (`ctx.kernels`).

    Norm              forward(x, delta=None, ctx) -> h
    PositionEncoding  rotary() -> RotaryTable or None
    Mixer             cache_spec() / state_spec(); forward(h, ctx, cache) -> y
    FeedForward       forward(h, ctx) -> y
    Block             sub_parts (name -> role); forward(x, pending, ctx, cache) -> (x, pending)

`x` is the float32 residual stream [tokens, hidden]; `h` and `y` are in the dtype
the run computes in.  `pending` is a delta that has not been added to `x` yet, so
that the next norm can add it and normalise in one kernel.  A delta (and so a `y`)
may be a plain tensor or what `ctx.kernels.linear(..., allow_partial=True)` returned:
the partial sums of a K-split product, which `add_rmsnorm`, `residual_add` and
`rope_append` add in the same pass; `ctx.kernels.materialize(y)` gives the tensor.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch

from ..config.plan import PartSpec
from ..weights.loader import TensorSpec


# --------------------------------------------------------------------- cache needs

@dataclass(frozen=True)
class KVCacheSpec:
    """What a mixer stores per token: keys and values of `num_kv_heads` heads of
    `head_dim`; `window` None keeps every key, an integer only the last `window`."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """What a mixer stores per request, whatever the request's length."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class RotaryTable:
    """A rotation of the first `rotary_dim` elements of every head: inverse
    frequencies [rotary_dim / 2] in float32 and how elements pair up."""
    inv_freq: torch.Tensor
    rotary_dim: int
    interleaved: bool            # False: (i, i + rotary_dim/2); True: (2i, 2i+1)


# ------------------------------------------------------------------ weight storage

class WeightBuffers:
    """The tensors a part keeps, carved out of ONE device allocation at offsets that are
    multiples of 256 bytes (TMA wants 16; 256 keeps every tensor on a fresh sector line).
    The reference packs a whole model into one cudaMalloc with no padding
    (runtime/backends/cuda/inferflux_cuda_executor.cpp:648-702); here each part packs its
    own, and a stacked matrix is filled slice by slice from the file's tensors, so that no
    second copy of it ever exists on the device.

        buf = WeightBuffers(device, {"w_qkv": ((q + 2 * kv, h), dtype), "b_qkv": ((q + 2 * kv,), torch.float32)})
        buf["w_qkv"][:q].copy_(tensors["q_proj.weight"])
    """

    ALIGN = 256

    def __init__(self, device, layout: Dict[str, Tuple[Tuple[int, ...], torch.dtype]]):
        offsets, total = {}, 0
        for name, (shape, dtype) in layout.items():
            n = torch.empty(0, dtype=dtype).element_size()
            for d in shape:
                n *= int(d)
            offsets[name] = (total, n)
            total += -(-n // self.ALIGN) * self.ALIGN
        self.storage = torch.empty(total + self.ALIGN, dtype=torch.uint8, device=device)
        shift = (-self.storage.data_ptr()) % self.ALIGN      # 0 on the GPU, whose allocator aligns to 512 bytes
        self.views = {name: self.storage[shift + off:shift + off + n].view(layout[name][1]).view(layout[name][0])
                      for name, (off, n) in offsets.items()}
        self.nbytes = total

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.views[name]


# --------------------------------------------------------------------------- parts

class Part:
    """Base of all parts."""

    # False for a part whose forward reads device data on the host or launches work whose
    # shape depends on the data: a step that holds such a part is never captured into a CUDA graph.
    graph_safe = True
    # True for a mixer or feed-forward that hands its input `h` only to `ctx.kernels.linear` /
    # `linear_swiglu`: the norm in front may then leave its row scale to that product
    # (`h` arrives as the kernels' pre-normed rows instead of a tensor).
    takes_scaled_rows = False

    def __init__(self, spec: PartSpec):
        self.spec = spec

    def param_specs(self) -> Dict[str, TensorSpec]:
        """Tensor names (relative to the part's prefix) this part expects."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Take the tensors named by `param_specs` (absent optional ones are left
        out of `tensors`) and keep them in the form the kernels want."""

    def step_sections(self, ctx) -> Dict[str, list]:
        """Int32 lists that parts of this class want on the device for the step `ctx`
        describes (`ctx.spans`, `ctx.slots_host`, `ctx.kv_lens_host` are set): work
        lists of its kernels, for instance.  They travel in the step's one metadata
        copy and are found in `ctx.extra[name]` (a flat int32 device array) with
        `ctx.extra_len[name]`; names carry the class's own prefix.  Called once per
        step on one part of each class, so the lists may depend on the step only, not
        on the part's parameters."""
        return {}


class Norm(Part):
    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], ctx, lazy: bool = False) -> torch.Tensor:
        """`lazy`: the consumer takes pre-normed rows (see Part.takes_scaled_rows)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary(self, device) -> Optional[RotaryTable]:
        """The rotation the mixer applies to queries and keys, or None."""
        return None


class Mixer(Part):
    def cache_spec(self) -> Optional[KVCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of parts around the residual stream.  A block kind says which
    parts it arranges (`sub_parts`: name -> role); the layer's spec must bring exactly
    those, and `forward` finds them under their names as attributes."""

    sub_parts: Dict[str, str] = {}

    def __init__(self, spec, parts: Dict[str, Part]):
        super().__init__(spec)
        missing = sorted(set(self.sub_parts) - set(parts))
        extra = sorted(set(parts) - set(self.sub_parts))
        if missing or extra:
            raise ValueError(f"block {spec.kind!r} arranges {sorted(self.sub_parts)}; the layer lacks {missing} "
                             f"and brings {extra} besides")
        self.parts = dict(parts)
        for name, part in parts.items():
            setattr(self, name, part)

    def cache_part(self) -> Optional[Part]:
        """The part whose `cache_spec()` / `state_spec()` say what this layer stores (None: nothing)."""
        return self.parts.get("mixer")

    def forward(self, x, pending, ctx, cache):
        raise NotImplementedError


# ---------------------------------------------------------------------- registries

_REGISTRIES: Dict[str, Dict[str, type]] = {
    "mixer": {}, "ffn": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "lm_head": {},
}


def register_part(role: str, kind: str) -> Callable[[type], type]:
    """Class decorator: make `kind` available for `role` (mixer, ffn, norm,
    position, block, embedding, lm_head)."""
    if role not in _REGISTRIES:
        raise KeyError(f"unknown part role {role!r}; roles: {sorted(_REGISTRIES)}")

    def deco(cls: type) -> type:
        _REGISTRIES[role][kind] = cls
        return cls
    return deco


def build_part(role: str, spec: PartSpec, *args, **kwargs):
    table = _REGISTRIES[role]
    if spec.kind not in table:
        raise KeyError(f"no {role} of kind {spec.kind!r} is registered; known: {sorted(table)}")
    return table[spec.kind](spec, *args, **kwargs)


def registered_parts(role: str):
    return sorted(_REGISTRIES[role])
