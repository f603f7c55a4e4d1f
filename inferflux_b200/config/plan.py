"""The architecture-neutral description of a model: which parts each layer is made
of, with which constants, and in which order the layers run.

A configuration class (one per architecture) turns its config.json keys into a
`ModelPlan`.  Everything below the plan (parts, cache manager, step function) reads
only the plan, never an architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part chosen by kind name, with its sizes and constants as parameters."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class SubPart:
    """One part of a layer: its role (mixer, ffn, norm, ...), what it is, and the
    tensor-name infix of its weights below the layer's prefix."""
    role: str
    spec: PartSpec
    infix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it arranges, by the names the
    block kind gives them.  Which parts a layer has is the block kind's business: a
    pre-norm block has `norm_mixer`, `mixer`, `norm_ffn`, `ffn`; another kind may have
    four norms and no feed-forward."""
    prefix: str                 # tensor-name prefix of this layer's weights
    block: PartSpec             # arrangement (e.g. pre-norm residual block)
    parts: Dict[str, SubPart] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.prefix, self.block, tuple(sorted((n, p.role, p.spec, p.infix) for n, p in self.parts.items()))))

    def __getattr__(self, name):            # layer.mixer, layer.norm_ffn, ...: the part's PartSpec
        parts = object.__getattribute__(self, "parts")
        if name in parts:
            return parts[name].spec
        raise AttributeError(name)


_PRENORM_INFIXES = {"mixer": "self_attn.", "ffn": "mlp.", "norm_mixer": "input_layernorm.",
                    "norm_ffn": "post_attention_layernorm."}


def prenorm_layer(prefix: str, mixer: PartSpec, ffn: PartSpec, norm_mixer: PartSpec, norm_ffn: PartSpec,
                  names: Optional[Dict[str, str]] = None, block: Optional[PartSpec] = None) -> LayerSpec:
    """The usual layer: x += mixer(norm(x)); x += ffn(norm(x)).  `names` overrides the
    tensor-name infixes of the four parts (default: the HF names of a Llama-style layer)."""
    infix = dict(_PRENORM_INFIXES)
    infix.update(names or {})
    return LayerSpec(prefix, block or PartSpec("prenorm"), {
        "norm_mixer": SubPart("norm", norm_mixer, infix["norm_mixer"]),
        "mixer": SubPart("mixer", mixer, infix["mixer"]),
        "norm_ffn": SubPart("norm", norm_ffn, infix["norm_ffn"]),
        "ffn": SubPart("ffn", ffn, infix["ffn"]),
    })


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `cache` names the cache (and state) index the mixer
    works on; two entries may name the same layer (weights run twice, each with a
    cache of its own) or the same cache (the later entry reads what the earlier one
    wrote and, with writes_cache False, stores nothing itself)."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    lm_head: PartSpec
    final_norm_prefix: str = "model.norm."
    embedding_prefix: str = "model.embed_tokens."
    lm_head_prefix: str = "lm_head."

    @property
    def num_caches(self) -> int:
        return 1 + max(e.cache for e in self.schedule) if self.schedule else 0

    def validate(self) -> None:
        if not self.schedule:
            raise ValueError("model plan: empty layer schedule")
        writers: Dict[int, int] = {}
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"model plan: schedule entry {i} names layer {e.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if e.cache < 0:
                raise ValueError(f"model plan: schedule entry {i} has a negative cache index")
            if e.writes_cache:
                if e.cache in writers:
                    raise ValueError(f"model plan: cache {e.cache} is written by schedule entries "
                                     f"{writers[e.cache]} and {i}")
                writers[e.cache] = i
            elif e.cache not in writers:
                raise ValueError(f"model plan: schedule entry {i} reads cache {e.cache} "
                                 f"before any entry has written it")
        for c in range(self.num_caches):
            if c not in writers:
                raise ValueError(f"model plan: cache index {c} is never written")

    def cache_owner_layer(self, cache: int) -> int:
        """The layer whose mixer defines what cache index `cache` stores."""
        for e in self.schedule:
            if e.cache == cache and e.writes_cache:
                return e.layer
        raise KeyError(cache)


def default_schedule(num_layers: int) -> List[ScheduleEntry]:
    return [ScheduleEntry(layer=i, cache=i) for i in range(num_layers)]
