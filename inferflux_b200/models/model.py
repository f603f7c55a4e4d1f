"""A model put together from a `ModelPlan`: embedding, layers (each a block of
parts), the order in which layers run, final norm and head.

The model knows no architecture.  `expected_tensors` gives every tensor name the
plan's parts declare (for checked loading and for random-weights mode); `Model.forward`
runs one step's tokens and returns float32 logits at the rows the step asks for.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.plan import ModelPlan
from ..parts import build_part
from ..weights.loader import TensorSpec


class Layer:
    """A layer's parts, built from its spec, and the block that arranges them."""

    def __init__(self, spec):
        self.spec = spec
        self.parts = {name: build_part(sub.role, sub.spec) for name, sub in spec.parts.items()}
        self.block = build_part("block", spec.block, self.parts)

    def __getattr__(self, name):            # layer.mixer, layer.ffn, ...: the built part
        parts = self.__dict__.get("parts", {})
        if name in parts:
            return parts[name]
        raise AttributeError(name)

    def named_parts(self):
        return [(self.spec.prefix + sub.infix, self.parts[name]) for name, sub in self.spec.parts.items()]


class Model:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding)
        self.layers: List[Layer] = [Layer(s) for s in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm)
        self.lm_head = build_part("lm_head", plan.lm_head)
        self.dtype = None
        self.device = None
        # one part of every class that wants arrays of its own in a step's metadata
        from ..parts.base import Part
        seen = {}
        for _prefix, part in self.named_parts():
            for p in [part] + list(getattr(part, "sub_parts", lambda: [])()):
                if type(p).step_sections is not Part.step_sections:
                    seen.setdefault(type(p), p)
        self.section_providers = list(seen.values())

    # ------------------------------------------------------------------- tensors
    def named_parts(self):
        out = [(self.plan.embedding_prefix, self.embedding)]
        for layer in self.layers:
            out.extend(layer.named_parts())
        out.append((self.plan.final_norm_prefix, self.final_norm))
        out.append((self.plan.lm_head_prefix, self.lm_head))
        return out

    def expected_tensors(self) -> Dict[str, TensorSpec]:
        out = {}
        for prefix, part in self.named_parts():
            for name, spec in part.param_specs().items():
                out[prefix + name] = spec
        return out

    def load(self, tensors, dtype: torch.dtype, device) -> "Model":
        """Hand every part its tensors (already checked against expected_tensors).  `tensors` is a
        dict name -> tensor, or a function that brings the tensors of the names it is given (a
        part at a time, so that only one part's unpacked tensors exist beside the model)."""
        self.dtype, self.device = dtype, torch.device(device)
        for prefix, part in self.named_parts():
            names = [prefix + n for n in part.param_specs()]
            got = tensors(names) if callable(tensors) else tensors
            own = {n[len(prefix):]: got[n] for n in names if n in got}
            del got
            if part is self.lm_head:
                part.load(own, dtype, device, tied_table=self.embedding.table)
            else:
                part.load(own, dtype, device)
            del own
        return self

    # ------------------------------------------------------------------ cache needs
    def cache_specs(self):
        """Per cache index: (KVCacheSpec or None, StateSpec or None), from the part
        that the block of the writing layer names as the one that stores."""
        out = []
        for c in range(self.plan.num_caches):
            part = self.layers[self.plan.cache_owner_layer(c)].block.cache_part()
            out.append((None, None) if part is None else (part.cache_spec(), part.state_spec()))
        return out

    # --------------------------------------------------------------------- forward
    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the step described by `ctx`; `caches.view(entry)` gives the cache of a
        schedule entry.  Returns float32 logits [len(ctx.logit_rows), vocab]."""
        k = ctx.kernels
        x = self.embedding.forward(ctx)                       # float32 [T, hidden]
        pending = None
        for entry in self.plan.schedule:
            x, pending = self.layers[entry.layer].block.forward(x, pending, ctx, caches.view(entry))
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=x.device)
        if pending is not None:
            k.residual_add(x, pending)
        rows = k.gather_rows(x, ctx.logit_rows)               # float32 [R, hidden]
        h = self.final_norm.forward(rows, None, ctx)
        return self.lm_head.forward(h, ctx)


def expected_tensors(plan: ModelPlan) -> Dict[str, TensorSpec]:
    return Model(plan).expected_tensors()
