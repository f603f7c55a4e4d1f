"""One step's batch: what the caller gives (`StepEntry`) and what the kernels read
(`StepContext`).

The reference's batch input is (sequence_id, n_past, tokens, request_logits) per
request (runtime/backends/common/backend_types.h:22-34); a row with one token and
logits is a decode row, anything else a prompt portion
(runtime/backends/cuda/inferflux_cuda_executor.cpp:3231-3263).  Here the spans of
all requests are laid end to end in one flat token array, and every per-token and
per-request array the kernels need is packed into one int32 buffer that crosses to
the device in a single copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import torch

@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)
    start: Optional[int] = None       # where the caller believes these tokens begin; checked against the cache


class StepContext:
    """Device arrays of one step.  All int32.

    token_ids[T], positions[T], token_req[T] (index of the token's request in this
    batch), cu_seqlens[R+1] (span boundaries in the flat arrays), kv_lens[R]
    (tokens stored once the step is done), req_slot[R] (row of the block tables and
    of the state tensors), logit_rows[W] (flat token indices whose logits are
    wanted).  What else a kind of part wants on the device for a step (work lists of
    its kernels, say) it declares through `Part.step_sections`; those arrays travel in
    the same copy and are found in `extra[name]`, their lengths in `extra_len[name]`.
    """

    def __init__(self, kernels, dtype, device):
        self.kernels = kernels
        self.dtype = dtype
        self.device = torch.device(device)
        self.num_tokens = 0
        self.num_requests = 0
        self.num_logit_rows = 0
        self.max_kv_len = 0
        self.max_span = 0
        # host copies, for parts written in plain torch and for tests
        self.spans: List[tuple] = []            # (first position, number of tokens) per request
        self.kv_lens_host: List[int] = []
        self.slots_host: List[int] = []
        self.request_ids: List[Hashable] = []
        self.extra: Dict[str, torch.Tensor] = {}
        self.extra_len: Dict[str, int] = {}

    @classmethod
    def build(cls, kernels, dtype, device, entries: Sequence[StepEntry], starts: Sequence[int],
              slots: Sequence[int], table_updates: Sequence[Sequence[tuple]] = (),
              relay: Optional[Sequence[tuple]] = None, providers: Sequence = ()):
        """Pack the arrays for `entries`; `starts[i]` is how many tokens request i
        already holds, `slots[i]` its slot, `table_updates[g]` the block-table
        entries of group g that changed since the last step; `providers` are parts
        whose `step_sections(ctx)` adds int32 lists of their own."""
        ctx = cls(kernels, dtype, device)
        token_ids, positions, token_req, cu, kv_lens = [], [], [], [0], []
        logit_rows = []
        for r, (e, start) in enumerate(zip(entries, starts)):
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request_id!r}: a step entry needs at least one token")
            base = cu[-1]
            token_ids.extend(int(t) for t in e.tokens)
            positions.extend(range(start, start + n))
            token_req.extend([r] * n)
            cu.append(base + n)
            kv_lens.append(start + n)
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"request {e.request_id!r}: wanted place {w} is outside its {n} tokens")
                logit_rows.append(base + int(w))
            ctx.spans.append((start, n))
        ctx.num_tokens = cu[-1]
        ctx.num_requests = len(entries)
        ctx.num_logit_rows = len(logit_rows)
        ctx.kv_lens_host = kv_lens
        ctx.slots_host = list(slots)
        ctx.request_ids = [e.request_id for e in entries]
        ctx.max_kv_len = max(kv_lens)
        ctx.max_span = max(n for _s, n in ctx.spans)

        sections: Dict[str, List[int]] = {
            "token_ids": token_ids, "positions": positions, "token_req": token_req,
            "cu_seqlens": cu, "kv_lens": kv_lens, "req_slot": list(slots),
            "logit_rows": logit_rows,
        }
        ctx._extra_names = []
        for part in providers:
            for name, vals in part.step_sections(ctx).items():
                if name in sections:
                    raise ValueError(f"step section {name!r} is declared twice")
                sections[name] = list(vals)
                ctx._extra_names.append(name)
        for g, ups in enumerate(table_updates):
            sections[f"upd_index_{g}"] = [u[0] for u in ups]
            sections[f"upd_page_{g}"] = [u[1] for u in ups]
        # tokens that the previous step sampled and that are still on the device: (flat position here, row there)
        sections["upd_relay_dst"] = [d for d, _s in (relay or ())]
        sections["upd_relay_src"] = [s_ for _d, s_ in (relay or ())]
        offsets, flat = {}, []
        core_len = 0
        for name, vals in sections.items():
            offsets[name] = (len(flat), len(vals))
            flat.extend(vals)
            flat.extend([0] * ((-len(flat)) % 4))                 # keep every section 16-byte aligned
            if not name.startswith("upd_"):
                core_len = len(flat)                              # the updates come last
        host = torch.tensor(flat if flat else [0], dtype=torch.int32)
        if ctx.device.type == "cuda":
            host = host.pin_memory()
            dev = host.to(ctx.device, non_blocking=True)
        else:
            dev = host
        ctx._host_buffer = host                                   # keep pinned memory alive until the copy ran
        ctx.meta_bytes = host.numel() * 4
        ctx._offsets, ctx._core_len, ctx._buffer = offsets, core_len, dev
        ctx._bind(dev)
        ctx.table_updates = [(dev[offsets[f"upd_index_{g}"][0]:][:offsets[f"upd_index_{g}"][1]],
                              dev[offsets[f"upd_page_{g}"][0]:][:offsets[f"upd_page_{g}"][1]])
                             for g in range(len(table_updates))]
        ctx.relay_dst = dev[offsets["upd_relay_dst"][0]:][:offsets["upd_relay_dst"][1]]
        ctx.relay_src = dev[offsets["upd_relay_src"][0]:][:offsets["upd_relay_src"][1]]
        return ctx

    _CORE = ("token_ids", "positions", "token_req", "cu_seqlens", "kv_lens", "req_slot", "logit_rows")

    def _bind(self, buffer):
        for name in self._CORE:
            off, n = self._offsets[name]
            setattr(self, name, buffer[off:off + n])
        for name in self._extra_names:
            off, n = self._offsets[name]
            self.extra[name] = buffer[off:off + n]
            self.extra_len[name] = n

    def layout_key(self):
        """Two steps with the same key have their arrays at the same offsets."""
        return tuple(self._offsets[n] for n in self._CORE) + tuple((n, self._offsets[n]) for n in self._extra_names)

    def core_buffer(self):
        return self._buffer[:self._core_len]

    def rebind(self, static_buffer):
        """Point the arrays at `static_buffer` (same layout), e.g. the fixed addresses a
        captured CUDA graph reads."""
        self._bind(static_buffer)
