"""The step function: run a batch of (request, its next tokens) through the model,
from the cache that earlier steps left, and return the logits at the wanted places.

The reference's counterpart is InferfluxCudaExecutor::ExecuteUnifiedBatch
(runtime/backends/cuda/inferflux_cuda_executor.cpp:3165-3769), which batches the
single-token rows and then runs each prompt portion in a forward call of its own.
Here every token of every entry goes through one forward: portions of prompts beside
single decoded tokens, cut anywhere.  Indices are checked on the host before
anything is launched (the reference does the same for slots and positions,
:3234-3253), so no kernel is ever handed an index outside its tables.
"""
from __future__ import annotations

import os

from typing import Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from .batch import StepContext, StepEntry


class StepError(ValueError):
    """A batch that cannot be run: bad token id, too long, duplicate request."""


class ModelRunner:
    """A loaded model, its cache and the kernel table: everything `step` needs."""

    MAX_GRAPHS = 24
    # A step that is one request's prompt portion of at least this many tokens (chunked prefill brings
    # the same portion size again and again) can be captured too, at its second occurrence; few of these
    # graphs are kept, because each holds the step's activations.  Off unless INFERFLUX_B200_PORTION_GRAPHS=1:
    # measured at the 7B shape a graph saves 0.3 ms on a portion of 129 tokens and nothing on 2,048 (the
    # host is ahead of the device anyway), while its capture stalls one step for 20 ms or more.
    PORTION_GRAPH_MIN_TOKENS = 64
    MAX_PORTION_GRAPHS = 4

    def __init__(self, model, kernels, page_size: int = 16, num_pages: int = 256, max_seqs: int = 8,
                 max_seq_len: Optional[int] = None, cache_dtype: Optional[torch.dtype] = None,
                 cuda_graphs: bool = False):
        self.model = model
        self.kernels = kernels
        self.dtype = model.dtype
        self.device = model.device
        self.vocab_size = model.plan.vocab_size
        limit = model.plan.max_positions
        self.max_seq_len = min(limit, max_seq_len) if max_seq_len else limit
        self.cache = CacheManager(model.cache_specs(), page_size=page_size, num_pages=num_pages,
                                  max_seqs=max_seqs, max_seq_len=self.max_seq_len,
                                  dtype=cache_dtype or model.dtype, device=self.device)
        self.steps = 0
        self.tokens_run = 0
        # Decode-only steps (one token per request, logits of every token) replay a CUDA graph
        # captured per (batch size, context bucket), as the reference does per batch size
        # (runtime/backends/cuda/native/transformer_forward.cu:3071-3101, 4369-4399).
        self.cuda_graphs = bool(cuda_graphs) and self.device.type == "cuda" and all(
            p.graph_safe for _n, p in model.named_parts())
        self._graphs = {}              # key -> [uses, graph or None, static buffer, static logits]
        self._portion_graphs = {}      # the same for prompt portions
        # All graphs allocate from one pool: they never run at the same time, so the activations of one
        # reuse the memory of the others (a graph of its own pool each would hold them all at once).
        self._graph_pool = torch.cuda.graph_pool_handle() if self.cuda_graphs else None
        self.portion_graphs = os.environ.get("INFERFLUX_B200_PORTION_GRAPHS", "0") == "1"
        self.graph_replays = 0

    # ---------------------------------------------------------------- requests
    def add_request(self, rid: Hashable) -> int:
        return self.cache.add_request(rid)

    def end_request(self, rid: Hashable) -> None:
        """Give back the pages and the slot of a finished request."""
        self.cache.free(rid)

    def length(self, rid: Hashable) -> int:
        return self.cache.length(rid)

    # -------------------------------------------------------------------- step
    def validate(self, entries: Sequence[StepEntry]) -> None:
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request_id!r}: no tokens")
            bad = [int(t) for t in e.tokens if not 0 <= int(t) < self.vocab_size]
            if bad:
                raise StepError(f"request {e.request_id!r}: token ids {bad[:8]} are outside the vocabulary "
                                f"of {self.vocab_size}")
            start = self.cache.length(e.request_id) if e.request_id in self.cache else 0
            if e.start is not None and int(e.start) != start:
                raise StepError(f"request {e.request_id!r}: the caller's tokens begin at {e.start}, the cache "
                                f"holds {start}")
            if start + len(e.tokens) > self.max_seq_len:
                raise StepError(f"request {e.request_id!r}: {start + len(e.tokens)} tokens exceed the longest "
                                f"sequence of {self.max_seq_len}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is outside its "
                                    f"{len(e.tokens)} tokens")

    def step(self, entries: Sequence[StepEntry], relay=None) -> torch.Tensor:
        """Run only the tokens given, as one batch.  Returns float32 logits
        [number of wanted places, vocab] in the order of the entries and of `want`.
        Raises OutOfPages (nothing taken, nothing run) when the pool cannot hold the step.
        `relay` = (pairs, ids): for each pair (flat position, row) the token at that position is
        ids[row], an int32 device tensor the previous step's sampling left (the host has not read it)."""
        entries = list(entries)
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        self.validate(entries)
        cache = self.cache
        fresh = [e.request_id for e in entries if e.request_id not in cache]
        if len(fresh) > cache.num_free_slots:
            raise OutOfPages(f"{len(fresh)} new requests but {cache.num_free_slots} free request slots")

        # ---- can the pool hold the whole step?  Decide before taking anything.
        need = [0] * len(cache.groups)
        for e in entries:
            if e.request_id in cache:
                per = cache.pages_needed(e.request_id, cache.length(e.request_id) + len(e.tokens))
            else:
                per = cache.pages_needed_fresh(len(e.tokens))
            need = [a + b for a, b in zip(need, per)]
        free = cache.free_pages()
        if any(n > f for n, f in zip(need, free)):
            raise OutOfPages(f"the step needs {need} pages per cache group, free: {free}")

        for rid in fresh:
            cache.add_request(rid)
        starts, slots = [], []
        try:
            for e in entries:
                start = cache.length(e.request_id)
                cache.reserve(e.request_id, start + len(e.tokens))
                starts.append(start)
                slots.append(cache.slot(e.request_id))
            ctx = StepContext.build(self.kernels, self.dtype, self.device, entries, starts, slots,
                                    cache.drain_table_updates(), relay[0] if relay else None,
                                    providers=getattr(self.model, "section_providers", ()))
            for group, (index, page) in zip(cache.groups, ctx.table_updates):
                self.kernels.scatter_i32(group.table, index, page)
            ctx.relay_ids = relay[1] if relay else None
            logits = self._forward(ctx, entries)
        except BaseException:
            # nothing of this step counts: new requests leave again, the others give back what they took
            for e in entries:
                if e.request_id in fresh:
                    if e.request_id in cache:
                        cache.free(e.request_id)
                elif e.request_id in cache:
                    cache.release_uncommitted(e.request_id)
            raise
        for e, start in zip(entries, starts):
            cache.commit(e.request_id, start + len(e.tokens))
        self.steps += 1
        self.tokens_run += ctx.num_tokens
        self.last_ctx = ctx
        return logits

    # ------------------------------------------------------------------ graphs
    def _relay(self, ctx: StepContext) -> None:
        """Put the tokens that are still on the device into the step's token ids."""
        if ctx.relay_ids is not None and ctx.relay_dst.numel():
            self.kernels.relay_i32(ctx.token_ids, ctx.relay_dst, ctx.relay_ids, ctx.relay_src)

    def _forward(self, ctx: StepContext, entries) -> torch.Tensor:
        decode_only = ctx.max_span == 1 and ctx.num_logit_rows == ctx.num_tokens
        one_portion = self.portion_graphs and len(entries) == 1 and ctx.num_tokens >= self.PORTION_GRAPH_MIN_TOKENS
        if not self.cuda_graphs or not (decode_only or one_portion):
            self._relay(ctx)
            return self.model.forward(ctx, self.cache)
        bucket = 256
        while bucket < ctx.max_kv_len:
            bucket *= 2
        key = (ctx.num_tokens, bucket, ctx.layout_key())
        graphs, most = (self._graphs, self.MAX_GRAPHS) if decode_only else (self._portion_graphs, self.MAX_PORTION_GRAPHS)
        slot = graphs.get(key)
        if slot is None:                                   # first time: run as is (also warms every kernel up)
            if len(graphs) >= most:
                graphs.pop(next(iter(graphs)))
            graphs[key] = [1, None, None, None]
            self._relay(ctx)
            return self.model.forward(ctx, self.cache)
        slot[0] += 1
        if slot[1] is None:                                # second time: capture
            static = torch.empty_like(ctx.core_buffer())
            static.copy_(ctx.core_buffer())
            ctx.rebind(static)
            self._relay(ctx)
            ctx.max_kv_len = bucket                        # what depends on the context is fixed per bucket
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            launches = self.kernels.launches
            with torch.cuda.graph(graph, pool=self._graph_pool):
                static_logits = self.model.forward(ctx, self.cache)
            slot[1], slot[2], slot[3] = graph, static, static_logits
            slot.append(self.kernels.launches - launches)
        else:
            slot[2].copy_(ctx.core_buffer(), non_blocking=True)
            ctx.rebind(slot[2])
            self._relay(ctx)
            self.kernels.launches += slot[4]
        slot[1].replay()
        self.graph_replays += 1
        return slot[3].clone()
