"""The Python entry point: from a model folder (or a configuration and a seed) to
generated token ids on one GPU.

The reference has no Python binding; its in-process surface is
NativeGpuBackend::LoadModel / Generate (runtime/backends/native/
native_gpu_backend.cpp:76-167, 594-834) and Scheduler::Generate
(scheduler/scheduler.cpp:1763).  Option names follow the reference where it has
them: SamplingParams fields (scheduler/request_batch.h:26-38), the scheduler's
max_batch_size / max_batch_tokens / chunked_prefill_tokens /
mixed_prefill_budget_ratio (scheduler/scheduler.h:74-84), `max_tokens` (default 256,
cli/main.cpp:1587), and the cache sizing knobs kv_max_batch / kv_max_seq /
kv_budget_mb / kv_budget_ratio (runtime/backends/cuda/native/
native_bootstrap_config.h:10-20) with 16-token pages (scheduler/scheduler.cpp:293).
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence, Union

import torch

from ..models.loading import load_model, parse_dtype, random_model
from ..sampling import Sampler, SamplingParams, SamplingRow
from .runner import ModelRunner
from .scheduler import PENDING, Request, Scheduler, SchedulerConfig, StepPlan


@dataclass
class GenerationResult:
    request_id: Hashable
    prompt_tokens: int
    token_ids: List[int]
    finish_reason: str
    preemptions: int = 0

    @property
    def completion_tokens(self) -> int:
        return len(self.token_ids)


@dataclass
class _Inflight:
    """A step that has been launched and whose sampled tokens have not been read yet."""
    plan: StepPlan
    ids: Optional[torch.Tensor]              # int32 on the device, one per entry that wanted logits
    host: Optional[torch.Tensor]             # pinned copy under way (CUDA)
    event: Optional[object]
    row_of: dict                             # request id -> its row in `ids`
    flag: Optional[torch.Tensor] = None      # pinned copy of the kernels' error flag, taken with the ids


@dataclass
class EngineStats:
    steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0


class Engine:
    def __init__(self, model=None, dtype="bfloat16", device="cuda:0", *, config=None, seed: int = 0,
                 kernels=None, kv_page_size: int = 16, kv_num_pages: Optional[int] = None,
                 kv_max_batch: int = 16, kv_max_seq: Optional[int] = None, kv_budget_mb: Optional[float] = None,
                 kv_budget_ratio: float = 0.20, max_batch_size: int = 32, max_batch_tokens: int = 16384,
                 chunked_prefill_tokens: int = 512, mixed_prefill_budget_ratio: float = 1.0,
                 sampling_seed: int = 0, cuda_graphs: bool = True, overlap_steps: bool = True,
                 loaded_model=None):
        """`model`: a folder with config.json and model.safetensors.  Without it,
        `config` (a typed configuration) and `seed` make random weights on the device."""
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        if kernels is None:
            from ..csrc import CudaKernels            # raises if the library cannot be built or no GPU is there
            kernels = CudaKernels(self.device)
        self.kernels = kernels
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        if loaded_model is not None:
            self.config, self.model = config, loaded_model
        elif model is not None:
            self.config, self.model = load_model(model, dtype=self.dtype, device=self.device)
        elif config is not None:
            self.config, self.model = config, random_model(config, seed=seed, dtype=self.dtype, device=self.device)
        else:
            raise ValueError("Engine needs a model folder, or a configuration for random weights")

        max_seq = min(self.model.plan.max_positions, kv_max_seq) if kv_max_seq else self.model.plan.max_positions
        max_seqs = max(int(kv_max_batch), 1)
        if kv_num_pages is None:
            kv_num_pages = self._plan_pages(kv_page_size, max_seqs, max_seq, kv_budget_mb, kv_budget_ratio)
        self.runner = ModelRunner(self.model, kernels, page_size=kv_page_size, num_pages=kv_num_pages,
                                  max_seqs=max_seqs, max_seq_len=max_seq, cuda_graphs=cuda_graphs)
        self.scheduler = Scheduler(SchedulerConfig(max_batch_size=min(max_batch_size, max_seqs),
                                                   max_batch_tokens=max_batch_tokens,
                                                   chunked_prefill_tokens=chunked_prefill_tokens,
                                                   mixed_prefill_budget_ratio=mixed_prefill_budget_ratio),
                                   self.runner.cache, max_seq)
        self.sampler = Sampler(kernels, self.device)
        # With overlap_steps a step is launched before the tokens of the one before are read: the
        # scheduler, the packing of the batch and the launches run while the GPU works, and a token
        # goes from one step's sampling to the next step's embedding on the device.
        self.overlap_steps = bool(overlap_steps)
        self._inflight: Optional[_Inflight] = None
        self._rng = random.Random(sampling_seed)
        self._next_id = 0
        self.stats = EngineStats()

    @classmethod
    def from_spec(cls, spec, **overrides) -> "Engine":
        """An engine for a `ModelLoadSpec` (what the command line and the replay program build)."""
        kw = spec.checked().engine_kwargs()
        kw.update(overrides)
        return cls(spec.path, **kw)

    # ------------------------------------------------------------------ sizing
    def bytes_per_token(self) -> int:
        """Cache bytes one token takes over all caches (2 . layers . kv_heads . head_dim . itemsize
        for a plain decoder, runtime/backends/cuda/native/kv_cache_planner.h:22-37)."""
        item = torch.empty(0, dtype=self.dtype).element_size()
        return sum(2 * kv.num_kv_heads * kv.head_dim * item for kv, _st in self.model.cache_specs() if kv)

    def state_bytes_per_request(self) -> int:
        """Bytes of fixed-size state one request slot takes over all caches."""
        total = 0
        for _kv, st in self.model.cache_specs():
            if st is not None:
                n = torch.empty(0, dtype=st.dtype).element_size()
                for s in st.shape:
                    n *= int(s)
                total += n
        return total

    def _plan_pages(self, page_size, max_seqs, max_seq, budget_mb, ratio) -> int:
        """Pages that fit the budget once the state slots of `max_seqs` requests are paid for."""
        per_page = max(1, self.bytes_per_token() * page_size)
        if budget_mb is not None:
            budget = int(budget_mb * 1024 * 1024)
        elif self.device.type == "cuda":
            free, _total = torch.cuda.mem_get_info(self.device)
            budget = int(free * ratio)
        else:
            budget = 64 * 1024 * 1024
        pages = max(0, budget - max_seqs * self.state_bytes_per_request()) // per_page
        most = max_seqs * (-(-max_seq // page_size))          # more than this can never be in use
        return int(max(1, min(pages, most)))

    # ---------------------------------------------------------------- requests
    def add_request(self, prompt_token_ids: Sequence[int], sampling_params: Optional[SamplingParams] = None,
                    max_tokens: int = 256, eos_token_id: Union[None, int, Sequence[int]] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        params = sampling_params or SamplingParams()
        vocab = self.model.plan.vocab_size
        prompt = [int(t) for t in prompt_token_ids]
        bad = [t for t in prompt if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"prompt token ids {bad[:8]} are outside the vocabulary of {vocab}")
        if request_id is None:
            request_id = f"req-{self._next_id}"
        self._next_id += 1
        eos = () if eos_token_id is None else ((eos_token_id,) if isinstance(eos_token_id, int) else tuple(eos_token_id))
        seed = params.seed if params.seed is not None else self._rng.getrandbits(63)
        self.scheduler.add(Request(request_id, prompt, params, max_tokens=max_tokens, eos_token_ids=eos, seed=seed))
        return request_id

    def abort(self, request_id: Hashable) -> Optional[GenerationResult]:
        """Stop a request now.  Its pages and slot go back to the pool at once, or, if the step in
        flight still owes it a token, when that step's tokens are read (the next `step()` or `drain()`
        then reports it with finish_reason "abort").  Returns the result if it is final already."""
        r = self.scheduler.abort(request_id)
        return None if r is None else self._result(r)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    # -------------------------------------------------------------------- step
    def step(self) -> List[GenerationResult]:
        """One scheduler decision, one model step, one sampling call.  Returns the requests
        that finished (failed ones included).  With `overlap_steps` the tokens of a step are
        read while the next step runs, so a request's finish is reported one step later."""
        results: List[GenerationResult] = []
        prev = self._inflight
        overlap = self.overlap_steps and not any(r.params.has_penalties for r in self.scheduler.running)
        if prev is not None and not overlap:
            results += self._finalize(prev)
            prev = self._inflight = None
        plan = self.scheduler.schedule(inflight=prev is not None)
        if plan.needs_drain:
            results += self._finalize(prev)
            prev = self._inflight = None
            plan = self.scheduler.schedule()
        results += [self._result(r) for r in plan.failed]
        launched = None
        if plan.entries:
            entries = plan.step_entries()
            relay, flat = [], 0
            for e, se in zip(plan.entries, entries):
                if se.tokens and se.tokens[-1] == PENDING:      # sampled by the step in flight, still on the device
                    se.tokens = list(se.tokens[:-1]) + [0]
                    relay.append((flat + len(se.tokens) - 1, prev.row_of[e.request.request_id]))
                flat += len(se.tokens)
            logits = self.runner.step(entries, relay=(relay, prev.ids) if relay else None)
            rows = [SamplingRow(e.request.params, e.request.seed, len(e.request.output), e.request.output)
                    for e in plan.entries if e.wants_logits]
            ids = host = event = flag = None
            if rows:
                ids = self.sampler.sample(logits, rows)
                if ids.is_cuda:
                    host = torch.empty(ids.shape, dtype=ids.dtype, pin_memory=True)
                    host.copy_(ids, non_blocking=True)          # the step's device-to-host read
                    err = getattr(self.kernels, "error_flag", None)
                    if err is not None:                         # a kernel whose bounded wait ran out set it
                        flag = torch.empty(1, dtype=err.dtype, pin_memory=True)
                        flag.copy_(err, non_blocking=True)
                    event = torch.cuda.Event()
                    event.record()
                self.stats.d2h_bytes += 4 * len(rows) + (4 if flag is not None else 0)
            self.scheduler.advance(plan)
            wanting = [e.request.request_id for e in plan.entries if e.wants_logits]
            launched = _Inflight(plan, ids, host, event, {rid: i for i, rid in enumerate(wanting)}, flag)
            self.stats.h2d_bytes += self.runner.last_ctx.meta_bytes
            self.stats.steps += 1
            self.stats.prompt_tokens += sum(e.count for e in plan.entries if e.count > 1 or not e.request.output)
            self.stats.generated_tokens += len(rows)
        if prev is not None:
            results += self._finalize(prev)
        self._inflight = launched
        if launched is not None and not overlap:
            results += self._finalize(launched)
            self._inflight = None
        self.stats.preemptions = self.scheduler.num_preemptions
        return results

    def _finalize(self, step: _Inflight) -> List[GenerationResult]:
        """Read a launched step's tokens and let the scheduler account for them."""
        if step.ids is None:
            sampled: List[int] = []
        elif step.host is not None:
            step.event.synchronize()
            sampled = step.host.tolist()
        else:
            sampled = step.ids.tolist()
        if step.flag is not None and int(step.flag[0]) != 0:
            self.kernels.check_errors()                     # raises before the tokens of an invalid step are used
        return [self._result(r) for r in self.scheduler.resolve(step.plan, sampled)]

    def drain(self) -> List[GenerationResult]:
        """Read the tokens of the step in flight, if any."""
        if self._inflight is None:
            return []
        out = self._finalize(self._inflight)
        self._inflight = None
        if hasattr(self.kernels, "check_errors"):
            self.kernels.check_errors()
        return out

    @staticmethod
    def _result(r: Request) -> GenerationResult:
        return GenerationResult(r.request_id, len(r.prompt), list(r.output), r.finish_reason or "", r.preemptions)

    # ---------------------------------------------------------------- generate
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[None, SamplingParams, Sequence[SamplingParams]] = None,
                 max_tokens: int = 256, eos_token_id=None) -> List[GenerationResult]:
        """Generate for every prompt (lists of token ids); results come back in the
        order of the prompts."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        ids = [self.add_request(p, sp, max_tokens=max_tokens, eos_token_id=eos_token_id)
               for p, sp in zip(prompts, sampling_params)]
        done = {}
        guard = 0
        while self.has_unfinished():
            for res in self.step():
                done[res.request_id] = res
            guard += 1
            if guard > 10_000_000:
                raise RuntimeError("generation did not finish")
        if hasattr(self.kernels, "check_errors"):
            self.kernels.check_errors()                     # steps without sampled tokens carry no flag copy
        return [done[i] for i in ids]
