"""One load contract for every way of starting the engine: the command line, the
replay program and Python callers build a `ModelLoadSpec` and hand it over.

The reference's struct of the same name (model/model_load_spec.h:17-37, validated in
model/model_load_spec.cpp:38-59) carries id, path, format, device, context_size,
max_parallel_sequences and kv_cache_type for a server that holds many models.  Here one
process holds one model, so the spec names that model and the sizes of its cache and
batches; the names the reference has are kept (`path`, `format`, `device`,
`context_size`, `max_parallel_sequences`, `kv_cache_type`), the rest are the engine's
own knobs under the names `Engine` takes them.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from pathlib import Path
from typing import Optional


@dataclass
class ModelLoadSpec:
    path: str                                   # folder with config.json and model.safetensors
    id: str = ""                                # name to report; default: the folder's name
    format: str = "auto"                        # auto | safetensors (the only format this engine reads)
    dtype: str = "bfloat16"                     # bfloat16 | float32: what the run computes in
    device: str = "cuda:0"
    context_size: Optional[int] = None          # longest sequence; default: the model's max_position_embeddings
    max_parallel_sequences: int = 16            # request slots
    kv_cache_type: str = "auto"                 # auto = the run's dtype (quantized caches are not built)
    kv_page_size: int = 16
    kv_num_pages: Optional[int] = None          # default: from the budget below
    kv_budget_mb: Optional[float] = None
    kv_budget_ratio: float = 0.20               # share of free device memory for the cache
    max_batch_size: int = 32
    max_batch_tokens: int = 16384
    chunked_prefill_tokens: int = 512
    cuda_graphs: bool = True
    overlap_steps: bool = True

    def validate(self) -> str:
        """"" if the spec can be loaded, else the reason (the reference's Validate() answers the same way)."""
        if not self.path:
            return "path must name a model folder"
        if self.format not in ("auto", "safetensors"):
            return "format must be auto or safetensors"
        if self.dtype not in ("bfloat16", "bf16", "float32", "fp32"):
            return "dtype must be bfloat16 or float32"
        if not re.fullmatch(r"cuda(:\d+)?", self.device):
            return "device must be cuda:N"
        if self.context_size is not None and self.context_size <= 0:
            return "context_size must be positive"
        if not 1 <= self.max_parallel_sequences <= 256:
            return "max_parallel_sequences must be between 1 and 256"
        if self.kv_cache_type not in ("auto", "bf16", "f32"):
            return "kv_cache_type must be auto (the run's dtype); quantized caches are not built"
        if self.kv_page_size <= 0:
            return "kv_page_size must be positive"
        if self.kv_num_pages is not None and self.kv_num_pages <= 0:
            return "kv_num_pages must be positive"
        if not 0 < self.kv_budget_ratio <= 1:
            return "kv_budget_ratio must be in (0, 1]"
        if min(self.max_batch_size, self.max_batch_tokens, self.chunked_prefill_tokens) <= 0:
            return "max_batch_size, max_batch_tokens and chunked_prefill_tokens must be positive"
        return ""

    def checked(self) -> "ModelLoadSpec":
        why = self.validate()
        if why:
            raise ValueError(f"model load spec: {why}")
        return self

    @property
    def name(self) -> str:
        return self.id or Path(self.path).name

    def engine_kwargs(self) -> dict:
        """The keyword arguments `Engine` takes for this spec."""
        return dict(dtype=self.dtype, device=self.device, kv_page_size=self.kv_page_size,
                    kv_num_pages=self.kv_num_pages, kv_max_batch=self.max_parallel_sequences,
                    kv_max_seq=self.context_size, kv_budget_mb=self.kv_budget_mb, kv_budget_ratio=self.kv_budget_ratio,
                    max_batch_size=self.max_batch_size, max_batch_tokens=self.max_batch_tokens,
                    chunked_prefill_tokens=self.chunked_prefill_tokens, cuda_graphs=self.cuda_graphs,
                    overlap_steps=self.overlap_steps)

    def make_runner(self):
        """(config, kernels, ModelRunner) for callers that drive the step function themselves (replay)."""
        import torch
        from ..csrc import CudaKernels
        from ..models import load_model
        from .runner import ModelRunner
        self.checked()
        device = torch.device(self.device)
        kernels = CudaKernels(device)                      # builds the library if need be; there is no fallback
        torch.cuda.set_device(device)
        config, model = load_model(self.path, dtype=self.dtype, device=device)
        runner = ModelRunner(model, kernels, page_size=self.kv_page_size, num_pages=self.kv_num_pages or 256,
                             max_seqs=self.max_parallel_sequences, max_seq_len=self.context_size,
                             cuda_graphs=self.cuda_graphs)
        return config, kernels, runner
