"""Weights by tensor name, checked against what the model's parts expect.

The reference resolves exact HF names and reports only the first missing layer,
without checking shapes (runtime/backends/cuda/native/weight_map.cpp:21-75).  Here
every expected tensor is declared by the part that owns it (name, shape, whether it
may be absent), and one `WeightError` lists everything that is missing, unexpected
or wrongly shaped.

Stored dtypes: 16-bit floats are kept as bfloat16, a tensor stored in 32-bit floats
stays 32-bit, integer tables become int32.  A float32 run takes float16 tensors
straight to float32, so that it does not compute with weights that lost three bits on
the way through bfloat16.  Converting to the dtype a run computes in is otherwise the
part's business when it takes its tensors.

Buffers that older exports carry and no part uses (`IGNORED_SUFFIXES`) are skipped with
a warning; so is the `lm_head.weight` of a model whose configuration ties the head to
the embedding (the reference would use the tensor, runtime/backends/cuda/native/
weight_map.cpp:33-37; here the configuration wins, and says so).
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .safetensors_io import open_model_shards


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one tensor."""
    shape: Tuple[int, ...]
    init: str = "normal"        # how random-weights mode fills it: normal | ones | zeros
    optional: bool = False      # may be absent from the file (the part then does without it)
    ignored: bool = False       # may be present but is not used (e.g. lm_head.weight of a tied model)
    invent: bool = True         # an optional tensor: whether random-weights mode makes it up


class WeightError(ValueError):
    """Missing, unexpected or wrongly shaped tensors, all in one message."""

    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"weights of {where} do not match the configuration:" if where
                 else "weights do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


IGNORED_SUFFIXES = ("rotary_emb.inv_freq", "masked_bias", "attn.bias")     # buffers, not parameters


def stored_dtype(dt: torch.dtype, run_dtype: Optional[torch.dtype] = None) -> torch.dtype:
    """The dtype a tensor of file dtype `dt` is kept in (for a run that computes in `run_dtype`)."""
    if dt in (torch.float32, torch.float64):
        return torch.float32
    if dt.is_floating_point:
        return torch.float32 if (dt == torch.float16 and run_dtype == torch.float32) else torch.bfloat16
    return torch.int32


def check_tensors(found: Dict[str, Tuple[int, ...]], expected: Dict[str, TensorSpec], where: str = "") -> None:
    """Raise one WeightError if the shapes in `found` do not fit `expected`."""
    missing = [n for n, s in expected.items() if n not in found and not s.optional and not s.ignored]
    skipped = [n for n in found if n not in expected and n.endswith(IGNORED_SUFFIXES)]
    if skipped:
        warnings.warn(f"{where or 'weights'}: {len(skipped)} tensors that no part uses are skipped "
                      f"({', '.join(sorted(skipped)[:3])}{', ...' if len(skipped) > 3 else ''})", stacklevel=3)
    unused = [n for n, s in expected.items() if s.ignored and n in found]
    if unused:
        warnings.warn(f"{where or 'weights'}: {', '.join(sorted(unused))} is present but not used "
                      f"(the configuration ties it to another tensor)", stacklevel=3)
    unexpected = [n for n in found if n not in expected and not n.endswith(IGNORED_SUFFIXES)]
    wrong = [(n, tuple(found[n]), tuple(s.shape)) for n, s in expected.items()
             if n in found and not s.ignored and tuple(found[n]) != tuple(s.shape)]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where)


class _Staging:
    """Two pinned buffers through which mapped file bytes go to the device: the host copy of one
    chunk runs while the other chunk's transfer is in flight."""

    CHUNK = 64 << 20

    def __init__(self, device):
        self.device = torch.device(device)
        self.bufs = [torch.empty(self.CHUNK, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.events = [torch.cuda.Event() for _ in range(2)]
        self.turn = 0

    def to_device(self, t: torch.Tensor) -> torch.Tensor:
        src = t.reshape(-1).view(torch.uint8)
        out = torch.empty(t.shape, dtype=t.dtype, device=self.device)
        dst = out.reshape(-1).view(torch.uint8)
        for off in range(0, src.numel(), self.CHUNK):
            n = min(self.CHUNK, src.numel() - off)
            i = self.turn
            self.turn ^= 1
            self.events[i].synchronize()                  # the buffer's last transfer is done
            self.bufs[i][:n].copy_(src[off:off + n])
            dst[off:off + n].copy_(self.bufs[i][:n], non_blocking=True)
            self.events[i].record()
        return out

    def finish(self):
        for e in self.events:
            e.synchronize()


class WeightSource:
    """The checked tensors of a model folder, handed out a few at a time: `take(names)` brings
    those tensors to the device (mapped file -> pinned buffers -> device), so that a model can be
    loaded part by part and only one part's unpacked tensors ever exist beside the model."""

    def __init__(self, model_dir, expected: Dict[str, TensorSpec], device="cpu",
                 run_dtype: Optional[torch.dtype] = None):
        self.shards = open_model_shards(model_dir)
        self.expected = expected
        self.device = torch.device(device)
        self.run_dtype = run_dtype
        self.staging = _Staging(self.device) if self.device.type == "cuda" else None
        try:
            self.owner = {}
            for sh in self.shards:
                for n in sh.names():
                    self.owner.setdefault(n, sh)      # first occurrence of a name wins, as in the reference
            check_tensors({n: sh.shape(n) for n, sh in self.owner.items()}, expected, where=str(model_dir))
        except BaseException:
            self.close()
            raise

    def names(self):
        return [n for n, spec in self.expected.items() if n in self.owner and not spec.ignored]

    def take(self, names) -> Dict[str, torch.Tensor]:
        out = {}
        for n in names:
            if n not in self.owner or self.expected[n].ignored:
                continue
            if self.staging is None:
                t = self.owner[n].tensor(n)
                out[n] = t.to(stored_dtype(t.dtype, self.run_dtype))
            else:
                t = self.owner[n].view(n)
                out[n] = self.staging.to_device(t).to(stored_dtype(t.dtype, self.run_dtype))
                del t
        if self.staging is not None:
            self.staging.finish()
        return out

    def close(self):
        for sh in self.shards:
            sh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def load_weights(model_dir, expected: Dict[str, TensorSpec], device="cpu",
                 run_dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """All tensors of a model folder that `expected` names, on `device`."""
    with WeightSource(model_dir, expected, device, run_dtype) as src:
        return src.take(src.names())
