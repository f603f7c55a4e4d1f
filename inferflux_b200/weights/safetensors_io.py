"""Reader and writer of the safetensors file layout.

Layout (as the reference parses it, runtime/backends/cuda/native/
safetensors_parser.cpp:144-303): 8 bytes little-endian header length N; N bytes of
JSON {name: {"dtype", "shape", "data_offsets": [begin, end)}} (keys starting with
"__" are metadata); the data section starts at byte 8 + N.  Unlike the reference,
a tensor whose byte count does not match shape x dtype is an error here, not a
warning, and the data start is exactly 8 + N.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Optional, Tuple

import torch

_MAX_HEADER = 100 * 1024 * 1024      # same sanity bound as the reference (safetensors_parser.cpp:156)

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def _itemsize(dt: torch.dtype) -> int:
    return torch.empty(0, dtype=dt).element_size()


class SafetensorsFile:
    """One memory-mapped .safetensors file; `tensor` copies a tensor out, `view` maps it."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise SafetensorsError(f"{self.path}: no such file")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: {size} bytes is too short for a safetensors header")
        self._fh = open(self.path, "rb")
        # a private (copy-on-write) mapping: nothing is written, but a writable buffer is what torch maps
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        (n,) = struct.unpack("<Q", self._mm[:8])
        if n > _MAX_HEADER or 8 + n > size:
            raise SafetensorsError(f"{self.path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._mm[8:8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header is not a JSON object")
        self._data_start = 8 + n
        self.metadata = header.get("__metadata__", {})
        self._info: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        data_size = size - self._data_start
        for name, info in header.items():
            if name.startswith("__"):
                continue
            try:
                dt = _DTYPES[info["dtype"]]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{self.path}: bad header entry for {name!r}: {info!r}") from e
            numel = 1
            for s in shape:
                numel *= s
            if begin < 0 or end < begin or end > data_size:
                raise SafetensorsError(f"{self.path}: tensor {name!r} spans bytes [{begin}, {end}) "
                                       f"but the data section has {data_size} bytes (truncated file?)")
            if end - begin != numel * _itemsize(dt):
                raise SafetensorsError(f"{self.path}: tensor {name!r} has {end - begin} bytes, "
                                       f"shape {list(shape)} of {info['dtype']} needs {numel * _itemsize(dt)}")
            self._info[name] = (dt, shape, begin, end)

    def names(self) -> Iterable[str]:
        return self._info.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._info

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._info[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self._info[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its memory (the mapping may be closed afterwards)."""
        dt, shape, begin, end = self._info[name]
        if end == begin:
            return torch.empty(shape, dtype=dt)
        buf = bytearray(self._mm[self._data_start + begin:self._data_start + end])
        return torch.frombuffer(buf, dtype=dt).reshape(shape)

    def view(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapping itself: no copy, valid until `close`.  Falls back to a copy
        where the tensor's bytes do not start on a multiple of its element size."""
        dt, shape, begin, end = self._info[name]
        start = self._data_start + begin
        if end == begin or start % _itemsize(dt):
            return self.tensor(name)
        numel = (end - begin) // _itemsize(dt)
        return torch.frombuffer(self._mm, dtype=dt, count=numel, offset=start).reshape(shape)

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass                       # a view still points into the mapping: it goes when the view does
        finally:
            self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    """Write `tensors` (any device) as one .safetensors file, tensor by tensor."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of {name!r}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())


def open_model_shards(model_dir):
    """The .safetensors files of a model folder: those named by
    model.safetensors.index.json's weight_map, else model.safetensors
    (runtime/backends/cuda/inferflux_cuda_executor.cpp:366-402)."""
    model_dir = Path(model_dir)
    index = model_dir / "model.safetensors.index.json"
    if index.is_file():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError) as e:
            raise SafetensorsError(f"{index}: no readable weight_map ({e})") from e
        names = sorted(set(weight_map.values()))
        return [SafetensorsFile(model_dir / n) for n in names]
    single = model_dir / "model.safetensors"
    if single.is_file():
        return [SafetensorsFile(single)]
    raise SafetensorsError(f"{model_dir}: no safetensors files found (model.safetensors or "
                           f"model.safetensors.index.json)")
