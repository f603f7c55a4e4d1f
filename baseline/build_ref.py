#!/usr/bin/env python3
"""Builds the reference arm: the UNMODIFIED dense model path of anvai-labs/inferflux
plus `ref_harness.cu` (this repository's own driver around it) into
`baseline/_ref/ref_harness`.

The reference is a C++/CMake server; pip cannot install it, and its CMake build wants
the llama.cpp submodule, which the checkout does not hold.  Its native CUDA model
path does not need llama.cpp: `transformer_forward.cu` only reaches
`runtime/backends/llama/llama_cpp_backend.h`, which includes `<llama.h>` to name a few
opaque types in member declarations.  A header of forward declarations
(`_ref/stub/llama.h`, written below; no llama.cpp code) satisfies it, and the link
closure of the model path is the 21 files of `SOURCES`.

    python baseline/build_ref.py [--reference DIR] [--force]

Sources and the headers they include are copied byte for byte from the reference
checkout into `_ref/src/` (MANIFEST.json records their sha256), so that the folder
can be rebuilt where the checkout is absent.  The reference checkout is found through
--reference, $INFERFLUX_REFERENCE, or `reference_path` of BASELINE.json.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
HARNESS = HERE / "ref_harness.cu"
HOST_PROBE = HERE / "ref_host_probe.cpp"
HOST_SOURCES = ["runtime/backends/cuda/native/safetensors_parser.cpp", "server/logging/logger.cpp"]
HOST_HEADERS = ["runtime/backends/cuda/native/kv_cache_planner.h"]

N = "runtime/backends/cuda/native/"
SOURCES = [
    N + "transformer_forward.cu", N + "cuda_kernels.cu", "runtime/backends/cuda/kernels/flash_attention.cu",
    N + "kv_cache_gpu.cu", N + "gpu_sampler.cu", N + "fused_quant_gemm.cu", N + "cublas_gemm.cpp",
    N + "dispatch_operator_health.cpp", N + "native_dispatch_policy.cpp", N + "native_dispatch_registry.cpp",
    N + "model_forward_factory.cpp", N + "weight_map.cpp", N + "gguf_util.cpp",
    "server/metrics/metrics.cpp", "server/logging/logger.cpp", "server/diagnostics/crash_handler.cpp",
    "runtime/rocr_spin_tamer.cpp",
]

STUB_LLAMA_H = """\
// Forward declarations only: the reference's llama_cpp_backend.h names these types in
// member declarations; nothing of llama.cpp is compiled, linked or called.
#pragma once
#include <cstddef>
#include <cstdint>
struct llama_model;
struct llama_context;
struct llama_vocab;
struct llama_sampler;
typedef int32_t llama_token;
typedef int32_t llama_pos;
typedef int32_t llama_seq_id;
extern "C" uint32_t llama_n_ctx(const struct llama_context *);
"""

FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-w", "-Xcompiler", "-fPIC"]
LINK = ["-Xlinker", "--gc-sections", "-lcublas", "-lcublasLt", "-lcurand"]


def say(msg):
    print(f"[reference arm] {msg}", file=sys.stderr, flush=True)


def nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise RuntimeError("nvcc not found")


def reference_root(arg):
    cands = [arg, os.environ.get("INFERFLUX_REFERENCE")]
    try:
        cands.append(json.loads((HERE.parent / "BASELINE.json").read_text()).get("reference_path"))
    except (OSError, ValueError):
        pass
    for c in cands:
        if c and (Path(c) / SOURCES[0]).is_file():
            return Path(c)
    return None


def sha(path):
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


def dependencies(root: Path, rel: str, stub: Path):
    """Headers under `root` that `rel` includes, from the compiler's own dependency list."""
    proc = subprocess.run([nvcc(), "-M", "-std=c++17", "-w", f"-I{root}", f"-I{root / 'external'}", f"-I{stub}",
                           str(root / rel)], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"dependency scan of {rel} failed:\n{proc.stderr[-2000:]}")
    deps = set()
    for tok in proc.stdout.replace("\\\n", " ").split():
        p = Path(tok)
        try:
            deps.add(str(p.resolve().relative_to(root.resolve())))
        except ValueError:
            continue
    deps.discard(rel)
    return deps


def copy_sources(root: Path):
    src = OUT / "src"
    stub = OUT / "stub"
    stub.mkdir(parents=True, exist_ok=True)
    (stub / "llama.h").write_text(STUB_LLAMA_H)
    say(f"copying the model path's sources from {root}")
    files = set(SOURCES) | set(HOST_SOURCES) | set(HOST_HEADERS)
    with ThreadPoolExecutor(max_workers=8) as pool:
        for deps in pool.map(lambda r: dependencies(root, r, stub), SOURCES + HOST_SOURCES):
            files |= deps
    manifest = {}
    for rel in sorted(files):
        dst = src / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(root / rel, dst)
        manifest[rel] = sha(dst)
    (OUT / "MANIFEST.json").write_text(json.dumps({"copied_unmodified_from": "anvai-labs/inferflux",
                                                   "sources": SOURCES, "sha256": manifest}, indent=1) + "\n")
    say(f"copied {len(manifest)} files")


def compile_all():
    src, obj = OUT / "src", OUT / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{src}", f"-I{src / 'external'}", f"-I{OUT / 'stub'}"]
    jobs = [(src / rel, obj / (Path(rel).name + ".o")) for rel in SOURCES] + [(HARNESS, obj / "ref_harness.o")]

    def one(job):
        s, o = job
        t0 = time.time()
        p = subprocess.run([nvcc(), *FLAGS, *inc, "-c", str(s), "-o", str(o)], capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s.name}:\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}")
        say(f"compiled {s.name} in {time.time() - t0:.1f}s")

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(one, jobs))
    exe = OUT / "ref_harness"
    cmd = [nvcc(), "-o", str(exe), *[str(o) for _s, o in jobs]]
    for d in ("/usr/local/cuda/lib64", "/usr/local/cuda/targets/x86_64-linux/lib"):
        if Path(d).is_dir():
            cmd += ["-L", d]
    p = subprocess.run(cmd + LINK, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"linking ref_harness failed:\n{p.stderr[-4000:]}")
    (OUT / "stamp.txt").write_text(stamp() + "\n")
    say(f"linked {exe}")
    return exe


def build_host_probe() -> Path:
    """The host-only probe (the reference's safetensors parser and its cache-size arithmetic): g++, no GPU."""
    exe = OUT / "ref_host_probe"
    src = OUT / "src"
    if exe.is_file() and exe.stat().st_mtime >= HOST_PROBE.stat().st_mtime:
        return exe
    if not (src / HOST_SOURCES[0]).is_file():
        root = reference_root(None)
        if root is None:
            raise RuntimeError("no reference checkout and no copied sources under baseline/_ref/src")
        copy_sources(root)
    cxx = shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise RuntimeError("no C++ compiler")
    cmd = [cxx, "-std=c++17", "-O1", "-w", f"-I{src}", f"-I{src / 'external'}", str(HOST_PROBE),
           *[str(src / r) for r in HOST_SOURCES], "-o", str(exe), "-lpthread"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"building ref_host_probe failed:\n{p.stderr[-3000:]}")
    return exe


def stamp():
    h = hashlib.sha256(HARNESS.read_bytes())
    m = OUT / "MANIFEST.json"
    if m.is_file():
        h.update(m.read_bytes())
    h.update(" ".join(FLAGS + LINK).encode())
    return h.hexdigest()


def build(reference=None, force=False) -> Path:
    """Path of the built harness; raises RuntimeError with the reason if it cannot be had."""
    exe, st = OUT / "ref_harness", OUT / "stamp.txt"
    if not force and exe.is_file() and st.is_file() and st.read_text().strip() == stamp():
        return exe
    if force or not (OUT / "src" / SOURCES[0]).is_file():
        root = reference_root(reference)
        if root is None:
            raise RuntimeError("no reference checkout (give --reference or $INFERFLUX_REFERENCE) and no copied "
                               "sources under baseline/_ref/src")
        copy_sources(root)
    return compile_all()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    try:
        print(build(a.reference, a.force))
    except RuntimeError as e:
        print(f"build_ref: {e}", file=sys.stderr)
        sys.exit(1)
