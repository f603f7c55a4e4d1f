"""Builds the sm_100a kernel library with nvcc and loads it.

Every .cu file of this folder is compiled to an object (`-gencode
arch=compute_100a,code=sm_100a`) and the objects are linked into one shared
library.  The library lives in `_build/` beside the sources when that folder can be
written, else in a per-user folder under the system's temporary directory.  A
stamp of the sources' contents and the flags decides whether a build is current, so
a fresh checkout compiles once, at its first call, and prints a line per file
while it does.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_NAME = "libinferflux_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
LINK_LIBS = ["-lcublas"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[inferflux_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels "
                     "cannot be built, and there is no other path")


def sources():
    return sorted(HERE.glob("*.cu"))


def _stamp() -> str:
    h = hashlib.sha256()
    for p in sorted(list(HERE.glob("*.cu")) + list(HERE.glob("*.cuh")) + list(HERE.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + LINK_LIBS).encode())
    return h.hexdigest()


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    in_tree = HERE / "_build"
    if _writable(in_tree):
        return in_tree
    d = Path(tempfile.gettempdir()) / f"inferflux_b200_build_{os.getuid()}"
    if _writable(d):
        return d
    raise BuildError(f"neither {in_tree} nor {d} can be written: nowhere to build the kernels")


def _cuda_lib_dirs():
    dirs = []
    for cand in ("/usr/local/cuda/lib64", "/usr/local/cuda/targets/x86_64-linux/lib",
                 "/usr/local/cuda/lib64/stubs"):
        if Path(cand).is_dir():
            dirs.append(cand)
    return dirs


def _compile_one(nvcc: str, src: Path, obj: Path, verbose_ptxas: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj), "-I", str(HERE)]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    t0 = time.time()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    _say(f"compiled {src.name} in {time.time() - t0:.1f}s")
    return proc.stderr


def build(force: bool = False, verbose_ptxas: bool = False) -> Path:
    """Compile what is stale and return the path of the shared library."""
    out = build_dir()
    lib, stamp_file = out / LIB_NAME, out / "stamp.txt"
    stamp = _stamp()
    if not force and lib.is_file() and stamp_file.is_file() and stamp_file.read_text().strip() == stamp:
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    _say(f"building {len(srcs)} CUDA sources for sm_100a into {out} (first call or sources changed)")
    objs = [out / (s.stem + ".o") for s in srcs]
    logs = []
    with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as pool:
        for log in pool.map(lambda so: _compile_one(nvcc, so[0], so[1], verbose_ptxas), zip(srcs, objs)):
            logs.append(log)
    tmp = out / (LIB_NAME + f".tmp{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs]]
    for d in _cuda_lib_dirs():
        cmd += ["-L", d]
    cmd += LINK_LIBS
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, lib)
    stamp_file.write_text(stamp + "\n")
    if verbose_ptxas:
        (out / "ptxas.log").write_text("\n".join(logs))
    _say(f"linked {lib}")
    return lib


_LIB = None


def load_library() -> ctypes.CDLL:
    """The kernel library, built if need be.  Raises if it cannot be had: there is
    no fallback."""
    global _LIB
    if _LIB is None:
        import torch  # noqa: F401  (loads the CUDA runtime and cuBLAS the library links against)
        path = build()
        try:
            _LIB = ctypes.CDLL(str(path))
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from e
    return _LIB
