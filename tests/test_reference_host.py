"""Two host-side anchors on the reference's own code (no GPU):

* a model file written by this repository's safetensors writer, parsed by the reference's
  SafetensorsParser (runtime/backends/cuda/native/safetensors_parser.cpp:144-303): same names,
  dtypes, shapes, offsets and bytes (through the parser's own data pointers) as this repository's reader sees;
* cache bytes per token against EstimateKvBytesPerTokenPerSequence
  (runtime/backends/cuda/native/kv_cache_planner.h:22-37) at the three real shapes.

The reference's outputs are kept in tests/golden/reference_host.json (the probe is
baseline/ref_host_probe.cpp, built by baseline/build_ref.py with g++); where the
reference's sources can be had, the probe is also run here and must still say the same.
"""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden" / "reference_host.json"
SHAPES = {"1.5b": (28, 2, 128), "7b": (28, 4, 128), "32b": (64, 8, 128)}


def _fnv1a(data: bytes) -> str:
    h = 1469598103934665603
    for b in data:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return format(h, "x")


def write_probe_file(folder: Path) -> Path:
    """A file with every dtype the writer knows, odd shapes, an empty-ish tensor and metadata of odd length."""
    from inferflux_b200.weights import write_safetensors
    from inferflux_b200.weights.random_init import counter_normal
    t = {
        "model.embed_tokens.weight": counter_normal((37, 24), 1, "e", 0.0, 0.02, torch.bfloat16),
        "model.layers.0.self_attn.q_proj.weight": counter_normal((24, 24), 1, "q", 0.0, 0.02, torch.float32),
        "model.layers.0.self_attn.q_proj.bias": counter_normal((24,), 1, "b", 0.0, 0.02).to(torch.float16),
        "model.norm.weight": torch.ones(24, dtype=torch.float32),
        "table": torch.arange(11, dtype=torch.int32),
        "one": counter_normal((1, 1, 3), 1, "o", 0.0, 1.0, torch.bfloat16),
    }
    path = folder / "model.safetensors"
    write_safetensors(path, t, metadata={"format": "pt", "note": "x" * 5})
    return path


def our_view(path: Path) -> dict:
    """What this repository's reader sees, in the shape of the probe's output."""
    from inferflux_b200.weights import SafetensorsFile
    raw = path.read_bytes()
    n = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + n])
    out = {}
    with SafetensorsFile(path) as f:
        for name in sorted(f.names()):
            b, e = header[name]["data_offsets"]
            t = f.tensor(name)
            data = t.contiguous().view(torch.uint8).numpy().tobytes() if t.numel() else b""
            assert data == raw[8 + n + b:8 + n + e], name
            out[name] = {"dtype": header[name]["dtype"], "shape": list(t.shape), "offset": b,
                         "byte_size": e - b, "fnv1a": _fnv1a(data)}
    return {"ok": True, "file_size": len(raw), "tensors": out}


def run_probe(*args):
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        from build_ref import build_host_probe
        exe = build_host_probe()
    except Exception as e:                               # no reference sources here: the stored outputs stand
        return None, str(e)
    proc = subprocess.run([str(exe), *map(str, args)], capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return json.loads(proc.stdout.strip().splitlines()[-1]), ""


def make_golden(folder: Path) -> dict:
    parsed, why = run_probe("parse", write_probe_file(folder))
    if parsed is None:
        raise RuntimeError(why)
    plan = {name: run_probe("kvplan", L, kv, d, 2)[0]["bytes_per_token"] for name, (L, kv, d) in SHAPES.items()}
    return {"parse": parsed, "kv_bytes_per_token_bf16": plan}


def test_the_reference_parser_reads_our_files_as_we_do(tmp_path):
    golden = json.loads(GOLDEN.read_text())
    path = write_probe_file(tmp_path)
    assert our_view(path) == golden["parse"]
    live, _why = run_probe("parse", path)
    if live is not None:
        assert live == golden["parse"]


def test_cache_bytes_per_token_match_the_reference_planner():
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.models import Model
    golden = json.loads(GOLDEN.read_text())["kv_bytes_per_token_bf16"]
    assert golden["7b"] == 57344
    for name, (L, kv, d) in SHAPES.items():
        cfg = Qwen2Config(hidden_size=kv * d, num_hidden_layers=L, num_attention_heads=kv * 2, num_key_value_heads=kv,
                          head_dim=d, intermediate_size=64, vocab_size=32)
        specs = Model(cfg.to_plan()).cache_specs()
        ours = sum(2 * s.num_kv_heads * s.head_dim * 2 for s, _st in specs)       # what Engine.bytes_per_token sums
        assert ours == golden[name], name
        live, _why = run_probe("kvplan", L, kv, d, 2)
        if live is not None:
            assert live["bytes_per_token"] == golden[name]


if __name__ == "__main__":                                # python tests/test_reference_host.py: rewrite the stored outputs
    import tempfile
    sys.path.insert(0, str(ROOT))
    with tempfile.TemporaryDirectory() as d:
        GOLDEN.write_text(json.dumps(make_golden(Path(d)), indent=1, sort_keys=True) + "\n")
    print(f"wrote {GOLDEN}")
