"""Trace replay: feed given token ids through a model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
    inferctl replay  (the same options)

Reads one JSON object per line from standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

runs all entries of a step as one batch through the engine's own step function
(the model, cache and kernels that generation uses), writes DIR/<step>.f32 with the
logits at the wanted places as little-endian float32 [wanted, vocab] when anything
is wanted, gives back what the requests named in `end` hold, and prints
`done <step>`.  It samples nothing.  The cache pool is made for --max-tokens tokens
(each request's count rounded up to 64), so pages are used again.  The kernels are
compiled at the first call.  The reference's nearest tools feed prompts and compare
tokens (tests/tools/batched_isolation_probe.cpp) or compare debug traces
(scripts/compare_decode_traces.py); neither feeds given ids or writes whole logits rows.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def add_arguments(ap):
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--max-seqs", type=int, default=8, help="request slots")


def run(args) -> int:
    from ..engine import ModelLoadSpec, StepEntry
    if args.page_size <= 0 or args.max_tokens <= 0:
        print("trace_run: --page-size and --max-tokens must be positive", file=sys.stderr)
        return 2
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    # A request of n x 64 tokens takes at most n x ceil(64 / page) pages, whatever the page size.
    units = -(-args.max_tokens // 64)
    num_pages = max(1, units * (-(-64 // args.page_size)))
    spec = ModelLoadSpec(path=str(args.model), dtype=args.dtype, kv_page_size=args.page_size, kv_num_pages=num_pages,
                         max_parallel_sequences=args.max_seqs)
    _config, kernels, runner = spec.make_runner()
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                   for e in rec.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                logits.detach().to("cpu").contiguous().numpy().astype("<f4").tofile(out_dir / f"{step}.f32")
            kernels.check_errors()
        for rid in rec.get("end", []):
            if rid in runner.cache:
                runner.end_request(rid)
        print(f"done {step}", flush=True)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    add_arguments(ap)
    return run(ap.parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
