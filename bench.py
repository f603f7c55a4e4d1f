#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the Qwen2.5-7B shape, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with the
context at 4,096 tokens, timed on the device with CUDA events around K decode
steps of the step function; `e2e` is the same through the Python entry point
(`Engine.step`: host token ids in through pinned memory, sampled ids read back,
every step).  `prefill` is one 2,048-token prompt in one step; `points` holds
decode at batch 1 and 64; `roofline` compares the bytes a decode step has to read
(every weight once and the cache of the live requests) with the measured HBM peak.
Weights are random (N(0, 0.02), norms 1.0), prompts are uniform random token ids.
A decode step reads ~14 GB of weights, far more than the 126 MB L2, so no L2 flush
is needed between timed steps (`l2` in `config` says so).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
CONTEXT = 4096
PREFILL_TOKENS = 2048


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            raw = json.loads(p.read_text())
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in raw.items() if isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        try:                                    # NVML in this process: a sample every 20 ms (reading only)
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(0)
            try:
                get_reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons
            except AttributeError:
                get_reasons = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            while not self._stop.is_set():
                bits = int(get_reasons(h))
                self.rows.append([str(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)), str(mx), "",
                                  "Active" if bits & 0x8 else "Not Active", "Active" if bits & 0x40 else "Not Active",
                                  "Active" if bits & 0x20 else "Not Active", "Active" if bits & 0x4 else "Not Active"])
                self._stop.wait(0.02)
            return
        except Exception:
            pass
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.rows.append([c.strip() for c in out.stdout.strip().splitlines()[0].split(",")])
            except (OSError, subprocess.SubprocessError):
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


SHAPES = {   # the three real-sized shapes of the benchmark description
    "7b": dict(hidden_size=3584, num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, vocab_size=152064, tie_word_embeddings=False),
    "1.5b": dict(hidden_size=1536, num_hidden_layers=28, num_attention_heads=12, num_key_value_heads=2,
                 intermediate_size=8960, vocab_size=151936, tie_word_embeddings=True),
    "32b": dict(hidden_size=5120, num_hidden_layers=64, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=27648, vocab_size=152064, tie_word_embeddings=False),
}


def qwen7b_config(shape="7b"):
    from inferflux_b200.config import Qwen2Config
    return Qwen2Config(head_dim=128, max_position_embeddings=32768, rope_theta=1000000.0, rms_norm_eps=1e-6,
                       **SHAPES[shape])


def weight_bytes(cfg, batch):
    """Bytes of weights a decode step reads once: every layer matrix, bias and norm,
    the final norm and the head; of the embedding table only the batch's rows."""
    h, i, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads * cfg.head_dim, \
        cfg.num_key_value_heads * cfg.head_dim
    per_layer = 2 * (h * (q + 2 * kv) + q * h + 3 * h * i) + 4 * (q + 2 * kv) + 4 * 2 * h
    head = 2 * cfg.vocab_size * h                       # tied or not, the head's table is read once
    return cfg.num_hidden_layers * per_layer + head + 4 * h + batch * h * 2


def kv_bytes_per_token(cfg):
    return 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * 2


def prefill_flops(cfg, tokens):
    h, i, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads * cfg.head_dim, \
        cfg.num_key_value_heads * cfg.head_dim
    linear = 2 * tokens * cfg.num_hidden_layers * (h * (q + 2 * kv) + q * h + 3 * h * i)
    attn = cfg.num_hidden_layers * 4 * cfg.num_attention_heads * cfg.head_dim * (tokens * (tokens + 1) // 2)
    head = 2 * cfg.vocab_size * h                       # logits of the last position only
    return linear + attn + head


def random_prompts(cfg, n, length, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (length,), generator=g).tolist() for _ in range(n)]


def bring_to_decode(engine, prompts, max_tokens):
    """Prefill every prompt through the engine until all requests are decoding."""
    from inferflux_b200.sampling import SamplingParams
    for p in prompts:
        engine.add_request(p, SamplingParams(temperature=0.0), max_tokens=max_tokens)
    guard = 0
    while engine.scheduler.waiting or any(r.remaining > 1 or not r.output for r in engine.scheduler.running):
        engine.step()
        guard += 1
        if guard > 100000:
            raise RuntimeError("prefill did not finish")


def drain(engine):
    for r in list(engine.scheduler.running):
        engine.scheduler._finish(r, "stop")
    engine.scheduler.waiting.clear()


def time_decode(engine, cfg, batch, steps, warmup, sampler_clock=None):
    """(device ms per step through the step function, wall ms per step through Engine.step,
    launches per step, h2d bytes per step, d2h bytes per step)."""
    import torch
    from inferflux_b200.engine import StepEntry
    total = warmup + steps
    # The last timed step ends at CONTEXT: the prompt leaves room for both timed loops and for the tokens
    # the first requests decode while the last prompts are still prefilled (8,192 prompt tokens a step).
    # So no step of the timed loops is the first of a longer context class (its CUDA graph would be
    # captured inside the timing).
    prompt_len = CONTEXT - 2 * total - 2 - (-(-batch * CONTEXT // 8192) + 2)
    prompts = random_prompts(cfg, batch, prompt_len, seed=batch)
    bring_to_decode(engine, prompts, max_tokens=4 * total + 8 + batch)   # the first ones decode while the last prefill
    runner, kernels = engine.runner, engine.kernels

    # ---- end to end through the entry point: scheduler, step, sampling, ids back to the host
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d0, d2h0 = engine.stats.h2d_bytes, engine.stats.d2h_bytes
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1000.0 / steps
    h2d = (engine.stats.h2d_bytes - h2d0) / steps
    d2h = (engine.stats.d2h_bytes - d2h0) / steps

    # ---- the step function alone, timed on the device
    engine.drain()
    rids = [r.request_id for r in engine.scheduler.running]
    assert len(rids) == batch, f"{len(rids)} of {batch} requests are still decoding"
    g = torch.Generator().manual_seed(1)
    feed = torch.randint(0, cfg.vocab_size, (total, batch), generator=g).tolist()

    def one(i):
        logits = runner.step([StepEntry(rid, [feed[i][b]], [0]) for b, rid in enumerate(rids)])
        return kernels.argmax(logits)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    l0 = kernels.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx_clock = sampler_clock if sampler_clock is not None else _Null()
    with ctx_clock:
        start.record()
        for i in range(warmup, total):
            one(i)
        end.record()
        torch.cuda.synchronize()
    dev_ms = start.elapsed_time(end) / steps
    launches = (kernels.launches - l0) / steps
    ctx_len = runner.cache.length(rids[0])
    # the requests' lengths moved outside the scheduler's books: end them here
    for r in list(engine.scheduler.running):
        r.status = "finished"
        engine.scheduler.running.remove(r)
        runner.end_request(r.request_id)
    return dev_ms, e2e_ms, launches, h2d, d2h, ctx_len


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def time_prefill(engine, cfg, tokens, warmup, reps):
    import torch
    from inferflux_b200.engine import StepEntry
    runner = engine.runner
    prompts = random_prompts(cfg, warmup + reps, tokens, seed=99)
    times = []
    for i, p in enumerate(prompts):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry(f"prefill-{i}", p, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.end_request(f"prefill-{i}")
        if i >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def serve_workload(engine, cfg, requests, new_tokens, seed=3, prompt_len=0):
    """Many requests with prompts of uniform random length through the scheduler: chunked
    prefill mixed with decode, as a server would run them.  Returns (seconds, prompt tokens,
    generated tokens, steps, preemptions)."""
    import torch
    from inferflux_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(seed)
    lens = [prompt_len] * requests if prompt_len else torch.randint(128, 2049, (requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    for p in prompts:
        engine.add_request(p, SamplingParams(temperature=0.0), max_tokens=new_tokens)
    torch.cuda.synchronize()
    steps0 = engine.stats.steps
    t0 = time.perf_counter()
    done = 0
    while engine.has_unfinished():
        done += len(engine.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert done == requests, f"{done} of {requests} requests finished"
    return dt, sum(lens), requests * new_tokens, engine.stats.steps - steps0, engine.stats.preemptions


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the 7B shape has (named in config)")
    ap.add_argument("--shape", default="7b", choices=sorted(SHAPES), help="model shape (default: the 7B headline shape)")
    ap.add_argument("--serve", type=int, default=0, metavar="REQUESTS",
                    help="instead of the decode/prefill numbers: REQUESTS prompts of 128..2048 tokens, 256 new tokens "
                         "each, chunked prefill of 512 mixed with decode, through the scheduler")
    ap.add_argument("--serve-prompt", type=int, default=0, metavar="TOKENS",
                    help="with --serve: every prompt has this length (default: uniform in [128, 2048])")
    ap.add_argument("--serve-new", type=int, default=256, metavar="TOKENS", help="with --serve: new tokens per request")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill (for profiling decode)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="time only the 2,048-token prefill and print a short line (for profiling prefill)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip cannot install the reference offline: it is a C++/CMake server with neither "
                          "setup.py nor pyproject.toml, and its native backend needs the absent llama.cpp submodule"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup, steps = max(3, args.warmup), max(1, args.steps)

    import torch
    from inferflux_b200 import Engine

    pk = peaks()
    cfg = qwen7b_config(args.shape)
    full_layers = cfg.num_hidden_layers
    if args.layers:
        cfg.num_hidden_layers = args.layers
    dev = torch.device("cuda:0")
    page = 16
    if args.serve:
        n = args.serve
        longest = (args.serve_prompt or 2048) + args.serve_new
        engine = Engine(config=cfg, seed=0, dtype="bfloat16", device=dev, kv_page_size=page,
                        kv_num_pages=n * (longest // page + 2), kv_max_batch=n, kv_max_seq=longest + 64, max_batch_size=n,
                        max_batch_tokens=8192, chunked_prefill_tokens=512)
        serve_workload(engine, cfg, min(n, 8), 16, prompt_len=min(args.serve_prompt, 1024))   # warm-up: kernels, graphs
        dt, pt, gt, steps_run, pre = serve_workload(engine, cfg, n, args.serve_new, prompt_len=args.serve_prompt)
        print(json.dumps({"metric": "served tokens/s (prompt + generated), chunked prefill mixed with decode",
                          "value": round((pt + gt) / dt, 1), "generated_tok_s": round(gt / dt, 1), "unit": "tokens/s",
                          "seconds": round(dt, 3), "steps": steps_run, "requests": n, "prompt_tokens": pt,
                          "generated_tokens": gt, "preemptions": pre, "dtype": "bf16", "n_gpus": 1,
                          "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": cfg.num_hidden_layers,
                                     "prompts": args.serve_prompt or "uniform in [128, 2048]", "prefill_chunk": 512,
                                     "new_tokens": args.serve_new, "kv_page": page}, "impl": "ours"}))
        return 0
    if args.prefill_only:
        engine = Engine(config=cfg, seed=0, dtype="bfloat16", device=dev, kv_page_size=page,
                        kv_num_pages=2 * (PREFILL_TOKENS // page + 2), kv_max_batch=2, kv_max_seq=PREFILL_TOKENS + 64,
                        max_batch_size=2, max_batch_tokens=8192, chunked_prefill_tokens=PREFILL_TOKENS)
        ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=warmup, reps=steps)
        frac = prefill_flops(cfg, PREFILL_TOKENS) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
        print(json.dumps({"metric": "prefill tok/s at 2,048 tokens", "value": round(PREFILL_TOKENS * 1000.0 / ms, 1),
                          "unit": "tokens/s", "ms": round(ms, 3), "frac": round(frac, 4), "dtype": "bf16", "n_gpus": 1,
                          "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": cfg.num_hidden_layers,
                                     "layers_full": full_layers, "kv_page": page, "peaks": pk["source"]},
                          "impl": "ours"}))
        return 0
    biggest = max(args.batch, 1 if args.no_points else 64)
    longest = CONTEXT + 4 * (warmup + steps) + 8 + biggest       # a prompt plus the most new tokens time_decode allows
    pages = biggest * (longest // page + 2)
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", device=dev, kv_page_size=page, kv_num_pages=pages,
                    kv_max_batch=biggest, kv_max_seq=longest, max_batch_size=biggest,
                    max_batch_tokens=8192, chunked_prefill_tokens=2048)

    clock = ClockSampler()
    dev_ms, e2e_ms, launches, h2d, d2h, ctx_len = time_decode(engine, cfg, args.batch, steps, warmup, clock)
    value = args.batch * 1000.0 / dev_ms
    step_bytes = weight_bytes(cfg, args.batch) + args.batch * ctx_len * kv_bytes_per_token(cfg)
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9

    prefill_ms = float("inf") if args.no_prefill else time_prefill(engine, cfg, PREFILL_TOKENS, warmup=3, reps=5)
    pf_flops = prefill_flops(cfg, PREFILL_TOKENS)
    pf_frac = pf_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)

    points = {}
    if not args.no_points:
        for b in (1, 64):
            k = min(steps, 32)
            ms, _e, _l, _h, _d, _c = time_decode(engine, cfg, b, k, 3)
            points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)

    line = {
        "metric": "decode tok/s at batch 8, Qwen2.5-7B bf16 (also batch 1/64 and prefill tok/s at 2,048 tokens)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": cfg.num_hidden_layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps, "global_batch": args.batch,
                   "seq_len": CONTEXT, "context_at_timing": ctx_len, "kv_page": page, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (GBs of weights per step), no flush",
                   "peaks": pk["source"]},
        "clocks": clock.summary(),
        "e2e": {"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_ms, 4)},
        "gpu_launches": int(round(launches * steps)),
        "prefill": None if args.no_prefill else
        {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
         "ms": round(prefill_ms, 3), "frac": round(pf_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
