#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the Qwen2.5-7B shape, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with the
context ending at 4,096 tokens, timed on the device with CUDA events around K decode
steps of the step function; the K-step loop is repeated until about half a second has
been timed and the median repeat is reported (`repeats`, `repeat_ms`, the SM clock
beside each).  `e2e` is the same through the Python entry point (`Engine.step`: host
token ids in through pinned memory, sampled ids read back, every step).  `prefill` is
one 2,048-token prompt in one step; `points` holds decode at batch 1 and 64, at
context 2,048 and averaged over 2,048 to 4,096, the prefill as four portions of 512,
and decode and a served workload at the Qwen2.5-1.5B shape; `roofline` compares the
bytes a decode step has to read (every weight once and the cache of the live requests)
with the measured HBM peak; `baselines` times the same model in plain PyTorch (matmul +
scaled_dot_product_attention) on the same GPU; `checked` compares the engine's logits at
the benchmarked depth, batch and context with a float32 PyTorch forward.
Weights are random (N(0, 0.02), norms 1.0), prompts are uniform random token ids.
A decode step reads ~14 GB of weights, far more than the 126 MB L2, so no L2 flush
is needed between timed steps (`l2` in `config` says so).

`--impl reference` runs the unmodified reference (its LlamaForwardTyped<bf16> model
path, built by baseline/build_ref.py with a small driver, baseline/ref_harness.cu) on
the same shape, batch, context and step counts and prints the same line.
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
        self.times = []
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
                self.times.append(time.time())
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
                    self.times.append(time.time())
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

    def summary(self, begin=None, end=None):
        """Median SM clock and the reasons seen, over all samples or those taken in [begin, end]."""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in zip(self.times, self.rows):
            if begin is not None and not (begin <= t <= end):
                continue
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


def end_all(engine):
    """End every live request outside the scheduler's books (their lengths were moved by direct steps)."""
    engine.drain()
    for r in list(engine.scheduler.running):
        r.status = "finished"
        engine.scheduler.running.remove(r)
        if r.request_id in engine.runner.cache:
            engine.runner.end_request(r.request_id)
    engine.scheduler.waiting.clear()


def time_decode(engine, cfg, batch, steps, warmup, repeats=1, context=4096, clock=None, e2e=True):
    """Decode at `batch` with the last timed step ending at `context` tokens.  Returns a dict:
    dev_ms (median over `repeats` loops of exactly `steps` steps, CUDA events around each loop),
    repeat_ms, repeat_spans (wall-clock begin/end of each loop), e2e_ms (through Engine.step),
    launches per step, h2d/d2h bytes per step, ctx (tokens per request after the last step)."""
    import torch
    from inferflux_b200.engine import StepEntry
    timed = repeats * steps
    total = warmup + timed
    # The last timed step ends at `context`: the prompt leaves room for both timed loops and for the tokens
    # the first requests decode while the last prompts are still prefilled (8,192 prompt tokens a step).
    # So no step of the timed loops is the first of a longer context class (its CUDA graph would be
    # captured inside the timing).
    loops = 2 if e2e else 1
    prompt_len = context - loops * total - 2 - (-(-batch * context // 8192) + 2)
    prompts = random_prompts(cfg, batch, prompt_len, seed=batch)
    bring_to_decode(engine, prompts, max_tokens=4 * total + 8 + batch)   # the first ones decode while the last prefill
    runner, kernels = engine.runner, engine.kernels
    out = {}

    # ---- end to end through the entry point: scheduler, step, sampling, ids back to the host
    if e2e:
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        h2d0, d2h0 = engine.stats.h2d_bytes, engine.stats.d2h_bytes
        walls = []
        for _ in range(repeats):
            t0 = time.perf_counter()
            for _ in range(steps):
                engine.step()
            torch.cuda.synchronize()
            walls.append((time.perf_counter() - t0) * 1000.0 / steps)
        out["e2e_ms"] = statistics.median(walls)
        out["h2d"] = (engine.stats.h2d_bytes - h2d0) / timed
        out["d2h"] = (engine.stats.d2h_bytes - d2h0) / timed

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
    ms, spans = [], []
    with (clock if clock is not None else _Null()):
        for r in range(repeats):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.time()
            start.record()
            for i in range(warmup + r * steps, warmup + (r + 1) * steps):
                one(i)
            end.record()
            torch.cuda.synchronize()
            spans.append((t0, time.time()))
            ms.append(start.elapsed_time(end) / steps)
    out["dev_ms"] = statistics.median(ms)
    out["repeat_ms"] = ms
    out["repeat_spans"] = spans
    out["launches"] = (kernels.launches - l0) / timed
    out["ctx"] = runner.cache.length(rids[0])
    kernels.check_errors()
    end_all(engine)
    return out


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def time_prefill(engine, cfg, tokens, warmup, reps, portion=0):
    """Median ms of one prompt of `tokens` tokens: in one step, or in portions of `portion`."""
    import torch
    from inferflux_b200.engine import StepEntry
    runner = engine.runner
    prompts = random_prompts(cfg, warmup + reps, tokens, seed=99)
    portion = portion or tokens
    times = []
    for i, p in enumerate(prompts):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for at in range(0, tokens, portion):
            part = p[at:at + portion]
            runner.step([StepEntry(f"prefill-{i}", part, [len(part) - 1] if at + portion >= tokens else [])])
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


def check_logits(engine, cfg, batch, context, rows, steps=4):
    """The engine's logits at the benchmarked depth, batch and context against a float32 PyTorch
    forward of the whole sequence: `batch` requests are prefilled through the engine to just under
    `context` tokens, then decoded for `steps` steps with given tokens through the step function (the
    path the timing uses: CUDA-graph replay from the second step on), and the last step's logits of
    `rows` are compared.  The yardstick for the error is the same model in plain bfloat16 PyTorch."""
    import torch
    from inferflux_b200.engine import StepEntry
    from baseline.torch_plain import TorchPlain
    torch.backends.cuda.matmul.allow_tf32 = False
    prompt_len = context - steps - 2 - (-(-batch * context // 8192) + 2)
    prompts = random_prompts(cfg, batch, prompt_len, seed=1000 + batch)
    bring_to_decode(engine, prompts, max_tokens=steps + 64 + batch)
    engine.drain()
    reqs = list(engine.scheduler.running)
    assert len(reqs) == batch
    g = torch.Generator().manual_seed(2)
    feed = torch.randint(0, cfg.vocab_size, (steps, batch), generator=g).tolist()
    # what each request holds so far: its prompt and the tokens it decoded while the others were prefilled;
    # its last sampled token has not been run yet and is replaced by the fed ones
    history = {b: list(r.prompt) + list(r.output[:engine.runner.cache.length(r.request_id) - len(r.prompt)])
               for b, r in enumerate(reqs)}
    logits = None
    for i in range(steps):
        logits = engine.runner.step([StepEntry(r.request_id, [feed[i][b]], [0]) for b, r in enumerate(reqs)])
        for b in range(batch):
            history[b].append(feed[i][b])
    engine.kernels.check_errors()
    got = logits.float()
    exact, plain16 = TorchPlain(engine.model, torch.float32), TorchPlain(engine.model, torch.bfloat16)
    worst = yard = scale = 0.0
    agree = 0
    for b in rows:
        want = exact.logits_last(history[b])[0]
        mine, theirs = got[b], plain16.logits_last(history[b])[0]
        worst = max(worst, float((mine - want).abs().max()))
        yard = max(yard, float((theirs - want).abs().max()))
        scale = max(scale, float(want.abs().max()))
        agree += int(int(mine.argmax()) == int(want.argmax()))
    ctx = engine.runner.cache.length(reqs[0].request_id)
    graphs = engine.runner.graph_replays
    end_all(engine)
    return {"batch": batch, "ctx": ctx, "rows": len(rows), "steps": steps, "max_err": round(worst, 4),
            "torch_bf16_err": round(yard, 4), "logit_scale": round(scale, 2), "argmax_agree": agree,
            "graph_replays": graphs, "ok": bool(worst <= 2.0 * yard + 1e-3 * scale)}


def run_reference(args, pk):
    """The reference arm: the unmodified reference model path (LlamaForwardTyped<bf16>::Forward /
    BatchForward + GpuSampler) driven by baseline/ref_harness at the same shape, batch, context and
    step counts.  None of this repository's kernels is loaded: the harness is a program of its own."""
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        from build_ref import build as build_reference
        exe = build_reference()
    except Exception as e:                                   # no sources, no nvcc, compile error
        print(json.dumps({"impl": "reference", "unavailable": f"the reference arm cannot be built: {e}"[:300]}))
        return 0
    cfg = qwen7b_config(args.shape)
    if args.layers:
        cfg.num_hidden_layers = args.layers
    warmup, steps = max(3, args.warmup), max(1, args.steps)
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    cmd = [str(exe), "bench", "dtype=bf16", f"hidden={cfg.hidden_size}", f"layers={cfg.num_hidden_layers}",
           f"heads={cfg.num_attention_heads}", f"kv_heads={cfg.num_key_value_heads}", f"head_dim={cfg.head_dim}",
           f"inter={cfg.intermediate_size}", f"vocab={cfg.vocab_size}", f"theta={cfg.rope_theta}",
           f"eps={cfg.rms_norm_eps}", f"tied={int(cfg.tie_word_embeddings)}", "bias=1", f"max_pos={CONTEXT}",
           f"ctx_end={CONTEXT}", f"steps={steps}", f"warmup={warmup}", f"prefill_tokens={PREFILL_TOKENS}",
           "batches=" + ",".join(map(str, batches))]
    clock = ClockSampler()
    with clock:
        proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the reference harness exited with {proc.returncode}: {proc.stderr.strip()[-200:]}"}))
        return 0
    raw = json.loads(proc.stdout.strip().splitlines()[-1])
    main = raw[f"b{args.batch}"]
    value = args.batch * 1000.0 / main["dev_ms"]
    step_bytes = weight_bytes(cfg, args.batch) + args.batch * main["ctx_end"] * kv_bytes_per_token(cfg)
    achieved = step_bytes / (main["dev_ms"] * 1e-3) / 1e9
    pf = prefill_flops(cfg, PREFILL_TOKENS) / (raw["prefill_ms"] * 1e-3)
    line = {
        "metric": "decode tok/s at batch 8, Qwen2.5-7B bf16 (also batch 1/64 and prefill tok/s at 2,048 tokens)",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["dev_ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": cfg.num_hidden_layers,
                   "layers_full": SHAPES[args.shape]["num_hidden_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
                   "seq_len": CONTEXT, "context_at_timing": main["ctx_end"], "kv_cache": "contiguous (the reference's)",
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (GBs of weights per step), no flush",
                   "peaks": pk["source"], "cuda_graph": bool(main["graph"])},
        "form": "stock model path: the reference's LlamaForwardTyped<bf16> (Forward, BatchForward), KvCacheGpuTyped, "
                "CublasGemm and GpuSampler, unmodified, driven by baseline/ref_harness.cu; the executor, scheduler and "
                "HTTP server above them are not built (they need llama.cpp)",
        "clocks": clock.summary(main["timed_begin"], main["timed_end"]),
        "e2e": {"value": round(args.batch * 1000.0 / main["e2e_ms"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": main["h2d_bytes"], "d2h_bytes_per_step": main["d2h_bytes"],
                "ms_per_step": round(main["e2e_ms"], 4)},
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / raw["prefill_ms"], 1), "tokens": PREFILL_TOKENS,
                    "ms": round(raw["prefill_ms"], 3), "frac": round(pf / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {f"decode_b{b}": round(b * 1000.0 / raw[f"b{b}"]["dev_ms"], 2) for b in batches if b != args.batch},
        "impl": "reference",
    }
    print(json.dumps(line))
    return 0


def _engine(cfg, page, slots, longest, pages=None, chunk=2048):
    import torch
    from inferflux_b200 import Engine
    return Engine(config=cfg, seed=0, dtype="bfloat16", device=torch.device("cuda:0"), kv_page_size=page,
                  kv_num_pages=pages or slots * (longest // page + 2), kv_max_batch=slots, kv_max_seq=longest,
                  max_batch_size=slots, max_batch_tokens=8192, chunked_prefill_tokens=chunk)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="tokens per request at the last timed decode step (default: the headline's 4,096)")
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the shape has (named in config)")
    ap.add_argument("--shape", default="7b", choices=sorted(SHAPES), help="model shape (default: the 7B headline shape)")
    ap.add_argument("--timed-seconds", type=float, default=0.5,
                    help="repeat the K-step loop until about this much has been timed (the median repeat is reported)")
    ap.add_argument("--serve", type=int, default=0, metavar="REQUESTS",
                    help="instead of the decode/prefill numbers: REQUESTS prompts of 128..2048 tokens, 256 new tokens "
                         "each, chunked prefill of 512 mixed with decode, through the scheduler")
    ap.add_argument("--serve-prompt", type=int, default=0, metavar="TOKENS",
                    help="with --serve: every prompt has this length (default: uniform in [128, 2048])")
    ap.add_argument("--serve-new", type=int, default=256, metavar="TOKENS", help="with --serve: new tokens per request")
    ap.add_argument("--no-points", action="store_true", help="skip the other decode points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill (for profiling decode)")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of logits with the float32 PyTorch forward")
    ap.add_argument("--no-extras", action="store_true", help="skip the PyTorch baseline and the 1.5B-shape points")
    ap.add_argument("--prefill-only", action="store_true",
                    help="time only the 2,048-token prefill and print a short line (for profiling prefill)")
    args = ap.parse_args()

    pk = peaks()
    if args.impl == "reference":
        return run_reference(args, pk)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup, steps = max(3, args.warmup), max(1, args.steps)
    context = args.context
    if context != CONTEXT:          # another context length: the headline's other points and checks do not apply
        args.no_points = args.no_check = args.no_extras = True

    import torch

    cfg = qwen7b_config(args.shape)
    full_layers = cfg.num_hidden_layers
    if args.layers:
        cfg.num_hidden_layers = args.layers
    page = 16
    model_name = f"Qwen2.5-{args.shape.upper()} shape"
    if args.serve:
        n = args.serve
        longest = (args.serve_prompt or 2048) + args.serve_new
        engine = _engine(cfg, page, n, longest + 64, chunk=512)
        serve_workload(engine, cfg, min(n, 8), 16, prompt_len=min(args.serve_prompt, 1024))   # warm-up: kernels, graphs
        dt, pt, gt, steps_run, pre = serve_workload(engine, cfg, n, args.serve_new, prompt_len=args.serve_prompt)
        print(json.dumps({"metric": "served tokens/s (prompt + generated), chunked prefill mixed with decode",
                          "value": round((pt + gt) / dt, 1), "generated_tok_s": round(gt / dt, 1), "unit": "tokens/s",
                          "seconds": round(dt, 3), "steps": steps_run, "requests": n, "prompt_tokens": pt,
                          "generated_tokens": gt, "preemptions": pre, "dtype": "bf16", "n_gpus": 1,
                          "config": {"model": model_name, "layers": cfg.num_hidden_layers,
                                     "prompts": args.serve_prompt or "uniform in [128, 2048]", "prefill_chunk": 512,
                                     "new_tokens": args.serve_new, "kv_page": page}, "impl": "ours"}))
        return 0
    if args.prefill_only:
        engine = _engine(cfg, page, 2, PREFILL_TOKENS + 64, chunk=PREFILL_TOKENS)
        ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=warmup, reps=steps)
        fl = prefill_flops(cfg, PREFILL_TOKENS) / (ms * 1e-3)
        print(json.dumps({"metric": "prefill tok/s at 2,048 tokens", "value": round(PREFILL_TOKENS * 1000.0 / ms, 1),
                          "unit": "tokens/s", "ms": round(ms, 3), "frac": round(fl / (pk["bf16_tflops"] * 1e12), 4),
                          "dtype": "bf16", "n_gpus": 1,
                          "config": {"model": model_name, "layers": cfg.num_hidden_layers,
                                     "layers_full": full_layers, "kv_page": page, "peaks": pk["source"]},
                          "impl": "ours"}))
        return 0

    # how often the K-step loop is repeated: about --timed-seconds at the rate the bytes allow
    est_ms = (weight_bytes(cfg, args.batch) + args.batch * context * kv_bytes_per_token(cfg)) / (0.7 * pk["hbm_gbs"] * 1e6)
    repeats = max(1, min(12, int(-(-args.timed_seconds * 1000.0 // (steps * est_ms)))))
    biggest = max(args.batch, 1 if args.no_points else 64)
    longest = context + 4 * (warmup + repeats * steps) + 8 + biggest   # a prompt plus the most new tokens time_decode allows
    cfg.max_position_embeddings = max(cfg.max_position_embeddings, longest)
    engine = _engine(cfg, page, biggest, longest)

    clock = ClockSampler()
    main_run = time_decode(engine, cfg, args.batch, steps, warmup, repeats=repeats, context=context, clock=clock)
    dev_ms = main_run["dev_ms"]
    value = args.batch * 1000.0 / dev_ms
    step_bytes = weight_bytes(cfg, args.batch) + args.batch * main_run["ctx"] * kv_bytes_per_token(cfg)
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9
    repeat_clocks = [clock.summary(b, e)["sm_mhz"] for b, e in main_run["repeat_spans"]]

    prefill = None
    points = {}
    if not args.no_prefill:
        pclock = ClockSampler()
        with pclock:
            prefill_ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=3, reps=9)
        pf = prefill_flops(cfg, PREFILL_TOKENS) / (prefill_ms * 1e-3) / 1e12
        pc = pclock.summary()
        prefill = {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                   "ms": round(prefill_ms, 3), "frac": round(pf / pk["bf16_tflops"], 4), "frac_of": "burst peak",
                   "frac_sustained": round(pf / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]), 4),
                   "sm_mhz": pc["sm_mhz"], "reasons": pc["reasons"]}
        if not args.no_points:
            ms4 = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=2, reps=3, portion=512)
            points["prefill_4x512"] = round(PREFILL_TOKENS * 1000.0 / ms4, 1)
    if not args.no_points:
        k = min(steps, 20)
        for b in (1, 64):
            r = time_decode(engine, cfg, b, k, 5, repeats=5, e2e=False)
            points[f"decode_b{b}"] = round(b * 1000.0 / r["dev_ms"], 1)
        window = [value]
        for ctx in (2048, 3072):
            r = time_decode(engine, cfg, args.batch, k, 5, repeats=4, context=ctx, e2e=False)
            window.append(args.batch * 1000.0 / r["dev_ms"])
            if ctx == 2048:
                points[f"decode_b{args.batch}_ctx2048"] = round(window[-1], 1)
        points[f"decode_b{args.batch}_avg_ctx2048_4096"] = round((window[1] + 2 * window[2] + window[0]) / 4, 1)

    checked = None
    if not args.no_check:
        checked = {"b%d" % args.batch: check_logits(engine, cfg, args.batch, context, rows=[0, args.batch - 1])}
        if not args.no_points:
            checked["b64"] = check_logits(engine, cfg, 64, context, rows=[0, 37])

    baselines = None
    if not args.no_extras:
        from baseline.torch_plain import time_torch_plain
        dec_ms, pre_ms = time_torch_plain(engine.model, cfg.vocab_size, args.batch, context, PREFILL_TOKENS)
        baselines = {"torch_plain": {"what": "the same weights in plain PyTorch (matmul + scaled_dot_product_attention, "
                                             "contiguous cache, eager)", "decode_tok_s": round(args.batch * 1000.0 / dec_ms, 1),
                                     "decode_ms_per_step": round(dec_ms, 3), "prefill_tok_s": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1),
                                     "prefill_ms": round(pre_ms, 3)}}

    if not args.no_extras and args.shape == "7b" and not args.layers:
        # the 1.5B shape (64 requests, chunks of 512 mixed with decode) on the same GPU
        del engine
        torch.cuda.empty_cache()
        small = qwen7b_config("1.5b")
        eng = _engine(small, page, 64, context + 4 * (5 + 2 * 20) + 80, chunk=512)
        r = time_decode(eng, small, 8, 20, 5, repeats=4, e2e=False)
        b15 = weight_bytes(small, 8) + 8 * r["ctx"] * kv_bytes_per_token(small)
        points["decode_b8_1p5b"] = round(8 * 1000.0 / r["dev_ms"], 1)
        points["decode_b8_1p5b_hbm_frac"] = round(b15 / (r["dev_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        serve_workload(eng, small, 8, 16, prompt_len=1024)
        runs = sorted(serve_workload(eng, small, 64, 256) for _ in range(3))      # the median of three: a shared host
        dt, pt, gt, _s, _p = runs[1]                                                # now and then stalls a run
        points["serve_1p5b"] = round((pt + gt) / dt, 1)
        points["serve_1p5b_generated"] = round(gt / dt, 1)

    line = {
        "metric": "decode tok/s at batch 8, Qwen2.5-7B bf16 (also batch 1/64 and prefill tok/s at 2,048 tokens)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": model_name, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps, "global_batch": args.batch,
                   "seq_len": context, "context_at_timing": main_run["ctx"], "kv_page": page, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (GBs of weights per step), no flush",
                   "peaks": pk["source"]},
        "repeats": repeats, "repeat_ms": [round(m, 4) for m in main_run["repeat_ms"]], "repeat_sm_mhz": repeat_clocks,
        "clocks": clock.summary(),
        "e2e": {"value": round(args.batch * 1000.0 / main_run["e2e_ms"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(main_run["h2d"]), "d2h_bytes_per_step": int(main_run["d2h"]),
                "ms_per_step": round(main_run["e2e_ms"], 4)},
        "gpu_launches": int(round(main_run["launches"] * steps)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "checked": checked,
        "baselines": baselines,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
