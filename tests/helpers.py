"""Helpers of the tests: tiny configurations, sharpened random weights, traces in
the replay format and their comparison with the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def tiny_configs():
    """Five tiny configurations that differ in every size and option.
    A and B follow the two tiny workloads the benchmark description names; C adds a
    window on its later layers, no biases, and sizes that are no power of two."""
    from inferflux_b200.config import Qwen2Config
    a = Qwen2Config(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=16, intermediate_size=176, vocab_size=512, max_position_embeddings=256,
                    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
    b = Qwen2Config(hidden_size=192, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2,
                    head_dim=32, intermediate_size=320, vocab_size=1000, max_position_embeddings=512,
                    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    c = Qwen2Config(hidden_size=120, num_hidden_layers=4, num_attention_heads=5, num_key_value_heads=1,
                    head_dim=48, intermediate_size=200, vocab_size=777, max_position_embeddings=384,
                    rope_theta=50000.0, rms_norm_eps=3e-4, tie_word_embeddings=False,
                    use_sliding_window=True, sliding_window=21, max_window_layers=2, qkv_bias=False)
    # D: nothing is a multiple of 8 except the head size's 8 itself: width 100, intermediate 150,
    # vocabulary 333, head size 24 - the sizes the tiled kernels refuse and the generic ones take.
    d = Qwen2Config(hidden_size=100, num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=3,
                    head_dim=24, intermediate_size=150, vocab_size=333, max_position_embeddings=300,
                    rope_theta=20000.0, rms_norm_eps=1e-5, tie_word_embeddings=True)
    # E: head size 64 and pages of 16, the sizes the tensor-core prompt attention takes; a window on
    # its second layer that ends inside the 128-key tiles.
    e = Qwen2Config(hidden_size=136, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2,
                    head_dim=64, intermediate_size=264, vocab_size=640, max_position_embeddings=512,
                    rope_theta=300000.0, rms_norm_eps=2e-6, tie_word_embeddings=False,
                    use_sliding_window=True, sliding_window=150, max_window_layers=1)
    return {"A": (a, 4), "B": (b, 8), "C": (c, 16), "D": (d, 16), "E": (e, 16)}


def write_tiny_model(cfg, out_dir, seed, dtype=torch.float32):
    """Random weights, then made sharp: query and key projections are scaled up so
    that attention is peaked (a wrong or missing key changes the result), and norm
    weights are jittered so that a norm weight used wrongly shows."""
    from inferflux_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    write_random_model(cfg, out_dir, seed=seed, dtype=dtype, norm_jitter=0.2)
    path = Path(out_dir) / "model.safetensors"
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    for n, t in tensors.items():
        if ".q_proj." in n or ".k_proj." in n:
            tensors[n] = (t.float() * 12.0).to(t.dtype)
        if n == "model.embed_tokens.weight":
            tensors[n] = (t.float() * 20.0).to(t.dtype)
    write_safetensors(path, tensors, metadata={"format": "pt"})
    return Path(out_dir)


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ----------------------------------------------------------------------- traces

def round64(n):
    return -(-n // 64) * 64


def trace_whole(requests):
    """Each request alone, whole, one after the other."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def trace_tail(requests, tail=32):
    """Most of a request in one step, then its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head],
                                                       "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


PORTIONS = [7, 2, 13, 3, 2, 31, 5, 2, 64, 9, 2, 17]


def trace_portions(requests):
    """Each request alone in portions of changing size, down to two tokens."""
    steps = []
    for k, (rid, toks) in enumerate(requests.items()):
        pos, i = 0, k
        while pos < len(toks):
            n = min(PORTIONS[i % len(PORTIONS)], len(toks) - pos)
            i += 1
            last = pos + n == len(toks)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[pos:pos + n],
                                                           "want": list(range(n))}],
                          "end": [rid] if last else []})
            pos += n
    return steps


def trace_mixed(requests, max_tokens, max_live=4, decode_tail=12):
    """Up to `max_live` requests at a time: prompt portions of some beside single
    decoded tokens of others; a request is admitted when the rounded sizes of the
    live ones leave room, so pages are freed and used again."""
    waiting = list(requests.items())
    live = []                      # [rid, toks, pos, portion index]
    steps = []
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live and \
                sum(round64(len(t)) for _r, t, _p, _i in live) + round64(len(waiting[0][1])) <= max_tokens:
            rid, toks = waiting.pop(0)
            live.append([rid, toks, 0, k])
            k += 3
        assert live, "a request does not fit the pool at all"
        entries, ended = [], []
        for item in live:
            rid, toks, pos, i = item
            if (len(steps) + i) % 5 == 4 and len(live) > 1:
                continue                                   # left out of this step, goes on later
            remaining = len(toks) - pos
            n = 1 if remaining <= decode_tail else min(PORTIONS[i % len(PORTIONS)], remaining - decode_tail)
            entries.append({"id": rid, "tokens": toks[pos:pos + n], "want": list(range(n))})
            item[2] += n
            item[3] += 1
            if item[2] == len(toks):
                ended.append(rid)
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        live = [it for it in live if it[0] not in ended]
    return steps


def collect(steps, outputs, vocab):
    """(request id -> [len, vocab] array) from per-step logits in trace order."""
    rows = {}
    for st in steps:
        out = outputs.get(st["step"])
        r = 0
        for e in st["entries"]:
            for _w in e["want"]:
                rows.setdefault(e["id"], []).append(out[r])
                r += 1
        if out is not None:
            assert r == out.shape[0], f"step {st['step']}: {out.shape[0]} rows written, {r} wanted"
    return {rid: np.stack(v) for rid, v in rows.items()}


def run_steps_in_process(runner, steps):
    """Drive the step function directly with a trace; returns step -> numpy logits."""
    from inferflux_b200.engine import StepEntry
    outputs = {}
    for st in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                outputs[st["step"]] = logits.detach().float().cpu().numpy()
        for rid in st["end"]:
            runner.end_request(rid)
        runner.cache.check()
    return outputs


def run_trace_cli(model_dir, dtype, steps, out_dir, max_tokens, vocab, page_size=None, timeout=600):
    """Drive bin/trace_run as a subprocess; returns step -> numpy logits."""
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], "a `done <step>` line is missing"
    outputs = {}
    for s in steps:
        f = Path(out_dir) / f"{s['step']}.f32"
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            assert f.is_file(), f"{f} was not written"
            outputs[s["step"]] = np.fromfile(f, dtype="<f4").reshape(wanted, vocab)
        else:
            assert not f.exists()
    return outputs


def plain_logits(model_dir, requests, weights_as=None, dtype=torch.float64):
    """request id -> float64 logits [len, vocab] of the plain implementation.
    `weights_as` rounds the stored weights first (what a bfloat16 run computes with);
    `dtype` is the arithmetic (bfloat16: the yardstick of what rounding does)."""
    from plain import plain_qwen2
    cfg, W = plain_qwen2.load_model_dir(model_dir)
    if weights_as is not None:
        W = {k: v.to(weights_as) for k, v in W.items()}
    return {rid: plain_qwen2.forward(cfg, W, toks, dtype=dtype).double().numpy() for rid, toks in requests.items()}


def max_abs_diff(got, want):
    return {rid: float(np.abs(got[rid].astype(np.float64) - want[rid]).max()) for rid in want}


def first_bad(got, want, tol):
    """(request, position, diff) of the first logits row beyond `tol`, or None."""
    for rid in want:
        d = np.abs(got[rid].astype(np.float64) - want[rid]).max(axis=1)
        bad = np.nonzero(d > tol)[0]
        if bad.size:
            return rid, int(bad[0]), float(d[bad[0]])
    return None


def plain_rows_layer_by_layer(cfg_raw, W, tokens, rows, dtype=torch.float64):
    """Logits of the plain implementation at `rows` of one whole sequence, run layer by layer so
    that only one layer's weights exist in `dtype` at a time (for models of many GB on the GPU).
    `W` holds the weights as stored (bfloat16 or float32), on the device the work should run on."""
    from plain import plain_qwen2 as P
    dev = W["model.embed_tokens.weight"].device
    toks = torch.as_tensor(tokens, dtype=torch.long, device=dev)
    positions = torch.arange(toks.numel())
    x = P.embedding(W["model.embed_tokens.weight"], toks).to(dtype)
    for layer in range(cfg_raw["num_hidden_layers"]):
        prefix = f"model.layers.{layer}."
        Wl = {k: v.to(dtype) for k, v in W.items() if k.startswith(prefix)}
        x = P.decoder_layer(x, Wl, cfg_raw, layer, positions)
        del Wl
    tied = cfg_raw.get("tie_word_embeddings", False) or "lm_head.weight" not in W
    table = "model.embed_tokens.weight" if tied else "lm_head.weight"
    head = {"model.norm.weight": W["model.norm.weight"].to(dtype), table: W[table].to(dtype)}
    return P.lm_head(x[torch.as_tensor(rows, device=dev)], head, cfg_raw)


def bf16_check(name, got, want, yard, rows=None):
    """bfloat16 results `got` against the exact ones `want`, row by row [rows, vocab].  The bound is not a
    chosen number: `yard` is the plain implementation run in bfloat16 arithmetic on the same rounded
    weights, and the engine, which keeps its sums and its residual stream in float32, has to be at least
    as close to `want` as that, in the worst row and on average, and to agree on the best token as often."""
    err = np.abs(got - want).max(axis=1)
    bound = np.abs(yard - want).max(axis=1)
    where = int(err.argmax()) if rows is None else rows[int(err.argmax())]
    assert float(err.max()) <= float(bound.max()), \
        f"{name}: row {where} is off by {float(err.max()):.4f}; plain bfloat16 arithmetic is off by at most {float(bound.max()):.4f}"
    assert float(err.mean()) <= float(bound.mean()), f"{name}: mean error {float(err.mean()):.4f} against {float(bound.mean()):.4f}"
    agree = float(np.mean(got.argmax(-1) == want.argmax(-1)))
    assert agree >= float(np.mean(yard.argmax(-1) == want.argmax(-1))) - 0.05, f"{name}: best token agrees at {agree:.2f}"
    return float(err.max()), float(bound.max())


def chosen_tokens_follow(raw, W16, prompt, out, name=""):
    """Every token of `out` (greedy) is the best, within rounding, under the plain logits of the sequence
    it continues: the gap to the best logit is at most twice what bfloat16 arithmetic moves that row."""
    from plain import plain_qwen2
    seq = list(prompt) + list(out)
    exact = plain_qwen2.forward(raw, W16, seq, dtype=torch.float64)
    rough = plain_qwen2.forward(raw, W16, seq, dtype=torch.bfloat16).double()
    for i, tok in enumerate(out):
        row = len(prompt) - 1 + i
        gap = float(exact[row].max() - exact[row, tok])
        slack = 2.0 * float((rough[row] - exact[row]).abs().max())
        assert gap <= slack, f"{name} token {i}: {gap:.4f} below the best logit, rounding allows {slack:.4f}"
