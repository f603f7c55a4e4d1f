"""`inferctl`: the command line, in the manner of the reference's client
(cli/main.cpp:1599-1641: `inferctl completion --prompt ... --model ... --max-tokens N
--stream`), but running the engine in this process instead of calling a server.
The engine works on token ids, so `--prompt` takes ids separated by commas or blanks.

    inferctl generate --model DIR --prompt "1 2 3" [--max-tokens 256] [--temperature 1.0]
                      [--top-p 1.0] [--top-k 0] [--seed N] [--stream] [--dtype bfloat16]
             (`completion` is the same command under the reference's name)
    inferctl replay --model DIR --dtype D --out DIR --max-tokens N      steps from standard input (trace replay)
    inferctl bench [options of bench.py]                                the benchmark of the checkout
    inferctl info [--model DIR]        configuration, tensors and cache bytes per token of a model; device,
                                       library and registered parts  (`models` and `status` give the halves)
    inferctl random-model --config FILE --seed N --out DIR [--dtype bfloat16]

It is Python by design: every command is a few calls into the package, the kernels are
reached through one C ABI either way, and a decode step's host work is hidden behind the
GPU by overlapped steps, so a second front end in C++ would restate the same calls.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def _add_engine_options(p):
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--kv-page-size", type=int, default=16)
    p.add_argument("--kv-max-batch", type=int, default=16, help="request slots")
    p.add_argument("--kv-max-seq", type=int, default=None, help="longest sequence (default: the model's)")
    p.add_argument("--kv-budget-mb", type=float, default=None)
    p.add_argument("--kv-budget-ratio", type=float, default=0.20, help="share of free memory for the cache")
    p.add_argument("--max-batch-size", type=int, default=32)
    p.add_argument("--max-batch-tokens", type=int, default=16384)
    p.add_argument("--chunked-prefill-tokens", type=int, default=512)


def _spec(args):
    from ..engine import ModelLoadSpec
    return ModelLoadSpec(path=str(args.model), dtype=args.dtype, kv_page_size=args.kv_page_size,
                         max_parallel_sequences=args.kv_max_batch, context_size=args.kv_max_seq,
                         kv_budget_mb=args.kv_budget_mb, kv_budget_ratio=args.kv_budget_ratio,
                         max_batch_size=args.max_batch_size, max_batch_tokens=args.max_batch_tokens,
                         chunked_prefill_tokens=args.chunked_prefill_tokens)


def cmd_completion(args) -> int:
    from .. import Engine, SamplingParams
    prompts = []
    if args.prompt:
        prompts.append(_ids(args.prompt))
    if args.prompt_file:
        for line in Path(args.prompt_file).read_text().splitlines():
            if line.strip():
                prompts.append(_ids(line))
    if not prompts:
        print("inferctl completion: give --prompt or --prompt-file", file=sys.stderr)
        return 2
    spec = _spec(args)
    why = spec.validate()
    if why:
        print(f"inferctl: {why}", file=sys.stderr)
        return 2
    engine = Engine.from_spec(spec)
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                            frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty,
                            repetition_penalty=args.repetition_penalty, seed=args.seed)
    ids = [engine.add_request(p, params, max_tokens=args.max_tokens, eos_token_id=args.eos_token_id) for p in prompts]
    shown = {i: 0 for i in ids}
    results = {}
    while engine.has_unfinished():
        for res in engine.step():
            results[res.request_id] = res
        if args.stream:
            for r in engine.scheduler.running + list(results.values()):
                rid = r.request_id
                toks = r.output if hasattr(r, "output") else r.token_ids
                for t in toks[shown[rid]:]:
                    if t < 0:               # sampled on the device, not read yet (steps overlap): next time
                        break
                    print(json.dumps({"id": rid, "token": t}), flush=True)
                    shown[rid] += 1
    for rid in ids:
        r = results[rid]
        print(json.dumps({"id": rid, "prompt_tokens": r.prompt_tokens, "completion_tokens": r.completion_tokens,
                          "finish_reason": r.finish_reason, "token_ids": r.token_ids}))
    return 0


def cmd_models(args) -> int:
    from ..config import load_config
    from ..models import expected_tensors
    cfg = load_config(args.model)
    specs = expected_tensors(cfg.to_plan())
    params = sum(int(__import__("math").prod(s.shape)) for s in specs.values() if not s.ignored)
    print(json.dumps({"id": str(args.model), "architecture": cfg.architecture, "config": cfg.to_dict(),
                      "tensors": len(specs), "parameters": params}, indent=2))
    return 0


def cmd_status(_args) -> int:
    import torch
    from ..config import registered_architectures
    from ..parts import registered_parts
    info = {"cuda": torch.cuda.is_available(), "architectures": registered_architectures(),
            "parts": {role: registered_parts(role) for role in ("mixer", "ffn", "norm", "position", "block")}}
    if torch.cuda.is_available():
        info["device"] = torch.cuda.get_device_name(0)
        from ..csrc import build
        info["library"] = str(build())
    print(json.dumps(info, indent=2))
    return 0


def cmd_info(args) -> int:
    """What `models` and `status` say, in one object; with --model also the cache bytes a token takes."""
    import io
    from contextlib import redirect_stdout
    out = {}
    buf = io.StringIO()
    with redirect_stdout(buf):
        cmd_status(args)
    out["engine"] = json.loads(buf.getvalue())
    if args.model:
        from ..config import load_config
        from ..models import Model
        buf = io.StringIO()
        with redirect_stdout(buf):
            cmd_models(args)
        out["model"] = json.loads(buf.getvalue())
        specs = Model(load_config(args.model).to_plan()).cache_specs()
        out["model"]["kv_bytes_per_token_bf16"] = sum(2 * kv.num_kv_heads * kv.head_dim * 2 for kv, _st in specs if kv)
    print(json.dumps(out, indent=2))
    return 0


def cmd_replay(args) -> int:
    from .replay import run
    return run(args)


def cmd_bench(args) -> int:
    """Runs bench.py of the checkout this package lies in, with the options given after `bench`."""
    import subprocess
    script = Path(__file__).resolve().parent.parent.parent / "bench.py"
    if not script.is_file():
        print(f"inferctl bench: {script} not found (the benchmark lives at the root of a source checkout)", file=sys.stderr)
        return 2
    return subprocess.call([sys.executable, str(script), *args.rest])


def cmd_random_model(args) -> int:
    import torch
    from ..config import config_from_dict
    from ..weights import write_random_model
    cfg = config_from_dict(json.loads(Path(args.config).read_text()))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    out = write_random_model(cfg, args.out, seed=args.seed, dtype=dtype)
    print(json.dumps({"written": str(out), "seed": args.seed, "dtype": args.dtype}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="inferctl", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    for name in ("generate", "completion"):
        c = sub.add_parser(name, help="generate from prompts of token ids")
        _add_engine_options(c)
        c.add_argument("--prompt", "--prompt-ids", help="token ids separated by commas or blanks")
        c.add_argument("--prompt-file", "--prompt-ids-file", help="one prompt of token ids per line")
        c.add_argument("--max-tokens", "--max_tokens", type=int, default=256)
        c.add_argument("--temperature", type=float, default=1.0, help="0 = greedy")
        c.add_argument("--top-p", type=float, default=1.0)
        c.add_argument("--top-k", type=int, default=0)
        c.add_argument("--min-p", type=float, default=0.0)
        c.add_argument("--frequency-penalty", type=float, default=0.0)
        c.add_argument("--presence-penalty", type=float, default=0.0)
        c.add_argument("--repetition-penalty", type=float, default=1.0)
        c.add_argument("--seed", "--sampling-seed", type=int, default=None)
        c.add_argument("--eos-token-id", type=int, default=None)
        c.add_argument("--stream", action="store_true", help="print each token as it is sampled")
        c.set_defaults(fn=cmd_completion)
    rp = sub.add_parser("replay", help="trace replay: steps as JSON lines on standard input, logits to files")
    from .replay import add_arguments as add_replay_arguments
    add_replay_arguments(rp)
    rp.set_defaults(fn=cmd_replay)
    b = sub.add_parser("bench", help="run the checkout's bench.py with the options that follow")
    b.add_argument("rest", nargs=argparse.REMAINDER)
    b.set_defaults(fn=cmd_bench)
    i = sub.add_parser("info", help="a model's configuration and sizes; device, library, registered parts")
    i.add_argument("--model", default=None)
    i.set_defaults(fn=cmd_info)
    m = sub.add_parser("models", help="describe a model folder")
    m.add_argument("--model", required=True)
    m.set_defaults(fn=cmd_models)
    s = sub.add_parser("status", help="device, library and registered parts")
    s.set_defaults(fn=cmd_status)
    r = sub.add_parser("random-model", help="write config.json and model.safetensors from a configuration and a seed")
    r.add_argument("--config", required=True, help="a config.json of a registered architecture")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(fn=cmd_random_model)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
