"""Logits at the depth, batch and context that the benchmark times: the Qwen2.5-7B layer sizes
with 4 layers in 32-bit and with all 28 layers in bfloat16, a request whole and with its last
tokens decoded one by one, and 64 requests decoding at a context of about 4,000 tokens through
`Engine.step` (CUDA-graph replay, overlapped steps, tokens relayed on the device).  The same
whole-and-tail check at the 1.5B (tied head, 6 query heads a group) and 32B (5 a group) sizes.

The oracle is the plain implementation, run on the GPU layer by layer.  For bfloat16 the bound is
not a chosen number: the plain implementation itself is run in bfloat16 arithmetic on the same
rounded weights, and the engine, which keeps its sums and its residual stream in float32, has to be
at least as close to the float64 result as that.
"""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

from test_real_shapes_gpu import SHAPES          # noqa: E402  (the three real layer shapes)


def build(shape, layers, dtype, cuda_kernels, max_pos, pages, max_seqs=4, seed=6):
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import random_model
    cfg = Qwen2Config(num_hidden_layers=layers, max_position_embeddings=max_pos, **SHAPES[shape])
    model = random_model(cfg, seed=seed, dtype=dtype, device="cuda:0")
    return cfg, model, ModelRunner(model, cuda_kernels, page_size=16, num_pages=pages, max_seqs=max_seqs, cuda_graphs=True)


def stored_weights(model, dtype, seed=6):
    from inferflux_b200.weights import random_tensors
    return random_tensors(model.expected_tensors(), seed, dtype=dtype, device="cuda:0")


def whole_and_tail(runner, toks, rows, tail=32):
    """The logits at `rows` from one step with the whole request, and from a step with all but the
    last `tail` tokens followed by `tail` single-token steps."""
    from inferflux_b200.engine import StepEntry
    T = len(toks)
    whole = runner.step([StepEntry("w", toks, rows)]).float().cpu().numpy()
    runner.end_request("w")
    head = T - tail
    got = {}
    out = runner.step([StepEntry("t", toks[:head], [r for r in rows if r < head])])
    for k, r in enumerate(r for r in rows if r < head):
        got[r] = out[k].float().cpu().numpy()
    for i in range(head, T):
        out = runner.step([StepEntry("t", [toks[i]], [0] if i in rows else [])])
        if i in rows:
            got[i] = out[0].float().cpu().numpy()
    runner.end_request("t")
    return whole, np.stack([got[r] for r in rows])


def test_7b_sizes_four_layers_in_32_bit(cuda_kernels):
    cfg, model, runner = build("7b", 4, "float32", cuda_kernels, 1024, 2 * 40)
    T = 600
    toks = helpers.random_tokens(cfg.vocab_size, T, 31)
    rows = sorted(set(range(0, T, 41)) | set(range(T - 34, T)))
    want = helpers.plain_rows_layer_by_layer(cfg.to_dict(), stored_weights(model, torch.float32), toks, rows).cpu().numpy()
    whole, tail = whole_and_tail(runner, toks, rows)
    for name, got in (("whole", whole), ("tail", tail)):
        d = np.abs(got - want).max(axis=1)
        assert float(d.max()) < 1e-4, f"{name}: position {rows[int(d.argmax())]} differs by {float(d.max()):.3e}"
    assert np.array_equal(whole, tail)                       # 32-bit sums depend on the position only
    assert not runner.cache.live_requests()


bf16_check = helpers.bf16_check


@pytest.mark.parametrize("shape,layers", [("7b", 28), ("7b", 4), ("1.5b", 28), ("32b", 4)])
def test_real_sizes_at_depth_in_bfloat16(shape, layers, cuda_kernels):
    cfg, model, runner = build(shape, layers, "bfloat16", cuda_kernels, 1024, 2 * 40)
    T = 600
    toks = helpers.random_tokens(cfg.vocab_size, T, 32)
    rows = sorted(set(range(5, T, 53)) | set(range(T - 34, T)))
    W = stored_weights(model, torch.bfloat16)
    raw = cfg.to_dict()
    want = helpers.plain_rows_layer_by_layer(raw, W, toks, rows, torch.float64).cpu().numpy()
    yard = helpers.plain_rows_layer_by_layer(raw, W, toks, rows, torch.bfloat16).float().cpu().numpy()
    del W
    torch.cuda.empty_cache()
    whole, tail = whole_and_tail(runner, toks, rows)
    e1, b = bf16_check(f"{shape} x{layers} whole", whole, want, yard, rows)
    e2, _ = bf16_check(f"{shape} x{layers} tail", tail, want, yard, rows)
    print(f"{shape} x{layers}: engine off by {e1:.4f} (whole) / {e2:.4f} (tail), plain bfloat16 by {b:.4f}, "
          f"logits up to {float(np.abs(want).max()):.2f}")
    cuda_kernels.check_errors()
    assert not runner.cache.live_requests()


def test_batch_64_decode_at_4k_context_through_the_entry_point(cuda_kernels):
    """What the benchmark's batch-64 point runs: 64 requests with prompts of about 4,000 tokens through
    `Engine` (chunked prefill, then decode steps as CUDA-graph replays with overlapped steps and the
    sampled token relayed on the device).  Four of the 64 are followed for 16 steps: the engine's own
    logits of each step (re-run through the step function on the same cache) against the plain
    implementation's for the sequence the request really has."""
    from inferflux_b200 import Engine, SamplingParams
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.engine import StepEntry
    layers, ctx, steps, B = 28, 3968, 16, 64
    cfg = Qwen2Config(num_hidden_layers=layers, max_position_embeddings=8192, **SHAPES["7b"])
    engine = Engine(config=cfg, seed=6, dtype="bfloat16", device="cuda:0", kv_page_size=16,
                    kv_num_pages=B * ((ctx + 160) // 16 + 2), kv_max_batch=B, kv_max_seq=ctx + 160, max_batch_size=B,
                    max_batch_tokens=8192, chunked_prefill_tokens=2048)
    g = torch.Generator().manual_seed(77)
    prompts = [torch.randint(0, cfg.vocab_size, (ctx - (i % 7),), generator=g).tolist() for i in range(B)]
    results = engine.generate(prompts, SamplingParams(temperature=0.0), max_tokens=steps + 40)
    assert engine.runner.graph_replays > steps and engine.stats.preemptions == 0
    engine.kernels.check_errors()
    W = stored_weights(engine.model, torch.bfloat16)
    raw = cfg.to_dict()
    followed = [0, 21, 42, 63]
    for b in followed:
        seq = prompts[b] + results[b].token_ids
        first = len(prompts[b]) - 1                          # the row that chose the first new token
        rows = list(range(first + 24, first + 24 + steps))   # steps well inside the decode-only graph replays
        want = helpers.plain_rows_layer_by_layer(raw, W, seq[:rows[-1] + 1], rows, torch.float32).cpu()
        yard = helpers.plain_rows_layer_by_layer(raw, W, seq[:rows[-1] + 1], rows, torch.bfloat16).float().cpu()
        chosen = torch.tensor([seq[r + 1] for r in rows])
        # the token the engine chose at every followed step is (within rounding) the best one of the plain logits
        best = want.max(-1).values
        picked = want.gather(1, chosen[:, None])[:, 0]
        slack = (yard - want).abs().max(-1).values
        assert bool(((best - picked) <= 2 * slack).all()), f"request {b}: a chosen token is not near the best plain logit"
        assert float((want.argmax(-1) == chosen).float().mean()) >= 0.75
    del W
