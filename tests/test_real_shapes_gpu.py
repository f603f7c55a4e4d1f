"""The three real layer shapes (Qwen2.5-1.5B, -7B, -32B: every size of a layer, of the
embedding and of the head as the models have them) with one layer and random weights:
the 32-bit path against the plain implementation under two cuttings, and the bfloat16
path against the same oracle with the tolerance its roundings need.

The plain implementation runs on the GPU here (float64, the same functions as on the
CPU) because of the size of the vocabulary; weights are made on the device by the
framework's seeded generator, so both sides draw the same values without a file.
"""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

SHAPES = {
    "1.5b": dict(hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, head_dim=128, intermediate_size=8960,
                 vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
               vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False),
    "32b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128, intermediate_size=27648,
                vocab_size=152064, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
}
LENS = [70, 37]


def make(shape, dtype, cuda_kernels, max_pos=512, num_pages=16):
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import random_model
    cfg = Qwen2Config(num_hidden_layers=1, max_position_embeddings=max_pos, **SHAPES[shape])
    model = random_model(cfg, seed=5, dtype=dtype, device="cuda:0", norm_jitter=0.2)
    return cfg, model, ModelRunner(model, cuda_kernels, page_size=16, num_pages=num_pages, max_seqs=4)


def oracle(cfg, model, reqs, weights_as):
    from inferflux_b200.weights import random_tensors
    from plain import plain_qwen2
    store = torch.float32 if weights_as is None else weights_as
    W = random_tensors(model.expected_tensors(), 5, dtype=store, device="cuda:0", norm_jitter=0.2)
    if cfg.tie_word_embeddings:
        W.pop("lm_head.weight", None)
    raw = cfg.to_dict()
    out = {rid: plain_qwen2.forward(raw, W, toks, dtype=torch.float64).cpu().numpy() for rid, toks in reqs.items()}
    del W
    torch.cuda.empty_cache()
    return out


@pytest.mark.parametrize("shape", ["1.5b", "7b", "32b"])
def test_real_layer_shapes_in_32_bit(shape, cuda_kernels):
    cfg, model, runner = make(shape, "float32", cuda_kernels)
    reqs = {f"r{i}": helpers.random_tokens(cfg.vocab_size, n, 700 + i) for i, n in enumerate(LENS)}
    want = oracle(cfg, model, reqs, None)
    for make_trace in (helpers.trace_whole, helpers.trace_portions, lambda r: helpers.trace_mixed(r, 256)):
        steps = make_trace(reqs)
        got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), cfg.vocab_size)
        bad = helpers.first_bad(got, want, 1e-4)
        assert bad is None, f"{shape}: first wrong row (request, position, diff) = {bad}"
        assert not runner.cache.live_requests()


@pytest.mark.parametrize("shape", ["1.5b", "7b", "32b"])
def test_real_layer_shapes_in_bfloat16(shape, cuda_kernels):
    cfg, model, runner = make(shape, "bfloat16", cuda_kernels)
    reqs = {f"r{i}": helpers.random_tokens(cfg.vocab_size, n, 700 + i) for i, n in enumerate(LENS)}
    want = oracle(cfg, model, reqs, torch.bfloat16)
    scale = max(float(np.abs(w).max()) for w in want.values())
    for make_trace in (helpers.trace_whole, helpers.trace_tail, lambda r: helpers.trace_mixed(r, 256)):
        steps = make_trace(reqs)
        got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), cfg.vocab_size)
        bad = helpers.first_bad(got, want, 0.03 * scale)
        assert bad is None, f"{shape}: first wrong row (request, position, diff) = {bad}, scale {scale}"
        agree = np.mean([np.mean(got[r].argmax(-1) == want[r].argmax(-1)) for r in want])
        assert agree > 0.9, f"{shape}: the best token agrees at only {agree:.2f} of the positions"
    cuda_kernels.check_errors()


def test_long_context_at_a_real_shape(cuda_kernels):
    """2,500 tokens through one layer of the 1.5B shape in bfloat16: whole, in portions of 512 and
    300 behind the growing prefix, and with the last tokens decoded one by one (clusters of blocks
    over thousands of keys); logits at a few dozen positions against the plain implementation."""
    from inferflux_b200.engine import StepEntry
    cfg, model, runner = make("1.5b", "bfloat16", cuda_kernels, max_pos=4096, num_pages=2 * 160)
    T = 2500
    toks = helpers.random_tokens(cfg.vocab_size, T, 901)
    wanted = sorted(set(list(range(0, T, 97)) + [127, 128, 255, 256, 511, 512, 1023, 1024, 2047, 2048] + list(range(T - 12, T))))
    from inferflux_b200.weights import random_tensors
    from plain import plain_qwen2
    W = random_tensors(model.expected_tensors(), 5, dtype=torch.bfloat16, device="cuda:0", norm_jitter=0.2)
    W.pop("lm_head.weight", None)
    full = plain_qwen2.forward(cfg.to_dict(), W, toks, dtype=torch.float64)
    want = full[torch.tensor(wanted, device=full.device)].cpu().numpy()
    del full, W
    torch.cuda.empty_cache()
    scale = float(np.abs(want).max())

    def run(cuts, name):
        got, pos = {}, 0
        for n in cuts:
            here = [p - pos for p in wanted if pos <= p < pos + n]
            out = runner.step([StepEntry(name, toks[pos:pos + n], here)])
            for k, p in enumerate(here):
                got[pos + p] = out[k].float().cpu().numpy()
            pos += n
        runner.end_request(name)
        assert pos == T
        return np.stack([got[p] for p in wanted])

    cuttings = {"whole": [T], "portions": [512, 300] * 3 + [T - 3 * 812], "tail": [T - 12] + [1] * 12}
    for name, cuts in cuttings.items():
        got = run(cuts, name)
        d = np.abs(got - want).max(axis=1)
        assert float(d.max()) < 0.03 * scale, f"{name}: position {wanted[int(d.argmax())]} differs by {float(d.max())} (scale {scale})"
    cuda_kernels.check_errors()
    assert not runner.cache.live_requests()


def test_mixed_steps_at_the_7b_layer_sizes_with_pages_used_again(cuda_kernels):
    """Head size 128, pages of 16, seven query heads a group: six requests, up to four live, portions of
    some beside decoded tokens of others, through a pool of 28 pages, so that a finished request's pages
    serve the next one.  Queries and keys are scaled up so that attention is peaked and a wrong or stale
    page moves the logits; every row against the plain implementation, in bfloat16, bounded by what
    plain bfloat16 arithmetic does to the same rows."""
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import Model
    from inferflux_b200.weights import random_tensors
    from plain import plain_qwen2
    cfg = Qwen2Config(num_hidden_layers=1, max_position_embeddings=512, **SHAPES["7b"])
    model = Model(cfg.to_plan())
    W = random_tensors(model.expected_tensors(), 12, dtype=torch.bfloat16, device="cuda:0", norm_jitter=0.2)
    for n in W:
        if ".q_proj." in n or ".k_proj." in n:
            W[n] = (W[n].float() * 3.0).to(torch.bfloat16)
    model.load(dict(W), torch.bfloat16, "cuda:0")
    pages = 28
    runner = ModelRunner(model, cuda_kernels, page_size=16, num_pages=pages, max_seqs=4, cuda_graphs=True)
    reqs = {f"m{i}": helpers.random_tokens(cfg.vocab_size, n, 800 + i) for i, n in enumerate([100, 70, 130, 40, 90, 60])}
    raw = cfg.to_dict()
    want = {r: plain_qwen2.forward(raw, W, t, dtype=torch.float64).cpu().numpy() for r, t in reqs.items()}
    yard = {r: plain_qwen2.forward(raw, W, t, dtype=torch.bfloat16).float().cpu().numpy() for r, t in reqs.items()}
    del W
    torch.cuda.empty_cache()
    steps = helpers.trace_mixed(reqs, pages * 16)
    assert max(len(s["entries"]) for s in steps) >= 3
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), cfg.vocab_size)
    g0 = runner.cache.stats()["groups"][0]
    assert g0["allocations"] > pages and g0["free"] == pages, "no page was used a second time"
    for rid in reqs:
        helpers.bf16_check(f"mixed at 7B sizes, {rid}", got[rid], want[rid], yard[rid])
    cuda_kernels.check_errors()
