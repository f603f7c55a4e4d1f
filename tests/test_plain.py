"""The plain implementation itself, and the engine's host logic run on the CPU with
the plain kernel table in place of the CUDA one (test-only: the engine has no CPU
path of its own)."""
import math

import numpy as np
import pytest
import torch

import helpers
from plain import plain_qwen2
from plain.plain_kernels import PlainKernels, philox_uniform


@pytest.fixture(scope="module")
def loaded(model_dirs):
    return {name: plain_qwen2.load_model_dir(d) for name, (d, _p) in model_dirs.items()}


def test_parts_against_hand_computed_values():
    x = torch.tensor([[3.0, 4.0]])
    y = plain_qwen2.rmsnorm(x, torch.tensor([2.0, 0.5]), 0.0)
    assert torch.allclose(y, torch.tensor([[6.0 / math.sqrt(12.5), 2.0 / math.sqrt(12.5)]]))
    assert torch.allclose(plain_qwen2.silu(torch.tensor([0.0, 1.0])), torch.tensor([0.0, 1.0 / (1.0 + math.exp(-1.0))]))
    # rotation by position p of the pair (x0, x2) with inv_freq 1 and of (x1, x3) with inv_freq theta^(-1/2)
    q = torch.tensor([[[1.0, 2.0, 0.0, 0.0]]])
    r = plain_qwen2.rope_neox(q, torch.tensor([3]), theta=100.0)
    want = [math.cos(3.0), 2 * math.cos(0.3), math.sin(3.0), 2 * math.sin(0.3)]
    assert torch.allclose(r[0, 0], torch.tensor(want), atol=1e-6)
    # rotation keeps q.k a function of the distance only
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(1, 1, 8, generator=g), torch.randn(1, 1, 8, generator=g)
    d1 = (plain_qwen2.rope_neox(a, torch.tensor([5]), 1e4) * plain_qwen2.rope_neox(b, torch.tensor([2]), 1e4)).sum()
    d2 = (plain_qwen2.rope_neox(a, torch.tensor([13]), 1e4) * plain_qwen2.rope_neox(b, torch.tensor([10]), 1e4)).sum()
    assert abs(float(d1 - d2)) < 1e-5


def test_attention_mask_window_and_groups():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(6, 4, 8, generator=g), torch.randn(6, 2, 8, generator=g), torch.randn(6, 2, 8, generator=g))
    out = plain_qwen2.attention_gqa_causal(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])     # one key; head 3 -> kv head 1
    w1 = plain_qwen2.attention_gqa_causal(q, k, v, window=1)
    assert torch.allclose(w1[:, 1], v[:, 0]) and torch.allclose(w1[:, 2], v[:, 1])       # a window of 1 sees itself
    w3 = plain_qwen2.attention_gqa_causal(q, k, v, window=3)
    s = (q[5, 0] @ k[3:6, 0].t()) / math.sqrt(8)
    assert torch.allclose(w3[5, 0], torch.softmax(s, 0) @ v[3:6, 0], atol=1e-6)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_causality_and_precision_of_the_whole_model(name, loaded, tiny_configs):
    cfg, W = loaded[name]
    toks = helpers.random_tokens(cfg["vocab_size"], 40, 5)
    full = plain_qwen2.forward(cfg, W, toks, dtype=torch.float64)
    part = plain_qwen2.forward(cfg, W, toks[:23], dtype=torch.float64)
    assert torch.allclose(full[:23], part, atol=1e-10), "a position depends on later tokens"
    f32 = plain_qwen2.forward(cfg, W, toks, dtype=torch.float32)
    assert float((f32.double() - full).abs().max()) < 2e-5
    assert float(full.abs().max()) > 0.3, "the test model's logits are too flat to show anything"
    if name == "C":       # the window changes the result once the sequence is longer than it
        nowin = dict(cfg, use_sliding_window=False)
        other = plain_qwen2.forward(nowin, W, toks, dtype=torch.float64)
        assert torch.allclose(other[:21], full[:21], atol=1e-10) and float((other[30:] - full[30:]).abs().max()) > 1e-3


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_engine_host_logic_on_plain_kernels(name, cutting, model_dirs, tiny_configs):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    lens = [40, 33, 50, 60, 97, 70, 25, 64]
    reqs = {f"r{i}": helpers.random_tokens(cfg.vocab_size, n, 100 + i) for i, n in enumerate(lens)}
    want = helpers.plain_logits(d, reqs)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](reqs)
    _c, model = load_model(d, dtype="float32", device="cpu")
    runner = ModelRunner(model, PlainKernels(), page_size=page, num_pages=256 // page, max_seqs=8)
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), cfg.vocab_size)
    bad = helpers.first_bad(got, want, 1e-4)
    assert bad is None, f"first wrong row (request, position, diff): {bad}"
    assert not runner.cache.live_requests()


def test_generation_on_plain_kernels_with_preemption(model_dirs, tiny_configs, loaded):
    from inferflux_b200 import Engine, SamplingParams
    name = "B"
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    raw, W = loaded[name]
    prompts = [helpers.random_tokens(cfg.vocab_size, n, 40 + i) for i, n in enumerate([7, 19, 33, 4])]
    want = [plain_qwen2.greedy_generate(raw, W, p, 16) for p in prompts]
    for pages in (64, 11):                                    # 11 pages of 8: the requests do not all fit
        eng = Engine(d, dtype="float32", device="cpu", kernels=PlainKernels(), kv_page_size=page, kv_num_pages=pages,
                     kv_max_batch=4, chunked_prefill_tokens=16, max_batch_tokens=48)
        res = eng.generate(prompts, SamplingParams(temperature=0.0), max_tokens=16)
        assert [r.token_ids for r in res] == want
        assert (eng.stats.preemptions > 0) == (pages == 11)
        assert eng.runner.cache.free_pages() == [pages]


def test_temperature_sampling_is_reproducible_and_independent_of_the_batch(model_dirs, tiny_configs):
    from inferflux_b200 import Engine, SamplingParams
    cfg, page = tiny_configs["A"]
    d, _ = model_dirs["A"]
    prompts = [helpers.random_tokens(cfg.vocab_size, n, 70 + i) for i, n in enumerate([1, 4, 50, 30, 13])]
    sp = [SamplingParams(temperature=0.8, seed=1000 + i) for i in range(len(prompts))]

    def run(subset, **kw):
        eng = Engine(d, dtype="float32", device="cpu", kernels=PlainKernels(), kv_page_size=page, kv_num_pages=128,
                     kv_max_batch=8, **kw)
        return [r.token_ids for r in eng.generate([prompts[i] for i in subset], [sp[i] for i in subset], max_tokens=12)]
    together = run(range(5), chunked_prefill_tokens=32, max_batch_tokens=64)
    assert together == run(range(5), chunked_prefill_tokens=32, max_batch_tokens=64)
    assert [together[2]] == run([2], chunked_prefill_tokens=512)
    assert [together[4], together[0]] == run([4, 0], chunked_prefill_tokens=5, max_batch_tokens=8)
    greedy = run(range(5))
    assert len({tuple(t) for t in together}) == 5
    # the sampler's own random numbers
    us = [philox_uniform(1234, 0, s) for s in range(2000)]
    assert 0.45 < float(np.mean(us)) < 0.55 and min(us) >= 0.0 and max(us) < 1.0 and len(set(us)) > 1990


@pytest.mark.parametrize("pages", [64, 12])
def test_overlapped_steps_give_the_same_tokens(pages, model_dirs, tiny_configs, loaded):
    """Launching a step before the last one's tokens are read (they travel on the device)
    changes nothing in what is generated: greedy and sampled, stopping on a token, on the
    token limit and on the context limit, with and without preemption."""
    from inferflux_b200 import Engine, SamplingParams
    name = "A"
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    raw, W = loaded[name]
    prompts = [helpers.random_tokens(cfg.vocab_size, n, 900 + i) for i, n in enumerate([5, 21, 33, 2, 40, 11])]
    free_run = plain_qwen2.greedy_generate(raw, W, prompts[1], 12)
    stop = free_run[5]
    until_stop = free_run[:free_run.index(stop) + 1]
    params = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.0), SamplingParams(temperature=0.9, seed=4),
              SamplingParams(temperature=0.0), SamplingParams(temperature=0.7, seed=9, top_k=20),
              SamplingParams(temperature=0.0)]

    def run(overlap):
        eng = Engine(d, dtype="float32", device="cpu", kernels=PlainKernels(), kv_page_size=page, kv_num_pages=pages,
                     kv_max_batch=4, kv_max_seq=48, chunked_prefill_tokens=16, max_batch_tokens=40, overlap_steps=overlap)
        ids = [eng.add_request(p, sp, max_tokens=m, eos_token_id=stop) for p, sp, m in
               zip(prompts, params, [9, 12, 14, 1, 30, 3])]
        done = {}
        while eng.has_unfinished():
            for r in eng.step():
                done[r.request_id] = r
        assert eng.runner.cache.free_pages() == [pages] and not eng.runner.cache.live_requests()
        return [(done[i].token_ids, done[i].finish_reason) for i in ids], eng.stats
    a, sa = run(False)
    b, sb = run(True)
    assert a == b
    assert a[1] == (until_stop, "stop") and a[3][1] == "length" and len(a[3][0]) == 1
    assert a[4][1] == "length" and len(prompts[4]) + len(a[4][0]) == 48        # the context limit
    assert all(PENDING not in toks for toks, _ in b)
    if pages == 12:
        assert sb.preemptions > 0


PENDING = -1
