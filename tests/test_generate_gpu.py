"""Generation through the Python entry point on the GPU: greedy tokens against the
plain implementation, long decoding, the first tokens of a sequence, sampling, and
what the engine does without its extension."""
import numpy as np
import pytest
import torch

import helpers
from plain import plain_qwen2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_the_plain_implementation(name, model_dirs, tiny_configs):
    from inferflux_b200 import Engine, SamplingParams
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    raw, W = plain_qwen2.load_model_dir(d)
    prompts = [helpers.random_tokens(cfg.vocab_size, n, 300 + i) for i, n in enumerate([7, 19, 33, 1])]
    want = [plain_qwen2.greedy_generate(raw, W, p, 16) for p in prompts]
    eng = Engine(d, dtype="float32", kv_page_size=page, kv_num_pages=64, kv_max_batch=4, chunked_prefill_tokens=16,
                 max_batch_tokens=40)
    res = eng.generate(prompts, SamplingParams(temperature=0.0), max_tokens=16)
    assert [r.token_ids for r in res] == want
    assert all(r.finish_reason == "length" and r.prompt_tokens == len(p) for r, p in zip(res, prompts))
    assert eng.runner.graph_replays > 0 and eng.kernels.launches > 0
    # few pages: requests are preempted and recomputed, the tokens stay the same
    small = Engine(d, dtype="float32", kv_page_size=page, kv_num_pages=-(-70 // page), kv_max_batch=4,
                   chunked_prefill_tokens=16, max_batch_tokens=40)
    res = small.generate(prompts, SamplingParams(temperature=0.0), max_tokens=16)
    assert [r.token_ids for r in res] == want and small.stats.preemptions > 0


def test_bfloat16_generation_follows_the_logits(model_dirs, tiny_configs):
    """In bfloat16 a near-tie may go the other way, so compare step by step: every
    token the engine picks must be (nearly) the best under the plain logits of the
    engine's own sequence so far."""
    from inferflux_b200 import Engine, SamplingParams
    cfg, page = tiny_configs["B"]
    d, _ = model_dirs["B"]
    raw, W = plain_qwen2.load_model_dir(d)
    W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    prompt = helpers.random_tokens(cfg.vocab_size, 25, 77)
    eng = Engine(d, dtype="bfloat16", kv_page_size=page, kv_num_pages=32, kv_max_batch=2)
    out = eng.generate([prompt], SamplingParams(temperature=0.0), max_tokens=24)[0].token_ids
    logits = plain_qwen2.forward(raw, W, prompt + out, dtype=torch.float64)
    scale = float(logits.abs().max())
    for i, tok in enumerate(out):
        row = logits[len(prompt) - 1 + i]
        assert float(row.max() - row[tok]) < 0.04 * scale, f"token {i} is not among the best of its position"


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", None)])
def test_long_decoding_and_first_tokens(dtype, tol, model_dirs, tiny_configs, cuda_kernels):
    """One request decoded token by token for hundreds of steps, across many pages and
    past the window; the very first positions (one key, two keys) are checked too."""
    from inferflux_b200.engine import ModelRunner, StepEntry
    from inferflux_b200.models import load_model
    cfg, page = tiny_configs["C"]
    d, _ = model_dirs["C"]
    toks = helpers.random_tokens(cfg.vocab_size, 330, 55)
    want = helpers.plain_logits(d, {"r": toks}, weights_as=torch.bfloat16 if dtype == "bfloat16" else None)["r"]
    _c, model = load_model(d, dtype=dtype, device="cuda:0")
    runner = ModelRunner(model, cuda_kernels, page_size=page, num_pages=24, max_seqs=2, cuda_graphs=True)
    rows = [runner.step([StepEntry("r", [t], [0])])[0].cpu().numpy() for t in toks]
    got = np.stack(rows)
    bound = tol if tol else 0.03 * float(np.abs(want).max())
    d_ = np.abs(got - want).max(axis=1)
    assert float(d_.max()) < bound, f"first wrong position {int(np.argmax(d_ > bound))}, diff {float(d_.max())}"
    assert runner.graph_replays > 300


def test_sampling_through_the_entry_point(model_dirs, tiny_configs):
    from inferflux_b200 import Engine, SamplingParams
    cfg, page = tiny_configs["B"]
    d, _ = model_dirs["B"]
    prompts = [helpers.random_tokens(cfg.vocab_size, n, 400 + i) for i, n in enumerate([1, 4, 50, 97, 130])]
    sp = [SamplingParams(temperature=0.8, seed=7 + i) for i in range(5)]

    def run(subset, **kw):
        eng = Engine(d, dtype="float32", kv_page_size=page, kv_num_pages=64, kv_max_batch=8, **kw)
        return [r.token_ids for r in eng.generate([prompts[i] for i in subset], [sp[i] for i in subset], max_tokens=12)]
    a = run(range(5), chunked_prefill_tokens=32, max_batch_tokens=64)
    assert a == run(range(5), chunked_prefill_tokens=32, max_batch_tokens=64), "a fixed seed did not repeat"
    assert [a[3]] == run([3], chunked_prefill_tokens=512), "a request's draw depends on its batch"
    # penalties, top-k = 1 and logit bias go through the same path
    eng = Engine(d, dtype="float32", kv_page_size=page, kv_num_pages=64, kv_max_batch=8)
    greedy = eng.generate([prompts[2]], SamplingParams(temperature=0.0), max_tokens=8)[0].token_ids
    topk1 = eng.generate([prompts[2]], SamplingParams(temperature=0.9, top_k=1, seed=3), max_tokens=8)[0].token_ids
    assert topk1 == greedy
    forced = eng.generate([prompts[2]], SamplingParams(temperature=0.0, logit_bias={5: 1000.0}), max_tokens=4)[0]
    assert forced.token_ids == [5, 5, 5, 5]
    pen = eng.generate([prompts[2]], SamplingParams(temperature=0.0, logit_bias={5: 1000.0}, presence_penalty=2000.0),
                       max_tokens=3)[0].token_ids
    assert pen[0] == 5 and pen[1] != 5
    stop = eng.generate([prompts[2]], SamplingParams(temperature=0.0), max_tokens=8, eos_token_id=greedy[2])[0]
    assert stop.finish_reason == "stop" and stop.token_ids == greedy[:3]


def test_no_extension_no_engine(monkeypatch, model_dirs):
    """If the kernel library cannot be had the engine refuses to start."""
    from inferflux_b200.csrc import BuildError, build, ops
    import inferflux_b200.csrc.build as b
    monkeypatch.setattr(ops, "load_library", lambda: (_ for _ in ()).throw(BuildError("nvcc not found")))
    from inferflux_b200 import Engine
    with pytest.raises(BuildError):
        Engine(model_dirs["A"][0], dtype="float32")


def test_overlapped_steps_give_the_same_tokens_on_the_gpu(model_dirs, tiny_configs):
    """A step launched before the previous one's tokens are read takes them on the device;
    the tokens generated are those of reading every step's tokens first."""
    from inferflux_b200 import Engine, SamplingParams
    cfg, page = tiny_configs["B"]
    d, _ = model_dirs["B"]
    prompts = [helpers.random_tokens(cfg.vocab_size, n, 700 + i) for i, n in enumerate([5, 21, 33, 2, 40, 11, 64, 17])]
    params = [SamplingParams(temperature=0.0 if i % 2 == 0 else 0.8, seed=50 + i) for i in range(len(prompts))]
    limits = [9, 40, 14, 1, 30, 3, 25, 33]

    def run(overlap, pages):
        eng = Engine(d, dtype="float32", kv_page_size=page, kv_num_pages=pages, kv_max_batch=8, kv_max_seq=96,
                     chunked_prefill_tokens=16, max_batch_tokens=48, overlap_steps=overlap)
        ids = [eng.add_request(p, sp, max_tokens=m) for p, sp, m in zip(prompts, params, limits)]
        done = {}
        while eng.has_unfinished():
            for r in eng.step():
                done[r.request_id] = r
        assert not eng.runner.cache.live_requests()
        return [(done[i].token_ids, done[i].finish_reason) for i in ids], eng
    base, _ = run(False, 128)
    over, eng = run(True, 128)
    assert base == over and eng.runner.graph_replays > 0
    tight, eng = run(True, 30)
    assert base == tight and eng.stats.preemptions > 0
    stop = base[1][0][7]
    cut = base[1][0][:base[1][0].index(stop) + 1]
    eng = Engine(d, dtype="float32", kv_page_size=page, kv_num_pages=128, kv_max_batch=8)
    got = eng.generate([prompts[1]], params[1], max_tokens=40, eos_token_id=stop)[0]
    assert got.token_ids == cut and got.finish_reason == "stop"


def test_command_line_streams_the_tokens_it_reports(model_dirs):
    """`inferctl completion --stream`: one line per token as it becomes known, then the result;
    the streamed ids are the result's ids (no placeholder of a token not yet read)."""
    import json
    import subprocess
    import sys
    d, _ = model_dirs["B"]
    proc = subprocess.run([sys.executable, str(helpers.ROOT / "bin" / "inferctl"), "completion", "--model", str(d),
                           "--prompt", "5 17 3 250 9", "--max-tokens", "9", "--temperature", "0.8", "--top-p", "0.9",
                           "--seed", "11", "--stream", "--kv-page-size", "8"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(x) for x in proc.stdout.splitlines() if x.startswith("{")]
    streamed = [x["token"] for x in lines if "token" in x]
    final = [x for x in lines if "token_ids" in x]
    assert len(final) == 1 and final[0]["completion_tokens"] == 9
    assert streamed == final[0]["token_ids"] and all(t >= 0 for t in streamed)


def test_many_requests_with_every_kind_of_sampling_twice(model_dirs, tiny_configs):
    """Sixty requests of random lengths and sampling settings (greedy, temperature, top-k, top-p, min-p,
    penalties, stop tokens) through a pool so small that requests are preempted, with overlapped steps:
    every request finishes, every page comes back, a second run draws the same tokens, so does a run whose
    layers are launched part by part, and the greedy requests' tokens are the best ones under the plain
    implementation's logits."""
    import random
    from inferflux_b200 import Engine, SamplingParams
    cfg, page = tiny_configs["E"]
    d, _ = model_dirs["E"]
    rng = random.Random(7)
    jobs = []
    for i in range(60):
        prompt = [rng.randrange(cfg.vocab_size) for _ in range(rng.choice([1, 2, 5, 17, 40, 90, 150]))]
        kind = i % 6
        sp = [SamplingParams(temperature=0.0),
              SamplingParams(temperature=0.9, seed=100 + i),
              SamplingParams(temperature=0.7, top_k=20, seed=100 + i),
              SamplingParams(temperature=1.1, top_p=0.8, min_p=0.02, seed=100 + i),
              SamplingParams(temperature=0.8, repetition_penalty=1.3, frequency_penalty=0.2, seed=100 + i),
              SamplingParams(temperature=0.0, presence_penalty=0.5)][kind]
        jobs.append((prompt, sp, rng.choice([1, 3, 12, 30]), rng.randrange(cfg.vocab_size) if i % 4 == 0 else None))

    def run(native_layers=True):
        eng = Engine(d, dtype="bfloat16", kv_page_size=page, kv_num_pages=40, kv_max_batch=12, kv_max_seq=256,
                     max_batch_size=12, max_batch_tokens=96, chunked_prefill_tokens=48)
        eng.kernels.native_layers = native_layers
        ids = [eng.add_request(p, sp, max_tokens=m, eos_token_id=eos) for p, sp, m, eos in jobs]
        done, guard = {}, 0
        while eng.has_unfinished():
            for r in eng.step():
                done[r.request_id] = r
            guard += 1
            assert guard < 5000, "the engine does not finish"
        assert not eng.runner.cache.live_requests()
        g0 = eng.runner.cache.stats()["groups"][0]
        assert g0["free"] == g0["pages"]
        eng.kernels.check_errors()
        return [(done[i].token_ids, done[i].finish_reason) for i in ids], eng.stats.preemptions

    first, preemptions = run()
    second, _ = run()
    assert first == second
    # the same with every kernel launched by its part instead of a layer at a time from native code: the logits
    # are the same bits, so every request draws the same tokens
    third, _ = run(native_layers=False)
    assert first == third
    # against the oracle: what the greedy requests chose is the best token of the plain logits of their
    # own sequence, within bfloat16 rounding (a wrong page or a stale key after a preemption would show)
    raw, W = plain_qwen2.load_model_dir(d)
    W16 = {k: v.to(torch.bfloat16) for k, v in W.items()}
    checked = 0
    for i, ((toks, _reason), (prompt, _sp, _m, _eos)) in enumerate(zip(first, jobs)):
        if i % 6 == 0:
            helpers.chosen_tokens_follow(raw, W16, prompt, toks, f"request {i}")
            checked += 1
    assert checked == 10
    assert preemptions > 0, "the pool was large enough that nothing was preempted"
    for (toks, reason), (_p, _sp, m, eos) in zip(first, jobs):
        assert 1 <= len(toks) <= m and all(0 <= t < cfg.vocab_size for t in toks)
        assert reason in ("length", "stop")
        if reason == "stop":
            assert toks[-1] == eos


def test_abort_with_a_step_in_flight_frees_pages_that_the_waiting_request_then_uses(model_dirs, tiny_configs):
    """Three requests fill the pool and a fourth waits.  One of the three is aborted while a step that
    owes it a token is in flight (steps overlap): it is reported with `abort`, its pages come back, the
    waiting request runs on them, and everyone else's tokens are what they are without the episode."""
    from inferflux_b200 import Engine, SamplingParams
    cfg, page = tiny_configs["B"]
    d, _ = model_dirs["B"]
    prompts = [helpers.random_tokens(cfg.vocab_size, n, 900 + i) for i, n in enumerate([40, 44, 36, 30])]
    raw, W = plain_qwen2.load_model_dir(d)
    want = [plain_qwen2.greedy_generate(raw, W, p, 14) for p in prompts]
    pages = 3 * (-(-(44 + 16) // page))                      # room for three, not for four
    eng = Engine(d, dtype="float32", kv_page_size=page, kv_num_pages=pages, kv_max_batch=3, kv_max_seq=96,
                 chunked_prefill_tokens=64, max_batch_tokens=256, overlap_steps=True)
    ids = [eng.add_request(p, SamplingParams(temperature=0.0), max_tokens=14) for p in prompts]
    done = {}
    for _ in range(4):
        for r in eng.step():
            done[r.request_id] = r
    assert eng._inflight is not None and ids[3] not in eng.runner.cache
    victim = ids[1]
    assert eng.abort(victim) is None                         # the step in flight still owes it a token
    assert eng.abort("no-such-request") is None
    while eng.has_unfinished():
        for r in eng.step():
            done[r.request_id] = r
    assert done[victim].finish_reason == "abort" and -1 not in done[victim].token_ids
    assert done[victim].token_ids == want[1][:len(done[victim].token_ids)] and len(done[victim].token_ids) < 14
    for i in (0, 2, 3):
        assert done[ids[i]].token_ids == want[i] and done[ids[i]].finish_reason == "length"
    assert not eng.runner.cache.live_requests()
    g0 = eng.runner.cache.stats()["groups"][0]
    assert g0["free"] == g0["pages"]
    eng.runner.cache.check()
    # a request that only waits is gone at once, one that runs with nothing pending too
    eng2 = Engine(d, dtype="float32", kv_page_size=page, kv_num_pages=pages, kv_max_batch=3, kv_max_seq=96, overlap_steps=False)
    a, b = (eng2.add_request(p, SamplingParams(temperature=0.0), max_tokens=6) for p in prompts[:2])
    assert eng2.abort(b).finish_reason == "abort"
    eng2.step()
    res = eng2.abort(a)
    assert res.finish_reason == "abort" and len(res.token_ids) == 1 and not eng2.has_unfinished()
    assert not eng2.runner.cache.live_requests()
