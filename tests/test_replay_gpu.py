"""Replay of the same requests cut in every way, in 32-bit and in bfloat16, through
the step function and through bin/trace_run, against the plain implementation.

Cuttings: each request whole; most of it in one step and the last 32 tokens one by
one; portions of changing size down to two tokens; up to four live requests mixed,
portions of some beside decoded tokens of others, with a pool so small that pages
are used again.
"""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

LENS = [40, 33, 50, 60, 97, 130, 25, 64]
MAX_TOKENS = 256
TOL = {"float32": 1e-4, "bfloat16": None}       # bfloat16: relative to the size of the logits, see below


def requests_for(cfg):
    return {f"r{i}": helpers.random_tokens(cfg.vocab_size, n, 100 + i) for i, n in enumerate(LENS)}


def make_runner(model_dir, page, dtype, cuda_kernels, max_tokens=MAX_TOKENS):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    _cfg, model = load_model(model_dir, dtype=dtype, device="cuda:0")
    return ModelRunner(model, cuda_kernels, page_size=page, num_pages=max_tokens // page, max_seqs=8)


def check(got, want, dtype, what, yard=None):
    if dtype == "float32":
        bad = helpers.first_bad(got, want, 1e-4)
        assert bad is None, f"{what}: first wrong row (request, position, diff) = {bad}"
    else:
        # bfloat16 keeps 8 bits: activations are rounded at every stage, so rows differ from the
        # float64 oracle by a few 2^-8 of the logits' scale.  The bound is fixed, not fitted per case.
        scale = max(float(np.abs(w).max()) for w in want.values())
        bad = helpers.first_bad(got, want, 0.03 * scale)
        assert bad is None, f"{what}: first wrong row (request, position, diff) = {bad}, scale {scale}"
        mean = np.mean([np.abs(got[r] - want[r]).mean() for r in want])
        assert mean < 0.006 * scale, f"{what}: mean error {mean} at scale {scale}"
        if yard is not None:         # and no further from the exact logits than plain bfloat16 arithmetic is
            for rid in want:
                helpers.bf16_check(f"{what} {rid}", got[rid], want[rid], yard[rid])


@pytest.fixture(scope="module")
def oracle(model_dirs, tiny_configs):
    out = {}
    for name, (d, _page) in model_dirs.items():
        reqs = requests_for(tiny_configs[name][0])
        out[name] = {"float32": helpers.plain_logits(d, reqs),
                     "bfloat16": helpers.plain_logits(d, reqs, weights_as=torch.bfloat16),
                     "yard": helpers.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16)}
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_step_function_cuttings(name, dtype, cutting, model_dirs, tiny_configs, oracle, cuda_kernels):
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    reqs = requests_for(cfg)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, MAX_TOKENS)}[cutting](reqs)
    runner = make_runner(d, page, dtype, cuda_kernels)
    outputs = helpers.run_steps_in_process(runner, steps)
    got = helpers.collect(steps, outputs, cfg.vocab_size)
    check(got, oracle[name][dtype], dtype, f"{name}/{dtype}/{cutting}", oracle[name]["yard"])
    assert not runner.cache.live_requests()
    if cutting == "mixed":
        g0 = runner.cache.stats()["groups"][0]
        assert g0["allocations"] > g0["pages"], "the pool was large enough that no page was used again"
        assert g0["free"] == g0["pages"]


LENS_E = [300, 150, 40, 260, 70, 385]
MAX_TOKENS_E = 832


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_long_requests_through_the_tensor_core_attention(dtype, cutting, model_dirs, tiny_configs, cuda_kernels):
    """Configuration E (head size 64, pages of 16) with requests of several hundred tokens: prompt
    portions of more than one 128-row query tile over several 128-key tiles, behind a cached prefix,
    with a window on the second layer, cut in every way."""
    cfg, page = tiny_configs["E"]
    d, _ = model_dirs["E"]
    assert cuda_kernels.tensor_core_prefill and cuda_kernels.lib.ifx_attention_prefill_tcgen05_supports(cfg.head_dim, page)
    reqs = {f"e{i}": helpers.random_tokens(cfg.vocab_size, n, 300 + i) for i, n in enumerate(LENS_E)}
    want = helpers.plain_logits(d, reqs, weights_as=torch.bfloat16 if dtype == "bfloat16" else None)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, MAX_TOKENS_E)}[cutting](reqs)
    runner = make_runner(d, page, dtype, cuda_kernels, max_tokens=MAX_TOKENS_E)
    before = cuda_kernels.launches
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), cfg.vocab_size)
    check(got, want, dtype, f"E/{dtype}/{cutting}")
    cuda_kernels.check_errors()
    assert cuda_kernels.launches > before and not runner.cache.live_requests()
    if cutting == "mixed":
        g0 = runner.cache.stats()["groups"][0]
        assert g0["allocations"] > g0["pages"], "the pool was large enough that no page was used again"


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_float32_is_the_same_under_every_cutting(name, model_dirs, tiny_configs, cuda_kernels):
    """The 32-bit kernels add in an order that depends on the position only, so
    every cutting gives the same bits."""
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    reqs = requests_for(cfg)
    results = []
    for make in (helpers.trace_whole, helpers.trace_portions, lambda r: helpers.trace_mixed(r, MAX_TOKENS)):
        steps = make(reqs)
        runner = make_runner(d, page, "float32", cuda_kernels)
        results.append(helpers.collect(steps, helpers.run_steps_in_process(runner, steps), cfg.vocab_size))
    for other in results[1:]:
        for rid in reqs:
            assert np.array_equal(results[0][rid], other[rid]), f"request {rid} differs between cuttings"


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("C", "bfloat16"), ("A", "bfloat16"), ("D", "bfloat16")])
def test_trace_run_program(name, dtype, model_dirs, tiny_configs, oracle, tmp_path):
    """bin/trace_run as a user calls it: one process, all four cuttings one after the other."""
    cfg, _page = tiny_configs[name]
    d, _ = model_dirs[name]
    reqs = requests_for(cfg)
    want = oracle[name][dtype]
    steps, owner = [], []
    for k, make in enumerate((helpers.trace_whole, helpers.trace_tail, helpers.trace_portions,
                              lambda r: helpers.trace_mixed(r, MAX_TOKENS))):
        renamed = {f"{rid}_{k}": toks for rid, toks in reqs.items()}
        for st in make(renamed):
            st["step"] = len(steps)
            steps.append(st)
    outputs = helpers.run_trace_cli(d, dtype, steps, tmp_path / "out", MAX_TOKENS, cfg.vocab_size)
    got = helpers.collect(steps, outputs, cfg.vocab_size)
    for k in range(4):
        part = {rid: got[f"{rid}_{k}"] for rid in reqs}
        check(part, want, dtype, f"trace_run {name}/{dtype}/cutting {k}")


def test_trace_run_refuses_a_bad_model(tmp_path):
    import json, subprocess, sys
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["NoSuchModel"], "model_type": "nosuch"}))
    proc = subprocess.run([sys.executable, str(helpers.ROOT / "bin" / "trace_run"), "--model", str(tmp_path),
                           "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                          input="", capture_output=True, text=True, timeout=300)
    assert proc.returncode != 0
    assert "unsupported architecture" in proc.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_replayed_from_a_cuda_graph(dtype, model_dirs, tiny_configs, oracle, cuda_kernels):
    """Decode-only steps run from a captured graph; the logits are those of the plain path."""
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    name = "B"
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    reqs = {k: v for k, v in list(requests_for(cfg).items())[:3]}
    steps = helpers.trace_tail(reqs, tail=20)
    _c, model = load_model(d, dtype=dtype, device="cuda:0")
    runner = ModelRunner(model, cuda_kernels, page_size=page, num_pages=MAX_TOKENS // page, max_seqs=8,
                         cuda_graphs=True)
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), cfg.vocab_size)
    assert runner.graph_replays >= 30
    check(got, {k: oracle[name][dtype][k] for k in reqs}, dtype, f"graph replay {dtype}", oracle[name]["yard"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_nine_live_requests_of_different_lengths_decode_from_a_cuda_graph(dtype, model_dirs, tiny_configs, cuda_kernels):
    """Nine requests of different lengths (some past the window, some inside their first page) decode
    together for twenty steps: from the second step on every step is a replay of one captured graph over
    metadata at fixed addresses.  Every logits row against the plain implementation."""
    from inferflux_b200.engine import ModelRunner, StepEntry
    from inferflux_b200.models import load_model
    name = "E"
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    lens = [3, 17, 64, 150, 151, 200, 33, 96, 129]
    tail = 20
    reqs = {f"g{i}": helpers.random_tokens(cfg.vocab_size, n + tail, 500 + i) for i, n in enumerate(lens)}
    want = helpers.plain_logits(d, reqs, weights_as=torch.bfloat16 if dtype == "bfloat16" else None)
    yard = helpers.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16) if dtype == "bfloat16" else None
    _c, model = load_model(d, dtype=dtype, device="cuda:0")
    runner = ModelRunner(model, cuda_kernels, page_size=page, num_pages=sum(-(-(n + tail) // page) for n in lens),
                         max_seqs=9, cuda_graphs=True)
    got = {rid: [] for rid in reqs}
    for (rid, toks), n in zip(reqs.items(), lens):          # prompts one by one, each whole
        out = runner.step([StepEntry(rid, toks[:n], list(range(n)))])
        got[rid] += list(out.float().cpu().numpy())
    before = runner.graph_replays
    for i in range(tail):
        out = runner.step([StepEntry(rid, [toks[n + i]], [0]) for (rid, toks), n in zip(reqs.items(), lens)])
        for k, rid in enumerate(reqs):
            got[rid].append(out[k].float().cpu().numpy())
    assert runner.graph_replays - before >= tail - 1
    check({rid: np.stack(v) for rid, v in got.items()}, want, dtype, f"nine live {dtype}", yard)
    cuda_kernels.check_errors()


@pytest.mark.parametrize("name,dtype", [("E", "bfloat16"), ("E", "float32"), ("C", "bfloat16")])
def test_prompt_portions_replayed_from_a_cuda_graph(name, dtype, model_dirs, tiny_configs, cuda_kernels):
    """Chunked prefill brings the same portion size again and again: from its second occurrence a
    one-request portion runs from a captured graph (behind a growing prefix, through the window,
    with and without wanted logits); the logits are those of the plain implementation."""
    from inferflux_b200.engine import ModelRunner, StepEntry
    from inferflux_b200.models import load_model
    cfg, page = tiny_configs[name]
    d, _ = model_dirs[name]
    toks = helpers.random_tokens(cfg.vocab_size, 370, 811)
    want = helpers.plain_logits(d, {"r": toks}, weights_as=torch.bfloat16 if dtype == "bfloat16" else None)["r"]
    _c, model = load_model(d, dtype=dtype, device="cuda:0")
    runner = ModelRunner(model, cuda_kernels, page_size=page, num_pages=64, max_seqs=2, cuda_graphs=True)
    runner.portion_graphs = True                             # an option (INFERFLUX_B200_PORTION_GRAPHS=1), off by default
    got, pos = {}, 0
    for k, n in enumerate([64] * 5 + [50]):
        here = list(range(n)) if k != 2 else []              # one portion asks for nothing
        out = runner.step([StepEntry("r", toks[pos:pos + n], here)])
        for j, p in enumerate(here):
            got[pos + p] = out[j].float().cpu().numpy()
        pos += n
    runner.end_request("r")
    assert runner.graph_replays >= 2, "no portion ran from a graph"
    rows = sorted(got)
    check({"r": np.stack([got[p] for p in rows])}, {"r": want[rows]}, dtype, f"portion graphs {name}/{dtype}")
    cuda_kernels.check_errors()


def test_twenty_thousand_tokens_against_the_plain_implementation(tmp_path, cuda_kernels):
    """Positions beyond 16 bits, a block table of 1,250 entries, a window of 9,000 keys on the second
    layer, head size 64 (the tensor-core prompt attention, clusters of blocks in decode): a request of
    20,000 tokens whole and in portions with decoded tokens at the end, against the plain
    implementation run on the GPU in float64."""
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.engine import ModelRunner, StepEntry
    from inferflux_b200.models import load_model
    from plain import plain_qwen2
    cfg = Qwen2Config(hidden_size=136, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
                      intermediate_size=264, vocab_size=640, max_position_embeddings=40000, rope_theta=300000.0,
                      rms_norm_eps=2e-6, tie_word_embeddings=False, use_sliding_window=True, sliding_window=9000,
                      max_window_layers=1)
    T = 20000
    d = helpers.write_tiny_model(cfg, tmp_path / "long", seed=3)
    toks = helpers.random_tokens(cfg.vocab_size, T, 77)
    wanted = sorted(set(list(range(0, T, 997)) + [T - 1 - i for i in range(6)] +
                        [8191, 8192, 8999, 9000, 9001, 16383, 16384]))
    raw, W = plain_qwen2.load_model_dir(d)
    W = {k: v.to(torch.bfloat16).cuda() for k, v in W.items()}
    full = plain_qwen2.forward(raw, W, toks, dtype=torch.float64)
    want = full[torch.tensor(wanted, device=full.device)].cpu().numpy()
    del full, W
    torch.cuda.empty_cache()
    scale = float(np.abs(want).max())
    _c, model = load_model(d, dtype="bfloat16", device="cuda:0")
    runner = ModelRunner(model, cuda_kernels, page_size=16, num_pages=T // 16 + 8, max_seqs=2, cuda_graphs=True)
    for name, cuts in (("whole", [T]), ("portions", [4096, 3000, 5000, 1, T - 12097 - 6] + [1] * 6)):
        got, pos = {}, 0
        for n in cuts:
            here = [p - pos for p in wanted if pos <= p < pos + n]
            out = runner.step([StepEntry(name, toks[pos:pos + n], here)])
            for j, p in enumerate(here):
                got[pos + p] = out[j].float().cpu().numpy()
            pos += n
        runner.end_request(name)
        assert pos == T
        diff = np.abs(np.stack([got[p] for p in wanted]) - want).max(axis=1)
        assert float(diff.max()) < 0.03 * scale, \
            f"{name}: position {wanted[int(diff.argmax())]} differs by {float(diff.max())} (scale {scale})"
    cuda_kernels.check_errors()
    assert not runner.cache.live_requests()
