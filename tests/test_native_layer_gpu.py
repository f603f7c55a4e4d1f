"""Whole layers launched from native code (csrc/layer_forward.cu) against the same layers run part by part
from Python: the kernels and their arguments are meant to be the same, so the logits must agree bit for bit,
however the tokens are cut into steps, with and without CUDA graphs."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def run(model, kernels, steps, vocab, native, monkeypatch, page_size=16, num_pages=24, cuda_graphs=False):
    from inferflux_b200.engine import ModelRunner
    monkeypatch.setattr(kernels, "native_layers", native)
    runner = ModelRunner(model, kernels, page_size=page_size, num_pages=num_pages, max_seqs=4, cuda_graphs=cuda_graphs)
    before = kernels.native_layer_calls
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), vocab)
    kernels.check_errors()
    assert not runner.cache.live_requests()
    return got, kernels.native_layer_calls - before


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_tiny_models_native_layers_equal_parts_one_by_one(name, model_dirs, tiny_configs, cuda_kernels, monkeypatch):
    from inferflux_b200.models import load_model
    cfg, page = tiny_configs[name]
    folder, _ = model_dirs[name]
    _c, model = load_model(folder, dtype="bfloat16", device="cuda:0")
    reqs = {f"r{i}": helpers.random_tokens(cfg.vocab_size, n, 40 + i) for i, n in enumerate((91, 50, 67))}
    for make_trace in (helpers.trace_whole, helpers.trace_tail, helpers.trace_portions, lambda r: helpers.trace_mixed(r, 256)):
        steps = make_trace(reqs)
        pages = 512 // page + 8
        parts, none = run(model, cuda_kernels, steps, cfg.vocab_size, False, monkeypatch, page_size=page, num_pages=pages)
        native, calls = run(model, cuda_kernels, steps, cfg.vocab_size, True, monkeypatch, page_size=page, num_pages=pages)
        assert none == 0 and calls > len(steps)
        for rid in reqs:
            assert np.array_equal(parts[rid], native[rid]), f"{name}/{rid}: {np.abs(parts[rid] - native[rid]).max()}"


@pytest.mark.parametrize("shape,rows", [("1.5b", (300, 45, 130)), ("7b", (170, 20))])
def test_real_layer_sizes_native_layers_equal_parts_one_by_one(shape, rows, cuda_kernels, monkeypatch):
    """Two layers of the real sizes: few rows (K slices, pre-normed rows), 129-160 rows, and many rows (cuBLAS and
    the tiled gate/up product) all occur among the steps; decoding runs as CUDA graphs too."""
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.models import random_model
    from test_real_shapes_gpu import SHAPES
    cfg = Qwen2Config(num_hidden_layers=2, max_position_embeddings=1024, **SHAPES[shape])
    model = random_model(cfg, seed=8, dtype="bfloat16", device="cuda:0", norm_jitter=0.2)
    reqs = {f"r{i}": helpers.random_tokens(cfg.vocab_size, n, 900 + i) for i, n in enumerate(rows)}
    for make_trace, graphs in ((helpers.trace_whole, False), (helpers.trace_tail, True),
                               (lambda r: helpers.trace_mixed(r, 640), False)):
        steps = make_trace(reqs)
        parts, _ = run(model, cuda_kernels, steps, cfg.vocab_size, False, monkeypatch, num_pages=48, cuda_graphs=graphs)
        native, calls = run(model, cuda_kernels, steps, cfg.vocab_size, True, monkeypatch, num_pages=48, cuda_graphs=graphs)
        assert calls > 0
        for rid in reqs:
            assert np.array_equal(parts[rid], native[rid]), f"{shape}/{rid}: {np.abs(parts[rid] - native[rid]).max()}"


def test_a_captured_graph_outlives_the_growth_of_the_layer_workspace(monkeypatch):
    """Decoding is captured into a CUDA graph while the layer workspace is small; a long prompt of another request
    then makes the kernel table take a larger one; the graph, replayed afterwards, still finds the memory it was
    captured with.  A kernel table of its own, so that the workspace starts empty."""
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.csrc import CudaKernels
    from inferflux_b200.models import random_model
    from test_real_shapes_gpu import SHAPES
    kernels = CudaKernels("cuda:0")
    cfg = Qwen2Config(num_hidden_layers=2, max_position_embeddings=2048, **SHAPES["1.5b"])
    model = random_model(cfg, seed=5, dtype="bfloat16", device="cuda:0", norm_jitter=0.2)
    a = helpers.random_tokens(cfg.vocab_size, 60, 1)
    b = helpers.random_tokens(cfg.vocab_size, 900, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [39]}], "end": []}]
    for i in range(40, 50):                                 # first seen, captured, then replayed
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [a[i]], "want": [0]}], "end": []})
    steps.append({"step": len(steps), "entries": [{"id": "b", "tokens": b, "want": [0, 899]}], "end": ["b"]})
    for i in range(50, 60):
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [a[i]], "want": [0]}],
                      "end": ["a"] if i == 59 else []})
    parts, _ = run(model, kernels, steps, cfg.vocab_size, False, monkeypatch, num_pages=96, cuda_graphs=True)
    assert kernels._layer_ws is None
    native, calls = run(model, kernels, steps, cfg.vocab_size, True, monkeypatch, num_pages=96, cuda_graphs=True)
    assert calls > 0 and len(kernels._layer_ws_all) >= 2, "the long prompt was meant to outgrow the first workspace"
    for rid in ("a", "b"):
        assert np.array_equal(parts[rid], native[rid]), f"{rid}: {np.abs(parts[rid] - native[rid]).max()}"


def test_native_layers_beside_layers_of_other_parts(cuda_kernels, monkeypatch):
    """A model whose schedule runs the framework's attention layer, then a layer of the tests' own parts (a mixer
    with state, a routed feed-forward), then the attention layer again: the first and the last run natively,
    the middle one part by part, and the unadded delta passes between them in both directions."""
    import test_parts_gpu as toys
    from inferflux_b200.models import Model
    from inferflux_b200.weights import random_tensors
    toys._register_toys()
    H, V, I = 64, 300, 96
    model = Model(toys._toy_plan(H, V, I))
    tensors = random_tensors(model.expected_tensors(), seed=3, dtype=torch.float32, std=0.08, norm_jitter=0.1)
    tensors["model.embed_tokens.weight"] *= 10
    model.load(tensors, torch.bfloat16, "cuda:0")
    reqs = {f"r{i}": helpers.random_tokens(V, n, 200 + i) for i, n in enumerate([40, 33, 50])}
    for make_trace in (helpers.trace_whole, helpers.trace_portions, lambda r: helpers.trace_mixed(r, 192)):
        steps = make_trace(reqs)
        parts, none = run(model, cuda_kernels, steps, V, False, monkeypatch, page_size=8, num_pages=24)
        native, calls = run(model, cuda_kernels, steps, V, True, monkeypatch, page_size=8, num_pages=24)
        assert none == 0 and calls > 0 and calls % 2 == 0          # two of the three schedule entries a step
        for rid in reqs:
            assert np.array_equal(parts[rid], native[rid]), f"{rid}: {np.abs(parts[rid] - native[rid]).max()}"


def test_a_block_of_other_parts_is_left_to_its_parts(cuda_kernels):
    """The native code runs exactly one arrangement of exactly these parts: a subclass may have changed a forward."""
    from inferflux_b200.parts.attention import Attention
    from inferflux_b200.parts.block import PreNormBlock

    class Block2(PreNormBlock):
        pass

    b = object.__new__(Block2)
    assert cuda_kernels._native_parts(b) is None and Attention is not None
