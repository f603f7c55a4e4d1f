"""Weights from a model folder straight to the device: mapped file -> pinned buffers -> GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tensors_reach_the_device_unchanged_through_small_staging_chunks(tmp_path, monkeypatch):
    from inferflux_b200.weights import SafetensorsFile, load_weights, write_safetensors
    from inferflux_b200.weights import loader
    from inferflux_b200.weights.loader import TensorSpec
    monkeypatch.setattr(loader._Staging, "CHUNK", 4096)            # many chunks, ragged last one
    g = torch.Generator().manual_seed(3)
    tensors = {
        "a.weight": torch.randn(333, 77, generator=g).to(torch.bfloat16),
        "b.weight": torch.randn(1000, 130, generator=g),                           # 32-bit stays 32-bit
        "c.table": torch.randint(0, 1000, (4097,), generator=g, dtype=torch.int64),  # integer tables become int32
        "d.weight": torch.randn(5, 3, generator=g).to(torch.float16),             # 16-bit is kept as bfloat16
    }
    write_safetensors(tmp_path / "model.safetensors", tensors, metadata={"x": "y" * 3})   # odd header length
    expected = {n: TensorSpec(tuple(t.shape)) for n, t in tensors.items()}
    got = load_weights(tmp_path, expected, device="cuda:0")
    assert got["a.weight"].dtype == torch.bfloat16 and torch.equal(got["a.weight"].cpu(), tensors["a.weight"])
    assert got["b.weight"].dtype == torch.float32 and torch.equal(got["b.weight"].cpu(), tensors["b.weight"])
    assert got["c.table"].dtype == torch.int32 and torch.equal(got["c.table"].cpu().long(), tensors["c.table"])
    assert got["d.weight"].dtype == torch.bfloat16
    assert torch.equal(got["d.weight"].cpu(), tensors["d.weight"].to(torch.bfloat16))
    with SafetensorsFile(tmp_path / "model.safetensors") as f:
        v = f.view("b.weight")
        assert torch.equal(v, tensors["b.weight"])
        del v


def test_the_same_seed_gives_the_same_bits_on_the_host_and_on_the_device(tmp_path):
    """`random_model` on the GPU, `write_random_model` on the host and a folder loaded back hold
    bit-identical weights: element i of a tensor depends on (seed, name, i) alone."""
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.models import expected_tensors
    from inferflux_b200.weights import SafetensorsFile, write_random_model
    from inferflux_b200.weights.random_init import counter_normal, random_tensors
    cfg = Qwen2Config(hidden_size=136, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
                      intermediate_size=264, vocab_size=641, max_position_embeddings=128)
    specs = expected_tensors(cfg.to_plan())
    for dtype in (torch.bfloat16, torch.float32):
        on_device = random_tensors(specs, seed=9, dtype=dtype, device="cuda:0", norm_jitter=0.1)
        write_random_model(cfg, tmp_path / str(dtype), seed=9, dtype=dtype, norm_jitter=0.1)
        with SafetensorsFile(tmp_path / str(dtype) / "model.safetensors") as f:
            assert sorted(f.names()) == sorted(on_device)
            for n in f.names():
                assert torch.equal(f.tensor(n), on_device[n].cpu()), (n, dtype)
    # a tensor of more than 2^21 elements (several host chunks), odd size, another seed and a large one
    for seed in (0, 2 ** 40 + 17):
        host = counter_normal((3, 1_400_001), seed, "x.weight", 0.0, 0.02, torch.float32, "cpu")
        dev = counter_normal((3, 1_400_001), seed, "x.weight", 0.0, 0.02, torch.float32, "cuda:0")
        assert torch.equal(host, dev.cpu())
    assert abs(float(host.std()) - 0.02) < 2e-4 and abs(float(host.mean())) < 1e-4


def test_a_float16_file_in_a_32_bit_run_matches_the_plain_implementation(tmp_path, cuda_kernels):
    """The 32-bit path computes with the float16 values of the file, not with their bfloat16 roundings."""
    import helpers
    from inferflux_b200.engine import ModelRunner, StepEntry
    from inferflux_b200.models import load_model
    from inferflux_b200.weights import SafetensorsFile, write_safetensors
    from plain import plain_qwen2
    cfg, _page = helpers.tiny_configs()["B"]
    d = helpers.write_tiny_model(cfg, tmp_path / "m", seed=21, dtype=torch.float32)
    with SafetensorsFile(d / "model.safetensors") as f:
        tensors = {n: f.tensor(n).to(torch.float16) for n in f.names()}
    write_safetensors(d / "model.safetensors", tensors, metadata={"format": "pt"})
    toks = helpers.random_tokens(cfg.vocab_size, 45, 5)
    raw, W = plain_qwen2.load_model_dir(d)
    want = plain_qwen2.forward(raw, W, toks, dtype=torch.float64)
    _c, model = load_model(d, dtype="float32", device="cuda:0")
    runner = ModelRunner(model, cuda_kernels, page_size=8, num_pages=8, max_seqs=2)
    got = runner.step([StepEntry("r", toks, list(range(len(toks))))]).double().cpu()
    assert float((got - want).abs().max()) < 1e-4


def test_loading_never_holds_much_more_than_the_model(tmp_path):
    """A folder of the 1.5B layer sizes (six layers, tied head) is loaded part by part: stacked matrices are
    filled slice by slice in their final place, so the peak of device memory stays within a tenth of the
    model's own bytes; every part's tensors sit in one allocation at offsets that are multiples of 256."""
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.models import expected_tensors, load_model
    from inferflux_b200.weights import random_tensors, write_safetensors
    import json
    cfg = Qwen2Config(hidden_size=1536, num_hidden_layers=6, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                      intermediate_size=8960, vocab_size=151936, tie_word_embeddings=True, max_position_embeddings=1024)
    W = random_tensors(expected_tensors(cfg.to_plan()), 3, dtype=torch.bfloat16, device="cuda:0")
    write_safetensors(tmp_path / "model.safetensors", {n: t.cpu() for n, t in W.items()}, metadata={"format": "pt"})
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    model_bytes = sum(t.numel() * t.element_size() for t in W.values())
    probe = {n: W[n].clone() for n in ("model.layers.3.self_attn.k_proj.weight", "model.layers.5.mlp.up_proj.weight")}
    del W
    torch.cuda.empty_cache()
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    _c, model = load_model(tmp_path, dtype="bfloat16", device="cuda:0")
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    held = torch.cuda.memory_allocated() - base
    assert held <= 1.02 * model_bytes + (8 << 20), (held, model_bytes)       # norms and biases are kept in float32
    assert peak <= 1.1 * model_bytes, f"peak {peak / 2**20:.0f} MiB for a model of {model_bytes / 2**20:.0f} MiB"
    a = model.layers[3].mixer
    q, kv = a.nq * a.d, a.nkv * a.d
    assert torch.equal(a.w_qkv[q:q + kv], probe["model.layers.3.self_attn.k_proj.weight"])
    f = model.layers[5].ffn
    assert torch.equal(f.w_gate_up[f.inter:], probe["model.layers.5.mlp.up_proj.weight"])
    for t in (a.w_qkv, a.w_o, a.b_qkv, f.w_gate_up, f.w_down):
        assert t.data_ptr() % 256 == 0 and t.is_contiguous()
    assert a.w_qkv.untyped_storage().data_ptr() == a.w_o.untyped_storage().data_ptr()      # one allocation a part
