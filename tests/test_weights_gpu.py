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
