"""Safetensors IO, checked loading by name, random-weights mode."""
import json
import struct

import pytest
import torch

from inferflux_b200.config import Qwen2Config
from inferflux_b200.models import expected_tensors, load_model
from inferflux_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights,
                                    write_random_model, write_safetensors)

CFG = Qwen2Config(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                  intermediate_size=48, vocab_size=100, max_position_embeddings=64)


def rewrite(path, change):
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    change(tensors)
    write_safetensors(path, tensors)


def test_round_trip_and_own_reader_agree(tmp_path):
    from plain.plain_qwen2 import read_safetensors
    t = {"a": torch.randn(3, 4), "b.c": torch.randn(5).to(torch.bfloat16), "i": torch.arange(6, dtype=torch.int64),
         "empty": torch.zeros(0, 2)}
    write_safetensors(tmp_path / "x.safetensors", t, metadata={"k": "v"})
    with SafetensorsFile(tmp_path / "x.safetensors") as f:
        assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
        for n in t:
            assert torch.equal(f.tensor(n), t[n]) and f.shape(n) == tuple(t[n].shape)
    other = read_safetensors(tmp_path / "x.safetensors")
    assert all(torch.equal(other[n], t[n]) for n in t)
    try:
        from safetensors.torch import load_file
    except ImportError:
        return
    lib = load_file(str(tmp_path / "x.safetensors"))          # the format's own library reads our files
    assert all(torch.equal(lib[n], t[n]) for n in t)


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "m.safetensors"
    write_safetensors(p, {"w": torch.randn(4, 4)})
    raw = p.read_bytes()
    p.write_bytes(raw[:-10])                                    # truncated data
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    p.write_bytes(raw[:5])
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 10 ** 9) + raw[8:])
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 4) + b"nope" + raw[8:])
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    header = json.dumps({"w": {"dtype": "F32", "shape": [4, 5], "data_offsets": [0, 64]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 64)
    with pytest.raises(SafetensorsError, match="needs 80"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="no safetensors files"):
        load_weights(tmp_path / "nowhere", {})


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(CFG, tmp_path / "m", seed=1, dtype=torch.bfloat16)

    def change(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.q_norm.weight"] = torch.ones(8)
        t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 31)
        t["lm_head.weight"] = torch.zeros(100, 33)
    rewrite(d / "model.safetensors", change)
    with pytest.raises(WeightError) as e:
        load_model(d, dtype="float32", device="cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert sorted(n for n, _g, _w in err.wrong_shape) == ["lm_head.weight", "model.layers.0.self_attn.k_proj.weight"]
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "is [16, 31], expected [16, 32]"):
        assert word in msg


def test_biases_are_optional_and_tied_head_is_not_required(tmp_path):
    import dataclasses
    cfg = dataclasses.replace(CFG, tie_word_embeddings=True, qkv_bias=False)
    d = write_random_model(cfg, tmp_path / "m", seed=2, dtype=torch.bfloat16)
    with SafetensorsFile(d / "model.safetensors") as f:
        names = set(f.names())
    assert "lm_head.weight" not in names and not any(n.endswith(".bias") for n in names)
    _c, model = load_model(d, dtype="float32", device="cpu")
    assert model.layers[0].mixer.b_qkv is None
    assert model.lm_head.weight is model.embedding.table
    # a tied model whose file also carries lm_head.weight: the configuration decides, the tensor is ignored
    rewrite(d / "model.safetensors", lambda t: t.update({"lm_head.weight": torch.zeros(100, 32)}))
    with pytest.warns(UserWarning, match="lm_head.weight is present but not used"):
        _c, model = load_model(d, dtype="float32", device="cpu")
    assert model.lm_head.weight is model.embedding.table
    # buffers of older exports that no part uses are skipped with a warning, not an error
    rewrite(d / "model.safetensors", lambda t: (t.pop("lm_head.weight"),
                                                t.update({"model.layers.0.self_attn.rotary_emb.inv_freq": torch.ones(8)})))
    with pytest.warns(UserWarning, match="skipped"):
        load_model(d, dtype="float32", device="cpu")


def test_a_float16_file_reaches_a_32_bit_run_without_passing_through_bfloat16(tmp_path):
    """float16 has three more bits than bfloat16: a float32 run computes with the file's own values."""
    d = write_random_model(CFG, tmp_path / "m", seed=4, dtype=torch.float32)
    rewrite(d / "model.safetensors", lambda t: t.update({n: v.to(torch.float16) for n, v in t.items()}))
    with SafetensorsFile(d / "model.safetensors") as f:
        halves = {n: f.tensor(n) for n in f.names()}
    assert all(v.dtype == torch.float16 for v in halves.values())
    _c, model = load_model(d, dtype="float32", device="cpu")
    assert torch.equal(model.layers[0].ffn.w_down, halves["model.layers.0.mlp.down_proj.weight"].float())
    assert not torch.equal(model.layers[0].ffn.w_down, halves["model.layers.0.mlp.down_proj.weight"].to(torch.bfloat16).float())
    _c, model16 = load_model(d, dtype="bfloat16", device="cpu")
    assert model16.layers[0].ffn.w_down.dtype == torch.bfloat16


def test_stored_dtypes(tmp_path):
    d = write_random_model(CFG, tmp_path / "m", seed=3, dtype=torch.bfloat16)
    def change(t):
        t["model.norm.weight"] = t["model.norm.weight"].float()          # stored in 32-bit: stays so
        t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].half()
    rewrite(d / "model.safetensors", change)
    got = load_weights(d, expected_tensors(CFG.to_plan()))
    assert got["model.norm.weight"].dtype == torch.float32
    assert got["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    a = write_random_model(CFG, tmp_path / "a", seed=7, dtype=torch.float32)
    b = write_random_model(CFG, tmp_path / "b", seed=7, dtype=torch.float32)
    c = write_random_model(CFG, tmp_path / "c", seed=8, dtype=torch.float32)
    import dataclasses
    e = write_random_model(dataclasses.replace(CFG, num_hidden_layers=3), tmp_path / "e", seed=7, dtype=torch.float32)
    fa, fb, fc, fe = (SafetensorsFile(x / "model.safetensors") for x in (a, b, c, e))
    n = "model.layers.1.self_attn.q_proj.weight"
    assert torch.equal(fa.tensor(n), fb.tensor(n)) and not torch.equal(fa.tensor(n), fc.tensor(n))
    assert torch.equal(fa.tensor(n), fe.tensor(n))                   # other tensors existing changes nothing
    w = fa.tensor(n)
    assert abs(float(w.std()) - 0.02) < 0.004 and torch.equal(fa.tensor("model.norm.weight"), torch.ones(32))
    cfg = json.loads((a / "config.json").read_text())
    assert cfg["architectures"] == ["Qwen2ForCausalLM"] and cfg["hidden_size"] == 32
    for f in (fa, fb, fc, fe):
        f.close()


def test_sharded_folder(tmp_path):
    d = write_random_model(CFG, tmp_path / "m", seed=4, dtype=torch.bfloat16)
    with SafetensorsFile(d / "model.safetensors") as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    (d / "model.safetensors").unlink()
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(d / "model-00001-of-00002.safetensors", {n: tensors[n] for n in names[:half]})
    write_safetensors(d / "model-00002-of-00002.safetensors", {n: tensors[n] for n in names[half:]})
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    got = load_weights(d, expected_tensors(CFG.to_plan()))
    assert all(torch.equal(got[n], tensors[n]) for n in names)


def test_made_up_weights_depend_on_seed_name_and_element_only():
    from inferflux_b200.weights.random_init import counter_normal, counter_normal_numpy, tensor_key
    a = counter_normal((7, 33), 5, "model.layers.0.mlp.up_proj.weight", 0.0, 0.02)
    again = counter_normal((7, 33), 5, "model.layers.0.mlp.up_proj.weight", 0.0, 0.02)
    assert torch.equal(a, again)
    # element i is the same whatever the tensor's shape or the chunk it is made in
    flat = counter_normal((231,), 5, "model.layers.0.mlp.up_proj.weight", 0.0, 0.02)
    assert torch.equal(a.reshape(-1), flat)
    k0, k1 = tensor_key(5, "model.layers.0.mlp.up_proj.weight")
    tail = counter_normal_numpy(31, k0, k1, 0.0, 0.02, first=200)
    assert (flat.numpy()[200:] == tail).all()
    # another name or another seed: other values
    assert not torch.equal(a, counter_normal((7, 33), 5, "model.layers.1.mlp.up_proj.weight", 0.0, 0.02))
    assert not torch.equal(a, counter_normal((7, 33), 6, "model.layers.0.mlp.up_proj.weight", 0.0, 0.02))
    big = counter_normal((400, 500), 1, "w", 0.0, 1.0).double()
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01
    kurt = float(((big - big.mean()) ** 4).mean() / big.var() ** 2) - 3.0
    assert abs(kurt) < 0.05
    # bfloat16 is the float32 value rounded once
    assert torch.equal(counter_normal((7, 33), 5, "n", 0.0, 0.02, torch.bfloat16), counter_normal((7, 33), 5, "n", 0.0, 0.02).to(torch.bfloat16))
