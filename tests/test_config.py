"""Configuration reading, validation and the architecture registry."""
import json

import pytest

from inferflux_b200.config import (ConfigError, Qwen2Config, ScheduleEntry, config_from_dict, load_config,
                                   registered_architectures)

BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 64, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 176, "vocab_size": 512,
        "max_position_embeddings": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True}


def test_reads_every_key_and_derives_head_dim():
    cfg = config_from_dict(dict(BASE))
    assert isinstance(cfg, Qwen2Config)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (64, 2, 4, 2)
    assert cfg.head_dim == 16 and cfg.intermediate_size == 176 and cfg.vocab_size == 512
    assert cfg.tie_word_embeddings and cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0
    cfg2 = config_from_dict({**BASE, "head_dim": 48})
    assert cfg2.head_dim == 48                       # head_dim need not be hidden_size / heads


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in BASE.items() if k not in ("rope_theta", "rms_norm_eps", "num_key_value_heads",
                                                      "tie_word_embeddings")}
    cfg = config_from_dict(raw)
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6
    assert cfg.num_key_value_heads == cfg.num_attention_heads and not cfg.tie_word_embeddings


def test_model_type_alone_is_enough():
    raw = dict(BASE)
    del raw["architectures"]
    assert isinstance(config_from_dict(raw), Qwen2Config)


@pytest.mark.parametrize("change,word", [
    ({"hidden_size": None}, "missing"), ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"), ({"rms_norm_eps": 0}, "rms_norm_eps"), ({"vocab_size": -1}, "positive"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"num_hidden_layers": 2.5}, "integer"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"hidden_size": 66}, "multiple")])
def test_bad_values_are_refused(change, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict({**BASE, **change})
    assert word in str(e.value)


def test_unknown_architecture_lists_the_known_ones():
    with pytest.raises(ConfigError) as e:
        config_from_dict({**BASE, "architectures": ["MambaForCausalLM"], "model_type": "mamba"})
    assert "Qwen2ForCausalLM" in str(e.value) and "Qwen2ForCausalLM" in registered_architectures()


def test_load_config_errors(tmp_path):
    with pytest.raises(ConfigError):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(BASE))
    assert load_config(tmp_path).vocab_size == 512


def test_round_trip_through_to_dict():
    cfg = config_from_dict({**BASE, "use_sliding_window": True, "sliding_window": 9, "max_window_layers": 1})
    again = config_from_dict(cfg.to_dict())
    assert again == cfg


def test_plan_layer_by_layer():
    cfg = config_from_dict({**BASE, "num_hidden_layers": 3, "use_sliding_window": True, "sliding_window": 9,
                            "max_window_layers": 1})
    plan = cfg.to_plan()
    assert [l.mixer.params["window"] for l in plan.layers] == [None, 9, 9]
    assert [l.mixer.params["head_dim"] for l in plan.layers] == [16, 16, 16]
    assert plan.layers[0].norm_mixer.params["eps"] == 1e-6
    assert [(e.layer, e.cache) for e in plan.schedule] == [(0, 0), (1, 1), (2, 2)]
    assert plan.lm_head.params["tied"] is True and plan.num_caches == 3


def test_schedule_is_checked():
    plan = config_from_dict(dict(BASE)).to_plan()
    plan.schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(1, 2), ScheduleEntry(0, 1, False)]
    plan.validate()                                   # a layer named twice, a layer reading another's cache
    plan.schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 0)]
    with pytest.raises(ValueError):
        plan.validate()                               # two writers of one cache
    plan.schedule = [ScheduleEntry(0, 1, False), ScheduleEntry(1, 1)]
    with pytest.raises(ValueError):
        plan.validate()                               # read before written
    plan.schedule = [ScheduleEntry(5, 0)]
    with pytest.raises(ValueError):
        plan.validate()


def test_a_head_size_the_kernels_do_not_take_is_refused_when_the_config_is_read():
    from inferflux_b200.config import ConfigError, config_from_dict
    raw = dict(architectures=["Qwen2ForCausalLM"], hidden_size=96, num_hidden_layers=1, num_attention_heads=8,
               num_key_value_heads=2, intermediate_size=64, vocab_size=100)
    with pytest.raises(ConfigError, match="head size 12"):          # hidden_size / heads, no head_dim given
        config_from_dict(raw)
    for head_dim in (12, 20, 264, 320):
        with pytest.raises(ConfigError, match="head size"):
            config_from_dict(dict(raw, head_dim=head_dim))
    for head_dim in (8, 24, 128, 256):
        assert config_from_dict(dict(raw, head_dim=head_dim)).head_dim == head_dim


def test_model_load_spec_validates_and_feeds_the_engine(tmp_path):
    from inferflux_b200.engine import ModelLoadSpec
    ok = ModelLoadSpec(path="m", dtype="float32", context_size=512, max_parallel_sequences=4, kv_num_pages=64)
    assert ok.validate() == "" and ok.name == "m"
    kw = ok.engine_kwargs()
    assert kw["kv_max_batch"] == 4 and kw["kv_max_seq"] == 512 and kw["dtype"] == "float32" and kw["kv_num_pages"] == 64
    for change, word in ((dict(path=""), "path"), (dict(format="gguf"), "format"), (dict(dtype="int8"), "dtype"),
                         (dict(device="rocm:0"), "device"), (dict(context_size=0), "context_size"),
                         (dict(max_parallel_sequences=300), "max_parallel_sequences"),
                         (dict(kv_cache_type="q8_0"), "kv_cache_type"), (dict(kv_page_size=0), "kv_page_size"),
                         (dict(kv_budget_ratio=0.0), "kv_budget_ratio"), (dict(max_batch_tokens=0), "max_batch_tokens")):
        import dataclasses
        bad = dataclasses.replace(ok, **change)
        assert word in bad.validate()
        with pytest.raises(ValueError, match="model load spec"):
            bad.checked()


def test_inferctl_info_describes_a_model_folder(tmp_path, capsys):
    import json
    import torch
    from inferflux_b200.cli.main import main
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.weights import write_random_model
    cfg = Qwen2Config(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                      intermediate_size=96, vocab_size=128)
    write_random_model(cfg, tmp_path, seed=1, dtype=torch.bfloat16)
    assert main(["info", "--model", str(tmp_path)]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["model"]["architecture"] == "Qwen2ForCausalLM" and out["model"]["kv_bytes_per_token_bf16"] == 2 * 3 * 2 * 16 * 2
    assert "attention" in out["engine"]["parts"]["mixer"]
