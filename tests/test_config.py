"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from helpers import TINY, config_dict
from kuiperllama_b200.config import (ConfigError, LlamaConfig, config_from_dict, config_from_folder,
                                     known_architectures)


def test_registry_maps_the_architecture_name():
    assert "LlamaForCausalLM" in known_architectures()
    cfg = config_from_dict(config_dict("tiny1"))
    assert isinstance(cfg, LlamaConfig)
    with pytest.raises(ConfigError, match="unknown architecture 'MambaForCausalLM'.*LlamaForCausalLM"):
        config_from_dict({"architectures": ["MambaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"hidden_size": 8})


@pytest.mark.parametrize("name", list(TINY))
def test_every_key_is_read_from_config_json(name):
    d = config_dict(name)
    cfg = config_from_dict(d)
    assert cfg.hidden_size == d["hidden_size"] and cfg.intermediate_size == d["intermediate_size"]
    assert cfg.num_hidden_layers == d["num_hidden_layers"] and cfg.vocab_size == d["vocab_size"]
    assert cfg.num_attention_heads == d["num_attention_heads"]
    assert cfg.num_key_value_heads == d["num_key_value_heads"]
    assert cfg.head_dim == d.get("head_dim", d["hidden_size"] // d["num_attention_heads"])
    assert cfg.rms_norm_eps == d["rms_norm_eps"] and cfg.rope_theta == d["rope_theta"]
    assert cfg.tie_word_embeddings == d["tie_word_embeddings"]
    assert cfg.max_position_embeddings == d["max_position_embeddings"]
    eos = d["eos_token_id"]
    assert cfg.eos_token_ids == (tuple(eos) if isinstance(eos, list) else (eos,))
    if d["rope_scaling"] is None:
        assert cfg.rope_scaling is None
    else:
        assert cfg.rope_scaling.factor == d["rope_scaling"]["factor"]
        assert cfg.rope_scaling.original_max_position_embeddings == d["rope_scaling"]["original_max_position_embeddings"]
    # round trip through to_dict
    assert config_from_dict(cfg.to_dict()) == cfg


def test_defaults_follow_the_reference():
    d = config_dict("tiny1")
    for k in ("num_key_value_heads", "rms_norm_eps", "rope_theta", "rope_scaling", "tie_word_embeddings"):
        d.pop(k, None)
    cfg = config_from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads      # tools/export_llama3.py:499
    assert cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0   # rmsnorm_kernel.cu:123, rope_kernel.cu:128
    assert cfg.rope_scaling is None and cfg.tie_word_embeddings is False


def test_all_faults_are_listed_in_one_error():
    d = config_dict("tiny2", num_key_value_heads=4, hidden_act="gelu", attention_bias=True)
    d["rope_scaling"] = {"rope_type": "yarn", "factor": 2.0}
    del d["vocab_size"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    msg = str(e.value)
    for needle in ('missing key "vocab_size"', "not a multiple", "yarn", "gelu", "attention_bias"):
        assert needle in msg, (needle, msg)


@pytest.mark.parametrize("bad", [{"hidden_size": "64"}, {"num_hidden_layers": 0}, {"rms_norm_eps": -1.0},
                                 {"head_dim": 15}, {"eos_token_id": "two"}, {"rope_theta": 0}])
def test_bad_values(bad):
    with pytest.raises(ConfigError):
        config_from_dict(config_dict("tiny1", **bad))


def test_from_folder(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_folder(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        config_from_folder(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(config_dict("tiny3")))
    assert config_from_folder(str(tmp_path)).head_dim == 64


def test_model_spec_is_layer_by_layer_data():
    cfg = config_from_dict(config_dict("tiny2"))
    spec = cfg.to_model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.lm_head_name is None and spec.stop_token_ids == (7, 9)
    layer = spec.layers[1]
    assert layer.prefix == "model.layers.1." and layer.arrangement == "pre_norm"
    assert layer.mixer.kind == "attention" and layer.mixer["num_kv_heads"] == 2 and layer.mixer["head_dim"] == 32
    assert layer.feed_forward.kind == "swiglu" and layer.feed_forward["intermediate_size"] == 512
    assert layer.mixer_norm["eps"] == 1e-6 and layer.position["theta"] == 500000.0
    assert layer.position["scaling"]["rope_type"] == "llama3"


def test_schedule_validation():
    import dataclasses
    from kuiperllama_b200.config import ScheduleEntry
    spec = config_from_dict(config_dict("tiny1")).to_model_spec()
    ok = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_from=1)))
    ok.validate()                                                  # a layer twice, a cache read from another entry
    for bad in [(ScheduleEntry(2),), (ScheduleEntry(0, cache_from=0),), (ScheduleEntry(0), ScheduleEntry(1, cache_from=3)),
                (ScheduleEntry(0), ScheduleEntry(1, cache_from=0), ScheduleEntry(0, cache_from=1))]:
        with pytest.raises(ValueError):
            dataclasses.replace(spec, schedule=bad).validate()
