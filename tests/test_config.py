"""Typed configuration from config.json keys, and the architecture registry."""
import json

import pytest

from tiny_llm_infer_b200 import models  # noqa: F401
from tiny_llm_infer_b200.config import (ConfigError, Qwen3Config, config_from_dict, describe_model,
                                        known_architectures, load_config)
from tiny import TINIES

RAW = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 96,
       "intermediate_size": 200, "num_hidden_layers": 3, "num_attention_heads": 6,
       "num_key_value_heads": 2, "head_dim": 32, "vocab_size": 384, "max_position_embeddings": 256,
       "rms_norm_eps": 1e-5, "rope_theta": 1e6, "tie_word_embeddings": False}


def test_reads_every_size_from_its_own_keys():
    cfg = config_from_dict(RAW)
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (96, 200, 3)
    assert (cfg.q_dim, cfg.kv_dim, cfg.group_size) == (192, 64, 3)      # query width != hidden
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and not cfg.tie_word_embeddings
    assert cfg.layer_types == ("full_attention",) * 3 and cfg.sliding_window is None


def test_defaults_of_the_reference():
    raw = {k: v for k, v in RAW.items() if k not in ("head_dim", "rms_norm_eps", "rope_theta", "architectures")}
    cfg = config_from_dict(raw)                 # found through model_type
    assert cfg.head_dim == 16 and cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 1e6


def test_round_trip_and_folder(tmp_path):
    for tiny in TINIES.values():
        cfg = tiny["cfg"]
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
        assert load_config(tmp_path) == cfg


def test_sliding_window_keys():
    raw = dict(RAW, use_sliding_window=True, sliding_window=24, max_window_layers=1)
    cfg = config_from_dict(raw)
    assert cfg.layer_types == ("full_attention", "sliding_attention", "sliding_attention")
    assert cfg.window_of_layer(0) is None and cfg.window_of_layer(2) == 24
    raw = dict(RAW, sliding_window=24, layer_types=["sliding_attention", "full_attention", "full_attention"])
    assert config_from_dict(raw).window_of_layer(0) == 24
    assert config_from_dict(dict(RAW, sliding_window=24)).sliding_window is None   # present but not enabled


@pytest.mark.parametrize("change,match", [
    ({"hidden_size": None}, "hidden_size"), ({"num_hidden_layers": 0}, "positive"),
    ({"num_key_value_heads": 4}, "multiple"), ({"head_dim": 15}, "even"),
    ({"architectures": ["LlamaForCausalLM"]}, "unknown architecture"),
    ({"model_type": "qwen2"}, "qwen3"), ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"attention_bias": True}, "attention_bias"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"vocab_size": "many"}, "integer"), ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"use_sliding_window": True, "max_window_layers": 0}, "sliding_window"),
    ({"eos_token_id": 99999}, "vocabulary"),
])
def test_errors(change, match):
    with pytest.raises(ConfigError, match=match):
        config_from_dict(dict(RAW, **change))


def test_registry_lists_known_names():
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict({"architectures": ["Nope"]})
    with pytest.raises(ConfigError, match="no config.json"):
        load_config("/nonexistent-folder")


def test_description_is_data():
    cfg = TINIES["C"]["cfg"]
    desc = describe_model(cfg)
    assert len(desc.layers) == 4 and [e.layer for e in desc.order] == [0, 1, 2, 3]
    windows = [l.parts["mixer"].params["window"] for l in desc.layers]
    assert windows == [24, None, 24, 24]
    assert desc.layers[2].parts["mixer"].prefix == "model.layers.2.self_attn."
    assert desc.head.params["tied"] is False
