"""Configuration: config.json keys, defaults, refusals, the registry, engine options."""

from __future__ import annotations

import json

import pytest

from mercury_b200.config import (ConfigError, EngineConfig, Qwen2Config, architecture_named,
                                 config_from_dict, known_architectures, read_model_config,
                                 register_architecture)
from tiny import RAW, TINY_A, TINY_C


def test_fields_come_from_config_json():
    _entry, cfg = config_from_dict(TINY_A)
    assert isinstance(cfg, Qwen2Config)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads) == (64, 2, 4)
    assert (cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size) == (2, 16, 128)
    assert (cfg.vocab_size, cfg.rope_theta, cfg.rms_norm_eps) == (256, 10000.0, 1e-6)
    assert cfg.tie_word_embeddings is True


def test_defaults_for_absent_keys_follow_the_reference():
    raw = {"hidden_size": 96, "intermediate_size": 10, "num_hidden_layers": 1,
           "num_attention_heads": 3, "vocab_size": 7}
    _entry, cfg = config_from_dict(raw)
    assert cfg.architecture == "Qwen2ForCausalLM"
    assert cfg.num_key_value_heads == 3 and cfg.head_dim == 32
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0
    assert cfg.max_position_embeddings == 32768 and cfg.tie_word_embeddings is False
    assert cfg.eos_token_ids == () and cfg.use_sliding_window is False


def test_eos_may_be_an_int_or_a_list():
    assert config_from_dict({**TINY_A, "eos_token_id": 5})[1].eos_token_ids == (5,)
    assert config_from_dict({**TINY_A, "eos_token_id": [5, 9]})[1].eos_token_ids == (5, 9)


@pytest.mark.parametrize("change,word", [
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": False}, "attention_bias"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"use_sliding_window": True, "sliding_window": 0}, "sliding_window"),
])
def test_what_is_not_built_is_refused_by_name(change, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict({**TINY_A, **change})


def test_a_missing_size_is_named():
    raw = dict(TINY_A)
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        config_from_dict(raw)


def test_window_layers():
    _entry, cfg = config_from_dict(TINY_C)
    assert [cfg.layer_window(i) for i in range(3)] == [0, 24, 24]
    _entry, cfg = config_from_dict(TINY_A)
    assert cfg.layer_window(1) == 0


@pytest.mark.parametrize("name", list(RAW))
def test_to_dict_reads_back_equal(name):
    _entry, cfg = config_from_dict(RAW[name])
    assert config_from_dict(cfg.to_dict())[1] == cfg


def test_registry_knows_qwen2_and_names_what_it_knows():
    assert "Qwen2ForCausalLM" in known_architectures()
    assert architecture_named("Qwen2ForCausalLM").config_class is Qwen2Config
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        config_from_dict({**TINY_A, "architectures": ["LlamaForCausalLM"]})


def test_an_architecture_can_be_registered(tmp_path):
    class OtherConfig(Qwen2Config):
        pass

    register_architecture("OtherForCausalLM", OtherConfig, lambda c: None)
    (tmp_path / "config.json").write_text(json.dumps({**TINY_A, "architectures": ["OtherForCausalLM"]}))
    entry, cfg = read_model_config(tmp_path)
    assert entry.name == "OtherForCausalLM" and isinstance(cfg, OtherConfig)


def test_engine_config_checks():
    with pytest.raises(ValueError, match="policy"):
        EngineConfig(policy="random")
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError, match="power of two"):
        EngineConfig(block_size=12)
    with pytest.raises(ValueError, match="max_batched_tokens"):
        EngineConfig(max_running=64, max_batched_tokens=8)
    cfg = EngineConfig(num_blocks=4, block_size=16, max_model_len=128)
    with pytest.raises(ValueError, match="page pool"):
        cfg.validate_against(4096)
    with pytest.raises(ValueError, match="positions"):
        EngineConfig(max_model_len=8192, num_blocks=4096).validate_against(2048)


def test_autosize_blocks_takes_the_fraction_of_what_is_left(monkeypatch):
    """mercury/config.py:164-185: (free - reserve) * fraction // (bytes per token * block)."""
    import torch

    from mercury_b200.config.engine_config import EngineConfig, autosize_blocks

    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda index=0: (10 * 2 ** 30, 16 * 2 ** 30))
    cfg = EngineConfig(block_size=16, gpu_memory_fraction=0.5)
    per_token = 24 * 2 * 2 * 64 * 2
    assert autosize_blocks(per_token, cfg, reserve_bytes=2 * 2 ** 30) == (4 * 2 ** 30) // (per_token * 16)
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda index=0: (2 ** 20, 16 * 2 ** 30))
    import pytest

    with pytest.raises(RuntimeError, match="no room for a cache"):
        autosize_blocks(per_token, cfg, reserve_bytes=2 ** 30)
