"""Configuration reading and the architecture registry."""

from __future__ import annotations

import json

import pytest

from acvram_b200.config import ConfigError, Qwen3Config, REGISTRY, load_config, register_architecture
from conftest import tiny_config


def write(tmp_path, cfg):
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    return str(tmp_path)


def test_round_trip_and_registry(tmp_path):
    cfg = tiny_config("B")
    again = load_config(write(tmp_path, cfg.to_dict()))
    assert again == cfg and isinstance(again, Qwen3Config)
    assert "Qwen3ForCausalLM" in REGISTRY


def test_defaults_are_the_references(tmp_path):
    """Absent keys take the reference's defaults (acvram/engine/config.py:891-906)."""
    cfg = load_config(write(tmp_path, {"architectures": ["Qwen3ForCausalLM"]}))
    assert (cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (4096, 11008, 32)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (32, 32, 128)
    assert (cfg.vocab_size, cfg.max_position_embeddings) == (32000, 4096)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0 and cfg.tie_word_embeddings is False
    cfg = load_config(write(tmp_path, {"architectures": ["Qwen3ForCausalLM"], "norm_epsilon": 3e-6}))
    assert cfg.rms_norm_eps == 3e-6


def test_real_qwen3_8b_keys(tmp_path):
    cfg = load_config(write(tmp_path, {
        "architectures": ["Qwen3ForCausalLM"], "attention_bias": False, "attention_dropout": 0.0, "bos_token_id": 151643,
        "eos_token_id": 151645, "head_dim": 128, "hidden_act": "silu", "hidden_size": 4096, "intermediate_size": 12288,
        "max_position_embeddings": 40960, "max_window_layers": 36, "model_type": "qwen3", "num_attention_heads": 32,
        "num_hidden_layers": 36, "num_key_value_heads": 8, "rms_norm_eps": 1e-06, "rope_scaling": None,
        "rope_theta": 1000000, "sliding_window": None, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
        "use_sliding_window": False, "vocab_size": 151936}))
    assert cfg.q_size == 4096 and cfg.kv_size == 1024 and cfg.eos_token_id == (151645,) and cfg.bos_token_id == 151643


@pytest.mark.parametrize("patch,word", [
    ({"architectures": ["LlamaForCausalLM"]}, "not built"),
    ({"architectures": []}, "architectures"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"use_sliding_window": True}, "use_sliding_window"),
    ({"hidden_size": "64"}, "integer"),
    ({"num_hidden_layers": 0}, ">= 1"),
    ({"rms_norm_eps": -1.0}, "> 0"),
    ({"eos_token_id": 999}, "vocabulary"),
    ({"attention_bias": True}, "biases"),
])
def test_named_errors(tmp_path, patch, word):
    cfg = {**tiny_config("A").to_dict(), **patch}
    with pytest.raises(ConfigError) as err:
        load_config(write(tmp_path, cfg))
    assert word in str(err.value)


def test_missing_file(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_another_architecture_registers_without_touching_the_package(tmp_path):
    class ToyConfig:
        @classmethod
        def from_dict(cls, cfg):
            self = cls()
            self.width = cfg["width"]
            return self

    register_architecture("ToyForTests", ToyConfig, lambda c: None)
    try:
        cfg = load_config(write(tmp_path, {"architectures": ["ToyForTests"], "width": 7}))
        assert cfg.width == 7
    finally:
        REGISTRY.pop("ToyForTests")


def test_generation_config_adds_its_end_of_sequence_ids(tmp_path):
    """generation_config.json beside config.json: its eos ids join config.json's (int or list in either file)."""
    import json
    from acvram_b200.config import load_config
    base = {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 300, "hidden_size": 64, "intermediate_size": 128,
            "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "eos_token_id": 45}
    (tmp_path / "config.json").write_text(json.dumps(base))
    assert load_config(tmp_path).eos_token_id == (45,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [45, 43], "temperature": 0.6}))
    assert load_config(tmp_path).eos_token_id == (43, 45)
    assert load_config(tmp_path / "config.json").eos_token_id == (43, 45)
    (tmp_path / "generation_config.json").write_text("{ not json")
    assert load_config(tmp_path).eos_token_id == (45,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 299}))
    assert load_config(tmp_path).eos_token_id == (45, 299)
