"""Configuration and registry (no GPU)."""
import json

import pytest

from gogguf_b200.config import ConfigError, Qwen3Config, config_from_dict, load_config, registered_architectures
from gogguf_b200.engine.model import expected_tensors
from helpers import TINY_A, TINY_B, TINY_W


def test_registry_knows_qwen3_and_rejects_others():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert isinstance(config_from_dict(TINY_A), Qwen3Config)
    assert isinstance(config_from_dict({**TINY_A, "architectures": None, "model_type": "qwen3"}), Qwen3Config)
    with pytest.raises(ConfigError) as e:
        config_from_dict({**TINY_A, "architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert "LlamaForCausalLM" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        config_from_dict({k: v for k, v in TINY_A.items() if k not in ("architectures", "model_type")})


def test_values_come_from_the_keys():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 6, 1, 32)
    assert b.q_width == 192 != b.hidden_size          # q width decoupled from hidden (config.go:70-82)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.rope_theta == 10000.0 and b.rope_theta == 1e6
    assert a.rms_norm_eps == 1e-6 and b.rms_norm_eps == 1e-5


def test_defaults_of_the_reference():
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "rms_norm_eps", "rope_theta", "num_key_value_heads")}
    c = config_from_dict(d)
    assert c.head_dim == 64 // 4            # hidden/heads when absent (config.go:70-73)
    assert c.rms_norm_eps == 1e-6           # config.go:60-63
    assert c.rope_theta == 1e6              # config.go:65-68
    assert c.num_key_value_heads == 4


@pytest.mark.parametrize("patch,word", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["sliding_attention", "full_attention"]}, "sliding_window"),
    ({"vocab_size": "many"}, "vocab_size"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict({**TINY_A, **patch})
    assert word in str(e.value)


def test_round_trip_and_windows(tmp_path):
    c = config_from_dict(TINY_W)
    assert c.layer_types == ("sliding_attention", "full_attention", "full_attention", "sliding_attention")
    p = tmp_path / "config.json"
    p.write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c
    spec = c.to_spec()
    assert [b.mixer["window"] for b in spec.blocks] == [37, None, None, 37]
    # use_sliding_window + max_window_layers form
    c2 = config_from_dict({**TINY_A, "use_sliding_window": True, "sliding_window": 8, "max_window_layers": 1})
    assert c2.layer_types == ("full_attention", "sliding_attention")


def test_spec_lists_every_tensor():
    exp = expected_tensors(config_from_dict(TINY_B).to_spec())
    assert exp["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    assert exp["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert exp["model.layers.1.mlp.down_proj.weight"].shape == (96, 160)
    assert exp["lm_head.weight"].shape == (384, 96) and not exp["lm_head.weight"].optional
    assert len(exp) == 3 * 11 + 3
    tied = expected_tensors(config_from_dict(TINY_A).to_spec())
    assert tied["lm_head.weight"].optional


def test_missing_config_file(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_schedule_validation():
    from dataclasses import replace
    from gogguf_b200.config import ScheduleEntry
    spec = config_from_dict(TINY_A).to_spec()
    replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))).validate()
    with pytest.raises(ValueError):
        replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(5))).validate()
    with pytest.raises(ValueError):
        replace(spec, schedule=(ScheduleEntry(0, cache_of=0),)).validate()


def test_generation_config_adds_stop_ids(tmp_path):
    import json
    from gogguf_b200.config import load_config
    from helpers import TINY_A
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, eos_token_id=7)))
    assert load_config(str(tmp_path)).eos_token_ids == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [9, 7], "temperature": 0.6}))
    cfg = load_config(str(tmp_path))
    assert cfg.eos_token_ids == (7, 9) and cfg.to_spec().stop_token_ids == (7, 9)
    (tmp_path / "generation_config.json").write_text("{")
    with pytest.raises(Exception, match="not valid JSON"):
        load_config(str(tmp_path))
