"""Configuration, specs and the architecture registry (no device needed)."""
import json
import os
import tempfile

import pytest

import tiny
from gopherllm_b200.config import (PhiConfig, load_config, resolve_architecture, ModelSpec, ScheduleEntry,
                                   default_schedule)
from gopherllm_b200.config.registry import architecture_from_config, known_architectures


@pytest.mark.parametrize("label", ["PhiForCausalLM", "phi", "Phi", "phi2", "PHI-2", "phi_2", "PhiModel",
                                   "phi-1_5", " phiforcausallm "])
def test_registry_spellings(label):
    # the reference maps "phi" to its phi2 graph and strips class-name suffixes (arch_detect.go:58-110)
    assert resolve_architecture(label).name == "phi"


@pytest.mark.parametrize("label", ["", "llama", "LlamaForCausalLM", "phi3", "ForCausalLM"])
def test_registry_rejects(label):
    assert resolve_architecture(label) is None


def test_unknown_architecture_error_lists_known():
    with pytest.raises(ValueError) as e:
        architecture_from_config({"architectures": ["MambaForCausalLM"], "model_type": "mamba"})
    assert "unsupported architecture" in str(e.value) and "phi" in str(e.value)
    assert "phi" in known_architectures()
    # model_type is the fallback when the class name is unknown
    assert architecture_from_config({"architectures": ["Whatever"], "model_type": "phi"}).name == "phi"


def test_config_from_json_keys():
    for name, (raw, _) in tiny.TINY.items():
        c = PhiConfig.from_dict(raw)
        spec = resolve_architecture("phi").build_spec(c)
        assert len(spec.layers) == raw["num_hidden_layers"] == len(spec.schedule)
        m = spec.layers[0].mixer
        assert m.num_heads == raw["num_attention_heads"]
        assert m.num_kv_heads == raw["num_key_value_heads"]
        assert m.head_dim == raw.get("head_dim", raw["hidden_size"] // raw["num_attention_heads"])
        assert m.position.rotary_dim == int(raw["partial_rotary_factor"] * m.head_dim)
        assert m.position.theta == raw["rope_theta"]
        assert spec.layers[0].norm.eps == raw["layer_norm_eps"]
        assert (m.qk_norm is not None) == raw["qk_layernorm"]
        assert spec.layers[0].ffn.intermediate == raw["intermediate_size"]
        assert spec.layers[0].ffn.activation == raw["hidden_act"]
        assert spec.tie_embeddings == raw["tie_word_embeddings"]
        assert spec.vocab == raw["vocab_size"] and spec.max_positions == raw["max_position_embeddings"]
        assert spec.stop_tokens == (raw["eos_token_id"],)
        assert spec.layers[0].arrangement == "parallel" and spec.layers[0].norm2 is None
        assert abs(m.q_scale - m.head_dim ** -0.5) < 1e-15
        assert PhiConfig.from_dict(c.to_dict()) == c


def test_config_defaults_and_phi2_sizes():
    c = PhiConfig.from_dict(dict(vocab_size=51200, hidden_size=2560, intermediate_size=10240,
                                 num_hidden_layers=32, num_attention_heads=32, partial_rotary_factor=0.4))
    assert (c.kv_heads, c.head_size, c.rotary_dim) == (32, 80, 32)
    assert c.layer_norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.hidden_act == "gelu_new"
    assert c.max_position_embeddings == 2048 and not c.qk_layernorm and not c.tie_word_embeddings


@pytest.mark.parametrize("change,needle", [
    (dict(num_attention_heads=0), "invalid model configuration"),
    (dict(hidden_size=65), "not divisible"),
    (dict(num_key_value_heads=3), "not a multiple"),
    (dict(partial_rotary_factor=0.45), "must be even"),
    (dict(partial_rotary_factor=1.5), "outside"),
    (dict(hidden_act="swish"), "unknown"),
    (dict(layer_norm_eps=0.0), "positive"),
    (dict(rope_scaling={"type": "yarn"}), "rope_scaling"),
])
def test_config_validation(change, needle):
    raw = dict(tiny.TINY_A)
    raw.update(change)
    with pytest.raises(ValueError) as e:
        PhiConfig.from_dict(raw)
    assert needle in str(e.value)


def test_missing_keys_are_named():
    with pytest.raises(ValueError) as e:
        PhiConfig.from_dict({"hidden_size": 8})
    assert "vocab_size" in str(e.value) and "num_hidden_layers" in str(e.value)


def test_load_config_from_folder():
    with tempfile.TemporaryDirectory() as d:
        with pytest.raises(FileNotFoundError):
            load_config(d)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(tiny.TINY_B, f)
        arch, cfg = load_config(d)
        assert arch.name == "phi" and isinstance(cfg, PhiConfig) and cfg.qk_layernorm


def test_schedule_is_data():
    spec = resolve_architecture("phi").build_spec(PhiConfig.from_dict(tiny.TINY_A))
    base = dict(hidden=spec.hidden, vocab=spec.vocab, max_positions=spec.max_positions,
                layers=spec.layers, final_norm=spec.final_norm)
    # a layer named twice, each run with a cache entry of its own
    s = ModelSpec(schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2)), **base)
    assert s.num_cache_entries == 3
    # a layer that reads the entry another run wrote
    s = ModelSpec(schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0, writes=False)), **base)
    assert s.num_cache_entries == 1
    with pytest.raises(ValueError):
        ModelSpec(schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 0)), **base)          # two writers
    with pytest.raises(ValueError):
        ModelSpec(schedule=(ScheduleEntry(0, 1, writes=False),), **base)                # nobody writes it
    with pytest.raises(ValueError):
        ModelSpec(schedule=(ScheduleEntry(5, 0),), **base)                              # no such layer
    assert default_schedule(3) == (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2))
