"""Typed configuration and the architecture registry."""

import json

import pytest

from oxr_inference_b200.config import ConfigError, EngineSettings, Qwen3Config, load_model_config, register_architecture, resolve_architecture
from oxr_inference_b200.config.registry import ARCHITECTURES, Architecture
from util import TINY_A, TINY_B


def test_reads_every_size_from_config_json():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (96, 160, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.group_size) == (6, 2, 32, 3)
    assert c.q_size == 192 and c.kv_size == 64 and c.q_size != c.hidden_size
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and c.vocab_size == 509
    assert not c.tie_word_embeddings and c.eos_token_ids == (507, 508)
    assert [c.window_of(i) for i in range(3)] == [0, 24, 0]


def test_head_dim_defaults_to_hidden_over_heads_and_tying_is_read():
    c = Qwen3Config.from_dict(TINY_A)
    assert c.head_dim == 16 and c.tie_word_embeddings and c.sliding_window is None
    assert c.layer_types == ("full_attention", "full_attention") and c.eos_token_ids == (255,)


def test_nested_llm_config_and_generation_config_eos():
    # the reference's wrapper nests the keys and prefers generation_config.json for eos (oxr_runtime/config.py:66-74)
    raw = {"architectures": ["Qwen3ForCausalLM"], "llm_config": {k: v for k, v in TINY_B.items() if k != "architectures"},
           "eos_token_id": 1}
    c = Qwen3Config.from_dict(raw, {"eos_token_id": [7, 9]})
    assert c.hidden_size == 96 and c.eos_token_ids == (7, 9)
    assert Qwen3Config.from_dict(raw, {}).eos_token_ids == (1,)


def test_max_window_layers_rule():
    raw = dict(TINY_B)
    del raw["layer_types"]
    raw["max_window_layers"] = 2
    assert Qwen3Config.from_dict(raw).layer_types == ("full_attention", "full_attention", "sliding_attention")
    raw["use_sliding_window"] = False
    assert Qwen3Config.from_dict(raw).sliding_window is None


@pytest.mark.parametrize("change,match", [
    ({"hidden_size": None}, "required"), ({"num_key_value_heads": 4}, "multiple"), ({"head_dim": 15}, "odd"),
    ({"attention_bias": True}, "attention_bias"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"), ({"layer_types": ["full_attention"]}, "entries"),
    ({"layer_types": ["full_attention", "linear_attention", "full_attention"]}, "unknown"), ({"vocab_size": 0}, "positive"),
])
def test_refuses_what_it_does_not_implement(change, match):
    raw = dict(TINY_B)
    for k, v in change.items():
        if v is None:
            del raw[k]
        else:
            raw[k] = v
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict(raw)


def test_round_trip_through_to_dict():
    for raw in (TINY_A, TINY_B):
        c = Qwen3Config.from_dict(raw)
        assert Qwen3Config.from_dict(c.to_dict()) == c


def test_registry_picks_the_model_by_architecture_name(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, cfg = load_model_config(tmp_path)
    assert arch.name == "Qwen3ForCausalLM" and isinstance(cfg, Qwen3Config)
    spec = arch.model_spec(cfg)
    assert len(spec.layers) == 2 and [e.layer for e in spec.schedule] == [0, 1]
    assert spec.layers[0].mixer.kind == "gqa_attention" and spec.layers[0].feed_forward.kind == "swiglu"
    assert spec.layers[1].mixer.prefix == "model.layers.1.self_attn." and spec.head.params["tied"] is True
    with pytest.raises(ConfigError, match="not registered.*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="no 'architectures'"):
        resolve_architecture({})


def test_registering_twice_is_refused_unless_replacing():
    arch = Architecture("ToyForTests", lambda raw, gen: raw, lambda cfg: None)
    try:
        register_architecture(arch)
        with pytest.raises(ValueError, match="already"):
            register_architecture(arch)
        register_architecture(arch, replace=True)
    finally:
        ARCHITECTURES.pop("ToyForTests", None)


def test_settings_validate():
    with pytest.raises(ValueError, match="dtype"):
        EngineSettings(dtype="float16")
    with pytest.raises(ValueError):
        EngineSettings(page_size=0)
    assert EngineSettings().cuda_graphs and EngineSettings().max_running == 256
