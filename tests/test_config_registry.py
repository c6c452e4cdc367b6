"""Configuration, architecture registry and model names (no GPU)."""

import json

import pytest

from tests.tiny_configs import TINY_A, TINY_B, TINY_C
from tokensprint_b200.config import registry
from tokensprint_b200.config.engine_config import Config, SamplingParams, canonical_dtype
from tokensprint_b200.config.model_config import ConfigError
from tokensprint_b200.models.qwen3 import Qwen3Config


def test_config_reads_every_size_from_its_keys():
    for d in (TINY_A, TINY_B, TINY_C):
        c = Qwen3Config.from_dict(d)
        assert c.hidden_size == d["hidden_size"] and c.head_dim == d["head_dim"]
        assert c.num_attention_heads == d["num_attention_heads"]
        assert c.num_key_value_heads == d["num_key_value_heads"]
        assert c.intermediate_size == d["intermediate_size"] and c.vocab_size == d["vocab_size"]
        assert c.rope_theta == d["rope_theta"] and c.rms_norm_eps == d["rms_norm_eps"]
        assert c.tie_word_embeddings == d["tie_word_embeddings"]
        assert len(c.layer_types) == d["num_hidden_layers"]
    c = Qwen3Config.from_dict(TINY_C)
    assert c.sliding_window == 24
    assert c.layer_types == ("full_attention", "sliding_attention", "sliding_attention", "full_attention")


def test_config_defaults_follow_the_reference_preset():
    d = {"vocab_size": 10, "hidden_size": 32, "num_hidden_layers": 1, "num_attention_heads": 4, "intermediate_size": 8}
    c = Qwen3Config.from_dict(d)
    assert c.head_dim == 8 and c.num_key_value_heads == 4
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-6 and not c.tie_word_embeddings
    assert c.sliding_window is None


def test_config_window_layers_from_max_window_layers():
    d = dict(TINY_A, use_sliding_window=True, sliding_window=8, max_window_layers=1)
    c = Qwen3Config.from_dict(d)
    assert c.layer_types == ("full_attention", "sliding_attention")
    # a window that no layer uses is dropped
    assert Qwen3Config.from_dict(dict(TINY_A, sliding_window=8, use_sliding_window=False)).sliding_window is None


@pytest.mark.parametrize(
    "change, word",
    [
        ({"hidden_act": "gelu"}, "hidden_act"),
        ({"attention_bias": True}, "attention_bias"),
        ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
        ({"num_key_value_heads": 3}, "num_key_value_heads"),
        ({"head_dim": 15}, "head_dim"),
        ({"vocab_size": None}, "vocab_size"),
        ({"layer_types": ["full_attention"]}, "layer_types"),
        ({"layer_types": ["full_attention", "sliding_attention"]}, "sliding_window"),
    ],
)
def test_config_rejects_what_the_engine_cannot_run(change, word):
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(dict(TINY_A, **change))


def test_config_round_trip(tmp_path):
    c = Qwen3Config.from_dict(TINY_C)
    c.save(tmp_path)
    assert Qwen3Config.from_json(tmp_path) == c
    arch, c2 = registry.load_model_config(tmp_path)
    assert arch.name == "Qwen3ForCausalLM" and c2 == c


def test_architecture_is_chosen_by_config_json():
    assert registry.architecture_for({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    assert registry.architecture_for({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(ValueError, match="Unsupported architecture"):
        registry.architecture_for({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_model_names_resolve_short_and_repo_id():
    assert registry.resolve_model_name("qwen3-0.6b") == "qwen3-0.6b"
    assert registry.resolve_model_name("qwen/qwen3-0.6b") == "qwen3-0.6b"
    assert registry.get_model_repo_id("qwen3-8b") == "qwen/qwen3-8b"
    assert registry.model_is_registered("qwen/qwen3-8b") and registry.model_is_registered("qwen3-32b")
    assert not registry.model_is_registered("meta-llama/qwen3-8b")
    assert not registry.model_is_registered("qwen3-9b")
    with pytest.raises(ValueError, match="Unsupported model_name 'llama-3-8b'. Available models:"):
        registry.resolve_model_name("llama-3-8b")
    assert registry.get_model_family("qwen3-14b") == "qwen"
    assert str(registry.get_local_model_dir("qwen/qwen3-8b", cache_dir="x")) == "x/qwen3-8b"


def test_presets_hold_the_published_sizes():
    c = registry.get_model_config("qwen3-0.6b")  # engine/models/qwen/_archs.py:92-125
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (1024, 16, 8, 128)
    assert (c.intermediate_size, c.vocab_size, c.num_hidden_layers) == (3072, 151936, 28)
    assert c.tie_word_embeddings and c.max_position_embeddings == 40960 and c.rope_theta == 1e6
    c = registry.get_model_config("qwen/qwen3-8b")
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.intermediate_size) == (36, 4096, 32, 12288)
    assert not c.tie_word_embeddings


def test_duplicate_registration_is_refused():
    with pytest.raises(ValueError, match="already registered"):
        registry.register_architecture("Qwen3ForCausalLM", config_from_dict=dict)(lambda c: None)
    with pytest.raises(ValueError, match="already registered"):
        registry.register_preset("qwen", "qwen3-8b", registry.PRESET_DIR / "qwen3-8b.json")


def test_listing_script():
    import model_registry

    out = model_registry.listing()
    assert out.startswith("Registered models:\n\nqwen:\n")
    assert "  - qwen3-0.6b (qwen/qwen3-0.6b)" in out
    for name in ("qwen3-1.7b", "qwen3-4b", "qwen3-8b", "qwen3-14b", "qwen3-32b"):
        assert f"  - {name} (qwen/{name})" in out
    assert registry.get_models_from_family("qwen", newest_first=False)[0] == "qwen3-0.6b"
    assert registry.get_models_from_family("nobody") == []


def test_engine_config_and_sampling_params(tmp_path):
    c = Config(model=str(tmp_path))
    assert c.kvcache_block_size == 16 and c.dtype == "bfloat16" and c.max_model_len == 4096
    assert Config(model=str(tmp_path), dtype="fp32").dtype == "float32"
    with pytest.raises(FileNotFoundError):
        Config(model=str(tmp_path / "nope"))
    with pytest.raises(ValueError):
        Config(model=str(tmp_path), kvcache_block_size=0)
    assert SamplingParams(temperature=0.0).greedy and not SamplingParams(temperature=0.8).greedy
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)
    assert canonical_dtype("torch.bfloat16") == "bfloat16"
    with pytest.raises(ValueError):
        canonical_dtype("float16")
