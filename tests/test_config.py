"""Configuration: keys, defaults, validation, registry."""
import json

import pytest

from allpaca_b200.config import ConfigError, EngineConfig, LlamaConfig
from allpaca_b200.config.presets import preset_config, preset_names
from allpaca_b200.models import known_architectures, load_config, resolve
from helpers import TINY_A, TINY_B


def test_defaults_follow_the_reference():
    cfg = LlamaConfig.from_dict({})
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads) == (32, 32, 1, 4)
    assert cfg.num_key_value_heads == 4          # defaults to the number of heads
    assert cfg.head_dim == 8                      # hidden / heads
    assert cfg.intermediate_size == 128           # 4 * hidden
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0
    assert cfg.rope_scaling is None and cfg.tie_word_embeddings is False


def test_every_size_comes_from_the_keys():
    a, b = LlamaConfig.from_dict(TINY_A), LlamaConfig.from_dict(TINY_B)
    assert (a.q_size, a.kv_size) == (64, 32)
    assert (b.q_size, b.kv_size) == (96, 32)
    assert b.rope_scaling.factor == 8.0 and b.rope_scaling.original_max_position_embeddings == 64
    assert b.tie_word_embeddings and not a.tie_word_embeddings
    assert a.to_dict()["intermediate_size"] == 176


def test_head_dim_may_differ_from_hidden_over_heads():
    cfg = LlamaConfig.from_dict({"hidden_size": 100, "num_attention_heads": 3, "head_dim": 16})
    assert cfg.q_size == 48


@pytest.mark.parametrize("bad, word", [
    ({"hidden_size": 100, "num_attention_heads": 3}, "divisible"),
    ({"num_attention_heads": 4, "num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 7}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_experts": 8}, "mixture"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "llama3"}}, "factor"),
    ({"vocab_size": 0}, "positive"),
    ({"vocab_size": 3.5}, "integer"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
])
def test_invalid_configs_are_named(bad, word):
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(bad)
    assert word in str(e.value)


def test_options_that_change_nothing_are_accepted():
    cfg = LlamaConfig.from_dict({"attention_bias": False, "mlp_bias": False, "rope_scaling": {"rope_type": "default"},
                                 "attention_dropout": 0.0, "bos_token_id": 1, "use_cache": True})
    assert cfg.rope_scaling is None


def test_registry_resolves_by_architecture_and_model_type(tmp_path):
    assert "LlamaForCausalLM" in known_architectures() and "llama" in known_architectures()
    assert resolve({"architectures": ["LlamaForCausalLM"]}).config_class is LlamaConfig
    assert resolve({"model_type": "llama"}).config_class is LlamaConfig
    with pytest.raises(ConfigError) as e:
        resolve({"architectures": ["MambaForCausalLM"], "model_type": "mamba"})
    assert "LlamaForCausalLM" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = load_config(str(tmp_path))
    spec = arch.spec_builder(cfg)
    assert len(spec.layers) == 3 and [r.layer for r in spec.order] == [0, 1, 2]
    assert spec.layers[0].params["mixer"].params["num_kv_heads"] == 1
    assert spec.layers[0].params["mixer_norm"].params["eps"] == 1e-6


def test_missing_or_broken_config_file(tmp_path):
    with pytest.raises(ConfigError):
        LlamaConfig.from_json_file(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        LlamaConfig.from_json_file(str(tmp_path))


def test_presets_parse():
    for n in preset_names():
        cfg = LlamaConfig.from_dict(preset_config(n))
        assert cfg.num_attention_heads % cfg.num_key_value_heads == 0
    big = LlamaConfig.from_dict(preset_config("llama-3.1-8b"))
    assert (big.hidden_size, big.intermediate_size, big.vocab_size) == (4096, 14336, 128256)


def test_engine_config_validation():
    EngineConfig(dtype="float32").validate()
    with pytest.raises(ConfigError):
        EngineConfig(dtype="float16").validate()
    with pytest.raises(ConfigError):
        EngineConfig(max_num_seqs=8, max_num_batched_tokens=4).validate()
    with pytest.raises(ConfigError):
        EngineConfig(page_size=0).validate()


def test_head_size_the_kernels_do_not_take_is_refused_when_the_model_is_described():
    """Multiples of 16 up to 256 are what the attention kernels are built for; any other head
    size is a configuration error before weights are read, not a build error at the first step."""
    from allpaca_b200.models import resolve
    for bad in (8, 24, 40, 272):
        raw = {"architectures": ["LlamaForCausalLM"], "hidden_size": 4 * bad, "num_attention_heads": 4,
               "head_dim": bad}
        arch = resolve(raw)
        cfg = arch.config_class.from_dict(raw)
        with pytest.raises(ConfigError, match="head_dim"):
            arch.spec_builder(cfg)
    raw = {"architectures": ["LlamaForCausalLM"], "hidden_size": 192, "num_attention_heads": 4, "head_dim": 48}
    arch = resolve(raw)
    assert arch.spec_builder(arch.config_class.from_dict(raw)).hidden_size == 192
