"""Typed configuration, registry and layout (CPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from mstar_b200.config.base import ConfigError
from mstar_b200.config.layout import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelLayout,
                                      NormSpec, RunEntry)
from mstar_b200.config.llama import LlamaConfig
from mstar_b200.config.registry import (config_from_dict, get_architecture,
                                        known_architectures, load_config)

ORPHEUS = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=28, num_attention_heads=24,
    num_key_value_heads=8, hidden_size=3072, head_dim=128, intermediate_size=8192,
    max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0, vocab_size=156940,
    rope_scaling={"factor": 32.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                  "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    tie_word_embeddings=True, eos_token_id=128258,
)


def test_every_size_comes_from_config_json():
    for raw in (TINY_A, TINY_B, ORPHEUS):
        cfg = config_from_dict(raw)
        assert isinstance(cfg, LlamaConfig)
        layout = cfg.layout()
        assert len(layout.blocks) == raw["num_hidden_layers"] == len(layout.order)
        attn = layout.blocks[0].mixer
        assert (attn.num_heads, attn.num_kv_heads, attn.head_dim) == (
            raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"])
        assert attn.position.theta == raw["rope_theta"]
        assert layout.blocks[0].ffn.intermediate_size == raw["intermediate_size"]
        assert layout.blocks[0].norm1.eps == raw["rms_norm_eps"] == layout.final_norm.eps
        assert layout.vocab_size == raw["vocab_size"]
        assert layout.tie_word_embeddings == raw["tie_word_embeddings"]
        scaling = attn.position.scaling
        if raw.get("rope_scaling"):
            assert scaling.factor == raw["rope_scaling"]["factor"]
            assert scaling.original_max_position_embeddings == raw["rope_scaling"][
                "original_max_position_embeddings"]
        else:
            assert scaling is None


def test_defaults_that_config_json_may_omit():
    raw = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "num_key_value_heads")}
    cfg = config_from_dict(raw)
    assert cfg.head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    assert cfg.num_key_value_heads == raw["num_attention_heads"]


def test_missing_keys_are_listed_together():
    raw = {k: v for k, v in TINY_A.items() if k not in ("rms_norm_eps", "vocab_size",
                                                        "rope_theta")}
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    for key in ("rms_norm_eps", "vocab_size", "rope_theta"):
        assert key in str(err.value)


@pytest.mark.parametrize("patch,word", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"), ({"num_key_value_heads": 3}, "multiple"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"), ({"hidden_size": "64"}, "integer"),
])
def test_unusable_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict({**TINY_A, **patch})


def test_registry_is_keyed_by_architecture_name(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    assert get_architecture("LlamaForCausalLM").config_cls is LlamaConfig
    with pytest.raises(KeyError, match="LlamaForCausalLM"):
        get_architecture("NoSuchModel")
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(tmp_path).to_dict()["intermediate_size"] == 160
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nowhere")


def test_stop_tokens_and_round_trip():
    cfg = config_from_dict(ORPHEUS)
    assert cfg.stop_token_ids() == (128258,)
    assert config_from_dict({**TINY_A, "eos_token_id": [1, 2]}).stop_token_ids() == (1, 2)
    again = config_from_dict(cfg.to_dict())
    assert again == cfg


def test_run_order_is_data_and_is_checked():
    norm = NormSpec(size=8, eps=1e-5)
    own = AttentionSpec(hidden_size=8, num_heads=2, num_kv_heads=1, head_dim=16)
    shared = AttentionSpec(hidden_size=8, num_heads=2, num_kv_heads=1, head_dim=16,
                           shares_kv=True)
    ffn = GatedMLPSpec(hidden_size=8, intermediate_size=16)
    b_own = BlockSpec("prenorm", own, ffn, norm, norm)
    b_shared = BlockSpec("prenorm", shared, ffn, norm, norm)

    def layout(order):
        return ModelLayout(vocab_size=10, hidden_size=8, blocks=[b_own, b_shared],
                           order=order, final_norm=norm)

    # a block named twice (each run with a cache of its own), and a block that reads
    # the cache another run wrote
    ok = layout([RunEntry(0, 0), RunEntry(1, 0), RunEntry(0, 1)])
    ok.validate()
    assert ok.num_caches() == 2
    with pytest.raises(ValueError, match="before any earlier"):
        layout([RunEntry(1, 0), RunEntry(0, 0)]).validate()
    with pytest.raises(ValueError, match="written by"):
        layout([RunEntry(0, 0), RunEntry(0, 0)]).validate()
    with pytest.raises(ValueError, match="names block"):
        layout([RunEntry(2, 0)]).validate()
