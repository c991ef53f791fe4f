"""Shared fixtures: the two tiny Llama configurations, random model folders, and the
``gpu`` marker for tests that need a B200."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# Two configurations that differ in every size and option: layers, width, heads and
# groups (GQA of 2 vs one kv head for 3 query heads), head size, intermediate size
# (160 is no multiple of 64), vocabulary, tied / untied head, theta, no scaling / llama3
# scaling with a 32-token original context (all three frequency bands occur), eps.
TINY_A = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=64,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
    vocab_size=256, tie_word_embeddings=True, rope_theta=10000.0, rope_scaling=None,
    rms_norm_eps=1e-5, max_position_embeddings=2048, hidden_act="silu",
)
TINY_B = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=3, hidden_size=96,
    num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=160,
    vocab_size=512, tie_word_embeddings=False, rope_theta=500000.0,
    rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                  "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
    rms_norm_eps=1e-6, max_position_embeddings=4096, hidden_act="silu",
)
TINY = {"tiny_a": (TINY_A, dict(seed=11, norm_noise=0.0)),
        "tiny_b": (TINY_B, dict(seed=23, norm_noise=0.1))}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> (folder, raw config, checkpoint tensors) for the two tiny models, written
    through the framework's random-weights mode into a temporary folder."""
    from mstar_b200.config.registry import config_from_dict
    from mstar_b200.weights.random_init import random_checkpoint, write_model_folder
    import torch

    out = {}
    for name, (raw, opts) in TINY.items():
        folder = tmp_path_factory.mktemp(name)
        cfg = config_from_dict(raw)
        # std 0.05 instead of 0.02: tiny widths need larger weights for logits that
        # differ visibly between tokens
        kwargs = dict(std=0.05, norm_noise=opts["norm_noise"], vector_dtype=torch.float32)
        tensors = random_checkpoint(cfg, opts["seed"], **kwargs)
        # sharper attention than N(0, 0.05) projections give: with near-uniform
        # attention weights a wrong or missing key would barely move the logits.  Not
        # sharper than x3: at x6 the model amplifies rounding so much that the plain
        # model run in float32 instead of float64 already differs by 8e-5.
        for key in tensors:
            if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
                tensors[key] = (tensors[key].float() * 3.0).to(torch.bfloat16)
        write_model_folder(folder, cfg, opts["seed"], tensors=tensors)
        out[name] = (folder, raw, tensors)
    return out
