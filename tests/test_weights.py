"""Weights by tensor name: packing, dtypes, tied head, and ONE error that lists every
missing tensor, unexpected tensor and wrong shape (CPU)."""
import json

import pytest
import torch
from safetensors.torch import save_file

from conftest import TINY_A, TINY_B
from mstar_b200.config.registry import config_from_dict, get_architecture
from mstar_b200.engine.model import model_param_specs
from mstar_b200.weights.loader import WeightsError, load_parameters
from mstar_b200.weights.random_init import random_checkpoint, write_model_folder


def load(raw, source, dtype=torch.float32):
    cfg = config_from_dict(raw)
    layout = cfg.layout()
    cmap = get_architecture(cfg.architecture).checkpoint_map(cfg, layout)
    return load_parameters(source, model_param_specs(layout), cmap, dtype, "cpu")


def test_random_folder_round_trip_and_packing(tmp_path):
    cfg = config_from_dict(TINY_B)
    write_model_folder(tmp_path, cfg, seed=3, std=0.05, norm_noise=0.1)
    assert json.loads((tmp_path / "config.json").read_text())["intermediate_size"] == 160
    tensors = random_checkpoint(cfg, seed=3, std=0.05, norm_noise=0.1)
    params = load(TINY_B, tmp_path)
    again = load(TINY_B, tensors)                     # same seed -> same weights, from memory
    for k in params:
        assert torch.equal(params[k], again[k]), k
    nq, nkv, inter = 3 * 32, 1 * 32, 160
    qkv = params["blocks.1.mixer.qkv.weight"]
    p = "model.layers.1"
    assert torch.equal(qkv[:nq], tensors[f"{p}.self_attn.q_proj.weight"].float())
    assert torch.equal(qkv[nq:nq + nkv], tensors[f"{p}.self_attn.k_proj.weight"].float())
    assert torch.equal(qkv[nq + nkv:], tensors[f"{p}.self_attn.v_proj.weight"].float())
    gu = params["blocks.2.ffn.gate_up.weight"]
    assert torch.equal(gu[:inter], tensors["model.layers.2.mlp.gate_proj.weight"].float())
    assert torch.equal(gu[inter:], tensors["model.layers.2.mlp.up_proj.weight"].float())
    assert params["head.weight"].data_ptr() != params["embed.weight"].data_ptr()
    # values are exact in bfloat16, so a bfloat16 load holds the same numbers
    bf = load(TINY_B, tmp_path, torch.bfloat16)
    assert bf["blocks.0.ffn.down.weight"].dtype == torch.bfloat16
    assert torch.equal(bf["blocks.0.ffn.down.weight"].float(), params["blocks.0.ffn.down.weight"])


def test_tied_head_is_an_alias(tmp_path):
    cfg = config_from_dict(TINY_A)
    tensors = random_checkpoint(cfg, seed=1)
    assert "lm_head.weight" not in tensors
    params = load(TINY_A, tensors)
    assert params["head.weight"].data_ptr() == params["embed.weight"].data_ptr()
    # a tied checkpoint that stores the head as well: accepted if equal, refused if not
    both = dict(tensors, **{"lm_head.weight": tensors["model.embed_tokens.weight"].clone()})
    loaded = load(TINY_A, both)
    assert loaded["head.weight"].data_ptr() == loaded["embed.weight"].data_ptr()
    both["lm_head.weight"] = both["lm_head.weight"] + 1
    with pytest.raises(WeightsError, match="differ"):
        load(TINY_A, both)
    # untied configuration: the head is required
    untied = {**TINY_A, "tie_word_embeddings": False}
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load(untied, tensors)


def test_dtype_rules(tmp_path):
    cfg = config_from_dict(TINY_A)
    tensors = random_checkpoint(cfg, seed=1, vector_dtype=torch.float32)
    bf = load(TINY_A, tensors, torch.bfloat16)
    assert bf["embed.weight"].dtype == torch.bfloat16
    assert bf["blocks.0.mixer.qkv.weight"].dtype == torch.bfloat16
    assert bf["blocks.0.norm1.weight"].dtype == torch.float32      # stored in 32-bit: stays so
    assert bf["final_norm.weight"].dtype == torch.float32
    f32 = load(TINY_A, tensors, torch.float32)
    assert all(t.dtype == torch.float32 for t in f32.values())
    # one float32 shard of a fused parameter keeps the whole parameter in 32-bit
    tensors["model.layers.0.self_attn.k_proj.weight"] = tensors[
        "model.layers.0.self_attn.k_proj.weight"].float()
    with pytest.warns(UserWarning, match="1 matrices .* stay float32 .*blocks.0.mixer.qkv.weight"):
        kept = load(TINY_A, tensors, torch.bfloat16)
    assert kept["blocks.0.mixer.qkv.weight"].dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY_B)
    tensors = random_checkpoint(cfg, seed=5)
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    tensors["something.else"] = torch.zeros(1)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(64, 96)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)   # ignored
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    with pytest.raises(WeightsError) as err:
        load(TINY_B, tmp_path)
    e = err.value
    assert e.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.7.mlp.up_proj.weight", "something.else"]
    assert [(n, tuple(g), tuple(w)) for n, g, w in e.wrong_shape] == [
        ("model.layers.1.self_attn.k_proj.weight", (64, 96), (32, 96))]
    text = str(e)
    for word in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (1)",
                 "checkpoint (64, 96), model (32, 96)"):
        assert word in text
    assert "rotary_emb" not in text


def test_sharded_checkpoint_and_missing_files(tmp_path):
    cfg = config_from_dict(TINY_A)
    tensors = {k: v.contiguous() for k, v in random_checkpoint(cfg, seed=2).items()}
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    weight_map = {k: ("model-00001-of-00002.safetensors" if i < half
                      else "model-00002-of-00002.safetensors") for i, k in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    params = load(TINY_A, tmp_path)
    assert torch.equal(params["final_norm.weight"], tensors["model.norm.weight"].float())
    with pytest.raises(FileNotFoundError):
        load(TINY_A, tmp_path / "empty")
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError, match="model.safetensors"):
        load(TINY_A, tmp_path / "empty")
