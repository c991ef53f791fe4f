"""The command line without a GPU: its options, the deployment file, the random-weights
mode (the reference's names: mstar/cli/main.py:138-167, docs/serving.rst:161-238)."""
import json

import pytest

from conftest import TINY_B
from mstar_b200.cli import main as cli


def test_generate_takes_the_reference_option_names():
    args = cli.build_parser().parse_args(
        ["generate", "/models/x", "--gpus", "0", "--config", "deploy.yaml", "--log-level", "DEBUG",
         "--log-stats", "--log-stats-file", "stats.txt", "--prompt-ids", "1,2,3", "--prompt-ids",
         "4, 5", "--temperature", "0.6", "--top-k", "0", "--top-p", "0.8", "--repetition-penalty",
         "1.3", "--ignore-eos", "--max-output-tokens", "7", "--seed", "3", "--page-size", "16",
         "--max-num-pages", "100", "--max-concurrent-requests", "8"])
    assert args.model == "/models/x" and args.gpus == "0" and args.config == "deploy.yaml"
    assert args.log_stats and args.log_stats_file == "stats.txt" and args.log_level == "DEBUG"
    assert (args.temperature, args.top_k, args.top_p, args.repetition_penalty) == (0.6, 0, 0.8, 1.3)
    assert cli._prompts(args) == [[1, 2, 3], [4, 5]]
    # what is not given stays None, so that the model folder's generation defaults apply
    bare = cli.build_parser().parse_args(["generate", "m", "--prompt-ids", "1"])
    assert bare.temperature is None and bare.top_p is None and bare.max_output_tokens is None
    with pytest.raises(SystemExit):
        cli.build_parser().parse_args(["serve", "orpheus"])        # not part of this engine


def test_prompt_file_and_deployment_file(tmp_path):
    prompts = tmp_path / "p.jsonl"
    prompts.write_text('[5, 6]\n\n{"prompt_token_ids": [7]}\n')
    args = cli.build_parser().parse_args(["generate", "m", "--prompt-file", str(prompts)])
    assert cli._prompts(args) == [[5, 6], [7]]
    with pytest.raises(SystemExit):
        cli._prompts(cli.build_parser().parse_args(["generate", "m"]))
    yml = tmp_path / "d.yaml"
    yml.write_text("max_concurrent_requests: 4\nautocast_dtype: float32\n"
                   "kv_cache:\n  page_size: 128\n  max_num_pages: 2048\n")
    d = cli._read_deployment(str(yml))
    assert d["max_concurrent_requests"] == 4 and d["kv_cache"] == {"page_size": 128,
                                                                   "max_num_pages": 2048}
    js = tmp_path / "d.json"
    js.write_text(json.dumps({"kv_cache": {"page_size": 16}}))
    assert cli._read_deployment(str(js))["kv_cache"]["page_size"] == 16
    assert cli._read_deployment(None) == {}
    with pytest.raises(SystemExit):
        cli._read_deployment(str(tmp_path / "missing.yaml"))


def test_random_model_writes_a_folder_that_loads_back(tmp_path, capsys):
    from mstar_b200.config.registry import load_config
    from safetensors import safe_open

    src = tmp_path / "config.json"
    src.write_text(json.dumps(TINY_B))
    out = tmp_path / "model"
    cli.main(["random-model", str(src), str(out), "--seed", "5", "--std", "0.05"])
    assert str(out) in capsys.readouterr().out
    cfg = load_config(out)
    assert cfg.hidden_size == TINY_B["hidden_size"] and cfg.num_hidden_layers == 3
    with safe_open(str(out / "model.safetensors"), framework="pt") as f:
        names = set(f.keys())
        assert "lm_head.weight" in names and "model.layers.2.mlp.up_proj.weight" in names
        assert tuple(f.get_tensor("model.embed_tokens.weight").shape) == (512, 96)
    # the same seed gives the same tensors
    out2 = tmp_path / "model2"
    cli.main(["random-model", str(src), str(out2), "--seed", "5", "--std", "0.05"])
    with safe_open(str(out / "model.safetensors"), framework="pt") as a, \
            safe_open(str(out2 / "model.safetensors"), framework="pt") as b:
        import torch

        assert torch.equal(a.get_tensor("model.norm.weight"), b.get_tensor("model.norm.weight"))
        assert torch.equal(a.get_tensor("lm_head.weight"), b.get_tensor("lm_head.weight"))
