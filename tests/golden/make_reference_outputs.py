"""Run t-avil/mstar's own Orpheus language-model code once on the CPU, on a tiny random
model, and store its logits beside the weights' seed so that tests can compare the
plain implementation (tests/plain_llama.py) with it.

    python tests/golden/make_reference_outputs.py /path/to/reference/checkout

What the reference's own code contributes: the module tree and its parameter names,
the fused qkv / gate_up layouts and split order, the loader's renaming of q/k/v_proj
and gate/up_proj, the pre-norm wiring of the decoder layer, the final norm and the
separate LM head.  What it cannot contribute on a CPU: RMSNorm, rotary encoding and
attention are library (FlashInfer) calls that need a GPU driver, so this script
supplies them through the reference's own seams -- ``run_rms_norm`` is replaced and a
stub cache handle provides ``apply_rope`` / ``run_attention`` -- with the plain
functions.  Those three therefore rest on the formulas cited in plain_llama.py, not
on this comparison.  The reference has no code for tied embeddings, so the golden
model is untied.

Output: tests/golden/reference_tiny.pt  {config, seed, token_ids, logits (float32)}.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

from plain_llama import plain_apply_rope, plain_attention, plain_rms_norm, plain_rope_frequencies  # noqa: E402

CFG = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=3, num_attention_heads=6,
    num_key_value_heads=2, hidden_size=96, head_dim=16, intermediate_size=176,
    max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=500000.0, vocab_size=320,
    rope_scaling={"factor": 8.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                  "original_max_position_embeddings": 32, "rope_type": "llama3"},
    tie_word_embeddings=False,
)
SEED = 20240607
TOKENS = [3, 17, 250, 9, 9, 41, 300, 7, 128, 64, 2, 319, 0, 77, 5, 190, 33, 33, 270, 11, 6,
          201, 154, 88, 13, 240, 99, 1, 45, 310, 222, 8, 19, 160, 75, 280, 52, 147, 4, 60]


def golden_weights(cfg: dict, seed: int) -> dict:
    """Checkpoint-named random tensors, float32 values that are exact in bfloat16."""
    g = torch.Generator().manual_seed(seed)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(*shape):
        return (0.05 * torch.randn(*shape, generator=g)).to(torch.bfloat16).float()

    def vec(n):
        return (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).float()

    w = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": vec(H),
         "lm_head.weight": mat(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[f"{p}.self_attn.q_proj.weight"] = mat(nh * hd, H)
        w[f"{p}.self_attn.k_proj.weight"] = mat(nkv * hd, H)
        w[f"{p}.self_attn.v_proj.weight"] = mat(nkv * hd, H)
        w[f"{p}.self_attn.o_proj.weight"] = mat(H, nh * hd)
        w[f"{p}.mlp.gate_proj.weight"] = mat(I, H)
        w[f"{p}.mlp.up_proj.weight"] = mat(I, H)
        w[f"{p}.mlp.down_proj.weight"] = mat(H, I)
        w[f"{p}.input_layernorm.weight"] = vec(H)
        w[f"{p}.post_attention_layernorm.weight"] = vec(H)
    return w


class StubCacheHandle:
    """Stands where the reference's BatchedCacheManager stands: whole sequence, no pages."""

    def __init__(self, cfg, num_tokens):
        self.positions = torch.arange(num_tokens)
        self.inv_freq = plain_rope_frequencies(cfg)

    def set_layer_idx(self, idx):
        pass

    def apply_rope(self, q, k, **kwargs):
        return (plain_apply_rope(q, self.positions, self.inv_freq).float(),
                plain_apply_rope(k, self.positions, self.inv_freq).float())

    def run_attention(self, q, k, v):
        return plain_attention(q, k, v).float()

    def advance_seq_lens(self):
        pass


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    import mstar.model.components.norm as ref_norm
    from mstar.distributed.communication import TPCommGroup
    from mstar.model.orpheus.components.language_model import OrpheusForCausalLM
    from mstar.model.orpheus.config import OrpheusModelConfig

    ref_norm.run_rms_norm = lambda x, w, eps: plain_rms_norm(x, w, eps).to(x.dtype)

    fields = {k: v for k, v in CFG.items()
              if k in OrpheusModelConfig.__dataclass_fields__}
    ref_cfg = OrpheusModelConfig(**fields)
    model = OrpheusForCausalLM(ref_cfg, TPCommGroup.trivial()).float()
    weights = golden_weights(CFG, SEED)
    loaded = model.load_weights(iter(weights.items()))
    expected = {n for n, _ in model.named_parameters()}
    assert loaded == expected, f"reference loader left parameters unset: {expected - loaded}"

    ids = torch.tensor(TOKENS, dtype=torch.long)
    with torch.no_grad():
        emb = model.model.embed_tokens(ids)
        hidden = model(query_sequence=emb, cache_handle=StubCacheHandle(CFG, ids.numel()))
        logits = model.lm_head(hidden)
    torch.save({"config": CFG, "seed": SEED, "token_ids": TOKENS,
                "logits": logits.float().contiguous()}, HERE / "reference_tiny.pt")
    print("wrote", HERE / "reference_tiny.pt", tuple(logits.shape))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
