"""Checkpoint tensor names of LlamaForCausalLM and where each goes.

The names are the ones the reference's module tree reproduces
(mstar/model/orpheus/components/language_model.py:61-70, 89-101) and the
packing is its stacked-parameter table: q/k/v_proj -> qkv_proj shards q, k, v;
gate/up_proj -> gate_up_proj shards 0, 1 (mstar/model/loader/base.py:159-165).
Names containing "rotary_emb" are skipped as there (base.py:151-153).

Unlike the reference, whose loader ignores unknown keys and never notices a
missing parameter (base.py:136-145), the loader that consumes this map reports
both; and a tied LM head, which the reference leaves uninitialised, is an alias
of the embedding table.
"""
from __future__ import annotations

from ..config.layout import ModelLayout
from .names import CheckpointMap, TensorSource


def llama_checkpoint_map(config, layout: ModelLayout) -> CheckpointMap:
    sources: list[TensorSource] = []
    vocab = layout.vocab_size
    sources.append(TensorSource("model.embed_tokens.weight", "embed.weight", 0, vocab))
    for i, block in enumerate(layout.blocks):
        attn, ffn = block.mixer, block.ffn
        q_rows = attn.num_heads * attn.head_dim
        kv_rows = attn.num_kv_heads * attn.head_dim
        hf = f"model.layers.{i}"
        me = f"blocks.{i}"
        sources.append(TensorSource(f"{hf}.self_attn.q_proj.weight", f"{me}.mixer.qkv.weight",
                                    0, q_rows))
        sources.append(TensorSource(f"{hf}.self_attn.k_proj.weight", f"{me}.mixer.qkv.weight",
                                    q_rows, kv_rows))
        sources.append(TensorSource(f"{hf}.self_attn.v_proj.weight", f"{me}.mixer.qkv.weight",
                                    q_rows + kv_rows, kv_rows))
        sources.append(TensorSource(f"{hf}.self_attn.o_proj.weight", f"{me}.mixer.o.weight",
                                    0, attn.hidden_size))
        inter = ffn.intermediate_size
        sources.append(TensorSource(f"{hf}.mlp.gate_proj.weight", f"{me}.ffn.gate_up.weight",
                                    0, inter))
        sources.append(TensorSource(f"{hf}.mlp.up_proj.weight", f"{me}.ffn.gate_up.weight",
                                    inter, inter))
        sources.append(TensorSource(f"{hf}.mlp.down_proj.weight", f"{me}.ffn.down.weight",
                                    0, ffn.hidden_size))
        sources.append(TensorSource(f"{hf}.input_layernorm.weight", f"{me}.norm1.weight",
                                    0, block.norm1.size))
        sources.append(TensorSource(f"{hf}.post_attention_layernorm.weight",
                                    f"{me}.norm2.weight", 0, block.norm2.size))
    sources.append(TensorSource("model.norm.weight", "final_norm.weight", 0,
                                layout.final_norm.size))
    sources.append(TensorSource("lm_head.weight", "head.weight", 0, vocab))
    tied = bool(layout.tie_word_embeddings)
    return CheckpointMap(
        sources=sources,
        aliases={"head.weight": "embed.weight"} if tied else {},
        optional=frozenset({"lm_head.weight"}) if tied else frozenset(),
        ignore=lambda name: "rotary_emb" in name,
    )
