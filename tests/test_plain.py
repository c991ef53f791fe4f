"""The plain implementation against the reference's own model code (stored outputs of
tests/golden/make_reference_outputs.py) and against itself."""
from pathlib import Path

import torch

import plain_llama as P
from golden.make_reference_outputs import golden_weights

GOLDEN = Path(__file__).parent / "golden" / "reference_tiny.pt"


def test_plain_matches_reference_model_code():
    blob = torch.load(GOLDEN)
    w = golden_weights(blob["config"], blob["seed"])
    mine = P.plain_logits(w, blob["config"], blob["token_ids"])
    ref = blob["logits"].double()
    assert mine.shape == ref.shape
    # the reference ran in float32 through its own modules
    assert (mine - ref).abs().max().item() < 2e-5
    assert torch.equal(mine.argmax(-1), ref.argmax(-1))


def test_causality_of_plain_logits():
    blob = torch.load(GOLDEN)
    w = golden_weights(blob["config"], blob["seed"])
    ids = blob["token_ids"]
    full = P.plain_logits(w, blob["config"], ids)
    part = P.plain_logits(w, blob["config"], ids[:17])
    assert (full[:17] - part).abs().max().item() < 1e-10


def test_rope_frequency_bands():
    cfg = dict(head_dim=32, hidden_size=96, num_attention_heads=3, rope_theta=500000.0,
               rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                             "high_freq_factor": 4.0, "original_max_position_embeddings": 32})
    scaled = P.plain_rope_frequencies(cfg)
    plain = P.plain_rope_frequencies({**cfg, "rope_scaling": None})
    ratio = (scaled / plain)
    assert torch.isclose(ratio[0], torch.tensor(1.0, dtype=torch.float64))      # high band
    assert torch.isclose(ratio[-1], torch.tensor(1 / 8.0, dtype=torch.float64))  # low band
    assert ((ratio > 1 / 8.0 + 1e-9) & (ratio < 1 - 1e-9)).any()                 # smoothed


def test_rope_is_a_rotation_and_relative():
    cfg = dict(head_dim=16, hidden_size=64, num_attention_heads=4, rope_theta=10000.0)
    inv = P.plain_rope_frequencies(cfg)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 16, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, 16, generator=g, dtype=torch.float64)
    def dot(pq, pk):
        a = P.plain_apply_rope(q, torch.tensor([pq]), inv)
        b = P.plain_apply_rope(k, torch.tensor([pk]), inv)
        return (a * b).sum().item()
    assert abs(P.plain_apply_rope(q, torch.tensor([7]), inv).norm().item() - q.norm().item()) < 1e-9
    assert abs(dot(9, 4) - dot(25, 20)) < 1e-5


def test_window_mask_limits_keys():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(10, 2, 16, generator=g, dtype=torch.float64)
    k = torch.randn(10, 1, 16, generator=g, dtype=torch.float64)
    v = torch.randn(10, 1, 16, generator=g, dtype=torch.float64)
    full = P.plain_attention(q, k, v)
    win = P.plain_attention(q, k, v, window=4)
    assert torch.allclose(full[:4], win[:4])
    tail = P.plain_attention(q[6:], k[6:], v[6:])     # last 4 keys only, same rotation-free q
    assert torch.allclose(win[9], tail[3])


def test_philox_reference_vector():
    # Random123 known-answer test for philox4x32-10 with zero key and counter
    assert P.plain_philox4x32_10(0, 0) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]


def test_sampling_distribution_filters():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0])
    p = P.plain_sampling_distribution(logits, 1.0, top_k=2)
    assert (p > 0).tolist() == [True, False, False, False, True]
    p = P.plain_sampling_distribution(logits, 1.0, top_p=0.6)
    assert (p > 0).sum().item() == 1 or (p > 0).sum().item() == 2
    seen = torch.tensor([0, 0, 0, 0, 1])
    p = P.plain_sampling_distribution(logits, 1.0, penalty=100.0, seen=seen)
    assert p.argmax().item() == 0
