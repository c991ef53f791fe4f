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


# ---- pins that do not rest on plain_llama's own formulas: numbers worked out by hand from
# the llama3 rule as published (wavelength 2*pi/f; shorter than C/high: kept; longer than
# C/low: f/factor; between: s = (C/wavelength - low)/(high - low), (1-s)*f/factor + s*f).
# The same rule is compared with the library call that the reference makes in
# tests/test_gpu_library_anchor.py; here it is pinned without a GPU, for the plain
# implementation and for the product's table alike.
ORPHEUS_ROPE = dict(head_dim=128, hidden_size=3072, num_attention_heads=24, rope_theta=500000.0,
                    rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                  "high_freq_factor": 4.0,
                                  "original_max_position_embeddings": 8192})
# frequency index -> scaled inverse frequency (theta 5e5, head size 128, factor 32, C 8192).
# Index 32 by hand: f = 500000^(-1/2) = 1.4142136e-3, C*f/(2*pi) = 1.843862,
# s = 0.843862/3 = 0.281287, f' = f*(0.718713/32 + 0.281287) = 4.295568e-4.
ORPHEUS_FREQS = {0: 1.0, 1: 0.8146172338565447, 28: 0.003211445994752591,      # kept
                 29: 0.002118406996779608, 31: 0.0007625412033563571,          # smoothed
                 32: 0.00042955679655936815, 34: 9.70828780262767e-05,
                 35: 2.3890530884911708e-05, 63: 7.672314972286278e-08}        # divided by 32
TINY_B_ROPE = dict(head_dim=32, hidden_size=96, num_attention_heads=3, rope_theta=500000.0,
                   rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                 "high_freq_factor": 4.0, "original_max_position_embeddings": 32})
TINY_B_FREQS = {0: 1.0, 1: 0.2146673579985814, 2: 0.02424034309358572,
                15: 5.677088100759837e-07}


def test_llama3_frequencies_against_hand_computed_values():
    from mstar_b200.config.llama import LlamaConfig  # noqa: F401  (the product's table too)
    from mstar_b200.config.layout import PositionSpec, RopeScalingSpec
    from mstar_b200.parts.rope import rope_inverse_frequencies

    for cfg, pins in ((ORPHEUS_ROPE, ORPHEUS_FREQS), (TINY_B_ROPE, TINY_B_FREQS)):
        plain = P.plain_rope_frequencies(cfg)
        rs = cfg["rope_scaling"]
        spec = PositionSpec(kind="rope", head_dim=cfg["head_dim"], rotary_dim=cfg["head_dim"],
                            theta=cfg["rope_theta"], scaling=RopeScalingSpec(
                                rs["rope_type"], rs["factor"], rs["low_freq_factor"],
                                rs["high_freq_factor"], rs["original_max_position_embeddings"]))
        product = rope_inverse_frequencies(spec)
        for j, value in pins.items():
            assert abs(plain[j].item() / value - 1) < 1e-12, (j, plain[j].item(), value)
            assert abs(product[j] / value - 1) < 1e-12, (j, product[j], value)


def test_split_half_rotation_of_one_hand_rotated_vector():
    """Head size 4, theta 10000 (frequencies 1 and 0.01), position 3: the pairs are
    (x0, x2) and (x1, x3).  x = (1, 2, 3, 4):
    x0' = cos 3 - 3 sin 3, x2' = 3 cos 3 + sin 3; x1' = 2 cos .03 - 4 sin .03, x3' = 4 cos .03 + 2 sin .03."""
    cfg = dict(head_dim=4, hidden_size=4, num_attention_heads=1, rope_theta=10000.0)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=torch.float64)
    out = P.plain_apply_rope(x, torch.tensor([3]), P.plain_rope_frequencies(cfg))[0, 0]
    want = [-1.413352520780047, 1.8791180666879925, -2.828857481741469, 4.058191135400942]
    for got, w in zip(out.tolist(), want):
        assert abs(got - w) < 1e-6, (out.tolist(), want)      # float32 angle: 0.03 is rounded


def test_attention_of_three_tokens_by_explicit_softmax():
    """One head of size 2, no position encoding: token t sees keys 0..t, scores scaled by
    2^-0.5, weights by explicit exponentials."""
    import math

    q = torch.tensor([[[1.0, 0.0]], [[0.0, 2.0]], [[1.0, 1.0]]], dtype=torch.float64)
    k = torch.tensor([[[1.0, 1.0]], [[2.0, 0.0]], [[0.0, 3.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0, 10.0]], [[2.0, 20.0]], [[4.0, 40.0]]], dtype=torch.float64)
    out = P.plain_attention(q, k, v)[:, 0]
    s = 2 ** -0.5
    rows = [[1.0],                                             # token 0: its own key only
            [math.exp(2 * s), math.exp(0.0)],                  # q1.k0 = 2, q1.k1 = 0
            [math.exp(2 * s), math.exp(2 * s), math.exp(3 * s)]]
    for t, weights in enumerate(rows):
        z = sum(weights)
        want0 = sum(w * v[j, 0, 0].item() for j, w in enumerate(weights)) / z
        assert abs(out[t, 0].item() - want0) < 1e-12 and abs(out[t, 1].item() - 10 * want0) < 1e-11
