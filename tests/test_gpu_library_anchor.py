"""The formulas that the reference never writes down, pinned on the calls it makes.

The reference hands the llama3 frequency rule and the RMSNorm arithmetic to a library:
``flashinfer.rope.apply_llama31_rope_pos_ids_inplace(q, k, pos_ids, rotary_dim=None,
interleave=False, rope_scale=factor, rope_theta=theta, low_freq_factor=..,
high_freq_factor=.., old_context_len=..)`` (mstar/engine/cache_manager.py:734-759, with the
parameters of mstar/model/components/distributed/attention.py:122-136 and the values of
mstar/model/orpheus/config.py:15-23) and ``flashinfer.norm.rmsnorm(input, weight, eps)``
(mstar/utils/flashinfer_utils.py:25-50).  These tests make the same calls with the same
arguments on the GPU and compare the results with the plain implementation's functions
(``plain_rope_frequencies`` + ``plain_apply_rope``, ``plain_rms_norm``), which are what
every other test compares the engine with.  The library is an oracle here and nothing
else: no product code path calls it.  If the package cannot be imported, or cannot
build or load its kernels on this machine, the tests are skipped with the error text.
"""
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

ORPHEUS = dict(head_dim=128, hidden_size=3072, num_attention_heads=24, rope_theta=500000.0,
               rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                             "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192})
# tiny-B's scaling parameters (a 32-token original context, so that all three bands lie
# within short sequences) at a head size of 64, the smallest the library takes
TINY_B = dict(head_dim=64, hidden_size=192, num_attention_heads=3, rope_theta=500000.0,
              rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                            "high_freq_factor": 4.0, "original_max_position_embeddings": 32})


def library():
    flashinfer = pytest.importorskip("flashinfer")
    return flashinfer


def call_or_skip(fn, *args, **kwargs):
    try:
        return fn(*args, **kwargs)
    except Exception as exc:                     # no compiler, no cache folder, wrong arch ...
        pytest.skip(f"the library call is not usable here: {type(exc).__name__}: {exc}"[:400])


@pytest.mark.parametrize("cfg,positions", [
    # every band of the rule at positions where a wrong frequency turns the pair visibly:
    # the smoothed band's frequencies are 7.7e-4 .. 3.1e-3 (Orpheus), so 10 % off is 2 rad
    # at position 8,000
    (ORPHEUS, [0, 1, 2, 17, 100, 1000, 2047, 4097, 8000, 8191]),
    (TINY_B, [0, 1, 2, 5, 17, 31, 32, 33, 100, 257]),
], ids=["orpheus", "tiny_b"])
def test_llama3_rope_as_the_reference_calls_it(cfg, positions):
    flashinfer = library()
    hd, heads, kv_heads = cfg["head_dim"], 4, 2
    g = torch.Generator().manual_seed(3)
    n = len(positions)
    q = torch.randn(n, heads, hd, generator=g).to(torch.bfloat16)      # bf16 values, exactly
    k = torch.randn(n, kv_heads, hd, generator=g).to(torch.bfloat16)
    rs = cfg["rope_scaling"]
    q_dev, k_dev = q.cuda().contiguous(), k.cuda().contiguous()
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    call_or_skip(flashinfer.rope.apply_llama31_rope_pos_ids_inplace, q_dev, k_dev, pos,
                 rotary_dim=None, interleave=False, rope_scale=rs["factor"],
                 rope_theta=cfg["rope_theta"], low_freq_factor=rs["low_freq_factor"],
                 high_freq_factor=rs["high_freq_factor"],
                 old_context_len=rs["original_max_position_embeddings"])
    inv_freq = P.plain_rope_frequencies(cfg)
    posl = torch.tensor(positions)
    for name, x, got in (("q", q, q_dev), ("k", k, k_dev)):
        want = P.plain_apply_rope(x, posl, inv_freq)
        err = (got.cpu().double() - want).abs()
        # two bfloat16 units in the last place of the rotated pair's length
        half = hd // 2
        length = torch.sqrt(x[..., :half].double() ** 2 + x[..., half:].double() ** 2)
        tol = 2.0 ** -7 * torch.cat([length, length], dim=-1) + 1e-6
        bad = (err > tol).nonzero()
        assert bad.numel() == 0, (f"{name}: {bad.shape[0]} elements off, first at token "
                                  f"{bad[0].tolist()} (position {positions[bad[0][0]]}, "
                                  f"frequency index {int(bad[0][2]) % half}): "
                                  f"{err[tuple(bad[0])].item():.4f}")


@pytest.mark.parametrize("hidden,eps", [(3072, 1e-5), (96, 1e-6)])
def test_rmsnorm_as_the_reference_calls_it(hidden, eps):
    flashinfer = library()
    g = torch.Generator().manual_seed(5)
    x = (3.0 * torch.randn(9, hidden, generator=g)).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    got = call_or_skip(flashinfer.norm.rmsnorm, x.cuda(), w.cuda(), eps=eps)
    want = P.plain_rms_norm(x, w, eps)
    err = (got.cpu().double() - want).abs()
    assert (err <= 2.0 ** -8 * want.abs() + 1e-6).all(), err.max().item()   # one bf16 ulp
