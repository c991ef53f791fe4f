"""The allocation-free decode attention entry point, called through its exported C
symbol, against the ordinary entry point.

Some callers of this library cannot obtain device memory at the time they need
attention: a process that is forbidden to allocate once it has started serving, a plugin
whose host hands out no device memory, code living inside someone else's memory pool.
For them ``mstar_paged_decode_attention_bf16_noalloc`` keeps the split-K scratch in a
4 MiB array inside the library.  This file checks that the variant computes what the
ordinary entry point computes and what the plain attention of tests/plain_llama.py
computes from the same keys and values, on two calls in a row (the second finds the first one's
leftovers in the shared array), and that it refuses a call that would need more scratch
than the array holds.  It is collected last on purpose: a run that stops at the first
failure has then already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def load_entry_point():
    from mstar_b200.ops.build import build_library

    lib = ctypes.CDLL(str(build_library("attention_decode_noalloc")))
    fn = lib.mstar_paged_decode_attention_bf16_noalloc
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, i, vp, vp, vp, i, vp, vp, i, i, i, i, i, i, f, i, i, vp]
    fn.restype = i
    return fn


def make_case(lens, nq, nkv, hd, page, seed):
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page) for n in lens]
    perm = iter(torch.randperm(sum(pages_per), generator=g).tolist())
    table = torch.full((len(lens), max(pages_per)), -1, dtype=torch.int32)
    for r, n in enumerate(pages_per):
        for p in range(n):
            table[r, p] = next(perm)
    kv = torch.randn(sum(pages_per), 2, nkv, page, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(len(lens), nq * hd, generator=g).to(torch.bfloat16)
    token_req = torch.arange(len(lens), dtype=torch.int32)
    cache_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    return [t.to(DEV) for t in (q, kv, table, token_req, cache_pos)]


def run_both(fn, lens, nq, nkv, hd, page, seed):
    from mstar_b200 import ops

    q, kv, table, token_req, cache_pos = make_case(lens, nq, nkv, hd, page, seed)
    tokens = len(lens)
    chunk, splits = ops.decode_split(tokens, nkv, max(lens))
    assert splits > 1, "the case must exercise the scratch"
    want = torch.empty(tokens, nq * hd, dtype=torch.bfloat16, device=DEV)
    ops.paged_decode_attention(q, nq * hd, want, kv, table, token_req, cache_pos, tokens, nq, nkv,
                               hd, page, 0, hd ** -0.5, max(lens))
    got = torch.full_like(want, float("nan"))
    rc = fn(q.data_ptr(), nq * hd, got.data_ptr(), kv.data_ptr(), table.data_ptr(),
            table.stride(0), token_req.data_ptr(), cache_pos.data_ptr(), tokens, nq, nkv, hd,
            page, 0, hd ** -0.5, chunk, splits, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f"entry point returned {rc}"
    torch.cuda.synchronize()
    return got, want, plain_decode(q, kv, table, cache_pos, nq, nkv, hd, page)


def plain_decode(q, kv, table, cache_pos, nq, nkv, hd, page):
    """The plain attention (tests/plain_llama.py) of each request's one query over the keys
    and values gathered from its pages, float64."""
    import plain_llama as P

    rows = []
    for r in range(q.shape[0]):
        n = int(cache_pos[r]) + 1
        pages = table[r, :-(-n // page)].long()
        k = kv[pages, 0].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:n].cpu()   # [keys, nkv, hd]
        v = kv[pages, 1].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:n].cpu()
        # a sequence whose last query is the decoded token: the causal mask of the last row
        # lets it see all n keys; the other rows are not looked at
        qs = q[r].cpu().view(1, nq, hd).expand(n, nq, hd)
        rows.append(P.plain_attention(qs, k, v)[-1].reshape(nq * hd))
    return torch.stack(rows)


def test_noalloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    fn = load_entry_point()
    allocated = torch.cuda.memory_allocated()
    # two calls in a row, different shapes: the second starts on the first one's leftovers
    for lens, nq, nkv, hd, page, seed in (([700, 33, 1500], 6, 2, 64, 16, 1),
                                          ([300, 2000], 24, 8, 128, 8, 2)):
        got, want, plain = run_both(fn, lens, nq, nkv, hd, page, seed)
        assert torch.isfinite(got.float()).all()
        # the tolerance of the kernel tests against the plain reference (bfloat16 outputs
        # of order 1), against the plain attention and against the ordinary entry point
        # (which cuts the keys into other chunks, so its float sums run in another order)
        assert (got.double().cpu() - plain).abs().max().item() < 2e-2
        assert (got.float() - want.float()).abs().max().item() < 2e-2
        del got, want, plain
    assert torch.cuda.memory_allocated() <= allocated + (1 << 20)   # nothing piled up


def test_noalloc_entry_point_refuses_more_scratch_than_it_has(capfd):
    fn = load_entry_point()
    z = torch.zeros(8, dtype=torch.int32, device=DEV)
    # 4096 tokens x 32 heads x 64 splits x 130 floats is far beyond the 1 Mi floats
    rc = fn(z.data_ptr(), 32 * 128, z.data_ptr(), z.data_ptr(), z.data_ptr(), 1, z.data_ptr(),
            z.data_ptr(), 4096, 32, 8, 128, 16, 0, 1.0, 64, 64, 0)
    assert rc == -2
    assert "exceed" in capfd.readouterr().err
