"""Each kernel alone against a plain float64 reference of the same op, at sizes other
than the engine's test models use (odd widths, head sizes in steps of 16, groups of
1, 3 and 5, permuted pages, windows)."""
import math
import os

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(dtype).to(DEV)


# --------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("table_dtype", DTYPES)
def test_embed_rows(table_dtype):
    from mstar_b200 import ops

    table = rnd(301, 100, dtype=table_dtype)
    ids = torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32, device=DEV)
    out = ops.embed_rows(table, ids)
    assert out.dtype == torch.float32
    assert torch.equal(out, table.float()[ids.long()])


def test_embed_rows_scaled_and_logit_scale_softcap():
    """The row multiplier of the embedding kernel and the scale / soft-cap kernel of the
    head, at widths that are no powers of two."""
    from mstar_b200 import ops

    table = rnd(77, 200, dtype=torch.bfloat16, seed=1)
    ids = torch.tensor([3, 76, 0, 3], dtype=torch.int32, device=DEV)
    out = ops.embed_rows(table, ids, scale=11.5)
    assert torch.equal(out, table[ids.long()].float() * 11.5)
    x = rnd(5, 1001, seed=2, scale=20.0)
    want = 30.0 * torch.tanh(x.double() * 0.25 / 30.0)
    got = ops.scale_softcap(x.clone(), 0.25, 30.0)
    assert (got.double() - want).abs().max() < 1e-5
    assert torch.equal(ops.scale_softcap(x.clone(), 0.5, None), x * 0.5)


@pytest.mark.parametrize("act", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("hidden", [100, 3000])
def test_add_rmsnorm(act, wdtype, hidden):
    from mstar_b200 import ops

    rows = 7
    resid = rnd(rows, hidden, seed=1)
    delta = rnd(rows, hidden, dtype=act, seed=2)
    w = (1 + 0.1 * rnd(hidden, seed=3)).to(wdtype)
    want_resid = resid.double() + delta.double()
    want = P.plain_rms_norm(want_resid.cpu(), w.cpu(), 1e-5)
    r = resid.clone()
    out = ops.add_rmsnorm(r, delta, w, 1e-5, act)
    assert (r.double() - want_resid).abs().max() < 1e-6          # the residual sum is float
    assert (out.double().cpu() - want).abs().max() < tol(act)
    # without a delta the residual is untouched; weight_offset gives the (1 + w) form
    r2 = resid.clone()
    out2 = ops.add_rmsnorm(r2, None, w, 1e-6, act, weight_offset=1.0)
    assert torch.equal(r2, resid)
    want2 = P.plain_rms_norm(resid.cpu(), (w.double() + 1).cpu(), 1e-6)
    assert (out2.double().cpu() - want2).abs().max() < tol(act, bf16=4e-2)
    # the promise that the kernel before did not write the residual changes when it is read,
    # not what comes out
    r3 = resid.clone()
    out3 = ops.add_rmsnorm(r3, delta, w, 1e-5, act, resid_static=True)
    assert torch.equal(out3, out) and torch.equal(r3, r)


@pytest.mark.parametrize("act", DTYPES)
def test_silu_mul_and_gather(act):
    from mstar_b200 import ops

    gu = rnd(5, 2 * 37, dtype=act, seed=4, scale=2.0)
    out = ops.silu_mul(gu)
    g, u = gu.double()[:, :37], gu.double()[:, 37:]
    assert (out.double() - g * torch.sigmoid(g) * u).abs().max() < tol(act, bf16=3e-2)

    resid = rnd(9, 50, seed=5)
    delta = rnd(9, 50, dtype=act, seed=6)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    got = ops.gather_add_rows(resid, delta, rows)
    assert (got.double() - (resid.double() + delta.double())[rows.long()]).abs().max() < 1e-6
    assert torch.equal(ops.gather_add_rows(resid, None, rows), resid[rows.long()])


def scatter_cache(num_pages, nkv, page, hd, dtype):
    return torch.zeros(num_pages, 2, nkv, page, hd, dtype=dtype, device=DEV)


def read_cache(kv, table, length, page):
    """Keys and values [length, nkv, hd] of one request, gathered through its table."""
    ks, vs = [], []
    for pos in range(length):
        pg = table[pos // page]
        ks.append(kv[pg, 0, :, pos % page])
        vs.append(kv[pg, 1, :, pos % page])
    return torch.stack(ks), torch.stack(vs)


@pytest.mark.parametrize("act", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,rot,inter", [(6, 3, 48, 48, False), (5, 1, 32, 16, False),
                                                 (4, 4, 16, 16, True), (2, 1, 64, 0, False)])
def test_rope_kv_write(act, nq, nkv, hd, rot, inter):
    from mstar_b200 import ops

    page, T = 4, 11
    # two requests: one continues at cache position 6, one starts at 0
    lens = [(6, 7), (0, 4)]
    token_req = torch.tensor([0] * 7 + [1] * 4, dtype=torch.int32, device=DEV)
    pos = torch.tensor([6 + i for i in range(7)] + list(range(4)), dtype=torch.int32, device=DEV)
    table = torch.tensor([[9, 2, 5, 0], [7, -1, -1, -1]], dtype=torch.int32, device=DEV)
    qkv = rnd(T, (nq + 2 * nkv) * hd, dtype=act, seed=7)
    kv = scatter_cache(10, nkv, page, hd, act)
    inv = None
    if rot:
        inv = torch.tensor([10000.0 ** (-2.0 * j / rot) for j in range(rot // 2)],
                           dtype=torch.float32, device=DEV)
    orig = qkv.clone()
    ops.rope_kv_write(qkv, pos, pos, token_req, table, inv, kv, nq, nkv, hd, rot, inter, page)

    def rotate(x):  # [T, heads, hd] float64 reference
        x = x.double().cpu()
        if not rot:
            return x
        xr = x[..., :rot]
        if inter:
            xr = torch.cat([xr[..., 0::2], xr[..., 1::2]], dim=-1)
        y = P.plain_apply_rope(xr, pos.cpu(), inv.double().cpu())
        if inter:
            z = torch.empty_like(y)
            z[..., 0::2], z[..., 1::2] = y[..., :rot // 2], y[..., rot // 2:]
            y = z
        return torch.cat([y, x[..., rot:]], dim=-1)

    q0 = orig[:, :nq * hd].view(T, nq, hd)
    k0 = orig[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
    v0 = orig[:, (nq + nkv) * hd:].view(T, nkv, hd)
    assert (qkv[:, :nq * hd].view(T, nq, hd).double().cpu() - rotate(q0)).abs().max() < tol(act)
    assert torch.equal(qkv[:, nq * hd:], orig[:, nq * hd:])       # k, v rows stay as they were
    kref, t0 = rotate(k0), 0
    for r, (start, n) in enumerate(lens):
        ks, vs = read_cache(kv, table[r].tolist(), start + n, page)
        assert (ks[start:].double().cpu() - kref[t0:t0 + n]).abs().max() < tol(act)
        assert torch.equal(vs[start:], v0[t0:t0 + n])
        assert ks[:start].abs().max() == 0 if start else True     # nothing else is touched
        t0 += n


# ----------------------------------------------------------------------- attention
def paged_case(lens_q, lens_kv, nq, nkv, hd, page, act, seed, window=0, spike=None,
               kernel="generic"):
    """Random q and paged k/v for requests with lens_kv keys of which the last lens_q are
    this step's queries; pages are handed out in a scrambled order.  ``spike`` =
    (request, key index): that key is made to dominate every query's softmax."""
    from mstar_b200 import ops

    g = torch.Generator().manual_seed(seed)
    n_req = len(lens_q)
    pages_per = [-(-n // page) for n in lens_kv]
    perm = torch.randperm(sum(pages_per) + 3, generator=g).tolist()
    width = max(pages_per)
    table = torch.full((n_req, width), -1, dtype=torch.int32)
    kv = torch.zeros(sum(pages_per) + 3, 2, nkv, page, hd, dtype=act)
    ks, vs = [], []
    it = iter(perm)
    for r in range(n_req):
        k = torch.randn(lens_kv[r], nkv, hd, generator=g)
        v = torch.randn(lens_kv[r], nkv, hd, generator=g)
        if spike and spike[0] == r:
            k[spike[1]] *= 0.0
            k[spike[1], :, 0] = 30.0
        k, v = k.to(act), v.to(act)
        ks.append(k), vs.append(v)
        for p in range(pages_per[r]):
            pg = next(it)
            table[r, p] = pg
            chunk = slice(p * page, min((p + 1) * page, lens_kv[r]))
            n = chunk.stop - chunk.start
            kv[pg, 0, :, :n] = k[chunk].transpose(0, 1)
            kv[pg, 1, :, :n] = v[chunk].transpose(0, 1)
    T = sum(lens_q)
    q = torch.randn(T, nq, hd, generator=g)
    if spike:
        q[..., 0] = 3.0 + q[..., 0].abs()
    q = q.to(act)
    token_req = torch.tensor([r for r in range(n_req) for _ in range(lens_q[r])],
                             dtype=torch.int32)
    cache_pos = torch.tensor([lens_kv[r] - lens_q[r] + i for r in range(n_req)
                              for i in range(lens_q[r])], dtype=torch.int32)
    out = torch.empty(T, nq * hd, dtype=act, device=DEV)
    qd = q.reshape(T, nq * hd).to(DEV).contiguous()
    if kernel == "generic":
        ops.paged_attention_generic(qd, nq * hd, out, kv.to(DEV), table.to(DEV),
                                    token_req.to(DEV), cache_pos.to(DEV), T, nq, nkv, hd, page,
                                    window, hd ** -0.5)
    elif kernel == "decode":
        assert all(n == 1 for n in lens_q)
        ops.paged_decode_attention(qd, nq * hd, out, kv.to(DEV), table.to(DEV), token_req.to(DEV),
                                   cache_pos.to(DEV), T, nq, nkv, hd, page, window, hd ** -0.5,
                                   max(lens_kv))
    else:
        indptr = [0]
        for n in lens_q:
            indptr.append(indptr[-1] + n)
        ops.paged_prefill_attention(
            qd, nq * hd, out, kv.to(DEV), table.to(DEV),
            torch.tensor(indptr, dtype=torch.int32, device=DEV),
            torch.tensor(lens_kv, dtype=torch.int32, device=DEV), 0, n_req, max(lens_q), nq, nkv,
            hd, page, window, hd ** -0.5)
    # plain reference: whole-sequence attention with the queries placed at the end
    want = torch.empty(T, nq, hd, dtype=torch.float64)
    t0 = 0
    for r in range(n_req):
        full_q = torch.zeros(lens_kv[r], nq, hd, dtype=torch.float64)
        full_q[lens_kv[r] - lens_q[r]:] = q[t0:t0 + lens_q[r]].double()
        ref = P.plain_attention(full_q, ks[r], vs[r], window=window or None)
        want[t0:t0 + lens_q[r]] = ref[lens_kv[r] - lens_q[r]:]
        t0 += lens_q[r]
    return out.view(T, nq, hd).double().cpu(), want, vs


@pytest.mark.parametrize("act", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,page", [(6, 2, 48, 4), (5, 1, 32, 16), (3, 3, 16, 8),
                                            (8, 2, 128, 16), (2, 1, 256, 2)])
def test_paged_attention_mixed_batch(act, nq, nkv, hd, page):
    got, want, _ = paged_case([1, 7, 1, 40, 2], [33, 7, 1, 75, 130], nq, nkv, hd, page, act,
                              seed=nq * 100 + hd)
    assert (got - want).abs().max() < tol(act, f32=2e-5, bf16=2e-2)


@pytest.mark.parametrize("act", DTYPES)
def test_paged_attention_far_key_among_hundreds(act):
    # key 3 of 700 dominates: the output must be its value, wherever its page lies
    got, want, vs = paged_case([1, 5], [700, 650], 6, 2, 32, 8, act, seed=11, spike=(0, 3))
    assert (got - want).abs().max() < tol(act, f32=2e-5, bf16=2e-2)
    v3 = vs[0][3].double()                        # [nkv, hd]
    for h in range(6):
        assert (got[0, h] - v3[h // 3]).abs().max() < 3e-2


@pytest.mark.parametrize("act", DTYPES)
def test_paged_attention_window_edge(act):
    # window 20 on 100 keys: key 80 is the oldest one the last query sees, key 79 is out
    for spike_key, inside in ((80, True), (79, False)):
        got, want, vs = paged_case([1], [100], 4, 2, 32, 8, act, seed=13, window=20,
                                   spike=(0, spike_key))
        assert (got - want).abs().max() < tol(act, f32=2e-5, bf16=2e-2)
        hit = (got[0, 0] - vs[0][spike_key, 0].double()).abs().max() < 3e-2
        assert bool(hit) == inside


# page sizes 8..64 with head sizes 64/128/256 take the TMA path of the decode kernel
SHAPES_FAST = [(6, 2, 64, 4), (5, 1, 32, 16), (3, 3, 16, 8), (24, 8, 128, 16), (2, 1, 256, 2),
               (16, 1, 64, 16), (4, 2, 256, 8), (6, 3, 128, 32), (8, 8, 64, 64),
               (6, 2, 128, 128), (4, 4, 64, 256), (3, 1, 256, 128)]   # pages larger than a tile


@pytest.mark.parametrize("nq,nkv,hd,page", SHAPES_FAST)
def test_decode_attention_kernel(nq, nkv, hd, page):
    # lengths around tile (64) and chunk edges, one long enough to be split many times
    lens = [1, 63, 64, 65, 200, 1500, 17]
    got, want, _ = paged_case([1] * len(lens), lens, nq, nkv, hd, page, torch.bfloat16,
                              seed=nq + hd, kernel="decode")
    assert (got - want).abs().max() < 2e-2
    got, want, _ = paged_case([1], [3000], nq, nkv, hd, page, torch.bfloat16, seed=3,
                              kernel="decode")              # one request: as many splits as fit
    assert (got - want).abs().max() < 2e-2
    assert tc_clean() == 0                                  # no bounded wait of a TMA copy ran out


@pytest.mark.parametrize("nq,nkv,hd,page", SHAPES_FAST)
def test_prefill_attention_kernel(nq, nkv, hd, page):
    # whole prompts, portions appended to cached keys, single tokens, sizes around 64 rows
    lens_q = [1, 7, 40, 2, 65, 130, 33]
    lens_kv = [33, 7, 75, 130, 65, 300, 33]
    got, want, _ = paged_case(lens_q, lens_kv, nq, nkv, hd, page, torch.bfloat16, seed=nq * 7 + hd,
                              kernel="prefill")
    assert (got - want).abs().max() < 2e-2


@pytest.mark.parametrize("which", ["tcgen05", "mma"])
@pytest.mark.parametrize("nq,nkv,page,hd", [(24, 8, 16, 128), (6, 3, 32, 128), (5, 1, 8, 128),
                                            (4, 4, 64, 128), (14, 2, 16, 128), (6, 2, 16, 64),
                                            (3, 1, 8, 64), (4, 2, 16, 256), (3, 3, 8, 256)])
def test_prefill_attention_both_kernels(which, nq, nkv, page, hd, monkeypatch):
    """The tcgen05 kernel (128-row tiles in tensor memory) and the mma.sync kernel on the
    same cases: rows around the tile sizes, portions behind cached keys, many key tiles."""
    from mstar_b200 import ops

    monkeypatch.setenv("MSTAR_PREFILL_ATTENTION", which)
    assert ops.prefill_attention_kernel(True, hd, page) == which
    lens_q = [1, 7, 43, 2, 65, 130, 700]
    lens_kv = [33, 7, 75, 130, 65, 300, 900]
    got, want, _ = paged_case(lens_q, lens_kv, nq, nkv, hd, page, torch.bfloat16,
                              seed=nq * 5 + page, kernel="prefill")
    assert (got - want).abs().max() < 2e-2
    # one key far back dominates every row: found among hundreds, in every tile row
    got, want, vs = paged_case([300], [640], nq, nkv, hd, page, torch.bfloat16, seed=5,
                               spike=(0, 3), kernel="prefill")
    assert (got - want).abs().max() < 2e-2
    for h in range(nq if hd <= 128 else 0):   # the far key carries most of the weight
        far = vs[0][3, h // (nq // nkv)].double()
        assert (want[17, h] - far).abs().max() < 0.2 * far.abs().max()
        assert (got[17, h] - far).abs().max() < 0.2 * far.abs().max()
    assert tc_clean() == 0


@pytest.mark.parametrize("nq,nkv,page,hd", [(24, 8, 16, 128), (5, 1, 8, 128), (14, 2, 64, 64),
                                            (4, 2, 16, 256), (4, 4, 32, 128), (9, 1, 16, 64),
                                            (32, 2, 64, 128), (128, 1, 32, 64)])
def test_prefill_attention_tcgen05_row_tiles(nq, nkv, page, hd, monkeypatch):
    """The tcgen05 kernel's row tiles are whole tokens (128 // G of them, G query heads per kv
    head: 126 rows at G 3, 125 at 5, 126 at 7) fetched by one TMA box per 64 features: prompts
    and portions around those sizes, behind cached keys, with one far key early or late in
    the context that the last token must find."""
    from mstar_b200 import ops

    monkeypatch.setenv("MSTAR_PREFILL_ATTENTION", "tcgen05")
    assert ops.prefill_attention_kernel(True, hd, page, nq // nkv) == "tcgen05"
    assert ops.prefill_attention_kernel(True, hd, page, 129) == "mma"    # more heads than a tile has rows
    per_tile = 128 // (nq // nkv)
    lens_q = [1, max(1, per_tile - 1), per_tile, per_tile + 1, 2 * per_tile, 2, 700 if nq < 100 else 90]
    lens_kv = [33, max(1, per_tile - 1), 300, per_tile + 1, 2 * per_tile + 5, 130, 900 if nq < 100 else 200]
    for seed in (1, 2):
        got, want, _ = paged_case(lens_q, lens_kv, nq, nkv, hd, page, torch.bfloat16, seed=seed,
                                  kernel="prefill")
        assert (got - want).abs().max() < 2e-2
    for far_key in (3, 600):
        got, want, vs = paged_case([300], [640], nq, nkv, hd, page, torch.bfloat16, seed=5,
                                   spike=(0, far_key), kernel="prefill")
        assert (got - want).abs().max() < 2e-2
        # the last token sees the key, which carries most of its weight: a tile that lost it
        # would be off by far more than the tolerance above
        far = vs[0][far_key, 0].double()
        assert hd > 128 or (want[299, 0] - far).abs().max() < 0.5 * far.abs().max()
    assert tc_clean() == 0


@pytest.mark.parametrize("page", [8, 16, 128])
def test_attention_kernels_over_long_contexts(page):
    """Thousands of keys: the producers fetch block-table entries 32 at a time and wrap
    their rings many times; one key far back carries a sixth of the weight."""
    got, want, _ = paged_case([2500, 1], [5000, 4100], 6, 2, 128, page, torch.bfloat16, seed=3,
                              kernel="prefill")
    assert (got - want).abs().max() < 2e-2
    got, want, vs = paged_case([1, 1, 1], [9000, 70, 4097], 6, 2, 128, page, torch.bfloat16,
                               seed=4, spike=(0, 8000), kernel="decode")
    assert (got - want).abs().max() < 2e-2
    assert tc_clean() == 0


def test_attention_kernels_on_cases_drawn_at_random():
    """Heads and groups, head sizes, page sizes (8 to 256), numbers of requests and their lengths
    drawn at random (a fixed seed): whole prompts, portions behind cached keys and single
    decoded tokens, against the plain attention; no bounded wait may run out."""
    from mstar_b200 import ops

    rng = np.random.default_rng(5)
    shapes = [(24, 8, 128), (6, 2, 128), (5, 1, 128), (4, 4, 128), (14, 2, 64), (32, 8, 64),
              (9, 1, 64), (4, 2, 256), (3, 3, 256), (12, 1, 128)]
    for trial in range(60):
        nq, nkv, hd = shapes[int(rng.integers(len(shapes)))]
        page = int(rng.choice([8, 16, 32, 64, 128, 256]))
        n_req = int(rng.integers(1, 6))
        lens_kv = [int(rng.integers(1, 700 if hd < 256 else 300)) for _ in range(n_req)]
        kind = "prefill" if trial % 2 == 0 else "decode"
        lens_q = [int(rng.integers(1, kv + 1)) for kv in lens_kv] if kind == "prefill" else [1] * n_req
        got, want, _ = paged_case(lens_q, lens_kv, nq, nkv, hd, page, torch.bfloat16, seed=trial,
                                  kernel=kind)
        err = (got - want).abs().max().item()
        assert err < 2e-2, (trial, kind, nq, nkv, hd, page, lens_q, lens_kv, err)
    assert tc_clean() == 0


def test_prefill_attention_kernel_choice(monkeypatch):
    from mstar_b200 import ops

    monkeypatch.delenv("MSTAR_PREFILL_ATTENTION", raising=False)
    assert ops.prefill_attention_kernel(True, 128, 16) == "tcgen05"
    assert ops.prefill_attention_kernel(True, 32, 16) == "mma"      # other head size
    assert ops.prefill_attention_kernel(False, 128, 4) == "mma"     # no TMA map of the cache
    monkeypatch.setenv("MSTAR_PREFILL_ATTENTION", "mma")
    assert ops.prefill_attention_kernel(True, 128, 16) == "mma"


@pytest.mark.parametrize("kernel", ["decode", "prefill"])
def test_fast_attention_far_key_and_window(kernel):
    act = torch.bfloat16
    got, want, vs = paged_case([1, 1], [700, 650], 6, 2, 32, 8, act, seed=11, spike=(0, 3),
                               kernel=kernel)
    assert (got - want).abs().max() < 2e-2
    for h in range(6):
        assert (got[0, h] - vs[0][3, h // 3].double()).abs().max() < 3e-2
    for spike_key, inside in ((80, True), (79, False)):
        got, want, vs = paged_case([1], [100], 4, 2, 32, 8, act, seed=13, window=20,
                                   spike=(0, spike_key), kernel=kernel)
        assert (got - want).abs().max() < 2e-2
        hit = (got[0, 0] - vs[0][spike_key, 0].double()).abs().max() < 3e-2
        assert bool(hit) == inside
    if kernel == "prefill":
        # a portion of 50 tokens with a window of 20 over 300 keys: every row has its own edge
        got, want, _ = paged_case([50, 9], [300, 9], 4, 2, 64, 16, act, seed=17, window=20,
                                  kernel="prefill")
        assert (got - want).abs().max() < 2e-2
    else:
        got, want, _ = paged_case([1, 1, 1], [300, 9, 150], 4, 2, 64, 16, act, seed=17,
                                  window=100, kernel="decode")
        assert (got - want).abs().max() < 2e-2


def test_fast_attention_refuses_other_head_sizes():
    from mstar_b200 import ops

    assert not ops.fast_attention_supported(torch.bfloat16, 4, 2, 48)
    assert not ops.fast_attention_supported(torch.float32, 4, 2, 64)
    assert not ops.fast_attention_supported(torch.bfloat16, 34, 2, 64)
    assert ops.fast_attention_supported(torch.bfloat16, 24, 8, 128)
    q = torch.zeros(1, 4 * 48, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError, match="refuses"):
        ops.paged_decode_attention(q, 4 * 48, q.clone(),
                                   torch.zeros(1, 2, 2, 4, 48, dtype=torch.bfloat16, device=DEV),
                                   z.view(1, 1), z, z, 1, 4, 2, 48, 4, 0, 1.0, 1)


def test_paged_attention_refuses_what_it_cannot_do():
    from mstar_b200 import ops
    from mstar_b200.ops import KernelError

    q = torch.zeros(1, 64 * 128, device=DEV)
    with pytest.raises(KernelError, match="refuses"):
        ops.paged_attention_generic(q, 64 * 128, q.clone(), torch.zeros(1, 2, 1, 4, 128, device=DEV),
                                    torch.zeros(1, 1, dtype=torch.int32, device=DEV),
                                    torch.zeros(1, dtype=torch.int32, device=DEV),
                                    torch.zeros(1, dtype=torch.int32, device=DEV),
                                    1, 64, 1, 128, 4, 0, 1.0)


# ---------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("m,n,k", [(1, 91, 53), (37, 130, 200), (130, 64, 17), (64, 1000, 96)])
def test_sgemm_is_true_float32(m, n, k):
    from mstar_b200 import ops

    a, w = rnd(m, k, seed=1), rnd(n, k, seed=2)
    got = ops.sgemm_nt(a, w)
    want = a.double() @ w.double().T
    # float rounding only: far below what a TF32 product (10-bit mantissa) would give
    assert (got.double() - want).abs().max() < 2e-5 * math.sqrt(k)
    # a row's result does not depend on the other rows of the batch
    assert torch.equal(ops.sgemm_nt(a[:1].contiguous(), w), got[:1])


@pytest.mark.parametrize("m,n,k", [(1, 200, 96), (50, 1000, 320)])
def test_linear_bf16_and_mixed(m, n, k):
    from mstar_b200 import ops

    x, w = rnd(m, k, dtype=torch.bfloat16, seed=3), rnd(n, k, dtype=torch.bfloat16, seed=4)
    want = x.double() @ w.double().T
    y = ops.linear(x, w)
    assert y.dtype == torch.bfloat16 and (y.double() - want).abs().max() < 0.02 * math.sqrt(k)
    y32 = ops.linear(x, w, out_dtype=torch.float32)
    assert y32.dtype == torch.float32 and (y32.double() - want).abs().max() < 1e-3 * math.sqrt(k)
    # a weight kept in 32-bit is multiplied in 32-bit even on the bfloat16 path
    ymix = ops.linear(x, w.float())
    assert ymix.dtype == torch.bfloat16
    assert (ymix.double() - want).abs().max() < 0.02 * math.sqrt(k)


# ------------------------------------------------------------------------ sampling
def test_argmax_and_greedy_rows():
    from mstar_b200 import ops

    logits = rnd(5, 1003, seed=5)
    logits[2, 17] = logits[2, 900] = 50.0          # equal maxima: the smaller index wins
    want = logits.argmax(-1).int()
    want[2] = 17
    assert torch.equal(ops.argmax(logits), want)
    temp = torch.zeros(5, device=DEV)
    assert torch.equal(ops.sample(logits, temp), want)


@pytest.mark.parametrize("rows,vocab", [(1, 7), (8, 156940), (64, 50001), (300, 1024), (3, 32768)])
def test_argmax_in_pieces(rows, vocab):
    """The greedy kernel cuts a row into pieces that meet in a 64-bit atomic maximum: rows
    whose width is no multiple of four and whose stride is not the width, equal maxima in
    different pieces (the smaller index wins), a maximum in the last element, negative rows,
    a NaN that must not win, and launch after launch on the same scratch."""
    from mstar_b200 import ops

    wide = rnd(rows, vocab + 3, seed=rows + vocab) - 3.0
    logits = wide[:, 1:vocab + 1]                      # a view: odd offset, stride != width
    assert logits.stride(0) != vocab and logits.data_ptr() % 16 != 0
    if vocab > 100:
        logits[0, 5] = logits[0, vocab - 2] = 40.0     # equal maxima far apart
        logits[rows - 1, vocab - 1] = 41.0             # the last element
        logits[rows // 2, 3] = float("nan")
    want = torch.nan_to_num(logits, nan=-float("inf")).argmax(-1).int()
    if vocab > 100:
        want[0] = 5 if rows > 1 else want[0]
    for _ in range(3):
        assert torch.equal(ops.argmax(logits), want)
    aligned = logits.contiguous() if vocab % 4 == 0 else None
    if aligned is not None:
        assert torch.equal(ops.argmax(aligned), want)  # the 16-byte loads


def draw(logits, temperature, seed, offset, **kw):
    from mstar_b200 import ops

    rows = logits.shape[0]
    t = torch.full((rows,), temperature, device=DEV)
    s = torch.tensor(seed, dtype=torch.int64, device=DEV)
    o = torch.tensor(offset, dtype=torch.int64, device=DEV)
    extra = {}
    if "top_k" in kw:
        extra["top_k"] = torch.full((rows,), kw["top_k"], dtype=torch.int32, device=DEV)
    if "top_p" in kw:
        extra["top_p"] = torch.full((rows,), kw["top_p"], device=DEV)
    return ops.sample(logits, t, seed=s, offset=o, **extra)


@pytest.mark.parametrize("opts", [{}, {"top_k": 5}, {"top_p": 0.7}, {"top_k": 40, "top_p": 0.5}])
def test_sample_is_the_inverse_cdf_of_the_plain_distribution(opts):
    vocab, rows = 1537, 64
    logits = rnd(1, vocab, seed=6, scale=2.0).repeat(rows, 1).contiguous()
    seeds, offsets = [1234] * rows, list(range(rows))
    got = draw(logits, 0.8, seeds, offsets, **opts).tolist()
    p = P.plain_sampling_distribution(logits[0].cpu(), 0.8, **opts)
    cdf = torch.cumsum(p, 0)
    for r, tok in enumerate(got):
        assert p[tok] > 0, f"row {r}: token {tok} is outside the kept set"
        u = P.plain_uniform(seeds[r], offsets[r])
        lo = cdf[tok - 1].item() if tok else 0.0
        assert lo - 1e-4 <= u <= cdf[tok].item() + 1e-4, (r, tok, u)
    # same (seed, offset) -> same token; another offset or seed -> another draw somewhere
    assert draw(logits, 0.8, seeds, offsets, **opts).tolist() == got
    assert draw(logits, 0.8, [99] * rows, offsets, **opts).tolist() != got


def test_sample_at_the_size_of_a_real_vocabulary():
    """156,940 logits a row, every option at once (the reference's defaults are a
    temperature, top-p and a repetition penalty): the kept set and the draw follow the
    plain distribution; rows of one batch with different options do not disturb each other."""
    from mstar_b200 import ops

    vocab, rows = 156940, 6
    logits = rnd(rows, vocab, seed=9, scale=3.0)
    seen = torch.zeros(rows, vocab, dtype=torch.uint8, device=DEV)
    seen[:, ::7] = 1
    temp = torch.tensor([0.6, 0.6, 1.3, 0.6, 0.0, 0.9], device=DEV)
    top_k = torch.tensor([0, 50, 0, 200, 0, 1], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([0.8, 1.0, 0.95, 0.5, 1.0, 1.0], device=DEV)
    pen = torch.tensor([1.3, 1.0, 1.3, 1.1, 1.3, 1.0], device=DEV)
    srows = torch.arange(rows, dtype=torch.int32, device=DEV)
    seeds = torch.arange(100, 100 + rows, dtype=torch.int64, device=DEV)
    offs = torch.arange(rows, dtype=torch.int64, device=DEV)
    before = seen.clone()
    got = ops.sample(logits, temp, top_k=top_k, top_p=top_p, penalty=pen, seen_mask=seen,
                     seen_rows=srows, seed=seeds, offset=offs).tolist()
    for r, tok in enumerate(got):
        x = logits[r].cpu()
        if temp[r] == 0:
            pl = P.plain_sampling_distribution(x, 1.0, penalty=float(pen[r]), seen=before[r].cpu())
            assert tok == int(pl.argmax())
            continue
        p = P.plain_sampling_distribution(x, float(temp[r]), top_k=int(top_k[r]),
                                          top_p=float(top_p[r]), penalty=float(pen[r]),
                                          seen=before[r].cpu())
        assert p[tok] > 0, f"row {r}: token {tok} is outside the kept set"
        cdf = torch.cumsum(p, 0)
        u = P.plain_uniform(100 + r, r)
        lo = cdf[tok - 1].item() if tok else 0.0
        assert lo - 1e-4 <= u <= cdf[tok].item() + 1e-4, (r, tok, u)
        assert seen[r, tok] == 1
    assert int(seen.sum() - before.sum()) <= rows
    again = ops.sample(logits, temp, top_k=top_k, top_p=top_p, penalty=pen, seen_mask=before,
                       seen_rows=srows, seed=seeds, offset=offs).tolist()
    assert again == got


def test_sample_frequencies_follow_the_distribution():
    vocab, rows = 50, 4096
    logits = rnd(1, vocab, seed=8).repeat(rows, 1).contiguous()
    got = draw(logits, 1.0, [7] * rows, list(range(rows)))
    freq = torch.bincount(got.long().cpu(), minlength=vocab).double() / rows
    p = torch.softmax(logits[0].double().cpu(), -1)
    assert (freq - p).abs().max() < 0.03


def test_repetition_penalty_and_seen_mask():
    from mstar_b200 import ops

    vocab = 300
    logits = torch.zeros(2, vocab, device=DEV)
    logits[:, 5] = 4.0
    logits[:, 9] = 3.0
    seen = torch.zeros(4, vocab, dtype=torch.uint8, device=DEV)
    seen[2, 5] = 1                                  # row 0 uses mask row 2, row 1 none
    rows = torch.tensor([2, -1], dtype=torch.int32, device=DEV)
    pen = torch.tensor([2.0, 2.0], device=DEV)
    temp = torch.zeros(2, device=DEV)
    got = ops.sample(logits, temp, penalty=pen, seen_mask=seen, seen_rows=rows)
    assert got.tolist() == [9, 5]                   # 4.0 / 2 < 3.0 where 5 was seen
    assert seen[2, 9] == 1 and seen.sum() == 2      # the sampled token is marked


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(16, 32), (100, 96), (3000, 1024), (157, 3072), (33001, 64),
                                 (1030, 2080)])
def test_small_m_gemm(m, n, k):
    """The weight-streaming products of decode steps (weights through a shared-memory ring of
    bulk copies with strips of 8, 16 and 32 rows): every M up to 16, N that is no multiple of
    the strip, K from one block of 32 up and K that is no multiple of the ring's chunk, both
    output types."""
    from mstar_b200 import ops

    x = rnd(m, k, dtype=torch.bfloat16, seed=m)
    w = rnd(n, k, dtype=torch.bfloat16, seed=n, scale=0.1)
    want = x.double() @ w.double().T
    y = ops._gemm_smallm(x, w, torch.bfloat16, gated=False)     # the kernel itself
    assert torch.equal(ops.linear(x, w), y) or m > ops.SMALL_M
    assert y.dtype == torch.bfloat16 and y.shape == (m, n)
    assert (y.double() - want).abs().max() < 0.01 * want.abs().max() + 1e-3
    y32 = ops._gemm_smallm(x, w, torch.float32, gated=False)
    assert (y32.double() - want).abs().max() < 2e-4 * math.sqrt(k)
    # a row's result does not depend on how many other rows the batch has
    if m > 1:
        assert torch.equal(ops._gemm_smallm(x[:1].contiguous(), w, torch.bfloat16, False), y[:1])
    # rows that are views into a wider buffer (stride larger than K)
    wide = torch.zeros(m, k + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :k] = x
    assert torch.equal(ops._gemm_smallm(wide[:, :k], w, torch.bfloat16, False), y)
    assert tc_clean() == 0                                  # no bounded wait ran out


@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("nq,nkv,hd,k,page", [(6, 3, 48, 96, 4), (5, 1, 32, 64, 8), (4, 4, 16, 32, 4),
                                              (24, 8, 128, 1056, 64), (3, 1, 256, 2080, 16)])
def test_qkv_product_with_rotary_and_cache_write(m, nq, nkv, hd, k, page):
    """The decode form of the mixer's first product (product, rotation, cache write in one
    kernel) against the float64 rotation of the float64 product, and against the two
    separate kernels: tokens of several requests at scattered cache positions, head sizes
    in steps of 16, a K that is no multiple of the ring's chunk."""
    from mstar_b200 import ops

    x = rnd(m, k, dtype=torch.bfloat16, seed=m + hd)
    w = rnd((nq + 2 * nkv) * hd, k, dtype=torch.bfloat16, seed=nq, scale=0.1)
    inv = torch.tensor([500000.0 ** (-2.0 * j / hd) for j in range(hd // 2)],
                       dtype=torch.float32, device=DEV)
    # token i belongs to request i % 3 and lies at a cache position of its own; positions
    # for the angles differ from the cache positions
    per_req = 6
    table = torch.randperm(3 * per_req, generator=torch.Generator().manual_seed(m)).to(
        torch.int32).view(3, per_req).to(DEV)
    token_req = torch.tensor([i % 3 for i in range(m)], dtype=torch.int32, device=DEV)
    cache_pos = torch.tensor([(7 * i + 3) % (per_req * page) for i in range(m)],
                             dtype=torch.int32, device=DEV)
    assert len({(int(r), int(c)) for r, c in zip(token_req, cache_pos)}) == m
    pos = cache_pos + 1000
    kv = scatter_cache(3 * per_req, nkv, page, hd, torch.bfloat16)
    q = ops.qkv_rope_write(x, w, pos, cache_pos, token_req, table, inv, kv, nq, nkv, hd, page)
    assert q is not None and q.shape == (m, nq * hd) and tc_clean() == 0

    # the two separate kernels
    kv2 = scatter_cache(3 * per_req, nkv, page, hd, torch.bfloat16)
    qkv = ops.linear(x, w)
    ops.rope_kv_write(qkv, pos, cache_pos, token_req, table, inv, kv2, nq, nkv, hd, hd, False, page)
    assert (q.float() - qkv[:, :nq * hd].float()).abs().max() <= 2 ** -7 * qkv.float().abs().max()
    assert (kv.float() - kv2.float()).abs().max() <= 2 ** -7 * kv2.float().abs().max()

    # float64: rotate the exact product
    y = (x.double() @ w.double().T).cpu()
    scale = y.abs().max()
    qr = P.plain_apply_rope(y[:, :nq * hd].view(m, nq, hd), pos.cpu(), inv.double().cpu())
    kr = P.plain_apply_rope(y[:, nq * hd:(nq + nkv) * hd].view(m, nkv, hd), pos.cpu(),
                            inv.double().cpu())
    vr = y[:, (nq + nkv) * hd:].view(m, nkv, hd)
    assert (q.double().cpu().view(m, nq, hd) - qr).abs().max() < 0.012 * scale
    written = torch.zeros(kv.shape[0], page, dtype=torch.bool)
    for i in range(m):
        cp = int(cache_pos[i])
        pg = int(table[int(token_req[i]), cp // page])
        written[pg, cp % page] = True
        assert (kv[pg, 0, :, cp % page].double().cpu() - kr[i]).abs().max() < 0.012 * scale
        assert (kv[pg, 1, :, cp % page].double().cpu() - vr[i]).abs().max() < 0.012 * scale
    # nothing else in the cache is touched
    untouched = kv.cpu().permute(0, 3, 1, 2, 4)[~written]
    assert untouched.abs().max() == 0


@pytest.mark.parametrize("tokens,ctx", [(8, 700), (3, 64), (16, 129), (1, 2000)])
def test_decode_sequence_with_promises(tokens, ctx):
    """A decode step's kernels in a row, as the engine launches them: the fused first product
    (rotation, cache write) and the attention that is promised static earlier keys, against
    the separate kernels without promises.  The token's own key is written by the kernel
    directly before the attention, the earlier keys long before; the results are the same
    bit for bit, launch after launch."""
    from mstar_b200 import ops

    nq, nkv, hd, page, k = 24, 8, 128, 64, 512
    x = rnd(tokens, k, dtype=torch.bfloat16, seed=tokens)
    w = rnd((nq + 2 * nkv) * hd, k, dtype=torch.bfloat16, seed=ctx, scale=0.05)
    inv = torch.tensor([500000.0 ** (-2.0 * j / hd) for j in range(hd // 2)],
                       dtype=torch.float32, device=DEV)
    pages_per = -(-(ctx + 1) // page)
    g = torch.Generator().manual_seed(5)
    table = torch.randperm(tokens * pages_per, generator=g).to(torch.int32).view(tokens, -1).to(DEV)
    old = rnd(tokens * pages_per, 2, nkv, page, hd, dtype=torch.bfloat16, seed=9)
    token_req = torch.arange(tokens, dtype=torch.int32, device=DEV)
    cache_pos = torch.tensor([ctx - (7 * i) % min(ctx, 50) for i in range(tokens)],
                             dtype=torch.int32, device=DEV)

    def step(fused):
        kv = old.clone()
        torch.cuda.synchronize()
        if fused:
            q = ops.qkv_rope_write(x, w, cache_pos, cache_pos, token_req, table, inv, kv, nq, nkv,
                                   hd, page)
        else:
            q = ops.linear(x, w)
            ops.rope_kv_write(q, cache_pos, cache_pos, token_req, table, inv, kv, nq, nkv, hd, hd,
                              False, page)
        out = torch.empty(tokens, nq * hd, dtype=torch.bfloat16, device=DEV)
        ops.paged_decode_attention(q, q.stride(0), out, kv, table, token_req, cache_pos, tokens,
                                   nq, nkv, hd, page, 0, hd ** -0.5, ctx + 1, static_keys=fused)
        return out, kv

    want, kv_want = step(False)
    for _ in range(5):
        got, kv_got = step(True)
        assert torch.equal(kv_got, kv_want)
        assert torch.equal(got, want)
    assert tc_clean() == 0


def test_small_m_gemm_refuses_more_rows():
    from mstar_b200 import ops

    x, w = rnd(17, 64, dtype=torch.bfloat16), rnd(32, 64, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="refuses"):
        ops._gemm_smallm(x, w, torch.bfloat16, gated=False)
    assert ops.linear(x, w).shape == (17, 32)             # the library product takes over


@pytest.mark.parametrize("inter,k", [(200, 96), (1500, 1120)])
@pytest.mark.parametrize("m", [1, 8, 13, 16, 100])
def test_gated_up_fused_and_unfused(m, inter, k):
    from mstar_b200 import ops

    x = rnd(m, k, dtype=torch.bfloat16, seed=1)
    w = rnd(2 * inter, k, dtype=torch.bfloat16, seed=2, scale=0.2)
    got = ops.gated_up(x, w) if m > 16 else ops._gemm_smallm(x, w, torch.bfloat16, gated=True)
    g = (x.double() @ w[:inter].double().T)
    u = (x.double() @ w[inter:].double().T)
    want = g * torch.sigmoid(g) * u
    assert got.shape == (m, inter)
    assert (got.double() - want).abs().max() < 0.02 * want.abs().max() + 2e-3
    # the fused kernel (m <= 16) and product + SiLU-multiply agree to bfloat16 rounding
    ref = ops.silu_mul(torch.mm(x, w.t()))
    assert (got.double() - ref.double()).abs().max() < 0.02 * want.abs().max() + 2e-3


# ------------------------------------------------------------------- tcgen05 GEMM
def tc_clean():
    from mstar_b200 import ops

    torch.cuda.synchronize()
    word = ops.tcgen05_error_word(DEV)
    code = int(word.item())
    word.zero_()
    return code


@pytest.mark.parametrize("bn", [128, 256, 512, 1024])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (1, 8, 8), (200, 300, 136), (513, 1000, 776),
                                   (64, 2048, 3072), (300, 130, 4096)])
def test_tcgen05_gemm(bn, m, n, k):
    """TMA + tcgen05.mma + TMEM product: lone CTAs (bn 128, 256) and CTA pairs (512); sizes
    that are no multiples of the tiles, K that is no multiple of the 64-wide block."""
    from mstar_b200 import ops

    x = rnd(m, k, dtype=torch.bfloat16, seed=m + k)
    w = rnd(n, k, dtype=torch.bfloat16, seed=n, scale=0.1)
    want = x.double() @ w.double().T
    y = ops.gemm_tcgen05(x, w, torch.bfloat16, bn)
    y32 = ops.gemm_tcgen05(x, w, torch.float32, bn)
    assert tc_clean() == 0
    assert (y32.double() - want).abs().max() < 2e-4 * math.sqrt(k) * max(1.0, want.abs().max().item() / 8)
    assert (y.double() - want).abs().max() < 0.01 * want.abs().max() + 1e-3
    # a view into a wider buffer: the row stride goes into the tensor map
    wide = torch.zeros(m, k + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :k] = x
    assert torch.equal(ops.gemm_tcgen05(wide[:, :k], w, torch.bfloat16, bn), y)
    assert tc_clean() == 0


@pytest.mark.parametrize("m,inter,k", [(256, 128, 64), (77, 200, 96), (2048, 1000, 512)])
def test_tcgen05_gated_gemm(m, inter, k):
    from mstar_b200 import ops

    x = rnd(m, k, dtype=torch.bfloat16, seed=1)
    w = rnd(2 * inter, k, dtype=torch.bfloat16, seed=2, scale=0.2)
    got = ops.gemm_tcgen05_gated(x, w)
    assert tc_clean() == 0
    g = x.double() @ w[:inter].double().T
    u = x.double() @ w[inter:].double().T
    want = g * torch.sigmoid(g) * u
    assert got.shape == (m, inter)
    assert (got.double() - want).abs().max() < 0.02 * want.abs().max() + 2e-3
    ref = ops.silu_mul(torch.mm(x, w.t()))
    assert (got.double() - ref.double()).abs().max() < 0.02 * want.abs().max() + 2e-3


def test_tcgen05_refusals_and_dispatch(monkeypatch):
    from mstar_b200 import ops

    x = rnd(32, 20, dtype=torch.bfloat16)          # K = 20 is no multiple of 8
    w = rnd(64, 20, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="refuses"):
        ops.gemm_tcgen05(x, w)
    assert ops.linear(x, w).shape == (32, 64)       # the library product takes it
    assert ops.tcgen05_tile(2048, 16384) == 1024 and ops.tcgen05_tile(64, 156940) == 256
    assert ops.tcgen05_tile(2048, 3072) is None
    monkeypatch.setenv("MSTAR_GEMM", "tcgen05")
    assert ops.tcgen05_tile(2048, 3072) == 1024
    monkeypatch.setenv("MSTAR_GEMM", "library")
    assert ops.tcgen05_tile(2048, 16384) is None


# ------------------------------------------------------------ swapped-operand tcgen05 GEMM
@pytest.mark.parametrize("m", [17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("n,k", [(300, 136), (130, 4096), (5120, 3072), (1000, 776), (33001, 64)])
def test_skinny_gemm(m, n, k):
    """17 to 128 rows with W as the MMA's M operand: row counts on both sides of the three
    token widths, output widths and K that are no multiples of the tiles."""
    from mstar_b200 import ops

    x = rnd(m, k, dtype=torch.bfloat16, seed=m + k)
    w = rnd(n, k, dtype=torch.bfloat16, seed=n, scale=0.1)
    want = x.double() @ w.double().T
    y = ops.gemm_skinny(x, w, torch.bfloat16)
    y32 = ops.gemm_skinny(x, w, torch.float32, static_weights=True)
    assert tc_clean() == 0
    assert (y32.double() - want).abs().max() < 2e-4 * math.sqrt(k) * max(1.0, want.abs().max().item() / 8)
    assert (y.double() - want).abs().max() < 0.01 * want.abs().max() + 1e-3
    # a view into a wider buffer: the row stride goes into the tensor map
    wide = torch.zeros(m, k + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :k] = x
    assert torch.equal(ops.gemm_skinny(wide[:, :k], w, torch.bfloat16), y)
    assert tc_clean() == 0


def test_skinny_gemm_refusals_and_dispatch(monkeypatch):
    from mstar_b200 import ops

    x = rnd(129, 64, dtype=torch.bfloat16)
    w = rnd(64, 64, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="refuses"):
        ops.gemm_skinny(x, w)
    with pytest.raises(ops.KernelError, match="refuses"):
        ops.gemm_skinny(rnd(20, 20, dtype=torch.bfloat16), rnd(64, 20, dtype=torch.bfloat16))
    assert ops.linear(x, w).shape == (129, 64)             # the library product takes it
    # chosen for a matrix of several tiles per SM only (a vocabulary-wide head)
    wide = torch.empty(ops.SKINNY_TILES_PER_SM * ops.num_sms() * 128, 64, dtype=torch.bfloat16,
                       device=DEV)
    assert ops._skinny_ok(x[:64], wide) and not ops._skinny_ok(x[:64], w)
    assert not ops._skinny_ok(x[:16], wide) and not ops._skinny_ok(x, wide)
    monkeypatch.setenv("MSTAR_SKINNY", "0")
    assert not ops._skinny_ok(x[:64], wide)
    monkeypatch.setenv("MSTAR_SKINNY", "1")
    assert ops._skinny_ok(x[:64], w)
    assert torch.equal(ops.linear(x[:64], w), ops.gemm_skinny(x[:64], w))
