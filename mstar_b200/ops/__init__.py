"""Python entry points of the hand-written kernels.

Each function validates shapes and dtypes, then launches a kernel from
``csrc/`` on the current CUDA stream.  Tensors must live on the GPU; nothing
here computes on the CPU.  Matrix products in bfloat16: this package's
weight-streaming kernels for up to 16 rows, its tcgen05 kernels for the LM head and
for gate/up at prompt size, and the library GEMM (cuBLAS through ``torch.mm``)
elsewhere, as the reference uses for every linear layer
(mstar/model/components/distributed/linear.py:101, 412); the float32 product
is this package's own true-32-bit kernel.
"""
from __future__ import annotations

import os

import torch

from . import lib
from .lib import BF16, F32, KernelError, check

_DT = {torch.float32: F32, torch.bfloat16: BF16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported (float32 and bfloat16 are)") from None


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw accessors cost a
    tenth of ``torch.cuda.current_stream()``, which matters at some 300 launches a step)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("mstar_b200 kernels run on CUDA tensors only; got a "
                              f"{t.device} tensor (there is no CPU path)")


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None,
               source=None, scale: float = 1.0):
    """out[t] = float(table[ids[t]]) * scale; the residual stream is float in both dtypes.
    ``source`` = (src, prev): where src[t] >= 0 the token is prev[src[t]] instead, a token
    that is on the device only (int32 tensors, src as long as ids)."""
    _need_cuda(table, ids)
    assert ids.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    n, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    src = prev = None
    if source is not None:
        src, prev = source
        _need_cuda(src, prev)
        assert src.dtype == torch.int32 and prev.dtype == torch.int32 and src.numel() == n
    check(lib.get("elementwise").mstar_embed_rows(
        table.data_ptr(), _dt(table), ids.data_ptr(), _ptr(src), _ptr(prev), out.data_ptr(), n,
        vocab, hidden, float(scale), _stream()), "embed_rows")
    return out


def scale_softcap(x: torch.Tensor, scale: float = 1.0, cap: float | None = None):
    """In place on float ``x``: x *= scale, then x = cap * tanh(x / cap) if ``cap``."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    check(lib.get("elementwise").mstar_scale_softcap(
        x.data_ptr(), x.numel(), float(scale), float(cap or 0.0), _stream()), "scale_softcap")
    return x


def add_rmsnorm(resid: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, weight_offset: float = 0.0, out=None,
                resid_static: bool = False):
    """resid += delta (if given), in place in float; returns rmsnorm(resid)*weight.
    ``resid_static`` promises that the kernel before this one on the stream did not write
    ``resid`` (it wrote ``delta``): the residual is then read while that kernel drains."""
    _need_cuda(resid, delta, weight)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    rows, hidden = resid.shape
    assert weight.numel() == hidden and weight.is_contiguous()
    if delta is not None:
        assert delta.shape == resid.shape and delta.dtype == out_dtype and delta.is_contiguous()
    if out is None:
        out = torch.empty((rows, hidden), dtype=out_dtype, device=resid.device)
    check(lib.get("elementwise").mstar_add_rmsnorm(
        resid.data_ptr(), _ptr(delta), weight.data_ptr(), _dt(weight), out.data_ptr(), _dt(out),
        rows, hidden, float(eps), float(weight_offset), int(resid_static), _stream()),
        "add_rmsnorm")
    return out


def gather_add_rows(resid: torch.Tensor, delta, rows: torch.Tensor):
    """float(resid[rows] + delta[rows]) as a new [len(rows), hidden] tensor."""
    _need_cuda(resid, delta, rows)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and rows.dtype == torch.int32
    hidden = resid.shape[1]
    out = torch.empty((rows.numel(), hidden), dtype=torch.float32, device=resid.device)
    act = _dt(delta) if delta is not None else F32
    if delta is not None:
        assert delta.shape == resid.shape and delta.is_contiguous()
    check(lib.get("elementwise").mstar_gather_add_rows(
        resid.data_ptr(), _ptr(delta), act, rows.data_ptr(), out.data_ptr(), rows.numel(),
        hidden, _stream()), "gather_add_rows")
    return out


def silu_mul(gate_up: torch.Tensor, out=None):
    """silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    check(lib.get("elementwise").mstar_silu_mul(
        gate_up.data_ptr(), out.data_ptr(), _dt(gate_up), rows, inter, _stream()), "silu_mul")
    return out


def convert(src: torch.Tensor, dtype: torch.dtype):
    _need_cuda(src)
    if src.dtype == dtype:
        return src
    assert src.is_contiguous()
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    check(lib.get("elementwise").mstar_convert(
        src.data_ptr(), _dt(src), out.data_ptr(), _dt(out), src.numel(), _stream()), "convert")
    return out


def rope_kv_write(qkv: torch.Tensor, positions, cache_pos, token_req, block_table,
                  inv_freq, kv_cache, num_heads: int, num_kv_heads: int, head_dim: int,
                  rotary_dim: int, interleaved: bool, page_size: int) -> None:
    """Rotate queries in place; rotate keys and copy values into their cache pages.

    ``kv_cache``: [pages, 2, kv_heads, page_size, head_dim] or None (queries only).
    ``inv_freq``: float [rotary_dim / 2] or None when rotary_dim == 0."""
    _need_cuda(qkv, positions, cache_pos, token_req, block_table, inv_freq, kv_cache)
    assert qkv.dim() == 2 and qkv.is_contiguous()
    n = qkv.shape[0]
    assert qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    assert rotary_dim % 2 == 0 and 0 <= rotary_dim <= head_dim
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype == torch.float32
        assert inv_freq.numel() == rotary_dim // 2
    if kv_cache is not None:
        assert kv_cache.dtype == qkv.dtype and kv_cache.is_contiguous()
        assert tuple(kv_cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim)
    check(lib.get("elementwise").mstar_rope_kv_write(
        qkv.data_ptr(), _dt(qkv), positions.data_ptr(), cache_pos.data_ptr(),
        token_req.data_ptr(), block_table.data_ptr(), block_table.stride(0), _ptr(inv_freq),
        _ptr(kv_cache), n, num_heads, num_kv_heads, head_dim, rotary_dim, int(interleaved),
        page_size, _stream()), "rope_kv_write")


def paged_attention_generic(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv_cache,
                            block_table, token_req, cache_pos, num_tokens: int, num_heads: int,
                            num_kv_heads: int, head_dim: int, page_size: int, window: int,
                            scale: float) -> None:
    """Attention of ``num_tokens`` query rows (portions and decoded tokens alike)
    over the paged cache; ``q`` may be a view into the fused qkv buffer with
    ``q_stride`` elements between tokens."""
    _need_cuda(q, out, kv_cache, block_table, token_req, cache_pos)
    assert out.is_contiguous() and kv_cache.is_contiguous()
    code = lib.get("attention_generic").mstar_paged_attention_generic(
        q.data_ptr(), q_stride, out.data_ptr(), kv_cache.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), token_req.data_ptr(), cache_pos.data_ptr(), num_tokens,
        num_heads, num_kv_heads, head_dim, page_size, window, float(scale), _dt(out), _stream())
    if code == -1:
        raise KernelError(
            f"paged attention refuses heads={num_heads}, kv_heads={num_kv_heads}, "
            f"head_dim={head_dim}: it needs head_dim <= 256 and (heads/kv_heads)*head_dim <= 4096")
    check(code, "paged_attention_generic")


FAST_ATTENTION_HEAD_DIMS = (16, 32, 64, 128, 256)

_sm_counts: dict = {}


def num_sms(device=None) -> int:
    """SMs of ``device`` (default: the current CUDA device), asked once per device."""
    index = torch.cuda.current_device() if device is None else (
        torch.device(device).index or 0)
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def fast_attention_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int,
                             head_dim: int) -> bool:
    """Whether the tensor-core attention kernels take this shape (else the generic
    kernel does)."""
    return (dtype == torch.bfloat16 and head_dim in FAST_ATTENTION_HEAD_DIMS
            and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16)


# CTAs of the decode attention grid per SM that the split of the keys aims for (the kernel
# with one CTA per work item), and CTAs per SM of the persistent ring kernel
DECODE_FILL = 6
RING_CTAS_PER_SM = 2


def decode_split(tokens: int, num_kv_heads: int, max_len: int, ring: bool = False,
                 sms: int | None = None) -> tuple:
    """(chunk, splits) of the keys for split-K decode attention, chunks in whole tiles of 64
    keys.  One CTA per work item (token, kv head, split): enough items to fill the GPU a
    few times over.  Persistent ring kernel: as many items as CTAs are resident or fewer
    (each CTA then streams one item of equal size), of at least 128 keys.  ``sms``: the
    device's SM count (default: asked of the current device)."""
    if sms is None:
        sms = num_sms()
    pairs = max(tokens * num_kv_heads, 1)
    if ring:
        want = max(1, (sms * RING_CTAS_PER_SM) // pairs)
        chunk = max(128, -(-(-(-max_len // want)) // 64) * 64)
    else:
        fill = int(os.environ.get("MSTAR_DECODE_FILL", DECODE_FILL))
        want = max(1, -(-sms * fill // pairs))
        want = min(want, 256)                   # the merge kernel takes up to 256 splits
        chunk = max(64, -(-(-(-max_len // want)) // 64) * 64)
    splits = max(1, -(-max_len // chunk))
    while splits > 256:                         # the merge kernel takes up to 256 splits
        chunk *= 2
        splits = max(1, -(-max_len // chunk))
    return chunk, splits


# page sizes whose caches the TMA kernels take: boxes of min(page, 64) keys
TMA_PAGE_SIZES = (8, 16, 32, 64, 128, 256)

_kv_maps: dict = {}


def kv_tensor_map(kv_cache: torch.Tensor):
    """The TMA tensor map (a 128-byte host buffer) of a cache tensor [pages, 2, kv_heads,
    page_size, head_dim], or None when the TMA kernels do not take its shape."""
    pages, _, nkv, page_size, hd = kv_cache.shape
    key = (kv_cache.data_ptr(), tuple(kv_cache.shape))
    if key not in _kv_maps:
        import ctypes

        buf = ctypes.create_string_buffer(128 + 64)
        addr = (ctypes.addressof(buf) + 63) & ~63          # the driver wants 64-byte alignment
        code = lib.get("attention_decode").mstar_make_kv_tensor_map(
            addr, kv_cache.data_ptr(), pages, nkv, page_size, hd)
        if code == -1:
            _kv_maps[key] = None
        elif code != 0:
            raise KernelError(f"could not make the TMA tensor map of a cache (code {code})")
        else:
            _kv_maps[key] = (buf, addr)
    entry = _kv_maps[key]
    return None if entry is None else entry[1]


def paged_decode_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv_cache,
                           block_table, token_req, cache_pos, tokens: int, num_heads: int,
                           num_kv_heads: int, head_dim: int, page_size: int, window: int,
                           scale: float, max_len: int, static_keys: bool = False) -> None:
    """bfloat16 attention of ``tokens`` single-query rows (token i of q/out/token_req/
    cache_pos); ``max_len`` bounds the keys any of them sees.  ``static_keys`` promises that
    the kernel before this one on the stream wrote nothing that is read here but the queries
    and each token's own key and value (a decode step of the engine: the keys before are from
    earlier steps, the index arrays from before the step's first kernel); the copies of the
    earlier keys then start while that kernel is still draining."""
    _need_cuda(q, out, kv_cache, block_table, token_req, cache_pos)
    assert q.dtype == torch.bfloat16 and kv_cache.dtype == torch.bfloat16
    assert (q_stride * 2) % 16 == 0 and q.data_ptr() % 16 == 0 and out.is_contiguous()
    if window:
        max_len = min(max_len, window)
    kv_map = kv_tensor_map(kv_cache) if not window else None
    ring = kv_map is not None and os.environ.get("MSTAR_DECODE_ATTENTION") != "per_item"
    if not ring and page_size > 64:
        kv_map = None                       # the per-item TMA kernel copies whole pages
    chunk, splits = decode_split(tokens, num_kv_heads, max(max_len, 1), ring=ring,
                                 sms=num_sms(q.device))
    scratch = None
    if splits > 1:
        scratch = torch.empty(tokens * num_heads * splits * (head_dim + 2), dtype=torch.float32,
                              device=q.device)
    if kv_map is not None:
        code = lib.get("attention_decode").mstar_paged_decode_attention_bf16_tma(
            kv_map, q.data_ptr(), q_stride, out.data_ptr(), kv_cache.data_ptr(),
            block_table.data_ptr(), block_table.stride(0), token_req.data_ptr(),
            cache_pos.data_ptr(), tokens, num_heads, num_kv_heads, head_dim, page_size,
            float(scale), chunk, splits, int(static_keys), _ptr(scratch),
            tcgen05_error_word(q.device).data_ptr(), _stream())
        if code == -1:
            raise KernelError("TMA decode attention refuses this shape")
        check(code, "paged_decode_attention_tma")
        if splits > 1:
            lib.add_launches(1)                 # the merge kernel
        return
    code = lib.get("attention_decode").mstar_paged_decode_attention_bf16(
        q.data_ptr(), q_stride, out.data_ptr(), kv_cache.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), token_req.data_ptr(), cache_pos.data_ptr(), tokens, num_heads,
        num_kv_heads, head_dim, page_size, window, float(scale), chunk, splits, _ptr(scratch),
        _stream())
    if code == -1:
        raise KernelError(f"decode attention refuses heads={num_heads}, kv_heads={num_kv_heads}, "
                          f"head_dim={head_dim} (head_dim in {FAST_ATTENTION_HEAD_DIMS}, at most "
                          "16 query heads per kv head)")
    check(code, "paged_decode_attention")
    if splits > 1:
        lib.add_launches(1)                     # the merge kernel


def prefill_attention_kernel(has_kv_map: bool, head_dim: int, page_size: int, group: int = 1) -> str:
    """"tcgen05" or "mma": which prefill attention kernel runs.  The tcgen05 kernel takes
    head_dim 64, 128 or 256, no window, the page sizes of ``TMA_PAGE_SIZES`` and up to 128
    query heads per kv head (``group``), and is the faster one from the shortest portions on;
    MSTAR_PREFILL_ATTENTION=mma selects the other."""
    import os

    takes = (has_kv_map and head_dim in (64, 128, 256) and page_size in TMA_PAGE_SIZES
             and group <= 128)
    if not takes or os.environ.get("MSTAR_PREFILL_ATTENTION") == "mma":
        return "mma"
    return "tcgen05"


def paged_prefill_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, kv_cache,
                            block_table, qo_indptr, kv_len, first_entry: int, entries: int,
                            max_q_len: int, num_heads: int, num_kv_heads: int, head_dim: int,
                            page_size: int, window: int, scale: float) -> None:
    """bfloat16 attention of the new tokens of batch entries [first_entry, first_entry +
    entries); q and out hold all tokens of the step, indexed through qo_indptr."""
    _need_cuda(q, out, kv_cache, block_table, qo_indptr, kv_len)
    assert q.dtype == torch.bfloat16 and kv_cache.dtype == torch.bfloat16
    assert (q_stride * 2) % 16 == 0 and q.data_ptr() % 16 == 0 and out.is_contiguous()
    kv_map = kv_tensor_map(kv_cache) if not window else None
    if prefill_attention_kernel(kv_map is not None, head_dim, page_size,
                                num_heads // num_kv_heads) == "tcgen05":
        code = lib.get("attention_prefill_tc").mstar_paged_prefill_attention_tc(
            kv_map, q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), qo_indptr.data_ptr(), kv_len.data_ptr(), first_entry, entries,
            max_q_len, num_heads, num_kv_heads, head_dim, page_size, float(scale),
            tcgen05_error_word(q.device).data_ptr(), _stream())
        if code == -1:
            raise KernelError("tcgen05 prefill attention refuses this shape")
        check(code, "paged_prefill_attention_tc")
        return
    code = lib.get("attention_prefill").mstar_paged_prefill_attention_bf16(
        kv_map or 0, q.data_ptr(), q_stride, out.data_ptr(), kv_cache.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), qo_indptr.data_ptr(), kv_len.data_ptr(),
        first_entry, entries, max_q_len, num_heads, num_kv_heads, head_dim, page_size, window,
        float(scale), tcgen05_error_word(q.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"prefill attention refuses heads={num_heads}, kv_heads={num_kv_heads}, "
                          f"head_dim={head_dim} (head_dim in {FAST_ATTENTION_HEAD_DIMS})")
    check(code, "paged_prefill_attention")


def sgemm_nt(a: torch.Tensor, w: torch.Tensor, out=None):
    """a[M,K] @ w[N,K]^T in true float32 (FMA, no tensor-core reduced precision)."""
    _need_cuda(a, w)
    assert a.dtype == torch.float32 and w.dtype == torch.float32
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1]
    assert a.stride(1) == 1 and w.stride(1) == 1
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    assert out.stride(1) == 1
    check(lib.get("gemm_f32").mstar_sgemm_nt(
        a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), w.stride(0),
        out.stride(0), _stream()), "sgemm_nt")
    return out


# Rows up to which the weight-streaming kernel is used (it takes up to 16); beyond, the
# library GEMM.
SMALL_M = 16


def _smallm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= SMALL_M
            and x.shape[1] % 32 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _gemm_smallm(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, gated: bool,
                 static_weights: bool = False):
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty((m, n // 2 if gated else n), dtype=out_dtype, device=x.device)
    code = lib.get("gemm_smallm_bulk").mstar_gemm_smallm_bulk_bf16(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), w.stride(0),
        out.stride(0), int(gated), _dt(out), int(static_weights),
        tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"small-M GEMM refuses M={m}, N={n}, K={k}")
    check(code, "gemm_smallm_bulk")
    return out


# Rows up to which the swapped-operand tcgen05 kernel is used (tokens are the MMA's N
# dimension: 32, 64 or 128), the rows of W to one of its tiles, and the tiles per SM from
# which on it is used: each CTA takes one tile and all of K, so only a matrix of many tiles
# (a vocabulary-wide head) fills the GPU several times over; with few tiles the library's
# cut along K wins.
SKINNY_MAX = 128
SKINNY_ROWS = 128
SKINNY_TILES_PER_SM = 4


def _skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the product of ``SMALL_M`` < M <= ``SKINNY_MAX`` bfloat16 rows goes to the
    swapped-operand tcgen05 kernel (MSTAR_SKINNY=0: nowhere, 1: for every width)."""
    if not (SMALL_M < x.shape[0] <= SKINNY_MAX and _tc_ok(x, w)):
        return False
    forced = os.environ.get("MSTAR_SKINNY")
    if forced is not None:
        return forced != "0"
    return -(-w.shape[0] // SKINNY_ROWS) >= SKINNY_TILES_PER_SM * num_sms(x.device)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
                static_weights: bool = False):
    """x[M,K] @ w[N,K]^T for up to 128 bfloat16 rows on the tcgen05 tensor cores with the
    operands swapped (rows of W are the MMA's M dimension, the tokens its N dimension)."""
    _need_cuda(x, w)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] == w.shape[1]
    m, k = x.shape
    n = w.shape[0]
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    code = lib.get("gemm_skinny").mstar_gemm_skinny_bf16(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), w.stride(0),
        out.stride(0), _dt(out), int(static_weights),
        tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"skinny GEMM refuses M={m}, N={n}, K={k} (at most {SKINNY_MAX} rows, "
                          "K and row strides multiples of 8, operands 16-byte aligned)")
    if code in (-3, -4):
        raise KernelError(f"skinny GEMM could not make its TMA tensor map (code {code})")
    check(code, "gemm_skinny")
    return out


def qkv_rope_write(x: torch.Tensor, w_qkv: torch.Tensor, positions, cache_pos, token_req,
                   block_table, inv_freq, kv_cache, num_heads: int, num_kv_heads: int,
                   head_dim: int, page_size: int, static_weights: bool = False):
    """For few bfloat16 rows (decoded tokens): the product x Wqkv^T, the split-half rotary
    encoding of q and k over the whole head, and the write of k and v into their cache
    pages, as one kernel.  Returns q [M, num_heads * head_dim], rotated; or None when this
    form does not apply (more than ``SMALL_M`` rows, another dtype, no cache to write, or
    MSTAR_FUSED_ROPE=0), and the caller runs ``linear`` and ``rope_kv_write`` instead."""
    if (kv_cache is None or inv_freq is None or not _smallm_ok(x, w_qkv)
            or kv_cache.dtype != torch.bfloat16 or head_dim % 16
            or inv_freq.numel() != head_dim // 2
            or w_qkv.shape[0] != (num_heads + 2 * num_kv_heads) * head_dim
            or os.environ.get("MSTAR_FUSED_ROPE") == "0"):
        return None
    _need_cuda(x, w_qkv, positions, cache_pos, token_req, block_table, inv_freq, kv_cache)
    assert kv_cache.is_contiguous() and inv_freq.dtype == torch.float32
    assert tuple(kv_cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim)
    m, k = x.shape
    q = torch.empty((m, num_heads * head_dim), dtype=torch.bfloat16, device=x.device)
    code = lib.get("gemm_smallm_bulk").mstar_qkv_rope_write_bulk_bf16(
        x.data_ptr(), w_qkv.data_ptr(), q.data_ptr(), m, k, x.stride(0), w_qkv.stride(0),
        q.stride(0), positions.data_ptr(), cache_pos.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), inv_freq.data_ptr(), kv_cache.data_ptr(),
        num_heads, num_kv_heads, head_dim, page_size, int(static_weights),
        tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"fused qkv/rotary product refuses M={m}, K={k}, heads={num_heads}, "
                          f"kv_heads={num_kv_heads}, head_dim={head_dim}")
    check(code, "qkv_rope_write")
    return q


_tc_error_words: dict = {}


def tcgen05_error_word(device) -> torch.Tensor:
    """Device int32 that a kernel with bounded mbarrier waits sets when one of them ran out:
    1-3 tcgen05 GEMM (producer, MMA issuer, epilogue), 4 decode attention copies, 6-12 tcgen05
    prefill attention, 13-14 bulk-copy small-M GEMM, 15-17 swapped-operand tcgen05 GEMM; zero
    otherwise."""
    key = torch.device(device).index or 0
    if key not in _tc_error_words:
        _tc_error_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_error_words[key]


WAIT_CODES = {
    1: "tcgen05 GEMM: the producer waited for a free operand stage",
    2: "tcgen05 GEMM: the MMA issuer waited for operand tiles",
    3: "tcgen05 GEMM: the epilogue waited for an accumulator",
    4: "decode attention: a wait for a key/value tile",
    5: "attention: a wait for the query tile or a key/value tile copied by TMA",
    13: "bulk-copy small-M GEMM: the producer waited for a free stage",
    14: "bulk-copy small-M GEMM: a consumer waited for weights",
}
WAIT_CODES.update({15: "swapped-operand tcgen05 GEMM: the producer waited for a free stage",
                   16: "swapped-operand tcgen05 GEMM: the MMA issuer waited for operand tiles",
                   17: "swapped-operand tcgen05 GEMM: the epilogue waited for the accumulator"})
WAIT_CODES.update({c: "tcgen05 prefill attention: a wait on one of its barriers ran out"
                   for c in range(6, 13)})


def raise_on_wait_code(code: int) -> None:
    """``code``: a value read from ``tcgen05_error_word``.  Non-zero means that a bounded
    wait inside a kernel ran out and the kernel returned with partial output, so whatever
    was computed since the word was last zero must not be used."""
    code = int(code)
    if code == 0:
        return
    what = WAIT_CODES.get(code, "an unknown kernel")
    raise KernelError(f"a kernel gave up a bounded wait (code {code}: {what}); the results "
                      "of the steps since the last check are not valid")


def check_error_word(device) -> None:
    """Read the device's error word (this waits for the work queued so far), zero it if it
    is set, and raise ``KernelError`` naming the code.  The engine's entry points call this
    (or read the word along with a step's results) before they hand results out."""
    word = tcgen05_error_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        raise_on_wait_code(code)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
                 bn: int = 256):
    """x[M,K] @ w[N,K]^T on the tcgen05 tensor cores (TMA operand tiles, TMEM
    accumulator).  bfloat16 operands, K and the row strides multiples of 8."""
    _need_cuda(x, w)
    out_dtype = out_dtype or torch.bfloat16
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1]
    assert x.stride(1) == 1 and w.stride(1) == 1
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    code = lib.get("gemm_tcgen05").mstar_gemm_tcgen05_bf16(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), w.stride(0),
        out.stride(0), _dt(out), bn, tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"tcgen05 GEMM refuses M={m}, N={n}, K={k} (K and row strides must be "
                          "multiples of 8, operands 16-byte aligned)")
    if code in (-3, -4):
        raise KernelError(f"tcgen05 GEMM could not make its TMA tensor map (code {code})")
    check(code, "gemm_tcgen05")
    return out


def gemm_tcgen05_gated(x: torch.Tensor, w_gate_up: torch.Tensor):
    """silu(x Wg^T) * (x Wu^T) for the fused [Wg; Wu] on pairs of CTAs (cta_group::2),
    the activation applied in the epilogue straight from tensor memory."""
    _need_cuda(x, w_gate_up)
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
    assert x.stride(1) == 1 and w_gate_up.stride(1) == 1 and x.shape[1] == w_gate_up.shape[1]
    m, k = x.shape
    n = w_gate_up.shape[0]
    out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
    code = lib.get("gemm_tcgen05").mstar_gemm_tcgen05_gated_bf16(
        x.data_ptr(), w_gate_up.data_ptr(), out.data_ptr(), m, n, k, x.stride(0),
        w_gate_up.stride(0), out.stride(0), tcgen05_error_word(x.device).data_ptr(), _stream())
    if code == -1:
        raise KernelError(f"gated tcgen05 GEMM refuses M={m}, N={n}, K={k}")
    if code in (-3, -4):
        raise KernelError(f"tcgen05 GEMM could not make its TMA tensor map (code {code})")
    check(code, "gemm_tcgen05_gated")
    return out


def _tc_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def tcgen05_tile(m: int, n: int, sms: int | None = None) -> int | None:
    """Which tcgen05 kernel takes an [m, K] x [n, K]^T product of more than ``SKINNY_MAX``
    rows, or None for the library GEMM: 256 = lone CTAs with 128 x 256 tiles, 1024 =
    persistent CTA pairs with 256 x 256 tiles (512: the same pairs, one tile each).
    The hand-written kernels are used where their tiles fill the GPU: up to 256 rows when
    there is a 128 x 256 tile or more for every SM (a vocabulary-wide head), beyond when the
    256 x 256 tiles make three waves or more over the CTA pairs (below, the library's finer
    tiles win: measured at 96 to 160 tiles on 74 pairs).
    ``MSTAR_GEMM=tcgen05`` forces them everywhere, ``MSTAR_GEMM=library`` nowhere."""
    forced = os.environ.get("MSTAR_GEMM", "")
    if forced == "library":
        return None
    if sms is None:
        sms = num_sms()
    if m <= 256:
        if -(-n // 256) >= sms:
            return 256
    elif -(-m // 256) * -(-n // 256) >= 3 * (sms // 2):
        return 1024
    if forced == "tcgen05":
        return 1024 if m > 128 else 256
    return None


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           static_weights: bool = False):
    """x[M,K] @ w[N,K]^T.  bfloat16: this package's weight-streaming kernel for at most
    ``SMALL_M`` rows, its swapped-operand tcgen05 kernel up to ``SKINNY_MAX`` rows, its
    tiled tcgen05 kernels where ``tcgen05_tile`` says so, else the library GEMM; anything
    involving a float32 operand runs in true float32.  ``static_weights`` promises that no
    kernel earlier on the stream writes ``w`` (model parameters): the kernels for few rows
    then start their weight copies while the kernel before them is still draining."""
    bf16 = x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and w.is_cuda
    m, n = x.shape[0], w.shape[0]
    if bf16 and out_dtype is None and m > SKINNY_MAX and tcgen05_tile(m, n) is None:
        # the common case of a prompt portion on a narrow projection, decided first: this
        # function runs a hundred times in a step that the host has to get launched
        return torch.mm(x, w.t())
    _need_cuda(x, w)
    out_dtype = out_dtype or x.dtype
    if out_dtype in (torch.bfloat16, torch.float32) and _smallm_ok(x, w):
        return _gemm_smallm(x, w, out_dtype, gated=False, static_weights=static_weights)
    if out_dtype in (torch.bfloat16, torch.float32) and _skinny_ok(x, w):
        return gemm_skinny(x, w, out_dtype, static_weights=static_weights)
    if out_dtype in (torch.bfloat16, torch.float32) and _tc_ok(x, w):
        tile = tcgen05_tile(x.shape[0], w.shape[0])
        if tile is not None:
            return gemm_tcgen05(x, w, out_dtype, tile)
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if out_dtype == torch.float32:
            try:
                return torch.mm(x, w.t(), out_dtype=torch.float32)
            except (TypeError, RuntimeError):
                return torch.mm(x, w.t()).float()
        return torch.mm(x, w.t())
    xf = convert(x, torch.float32)
    wf = convert(w, torch.float32)
    y = sgemm_nt(xf, wf)
    return convert(y, out_dtype)


def gated_up(x: torch.Tensor, w_gate_up: torch.Tensor, static_weights: bool = False):
    """silu(x Wg^T) * (x Wu^T) for the fused matrix [Wg; Wu]: one kernel for few
    bfloat16 rows, else the product followed by the SiLU-multiply kernel."""
    _need_cuda(x, w_gate_up)
    if _smallm_ok(x, w_gate_up) and w_gate_up.shape[0] % 2 == 0:
        return _gemm_smallm(x, w_gate_up, torch.bfloat16, gated=True, static_weights=static_weights)
    if (_tc_ok(x, w_gate_up) and w_gate_up.shape[0] % 16 == 0
            and tcgen05_tile(x.shape[0], w_gate_up.shape[0]) is not None):
        return gemm_tcgen05_gated(x, w_gate_up)
    return silu_mul(linear(x, w_gate_up))


_argmax_scratch: dict = {}


def _argmax_buffers(device, rows: int):
    """Zeroed scratch of the argmax kernel (a 64-bit key and a counter per row); the kernel
    leaves it zeroed.  One per device: launches that share it run on one stream."""
    key = torch.device(device).index or 0
    have = _argmax_scratch.get(key)
    if have is None or have[1].numel() < rows:
        n = max(rows, 1024)
        have = _argmax_scratch[key] = (torch.zeros(n, dtype=torch.int64, device=device),
                                       torch.zeros(n, dtype=torch.int32, device=device))
    return have


def argmax(logits: torch.Tensor):
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    rows, vocab = logits.shape
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    best, arrived = _argmax_buffers(logits.device, rows)
    check(lib.get("sampling").mstar_argmax(
        logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), best.data_ptr(),
        arrived.data_ptr(), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature, top_k=None, top_p=None, penalty=None,
           seen_mask=None, seen_rows=None, seed=None, offset=None):
    """One token per row.  Per-row tensors: temperature float32, top_k int32,
    top_p float32, penalty float32, seed/offset int64; ``seen_mask`` uint8
    [slots, vocab] with ``seen_rows`` int32 naming each row's slot (or -1)."""
    _need_cuda(logits, temperature, top_k, top_p, penalty, seen_mask, seen_rows, seed, offset)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    rows, vocab = logits.shape
    assert temperature.dtype == torch.float32 and temperature.numel() == rows
    for t, dt in ((top_k, torch.int32), (top_p, torch.float32), (penalty, torch.float32),
                  (seen_rows, torch.int32), (seed, torch.int64), (offset, torch.int64)):
        assert t is None or (t.dtype == dt and t.numel() == rows)
    if seen_mask is not None:
        assert seen_mask.dtype == torch.uint8 and seen_mask.shape[1] == vocab
        assert seen_mask.is_contiguous()
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(lib.get("sampling").mstar_sample(
        logits.data_ptr(), logits.stride(0), rows, vocab, temperature.data_ptr(), _ptr(top_k),
        _ptr(top_p), _ptr(penalty), _ptr(seen_mask), _ptr(seen_rows), _ptr(seed), _ptr(offset),
        out.data_ptr(), _stream()), "sample")
    return out
