// Paged causal prefill attention in bfloat16 for portions of prompts: every entry of
// the batch brings q_len new tokens that attend to the entry's cached keys and to each
// other (causally), all read from the paged cache, where this step's keys already are.
//
// The rows of one (entry, kv head) are the pairs (token, query head of the group),
// token-major; a CTA takes 64 consecutive rows (four warps of 16) and streams the keys
// and values its rows can see through shared memory in tiles of 64 keys (cp.async, two
// stages).  S = Q K^T and O += P V are m16n8k16 tensor-core MMAs with float
// accumulation, the softmax is online and float, each row is masked by its own
// position (causal, end-aligned, optional window).  Packing the group into the rows
// lets any group size use full tiles and makes each key/value tile serve all query
// heads of the group.
//
// Semantics as attention_generic.cu; the reference uses a library here
// (mstar/utils/flashinfer_utils.py:136-156, 259-269).
#include <string.h>

#include "common.cuh"
#include "mma_util.cuh"
#include "tma_util.cuh"

#define PRE_THREADS 128
#define PRE_ROWS 64
#define PRE_TILE 64

struct PrefillArgs {
    const bf16* q;
    const bf16* kv;
    const int* block_table;
    const int* qo_indptr;
    const int* kv_len;
    bf16* out;
    int q_stride, bt_stride, nq, nkv, page_size, window, first_entry;
    float scale_log2e;
};

// Position (in elements) of 16-byte chunk c of key `row` in a key/value tile.  With TMA a
// tile is HD/64 halves of [64 keys x 64 features] with the hardware's 128-byte swizzle;
// with cp.async it is [64 keys x HD] with this file's own XOR swizzle.
template <int HD, bool TMA> __device__ __forceinline__ int kv_off(int row, int c) {
    if (TMA) return (c >> 3) * (64 * 64) + row * 64 + (((c & 7) ^ (row & 7)) << 3);
    return tile_off<HD / 8>(row, c);
}

// TMA = true: keys and values come by bulk tensor copies, one box of [page_size x 64] per
// page and 64-feature half, issued by one thread and awaited on an mbarrier (head_dim 64,
// 128 or 256, page size 8..64 dividing 64, no window).  TMA = false: every thread copies
// its 16-byte pieces with cp.async (any page size, windows).
template <int HD, bool TMA>
__global__ void __launch_bounds__(PRE_THREADS)
prefill_attention_kernel(const __grid_constant__ CUtensorMap kv_map, PrefillArgs a,
                         int* __restrict__ error_word) {
    constexpr int CPR = HD / 8;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* aligned = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    bf16* stages = reinterpret_cast<bf16*>(aligned);   // [2]{K [64][HD], V [64][HD]}, 1024-aligned
    bf16* Qs = stages + 2 * 2 * PRE_TILE * HD;         // [64][HD]
    __shared__ __align__(8) uint64_t full_bar[2];

    // the last row tiles see the most keys: schedule them first, so that the short tiles of
    // the prompt's start fill the tail of the grid
    const int tile = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y, e = a.first_entry + blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.nq / a.nkv;
    const int q_start = a.qo_indptr[e];
    const int q_len = a.qo_indptr[e + 1] - q_start;
    const int rows_total = q_len * G;
    const int row0 = tile * PRE_ROWS;
    if (row0 >= rows_total) return;
    const int past = a.kv_len[e] - q_len;  // cache position of the entry's first new token
    const int last_row = min(rows_total, row0 + PRE_ROWS) - 1;
    const int hi = past + last_row / G + 1;
    const int lo = a.window > 0 ? max(0, past + row0 / G - a.window + 1) : 0;

    const int* bt = a.block_table + (size_t)e * a.bt_stride;
    const size_t page_elems = (size_t)2 * a.nkv * a.page_size * HD;
    const size_t head_off = (size_t)kvh * a.page_size * HD;
    const size_t v_off = (size_t)a.nkv * a.page_size * HD;

    // ---- the 64 query rows -> shared
    for (int i = tid; i < PRE_ROWS * CPR; i += PRE_THREADS) {
        const int r = i / CPR, c = i - r * CPR;
        const int row = row0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows_total) {
            const int tok = q_start + row / G, head = kvh * G + row % G;
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)tok * a.q_stride + (size_t)head * HD + c * 8);
        }
        *reinterpret_cast<uint4*>(Qs + tile_off<CPR>(r, c)) = v;
    }

    if (TMA) {
        if (tid == 0) {
            mbar_init(tc_smem(&full_bar[0]), 1);
            mbar_init(tc_smem(&full_bar[1]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        // rows no copy fills must hold finite numbers (their probabilities are zero)
        for (int i = tid; i < 2 * 2 * PRE_TILE * HD / 8; i += PRE_THREADS)
            reinterpret_cast<uint4*>(stages)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
    }
    auto issue_tile = [&](int stage, int base) {  // TMA: one thread
        const int ps = a.page_size;
        const int pages = (min(hi, base + PRE_TILE) - base + ps - 1) / ps;
        const uint32_t bar = tc_smem(&full_bar[stage]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, (uint32_t)pages * ps * HD * 2 * 2);
        unsigned char* kdst = reinterpret_cast<unsigned char*>(stages) +
                              (size_t)stage * 2 * PRE_TILE * HD * 2;
        unsigned char* vdst = kdst + (size_t)PRE_TILE * HD * 2;
        for (int p = 0; p < pages; ++p) {
            const int page = bt[base / ps + p];
            const int krow = ((page * 2) * a.nkv + kvh) * ps;
            const int vrow = ((page * 2 + 1) * a.nkv + kvh) * ps;
#pragma unroll
            for (int h = 0; h < HD / 64; ++h) {
                const uint32_t off = (uint32_t)h * (64 * 128) + (uint32_t)p * ps * 128;
                tma_load_2d(tc_smem(kdst + off), &kv_map, bar, h * 64, krow);
                tma_load_2d(tc_smem(vdst + off), &kv_map, bar, h * 64, vrow);
            }
        }
    };
    auto load_tile = [&](int stage, int base) {
        bf16* Ks = stages + (size_t)stage * 2 * PRE_TILE * HD;
        bf16* Vs = Ks + PRE_TILE * HD;
        for (int i = tid; i < PRE_TILE * CPR; i += PRE_THREADS) {
            const int r = i / CPR, c = i - r * CPR;
            const int key = base + r;
            const bool ok = key < hi;
            const bf16* src = a.kv;
            if (ok) {
                const int pg = key / a.page_size;
                src = a.kv + (size_t)bt[pg] * page_elems + head_off +
                      (size_t)(key - pg * a.page_size) * HD + c * 8;
            }
            const int off = tile_off<CPR>(r, c);
            cp_async_16(smem_u32(Ks + off), src, ok ? 16 : 0);
            cp_async_16(smem_u32(Vs + off), ok ? src + v_off : src, ok ? 16 : 0);
        }
    };

    // this thread's two rows (g and g+8 of the warp's 16) and the keys they may see
    const int rowA = row0 + warp * 16 + (lane >> 2), rowB = rowA + 8;
    const int cpA = past + min(rowA, rows_total - 1) / G;
    const int cpB = past + min(rowB, rows_total - 1) / G;
    const int loA = a.window > 0 ? max(0, cpA - a.window + 1) : 0;
    const int loB = a.window > 0 ? max(0, cpB - a.window + 1) : 0;
    // the warp's rows together: newest key any row sees, oldest key any row sees
    const int warp_hi = past + min(row0 + warp * 16 + 15, rows_total - 1) / G;
    const int warp_lo = a.window > 0
                            ? max(0, past + min(row0 + warp * 16, rows_total - 1) / G - a.window + 1)
                            : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const int ntiles = (hi - lo + PRE_TILE - 1) / PRE_TILE;
    if (TMA) {
        if (tid == 0) issue_tile(0, lo);
    } else {
        load_tile(0, lo);
        cp_async_commit();
    }
    for (int it = 0; it < ntiles; ++it) {
        if (TMA) {
            if (tid == 0 && it + 1 < ntiles) issue_tile((it + 1) & 1, lo + (it + 1) * PRE_TILE);
            const bool arrived = mbar_wait(tc_smem(&full_bar[it & 1]), (uint32_t)(it >> 1) & 1u);
            if (!__syncthreads_and(arrived ? 1 : 0)) {  // a copy never completed
                if (tid == 0) atomicExch(error_word, 5);
                return;
            }
        } else {
            if (it + 1 < ntiles) load_tile((it + 1) & 1, lo + (it + 1) * PRE_TILE);
            cp_async_commit();
            cp_async_wait<1>();
            __syncthreads();
        }
        const bf16* Ks = stages + (size_t)(it & 1) * 2 * PRE_TILE * HD;
        const bf16* Vs = Ks + PRE_TILE * HD;
        const int base = lo + it * PRE_TILE;
        if (base <= warp_hi && base + PRE_TILE > warp_lo) {
            // ---- S[16 rows x 64 keys] = Q K^T
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t qa[4];
                const int arow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(qa, smem_u32(Qs + tile_off<CPR>(arow, 2 * kk + (lane >> 4))));
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {
                    uint32_t kb[4];
                    const int brow = jp * 16 + (lane & 7) + (lane >> 4) * 8;
                    ldmatrix_x4(kb, smem_u32(Ks + kv_off<HD, TMA>(brow, 2 * kk + ((lane >> 3) & 1))));
                    mma_bf16_16816(s[2 * jp], qa, kb[0], kb[1]);
                    mma_bf16_16816(s[2 * jp + 1], qa, kb[2], kb[3]);
                }
            }
            // ---- scale, mask each row by its own position, online softmax
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int key = base + j * 8 + (lane & 3) * 2 + (q4 & 1);
                    const bool upper = q4 < 2;
                    const bool ok = upper ? (key <= cpA && key >= loA) : (key <= cpB && key >= loB);
                    const float v = ok ? s[j][q4] * a.scale_log2e : -INFINITY;
                    s[j][q4] = v;
                    if (upper) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            // a row may have seen no key yet (all of this tile is masked for it)
            const float b0 = mn0 == -INFINITY ? 0.f : mn0, b1 = mn1 == -INFINITY ? 0.f : mn1;
            const float al0 = exp2f(m0 - b0), al1 = exp2f(m1 - b1);
            m0 = mn0;
            m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[j][0] = exp2f(s[j][0] - b0);
                s[j][1] = exp2f(s[j][1] - b0);
                s[j][2] = exp2f(s[j][2] - b1);
                s[j][3] = exp2f(s[j][3] - b1);
                ps0 += s[j][0] + s[j][1];
                ps1 += s[j][2] + s[j][3];
            }
            l0 = l0 * al0 + ps0;
            l1 = l1 * al1 + ps1;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1;
            }
            // ---- O[16 rows x HD] += P[16 x 64 keys] V[64 keys x HD]
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pa[4];
                pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < HD / 16; ++n2) {
                    uint32_t vb[4];
                    const int vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4_trans(vb, smem_u32(Vs + kv_off<HD, TMA>(vrow, 2 * n2 + (lane >> 4))));
                    mma_bf16_16816(o[2 * n2], pa, vb[0], vb[1]);
                    mma_bf16_16816(o[2 * n2 + 1], pa, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();
    }
    if (!TMA) cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
    if (rowA < rows_total) {
        const int tok = q_start + rowA / G, head = kvh * G + rowA % G;
        bf16* dst = a.out + (size_t)tok * a.nq * HD + (size_t)head * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) =
                __floats2bfloat162_rn(o[n][0] * inv0, o[n][1] * inv0);
    }
    if (rowB < rows_total) {
        const int tok = q_start + rowB / G, head = kvh * G + rowB % G;
        bf16* dst = a.out + (size_t)tok * a.nq * HD + (size_t)head * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) =
                __floats2bfloat162_rn(o[n][2] * inv1, o[n][3] * inv1);
    }
}

template <int HD, bool TMA>
static int launch_prefill(const CUtensorMap& map, const PrefillArgs& a, int entries, int max_q_len,
                          int* error_word, cudaStream_t s) {
    const size_t smem = (size_t)(PRE_ROWS * HD + 2 * 2 * PRE_TILE * HD) * sizeof(bf16) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<HD, TMA>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int G = a.nq / a.nkv;
    const long long tiles = ((long long)max_q_len * G + PRE_ROWS - 1) / PRE_ROWS;
    if (tiles > 2147483647LL) return -1;
    dim3 grid((unsigned)tiles, a.nkv, entries);
    prefill_attention_kernel<HD, TMA><<<grid, PRE_THREADS, smem, s>>>(map, a, error_word);
    return launch_status();
}

// Entries [first_entry, first_entry + entries) of the batch; qo_indptr and kv_len are
// indexed by entry, block_table rows too.  Returns 0, a CUDA error code, or -1 when
// the shape is refused (head_dim not one of 16/32/64/128/256).
// `kv_map`: the cache's tensor map (mstar_make_kv_tensor_map of the decode library) or
// null; with a map, no window and a page size of 8..64 that divides 64, keys and values
// are fetched by TMA.  `error_word`: device int, set to 5 if a TMA copy never completed.
MSTAR_API int mstar_paged_prefill_attention_bf16(
    const void* kv_map, const void* q, int q_stride, void* out, const void* kv_cache,
    const int* block_table, int bt_stride, const int* qo_indptr, const int* kv_len, int first_entry,
    int entries, int max_q_len, int nq, int nkv, int hd, int page_size, int window, float scale,
    int* error_word, void* stream) {
    if (entries <= 0 || max_q_len <= 0) return 0;
    if (nkv <= 0 || nq % nkv != 0 || entries > 65535 || nkv > 65535) return -1;
    PrefillArgs a;
    a.q = (const bf16*)q;
    a.kv = (const bf16*)kv_cache;
    a.block_table = block_table;
    a.qo_indptr = qo_indptr;
    a.kv_len = kv_len;
    a.out = (bf16*)out;
    a.q_stride = q_stride;
    a.bt_stride = bt_stride;
    a.nq = nq;
    a.nkv = nkv;
    a.page_size = page_size;
    a.window = window;
    a.first_entry = first_entry;
    a.scale_log2e = scale * 1.4426950408889634f;
    cudaStream_t s = (cudaStream_t)stream;
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    const bool tma = kv_map != nullptr && window == 0 && hd % 64 == 0 && page_size >= 8 &&
                     page_size <= 64 && PRE_TILE % page_size == 0 && error_word != nullptr;
    if (tma) {
        memcpy(&map, kv_map, sizeof(map));
        switch (hd) {
            case 64: return launch_prefill<64, true>(map, a, entries, max_q_len, error_word, s);
            case 128: return launch_prefill<128, true>(map, a, entries, max_q_len, error_word, s);
            case 256: return launch_prefill<256, true>(map, a, entries, max_q_len, error_word, s);
            default: return -1;
        }
    }
    switch (hd) {
        case 16: return launch_prefill<16, false>(map, a, entries, max_q_len, error_word, s);
        case 32: return launch_prefill<32, false>(map, a, entries, max_q_len, error_word, s);
        case 64: return launch_prefill<64, false>(map, a, entries, max_q_len, error_word, s);
        case 128: return launch_prefill<128, false>(map, a, entries, max_q_len, error_word, s);
        case 256: return launch_prefill<256, false>(map, a, entries, max_q_len, error_word, s);
        default: return -1;
    }
}
