// Split-K paged grouped-query decode attention in bfloat16: one query token per
// request, keys and values streamed from cache pages.
//
// The work of one (token, kv head) is cut along the keys into `splits` chunks; each
// CTA streams its chunk through shared memory in tiles of 64 keys (cp.async, two
// stages), its four warps take 16 keys each, compute S = Q K^T and O += P V with
// m16n8k16 tensor-core MMAs (the group of query heads padded to the 16 rows of the
// tile) and keep an online softmax in float.  Warps are merged in shared memory; if
// the keys were split, partial (max, sum, O) go to a scratch buffer and a second
// kernel merges them.  Decode attention is bound by the bytes of the cache, so the
// padded rows cost nothing that matters.
//
// Semantics are those of attention_generic.cu: scale, causal end-aligned mask,
// optional window, float softmax.  The reference calls a library for this
// (mstar/utils/flashinfer_utils.py:348-366, 452-465).
#include "common.cuh"
#include "mma_util.cuh"
#include "tma_util.cuh"
#include <stdlib.h>
#include <string.h>

#define DEC_THREADS 128
#define DEC_TILE 64

struct DecodeArgs {
    const bf16* q;
    const bf16* kv;
    const int* block_table;
    const int* token_req;
    const int* cache_pos;
    float* part_o;   // [tokens, nq, splits, HD]
    float* part_ml;  // [tokens, nq, splits, 2]
    bf16* out;       // [tokens, nq * HD]
    int q_stride, bt_stride, nq, nkv, page_size, window, chunk, splits;
    float scale_log2e;
    // > 0: the chunk is made on the device from the longest of these tokens' key ranges (see
    // live_chunk), `chunk` being its upper bound; 0: `chunk` as given
    int live_tokens;
    // nonzero: the caller promises that the kernel before this one on the stream wrote, of the
    // cache, nothing but each token's own key and value (the keys before them are from earlier
    // steps), and none of the index arrays
    int keys_static;
};

// The chunk that cuts the longest key range among the launch's tokens into `splits` equal
// parts, in whole tiles, at least 128 keys, at most the chunk the launch was sized for.  A
// launch replayed from a CUDA graph is sized for the longest range its block tables could
// hold; the ranges that are there may be half as long, and chunks cut for the bound would
// leave half of the splits empty.  Every warp of every CTA (and the merge kernel) computes
// the same value from the same array.
__device__ __forceinline__ int live_chunk(const DecodeArgs& a) {
    if (a.live_tokens <= 0) return a.chunk;
    int longest = 1;
    for (int i = threadIdx.x & 31; i < a.live_tokens; i += 32) longest = max(longest, a.cache_pos[i] + 1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o));
    const int c = max(128, ((longest + a.splits - 1) / a.splits + DEC_TILE - 1) / DEC_TILE * DEC_TILE);
    return min(c, a.chunk);
}

template <int HD>
__global__ void __launch_bounds__(DEC_THREADS) decode_attention_kernel(DecodeArgs a) {
    constexpr int CPR = HD / 8;  // 16-byte chunks per row
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);  // [16][HD]
    bf16* stages = Qs + 16 * HD;                   // [2]{K [64][HD], V [64][HD]}

    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.nq / a.nkv;

    const int hi = a.cache_pos[t] + 1;
    const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
    const int ks = lo + split * a.chunk;
    const int ke = min(hi, ks + a.chunk);
    if (ks >= ke) return;  // this token has fewer chunks than the launch has splits

    const int* bt = a.block_table + (size_t)a.token_req[t] * a.bt_stride;
    const size_t page_elems = (size_t)2 * a.nkv * a.page_size * HD;
    const size_t head_off = (size_t)kvh * a.page_size * HD;
    const size_t v_off = (size_t)a.nkv * a.page_size * HD;

    // ---- queries of the group -> shared, rows beyond the group are zero
    const bf16* qrow = a.q + (size_t)t * a.q_stride + (size_t)kvh * G * HD;
    for (int i = tid; i < 16 * CPR; i += DEC_THREADS) {
        const int r = i / CPR, c = i - r * CPR;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < G) v = *reinterpret_cast<const uint4*>(qrow + (size_t)r * HD + c * 8);
        *reinterpret_cast<uint4*>(Qs + tile_off<CPR>(r, c)) = v;
    }

    auto load_tile = [&](int stage, int base) {
        bf16* Ks = stages + (size_t)stage * 2 * DEC_TILE * HD;
        bf16* Vs = Ks + DEC_TILE * HD;
        for (int i = tid; i < DEC_TILE * CPR; i += DEC_THREADS) {
            const int r = i / CPR, c = i - r * CPR;
            const int key = base + r;
            const bool ok = key < ke;
            const bf16* src = a.kv;
            if (ok) {
                const int page = bt[key / a.page_size];
                const int slot = key - (key / a.page_size) * a.page_size;
                src = a.kv + (size_t)page * page_elems + head_off + (size_t)slot * HD + c * 8;
            }
            const int off = tile_off<CPR>(r, c);
            cp_async_16(smem_u32(Ks + off), src, ok ? 16 : 0);
            cp_async_16(smem_u32(Vs + off), ok ? src + v_off : src, ok ? 16 : 0);
        }
    };

    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g+8 of the tile

    const int ntiles = (ke - ks + DEC_TILE - 1) / DEC_TILE;
    load_tile(0, ks);
    cp_async_commit();
    for (int it = 0; it < ntiles; ++it) {
        if (it + 1 < ntiles) load_tile((it + 1) & 1, ks + (it + 1) * DEC_TILE);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* Ks = stages + (size_t)(it & 1) * 2 * DEC_TILE * HD;
        const bf16* Vs = Ks + DEC_TILE * HD;
        const int key0 = ks + it * DEC_TILE + warp * 16;  // first key of this warp's 16
        if (key0 < ke) {
            // ---- S[16 heads x 16 keys] = Q K^T
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t qa[4], kb[4];
                const int arow = (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(qa, smem_u32(Qs + tile_off<CPR>(arow, 2 * kk + (lane >> 4))));
                const int brow = warp * 16 + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(kb, smem_u32(Ks + tile_off<CPR>(brow, 2 * kk + ((lane >> 3) & 1))));
                mma_bf16_16816(s[0], qa, kb[0], kb[1]);
                mma_bf16_16816(s[1], qa, kb[2], kb[3]);
            }
            // ---- scale (log2 domain), mask the tail, online softmax per head row
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                    const float v = key < ke ? s[j][e] * a.scale_log2e : -INFINITY;
                    s[j][e] = v;
                    if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: key0 is valid
            const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
            m0 = mn0;
            m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[j][0] = exp2f(s[j][0] - mn0);
                s[j][1] = exp2f(s[j][1] - mn0);
                s[j][2] = exp2f(s[j][2] - mn1);
                s[j][3] = exp2f(s[j][3] - mn1);
                ps0 += s[j][0] + s[j][1];
                ps1 += s[j][2] + s[j][3];
            }
            l0 = l0 * al0 + ps0;
            l1 = l1 * al1 + ps1;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1;
            }
            // ---- O[16 heads x HD] += P[16 x 16 keys] V[16 keys x HD]
            uint32_t pa[4];
            pa[0] = pack_bf16(s[0][0], s[0][1]);
            pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]);
            pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
            for (int n2 = 0; n2 < HD / 16; ++n2) {
                uint32_t vb[4];
                const int vrow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(vb, smem_u32(Vs + tile_off<CPR>(vrow, 2 * n2 + (lane >> 4))));
                mma_bf16_16816(o[2 * n2], pa, vb[0], vb[1]);
                mma_bf16_16816(o[2 * n2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    // ---- merge the four warps (the stage buffers are free now)
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* Om = reinterpret_cast<float*>(stages);  // [4][16][HD]
    float* MLm = Om + 4 * 16 * HD;                 // [4][16][2]
    const int r0 = lane >> 2;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        float* p0 = Om + ((size_t)warp * 16 + r0) * HD + col;
        p0[0] = o[n][0];
        p0[1] = o[n][1];
        float* p1 = p0 + 8 * HD;
        p1[0] = o[n][2];
        p1[1] = o[n][3];
    }
    if ((lane & 3) == 0) {
        MLm[(warp * 16 + r0) * 2 + 0] = m0;
        MLm[(warp * 16 + r0) * 2 + 1] = l0;
        MLm[(warp * 16 + r0 + 8) * 2 + 0] = m1;
        MLm[(warp * 16 + r0 + 8) * 2 + 1] = l1;
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += DEC_THREADS) {
        const int g = idx / HD, d = idx - g * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, MLm[(w * 16 + g) * 2]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = MLm[(w * 16 + g) * 2];
            const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - m);
            acc += wgt * Om[((size_t)w * 16 + g) * HD + d];
            L += wgt * MLm[(w * 16 + g) * 2 + 1];
        }
        const int head = kvh * G + g;
        if (a.splits == 1) {
            a.out[(size_t)t * a.nq * HD + (size_t)head * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            const size_t slot = ((size_t)t * a.nq + head) * a.splits + split;
            a.part_o[slot * HD + d] = acc;
            if (d == 0) {
                a.part_ml[slot * 2] = m;
                a.part_ml[slot * 2 + 1] = L;
            }
        }
    }
}

// Merge the partial results of the splits of one (token, head): the first warp finds
// the overall maximum and each split's weight, then every thread sums its features.
#define MERGE_MAX_SPLITS 256
template <int HD>
__global__ void decode_merge_kernel(DecodeArgs a) {
    pdl_launch_dependents();   // a short kernel: the long one after it may be scheduled now
    __shared__ float wgt[MERGE_MAX_SPLITS];
    const int head = blockIdx.x, t = blockIdx.y;
    // the step's index arrays were there before the step's first kernel
    const int hi = a.cache_pos[t] + 1;
    const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
    const int chunk = live_chunk(a);               // every warp computes it (uniform)
    const int n = min(a.splits, (hi - lo + chunk - 1) / chunk);
    const size_t base = ((size_t)t * a.nq + head) * a.splits;
    pdl_wait();
    // a thread's features of the first splits are asked for together with the maxima and sums,
    // not after the weights are known: one round trip to memory instead of two
    constexpr int PD = (HD + 127) / 128, PS = 16;
    float po[PD][PS];
#pragma unroll
    for (int i = 0; i < PD; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
#pragma unroll
        for (int s = 0; s < PS; ++s) po[i][s] = (s < n && d < HD) ? a.part_o[(base + s) * HD + d] : 0.f;
    }
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m = -INFINITY;
        for (int s = lane; s < n; s += 32) m = fmaxf(m, a.part_ml[(base + s) * 2]);
        m = warp_max(m);
        float L = 0.f;
        for (int s = lane; s < n; s += 32) {
            const float w = exp2f(a.part_ml[(base + s) * 2] - m);
            wgt[s] = w;
            L += a.part_ml[(base + s) * 2 + 1] * w;
        }
        L = warp_sum(L);
        const float inv = 1.f / L;
        __syncwarp();
        for (int s = lane; s < n; s += 32) wgt[s] *= inv;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < PD; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        if (d >= HD) continue;
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < PS; ++s)
            if (s < n) acc = fmaf(po[i][s], wgt[s], acc);
        for (int s = PS; s < n; ++s) acc = fmaf(a.part_o[(base + s) * HD + d], wgt[s], acc);
        a.out[(size_t)t * a.nq * HD + (size_t)head * HD + d] = __float2bfloat16_rn(acc);
    }
}

template <int HD> static int launch_decode(const DecodeArgs& a, int tokens, cudaStream_t s) {
    const size_t smem = (size_t)(16 * HD + 2 * 2 * DEC_TILE * HD) * sizeof(bf16);
    static_assert((size_t)(4 * 16 * HD + 4 * 16 * 2) * sizeof(float) <=
                      (size_t)(2 * 2 * DEC_TILE * HD) * sizeof(bf16),
                  "merge buffer must fit in the stage buffers");
    static bool configured = false;  // once per head size: not repeated inside graph captures
    if (smem > 48 * 1024 && !configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(a.splits, a.nkv, tokens);
    decode_attention_kernel<HD><<<grid, DEC_THREADS, smem, s>>>(a);
    if (a.splits > 1) {
        dim3 mgrid(a.nq, tokens);
        mstar_launch((decode_merge_kernel<HD>), mgrid, dim3(HD < 32 ? 32 : (HD < 128 ? HD : 128)), 0, s, a);
    }
    return launch_status();
}

// ------------------------------------------------------------- TMA variant of the kernel
// Same arithmetic, other way of getting keys and values into shared memory: instead of
// every thread computing page addresses for its 16-byte pieces, one thread issues bulk
// tensor copies (TMA), one box of [page_size rows x 64 features] per page and 64-feature
// half, which land with the hardware's 128-byte swizzle and signal an mbarrier.  The
// cache is described as a matrix [(page, k/v, head, slot), head_dim] by a tensor map made
// on the host.  That takes the address arithmetic out of the instruction stream, which is
// what bounded the cp.async kernel.  Used when head_dim is 64, 128 or 256, the page size
// divides 64 and is at least 8, and there is no window (tiles then start on page
// boundaries); everything else takes the kernel above.
template <int HD> __device__ __forceinline__ int tma_off(int row, int c) {
    // element offset of 16-byte chunk c of key `row` in a tile stored as HD/64 halves of
    // [64 keys x 64 features], chunks XOR-swizzled by the row as TMA's SWIZZLE_128B does
    return (c >> 3) * (64 * 64) + row * 64 + ((((c & 7) ^ (row & 7))) << 3);
}

template <int HD>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap kv_map, DecodeArgs a,
                            int* __restrict__ error_word) {
    constexpr int CPR = HD / 8;
    constexpr int HALVES = HD / 64;
    constexpr uint32_t TILE_BYTES = DEC_TILE * HD * 2;  // keys (or values) of one tile
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* aligned = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    bf16* stages = reinterpret_cast<bf16*>(aligned);              // [2]{K, V}, 1024-aligned
    bf16* Qs = stages + 2 * 2 * DEC_TILE * HD;                    // [16][HD]
    __shared__ __align__(8) uint64_t full_bar[2];

    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.nq / a.nkv;
    const int hi = a.cache_pos[t] + 1;
    const int ks = split * a.chunk;
    const int ke = min(hi, ks + a.chunk);
    if (ks >= ke) return;
    const int* bt = a.block_table + (size_t)a.token_req[t] * a.bt_stride;
    const int ps = a.page_size;

    if (tid == 0) {
        mbar_init(tc_smem(&full_bar[0]), 1);
        mbar_init(tc_smem(&full_bar[1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const bf16* qrow = a.q + (size_t)t * a.q_stride + (size_t)kvh * G * HD;
    for (int i = tid; i < 16 * CPR; i += DEC_THREADS) {
        const int r = i / CPR, c = i - r * CPR;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < G) v = *reinterpret_cast<const uint4*>(qrow + (size_t)r * HD + c * 8);
        *reinterpret_cast<uint4*>(Qs + tile_off<CPR>(r, c)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    // Every tile is filled completely: pages beyond the request's last one are replaced by
    // that last page, so that rows whose keys are masked still hold finite numbers (their
    // probabilities are zero, but 0 * NaN is not) without clearing shared memory first.
    const int last_page = (hi - 1) / ps;
    auto issue_tile = [&](int stage, int base) {  // one thread
        const int npages = DEC_TILE / ps;
        const uint32_t bar = tc_smem(&full_bar[stage]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, 2 * TILE_BYTES);
        unsigned char* kdst = reinterpret_cast<unsigned char*>(stages) + (size_t)stage * 2 * TILE_BYTES;
        unsigned char* vdst = kdst + TILE_BYTES;
        for (int p = 0; p < npages; ++p) {
            const int page = bt[min(base / ps + p, last_page)];
            const int krow = ((page * 2) * a.nkv + kvh) * ps;
            const int vrow = ((page * 2 + 1) * a.nkv + kvh) * ps;
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
                const uint32_t off = (uint32_t)h * (64 * 128) + (uint32_t)p * ps * 128;
                tma_load_2d(tc_smem(kdst + off), &kv_map, bar, h * 64, krow);
                tma_load_2d(tc_smem(vdst + off), &kv_map, bar, h * 64, vrow);
            }
        }
    };

    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const int ntiles = (ke - ks + DEC_TILE - 1) / DEC_TILE;
    if (tid == 0) issue_tile(0, ks);
    bool alive = true;
    for (int it = 0; it < ntiles; ++it) {
        if (tid == 0 && it + 1 < ntiles) issue_tile((it + 1) & 1, ks + (it + 1) * DEC_TILE);
        const bool arrived = mbar_wait(tc_smem(&full_bar[it & 1]), (uint32_t)(it >> 1) & 1u);
        if (!__syncthreads_and(arrived ? 1 : 0)) {  // a copy never completed: give up together
            if (tid == 0) atomicExch(error_word, 4);
            alive = false;
            break;
        }
        const bf16* Ks = stages + (size_t)(it & 1) * 2 * DEC_TILE * HD;
        const bf16* Vs = Ks + DEC_TILE * HD;
        const int key0 = ks + it * DEC_TILE + warp * 16;
        if (key0 < ke) {
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t qa[4], kb[4];
                const int arow = (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(qa, smem_u32(Qs + tile_off<CPR>(arow, 2 * kk + (lane >> 4))));
                const int brow = warp * 16 + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(kb, smem_u32(Ks + tma_off<HD>(brow, 2 * kk + ((lane >> 3) & 1))));
                mma_bf16_16816(s[0], qa, kb[0], kb[1]);
                mma_bf16_16816(s[1], qa, kb[2], kb[3]);
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                    const float v = key < ke ? s[j][e] * a.scale_log2e : -INFINITY;
                    s[j][e] = v;
                    if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
            m0 = mn0;
            m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[j][0] = exp2f(s[j][0] - mn0);
                s[j][1] = exp2f(s[j][1] - mn0);
                s[j][2] = exp2f(s[j][2] - mn1);
                s[j][3] = exp2f(s[j][3] - mn1);
                ps0 += s[j][0] + s[j][1];
                ps1 += s[j][2] + s[j][3];
            }
            l0 = l0 * al0 + ps0;
            l1 = l1 * al1 + ps1;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1;
            }
            uint32_t pa[4];
            pa[0] = pack_bf16(s[0][0], s[0][1]);
            pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]);
            pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
            for (int n2 = 0; n2 < HD / 16; ++n2) {
                uint32_t vb[4];
                const int vrow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(vb, smem_u32(Vs + tma_off<HD>(vrow, 2 * n2 + (lane >> 4))));
                mma_bf16_16816(o[2 * n2], pa, vb[0], vb[1]);
                mma_bf16_16816(o[2 * n2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();  // everyone is done with this stage before it is filled again
    }
    if (!alive) return;

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* Om = reinterpret_cast<float*>(stages);
    float* MLm = Om + 4 * 16 * HD;
    const int r0 = lane >> 2;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        float* p0 = Om + ((size_t)warp * 16 + r0) * HD + col;
        p0[0] = o[n][0];
        p0[1] = o[n][1];
        float* p1 = p0 + 8 * HD;
        p1[0] = o[n][2];
        p1[1] = o[n][3];
    }
    if ((lane & 3) == 0) {
        MLm[(warp * 16 + r0) * 2 + 0] = m0;
        MLm[(warp * 16 + r0) * 2 + 1] = l0;
        MLm[(warp * 16 + r0 + 8) * 2 + 0] = m1;
        MLm[(warp * 16 + r0 + 8) * 2 + 1] = l1;
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += DEC_THREADS) {
        const int g = idx / HD, d = idx - g * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, MLm[(w * 16 + g) * 2]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = MLm[(w * 16 + g) * 2];
            const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - m);
            acc += wgt * Om[((size_t)w * 16 + g) * HD + d];
            L += wgt * MLm[(w * 16 + g) * 2 + 1];
        }
        const int head = kvh * G + g;
        if (a.splits == 1) {
            a.out[(size_t)t * a.nq * HD + (size_t)head * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            const size_t slot = ((size_t)t * a.nq + head) * a.splits + split;
            a.part_o[slot * HD + d] = acc;
            if (d == 0) {
                a.part_ml[slot * 2] = m;
                a.part_ml[slot * 2 + 1] = L;
            }
        }
    }
}

template <int HD>
static int launch_decode_tma(const CUtensorMap& map, const DecodeArgs& a, int tokens, int* error_word,
                             cudaStream_t s) {
    const size_t smem = (size_t)(16 * HD + 2 * 2 * DEC_TILE * HD) * sizeof(bf16) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_tma_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(a.splits, a.nkv, tokens);
    decode_attention_tma_kernel<HD><<<grid, DEC_THREADS, smem, s>>>(map, a, error_word);
    if (a.splits > 1) {
        dim3 mgrid(a.nq, tokens);
        mstar_launch((decode_merge_kernel<HD>), mgrid, dim3(HD < 128 ? HD : 128), 0, s, a);
    }
    return launch_status();
}

// ------------------------------------------------------------- persistent ring variant
// The same tiles and arithmetic once more, with the launch turned inside out: the grid is
// what fits on the GPU at once, every CTA walks over work items (token, kv head, split),
// and two producer warps (one for the keys, one for the values) keep a ring of key/value
// tiles filled across item boundaries, so that the copies of the next item are in flight
// while this one is computed.  With one
// CTA per item a CTA lives for a launch plus two or three DRAM latencies, and at small
// batches most of a decode step's attention time was that; here the latencies overlap.
// A producer's lanes fetch 32 block-table entries at a time and issue the copies of a
// tile side by side (its loop has no division and no exchange but the page numbers: with
// few tiles per CTA its length is the CTA's pace); the four consumer warps take 16 keys of a tile each, as above, and
// are merged in shared memory at the end of an item.
#define RING_THREADS (DEC_THREADS + 64)   // four consumer warps, a copy warp for the keys, one for the values

struct RingLayout {   // byte offsets into dynamic shared memory, made on the host
    int stages, q_off, om_off, ml_off, bar_off, total;
};

template <int HD>
__global__ void __launch_bounds__(RING_THREADS)
decode_attention_ring_kernel(const __grid_constant__ CUtensorMap kv_map, DecodeArgs a, int tokens,
                             RingLayout lay, int* __restrict__ error_word) {
    // With `keys_static` the kernel before this one wrote the queries and each token's own key
    // and value, and nothing else that is read here: the keys before them were written by
    // earlier steps and the step's index arrays before its first kernel.  The copies of all
    // tiles but a token's last then start at once, while that kernel is still draining, and
    // only the consumers and the last tile wait for it.
    if (!a.keys_static) pdl_wait();
    constexpr int CPR = HD / 8;
    constexpr int HALVES = HD / 64;
    constexpr uint32_t TILE_BYTES = DEC_TILE * HD * 2;  // keys (or values) of one tile
    extern __shared__ __align__(1024) unsigned char ring_smem[];
    unsigned char* ring = ring_smem;                                  // [stages]{K, V}
    bf16* Qs = reinterpret_cast<bf16*>(ring_smem + lay.q_off);        // [16][HD]
    float* Om = reinterpret_cast<float*>(ring_smem + lay.om_off);     // [4 warps][G][HD]
    float* MLm = reinterpret_cast<float*>(ring_smem + lay.ml_off);    // [4 warps][G][2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_smem + lay.bar_off);
    const int S = lay.stages;
    const uint32_t full = tc_smem(bars), empty = tc_smem(bars + S);
    volatile int* failed = reinterpret_cast<volatile int*>(bars + 2 * S);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.nq / a.nkv;
    const int ps = a.page_size;
    const int items = tokens * a.nkv * a.splits;
    const int chunk = live_chunk(a);

    if ((tc_smem(ring_smem) & 1023u) != 0) {          // the swizzled tiles need this alignment
        if (tid == 0) atomicExch(error_word, 5);
        return;
    }
    if (tid == 0) {
        *failed = 0;
        for (int s = 0; s < S; ++s) {
            mbar_init(full + 8 * s, 2);                     // the keys' warp and the values'
            mbar_init(empty + 8 * s, DEC_THREADS / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp >= DEC_THREADS / 32) {
        // ----------------------------------------- producers: a warp for the keys, one for the values
        // st: the ring's stage, round: how often the ring has been filled before (counted, not
        // divided: the loop is the pace of a CTA with few tiles); page sizes are powers of two
        const int which = warp - DEC_THREADS / 32;
        int st = 0, round = 0;
        const int ps_log = 31 - __clz(ps);
        bool ok = true, waited = !a.keys_static;
        for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
            const int split = item % a.splits, kvh = (item / a.splits) % a.nkv, t = item / (a.splits * a.nkv);
            const int hi = a.cache_pos[t] + 1;
            const int ks = split * chunk;
            const int ke = min(hi, ks + chunk);
            if (ks >= ke) continue;
            const int* bt = a.block_table + (size_t)a.token_req[t] * a.bt_stride;
            // pages beyond the request's last one are replaced by it: masked keys stay finite
            const int last_page = (hi - 1) >> ps_log;
            // a tile is DEC_TILE / ps whole pages, or, with pages of 128 or 256 keys, a part of one
            const int per_tile = ps < DEC_TILE ? DEC_TILE >> ps_log : 1;
            const int box_rows = ps < DEC_TILE ? ps : DEC_TILE;
            const int ntiles = (ke - ks + DEC_TILE - 1) / DEC_TILE;
            int mine = 0, have_from = -1;              // lanes hold pages have_from .. +31
            const int p = lane / HALVES, h = lane % HALVES;   // this lane's page and block of a tile
            for (int it = 0; it < ntiles; ++it) {
                const int key0 = ks + it * DEC_TILE;
                if (!waited && key0 + DEC_TILE >= hi) {   // the tile with the token's own key
                    pdl_wait();
                    waited = true;
                }
                const int base_page = key0 >> ps_log;
                if (have_from < 0 || base_page + per_tile > have_from + 32) {
                    have_from = base_page;
                    mine = bt[min(base_page + lane, last_page)];
                }
                // lane HALVES p + h waits for the stage and copies 64-feature block h of page p
                const int page = __shfl_sync(0xffffffffu, mine, (base_page + p - have_from) & 31);
                if (p < per_tile) {
                    if (round > 0 && !mbar_wait(empty + 8 * st, ((uint32_t)round - 1u) & 1u)) {
                        atomicExch(error_word, 4);
                        ok = false;
                    } else {
                        // the bytes may land before lane 0 has announced them: the phase cannot
                        // end before the two warps' arrivals
                        if (lane == 0) mbar_expect_tx(full + 8 * st, TILE_BYTES);
                        unsigned char* dst = ring + (size_t)st * 2 * TILE_BYTES + which * TILE_BYTES +
                                             h * (64 * 128) + p * box_rows * 128;
                        const int in_page = key0 & (ps - 1);   // 0 unless the page is larger than the tile
                        tma_load_2d(tc_smem(dst), &kv_map, full + 8 * st, h * 64,
                                    ((page * 2 + which) * a.nkv + kvh) * ps + in_page);
                    }
                }
                if (!__all_sync(0xffffffffu, ok)) {
                    ok = false;
                    break;
                }
                if (++st == S) {
                    st = 0;
                    ++round;
                }
            }
        }
        pdl_launch_dependents();          // the last keys are asked for
        return;
    }

    // ---------------------------------------------------------------------- consumers
    if (a.keys_static) pdl_wait();        // the queries are the output of the kernel before
    int st = 0, round = 0;                // as the producer counts them
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int split = item % a.splits, kvh = (item / a.splits) % a.nkv, t = item / (a.splits * a.nkv);
        const int hi = a.cache_pos[t] + 1;
        const int ks = split * chunk;
        const int ke = min(hi, ks + chunk);
        if (ks >= ke) continue;   // this token has fewer chunks than the launch has splits
        // the last item's Q and merge buffers are free: every warp is past its last barrier
        const bf16* qrow = a.q + (size_t)t * a.q_stride + (size_t)kvh * G * HD;
        for (int i = tid; i < 16 * CPR; i += DEC_THREADS) {
            const int r = i / CPR, cc = i - r * CPR;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < G) v = *reinterpret_cast<const uint4*>(qrow + (size_t)r * HD + cc * 8);
            *reinterpret_cast<uint4*>(Qs + tile_off<CPR>(r, cc)) = v;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(DEC_THREADS) : "memory");

        float o[HD / 8][4];
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        const int ntiles = (ke - ks + DEC_TILE - 1) / DEC_TILE;
        for (int it = 0; it < ntiles; ++it) {
            // one outcome for the warp: the matrix instructions below are warp-wide
            if (!__all_sync(0xffffffffu, mbar_wait(full + 8 * st, (uint32_t)round & 1u))) {
                // give up, but together with the other warps (they wait at the barrier below)
                if (lane == 0) atomicExch(error_word, 4);
                *failed = 1;
                break;
            }
            const bf16* Ks = reinterpret_cast<const bf16*>(ring + (size_t)st * 2 * TILE_BYTES);
            const bf16* Vs = Ks + DEC_TILE * HD;
            const int key0 = ks + it * DEC_TILE + warp * 16;
            if (key0 < ke) {
                float s[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    uint32_t qa[4], kb[4];
                    const int arow = (lane & 7) + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(qa, smem_u32(Qs + tile_off<CPR>(arow, 2 * kk + (lane >> 4))));
                    const int brow = warp * 16 + (lane & 7) + (lane >> 4) * 8;
                    ldmatrix_x4(kb, smem_u32(Ks + tma_off<HD>(brow, 2 * kk + ((lane >> 3) & 1))));
                    mma_bf16_16816(s[0], qa, kb[0], kb[1]);
                    mma_bf16_16816(s[1], qa, kb[2], kb[3]);
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                        const float v = key < ke ? s[j][e] * a.scale_log2e : -INFINITY;
                        s[j][e] = v;
                        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                    }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: key0 is valid
                const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
                m0 = mn0;
                m1 = mn1;
                float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    s[j][0] = exp2f(s[j][0] - mn0);
                    s[j][1] = exp2f(s[j][1] - mn0);
                    s[j][2] = exp2f(s[j][2] - mn1);
                    s[j][3] = exp2f(s[j][3] - mn1);
                    ps0 += s[j][0] + s[j][1];
                    ps1 += s[j][2] + s[j][3];
                }
                l0 = l0 * al0 + ps0;
                l1 = l1 * al1 + ps1;
#pragma unroll
                for (int n = 0; n < HD / 8; ++n) {
                    o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1;
                }
                uint32_t pa[4];
                pa[0] = pack_bf16(s[0][0], s[0][1]);
                pa[1] = pack_bf16(s[0][2], s[0][3]);
                pa[2] = pack_bf16(s[1][0], s[1][1]);
                pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
                for (int n2 = 0; n2 < HD / 16; ++n2) {
                    uint32_t vb[4];
                    const int vrow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4_trans(vb, smem_u32(Vs + tma_off<HD>(vrow, 2 * n2 + (lane >> 4))));
                    mma_bf16_16816(o[2 * n2], pa, vb[0], vb[1]);
                    mma_bf16_16816(o[2 * n2 + 1], pa, vb[2], vb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty + 8 * st) : "memory");
            }
            if (++st == S) {
                st = 0;
                ++round;
            }
        }

        if (item + (int)gridDim.x >= items) pdl_launch_dependents();   // the last keys are here
        // ---- the warps' parts of the keys -> shared (rows of the group only), then merged
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const int r0 = lane >> 2;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            const int col = n * 8 + (lane & 3) * 2;
            if (r0 < G) {
                float* p0 = Om + ((size_t)warp * G + r0) * HD + col;
                p0[0] = o[n][0];
                p0[1] = o[n][1];
            }
            if (r0 + 8 < G) {
                float* p1 = Om + ((size_t)warp * G + r0 + 8) * HD + col;
                p1[0] = o[n][2];
                p1[1] = o[n][3];
            }
        }
        if ((lane & 3) == 0) {
            if (r0 < G) {
                MLm[(warp * G + r0) * 2 + 0] = m0;
                MLm[(warp * G + r0) * 2 + 1] = l0;
            }
            if (r0 + 8 < G) {
                MLm[(warp * G + r0 + 8) * 2 + 0] = m1;
                MLm[(warp * G + r0 + 8) * 2 + 1] = l1;
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(DEC_THREADS) : "memory");
        if (*failed) return;
        for (int idx = tid; idx < G * HD; idx += DEC_THREADS) {
            const int g = idx / HD, d = idx - g * HD;
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) m = fmaxf(m, MLm[(w * G + g) * 2]);
            float acc = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = MLm[(w * G + g) * 2];
                const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - m);
                acc += wgt * Om[((size_t)w * G + g) * HD + d];
                L += wgt * MLm[(w * G + g) * 2 + 1];
            }
            const int head = kvh * G + g;
            if (a.splits == 1) {
                a.out[(size_t)t * a.nq * HD + (size_t)head * HD + d] = __float2bfloat16_rn(acc / L);
            } else {
                const size_t slot = ((size_t)t * a.nq + head) * a.splits + split;
                a.part_o[slot * HD + d] = acc;
                if (d == 0) {
                    a.part_ml[slot * 2] = m;
                    a.part_ml[slot * 2 + 1] = L;
                }
            }
        }
        // Q and the merge buffers are written again only after every warp has passed this
        asm volatile("bar.sync 1, %0;" ::"n"(DEC_THREADS) : "memory");
    }
}

// Shared memory of the ring kernel for a group of G query heads: as many stages (3 or 2) as
// leave room for two CTAs per SM.
template <int HD> static RingLayout ring_layout(int G, int stages) {
    RingLayout l;
    l.stages = stages;
    l.q_off = stages * 2 * DEC_TILE * HD * 2;
    l.om_off = l.q_off + 16 * HD * 2;
    l.ml_off = l.om_off + 4 * G * HD * 4;
    l.bar_off = (l.ml_off + 4 * G * 2 * 4 + 7) & ~7;
    l.total = l.bar_off + (2 * stages + 1) * 8;
    return l;
}

template <int HD>
static int launch_decode_ring(const CUtensorMap& map, const DecodeArgs& a, int tokens, int* error_word,
                              cudaStream_t s) {
    const int G = a.nq / a.nkv;
    static int sms = 0, max_smem = 0, configured_for = 0;
    auto kernel = decode_attention_ring_kernel<HD>;
    if (sms == 0) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev)) != cudaSuccess)
            return (int)e;
    }
    // 3 stages if two such CTAs fit on an SM (1 KB per CTA is the system's), else 2; one CTA
    // per SM if even that is too much (head_dim 256)
    RingLayout lay = ring_layout<HD>(G, 3);
    int per_sm = 2;
    if (2 * (lay.total + 1024) > max_smem) {
        lay = ring_layout<HD>(G, 2);
        if (2 * (lay.total + 1024) > max_smem) per_sm = 1;
    }
    if (lay.total + 1024 > max_smem) return -1;
    if (lay.total > configured_for) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lay.total);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured_for = lay.total;
    }
    const long long items = (long long)tokens * a.nkv * a.splits;
    if (items > 2147483647LL) return -1;
    DecodeArgs live = a;
    live.live_tokens = tokens;
    static int occ_for = -1, occ = 0;   // registers may allow fewer CTAs than shared memory does
    if (occ_for != lay.total) {
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, RING_THREADS, lay.total);
        if (e != cudaSuccess) return (int)e;
        if (occ < 1) return -1;
        occ_for = lay.total;
    }
    if (occ < per_sm) per_sm = occ;
    const int resident = per_sm * sms;
    const int grid = items < resident ? (int)items : resident;
    mstar_launch(kernel, dim3(grid), dim3(RING_THREADS), lay.total, s, map, live, tokens, lay, error_word);
    if (a.splits > 1) {
        dim3 mgrid(a.nq, tokens);
        mstar_launch((decode_merge_kernel<HD>), mgrid, dim3(HD < 128 ? HD : 128), 0, s, live);
    }
    return launch_status();
}

// Tensor map of a cache [pages, 2, nkv, page_size, hd] (bfloat16) seen as the matrix
// [pages * 2 * nkv * page_size, hd] with boxes of min(page_size, 64) rows x 64 features,
// 128-byte swizzle; page sizes 8..64 that divide 64, 128 and 256.  `out_map` receives the 128-byte map.  Returns 0, -1 (shape not taken), -3 / -4.
MSTAR_API int mstar_make_kv_tensor_map(void* out_map, const void* kv_cache, long long pages, int nkv,
                                       int page_size, int hd) {
    const bool small_page = page_size >= 8 && page_size <= 64 && DEC_TILE % page_size == 0;
    if (hd % 64 != 0 || hd > 256 || !(small_page || page_size == 128 || page_size == 256)) return -1;
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return -3;
    const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)pages * 2 * nkv * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)(page_size < DEC_TILE ? page_size : DEC_TILE)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(reinterpret_cast<CUtensorMap*>(out_map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                          const_cast<void*>(kv_cache), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -4;
}

// The TMA variant: `kv_map` from mstar_make_kv_tensor_map for this cache; no window.
// `error_word`: device int, set to 4 if a copy's barrier never completed.  `keys_static`:
// nonzero promises that the kernel before this one on the stream wrote nothing that is read
// here but the queries and each token's own key and value (see DecodeArgs).
MSTAR_API int mstar_paged_decode_attention_bf16_tma(
    const void* kv_map, const void* q, int q_stride, void* out, const void* kv_cache,
    const int* block_table, int bt_stride, const int* token_req, const int* cache_pos, int tokens,
    int nq, int nkv, int hd, int page_size, float scale, int chunk, int splits, int keys_static,
    float* scratch, int* error_word, void* stream) {
    if (tokens <= 0) return 0;
    if (nkv <= 0 || nq % nkv != 0 || nq / nkv > 16) return -1;
    if (chunk <= 0 || chunk % DEC_TILE != 0 || splits < 1 || splits > MERGE_MAX_SPLITS) return -1;
    if (splits > 1 && scratch == nullptr) return -1;
    if (tokens > 65535 || nkv > 65535) return -1;
    const bool small_page = page_size >= 8 && page_size <= 64 && DEC_TILE % page_size == 0;
    if (!(small_page || page_size == 128 || page_size == 256)) return -1;
    DecodeArgs a;
    a.q = (const bf16*)q;
    a.kv = (const bf16*)kv_cache;
    a.block_table = block_table;
    a.token_req = token_req;
    a.cache_pos = cache_pos;
    a.part_o = scratch;
    a.part_ml = scratch ? scratch + (size_t)tokens * nq * splits * hd : nullptr;
    a.out = (bf16*)out;
    a.q_stride = q_stride;
    a.bt_stride = bt_stride;
    a.nq = nq;
    a.nkv = nkv;
    a.page_size = page_size;
    a.window = 0;
    a.chunk = chunk;
    a.splits = splits;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.live_tokens = 0;
    a.keys_static = keys_static;
    CUtensorMap map;
    memcpy(&map, kv_map, sizeof(map));
    cudaStream_t s = (cudaStream_t)stream;
    static int per_item = -1;   // MSTAR_DECODE_ATTENTION=per_item: one CTA per work item
    if (per_item < 0) {
        const char* e = getenv("MSTAR_DECODE_ATTENTION");
        per_item = (e != nullptr && strcmp(e, "per_item") == 0) ? 1 : 0;
    }
    if (per_item) {
        if (!small_page) return -1;       // that kernel copies whole pages
        switch (hd) {
            case 64: return launch_decode_tma<64>(map, a, tokens, error_word, s);
            case 128: return launch_decode_tma<128>(map, a, tokens, error_word, s);
            case 256: return launch_decode_tma<256>(map, a, tokens, error_word, s);
            default: return -1;
        }
    }
    switch (hd) {
        case 64: return launch_decode_ring<64>(map, a, tokens, error_word, s);
        case 128: return launch_decode_ring<128>(map, a, tokens, error_word, s);
        case 256: return launch_decode_ring<256>(map, a, tokens, error_word, s);
        default: return -1;
    }
}

// Scratch floats needed for `tokens` query tokens cut into `splits` chunks.
MSTAR_API long long mstar_decode_attention_scratch_floats(int tokens, int nq, int hd, int splits) {
    return splits <= 1 ? 0 : (long long)tokens * nq * splits * (hd + 2);
}

// Returns 0, a CUDA error code, or -1 when the shape is refused (head_dim not one of
// 16/32/64/128/256, more than 16 query heads per kv head, chunk no multiple of 64).
MSTAR_API int mstar_paged_decode_attention_bf16(
    const void* q, int q_stride, void* out, const void* kv_cache, const int* block_table,
    int bt_stride, const int* token_req, const int* cache_pos, int tokens, int nq, int nkv, int hd,
    int page_size, int window, float scale, int chunk, int splits, float* scratch, void* stream) {
    if (tokens <= 0) return 0;
    if (nkv <= 0 || nq % nkv != 0 || nq / nkv > 16) return -1;
    if (chunk <= 0 || chunk % DEC_TILE != 0 || splits < 1 || splits > MERGE_MAX_SPLITS) return -1;
    if (splits > 1 && scratch == nullptr) return -1;
    if (tokens > 65535 || nkv > 65535) return -1;
    DecodeArgs a;
    a.q = (const bf16*)q;
    a.kv = (const bf16*)kv_cache;
    a.block_table = block_table;
    a.token_req = token_req;
    a.cache_pos = cache_pos;
    a.part_o = scratch;
    a.part_ml = scratch ? scratch + (size_t)tokens * nq * splits * hd : nullptr;
    a.out = (bf16*)out;
    a.q_stride = q_stride;
    a.bt_stride = bt_stride;
    a.nq = nq;
    a.nkv = nkv;
    a.page_size = page_size;
    a.window = window;
    a.chunk = chunk;
    a.splits = splits;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.live_tokens = 0;
    a.keys_static = 0;
    cudaStream_t s = (cudaStream_t)stream;
    switch (hd) {
        case 16: return launch_decode<16>(a, tokens, s);
        case 32: return launch_decode<32>(a, tokens, s);
        case 64: return launch_decode<64>(a, tokens, s);
        case 128: return launch_decode<128>(a, tokens, s);
        case 256: return launch_decode<256>(a, tokens, s);
        default: return -1;
    }
}
