// y[M,N] = x[M,K] W[N,K]^T for few rows (M <= 16), bfloat16 in, float accumulation, with
// the weights brought by bulk asynchronous copies (cp.async.bulk, global -> shared, mbarrier
// completion) instead of register loads.
//
// Why: at these sizes the time of a product is the time to stream W once from HBM, and with
// register loads a warp has at most a few kilobytes in flight, so a CTA lives through
// several rounds of DRAM latency and the narrow projections (N = 3072 .. 5120) reach 40 %
// of the memory bandwidth.  Here one lane asks for a CTA's rows as whole row segments of up
// to 2 KB, three stages deep; with four CTAs on an SM about 200 KB per SM are in flight from
// the first microsecond on, which is several times the latency-bandwidth product, and the
// consumer warps only ever wait for data that is already on its way.
//
// A CTA owns strips of 8 NT output features (8 NT rows of W; twice that for the fused gate/up
// form: rows n and inter + n) and walks over its strips (grid = at most what is resident at
// once, cut so that every CTA takes the same number of strips; further strips are taken in
// further turns without draining the ring).  NT is 1, 2 or 4:
// the more rows share one read of x, the less traffic x causes (with 8 tokens and NT = 1 it
// equals the traffic of W), so wide matrices, which have strips enough, take larger ones.
// The bytes in flight per SM stay near 200 KB: 4, 2 or 1 CTAs per SM.  The K range of a strip is cut
// into chunks of `KC` elements; a stage of the ring holds one chunk of every row, rows 64
// bytes more than a chunk apart, which makes the 16-byte fragment reads free of bank
// conflicts.  Eight consumer warps take the 32-element blocks of a chunk in turn, read their
// fragments from shared memory (W rows as the 8-wide N of m16n8k16, the tokens as its M, k
// assigned to threads so that 16 consecutive bytes of a row are one thread's: permuted alike
// in both operands) and x from global memory (it is small and stays
// in L1/L2), and are summed through shared memory at the end of a strip.
//
// A third form is the attention mixer's first product for decoded tokens: y = x Wqkv^T with
// the rotary encoding of q and k and the write of k and v into their cache pages done where
// the sums are made.  A strip then holds rows j .. j + 8 NT - 1 and hd/2 + the same of one
// head, the two halves of 8 NT rotated pairs (the gated form's row layout with another
// distance), so both partners of a pair meet in one thread; q leaves rotated, k and v go to
// (page, slot) of the token's cache position and nowhere else.  Arithmetic as in the separate
// kernel (elementwise.cu): sums rounded to bfloat16, angle = float(position) * inv_freq[j],
// sincosf, rotation in float.
//
// Every mbarrier wait is bounded; a wait that runs out sets the error word (13 producer, 14
// consumer) and the CTA leaves (the consumer warps together, after their next barrier).
// The reference uses the library GEMM for these products
// (mstar/model/components/distributed/linear.py:101, mlp.py:78-81 for the gated form).
#include <stdlib.h>

#include "common.cuh"
#include "mma_util.cuh"
#include "tma_util.cuh"

#define SB_WARPS 8                       // consumer warps
#define SB_THREADS ((SB_WARPS + 1) * 32) // + the producer warp
#define SB_STAGES 3
#define SB_KC 1024                       // elements of K per chunk
#define SB_PAD 64                        // bytes between the end of a row's chunk and the next row

template <typename T> __device__ __forceinline__ void sb_store(T* p, float v);
template <> __device__ __forceinline__ void sb_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void sb_store<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void sb_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// the forms of the kernel; the last two have two 8 NT-row groups per strip
#define SB_PLAIN 0
#define SB_GATED 1
#define SB_ROPE 2

// what the rotary form needs beside the product's operands
struct SbRope {
    const int* positions;    // [M] position of a token for the angles
    const int* cache_pos;    // [M] its place in its request's cache
    const int* token_req;    // [M] row of the block table
    const int* block_table;
    const float* inv_freq;   // [hd / 2]
    bf16* kv_cache;          // [pages, 2, nkv, page_size, hd]
    int nq, nkv, hd, page_size, bt_stride;
};

__host__ __device__ constexpr int sb_rows(bool gated, int nt) { return (gated ? 16 : 8) * nt; }
__host__ __device__ constexpr int sb_pitch() { return SB_KC * 2 + SB_PAD; }
__host__ __device__ constexpr int sb_stage_bytes(bool gated, int nt) { return sb_rows(gated, nt) * sb_pitch(); }
// ring, the warps' partial sums [row groups][warps][16][8], barriers
__host__ __device__ constexpr int sb_smem(bool gated, int nt) {
    return SB_STAGES * sb_stage_bytes(gated, nt) + (gated ? 2 : 1) * nt * SB_WARPS * 16 * 8 * 4 + 64;
}

// M16: tokens 8..15 exist (else the upper half of the MMA's rows is zero)
// first output feature of a strip
template <int MODE, int NT>
__device__ __forceinline__ int sb_strip_n0(int strip, const SbRope& rp) {
    if (MODE != SB_ROPE) return strip * 8 * NT;
    const int per_head = (rp.hd / 2) / (8 * NT);
    const int h = strip / per_head;
    return h * rp.hd + (strip - h * per_head) * 8 * NT;
}

template <int MODE, bool M16, int NT, typename OutT>
__global__ void __launch_bounds__(SB_THREADS, (MODE ? 2 : 4) / NT >= 1 ? (MODE ? 2 : 4) / NT : 1)
smallm_bulk_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, OutT* __restrict__ out, int M,
                   int n_out, int K, int ldx, int ldw, int ldo, int inter, int w_static,
                   int* __restrict__ error_word, SbRope rp) {
    constexpr bool GATED = MODE != SB_PLAIN;          // two row groups per strip
    constexpr int STRIPS = GATED ? 2 : 1;
    constexpr int GROUPS = STRIPS * NT;               // 8-row groups of a stage
    constexpr int ROWS = 8 * GROUPS;
    constexpr int PITCH = sb_pitch();
    constexpr int STAGE = sb_stage_bytes(GATED, NT);
    extern __shared__ __align__(128) unsigned char sb_smem_raw[];
    unsigned char* ring = sb_smem_raw;
    float* red = reinterpret_cast<float*>(ring + SB_STAGES * STAGE);           // [GROUPS][warps][16][8]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + GROUPS * SB_WARPS * 128);
    const uint32_t full = tc_smem(bars), empty = tc_smem(bars + SB_STAGES);     // [SB_STAGES] each
    volatile int* failed = reinterpret_cast<volatile int*>(bars + 2 * SB_STAGES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nstrips = MODE == SB_ROPE ? n_out / (16 * NT) : (n_out + 8 * NT - 1) / (8 * NT);
    const int nch = (K + SB_KC - 1) / SB_KC;

    if (tid == 0) {
        *failed = 0;
        for (int s = 0; s < SB_STAGES; ++s) {
            mbar_init(full + 8 * s, 1);
            mbar_init(empty + 8 * s, SB_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == SB_WARPS) {
        // ------------------------------------------------------------------ producer
        // Weights that nothing writes while the engine runs are asked for at once, while the
        // kernel before this one is still draining; otherwise W is the output of some kernel
        // like x, and the copies wait for it.
        if (!w_static) pdl_wait();
        // lane r asks for row r of the stage: rows n0 .. n0 + 8 NT - 1 (and inter + the same)
        int c = 0;
        bool ok = true;
        for (int strip = blockIdx.x; strip < nstrips && ok; strip += gridDim.x) {
            const int n0 = sb_strip_n0<MODE, NT>(strip, rp);
            const int row = min(n0 + lane % (8 * NT), n_out - 1) + (lane / (8 * NT)) * inter;
            const bf16* src_row = W + (size_t)(lane < ROWS ? row : 0) * ldw;
            for (int ch = 0; ch < nch; ++ch, ++c) {
                const int st = c % SB_STAGES;
                const uint32_t bytes = (uint32_t)min(SB_KC, K - ch * SB_KC) * 2;
                if (lane == 0) {
                    if (c >= SB_STAGES && !mbar_wait(empty + 8 * st, ((uint32_t)(c / SB_STAGES) - 1u) & 1u)) {
                        atomicExch(error_word, 13);
                        ok = false;
                    } else {
                        mbar_expect_tx(full + 8 * st, bytes * ROWS);
                    }
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                if (!ok) break;
                if (lane < ROWS)
                    bulk_load(tc_smem(ring + st * STAGE + lane * PITCH), src_row + (size_t)ch * SB_KC, bytes,
                              full + 8 * st);
            }
        }
        pdl_launch_dependents();          // the last weights are asked for
        return;
    }

    // ---------------------------------------------------------------------- consumers
    // x is the output of the kernel before: its addresses are formed from the wait's result and
    // it is read with ordinary loads (a kernel launched early lives while x is being written,
    // which loads of never-changing memory, __ldg, do not allow)
    x = pdl_after(x, pdl_wait());
    const int g = lane >> 2, t = lane & 3;
    const bf16* xa = x + (size_t)min(g, M - 1) * ldx + 8 * t;
    const bf16* xb = x + (size_t)min(g + 8, M - 1) * ldx + 8 * t;
    // this warp's blocks of a chunk: warp, warp + 8, ...  (at most 4 of 32)
    constexpr int PER = SB_KC / 32 / SB_WARPS;
    auto load_x = [&](int ch, uint4 (&xv)[PER], uint4 (&xw)[PER]) {
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int k = ch * SB_KC + (warp + u * SB_WARPS) * 32;
            xv[u] = xw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (k < K) {
                xv[u] = *reinterpret_cast<const uint4*>(xa + k);
                if (M16) xw[u] = *reinterpret_cast<const uint4*>(xb + k);
            }
        }
    };
    // With at most 8 tokens x is asked for one chunk ahead (it does not depend on the strip, so
    // a strip's last chunk asks for the first of the next): when the weights are there before
    // x, as in a short product whose ring was filled while the kernel before it drained, the
    // latency of x would otherwise show once per chunk.  With 16 tokens, and in the rotary form,
    // the registers do not allow it (measured: slower), and x is asked for just before the wait
    // for W.
    constexpr bool AHEAD = !M16 && MODE != SB_ROPE;
    uint4 xn[PER], xwn[PER];
    if (AHEAD && (int)blockIdx.x < nstrips) load_x(0, xn, xwn);
    int c = 0;
    for (int strip = blockIdx.x; strip < nstrips; strip += gridDim.x) {
        const int n0 = sb_strip_n0<MODE, NT>(strip, rp);
        float acc[GROUPS][4];
#pragma unroll
        for (int s = 0; s < GROUPS; ++s) acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.f;
        for (int ch = 0; ch < nch; ++ch, ++c) {
            const int st = c % SB_STAGES;
            const int nkb = min(SB_KC, K - ch * SB_KC) / 32;
            uint4 xv[PER], xw[PER];
            if (AHEAD) {
#pragma unroll
                for (int u = 0; u < PER; ++u) {
                    xv[u] = xn[u];
                    xw[u] = xwn[u];
                }
                const bool more = ch + 1 < nch || strip + (int)gridDim.x < nstrips;
                if (more) load_x(ch + 1 < nch ? ch + 1 : 0, xn, xwn);
            } else {
                load_x(ch, xv, xw);
            }
            // one outcome for the warp: the matrix instructions below are warp-wide
            if (!__all_sync(0xffffffffu, mbar_wait(full + 8 * st, (uint32_t)(c / SB_STAGES) & 1u))) {
                // give up, but only together with the other warps (they wait at the barrier below)
                if (lane == 0) atomicExch(error_word, 14);
                *failed = 1;
                break;
            }
            const unsigned char* stage = ring + st * STAGE;
#pragma unroll
            for (int u = 0; u < PER; ++u) {
                const int kb = warp + u * SB_WARPS;
                if (kb < nkb) {
                    const uint32_t a1[4] = {xv[u].x, xw[u].x, xv[u].y, xw[u].y};
                    const uint32_t a2[4] = {xv[u].z, xw[u].z, xv[u].w, xw[u].w};
#pragma unroll
                    for (int s = 0; s < GROUPS; ++s) {
                        const uint4 wv = *reinterpret_cast<const uint4*>(stage + (s * 8 + g) * PITCH + kb * 64 + t * 16);
                        mma_bf16_16816(acc[s], a1, wv.x, wv.y);
                        mma_bf16_16816(acc[s], a2, wv.z, wv.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) sb_arrive(empty + 8 * st);
        }
        // the last strip's weights are here: the next kernel may be scheduled while the sums
        // are made
        if (strip + (int)gridDim.x >= nstrips) pdl_launch_dependents();
        // ---- sum the warps' parts in shared memory: red[group][warp][token][W row]
#pragma unroll
        for (int s = 0; s < GROUPS; ++s) {
            float* mine = red + ((s * SB_WARPS + warp) * 16) * 8;
            mine[g * 8 + 2 * t] = acc[s][0];
            mine[g * 8 + 2 * t + 1] = acc[s][1];
            mine[(g + 8) * 8 + 2 * t] = acc[s][2];
            mine[(g + 8) * 8 + 2 * t + 1] = acc[s][3];
        }
        asm volatile("bar.sync 1, %0;" ::"n"(SB_WARPS * 32) : "memory");
        if (*failed) return;
        // thread -> (token m, row r of an 8-row group, group j): r fastest, so that consecutive
        // threads store consecutive features
        for (int idx = tid; idx < 128 * NT; idx += SB_WARPS * 32) {
            const int r = idx & 7, j = (idx >> 3) % NT, m = idx / (8 * NT);
            const int n = n0 + 8 * j + r;
            if (m < M && n < n_out) {
                float v[STRIPS];
#pragma unroll
                for (int s = 0; s < STRIPS; ++s) {
                    float sum = 0.f;
#pragma unroll
                    for (int w = 0; w < SB_WARPS; ++w)
                        sum += red[(((s * NT + j) * SB_WARPS + w) * 16 + m) * 8 + r];
                    v[s] = sum;
                }
                if (MODE == SB_ROPE) {
                    // n is the first partner's feature: head h, pair i of its hd/2
                    const int hd = rp.hd, half = hd / 2;
                    const int h = n0 / hd, i = n - h * hd;
                    float y0 = __bfloat162float(__float2bfloat16_rn(v[0]));
                    float y1 = __bfloat162float(__float2bfloat16_rn(v[STRIPS - 1]));
                    if (h < rp.nq + rp.nkv) {
                        float sn, cs;
                        sincosf((float)rp.positions[m] * rp.inv_freq[i], &sn, &cs);
                        const float x0 = y0, x1 = y1;
                        y0 = x0 * cs - x1 * sn;
                        y1 = x1 * cs + x0 * sn;
                    }
                    bf16* dst;
                    if (h < rp.nq) {
                        dst = reinterpret_cast<bf16*>(out) + (size_t)m * ldo + h * hd + i;
                    } else {
                        const int cp = rp.cache_pos[m];
                        const int page = rp.block_table[(size_t)rp.token_req[m] * rp.bt_stride + cp / rp.page_size];
                        const int slot = cp - (cp / rp.page_size) * rp.page_size;
                        const int hk = h - rp.nq;        // key heads, then value heads: the page's order
                        dst = rp.kv_cache + ((size_t)page * 2 * rp.nkv + hk) * rp.page_size * hd +
                              (size_t)slot * hd + i;
                    }
                    dst[0] = __float2bfloat16_rn(y0);
                    dst[half] = __float2bfloat16_rn(y1);
                    continue;
                }
                float y = v[0];
                if (MODE == SB_GATED) {
                    // gate and up are rounded to bfloat16 first, as the unfused path stores them
                    const float gate = __bfloat162float(__float2bfloat16_rn(v[0]));
                    const float up = __bfloat162float(__float2bfloat16_rn(v[STRIPS - 1]));
                    y = gate / (1.f + expf(-gate)) * up;
                }
                sb_store<OutT>(out + (size_t)m * ldo + n, y);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(SB_WARPS * 32) : "memory");  // red is reused by the next strip
    }
}

template <int MODE, bool M16, int NT, typename OutT>
static int launch_bulk_nt(const bf16* x, const bf16* W, OutT* out, int M, int n_out, int K, int ldx, int ldw,
                          int ldo, int inter, int w_static, int* error_word, cudaStream_t s,
                          const SbRope& rp = SbRope{}) {
    static int resident = 0;   // CTAs of this variant that fit on the GPU at once
    auto kernel = smallm_bulk_kernel<MODE, M16, NT, OutT>;
    constexpr int SMEM = sb_smem(MODE != SB_PLAIN, NT);
    if (resident == 0) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0, dev = 0, sms = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, SB_THREADS, SMEM);
        if (e != cudaSuccess) return (int)e;
        if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        if (per_sm < 1) return -2;
        resident = per_sm * sms;
    }
    // as many CTAs as give every CTA the same number of strips (within one): 320 strips on
    // 296 resident CTAs would leave 272 of them waiting for the 24 that take a second strip
    const int nstrips = MODE == SB_ROPE ? n_out / (16 * NT) : (n_out + 8 * NT - 1) / (8 * NT);
    const int rounds = (nstrips + resident - 1) / resident;
    const int grid = (nstrips + rounds - 1) / rounds;
    mstar_launch(kernel, dim3(grid), dim3(SB_THREADS), SMEM, s, x, W, out, M, n_out, K, ldx, ldw, ldo, inter, w_static, error_word, rp);
    return launch_status();
}

// Rows of W per strip by the number of output features: 8 while the strips barely fill the
// GPU, 16 and 32 where there are many (less traffic for x); the gated form has twice the rows
// per strip already, and with at most 8 tokens it keeps to them (two CTAs on an SM: measured
// faster than one with 32 rows).  MSTAR_SMALLM_NT=1|2|4 forces one (for measurements).
static int pick_nt(int n_out, bool gated, bool m16) {
    static int forced = -1;
    if (forced < 0) {
        const char* e = getenv("MSTAR_SMALLM_NT");
        forced = e ? atoi(e) : 0;
    }
    int nt = n_out >= 32768 ? 4 : (n_out >= 1024 ? 2 : 1);
    if (gated && !m16) nt = 1;
    if (forced == 1 || forced == 2 || forced == 4) nt = forced;
    if (gated && nt > 2) nt = 2;
    return nt;
}

template <bool GATED, bool M16, typename OutT>
static int launch_bulk(const bf16* x, const bf16* W, OutT* out, int M, int n_out, int K, int ldx, int ldw,
                       int ldo, int inter, int w_static, int* error_word, cudaStream_t s) {
    switch (pick_nt(n_out, GATED, M16)) {
        case 4:
            if constexpr (!GATED)
                return launch_bulk_nt<GATED ? SB_GATED : SB_PLAIN, M16, 4, OutT>(x, W, out, M, n_out, K, ldx, ldw, ldo, inter, w_static, error_word, s);
        case 2: return launch_bulk_nt<GATED ? SB_GATED : SB_PLAIN, M16, 2, OutT>(x, W, out, M, n_out, K, ldx, ldw, ldo, inter, w_static, error_word, s);
        default: return launch_bulk_nt<GATED ? SB_GATED : SB_PLAIN, M16, 1, OutT>(x, W, out, M, n_out, K, ldx, ldw, ldo, inter, w_static, error_word, s);
    }
}

// out[M, N] = x W^T (gated == 0), or out[M, N/2] = silu(x Wg^T) * (x Wu^T) for W = [Wg; Wu]
// (gated == 1, N even, bfloat16 out).  x: [M, K] bf16 with row stride ldx, W: [N, K] bf16 with
// row stride ldw, out: bf16 or float (out_dtype) with row stride ldo.  Returns 0, a CUDA error
// code, or -1 when the shape is refused: M outside 1..16, K no multiple of 32, leading
// dimensions not multiples of 8 elements or pointers not 16-byte aligned (bulk copies), N odd
// for the gated form.  `w_static`: nonzero promises that nothing earlier on the stream writes W
// (model weights), which lets the copies start before the kernel before this one has ended.
// `error_word`: device int, set to 13 / 14 if a bounded wait ran out.
MSTAR_API int mstar_gemm_smallm_bulk_bf16(const void* x, const void* W, void* out, int M, int N, int K,
                                          int ldx, int ldw, int ldo, int gated, int out_dtype,
                                          int w_static, int* error_word, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || K % 32 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || error_word == nullptr) return -1;
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)W & 15) != 0) return -1;
    if (gated && (N % 2 != 0 || out_dtype != MSTAR_BF16)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
    if (gated) {
        if (M > 8)
            return launch_bulk<true, true, bf16>(xp, wp, (bf16*)out, M, N / 2, K, ldx, ldw, ldo, N / 2, w_static, error_word, s);
        return launch_bulk<true, false, bf16>(xp, wp, (bf16*)out, M, N / 2, K, ldx, ldw, ldo, N / 2, w_static, error_word, s);
    }
    if (out_dtype == MSTAR_F32) {
        if (M > 8) return launch_bulk<false, true, float>(xp, wp, (float*)out, M, N, K, ldx, ldw, ldo, 0, w_static, error_word, s);
        return launch_bulk<false, false, float>(xp, wp, (float*)out, M, N, K, ldx, ldw, ldo, 0, w_static, error_word, s);
    }
    if (M > 8) return launch_bulk<false, true, bf16>(xp, wp, (bf16*)out, M, N, K, ldx, ldw, ldo, 0, w_static, error_word, s);
    return launch_bulk<false, false, bf16>(xp, wp, (bf16*)out, M, N, K, ldx, ldw, ldo, 0, w_static, error_word, s);
}

// The attention mixer's first product for few tokens, with the rotary encoding and the cache
// write where the sums are made: q_out[M, nq hd] = rotated (x Wq^T); rotated x Wk^T and
// x Wv^T go to the tokens' cache slots.  W: [(nq + 2 nkv) hd, K], rows [q heads | k heads |
// v heads]; split-half pairs over the whole head (rotary_dim == hd); kv_cache bfloat16
// [pages, 2, nkv, page_size, hd].  Returns -1 when the shape is refused: M outside 1..16, hd no
// multiple of 16, K no multiple of 32, strides or pointers unaligned, a null pointer.
MSTAR_API int mstar_qkv_rope_write_bulk_bf16(const void* x, const void* W, void* q_out, int M, int K, int ldx,
                                             int ldw, int ldo, const int* positions, const int* cache_pos,
                                             const int* token_req, const int* block_table, int bt_stride,
                                             const float* inv_freq, void* kv_cache, int nq, int nkv, int hd,
                                             int page_size, int w_static, int* error_word, void* stream) {
    if (M <= 0) return 0;
    if (M > 16 || K <= 0 || K % 32 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || error_word == nullptr) return -1;
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)W & 15) != 0) return -1;
    if (nq <= 0 || nkv <= 0 || hd <= 0 || hd % 16 != 0 || page_size <= 0) return -1;
    if (!positions || !cache_pos || !token_req || !block_table || !inv_freq || !kv_cache || !q_out) return -1;
    const SbRope rp{positions, cache_pos, token_req, block_table, inv_freq, (bf16*)kv_cache,
                    nq, nkv, hd, page_size, bt_stride};
    const int n_out = (nq + 2 * nkv) * hd;
    cudaStream_t s = (cudaStream_t)stream;
    // Strips of 32 rows (two 8-row groups of each half) for 9 to 16 tokens where the head size
    // allows: x is read half as often (12.0 -> 10.6 us at 16 tokens); with up to 8 tokens
    // strips of 16 rows are faster (8.5 against 10.1 us).  MSTAR_ROPE_NT=1|2 forces one.
    static int rope_nt = -1;
    if (rope_nt < 0) {
        const char* e = getenv("MSTAR_ROPE_NT");
        rope_nt = e ? atoi(e) : 0;
    }
    const bool wide = rope_nt == 2 || (rope_nt != 1 && M > 8);
    if (wide && hd % 32 == 0) {
        if (M > 8)
            return launch_bulk_nt<SB_ROPE, true, 2, bf16>((const bf16*)x, (const bf16*)W, (bf16*)q_out, M, n_out, K,
                                                          ldx, ldw, ldo, hd / 2, w_static, error_word, s, rp);
        return launch_bulk_nt<SB_ROPE, false, 2, bf16>((const bf16*)x, (const bf16*)W, (bf16*)q_out, M, n_out, K,
                                                       ldx, ldw, ldo, hd / 2, w_static, error_word, s, rp);
    }
    if (M > 8)
        return launch_bulk_nt<SB_ROPE, true, 1, bf16>((const bf16*)x, (const bf16*)W, (bf16*)q_out, M, n_out, K,
                                                      ldx, ldw, ldo, hd / 2, w_static, error_word, s, rp);
    return launch_bulk_nt<SB_ROPE, false, 1, bf16>((const bf16*)x, (const bf16*)W, (bf16*)q_out, M, n_out, K,
                                                   ldx, ldw, ldo, hd / 2, w_static, error_word, s, rp);
}
