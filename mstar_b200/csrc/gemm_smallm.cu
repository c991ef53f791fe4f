// y[M,N] = x[M,K] W[N,K]^T for few rows (M <= 16), bfloat16 in, float accumulation:
// the matrix product of decode steps, where every weight is read once and the time is
// the time to stream W from HBM.
//
// A CTA owns 8 output features (8 rows of W); its eight warps split K among them and
// are summed in shared memory.  Each warp streams its part of the 8 rows straight from
// global memory into MMA fragments: the rows of W are the 8-wide N of m16n8k16, the
// tokens (padded to 16) its M.  Within a block of 32 k-values a thread takes 8
// consecutive ones (one 16-byte load per row) instead of the canonical interleaved
// ones; the sum over k does not care, and x is read with the same assignment, so the
// products pair up correctly.  A warp issues the loads of eight blocks before it uses
// the first, and the small strips give several CTAs per SM, which together keep enough
// bytes in flight to saturate HBM even for the narrow projections (N = 3072).
//
// Variants: GATED computes two strips at once, rows n and inter + n of a fused
// [gate; up] matrix, and writes silu(gate) * up (mstar/model/components/distributed/
// mlp.py:78-81), which saves the [M, 2*inter] round trip and one launch.  The output
// type is bfloat16 or float (logits).  The reference uses the library GEMM for all of
// these (mstar/model/components/distributed/linear.py:101).
#include "common.cuh"
#include "mma_util.cuh"

#define SM_WARPS 8
#define SM_THREADS (SM_WARPS * 32)
#define SM_UNROLL 8

__device__ __forceinline__ uint4 ld_stream(const bf16* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}
// x: an ordinary load (cached in L1, coherent after the dependency wait; not __ldg, which is
// for memory that does not change while the kernel lives)
__device__ __forceinline__ uint4 ld_cached(const bf16* p) {
    return *reinterpret_cast<const uint4*>(p);
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// M16: tokens 8..15 exist (else the upper half of the MMA's rows is zero)
template <bool GATED, bool M16, typename OutT>
__global__ void __launch_bounds__(SM_THREADS)
smallm_gemm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, OutT* __restrict__ out,
                   int M, int n_out, int K, int ldx, int ldw, int ldo, int inter, int w_static) {
    // Weights that nothing writes while the engine runs are asked for before the wait for
    // the kernel before this one (whose output x is); see the loop.
    unsigned long long waited = 0;
    if (!w_static) waited = pdl_wait();
    constexpr int STRIPS = GATED ? 2 : 1;
    __shared__ float red[STRIPS][SM_WARPS][16][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 8;
    const int kblocks = K / 32;
    const int kb0 = (int)((long long)warp * kblocks / SM_WARPS);
    const int kb1 = (int)((long long)(warp + 1) * kblocks / SM_WARPS);

    const int row = min(n0 + g, n_out - 1);
    const bf16* wp[STRIPS];
#pragma unroll
    for (int s = 0; s < STRIPS; ++s) wp[s] = W + ((size_t)row + (size_t)s * inter) * ldw + 8 * t;
    // x is what the kernel before wrote: its addresses are formed after the wait
    const bf16* xa = pdl_after(x, waited) + (size_t)min(g, M - 1) * ldx + 8 * t;
    const bf16* xb = pdl_after(x, waited) + (size_t)min(g + 8, M - 1) * ldx + 8 * t;

    float acc[STRIPS][4];
#pragma unroll
    for (int s = 0; s < STRIPS; ++s) acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.f;

    for (int kb = kb0; kb < kb1; kb += SM_UNROLL) {
        uint4 wv[STRIPS][SM_UNROLL];
#pragma unroll
        for (int u = 0; u < SM_UNROLL; ++u) {
            if (kb + u < kb1) {
#pragma unroll
                for (int s = 0; s < STRIPS; ++s) wv[s][u] = ld_stream(wp[s] + (kb + u) * 32);
            }
        }
        if (w_static && kb == kb0) {             // the first weights are on their way
            const unsigned long long z = pdl_wait();
            xa = pdl_after(xa, z);
            xb = pdl_after(xb, z);
        }
#pragma unroll
        for (int u = 0; u < SM_UNROLL; ++u) {
            if (kb + u < kb1) {
                const int k = (kb + u) * 32;
                const uint4 xv = ld_cached(xa + k);
                uint4 xw = make_uint4(0u, 0u, 0u, 0u);
                if (M16) xw = ld_cached(xb + k);
                const uint32_t a1[4] = {xv.x, xw.x, xv.y, xw.y};
                const uint32_t a2[4] = {xv.z, xw.z, xv.w, xw.w};
#pragma unroll
                for (int s = 0; s < STRIPS; ++s) {
                    mma_bf16_16816(acc[s], a1, wv[s][u].x, wv[s][u].y);
                    mma_bf16_16816(acc[s], a2, wv[s][u].z, wv[s][u].w);
                }
            }
        }
    }

    if (w_static) pdl_wait();  // a warp without a part of K has not waited yet; nothing is stored before
    pdl_launch_dependents();   // the weights are here: the next kernel may be scheduled
    // ---- sum the warps' parts of K in shared memory: red[..][token][W row]
#pragma unroll
    for (int s = 0; s < STRIPS; ++s) {
        red[s][warp][g][2 * t] = acc[s][0];
        red[s][warp][g][2 * t + 1] = acc[s][1];
        red[s][warp][g + 8][2 * t] = acc[s][2];
        red[s][warp][g + 8][2 * t + 1] = acc[s][3];
    }
    __syncthreads();
    if (tid < 128) {
        const int r = tid & 7, m = tid >> 3;  // r fastest: consecutive threads, consecutive n
        if (m < M && n0 + r < n_out) {
            float v[STRIPS];
#pragma unroll
            for (int s = 0; s < STRIPS; ++s) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < SM_WARPS; ++w) sum += red[s][w][m][r];
                v[s] = sum;
            }
            float y = v[0];
            if (GATED) {
                // gate and up are rounded to bfloat16 first, as the unfused path stores them
                const float gate = __bfloat162float(__float2bfloat16_rn(v[0]));
                const float up = __bfloat162float(__float2bfloat16_rn(v[STRIPS - 1]));
                y = gate / (1.f + expf(-gate)) * up;
            }
            store_out<OutT>(out + (size_t)m * ldo + n0 + r, y);
        }
    }
}

// ---- wide strips: 16 rows of W per CTA as the A operand (the MMA's M), up to 8 tokens as
// its N.  Half as many CTAs, each with twice the bytes: the better shape for matrices with
// many rows (the fused gate/up matrix), where there are CTAs enough anyway.
template <int NT, bool GATED, typename OutT>
__global__ void __launch_bounds__(SM_THREADS)
smallm_wide_gemm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, OutT* __restrict__ out,
                   int M, int n_out, int K, int ldx, int ldw, int ldo, int inter, int w_static) {
    unsigned long long waited = 0;
    if (!w_static) waited = pdl_wait();   // as in the kernel above
    extern __shared__ float red[];  // [strips][SM_WARPS][16][8*NT]
    constexpr int COLS = 8 * NT;
    constexpr int STRIPS = GATED ? 2 : 1;
    constexpr int UNROLL = GATED ? 4 : 8;  // k-blocks of W in flight per thread
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int kblocks = K / 32;
    const int kb0 = (int)((long long)warp * kblocks / SM_WARPS);
    const int kb1 = (int)((long long)(warp + 1) * kblocks / SM_WARPS);

    const int ra = min(n0 + g, n_out - 1), rb = min(n0 + g + 8, n_out - 1);
    const bf16* wa[STRIPS];
    const bf16* wb[STRIPS];
#pragma unroll
    for (int s = 0; s < STRIPS; ++s) {
        wa[s] = W + ((size_t)ra + (size_t)s * inter) * ldw + 8 * t;
        wb[s] = W + ((size_t)rb + (size_t)s * inter) * ldw + 8 * t;
    }
    const bf16* xr[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) xr[j] = pdl_after(x, waited) + (size_t)min(8 * j + g, M - 1) * ldx + 8 * t;

    float acc[STRIPS][NT][4];
#pragma unroll
    for (int s = 0; s < STRIPS; ++s)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.f;

    for (int kb = kb0; kb < kb1; kb += UNROLL) {
        uint4 va[STRIPS][UNROLL], vb[STRIPS][UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (kb + u < kb1) {
                const int k = (kb + u) * 32;
#pragma unroll
                for (int s = 0; s < STRIPS; ++s) {
                    va[s][u] = ld_stream(wa[s] + k);
                    vb[s][u] = ld_stream(wb[s] + k);
                }
            }
        }
        if (w_static && kb == kb0) {             // the first weights are on their way
            const unsigned long long z = pdl_wait();
#pragma unroll
            for (int j = 0; j < NT; ++j) xr[j] = pdl_after(xr[j], z);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (kb + u < kb1) {
                const int k = (kb + u) * 32;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint4 xv = ld_cached(xr[j] + k);
#pragma unroll
                    for (int s = 0; s < STRIPS; ++s) {
                        const uint32_t a1[4] = {va[s][u].x, vb[s][u].x, va[s][u].y, vb[s][u].y};
                        const uint32_t a2[4] = {va[s][u].z, vb[s][u].z, va[s][u].w, vb[s][u].w};
                        mma_bf16_16816(acc[s][j], a1, xv.x, xv.y);
                        mma_bf16_16816(acc[s][j], a2, xv.z, xv.w);
                    }
                }
            }
        }
    }

    if (w_static) pdl_wait();  // a warp without a part of K has not waited yet; nothing is stored before
    pdl_launch_dependents();   // the weights are here: the next kernel may be scheduled
    // ---- sum the warps' parts of K in shared memory
#pragma unroll
    for (int s = 0; s < STRIPS; ++s) {
        float* mine = red + ((size_t)(s * SM_WARPS + warp) * 16) * COLS;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int col = 8 * j + 2 * t;
            mine[g * COLS + col] = acc[s][j][0];
            mine[g * COLS + col + 1] = acc[s][j][1];
            mine[(g + 8) * COLS + col] = acc[s][j][2];
            mine[(g + 8) * COLS + col + 1] = acc[s][j][3];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * COLS; idx += SM_THREADS) {
        const int r = idx & 15, m = idx >> 4;  // r fastest: consecutive threads, consecutive n
        if (m >= M || n0 + r >= n_out) continue;
        float v[STRIPS];
#pragma unroll
        for (int s = 0; s < STRIPS; ++s) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < SM_WARPS; ++w)
                sum += red[((size_t)(s * SM_WARPS + w) * 16 + r) * COLS + m];
            v[s] = sum;
        }
        float y = v[0];
        if (GATED) {
            // the gate is rounded to bfloat16 first, as the unfused path stores it
            const float gate = __bfloat162float(__float2bfloat16_rn(v[0]));
            const float up = __bfloat162float(__float2bfloat16_rn(v[STRIPS - 1]));
            y = gate / (1.f + expf(-gate)) * up;
        }
        store_out<OutT>(out + (size_t)m * ldo + n0 + r, y);
    }
}

template <bool GATED, typename OutT>
static int launch_smallm(const bf16* x, const bf16* W, OutT* out, int M, int n_out, int K, int ldx,
                         int ldw, int ldo, int inter, int w_static, cudaStream_t s) {
    if (M <= 8 && n_out >= 8192 && n_out < 65536) {
        const size_t smem = (size_t)(GATED ? 2 : 1) * SM_WARPS * 16 * 8 * sizeof(float);
        mstar_launch((smallm_wide_gemm_kernel<1, GATED, OutT>), dim3((n_out + 15) / 16), dim3(SM_THREADS), smem, s, 
            x, W, out, M, n_out, K, ldx, ldw, ldo, inter, w_static);
        return launch_status();
    }
    const int grid = (n_out + 7) / 8;
    if (M <= 8)
        mstar_launch((smallm_gemm_kernel<GATED, false, OutT>), dim3(grid), dim3(SM_THREADS), 0, s, x, W, out, M, n_out, K,
                                                                           ldx, ldw, ldo, inter, w_static);
    else
        mstar_launch((smallm_gemm_kernel<GATED, true, OutT>), dim3(grid), dim3(SM_THREADS), 0, s, x, W, out, M, n_out, K,
                                                                          ldx, ldw, ldo, inter, w_static);
    return launch_status();
}

// out[M, N] = x W^T (gated == 0), or out[M, N/2] = silu(x Wg^T) * (x Wu^T) for W = [Wg; Wu]
// (gated == 1).  out_dtype: MSTAR_BF16 or MSTAR_F32.  Returns 0, a CUDA error code, or -1
// when the shape is refused: M outside 1..16, K no multiple of 32, leading dimensions not
// multiples of 8 elements (16-byte loads), N odd for the gated form.  `w_static`: nonzero
// promises that nothing earlier on the stream writes W (model weights); the first weight
// loads are then issued before the wait for the kernel before this one.
MSTAR_API int mstar_gemm_smallm_bf16(const void* x, const void* W, void* out, int M, int N, int K,
                                     int ldx, int ldw, int ldo, int gated, int out_dtype,
                                     int w_static, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || K % 32 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return -1;
    if (gated && (N % 2 != 0 || out_dtype != MSTAR_BF16)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
    if (gated) return launch_smallm<true, bf16>(xp, wp, (bf16*)out, M, N / 2, K, ldx, ldw, ldo, N / 2, w_static, s);
    if (out_dtype == MSTAR_F32)
        return launch_smallm<false, float>(xp, wp, (float*)out, M, N, K, ldx, ldw, ldo, 0, w_static, s);
    return launch_smallm<false, bf16>(xp, wp, (bf16*)out, M, N, K, ldx, ldw, ldo, 0, w_static, s);
}
