// y[M,N] = x[M,K] W[N,K]^T in bfloat16 on the fifth-generation tensor cores:
// tcgen05.mma with both operands in shared memory and the float accumulator in tensor
// memory (TMEM), operand tiles brought in by TMA (cp.async.bulk.tensor) behind
// mbarriers, the accumulator read back with tcgen05.ld for the epilogue.
//
// One CTA computes one 128 x BN tile of y (BN = 256 or 128).  Six warps, three roles:
//   warp 0   producer: one lane issues the TMA loads of the x tile [128 x 64] and the W
//            tile [BN x 64] of each 64-wide k-block into a ring of STAGES buffers;
//   warp 1   owns the TMEM allocation; one lane issues four M128 x N(BN) x K16 MMAs per
//            k-block and commits them to the stage's "empty" barrier, and at the end to
//            the "accumulator ready" barrier;
//   warps 2-5  epilogue: each reads its 32 TMEM lanes (rows) in chunks of 32 columns,
//            converts and stores.
// Both operands are K-major (x is [M,K], W is [N,K], row-major), so the tiles are loaded
// with the 128-byte swizzle and described to the MMA by a shared-memory descriptor with
// an 8-row group stride of 1024 bytes; a k-step of 16 elements advances the descriptor's
// start address by 32 bytes inside the swizzle atom.
//
// No cluster, no multicast.  Rows beyond M, N or K are zero-filled by TMA and masked in
// the epilogue.  Every wait on an mbarrier is bounded: on a timeout the kernel records
// where it gave up in an error word, stops issuing work, frees its TMEM and returns.
//
// The reference uses the library GEMM for every linear layer
// (mstar/model/components/distributed/linear.py:101, 412).
#include "common.cuh"
#include "tma_util.cuh"
#include "tcgen05_util.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192

template <typename T> __device__ __forceinline__ void store32(T* dst, const uint32_t (&r)[32], int valid,
                                                               bool vec_ok);
template <> __device__ __forceinline__ void store32<float>(float* dst, const uint32_t (&r)[32], int valid,
                                                            bool vec_ok) {
    if (valid == 32 && vec_ok) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = __uint_as_float(r[i]);
    }
}
template <> __device__ __forceinline__ void store32<bf16>(bf16* dst, const uint32_t (&r)[32], int valid,
                                                           bool vec_ok) {
    if (valid == 32 && vec_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 v;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
            v.x = *reinterpret_cast<uint32_t*>(&p0);
            v.y = *reinterpret_cast<uint32_t*>(&p1);
            v.z = *reinterpret_cast<uint32_t*>(&p2);
            v.w = *reinterpret_cast<uint32_t*>(&p3);
            reinterpret_cast<uint4*>(dst)[i] = v;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
    }
}

// ----------------------------------------------------------------------------- kernel
template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    OutT* __restrict__ out, int M, int N, int K, int ldo, int* __restrict__ error_word) {
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;  // 16 KB
    constexpr uint32_t B_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ unsigned char smem_dyn[];
    // the swizzle pattern is a function of the address: stage buffers start on 1024 bytes
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t accum_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * TC_BM;
    const int num_kb = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(tc_smem(&full_bar[s]), 1);
            mbar_init(tc_smem(&empty_bar[s]), 1);
        }
        mbar_init(tc_smem(&accum_bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // TMEM: BN columns of 128 lanes x 32 bits for the accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         tc_smem(&tmem_base_slot)),
                     "r"((uint32_t)BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
                if (!mbar_wait(tc_smem(&empty_bar[s]), phase ^ 1u)) {  // first pass: free at once
                    atomicExch(error_word, 1);
                    abort_flag = 1;
                    break;
                }
                if (*(volatile int*)&abort_flag) break;
                const uint32_t bar = tc_smem(&full_bar[s]);
                mbar_expect_tx(bar, STAGE_BYTES);
                unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
                tma_load_2d(tc_smem(stage), &map_a, bar, kb * TC_BK, m0);
                tma_load_2d(tc_smem(stage + A_BYTES), &map_b, bar, kb * TC_BK, n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(TC_BM, BN);
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
                if (!mbar_wait(tc_smem(&full_bar[s]), phase)) {
                    atomicExch(error_word, 2);
                    abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_addr = tc_smem(tiles + (size_t)s * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
                    const uint64_t da = smem_desc_sw128(a_addr + k4 * 32);
                    const uint64_t db = smem_desc_sw128(b_addr + k4 * 32);
                    tc_mma(tmem_base, da, db, idesc, (kb | k4) != 0 ? 1u : 0u);
                }
                tc_commit(tc_smem(&empty_bar[s]));  // the stage is free when these MMAs are done
            }
            tc_commit(tc_smem(&accum_bar));          // all MMAs done: the accumulator is ready
        }
    } else {
        // epilogue warps 2..5: warp w may touch TMEM lanes 32*(w%4) .. +31
        const int quarter = warp & 3;
        const bool ready = mbar_wait(tc_smem(&accum_bar), 0);
        if (!ready && lane == 0) {
            atomicExch(error_word, 3);
            abort_flag = 1;
        }
        tc_fence_after_sync();
        // one outcome for the warp: the loads from tensor memory below are warp-wide
        if (__all_sync(0xffffffffu, ready && !*(volatile int*)&abort_flag)) {
            const int row = m0 + quarter * 32 + lane;
            const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tc_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
                tc_wait_ld();
                const int col = n0 + c0;
                if (row < M && col < N)
                    store32<OutT>(out + (size_t)row * ldo + col, r, min(32, N - col), vec_ok);
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)BN)
                     : "memory");
    }
}

// ------------------------------------------------------------- two-CTA pairs (cta_group::2)
// A pair of CTAs on two SMs (a cluster of 2) computes a 256 x 256 tile: each CTA holds the
// x tile of its own 128 rows and HALF of the W tile (128 of the 256 rows), and one MMA of
// the leader CTA reads both halves from both shared memories and writes each CTA's 128
// rows of the accumulator into that CTA's tensor memory.  Per byte loaded this does 1.5x
// the work of a lone 128 x 256 CTA, which is what counts: the lone-CTA kernel is bound
// by the rate at which L2 feeds shared memory.  Both CTAs' loads complete on the
// leader's "full" barrier; the MMA's commit arrives on the "empty" barriers of both CTAs
// (tcgen05.commit with a CTA mask).  No load is multicast.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], "
        "[%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(both)
        : "memory");
}

//
// GATED: W is a fused [gate; up] matrix of 2 * N rows.  The leader loads 128 gate rows, its
// peer the 128 up rows of the same output columns, so the accumulator holds gate in columns
// 0..127 and up in columns 128..255, and the epilogue writes silu(gate) * up: 128 output
// columns per tile, no [M, 2N] round trip and no separate activation kernel
// (mstar/model/components/distributed/mlp.py:78-81).
template <int STAGES, bool GATED, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         OutT* __restrict__ out, int M, int N, int K, int ldo,
                         int* __restrict__ error_word) {
    constexpr int BN = 256;                           // accumulator columns of the pair's tile
    constexpr int OUT_COLS = GATED ? BN / 2 : BN;     // output columns of the pair's tile
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;   // this CTA's 128 rows of x
    constexpr uint32_t B_BYTES = (BN / 2) * TC_BK * 2;  // this CTA's half of the W tile
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t accum_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int m0 = (blockIdx.x >> 1) * 2 * TC_BM + (int)rank * TC_BM;
    const int n0 = blockIdx.y * OUT_COLS;
    // rows of W this CTA loads: its half of the tile, or (gated) gate rows / up rows
    const int w_row0 = GATED ? (int)rank * N + n0 : n0 + (int)rank * (BN / 2);
    const int num_kb = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(tc_smem(&full_bar[s]), 1);
            mbar_init(tc_smem(&empty_bar[s]), 1);
        }
        mbar_init(tc_smem(&accum_bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         tc_smem(&tmem_base_slot)),
                     "r"((uint32_t)BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before either signals the other's
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
                if (!mbar_wait(tc_smem(&empty_bar[s]), phase ^ 1u)) {
                    atomicExch(error_word, 1);
                    abort_flag = 1;
                    break;
                }
                if (*(volatile int*)&abort_flag) break;
                // all four loads of the pair complete on the leader's barrier
                const uint32_t leader_bar = map_to_rank(tc_smem(&full_bar[s]), 0);
                if (rank == 0) mbar_expect_tx(tc_smem(&full_bar[s]), 2 * STAGE_BYTES);
                unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
                tma_load_2d_pair(tc_smem(stage), &map_a, leader_bar, kb * TC_BK, m0);
                tma_load_2d_pair(tc_smem(stage + A_BYTES), &map_b, leader_bar, kb * TC_BK, w_row0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(2 * TC_BM, BN);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
                if (!mbar_wait(tc_smem(&full_bar[s]), phase)) {
                    atomicExch(error_word, 2);
                    abort_flag = 1;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_addr = tc_smem(tiles + (size_t)s * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                    tc_mma_pair(tmem_base, smem_desc_sw128(a_addr + k4 * 32),
                                smem_desc_sw128(b_addr + k4 * 32), idesc, (kb | k4) != 0 ? 1u : 0u);
                tc_commit_pair(tc_smem(&empty_bar[s]));
            }
            tc_commit_pair(tc_smem(&accum_bar));
        }
    } else {
        const int quarter = warp & 3;
        const bool ready = mbar_wait(tc_smem(&accum_bar), 0);
        if (!ready && lane == 0) {
            atomicExch(error_word, 3);
            abort_flag = 1;
        }
        tc_fence_after_sync();
        // one outcome for the warp: the loads from tensor memory below are warp-wide
        if (__all_sync(0xffffffffu, ready && !*(volatile int*)&abort_flag)) {
            const int row = m0 + quarter * 32 + lane;
            const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
                tc_ld32(taddr, r);
                if (GATED) {
                    uint32_t u[32];
                    tc_ld32(taddr + BN / 2, u);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        // gate and up rounded to bfloat16 first, as the unfused path stores them
                        const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[i])));
                        const float v = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[i])));
                        r[i] = __float_as_uint(g / (1.f + expf(-g)) * v);
                    }
                } else {
                    tc_wait_ld();
                }
                const int col = n0 + c0;
                if (row < M && col < N)
                    store32<OutT>(out + (size_t)row * ldo + col, r, min(32, N - col), vec_ok);
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves while the other may still read its memory
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)BN)
                     : "memory");
    }
}

// [rows, K] bf16 row-major with leading dimension ld (elements); box = box_rows x 64
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return -3;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                          box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -4;
}

static int pairs_on_gpu() {
    static int pairs = 0;
    if (pairs == 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        pairs = sms > 1 ? sms / 2 : 1;
    }
    return pairs;
}

// ------------------------------------------------- persistent pairs, overlapped epilogue
// As many CTA pairs as the GPU holds at once walk over the tiles (row tiles fastest, so
// that pairs working at the same time share W tiles in L2).  Each CTA's tensor memory
// holds two accumulators of 256 columns: while the epilogue warps read and store tile j,
// the MMAs of tile j+1 already run into the other one.  Two more barrier pairs do the
// hand-over: "accumulator full" (the leader's commit, arriving in both CTAs) and
// "accumulator empty" (one arrival per epilogue warp of both CTAs on the leader's barrier).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
                 : "memory");
}

template <int BN, int STAGES, bool GATED, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                               const __grid_constant__ CUtensorMap map_b, OutT* __restrict__ out, int M,
                               int N, int K, int ldo, int tiles_m, int tiles_total,
                               int* __restrict__ error_word) {
    static_assert(BN == 256 || BN == 192 || BN == 128, "pair tile width");
    static_assert(!GATED || BN == 256, "the gated form keeps gate and up in 128 columns each");
    constexpr int OUT_COLS = GATED ? BN / 2 : BN;
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
    constexpr uint32_t B_BYTES = (BN / 2) * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(tc_smem(&full_bar[s]), 1);
            mbar_init(tc_smem(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tc_smem(&acc_full[b]), 1);
            mbar_init(tc_smem(&acc_empty[b]), 8);  // four epilogue warps in each of two CTAs
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         tc_smem(&tmem_base_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;  // k-blocks loaded so far, over all tiles
            for (int t = pair; t < tiles_total; t += num_pairs) {
                const int m0 = (t % tiles_m) * 2 * TC_BM + (int)rank * TC_BM;
                const int n0 = (t / tiles_m) * OUT_COLS;
                const int w_row0 = GATED ? (int)rank * N + n0 : n0 + (int)rank * (BN / 2);
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1u;
                    if (!mbar_wait(tc_smem(&empty_bar[s]), phase ^ 1u)) {
                        atomicExch(error_word, 1);
                        abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t leader_bar = map_to_rank(tc_smem(&full_bar[s]), 0);
                    if (rank == 0) mbar_expect_tx(tc_smem(&full_bar[s]), 2 * STAGE_BYTES);
                    unsigned char* stage = tiles + (size_t)s * STAGE_BYTES;
                    tma_load_2d_pair(tc_smem(stage), &map_a, leader_bar, kb * TC_BK, m0);
                    tma_load_2d_pair(tc_smem(stage + A_BYTES), &map_b, leader_bar, kb * TC_BK, w_row0);
                }
                if (!ok || *(volatile int*)&abort_flag) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(2 * TC_BM, BN);
            uint32_t it = 0;
            int j = 0;  // tiles done by this pair
            bool ok = true;
            for (int t = pair; t < tiles_total && ok; t += num_pairs, ++j) {
                const int b = j & 1;
                if (!mbar_wait(tc_smem(&acc_empty[b]), (((uint32_t)j >> 1) & 1u) ^ 1u)) {
                    atomicExch(error_word, 6);
                    abort_flag = 1;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + (uint32_t)b * 256;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1u;
                    if (!mbar_wait(tc_smem(&full_bar[s]), phase)) {
                        atomicExch(error_word, 2);
                        abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = tc_smem(tiles + (size_t)s * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                        tc_mma_pair(tmem_d, smem_desc_sw128(a_addr + k4 * 32),
                                    smem_desc_sw128(b_addr + k4 * 32), idesc, (kb | k4) != 0 ? 1u : 0u);
                    tc_commit_pair(tc_smem(&empty_bar[s]));
                }
                if (ok) tc_commit_pair(tc_smem(&acc_full[b]));
            }
        }
    } else {
        const int quarter = warp & 3;
        const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
        int j = 0;
        for (int t = pair; t < tiles_total; t += num_pairs, ++j) {
            const int b = j & 1;
            const bool ready = mbar_wait(tc_smem(&acc_full[b]), ((uint32_t)j >> 1) & 1u);
            // one outcome for the warp: the loads from tensor memory below are warp-wide
            if (!__all_sync(0xffffffffu, ready && !*(volatile int*)&abort_flag)) {
                if (!ready && lane == 0) {
                    atomicExch(error_word, 3);
                    abort_flag = 1;
                }
                break;
            }
            tc_fence_after_sync();
            const int m0 = (t % tiles_m) * 2 * TC_BM + (int)rank * TC_BM;
            const int n0 = (t / tiles_m) * OUT_COLS;
            const int row = m0 + quarter * 32 + lane;
            const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)b * 256;
            if (!GATED) {
                // read 64 columns at a time; after the last read the accumulator is free
                // for the MMAs of the tile after next, the stores follow
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    uint32_t r[2][32];
                    tc_ld32(tbase + (uint32_t)c0, r[0]);
                    tc_ld32(tbase + (uint32_t)(c0 + 32), r[1]);
                    tc_wait_ld();
                    if (c0 + 64 == BN) {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_remote(map_to_rank(tc_smem(&acc_empty[b]), 0));
                    }
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int col = n0 + c0 + c * 32;
                        if (row < M && col < N)
                            store32<OutT>(out + (size_t)row * ldo + col, r[c], min(32, N - col), vec_ok);
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
                    uint32_t r[32], u[32];
                    tc_ld32(tbase + (uint32_t)c0, r);
                    tc_ld32(tbase + (uint32_t)(c0 + BN / 2), u);
                    tc_wait_ld();
                    if (c0 + 32 == OUT_COLS) {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_remote(map_to_rank(tc_smem(&acc_empty[b]), 0));
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[i])));
                        const float v = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[i])));
                        r[i] = __float_as_uint(g / (1.f + expf(-g)) * v);
                    }
                    const int col = n0 + c0;
                    if (row < M && col < N)
                        store32<OutT>(out + (size_t)row * ldo + col, r, min(32, N - col), vec_ok);
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                     : "memory");
    }
}

template <int BN, int STAGES, bool GATED, typename OutT>
static int launch_tc_persistent(const CUtensorMap& ma, const CUtensorMap& mb, OutT* out, int M, int N,
                                int K, int ldo, int* error_word, cudaStream_t s) {
    const size_t smem = (size_t)STAGES * (TC_BM + BN / 2) * TC_BK * 2 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<BN, STAGES, GATED, OutT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int out_cols = GATED ? BN / 2 : BN;
    const int tiles_m = (M + 2 * TC_BM - 1) / (2 * TC_BM);
    const int tiles_n = (N + out_cols - 1) / out_cols;
    const int total = tiles_m * tiles_n;
    const int on_gpu = pairs_on_gpu();
    const int pairs = total < on_gpu ? total : on_gpu;
    gemm_tcgen05_persistent_kernel<BN, STAGES, GATED, OutT><<<2 * pairs, TC_THREADS, smem, s>>>(
        ma, mb, out, M, N, K, ldo, tiles_m, total, error_word);
    return launch_status();
}

template <int STAGES, bool GATED, typename OutT>
static int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mb, OutT* out, int M, int N, int K,
                          int ldo, int* error_word, cudaStream_t s) {
    const size_t smem = (size_t)STAGES * (TC_BM + 128) * TC_BK * 2 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<STAGES, GATED, OutT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int out_cols = GATED ? 128 : 256;  // N is the number of output columns
    dim3 grid(2 * ((M + 2 * TC_BM - 1) / (2 * TC_BM)), (N + out_cols - 1) / out_cols);
    gemm_tcgen05_pair_kernel<STAGES, GATED, OutT><<<grid, TC_THREADS, smem, s>>>(ma, mb, out, M, N, K,
                                                                                  ldo, error_word);
    return launch_status();
}

// ------------------------------------------------------------------------------- host
template <int BN, int STAGES, typename OutT>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, OutT* out, int M, int N, int K, int ldo,
                     int* error_word, cudaStream_t s) {
    const size_t smem = (size_t)STAGES * (TC_BM + BN) * TC_BK * 2 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, OutT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + TC_BM - 1) / TC_BM);
    gemm_tcgen05_kernel<BN, STAGES, OutT><<<grid, TC_THREADS, smem, s>>>(ma, mb, out, M, N, K, ldo,
                                                                         error_word);
    return launch_status();
}

// out[M,N] = x[M,K] W[N,K]^T.  out_dtype MSTAR_BF16 or MSTAR_F32; bn 128 or 256: lone CTAs
// with 128 x bn tiles; bn 512: pairs of CTAs with 256 x 256 tiles, one tile per pair; bn
// 1024: persistent pairs that walk over the tiles and overlap each tile's epilogue with
// the next tile's MMAs.
// `error_word`: device int, zero before the call; a kernel that gave up on a wait writes
// 1 (producer), 2 (MMA issuer) or 3 (epilogue) there.  Returns 0, a CUDA error code, -1
// when the shape is refused (K or a leading dimension not a multiple of 8 elements,
// operands not 16-byte aligned, bn not 128 or 256), -3 / -4 when the tensor map cannot
// be made.
// out[M, N/2] = silu(x Wg^T) * (x Wu^T) for the fused W = [Wg; Wu] of N rows, bfloat16, on
// pairs of CTAs.  Refusals and error word as mstar_gemm_tcgen05_bf16; N/2 must be a
// multiple of 8.
MSTAR_API int mstar_gemm_tcgen05_gated_bf16(const void* x, const void* W, void* out, int M, int N,
                                            int K, int ldx, int ldw, int ldo, int* error_word,
                                            void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || N % 16 != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return -1;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, x, M, K, ldx, TC_BM);
    if (rc != 0) return rc;
    rc = make_map(&mb, W, N, K, ldw, 128);
    if (rc != 0) return rc;
    return launch_tc_persistent<256, 6, true, bf16>(ma, mb, (bf16*)out, M, N / 2, K, ldo, error_word,
                                                    (cudaStream_t)stream);
}

MSTAR_API int mstar_gemm_tcgen05_bf16(const void* x, const void* W, void* out, int M, int N, int K,
                                      int ldx, int ldw, int ldo, int out_dtype, int bn,
                                      int* error_word, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return -1;
    if (bn != 128 && bn != 256 && bn != 512 && bn != 1024) return -1;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, x, M, K, ldx, TC_BM);
    if (rc != 0) return rc;
    rc = make_map(&mb, W, N, K, ldw, bn >= 512 ? 128 : bn);
    if (rc != 0) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (bn == 1024) {  // persistent pairs with overlapped epilogue
        // (narrower pair tiles, 192 or 128 columns, were measured for the shapes whose 256-wide
        // tiles fill the pairs unevenly: no gain, the kernel is bound by operand traffic per
        // k-block, which narrower tiles do not reduce)
        if (out_dtype == MSTAR_F32)
            return launch_tc_persistent<256, 6, false, float>(ma, mb, (float*)out, M, N, K, ldo,
                                                              error_word, s);
        return launch_tc_persistent<256, 6, false, bf16>(ma, mb, (bf16*)out, M, N, K, ldo, error_word, s);
    }
    if (bn == 512) {  // pairs of CTAs, 256 x 256 tiles
        if (out_dtype == MSTAR_F32)
            return launch_tc_pair<6, false, float>(ma, mb, (float*)out, M, N, K, ldo, error_word, s);
        return launch_tc_pair<6, false, bf16>(ma, mb, (bf16*)out, M, N, K, ldo, error_word, s);
    }
    if (out_dtype == MSTAR_F32) {
        if (bn == 256) return launch_tc<256, 4, float>(ma, mb, (float*)out, M, N, K, ldo, error_word, s);
        return launch_tc<128, 6, float>(ma, mb, (float*)out, M, N, K, ldo, error_word, s);
    }
    if (bn == 256) return launch_tc<256, 4, bf16>(ma, mb, (bf16*)out, M, N, K, ldo, error_word, s);
    return launch_tc<128, 6, bf16>(ma, mb, (bf16*)out, M, N, K, ldo, error_word, s);
}
