// y[M,N] = x[M,K] W[N,K]^T in bfloat16 for a few dozen rows of x (17 to 128: decode steps
// of many requests) and a very wide W (a vocabulary-wide head), on the fifth-generation
// tensor cores with the operands swapped: the rows of W are the M dimension of the MMA
// (128 to a tile) and the tokens its N dimension (32, 64 or 128), so no half of a tile is
// spent on rows that do not exist.  The product is bound by the one pass over W:
//
//   * a CTA takes one tile of 128 rows of W and all of K; two CTAs share an SM (their
//     rings hold 192 KB of tiles on their way between them), so that one CTA's start and
//     epilogue lie under the other's stream;
//   * warp 0 issues the TMA loads (128-byte swizzle, ring of stages behind mbarriers).  W
//     is a model parameter: its first loads are issued before the wait of programmatic
//     dependent launch, while the kernel before is still draining; x is loaded after it;
//   * warp 1 issues tcgen05.mma (M 128, N = tokens, K 16) into a float accumulator in
//     tensor memory; warps 2-5 read it back with tcgen05.ld and store straight from their
//     registers: a warp's lanes are consecutive rows of W, that is consecutive features
//     of a token.
//
// Narrow matrices (a few dozen tiles) would have to be cut along K to fill the GPU; that
// was built (partial tiles exchanged through scratch memory, summed in fixed order by the
// CTA that arrives last at a counter) and measured at 64 rows: 17 to 22 us for the
// attention and feed-forward projections of a 3072-wide model against 7 to 14 us of the
// library GEMM, each extra slice costing about 5 us.  A second form cut K over the CTAs of a
// thread-block cluster (each CTA its share of the k-blocks of one tile, its float partial
// tile left in its own shared memory, every CTA adding up one share of the elements from all
// of them through distributed shared memory, in rank order, 16 bytes a load): right in every
// test and as fast as the library's kernels when timed alone (64 rows: O 8.4 against 7.3 us,
// down 14.0 against 14.2, QKV 11.1 against 8.5), but a decode step of 64 requests took 4.49
// instead of 4.28 ms with it.  A CTA with an SM to itself and a ring of 96 KB moves 64 GB/s;
// twice the ring shuts the next kernel's CTAs out of the SM, and with them the overlap of
// its weight copies with this kernel's end.  So those stay with the library and this kernel
// keeps one slice.
//
// Every mbarrier wait is bounded and reports into an error word.  No cluster, no multicast.
// The reference uses the library GEMM for every linear layer
// (mstar/model/components/distributed/linear.py:101, 412).
#include "common.cuh"
#include "tma_util.cuh"
#include "tcgen05_util.cuh"

#define SK_ROWS 128        // rows of W to a tile
#define SK_BK 64           // k-block: one 128-byte swizzle atom of bfloat16
#define SK_THREADS 192
// Stages of a CTA's ring, so that two CTAs fit an SM (96 to 100 KB each).
__host__ __device__ constexpr int sk_stages(int tok) { return tok <= 32 ? 5 : (tok <= 64 ? 4 : 3); }

template <typename T> __device__ __forceinline__ void sk_store(T* p, float v);
template <> __device__ __forceinline__ void sk_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void sk_store<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// TOK: tokens of the MMA's N dimension (M <= TOK); N: rows of W = output features.
template <int TOK, typename OutT>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   OutT* __restrict__ out, int M, int N, int K, int ldo, int w_static,
                   int* __restrict__ error_word) {
    constexpr int STAGES = sk_stages(TOK);
    constexpr uint32_t W_BYTES = SK_ROWS * SK_BK * 2;   // 16 KB
    constexpr uint32_t X_BYTES = TOK * SK_BK * 2;
    constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;
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
    const int n0 = blockIdx.x * SK_ROWS;
    const int num_kb = (K + SK_BK - 1) / SK_BK;

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
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         tc_smem(&tmem_base_slot)),
                     "r"((uint32_t)TOK)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            auto load_w = [&](int kb, int s) {
                const uint32_t bar = tc_smem(&full_bar[s]);
                mbar_expect_tx(bar, STAGE_BYTES);       // the stage's W and x tiles
                tma_load_2d(tc_smem(tiles + (size_t)s * STAGE_BYTES), &map_w, bar, kb * SK_BK, n0);
            };
            auto load_x = [&](int kb, int s) {
                tma_load_2d(tc_smem(tiles + (size_t)s * STAGE_BYTES + W_BYTES), &map_x,
                            tc_smem(&full_bar[s]), kb * SK_BK, 0);
            };
            // the first ring of weights before the dependency wait: nothing earlier on the
            // stream writes them
            const int early = w_static ? min(num_kb, STAGES) : 0;
            for (int kb = 0; kb < early; ++kb) load_w(kb, kb);
            pdl_wait();
            for (int kb = 0; kb < early; ++kb) load_x(kb, kb);
            for (int kb = early; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
                if (!mbar_wait(tc_smem(&empty_bar[s]), phase ^ 1u)) {  // first pass: free at once
                    atomicExch(error_word, 15);
                    abort_flag = 1;
                    break;
                }
                if (*(volatile int*)&abort_flag) break;
                load_w(kb, s);
                load_x(kb, s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(SK_ROWS, TOK);
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t phase = (uint32_t)(kb / STAGES) & 1u;
                if (!mbar_wait(tc_smem(&full_bar[s]), phase)) {
                    atomicExch(error_word, 16);
                    abort_flag = 1;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t w_addr = tc_smem(tiles + (size_t)s * STAGE_BYTES);
                const uint32_t x_addr = w_addr + W_BYTES;
#pragma unroll
                for (int k4 = 0; k4 < SK_BK / 16; ++k4)
                    tc_mma(tmem_base, smem_desc_sw128(w_addr + k4 * 32), smem_desc_sw128(x_addr + k4 * 32),
                           idesc, (kb | k4) != 0 ? 1u : 0u);
                tc_commit(tc_smem(&empty_bar[s]));  // the stage is free when these MMAs are done
            }
            tc_commit(tc_smem(&accum_bar));          // all MMAs done: the accumulator is ready
        }
    } else {
        // warps 2-5: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        const bool ready = mbar_wait(tc_smem(&accum_bar), 0);
        if (!ready && lane == 0) {
            atomicExch(error_word, 17);
            abort_flag = 1;
        }
        tc_fence_after_sync();
        // every byte of W this CTA needs has been consumed: the next kernel may be scheduled
        pdl_launch_dependents();
        // `out` may be memory that the kernel before still reads: nothing is written before
        // that kernel has ended
        pdl_wait();
        // one outcome for the warp: the loads from tensor memory below are warp-wide
        if (__all_sync(0xffffffffu, ready && !*(volatile int*)&abort_flag)) {
            const int n = n0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < TOK; c0 += 32) {
                uint32_t v[32];
                tc_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                tc_wait_ld();
                if (n < N) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c0 + i < M) sk_store<OutT>(out + (size_t)(c0 + i) * ldo + n, __uint_as_float(v[i]));
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TOK)
                     : "memory");
    }
}

// ------------------------------------------------------------------------------- host
// [rows, K] bf16 row-major with leading dimension ld (elements); box = box_rows x 64
static int sk_make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return -3;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {SK_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                          box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -4;
}

template <int TOK, typename OutT>
static int sk_launch(const CUtensorMap& mw, const CUtensorMap& mx, OutT* out, int M, int N, int K, int ldo,
                     int w_static, int* error_word, cudaStream_t s) {
    constexpr size_t smem = (size_t)sk_stages(TOK) * (SK_ROWS + TOK) * SK_BK * 2 + 1024;
    auto kernel = gemm_skinny_kernel<TOK, OutT>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    mstar_launch(kernel, dim3((N + SK_ROWS - 1) / SK_ROWS), dim3(SK_THREADS), smem, s, mw, mx, out, M, N, K, ldo,
                 w_static, error_word);
    return launch_status();
}

template <typename OutT>
static int sk_dispatch(const void* x, const void* W, OutT* out, int M, int N, int K, int ldx, int ldw, int ldo,
                       int w_static, int* error_word, cudaStream_t s) {
    const int tok = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
    CUtensorMap mw, mx;
    int rc = sk_make_map(&mw, W, N, K, ldw, SK_ROWS);
    if (rc != 0) return rc;
    rc = sk_make_map(&mx, x, M, K, ldx, tok);
    if (rc != 0) return rc;
    switch (tok) {
        case 32: return sk_launch<32, OutT>(mw, mx, out, M, N, K, ldo, w_static, error_word, s);
        case 64: return sk_launch<64, OutT>(mw, mx, out, M, N, K, ldo, w_static, error_word, s);
        default: return sk_launch<128, OutT>(mw, mx, out, M, N, K, ldo, w_static, error_word, s);
    }
}

// out[M, N] = x W^T for M <= 128; out_dtype MSTAR_BF16 or MSTAR_F32.  `w_static`: nonzero
// promises that no kernel earlier on the stream writes W.  `error_word`: device int, zero
// before the call; a kernel that gave up on a wait writes 15 (producer), 16 (MMA issuer) or
// 17 (epilogue) there.  Returns 0, a CUDA error code, -1 when the shape is refused (more
// than 128 rows, K or a leading dimension not a multiple of 8 elements, operands not
// 16-byte aligned), -3 / -4 when the tensor map cannot be made.
MSTAR_API int mstar_gemm_skinny_bf16(const void* x, const void* W, void* out, int M, int N, int K, int ldx,
                                     int ldw, int ldo, int out_dtype, int w_static, int* error_word,
                                     void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 128 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || error_word == nullptr) return -1;
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)W & 15) != 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == MSTAR_F32)
        return sk_dispatch<float>(x, W, (float*)out, M, N, K, ldx, ldw, ldo, w_static, error_word, s);
    return sk_dispatch<bf16>(x, W, (bf16*)out, M, N, K, ldx, ldw, ldo, w_static, error_word, s);
}
