// Paged causal prefill attention on the fifth-generation tensor cores (tcgen05), bfloat16,
// head_dim 64, 128 or 256.  Same semantics as attention_prefill.cu (rows are (token, query head of
// the group) pairs, causal end-aligned mask, float softmax); what differs is where the
// work runs.
//
// One CTA owns the rows of 128 / G whole tokens (G query heads per kv head: 128 rows, or
// 126 where G is 3) and one kv head; the CTAs with the most keys are launched first.  Its
// query rows come by one TMA copy per 64 features: a box of [tokens x G heads x 64] from the
// projection's output lands as the K-major swizzled tile that the MMA reads (loads and
// stores by the softmax threads took 5 to 9 us per CTA before the first product could start).
// Per tile of 64 keys:
//   * two producer warps bring the keys and the values by TMA (one box of [page_size x 64]
//     per page and 64-feature half, 128-byte swizzle, issued side by side from several
//     lanes) into two rings of two stages;
//   * a lane of the S warp issues S = Q K^T as tcgen05.mma (M 128, N 64, K 16 per step) into
//     one of two buffers in tensor memory, a tile ahead of the softmax threads: the buffer
//     is free when O += P V of the tile before last is done;
//   * 128 softmax threads each own one row: they read their row of S from tensor memory
//     (tcgen05.ld; the row maximum and sum need no shuffles), and write the probabilities
//     as packed bfloat16 over the first half of the same row (tcgen05.st), so P never
//     passes through shared memory; they rescale their row of the running output O in
//     tensor memory only when the row maximum grew by more than 2^8;
//   * a lane of the O warp issues O += P V (M 128, N head_dim, K 16 x 4) with P as the A
//     operand from tensor memory and V as the N-major B operand straight from the
//     cache's [key][feature] tiles.
// At the end each thread reads its row of O, divides by the softmax sum and stores.
// At head_dim 128 two CTAs fit on an SM (97 KB of shared memory, 256 TMEM columns each:
// S and P 2 x 64, O 128), so one CTA's softmax overlaps the other's MMAs; at 64 there is
// room for more, at 256 (193 KB, 512 columns) for one.
//
// With one prompt alone the CTAs are few (a few hundred, of 1 to 32 key tiles) and the
// longest sets the time.  Sharing the long row tiles between two CTAs was built twice and is
// not kept: as a cluster of two with the second CTA's part read through distributed shared
// memory (63 us instead of 42 for 2,048 tokens: launched as clusters the CTAs no longer
// overlapped on the SMs), and as independent CTAs that leave their parts in scratch memory,
// the one that comes second adding them up (46 to 56 us against 38: a CTA's start and end
// cost as much as four key tiles, writing and reading a part as much as seven).
//
// Shared-memory descriptors: Q and K are K-major with the 128-byte swizzle (8-row groups
// 1024 bytes apart); V is MN-major (features contiguous): 8-key groups 1024 bytes apart
// (stride byte offset), the 64-feature blocks 8192 bytes apart (leading byte offset).
// Every mbarrier wait is bounded; a timeout is recorded in the error word.
//
// The reference calls a library for this (mstar/utils/flashinfer_utils.py:136-156).
#include <string.h>

#include "common.cuh"
#include "tma_util.cuh"

#define PT_ROWS 128
#define PT_KEYS 64
#define PT_THREADS 256  // 4 softmax warps, the S-issuing warp, the key warp, the O-issuing warp, the value warp

struct PrefillTcArgs {
    const int* block_table;
    const int* qo_indptr;
    const int* kv_len;
    bf16* out;
    int bt_stride, nq, nkv, page_size, first_entry;
    float scale_log2e;
};

__device__ __forceinline__ void pt_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pt_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pt_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void pt_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the same with the A operand in tensor memory (M lanes x K/2 columns of packed pairs)
__device__ __forceinline__ void pt_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void pt_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void pt_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
          "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
          "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
          "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void pt_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void pt_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// A wait of a whole warp whose outcome all its lanes share: the tcgen05.ld / st that follow
// are warp-wide instructions and must not be reached by a part of the warp only.
__device__ __forceinline__ bool pt_wait_warp(uint32_t bar, uint32_t parity) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity)) != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void pt_tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0,
                                               int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
        "%4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// descriptor bits common to all operands here: version 1 [46,48), SWIZZLE_128B [61,64)
__device__ __forceinline__ uint64_t pt_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D float, A and B bfloat16, b_major (bit 16) = 1 for an
// MN-major B operand
__host__ __device__ constexpr uint32_t pt_idesc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Shared memory of one CTA: Q as blocks of [128 rows x 64 features], two stages of keys and
// two of values as blocks of [64 keys x 64 features], then the barriers.
__host__ __device__ constexpr int pt_q_bytes(int hd) { return PT_ROWS * hd * 2; }
__host__ __device__ constexpr int pt_kv_tile(int hd) { return PT_KEYS * hd * 2; }
__host__ __device__ constexpr int pt_smem(int hd) { return pt_q_bytes(hd) + 4 * pt_kv_tile(hd) + 128; }
// What a launch asks for: at head_dim 64 more than the kernel uses, so that no more CTAs
// land on an SM than its 512 TMEM columns serve (a further one would wait in its allocation).
__host__ __device__ constexpr int pt_smem_launch(int hd) { return pt_smem(hd) < 77 * 1024 ? 77 * 1024 : pt_smem(hd); }
// Tensor memory: S / P 2 x 64 columns, O head_dim; allocations are powers of two.
__host__ __device__ constexpr uint32_t pt_tmem_cols(int hd) { return hd <= 128 ? 256u : 512u; }
// The running maximum of a row follows the tile maxima only when they exceed it by more
// than this (in powers of two): probabilities then reach 2^8 at most, which float sums and
// bfloat16's relative precision take, and the output in tensor memory is rarely rescaled.
#define PT_MAX_SLACK 8.0f

__device__ __forceinline__ float pt_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD>
__global__ void __launch_bounds__(PT_THREADS)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap kv_map,
                            const __grid_constant__ CUtensorMap q_map, PrefillTcArgs a,
                            int* __restrict__ error_word) {
    constexpr int PT_Q_BYTES = pt_q_bytes(HD), PT_KV_TILE = pt_kv_tile(HD);
    constexpr int NB = HD / 64;                     // 64-feature blocks of a row
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char* q_s = smem_dyn;
    unsigned char* k_s = q_s + PT_Q_BYTES;          // [2 stages]
    unsigned char* v_s = k_s + 2 * PT_KV_TILE;      // [2 stages]
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * PT_KV_TILE);
    // k_full[2], v_full[2]: a stage's copies have landed.  k_empty[2]: S of the stage's tile
    // is done.  v_empty[2]: O += P V of the stage's tile is done (the values may be refilled,
    // the tile's S / P buffer overwritten by S of the tile after next, O rescaled or read).
    // s_full[2]: S of a tile is done.  p_ready[2]: P of a tile is written (one arrival per
    // softmax thread).  All go through one phase per two tiles.
    const uint32_t k_full = tc_smem(bars + 0), v_full = tc_smem(bars + 2), k_empty = tc_smem(bars + 4),
                   v_empty = tc_smem(bars + 6), p_ready = tc_smem(bars + 8), s_full = tc_smem(bars + 10);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);

    // grid: x the kv head, y the row tile with the longest first (the tiles with the most keys
    // are launched before the short ones), z the entry
    const int tile = gridDim.y - 1 - blockIdx.y, e = a.first_entry + blockIdx.z;
    const int kvh = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.nq / a.nkv;
    const int TPT = PT_ROWS / G, RPT = TPT * G;      // tokens and rows of a tile
    const int q_start = a.qo_indptr[e];
    const int q_len = a.qo_indptr[e + 1] - q_start;
    const int tok0 = tile * TPT;
    if (tok0 >= q_len) return;
    if ((tc_smem(smem_dyn) & 1023u) != 0) {         // the swizzled tiles need this alignment
        if (tid == 0) atomicExch(error_word, 6);
        return;
    }
    const int past = a.kv_len[e] - q_len;
    const int hi = past + min(q_len, tok0 + TPT);   // keys 0 .. hi-1 are visible to some row
    const int ntiles = (hi + PT_KEYS - 1) / PT_KEYS;
    const int* bt = a.block_table + (size_t)e * a.bt_stride;
    const int ps = a.page_size;

    const uint32_t q_ready = tc_smem(bars + 12);
    if (tid == 0) {
        for (int i = 0; i < 13; ++i)
            mbar_init(tc_smem(bars + i), i == 8 || i == 9 ? 128 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid >= RPT && tid < PT_ROWS) {
        // rows of the tile that the copy of the query rows leaves out (128 is no multiple of G)
        for (int c = 0; c < HD / 8; ++c)
            *reinterpret_cast<uint4*>(q_s + (c >> 3) * (PT_ROWS * 128) + tid * 128 + (c & 7) * 16) =
                make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         tc_smem(tmem_slot)),
                     "r"(pt_tmem_cols(HD))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pt_fence_before();
    __syncthreads();
    pt_fence_after();
    const uint32_t tmem = *tmem_slot;
    // S / P: two buffers of 64 columns; a tile's S (64 floats per row) is replaced in place by
    // its P (64 packed bfloat16 = 32 columns), each thread overwriting what it alone has read
    const uint32_t tmem_sp = tmem;
    const uint32_t tmem_o = tmem + 128;   // O: head_dim columns from 128 on

    if (warp == 5 || warp == 7) {
        // ------------------------------------------- TMA producers: warp 5 the keys, 7 the values
        // All lanes run the loop: they fetch 32 block-table entries at a time (one dependent
        // global load per page would cost more than the copies); lane NB p + h waits for the
        // stage and copies block h of page p (at most 8 pages x 4 blocks), side by side with
        // the others.  Keys and values have a warp each and the loop is kept short (page
        // sizes are powers of two: shifts; no exchange between the lanes but the page
        // numbers): one warp doing both, with divisions, took 1,850 cycles per tile, which
        // was the whole kernel's pace.
        const int which = warp == 7;
        const int ps_log = 31 - __clz(ps);
        const int last_page = (hi - 1) >> ps_log;
        // a tile is 1, 2, 4 or 8 whole pages, or, with pages of 128 or 256 keys, a part of one
        const int per_tile = ps < PT_KEYS ? PT_KEYS >> ps_log : 1;
        const int box_rows = ps < PT_KEYS ? ps : PT_KEYS;
        const int p = lane / NB, h = lane % NB;
        const bool issues = p < per_tile;
        const uint32_t full0 = which ? v_full : k_full, empty0 = which ? v_empty : k_empty;
        const uint32_t dst0 = tc_smem(which ? v_s : k_s) + (uint32_t)(h * (PT_KEYS * 128) + p * box_rows * 128);
        // row of the cache seen as a matrix: ((page * 2 + which) * nkv + kvh) * ps + key in page
        const int page_rows = 2 * a.nkv * ps, row0 = (which * a.nkv + kvh) * ps;
        if (which == 0 && lane == 0) {
            // the query rows: tokens tok0 .. tok0+TPT-1 (past the last row of the batch: zeros)
            mbar_expect_tx(q_ready, (uint32_t)(NB * RPT * 128));
            for (int hh = 0; hh < NB; ++hh)
                pt_tma_load_4d(tc_smem(q_s + hh * (PT_ROWS * 128)), &q_map, q_ready, hh * 64, 0, kvh,
                               q_start + tok0);
        }
        int mine = 0, have_from = -1;                 // lanes hold pages have_from .. +31
        bool ok = true;
        for (int j = 0; j < ntiles; ++j) {
            const int s = j & 1;
            const uint32_t free_parity = (((uint32_t)j >> 1) & 1u) ^ 1u;
            const int key0 = j * PT_KEYS;
            const int base_page = key0 >> ps_log;
            const int in_page = key0 & (ps - 1);      // 0 unless the page is larger than the tile
            if (have_from < 0 || base_page + per_tile > have_from + 32) {
                have_from = base_page;
                // pages beyond the last are replaced by the last: masked rows stay finite
                mine = bt[min(base_page + lane, last_page)];
            }
            const int page = __shfl_sync(0xffffffffu, mine, (base_page + p - have_from) & 31);
            if (issues) {
                // the stage is free once S (keys) or O += P V (values) of tile j-2 is done
                if (!mbar_wait(empty0 + 8 * s, free_parity)) {
                    atomicExch(error_word, 7);
                    ok = false;
                } else {
                    // the bytes may land before lane 0 has announced them: the phase cannot
                    // end before its one arrival
                    if (lane == 0) mbar_expect_tx(full0 + 8 * s, PT_KV_TILE);
                    tma_load_2d(dst0 + (uint32_t)(s * PT_KV_TILE), &kv_map, full0 + 8 * s, h * 64,
                                page * page_rows + row0 + in_page);
                }
            }
            if (!__all_sync(0xffffffffu, ok)) break;
        }
    } else if (warp == 4) {
        // ------------------------------------------------ S = Q K^T, while the softmax works on
        // the tile before
        if (lane == 0) {
            constexpr uint32_t idesc_s = pt_idesc(PT_ROWS, PT_KEYS, 0);
            const uint32_t q_addr = tc_smem(q_s);
            bool q_there = mbar_wait(q_ready, 0);
            if (!q_there) atomicExch(error_word, 8);
            for (int j = 0; j < ntiles && q_there; ++j) {
                const int s = j & 1;
                const uint32_t parity = ((uint32_t)j >> 1) & 1u;
                if (!mbar_wait(k_full + 8 * s, parity)) {
                    atomicExch(error_word, 8);
                    break;
                }
                // 8 k-steps of 16 features; features 64.. live in the second half-tile.  The
                // descriptors are made before the wait that the softmax threads end.
                const uint32_t k_addr = tc_smem(k_s + s * PT_KV_TILE);
                uint64_t dq[HD / 16], dk[HD / 16];
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    dq[kk] = pt_desc(q_addr + (uint32_t)(kk >> 2) * (PT_ROWS * 128) + (uint32_t)(kk & 3) * 32, 16, 1024);
                    dk[kk] = pt_desc(k_addr + (uint32_t)(kk >> 2) * (PT_KEYS * 128) + (uint32_t)(kk & 3) * 32, 16, 1024);
                }
                // the buffer is free once O += P V of tile j-2, which read P from it, is done:
                // S runs a tile ahead of the softmax threads
                if (j >= 2 && !mbar_wait(v_empty + 8 * s, (((uint32_t)j >> 1) & 1u) ^ 1u)) {
                    atomicExch(error_word, 8);
                    break;
                }
                pt_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    pt_mma(tmem_sp + (uint32_t)s * 64, dq[kk], dk[kk], idesc_s, kk != 0);
                pt_commit(s_full + 8 * s);
                pt_commit(k_empty + 8 * s);
            }
        }
    } else if (warp == 6) {
        // ------------------------------------------------ O += P V, V the N-major operand
        if (lane == 0) {
            constexpr uint32_t idesc_o = pt_idesc(PT_ROWS, HD, 1);
            for (int j = 0; j < ntiles; ++j) {
                const int s = j & 1;
                const uint32_t parity = ((uint32_t)j >> 1) & 1u;
                if (!mbar_wait(v_full + 8 * s, parity)) {
                    atomicExch(error_word, 9);
                    break;
                }
                // the softmax threads have replaced S by P and rescaled O where needed
                if (!mbar_wait(p_ready + 8 * s, parity)) {
                    atomicExch(error_word, 9);
                    break;
                }
                pt_fence_after();
                // 4 k-steps of 16 keys (8 columns of packed P); V rows are keys, 8-key
                // groups 1024 bytes apart, the two 64-feature halves 8192 bytes apart
                const uint32_t v_addr = tc_smem(v_s + s * PT_KV_TILE);
#pragma unroll
                for (int kk = 0; kk < PT_KEYS / 16; ++kk) {
                    const uint64_t db = pt_desc(v_addr + (uint32_t)kk * 16 * 128, PT_KEYS * 128, 1024);
                    pt_mma_ts(tmem_o, tmem_sp + (uint32_t)s * 64 + (uint32_t)kk * 8, db, idesc_o, (j | kk) != 0);
                }
                pt_commit(v_empty + 8 * s);   // the values are consumed, O holds tiles 0..j
            }
        }
    } else if (warp < 4) {
        // ------------------------------------------------------ softmax, one row per thread
        const int r = tid;                              // row of the tile = TMEM lane
        const int tok = tok0 + min(r, RPT - 1) / G;
        const bool valid = r < RPT && tok < q_len;
        const int cp = past + min(tok, q_len - 1);      // newest key this row sees
        const int cp_min = past + tok0;                 // ... and any row of this CTA
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const float scale = a.scale_log2e;
        float m = -INFINITY, l = 0.f;     // m: the reference maximum, in scaled (log2) units
        bool ok = true;
        for (int j = 0; j < ntiles; ++j) {
            if (!pt_wait_warp(s_full + 8 * (j & 1), ((uint32_t)j >> 1) & 1u)) {
                if (lane == 0) atomicExch(error_word, 10);
                ok = false;
                break;
            }
            pt_fence_after();
            uint32_t s0[32], s1[32];
            pt_ld32(tmem_sp + lane_off + (uint32_t)(j & 1) * 64, s0);
            pt_ld32(tmem_sp + lane_off + (uint32_t)(j & 1) * 64 + 32, s1);
            pt_wait_ld();
            const int key0 = j * PT_KEYS;
            if (key0 + PT_KEYS - 1 > cp_min) {            // the tile touches the diagonal
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (key0 + i > cp) s0[i] = 0xff800000u;          // -inf
                    if (key0 + 32 + i > cp) s1[i] = 0xff800000u;
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                mx0 = fmaxf(mx0, __uint_as_float(s0[i]));
                mx1 = fmaxf(mx1, __uint_as_float(s1[i]));
            }
            const float mx = fmaxf(mx0, mx1) * scale;     // scale > 0
            // key 0 is visible to every row, so m is finite from the first tile on
            float alpha = 1.f;
            if (mx > m + PT_MAX_SLACK) {
                alpha = pt_ex2(m - mx);
                m = mx;
            }
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t packed[32];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float p0 = pt_ex2(fmaf(__uint_as_float(s0[i]), scale, -m));
                const float p1 = pt_ex2(fmaf(__uint_as_float(s0[i + 1]), scale, -m));
                const float p2 = pt_ex2(fmaf(__uint_as_float(s1[i]), scale, -m));
                const float p3 = pt_ex2(fmaf(__uint_as_float(s1[i + 1]), scale, -m));
                sum0 += p0 + p1;
                sum1 += p2 + p3;
                __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi2 = __floats2bfloat162_rn(p2, p3);
                packed[i >> 1] = *reinterpret_cast<uint32_t*>(&lo);
                packed[16 + (i >> 1)] = *reinterpret_cast<uint32_t*>(&hi2);
            }
            l = l * alpha + (sum0 + sum1);
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // O += P V of tile j-1 must be done before O is rescaled
                if (!pt_wait_warp(v_empty + 8 * ((j - 1) & 1), ((uint32_t)(j - 1) >> 1) & 1u)) {
                    if (lane == 0) atomicExch(error_word, 11);
                    ok = false;
                    break;
                }
                pt_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t o[32];
                    pt_ld32(tmem_o + lane_off + (uint32_t)c0, o);
                    pt_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    pt_st32(tmem_o + lane_off + (uint32_t)c0, o);
                }
            }
            // P over the first half of this row's S: column c holds keys 2c, 2c+1
            pt_st32(tmem_sp + lane_off + (uint32_t)(j & 1) * 64, packed);
            pt_wait_st();
            pt_fence_before();
            mbar_arrive(p_ready + 8 * (j & 1));
        }
        if (ok && !pt_wait_warp(v_empty + 8 * ((ntiles - 1) & 1), ((uint32_t)(ntiles - 1) >> 1) & 1u)) {
            if (lane == 0) atomicExch(error_word, 12);
            ok = false;
        }
        pt_fence_after();
        // ---------------------------------------------------------------- epilogue
        // (`ok` is the same in all lanes of a warp; rows past the entry's last token are read
        // with the others, the load being a warp's, and not stored)
        if (ok) {
            const float inv = 1.f / l;
            bf16* dst = a.out + (size_t)(q_start + tok) * a.nq * HD + (size_t)(kvh * G + r % G) * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t o[32];
                pt_ld32(tmem_o + lane_off + (uint32_t)c0, o);
                pt_wait_ld();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float f[8];
#pragma unroll
                        for (int t = 0; t < 8; ++t) f[t] = __uint_as_float(o[8 * i + t]) * inv;
                        store8(dst + c0 + 8 * i, f);
                    }
                }
            }
        }
    }
    pt_fence_before();
    __syncthreads();
    if (warp == 4) {
        pt_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(pt_tmem_cols(HD))
                     : "memory");
    }
}

template <int HD>
static int launch_prefill_tc(const CUtensorMap& map, const CUtensorMap& q_map, const PrefillTcArgs& a,
                             dim3 grid, int* error_word, cudaStream_t stream) {
    auto kernel = prefill_attention_tc_kernel<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             pt_smem_launch(HD));
        if (e != cudaSuccess) return (int)e;
        // several CTAs per SM need nearly all of the SM's shared memory
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    kernel<<<grid, PT_THREADS, pt_smem_launch(HD), stream>>>(map, q_map, a, error_word);
    return launch_status();
}

// Entries [first_entry, first_entry + entries) of the batch.  head_dim must be 64, 128 or
// 256, the page size 8..64 dividing 64, or 128 or 256, no window, at most 128 query heads per
// kv head.  `kv_map`: the cache's tensor map.  `q`: `q_rows` rows of `q_stride` elements, of
// which the first nq * hd are the query heads; 16-byte aligned, the stride a multiple of 8.
// Returns 0, a CUDA error code or -1 (shape refused).  `error_word` receives 6..12 if a wait
// ran out (6: the shared memory was not aligned as the swizzle needs).
MSTAR_API int mstar_paged_prefill_attention_tc(
    const void* kv_map, const void* q, int q_stride, int q_rows, void* out, const int* block_table, int bt_stride,
    const int* qo_indptr, const int* kv_len, int first_entry, int entries, int max_q_len, int nq,
    int nkv, int hd, int page_size, float scale, int* error_word, void* stream) {
    if (entries <= 0 || max_q_len <= 0) return 0;
    if ((hd != 64 && hd != 128 && hd != 256) || !(scale > 0.f) || nkv <= 0 || nq % nkv != 0 ||
        kv_map == nullptr || error_word == nullptr)
        return -1;
    if (!((page_size >= 8 && page_size <= 64 && PT_KEYS % page_size == 0) || page_size == 128 ||
          page_size == 256))
        return -1;
    if (entries > 65535) return -1;
    const int G = nq / nkv;
    if (G > PT_ROWS || q == nullptr || q_rows <= 0 || ((uintptr_t)q & 15) != 0 || q_stride % 8 != 0 ||
        q_stride < nq * hd)
        return -1;
    const int per_tile = PT_ROWS / G;                     // tokens of a row tile
    // the query rows as [token][kv head][head of the group][feature]; a box is a tile's rows
    // for one kv head and 64 features
    CUtensorMap q_map;
    {
        EncodeTiledFn encode = encode_tiled_fn();
        if (encode == nullptr) return (int)cudaErrorNotSupported;
        const cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)G, (cuuint64_t)nkv, (cuuint64_t)q_rows};
        const cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)G * hd * 2, (cuuint64_t)q_stride * 2};
        const cuuint32_t box[4] = {64, (cuuint32_t)G, 1, (cuuint32_t)per_tile};
        const cuuint32_t elem[4] = {1, 1, 1, 1};
        if (encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(q), dims, strides, box,
                   elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return -1;
    }
    PrefillTcArgs a;
    a.block_table = block_table;
    a.qo_indptr = qo_indptr;
    a.kv_len = kv_len;
    a.out = (bf16*)out;
    a.bt_stride = bt_stride;
    a.nq = nq;
    a.nkv = nkv;
    a.page_size = page_size;
    a.first_entry = first_entry;
    a.scale_log2e = scale * 1.4426950408889634f;
    CUtensorMap map;
    memcpy(&map, kv_map, sizeof(map));
    const long long tiles = ((long long)max_q_len + per_tile - 1) / per_tile;
    if (tiles > 65535) return -1;
    dim3 grid(nkv, (unsigned)tiles, entries);
    cudaStream_t s = (cudaStream_t)stream;
    switch (hd) {
        case 64: return launch_prefill_tc<64>(map, q_map, a, grid, error_word, s);
        case 128: return launch_prefill_tc<128>(map, q_map, a, grid, error_word, s);
        default: return launch_prefill_tc<256>(map, q_map, a, grid, error_word, s);
    }
}
