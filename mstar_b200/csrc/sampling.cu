// Token sampling from float logits, one block per request row.
//
// Options and their meaning are the reference's (mstar/utils/sampling.py:207-226):
//   repetition_penalty  seen token: x > 0 ? x / penalty : x * penalty  (:97-98)
//   temperature         0 = greedy, argmax of the penalised logits (:60-74, :151-154);
//                       otherwise softmax(x / temperature)
//   top_k               0 = off; keep the k most probable, renormalise
//   top_p               1 = off; smallest set of most probable tokens whose mass
//                       reaches top_p (after top-k); tokens tied with the last
//                       kept one are kept too
//   seed, offset        per-request Philox key and counter (:354-363, :415-416):
//                       the same (seed, offset) always draws the same token
// The reference computes probabilities with a Triton kernel and samples with a
// library call; here one kernel does penalty, max, thresholds for top-k / top-p by
// bisection over the ordered bit patterns of the logits, and an inverse-CDF draw in
// index order.  The sampled token is marked in the request's seen-mask row.
#include <cooperative_groups.h>
#include <string.h>

#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned ordered_bits(float f) {
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(unsigned u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
__device__ __forceinline__ void philox4x32_10(unsigned k0, unsigned k1, unsigned c[4]) {
    const unsigned M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
        const unsigned hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
        const unsigned n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += W0; k1 += W1;
    }
}

struct RowView {
    const float* x;
    const unsigned char* seen;  // may be null
    float penalty;
    __device__ __forceinline__ float at(int i) const {
        float v = x[i];
        if (seen != nullptr && seen[i]) v = v > 0.f ? v / penalty : v * penalty;
        return v;
    }
};

__device__ __forceinline__ float block_sum_1024(float v, float* scratch) { return block_sum(v, scratch); }

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int r = (lane < (int)(blockDim.x >> 5)) ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ penalty,
              unsigned char* __restrict__ seen_mask, const int* __restrict__ seen_rows,
              const long long* __restrict__ seed, const long long* __restrict__ offset,
              int* __restrict__ out) {
    logits = pdl_after(logits, pdl_wait());   // written by the kernel before
    __shared__ float fs[32];
    __shared__ int is[32];
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    __shared__ float scan[SAMPLE_THREADS];
    __shared__ int chosen;

    const int row = blockIdx.x, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    RowView rv;
    rv.x = logits + (size_t)row * ld;
    rv.penalty = penalty != nullptr ? penalty[row] : 1.f;
    const int srow = (seen_mask != nullptr && seen_rows != nullptr) ? seen_rows[row] : -1;
    unsigned char* my_seen = srow >= 0 ? seen_mask + (size_t)srow * vocab : nullptr;
    rv.seen = (my_seen != nullptr && rv.penalty != 1.f) ? my_seen : nullptr;

    // ---- max and argmax (smallest index among equal maxima)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = rv.at(i);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = best_v[lane]; bi = best_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { best_v[0] = bv; best_i[0] = bi; }
    }
    __syncthreads();
    const float vmax = best_v[0];
    const int amax = best_i[0];

    const float temp = temperature[row];
    if (temp <= 0.f) {
        if (tid == 0) {
            out[row] = amax;
            if (my_seen != nullptr) my_seen[amax] = 1;
        }
        return;
    }
    const float inv_temp = 1.f / temp;

    // ---- threshold tau (in ordered-bit space of the penalised logits): keep x >= tau
    unsigned tau = 0u;
    const int k = top_k != nullptr ? top_k[row] : 0;
    if (k > 0 && k < vocab) {
        // largest tau with count(x >= tau) >= k, i.e. the k-th largest value
        unsigned cur = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = cur | (1u << bit);
            int cnt = 0;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) cnt += ordered_bits(rv.at(i)) >= cand;
            cnt = block_sum_int(cnt, is);
            if (cnt >= k) cur = cand;
        }
        tau = cur;
    }
    float total = 0.f;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = rv.at(i);
        if (ordered_bits(v) >= tau) total += expf((v - vmax) * inv_temp);
    }
    total = block_sum(total, fs);

    const float p = top_p != nullptr ? top_p[row] : 1.f;
    if (p < 1.f) {
        // largest tau2 >= tau with mass(x >= tau2) >= p * total
        const float need = p * total;
        unsigned cur = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = cur | (1u << bit);
            float mass = 0.f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                const float v = rv.at(i);
                if (ordered_bits(v) >= cand) mass += expf((v - vmax) * inv_temp);
            }
            mass = block_sum(mass, fs);
            if (mass >= need) cur = cand;
        }
        if (cur > tau) {
            tau = cur;
            total = 0.f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                const float v = rv.at(i);
                if (ordered_bits(v) >= tau) total += expf((v - vmax) * inv_temp);
            }
            total = block_sum(total, fs);
        }
    }

    // ---- inverse-CDF draw over the kept tokens in index order
    unsigned c[4];
    const unsigned long long sd = seed != nullptr ? (unsigned long long)seed[row] : 0ull;
    const unsigned long long of = offset != nullptr ? (unsigned long long)offset[row] : 0ull;
    c[0] = (unsigned)of; c[1] = (unsigned)(of >> 32); c[2] = 0u; c[3] = 0u;
    philox4x32_10((unsigned)sd, (unsigned)(sd >> 32), c);
    const float u = (float)(c[0] >> 8) * (1.0f / 16777216.0f);  // [0, 1)

    const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = tid * chunk;
    const int end = min(begin + chunk, vocab);
    float mine = 0.f;
    for (int i = begin; i < end; ++i) {
        const float v = rv.at(i);
        if (ordered_bits(v) >= tau) mine += expf((v - vmax) * inv_temp);
    }
    scan[tid] = mine;
    if (tid == 0) chosen = -1;
    __syncthreads();
    // inclusive scan over the 1024 chunk sums (Hillis-Steele)
    for (int off = 1; off < SAMPLE_THREADS; off <<= 1) {
        const float add = tid >= off ? scan[tid - off] : 0.f;
        __syncthreads();
        scan[tid] += add;
        __syncthreads();
    }
    const float grand = scan[SAMPLE_THREADS - 1];
    const float target = u * grand;
    const float incl = scan[tid];
    const float excl = tid > 0 ? scan[tid - 1] : 0.f;
    if (mine > 0.f && target >= excl && target < incl) {
        float run = excl;
        int pick = -1;
        for (int i = begin; i < end; ++i) {
            const float v = rv.at(i);
            if (ordered_bits(v) >= tau) {
                run += expf((v - vmax) * inv_temp);
                pick = i;  // last kept token seen so far
                if (target < run) break;
            }
        }
        atomicMax(&chosen, pick);
    }
    __syncthreads();
    if (tid == 0) {
        // rounding can leave the target in no chunk's interval: the argmax is always kept
        const int tok = chosen >= 0 ? chosen : amax;
        out[row] = tok;
        if (my_seen != nullptr) my_seen[tok] = 1;
    }
}

// ------------------------------------------------------------------ cluster variant
// The same sampling with a thread-block cluster of 8 CTAs per row: each CTA keeps an
// eighth of the row in shared memory (the penalised logits and their exponentials), so the
// row is read from global memory once; the thresholds of top-k and top-p are found by radix
// selection (three rounds of 11, 11 and 10 bits with a histogram per round, summed across
// the cluster through distributed shared memory) instead of 32 passes of bisection each.
// The selection runs on keys that spread the row's range [min, max] linearly over 32 bits
// (a monotone map of the penalised logits: the bit patterns themselves would put nearly
// all tokens into the few bins of their common exponents, and the histogram's atomics
// would serialise); logits closer than range / 2^32 count as tied, and ties with the last
// kept token are kept, as before.  Probability mass is counted in 64-bit fixed
// point (exp * 2^40, exact integer sums), so that no sum depends on the order in which it
// is made: the same (seed, offset) always draws the same token.  With the reference's
// default options (temperature, top-p and a repetition penalty) a row of 157 k logits takes
// tens of microseconds instead of three milliseconds.
#define CS_CLUSTER 8
#define CS_THREADS 512
#define CS_BINS 2048
#define CS_SCALE 1099511627776.f      // 2^40

namespace cg = cooperative_groups;

__device__ __forceinline__ unsigned long long cs_fixed(float e) { return __float2ull_rz(e * CS_SCALE); }

// Sum of one u64 per thread over the block; every thread gets it.  `scratch`: 32 u64.
__device__ __forceinline__ unsigned long long cs_block_sum(unsigned long long v, unsigned long long* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    unsigned long long r = lane < CS_THREADS / 32 ? scratch[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

// One value per CTA -> the values of all CTAs of the cluster, in rank order.  `slot`: 8 u64
// in this CTA's shared memory (the same variable in every CTA).
__device__ __forceinline__ void cs_gather(cg::cluster_group& cluster, unsigned long long mine,
                                          unsigned long long* slot, unsigned long long (&all)[CS_CLUSTER]) {
    if (threadIdx.x == 0) slot[0] = mine;
    cluster.sync();
#pragma unroll
    for (int r = 0; r < CS_CLUSTER; ++r) all[r] = *cluster.map_shared_rank(slot, r);
    cluster.sync();          // nobody overwrites its slot before everybody has read it
}

// The bin of a radix round.  hist: this CTA's histogram (counts or masses, u64), complete for
// this CTA's threads only after the barrier inside; ghist: the cluster-wide histogram, kept
// in rank 0's shared memory and zero between rounds.  Every CTA adds its non-empty bins to it
// (remote atomics: stores, no round trips); rank 0 walks the bins from the top and finds the
// bin b where the running sum `above + sum(bins > b)` is still below `need` and `above +
// sum(bins >= b)` reaches it, and writes (b, above + sum(bins > b)) into every CTA's `result`.
// Returns b (0 if the need is never reached) and updates `above`.
__device__ __forceinline__ int cs_pick_bin(cg::cluster_group& cluster, int rank, unsigned long long* hist,
                                           unsigned long long* ghist, unsigned long long* scratch,
                                           unsigned long long* result, unsigned long long need,
                                           unsigned long long& above) {
    constexpr int PER = CS_BINS / CS_THREADS;      // bins per thread: 4
    const int tid = threadIdx.x;
    __syncthreads();                                // this CTA's histogram is complete
    unsigned long long* total = cluster.map_shared_rank(ghist, 0);
    for (int bin = tid; bin < CS_BINS; bin += CS_THREADS) {
        const unsigned long long v = hist[bin];
        if (v != 0ull) atomicAdd(total + bin, v);
    }
    cluster.sync();                                 // every CTA's bins have arrived
    if (rank == 0) {
        unsigned long long mine[PER];
        unsigned long long local = 0ull;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            mine[j] = ghist[tid * PER + j];
            ghist[tid * PER + j] = 0ull;            // ready for the next round
            local += mine[j];
        }
        // suffix sums over the threads' totals: after = sum of the bins of threads > tid
        const int lane = tid & 31, warp = tid >> 5;
        unsigned long long incl = local;            // inclusive suffix within the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_down_sync(0xffffffffu, incl, o);
            if (lane + o < 32) incl += up;
        }
        if (lane == 0) scratch[warp] = incl;        // the warp's total
        __syncthreads();
        unsigned long long after = incl - local;    // bins of higher lanes of this warp
        for (int w = warp + 1; w < CS_THREADS / 32; ++w) after += scratch[w];
        const unsigned long long before = above + after;        // everything in higher bins
        if (tid == 0) {                             // the answer if nothing reaches the need
            for (int r = 0; r < CS_CLUSTER; ++r) {
                unsigned long long* dst = cluster.map_shared_rank(result, r);
                dst[0] = 0ull;
                dst[1] = above;
            }
        }
        __syncthreads();
        if (before < need && before + local >= need) {          // at most one thread
            unsigned long long run = before;
            for (int j = PER - 1; j >= 0; --j) {
                if (run + mine[j] >= need) {
                    for (int r = 0; r < CS_CLUSTER; ++r) {
                        unsigned long long* dst = cluster.map_shared_rank(result, r);
                        dst[0] = (unsigned long long)(tid * PER + j);
                        dst[1] = run;
                    }
                    break;
                }
                run += mine[j];
            }
        }
    }
    cluster.sync();                                 // the result has been written everywhere
    above = result[1];
    return (int)result[0];
}

__global__ void __cluster_dims__(CS_CLUSTER, 1, 1) __launch_bounds__(CS_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int ld, int vocab, int chunk,
                      const float* __restrict__ temperature, const int* __restrict__ top_k,
                      const float* __restrict__ top_p, const float* __restrict__ penalty,
                      unsigned char* __restrict__ seen_mask, const int* __restrict__ seen_rows,
                      const long long* __restrict__ seed, const long long* __restrict__ offset,
                      int* __restrict__ out) {
    logits = pdl_after(logits, pdl_wait());   // written by the kernel before
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(16) unsigned char cs_smem[];
    float* sv = reinterpret_cast<float*>(cs_smem);                  // penalised logits [chunk]
    float* se = sv + chunk;                                         // exponentials [chunk]
    unsigned long long* hist = reinterpret_cast<unsigned long long*>(se + chunk);
    unsigned long long* ghist = hist + CS_BINS;
    __shared__ unsigned long long scratch[32];
    __shared__ unsigned long long slot[1];
    __shared__ unsigned long long result[2];
    __shared__ float best_v[32], low_v[32];
    __shared__ int best_i[32];

    const int row = blockIdx.x / CS_CLUSTER, rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int base = rank * chunk;
    const int n = max(0, min(chunk, vocab - base));
    const float* x = logits + (size_t)row * ld;
    const float pen = penalty != nullptr ? penalty[row] : 1.f;
    const int srow = (seen_mask != nullptr && seen_rows != nullptr) ? seen_rows[row] : -1;
    unsigned char* my_seen = srow >= 0 ? seen_mask + (size_t)srow * vocab : nullptr;
    const unsigned char* seen = (my_seen != nullptr && pen != 1.f) ? my_seen : nullptr;

    for (int b = tid; b < CS_BINS; b += CS_THREADS) ghist[b] = 0ull;   // before the first cluster barrier
    // ---- the row, once: penalty, maximum and argmax (smallest index among equal maxima)
    float bv = -INFINITY, lowest = INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < n; i += CS_THREADS) {
        float v = x[base + i];
        if (seen != nullptr && seen[base + i]) v = v > 0.f ? v / pen : v * pen;
        sv[i] = v;
        if (v > bv || (v == bv && base + i < bi)) { bv = v; bi = base + i; }
        if (v > -INFINITY) lowest = fminf(lowest, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        lowest = fminf(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
    }
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; low_v[warp] = lowest; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < CS_THREADS / 32 ? best_v[lane] : -INFINITY;
        bi = lane < CS_THREADS / 32 ? best_i[lane] : 0x7fffffff;
        lowest = lane < CS_THREADS / 32 ? low_v[lane] : INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            lowest = fminf(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
        }
        if (lane == 0) low_v[0] = lowest;
    }
    __syncthreads();
    lowest = low_v[0];
    unsigned long long all[CS_CLUSTER];
    // (value, index) packed: the ordered bits of the value above, the index below (inverted,
    // so that the larger word is the larger value or, among equals, the smaller index)
    cs_gather(cluster, ((unsigned long long)ordered_bits(bv) << 32) | (unsigned)(0x7fffffff - bi), slot, all);
    unsigned long long top = 0ull;
#pragma unroll
    for (int r = 0; r < CS_CLUSTER; ++r) top = all[r] > top ? all[r] : top;
    const float vmax = from_ordered_bits((unsigned)(top >> 32));
    const int amax = 0x7fffffff - (int)(unsigned)(top & 0xffffffffu);

    const float temp = temperature[row];
    if (temp <= 0.f) {                      // uniform over the cluster; all reads are done
        if (rank == 0 && tid == 0) {
            out[row] = amax;
            if (my_seen != nullptr) my_seen[amax] = 1;
        }
        return;
    }
    const float inv_temp = 1.f / temp;
    // the row's minimum over the cluster (ordered bits inverted: the largest word is the smallest value)
    cs_gather(cluster, (unsigned long long)(~ordered_bits(lowest)), slot, all);
    unsigned long long low_word = 0ull;
#pragma unroll
    for (int r = 0; r < CS_CLUSTER; ++r) low_word = all[r] > low_word ? all[r] : low_word;
    const float vmin = fminf(from_ordered_bits(~(unsigned)low_word), vmax);
    // exponentials, and the selection keys in place of the logits
    const double spread = vmax > vmin ? 4294967295.0 / ((double)vmax - (double)vmin) : 0.0;
    unsigned* sq = reinterpret_cast<unsigned*>(sv);
    for (int i = tid; i < n; i += CS_THREADS) {
        const float v = sv[i];
        se[i] = expf((v - vmax) * inv_temp);
        const double q = v > vmin ? ((double)v - (double)vmin) * spread : 0.0;
        sq[i] = q >= 4294967295.0 ? 0xffffffffu : (unsigned)q;
    }
    __syncthreads();

    // ---- top-k: tau = the k-th largest key, by radix selection on counts
    unsigned tau = 0u;
    const int k = top_k != nullptr ? top_k[row] : 0;
    if (k > 0 && k < vocab) {
        unsigned prefix = 0u;
        unsigned long long above = 0ull;
        int decided = 0;
        for (int round = 0; round < 3; ++round) {
            const int bits = round < 2 ? 11 : 10;
            const int shift = 32 - decided - bits;
            for (int b = tid; b < CS_BINS; b += CS_THREADS) hist[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < n; i += CS_THREADS) {
                const unsigned key = sq[i];
                if (decided == 0 || (key >> (32 - decided)) == prefix)
                    atomicAdd(&hist[(key >> shift) & ((1u << bits) - 1u)], 1ull);
            }
            const int bin = cs_pick_bin(cluster, rank, hist, ghist, scratch, result, (unsigned long long)k, above);
            prefix = (prefix << bits) | (unsigned)bin;
            decided += bits;
        }
        tau = prefix;
    }

    // ---- mass of the kept tokens
    unsigned long long mass = 0ull;
    for (int i = tid; i < n; i += CS_THREADS)
        if (sq[i] >= tau) mass += cs_fixed(se[i]);
    mass = cs_block_sum(mass, scratch);
    cs_gather(cluster, mass, slot, all);
    unsigned long long total = 0ull;
#pragma unroll
    for (int r = 0; r < CS_CLUSTER; ++r) total += all[r];

    // ---- top-p: the largest tau2 >= tau whose tokens (x >= tau2) hold p of that mass
    const float p = top_p != nullptr ? top_p[row] : 1.f;
    if (p < 1.f) {
        const unsigned long long need = (unsigned long long)((double)p * (double)total);
        unsigned prefix = 0u;
        unsigned long long above = 0ull;
        int decided = 0;
        for (int round = 0; round < 3; ++round) {
            const int bits = round < 2 ? 11 : 10;
            const int shift = 32 - decided - bits;
            for (int b = tid; b < CS_BINS; b += CS_THREADS) hist[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < n; i += CS_THREADS) {
                const unsigned key = sq[i];
                if (key >= tau && (decided == 0 || (key >> (32 - decided)) == prefix))
                    atomicAdd(&hist[(key >> shift) & ((1u << bits) - 1u)], cs_fixed(se[i]));
            }
            const int bin = cs_pick_bin(cluster, rank, hist, ghist, scratch, result, need > 0ull ? need : 1ull, above);
            prefix = (prefix << bits) | (unsigned)bin;
            decided += bits;
        }
        if (prefix > tau) {
            tau = prefix;
            mass = 0ull;
            for (int i = tid; i < n; i += CS_THREADS)
                if (sq[i] >= tau) mass += cs_fixed(se[i]);
            mass = cs_block_sum(mass, scratch);
            cs_gather(cluster, mass, slot, all);
            total = 0ull;
#pragma unroll
            for (int r = 0; r < CS_CLUSTER; ++r) total += all[r];
        }
    }

    // ---- inverse-CDF draw over the kept tokens in index order (exact integer prefix sums)
    unsigned c[4];
    const unsigned long long sd = seed != nullptr ? (unsigned long long)seed[row] : 0ull;
    const unsigned long long of = offset != nullptr ? (unsigned long long)offset[row] : 0ull;
    c[0] = (unsigned)of; c[1] = (unsigned)(of >> 32); c[2] = 0u; c[3] = 0u;
    philox4x32_10((unsigned)sd, (unsigned)(sd >> 32), c);
    const double u = (double)(c[0] >> 8) * (1.0 / 16777216.0);   // [0, 1)
    unsigned long long target = (unsigned long long)(u * (double)total);
    if (target >= total) target = total - 1;                      // total > 0: the maximum counts 2^40
    unsigned long long before_me = 0ull;                          // mass of the CTAs of lower rank
#pragma unroll
    for (int r = 0; r < CS_CLUSTER; ++r)
        if (r < rank) before_me += all[r];
    if (target >= before_me && target < before_me + all[rank]) {  // the token is in this CTA
        const int per = (n + CS_THREADS - 1) / CS_THREADS;
        const int begin = min(tid * per, n), end = min(begin + per, n);
        unsigned long long mine = 0ull;
        for (int i = begin; i < end; ++i)
            if (sq[i] >= tau) mine += cs_fixed(se[i]);
        // exclusive prefix of `mine` over the threads
        unsigned long long incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        __syncthreads();
        if (lane == 31) scratch[warp] = incl;
        __syncthreads();
        unsigned long long excl = before_me + incl - mine;
        for (int w = 0; w < warp; ++w) excl += scratch[w];
        if (mine > 0ull && target >= excl && target < excl + mine) {
            unsigned long long run = excl;
            int pick = amax;
            for (int i = begin; i < end; ++i) {
                if (sq[i] >= tau) {
                    run += cs_fixed(se[i]);
                    if (target < run) { pick = base + i; break; }
                }
            }
            out[row] = pick;
            if (my_seen != nullptr) my_seen[pick] = 1;
        }
    }
}

static int cs_chunk(int vocab) { return ((vocab + CS_CLUSTER - 1) / CS_CLUSTER + 3) & ~3; }
static size_t cs_smem_bytes(int vocab) {
    return (size_t)cs_chunk(vocab) * 8 + 2 * CS_BINS * sizeof(unsigned long long);
}

MSTAR_API int mstar_sample(const float* logits, int ld, int rows, int vocab,
                           const float* temperature, const int* top_k, const float* top_p,
                           const float* penalty, unsigned char* seen_mask, const int* seen_rows,
                           const long long* seed, const long long* offset, int* out,
                           void* stream) {
    if (rows <= 0) return 0;
    // rows of up to ~200 k logits fit the shared memory of a cluster of 8 CTAs
    static int one_block = -1;          // MSTAR_SAMPLER=block: the one-block-per-row kernel
    if (one_block < 0) {
        const char* e = getenv("MSTAR_SAMPLER");
        one_block = (e != nullptr && strcmp(e, "block") == 0) ? 1 : 0;
    }
    const size_t smem = cs_smem_bytes(vocab);
    if (!one_block && smem <= 200 * 1024 && rows <= 65535 / CS_CLUSTER * CS_CLUSTER) {
        static size_t configured = 0;
        if (smem > configured) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = smem;
        }
        mstar_launch((sample_cluster_kernel), dim3(rows * CS_CLUSTER), dim3(CS_THREADS), smem,
                     (cudaStream_t)stream, logits, ld, vocab, cs_chunk(vocab), temperature, top_k, top_p,
                     penalty, seen_mask, seen_rows, seed, offset, out);
        return launch_status();
    }
    mstar_launch((sample_kernel), dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, 
        logits, ld, vocab, temperature, top_k, top_p, penalty, seen_mask, seen_rows, seed, offset,
        out);
    return launch_status();
}

// Greedy only: argmax of each row (smallest index among equal maxima).  A row is cut into
// `gridDim.y` pieces, a CTA each (one CTA alone reads a row of 157 k logits in some 15 us, at
// the rate of a single SM); a piece's best is a 64-bit key, the value's ordered bits above the
// complemented index, so that the maximum over keys is the largest value and, among equal
// values, the smallest index; keys meet in `best[row]` by atomicMax, and the CTA that counts
// itself last at `arrived[row]` writes the token and puts both back to zero for the next
// launch.  Nobody waits.  `best` and `arrived` must be zero at the first launch and belong to
// one stream at a time.
#define ARGMAX_THREADS 256
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out,
              unsigned long long* __restrict__ best, int* __restrict__ arrived) {
    logits = pdl_after(logits, pdl_wait());   // written by the kernel before
    __shared__ unsigned long long best_k[ARGMAX_THREADS / 32];
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * ld;
    // this CTA's piece: whole groups of four, so that aligned rows are read 16 bytes at a time
    const int groups = (vocab + 3) / 4;
    const int per = (groups + (int)gridDim.y - 1) / (int)gridDim.y;
    const int g0 = (int)blockIdx.y * per, g1 = min(groups, g0 + per);
    const bool vec = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    unsigned long long key = 0ull;             // below every real key (ordered bits are never 0 for a number)
    auto take = [&](float f, int i) {
        f = f == f ? f : -INFINITY;                                   // a NaN never wins
        const unsigned long long k =
            ((unsigned long long)ordered_bits(f) << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
        key = k > key ? k : key;
    };
    int g = g0 + tid;
    if (vec) {
        // four loads of 16 bytes in flight per thread
        for (; g + 3 * ARGMAX_THREADS < g1 && 4 * (g + 3 * ARGMAX_THREADS) + 3 < vocab; g += 4 * ARGMAX_THREADS) {
            float4 q[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) q[u] = *reinterpret_cast<const float4*>(x + 4 * (g + u * ARGMAX_THREADS));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i0 = 4 * (g + u * ARGMAX_THREADS);
                take(q[u].x, i0);
                take(q[u].y, i0 + 1);
                take(q[u].z, i0 + 2);
                take(q[u].w, i0 + 3);
            }
        }
    }
    for (; g < g1; g += ARGMAX_THREADS) {
        const int i0 = 4 * g;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (i0 + j < vocab) take(x[i0 + j], i0 + j);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = other > key ? other : key;
    }
    if (lane == 0) best_k[warp] = key;
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int w = 1; w < ARGMAX_THREADS / 32; ++w) key = best_k[w] > key ? best_k[w] : key;
        atomicMax(best + row, key);
        __threadfence();
        if (atomicAdd(arrived + row, 1) == (int)gridDim.y - 1) {
            __threadfence();
            const unsigned long long top = atomicExch(best + row, 0ull);
            out[row] = (int)(0xffffffffu - (unsigned)(top & 0xffffffffull));
            arrived[row] = 0;
        }
    }
}

// `best` [rows] of 64 bits and `arrived` [rows] ints: scratch that is zero before the first
// launch; the kernel leaves it zero.
MSTAR_API int mstar_argmax(const float* logits, int ld, int rows, int vocab, int* out, void* best,
                           int* arrived, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || best == nullptr || arrived == nullptr) return -1;
    // pieces of 8 k logits or more, as many CTAs as fill the GPU about once (eight of these
    // CTAs fit on an SM)
    int pieces = (vocab + 8191) / 8192;
    const int fit = 8 * device_sm_count() / rows;
    if (pieces > fit) pieces = fit;
    if (pieces < 1) pieces = 1;
    if (pieces > 64) pieces = 64;
    mstar_launch((argmax_kernel), dim3(rows, pieces), dim3(ARGMAX_THREADS), 0, (cudaStream_t)stream, logits, ld,
                 vocab, out, (unsigned long long*)best, arrived);
    return launch_status();
}
