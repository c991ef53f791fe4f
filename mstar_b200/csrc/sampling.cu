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
    pdl_wait();
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

MSTAR_API int mstar_sample(const float* logits, int ld, int rows, int vocab,
                           const float* temperature, const int* top_k, const float* top_p,
                           const float* penalty, unsigned char* seen_mask, const int* seen_rows,
                           const long long* seed, const long long* offset, int* out,
                           void* stream) {
    if (rows <= 0) return 0;
    mstar_launch((sample_kernel), dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, 
        logits, ld, vocab, temperature, top_k, top_p, penalty, seen_mask, seen_rows, seed, offset,
        out);
    return launch_status();
}

// Greedy only: argmax of each row (smallest index among equal maxima).
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out) {
    pdl_wait();
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * ld;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = x[i];
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
        if (lane == 0) out[row] = bi;
    }
}

MSTAR_API int mstar_argmax(const float* logits, int ld, int rows, int vocab, int* out,
                           void* stream) {
    if (rows <= 0) return 0;
    mstar_launch((argmax_kernel), dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, ld, vocab, out);
    return launch_status();
}
