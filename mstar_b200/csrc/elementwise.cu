// Memory-bound kernels of the decoder: embedding gather, fused residual-add +
// RMSNorm, rotary position encoding fused with the write of keys and values into
// cache pages, SiLU(gate)*up, row gather, dtype conversion.
//
// Formulas follow the reference model: RMSNorm x*rsqrt(mean(x^2)+eps)*w
// (mstar/model/components/norm.py:45-59, mstar/utils/attention.py:457-474),
// split-half rotary pairs (mstar/utils/attention.py:224-253), down(silu(gate)*up)
// (mstar/model/components/distributed/mlp.py:78-81), plain residual adds
// (mstar/model/components/decoder_layer.py:58-71).  The residual stream is kept in
// float in both dtypes so that the residual sum is a 32-bit sum.
#include <stdlib.h>

#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[t] = float(table[id]) with id = ids[t], or, where `src` is given and src[t] >= 0,
// id = prev[src[t]]: a token that the step before sampled and that is still on the device
// (the engine launches a step before it has read the last one's tokens).
template <typename W>
__global__ void embed_rows_kernel(const W* __restrict__ table, const int* __restrict__ ids,
                                  const int* __restrict__ src, const int* __restrict__ prev,
                                  float* __restrict__ out, int vocab, int hidden, float scale) {
    prev = pdl_after(prev, pdl_wait());       // sampled by the step before
    const int t = blockIdx.x;
    int id = ids[t];
    if (src != nullptr) {
        const int from = src[t];
        if (from >= 0) id = prev[from];
    }
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {  // host validates ids; never read out of the table
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const W* row = table + (size_t)id * hidden;
    if (scale == 1.f)
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
    else
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// `src` and `prev` are both null or both given (src: [num_tokens] ints, -1 where ids holds
// the token; prev: int tokens on the device).  Rows are multiplied by `scale` in float.
MSTAR_API int mstar_embed_rows(const void* table, int table_dtype, const int* ids, const int* src,
                               const int* prev, float* out, int num_tokens, int vocab, int hidden,
                               float scale, void* stream) {
    if (num_tokens <= 0) return 0;
    if ((src == nullptr) != (prev == nullptr)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == MSTAR_F32)
        mstar_launch((embed_rows_kernel<float>), dim3(num_tokens), dim3(threads), 0, s, (const float*)table, ids,
                     src, prev, out, vocab, hidden, scale);
    else
        mstar_launch((embed_rows_kernel<bf16>), dim3(num_tokens), dim3(threads), 0, s, (const bf16*)table, ids,
                     src, prev, out, vocab, hidden, scale);
    return launch_status();
}

// ------------------------------------------------- residual add + RMSNorm
// resid (float, [rows, hidden]) is updated in place with resid + delta when delta
// is given; out = resid * rsqrt(mean(resid^2) + eps) * (w + w_offset) in type A.
// One block per row.  The sum of squares is accumulated per thread over a fixed
// stride and then reduced in a fixed tree, so a row's result does not depend on
// which other rows are in the batch.  `resid_static`: nonzero promises that the kernel
// before this one on the stream did not write resid (it wrote delta), so resid may be
// read while that kernel is still draining.
template <typename A, typename W, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const A* __restrict__ delta,
                                   const W* __restrict__ weight, A* __restrict__ out, int hidden,
                                   float eps, float w_offset, int resid_static) {
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * hidden;
    float* r = resid + base;
    float ss = 0.f;
    if (VEC) {
        // eight elements per thread and step, 16-byte accesses; the order in which a row's
        // squares are summed depends only on the row's width and the block size
        const int chunks = hidden >> 3;
        if (chunks <= 2 * (int)blockDim.x) {
            // a thread's one or two chunks stay in registers.  The weight is a parameter, and
            // with `resid_static` the kernel before this one wrote the delta only: both are
            // asked for while that kernel is still draining.
            const int c0 = threadIdx.x, c1 = threadIdx.x + blockDim.x;
            const bool h0 = c0 < chunks, h1 = c1 < chunks;
            float v0[8], v1[8], w0[8], w1[8];
            if (h0) load8(weight + 8 * c0, w0);
            if (h1) load8(weight + 8 * c1, w1);
            if (resid_static) {
                if (h0) load8(r + 8 * c0, v0);
                if (h1) load8(r + 8 * c1, v1);
            }
            delta = pdl_after(delta, pdl_wait());
            if (!resid_static) {
                if (h0) load8(r + 8 * c0, v0);
                if (h1) load8(r + 8 * c1, v1);
            }
            if (delta != nullptr) {
                float d[8];
                if (h0) {
                    load8(delta + base + 8 * c0, d);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v0[i] += d[i];
                    store8(r + 8 * c0, v0);
                }
                if (h1) {
                    load8(delta + base + 8 * c1, d);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v1[i] += d[i];
                    store8(r + 8 * c1, v1);
                }
            }
            if (h0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(v0[i], v0[i], ss);
            }
            if (h1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(v1[i], v1[i], ss);
            }
            const float total = block_sum(ss, scratch);
            const float inv = rsqrtf(total / (float)hidden + eps);
            if (h0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v0[i] = v0[i] * inv * (w0[i] + w_offset);
                store8(out + base + 8 * c0, v0);
            }
            if (h1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v1[i] = v1[i] * inv * (w1[i] + w_offset);
                store8(out + base + 8 * c1, v1);
            }
            return;
        }
        delta = pdl_after(delta, pdl_wait());
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            float v[8];
            load8(r + 8 * c, v);
            if (delta != nullptr) {
                float d[8];
                load8(delta + base + 8 * c, d);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += d[i];
                store8(r + 8 * c, v);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
        }
        const float total = block_sum(ss, scratch);
        const float inv = rsqrtf(total / (float)hidden + eps);
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            float v[8], w[8];
            load8(r + 8 * c, v);  // what this thread wrote itself
            load8(weight + 8 * c, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * (w[i] + w_offset);
            store8(out + base + 8 * c, v);
        }
        return;
    }
    delta = pdl_after(delta, pdl_wait());
    if (delta != nullptr) {
        const A* d = delta + base;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = r[i] + to_float(d[i]);
            r[i] = v;
            ss = fmaf(v, v, ss);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = r[i];
            ss = fmaf(v, v, ss);
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    A* o = out + base;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        // each thread re-reads only what it wrote itself, so no barrier is needed
        o[i] = from_float<A>(r[i] * inv * (to_float(weight[i]) + w_offset));
    }
}

MSTAR_API int mstar_add_rmsnorm(float* resid, const void* delta, const void* weight,
                                int weight_dtype, void* out, int act_dtype, int rows, int hidden,
                                float eps, float w_offset, int resid_static, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = hidden % 8 == 0 && ((uintptr_t)resid % 32 == 0) && ((uintptr_t)out % 16 == 0) &&
                     ((uintptr_t)weight % 32 == 0) && (delta == nullptr || (uintptr_t)delta % 16 == 0);
    int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (vec) threads = hidden >= 4096 ? 512 : (hidden >= 2048 ? 256 : 128);
    // a thread per 8-element chunk where 512 threads suffice: one load of each kind per thread
    // and a tree that starts at once (a decode step's norm 1.92 -> 1.68 us at width 3072)
    if (vec && hidden / 8 <= 512) threads = ((hidden / 8 + 31) / 32) * 32;
#define LAUNCH(A, W)                                                                             \
    if (vec)                                                                                     \
        mstar_launch((add_rmsnorm_kernel<A, W, true>), dim3(rows), dim3(threads), 0, s,                                  \
            resid, (const A*)delta, (const W*)weight, (A*)out, hidden, eps, w_offset,           \
            resid_static);                                                                       \
    else                                                                                         \
        mstar_launch((add_rmsnorm_kernel<A, W, false>), dim3(rows), dim3(threads), 0, s,                                 \
            resid, (const A*)delta, (const W*)weight, (A*)out, hidden, eps, w_offset, resid_static)
    if (act_dtype == MSTAR_F32) {
        if (weight_dtype == MSTAR_F32) { LAUNCH(float, float); } else { LAUNCH(float, bf16); }
    } else {
        if (weight_dtype == MSTAR_F32) { LAUNCH(bf16, float); } else { LAUNCH(bf16, bf16); }
    }
#undef LAUNCH
    return launch_status();
}

// ------------------------------------------------------ gather (+add) rows
// out[i] = resid[rows[i]] (+ delta[rows[i]]), float.  Used to pick the rows whose
// logits are wanted before the final norm, so norm and LM head run on those only.
template <typename A>
__global__ void gather_add_rows_kernel(const float* __restrict__ resid, const A* __restrict__ delta,
                                       const int* __restrict__ rows, float* __restrict__ out,
                                       int hidden) {
    const unsigned long long waited = pdl_wait();
    resid = pdl_after(resid, waited);
    delta = pdl_after(delta, waited);
    const size_t src = (size_t)rows[blockIdx.x] * hidden;
    const size_t dst = (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = resid[src + i];
        if (delta != nullptr) v += to_float(delta[src + i]);
        out[dst + i] = v;
    }
}

MSTAR_API int mstar_gather_add_rows(const float* resid, const void* delta, int act_dtype,
                                    const int* rows, float* out, int num_rows, int hidden,
                                    void* stream) {
    if (num_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == MSTAR_F32)
        mstar_launch((gather_add_rows_kernel<float>), dim3(num_rows), dim3(256), 0, s, resid, (const float*)delta, rows, out, hidden);
    else
        mstar_launch((gather_add_rows_kernel<bf16>), dim3(num_rows), dim3(256), 0, s, resid, (const bf16*)delta, rows, out, hidden);
    return launch_status();
}

// ------------------------------------------------------------ SiLU(gate)*up
// gate_up: [rows, 2*inter] with gate first (mstar/model/components/distributed/
// mlp.py:78-81); out: [rows, inter].  silu(x) = x / (1 + exp(-x)) in float.
template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gate_up, A* __restrict__ out, int inter,
                                size_t total) {
    gate_up = pdl_after(gate_up, pdl_wait());
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t row = idx / inter;
        const int col = (int)(idx - row * inter);
        const A* p = gate_up + row * 2 * (size_t)inter;
        const float g = to_float(p[col]);
        const float u = to_float(p[inter + col]);
        const float act = g / (1.f + expf(-g));
        out[idx] = from_float<A>(act * u);
    }
}

MSTAR_API int mstar_silu_mul(const void* gate_up, void* out, int act_dtype, int rows, int inter,
                             void* stream) {
    const size_t total = (size_t)rows * inter;
    if (total == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    const size_t most = (size_t)device_sm_count() * 32;   // a grid-stride loop takes the rest
    if (blocks > most) blocks = most;
    if (act_dtype == MSTAR_F32)
        mstar_launch((silu_mul_kernel<float>), dim3((int)blocks), dim3(threads), 0, s, (const float*)gate_up, (float*)out, inter, total);
    else
        mstar_launch((silu_mul_kernel<bf16>), dim3((int)blocks), dim3(threads), 0, s, (const bf16*)gate_up, (bf16*)out, inter, total);
    return launch_status();
}

// ------------------------------------------------- logit scale and soft cap
// x = x * scale, then x = cap * tanh(x / cap) when cap > 0; float, in place.
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t n, float scale, float cap) {
    x = pdl_after(x, pdl_wait());
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v * inv_cap);
        x[i] = v;
    }
}

MSTAR_API int mstar_scale_softcap(float* x, long long n, float scale, float cap, void* stream) {
    if (n <= 0) return 0;
    size_t blocks = ((size_t)n + 255) / 256;
    const size_t most = (size_t)device_sm_count() * 32;
    if (blocks > most) blocks = most;
    mstar_launch(scale_softcap_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, x,
                 (size_t)n, scale, cap);
    return launch_status();
}

// ------------------------------------------------------------- conversion
template <typename S, typename D>
__global__ void convert_kernel(const S* __restrict__ src, D* __restrict__ dst, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = from_float<D>(to_float(src[i]));
}

MSTAR_API int mstar_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
                            void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    size_t blocks = ((size_t)n + 255) / 256;
    const size_t most = (size_t)device_sm_count() * 32;   // a grid-stride loop takes the rest
    if (blocks > most) blocks = most;
    if (src_dtype == MSTAR_F32 && dst_dtype == MSTAR_BF16)
        convert_kernel<float, bf16><<<(int)blocks, 256, 0, s>>>((const float*)src, (bf16*)dst, (size_t)n);
    else if (src_dtype == MSTAR_BF16 && dst_dtype == MSTAR_F32)
        convert_kernel<bf16, float><<<(int)blocks, 256, 0, s>>>((const bf16*)src, (float*)dst, (size_t)n);
    else if (src_dtype == MSTAR_F32 && dst_dtype == MSTAR_F32)
        convert_kernel<float, float><<<(int)blocks, 256, 0, s>>>((const float*)src, (float*)dst, (size_t)n);
    else
        convert_kernel<bf16, bf16><<<(int)blocks, 256, 0, s>>>((const bf16*)src, (bf16*)dst, (size_t)n);
    return launch_status();
}

// ------------------------------------- rotary encoding + key/value page write
// qkv: [T, (nq + 2*nkv) * hd], rows [q heads | k heads | v heads].  Queries are
// rotated in place; keys are rotated and written, values copied, into the paged
// cache [pages, 2, nkv, page_size, hd] at (page, slot) of the token's cache
// position.  Angle = float(position) * inv_freq[j] in float, sincosf without
// fast-math (full range reduction).  rotary_dim == 0 writes keys unrotated.
// kv_cache == nullptr (a layer that reads another layer's cache): queries only.
struct RopeArgs {
    int nq, nkv, hd, rotary_dim, interleaved;
    int page_size, bt_stride;
};

template <typename A>
__global__ void rope_kv_write_kernel(A* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ cache_pos,
                                     const int* __restrict__ token_req,
                                     const int* __restrict__ block_table,
                                     const float* __restrict__ inv_freq, A* __restrict__ kv_cache,
                                     RopeArgs a) {
    pdl_launch_dependents();   // a short kernel: the long one after it may be scheduled now
    pdl_wait();
    // grid (token, slice): the items of a token (rotated pairs of q and k, unrotated tail
    // of k, values) are spread over all threads of its slices, one or a few each, so that
    // the dependent loads of different items overlap instead of queueing in one thread
    const int t = blockIdx.x;
    const int hd = a.hd, half = a.rotary_dim / 2;
    const int row_elems = (a.nq + 2 * a.nkv) * hd;
    A* row = qkv + (size_t)t * row_elems;
    const bool write = kv_cache != nullptr;
    const int rot_items = (write ? a.nq + a.nkv : a.nq) * half;
    const int tail = hd - a.rotary_dim;
    const int tail_items = write ? a.nkv * tail : 0;
    const int v_items = write ? a.nkv * hd : 0;
    const int total = rot_items + tail_items + v_items;
    const int first = blockIdx.y * blockDim.x + threadIdx.x;
    const int stride = gridDim.y * blockDim.x;
    if (first >= total) return;

    A* kdst = nullptr;
    A* vdst = nullptr;
    if (write) {
        const int cp = cache_pos[t];
        const int page = block_table[(size_t)token_req[t] * a.bt_stride + cp / a.page_size];
        const int slot = cp % a.page_size;
        const size_t page_elems = (size_t)2 * a.nkv * a.page_size * hd;
        kdst = kv_cache + (size_t)page * page_elems + (size_t)slot * hd;
        vdst = kdst + (size_t)a.nkv * a.page_size * hd;
    }
    const float pos = (float)positions[t];
    for (int item = first; item < total; item += stride) {
        if (item < rot_items) {
            const int h = item / half, j = item - h * half;
            const int i0 = a.interleaved ? 2 * j : j;
            const int i1 = a.interleaved ? 2 * j + 1 : j + half;
            float sn, cs;
            sincosf(pos * inv_freq[j], &sn, &cs);
            A* src = row + (size_t)h * hd;
            const float x0 = to_float(src[i0]), x1 = to_float(src[i1]);
            const float y0 = x0 * cs - x1 * sn;
            const float y1 = x1 * cs + x0 * sn;
            A* dst = h < a.nq ? src : kdst + (size_t)(h - a.nq) * a.page_size * hd;
            dst[i0] = from_float<A>(y0);
            dst[i1] = from_float<A>(y1);
        } else if (item < rot_items + tail_items) {
            // features of k beyond rotary_dim are copied unrotated
            const int it = item - rot_items;
            const int h = it / tail, d = a.rotary_dim + (it - h * tail);
            kdst[(size_t)h * a.page_size * hd + d] = row[(size_t)(a.nq + h) * hd + d];
        } else {
            const int it = item - rot_items - tail_items;
            const int h = it / hd, d = it - h * hd;
            vdst[(size_t)h * a.page_size * hd + d] = row[(size_t)(a.nq + a.nkv + h) * hd + d];
        }
    }
}

// Vector form of the kernel above for split-half pairs whose halves are multiples of 8
// features: a thread rotates 8 pairs (two 16-byte loads, two 16-byte stores) or copies
// 8 values; same arithmetic per element.
template <typename A>
__global__ void rope_kv_write_vec_kernel(A* __restrict__ qkv, const int* __restrict__ positions,
                                         const int* __restrict__ cache_pos,
                                         const int* __restrict__ token_req,
                                         const int* __restrict__ block_table,
                                         const float* __restrict__ inv_freq,
                                         A* __restrict__ kv_cache, RopeArgs a) {
    pdl_launch_dependents();   // a short kernel: the long one after it may be scheduled now
    pdl_wait();
    const int t = blockIdx.x;
    const int hd = a.hd, half = a.rotary_dim / 2;
    const int row_elems = (a.nq + 2 * a.nkv) * hd;
    A* row = qkv + (size_t)t * row_elems;
    const bool write = kv_cache != nullptr;
    const int hchunks = half >> 3;                         // 8-pair chunks per head
    const int rot_items = (write ? a.nq + a.nkv : a.nq) * hchunks;
    const int tail = hd - a.rotary_dim;                    // multiple of 8 on this path
    const int tail_items = write ? a.nkv * (tail >> 3) : 0;
    const int v_items = write ? a.nkv * (hd >> 3) : 0;
    const int total = rot_items + tail_items + v_items;
    const int first = blockIdx.y * blockDim.x + threadIdx.x;
    const int stride = gridDim.y * blockDim.x;
    // the token's sines and cosines once per block (every head uses the same); half <= 128
    __shared__ float tab_sn[128], tab_cs[128];
    {
        const float p = (float)positions[t];
        for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(p * inv_freq[j], &tab_sn[j], &tab_cs[j]);
    }
    __syncthreads();
    if (first >= total) return;

    A* kdst = nullptr;
    A* vdst = nullptr;
    if (write) {
        const int cp = cache_pos[t];
        const int page = block_table[(size_t)token_req[t] * a.bt_stride + cp / a.page_size];
        const int slot = cp % a.page_size;
        const size_t page_elems = (size_t)2 * a.nkv * a.page_size * hd;
        kdst = kv_cache + (size_t)page * page_elems + (size_t)slot * hd;
        vdst = kdst + (size_t)a.nkv * a.page_size * hd;
    }
    for (int item = first; item < total; item += stride) {
        if (item < rot_items) {
            const int h = item / hchunks, j0 = (item - h * hchunks) * 8;
            A* src = row + (size_t)h * hd;
            float x0[8], x1[8], y0[8], y1[8];
            load8(src + j0, x0);
            load8(src + j0 + half, x1);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float sn = tab_sn[j0 + i], cs = tab_cs[j0 + i];
                y0[i] = x0[i] * cs - x1[i] * sn;
                y1[i] = x1[i] * cs + x0[i] * sn;
            }
            A* dst = h < a.nq ? src : kdst + (size_t)(h - a.nq) * a.page_size * hd;
            store8(dst + j0, y0);
            store8(dst + j0 + half, y1);
        } else if (item < rot_items + tail_items) {
            const int it = item - rot_items;
            const int per = tail >> 3;
            const int h = it / per, d = a.rotary_dim + (it - h * per) * 8;
            *reinterpret_cast<uint4*>(kdst + (size_t)h * a.page_size * hd + d) =
                *reinterpret_cast<const uint4*>(row + (size_t)(a.nq + h) * hd + d);
        } else {
            const int it = item - rot_items - tail_items;
            const int per = hd >> 3;
            const int h = it / per, d = (it - h * per) * 8;
            float v[8];
            load8(row + (size_t)(a.nq + a.nkv + h) * hd + d, v);
            store8(vdst + (size_t)h * a.page_size * hd + d, v);
        }
    }
}

MSTAR_API int mstar_rope_kv_write(void* qkv, int act_dtype, const int* positions,
                                  const int* cache_pos, const int* token_req,
                                  const int* block_table, int bt_stride, const float* inv_freq,
                                  void* kv_cache, int num_tokens, int nq, int nkv, int hd,
                                  int rotary_dim, int interleaved, int page_size, void* stream) {
    if (num_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    RopeArgs a{nq, nkv, hd, rotary_dim, interleaved, page_size, bt_stride};
    const int threads = 256;
    // split-half pairs, halves and the unrotated tail in whole groups of 8, float angles
    // table aligned: the vector kernel; else one pair per item
    const bool vec = !interleaved && rotary_dim > 0 && rotary_dim <= 256 && (rotary_dim / 2) % 8 == 0 && hd % 8 == 0 &&
                     (hd - rotary_dim) % 8 == 0 && ((uintptr_t)qkv % 32 == 0) &&
                     ((uintptr_t)inv_freq % 32 == 0) && (kv_cache == nullptr || (uintptr_t)kv_cache % 32 == 0) &&
                     act_dtype == MSTAR_BF16;
    if (vec) {
        const int items = (nq + nkv) * (rotary_dim / 16) + nkv * ((hd - rotary_dim) / 8) + nkv * (hd / 8);
        int slices = (items + threads - 1) / threads;
        if (num_tokens >= 256 && slices > 1) slices = 1;
        if (slices < 1) slices = 1;
        dim3 grid(num_tokens, slices);
        mstar_launch((rope_kv_write_vec_kernel<bf16>), dim3(grid), dim3(threads), 0, s, 
            (bf16*)qkv, positions, cache_pos, token_req, block_table, inv_freq, (bf16*)kv_cache, a);
        return launch_status();
    }
    const int items = (nq + nkv) * (rotary_dim / 2) + nkv * (hd - rotary_dim) + nkv * hd;
    // few tokens: one item per thread; many tokens: fewer, longer-running slices
    int slices = (items + threads - 1) / threads;
    if (num_tokens >= 256 && slices > 2) slices = 2;
    if (slices < 1) slices = 1;
    dim3 grid(num_tokens, slices);
    if (act_dtype == MSTAR_F32)
        mstar_launch((rope_kv_write_kernel<float>), dim3(grid), dim3(threads), 0, s, 
            (float*)qkv, positions, cache_pos, token_req, block_table, inv_freq, (float*)kv_cache, a);
    else
        mstar_launch((rope_kv_write_kernel<bf16>), dim3(grid), dim3(threads), 0, s, 
            (bf16*)qkv, positions, cache_pos, token_req, block_table, inv_freq, (bf16*)kv_cache, a);
    return launch_status();
}
