// Paged grouped-query attention for any mix of prompt portions and decoded tokens,
// in float arithmetic on CUDA cores.  It is the attention of the true 32-bit path
// and the fallback of the bfloat16 path for shapes the tensor-core kernels refuse.
//
// Semantics (mstar/engine/cache_manager.py:653-701 for the call, scale 1/sqrt(hd)
// as in mstar/utils/attention.py:116-117): query head i uses key/value head
// i / (nq/nkv); the token whose key sits at cache position p sees keys lo..p with
// lo = max(0, p - window + 1) (window 0: lo = 0), which is the causal mask aligned
// to the end of the sequence; softmax statistics and the output sum are float.
//
// One block per (token, kv head) handles the whole group of query heads, streaming
// the keys and values of that head through shared memory in tiles of 32 keys with
// an online softmax.  The keys of the current step are already in the cache.
#include "common.cuh"

#define ATT_TILE 32
#define ATT_THREADS 128
#define ATT_MAX_ACC 32

struct AttnArgs {
    int nq, nkv, hd, page_size, bt_stride, window;
    int q_stride;  // elements between consecutive tokens in q
    float scale;
};

template <typename A>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_generic_kernel(const A* __restrict__ q, A* __restrict__ out,
                               const A* __restrict__ kv_cache, const int* __restrict__ block_table,
                               const int* __restrict__ token_req, const int* __restrict__ cache_pos,
                               AttnArgs a) {
    extern __shared__ float smem[];
    const int t = blockIdx.x, kvh = blockIdx.y;
    const int hd = a.hd, G = a.nq / a.nkv;
    const int ldk = hd + 1;
    float* qs = smem;                        // [G][hd]
    float* tile = qs + G * hd;               // [ATT_TILE][hd+1]
    float* sc = tile + ATT_TILE * ldk;       // [G][ATT_TILE]
    float* m_s = sc + G * ATT_TILE;          // [G]
    float* l_s = m_s + G;                    // [G]
    float* alpha_s = l_s + G;                // [G]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hi = cache_pos[t] + 1;
    const int lo = (a.window > 0 && hi > a.window) ? hi - a.window : 0;
    const int* bt = block_table + (size_t)token_req[t] * a.bt_stride;
    const size_t page_elems = (size_t)2 * a.nkv * a.page_size * hd;
    const size_t head_off = (size_t)kvh * a.page_size * hd;
    const size_t v_off = (size_t)a.nkv * a.page_size * hd;

    const A* qrow = q + (size_t)t * a.q_stride + (size_t)kvh * G * hd;
    for (int i = tid; i < G * hd; i += ATT_THREADS) qs[i] = to_float(qrow[i]);
    for (int i = tid; i < G; i += ATT_THREADS) {
        m_s[i] = -INFINITY;
        l_s[i] = 0.f;
    }
    float acc[ATT_MAX_ACC];
#pragma unroll
    for (int k = 0; k < ATT_MAX_ACC; ++k) acc[k] = 0.f;
    const int n_out = G * hd;
    __syncthreads();

    for (int base = lo; base < hi; base += ATT_TILE) {
        // ---- keys of this tile -> shared (zero rows beyond hi)
        for (int idx = tid; idx < ATT_TILE * hd; idx += ATT_THREADS) {
            const int j = idx / hd, d = idx - j * hd;
            const int key = base + j;
            float v = 0.f;
            if (key < hi) {
                const int page = bt[key / a.page_size];
                const int slot = key % a.page_size;
                v = to_float(kv_cache[(size_t)page * page_elems + head_off + (size_t)slot * hd + d]);
            }
            tile[j * ldk + d] = v;
        }
        __syncthreads();
        // ---- scores
        for (int idx = tid; idx < G * ATT_TILE; idx += ATT_THREADS) {
            const int g = idx / ATT_TILE, j = idx - g * ATT_TILE;
            float s = -INFINITY;
            if (base + j < hi) {
                const float* qv = qs + g * hd;
                const float* kv = tile + j * ldk;
                float dot = 0.f;
                for (int d = 0; d < hd; ++d) dot = fmaf(qv[d], kv[d], dot);
                s = dot * a.scale;
            }
            sc[idx] = s;
        }
        __syncthreads();
        // ---- online softmax statistics, one warp per query head
        for (int g = warp; g < G; g += ATT_THREADS / 32) {
            const float s = sc[g * ATT_TILE + lane];
            const float m_old = m_s[g];
            const float m_new = fmaxf(m_old, warp_max(s));  // key `base` is always valid
            const float p = expf(s - m_new);                 // exp(-inf) = 0 for masked keys
            const float psum = warp_sum(p);
            sc[g * ATT_TILE + lane] = p;
            if (lane == 0) {
                const float al = expf(m_old - m_new);        // 0 on the first tile
                alpha_s[g] = al;
                l_s[g] = l_s[g] * al + psum;
                m_s[g] = m_new;
            }
        }
        __syncthreads();
        // ---- values of this tile -> shared (reusing the key buffer)
        for (int idx = tid; idx < ATT_TILE * hd; idx += ATT_THREADS) {
            const int j = idx / hd, d = idx - j * hd;
            const int key = base + j;
            float v = 0.f;
            if (key < hi) {
                const int page = bt[key / a.page_size];
                const int slot = key % a.page_size;
                v = to_float(kv_cache[(size_t)page * page_elems + v_off + head_off + (size_t)slot * hd + d]);
            }
            tile[j * ldk + d] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < ATT_MAX_ACC; ++k) {
            const int o = tid + k * ATT_THREADS;
            if (o < n_out) {
                const int g = o / hd, d = o - g * hd;
                const float* p = sc + g * ATT_TILE;
                float sum = acc[k] * alpha_s[g];
#pragma unroll 8
                for (int j = 0; j < ATT_TILE; ++j) sum = fmaf(p[j], tile[j * ldk + d], sum);
                acc[k] = sum;
            }
        }
        __syncthreads();
    }

    A* orow = out + (size_t)t * a.nq * hd + (size_t)kvh * G * hd;
#pragma unroll
    for (int k = 0; k < ATT_MAX_ACC; ++k) {
        const int o = tid + k * ATT_THREADS;
        if (o < n_out) {
            const int g = o / hd;
            orow[o] = from_float<A>(acc[k] / l_s[g]);
        }
    }
}

// Returns 0, a CUDA error code, or -1 when the shape is refused
// (group * head_dim > 4096 or head_dim > 256).
MSTAR_API int mstar_paged_attention_generic(const void* q, int q_stride, void* out,
                                            const void* kv_cache, const int* block_table,
                                            int bt_stride, const int* token_req,
                                            const int* cache_pos, int num_tokens, int nq, int nkv,
                                            int hd, int page_size, int window, float scale,
                                            int act_dtype, void* stream) {
    if (num_tokens <= 0) return 0;
    if (nkv <= 0 || nq % nkv != 0) return -1;
    const int G = nq / nkv;
    if (G * hd > ATT_MAX_ACC * ATT_THREADS || hd > 256) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    AttnArgs a{nq, nkv, hd, page_size, bt_stride, window, q_stride, scale};
    const size_t smem = sizeof(float) * ((size_t)G * hd + (size_t)ATT_TILE * (hd + 1) +
                                         (size_t)G * ATT_TILE + 3 * (size_t)G);
    dim3 grid(num_tokens, nkv);
    static size_t configured_f32 = 0, configured_bf16 = 0;  // largest size set so far
    if (act_dtype == MSTAR_F32) {
        if (smem > 48 * 1024 && smem > configured_f32) {
            cudaFuncSetAttribute(paged_attention_generic_kernel<float>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_f32 = smem;
        }
        paged_attention_generic_kernel<float><<<grid, ATT_THREADS, smem, s>>>(
            (const float*)q, (float*)out, (const float*)kv_cache, block_table, token_req, cache_pos, a);
    } else {
        if (smem > 48 * 1024 && smem > configured_bf16) {
            cudaFuncSetAttribute(paged_attention_generic_kernel<bf16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured_bf16 = smem;
        }
        paged_attention_generic_kernel<bf16><<<grid, ATT_THREADS, smem, s>>>(
            (const bf16*)q, (bf16*)out, (const bf16*)kv_cache, block_table, token_req, cache_pos, a);
    }
    return launch_status();
}
