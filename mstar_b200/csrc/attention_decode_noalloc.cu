// The allocation-free variant of split-K paged decode attention: the same kernels as
// attention_decode.cu, with the partial results of the splits kept in a fixed array of
// this library instead of caller-provided scratch.  See attention_decode_noalloc.h for
// who needs this and what the limits are.
#include <cstdio>

#include "attention_decode.cu"
#include "attention_decode_noalloc.h"

// Scratch for the splits' partial (max, sum, O).  Lives in the library image: each GPU
// that loads the library holds it until the process ends.
static __device__ __align__(256) float g_noalloc_scratch[MSTAR_NOALLOC_SCRATCH_FLOATS];

#define NOALLOC_MAX_DEVICES 64
// Device address of g_noalloc_scratch per device.  In host code the array's name is
// only a handle for cudaGetSymbolAddress, never a pointer a kernel may be given.
static float* g_scratch_addr[NOALLOC_MAX_DEVICES];

static int scratch_for_current_device(float** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (g_scratch_addr[dev] == nullptr) {
        // once per device, with that device current (it is: we just asked which one)
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

extern "C" __attribute__((visibility("default"))) int mstar_paged_decode_attention_bf16_noalloc(
    const void* q, int q_stride, void* out, const void* kv_cache, const int* block_table,
    int bt_stride, const int* token_req, const int* cache_pos, int tokens, int nq, int nkv, int hd,
    int page_size, int window, float scale, int chunk, int splits, void* stream) {
    if (tokens <= 0) return 0;
    const long long need = mstar_decode_attention_scratch_floats(tokens, nq, hd, splits);
    if (need > (long long)MSTAR_NOALLOC_SCRATCH_FLOATS) {
        fprintf(stderr,
                "mstar_paged_decode_attention_bf16_noalloc: %d tokens x %d heads x %d splits x "
                "(%d + 2) = %lld floats of scratch exceed the built-in %d; use fewer splits or "
                "tokens per call, or the ordinary entry point with your own scratch\n",
                tokens, nq, splits, hd, need, MSTAR_NOALLOC_SCRATCH_FLOATS);
        return -2;
    }
    float* scratch = nullptr;
    if (splits > 1) {
        const int rc = scratch_for_current_device(&scratch);
        if (rc != 0) return rc;
    }
    // Nothing in the scratch has to start at zero: every (token, head, split) slot that
    // the merge kernel reads is written by the attention kernel of this same call.
    return mstar_paged_decode_attention_bf16(q, q_stride, out, kv_cache, block_table, bt_stride,
                                             token_req, cache_pos, tokens, nq, nkv, hd, page_size,
                                             window, scale, chunk, splits, scratch, stream);
}
