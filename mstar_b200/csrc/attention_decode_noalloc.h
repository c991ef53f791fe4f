// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (t-avil/mstar); it exists for
// programs that want the split-K paged decode attention of this library but are not in
// a position to hand it a scratch buffer: code that runs where cudaMalloc is off limits
// (a real-time or safety-certified process that may not allocate after start-up, a
// plugin whose host owns all device memory and gives out none, a caller sitting inside
// another framework's memory pool it must not touch).  The ordinary entry point,
// mstar_paged_decode_attention_bf16, needs `tokens * nq * splits * (hd + 2)` floats of
// scratch from its caller whenever the keys are split; here that scratch is a fixed
// array inside the library.
//
// Limit: MSTAR_NOALLOC_SCRATCH_FLOATS floats (4 MiB).  The array is part of the library
// image, so every GPU on which this library is loaded keeps 4 MiB for it until the
// process exits, whether the function is ever called or not.  A call that would need
// more is refused with -2 and a message on stderr; nothing is launched.
//
// Behaviour to know about:
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) and keeps it.  Make that first call outside of any CUDA
//     stream capture.  The kept address is stored without a lock: two host threads that
//     make their first calls on a device at the same time both look the address up and
//     both store the same value, which is harmless.
//   * No call allocates or frees: no cudaMalloc, cudaFree or allocating library routine.
//   * All calls on a device share the one array.  It still holds the previous call's
//     partial results when the next one starts; that is harmless, because every partial
//     result that the merge step reads is written earlier in the same call, so nothing
//     has to be cleared.  But two calls that overlap on the GPU (different streams, or
//     different host threads) race on it: serialise them.
//   * Inputs, output and all index arrays are the caller's, exactly as for the ordinary
//     entry point, and so are the meaning of the arguments and the shapes it accepts.
//
// Returns 0 on success, -1 if the shape is refused (as the ordinary entry point), -2 if
// the scratch needed exceeds the limit, or a CUDA error code.
#pragma once

#define MSTAR_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int mstar_paged_decode_attention_bf16_noalloc(
    const void* q, int q_stride, void* out, const void* kv_cache, const int* block_table,
    int bt_stride, const int* token_req, const int* cache_pos, int tokens, int nq, int nkv, int hd,
    int page_size, int window, float scale, int chunk, int splits, void* stream);

#ifdef __cplusplus
}
#endif
