// Shared helpers for the sm_100a kernels: element types, conversions, reductions.
//
// Every kernel that touches activations is templated on the activation type
// (float for the true 32-bit path, __nv_bfloat16 for serving); arithmetic that
// decides accuracy (norm sums, softmax, rotary angles, residual sums) is float
// in both.  No file in this tree is compiled with fast-math.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define MSTAR_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side (mstar_b200/ops/lib.py)
enum MstarDType : int { MSTAR_F32 = 0, MSTAR_BF16 = 1 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// Eight consecutive elements as floats, by 16-byte accesses (the pointer must be aligned
// to 8 elements of T).
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a whole block; `scratch` holds at least 32 floats of shared memory.
// Every thread gets the result.  Safe to call repeatedly with the same scratch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch
// A kernel launched through mstar_launch may be scheduled while the kernel before it on the
// stream is still draining: its CTAs become resident, run up to pdl_wait() and stay there
// until that kernel has completed and its memory is visible.  This takes launch latency and
// the ramp of CTA scheduling out of the gaps between the many short kernels of a decode step
// (measured: 2.35 -> 2.22 ms per step at batch 8).  A successor is scheduled once every CTA
// of the running kernel has called pdl_launch_dependents() or has ended.  The long kernels
// call it where their last weights or keys have arrived, before their reductions; the rotary
// and the split-merge kernel, short ones before long ones, call it at their top (2.16 ->
// 2.12 ms); the norm kernel leaves it to its end (calling it at its top lets the product
// after it crowd in on the product before it: 2.37 ms).  Calling it at the top of every kernel lets waiting successors
// pile up on the SMs and was slower than no overlap at all (2.93 ms).  Every kernel calls
// pdl_wait() before it touches what the kernel before it wrote; what that kernel did not
// write (model weights, the step's index arrays, keys of earlier steps, the residual when the
// caller says so) may be read before.  MSTAR_PDL=0 launches everything with full
// serialization (the calls in the kernels are then no-ops).
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Returns zero, in a way the compiler cannot see through.  A pointer to data that the kernel
// before this one wrote is passed through pdl_after() with that zero before its first use: a
// load through a `const __restrict__` pointer (or __ldg) may be compiled as a load of memory
// that never changes, which the compiler is free to move above the wait; an address that
// depends on the wait's result cannot be formed before it.
__device__ __forceinline__ unsigned long long pdl_wait() {
    unsigned long long zero;
    asm volatile("griddepcontrol.wait;\n\tmov.u64 %0, 0;" : "=l"(zero)::"memory");
    return zero;
}
template <typename T> __device__ __forceinline__ T* pdl_after(T* p, unsigned long long zero_of_wait) {
    return reinterpret_cast<T*>(reinterpret_cast<unsigned long long>(p) + zero_of_wait);
}

// Number of SMs of the current device, asked once per device (grids are sized from it).
static inline int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] <= 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            sms <= 0)
            return 1;
        cached[dev] = sms;
    }
    return cached[dev];
}

static inline int pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MSTAR_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t mstar_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
