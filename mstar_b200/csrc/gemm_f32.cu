// C[M,N] = A[M,K] * W[N,K]^T in true 32-bit: float inputs, float FMA accumulation on
// CUDA cores, no tensor-core mode of reduced precision.  This is the matrix product
// of the float32 path of the whole model (the reference has no such path: it lets
// float matmuls run as TF32, mstar/engine/__init__.py:6).  Every output element is
// one sequential sum over K, so a row's result does not depend on what else is in
// the batch.
#include "common.cuh"

#define SG_BM 64
#define SG_BN 64
#define SG_BK 16

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ __align__(16) float As[SG_BK][SG_BM + 4];
    __shared__ __align__(16) float Ws[SG_BK][SG_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;      // 0..1023
            const int r = idx >> 4, kk = idx & 15;
            const int gk = k0 + kk;
            float va = 0.f, vw = 0.f;
            if (gk < K) {
                if (m0 + r < M) va = A[(size_t)(m0 + r) * lda + gk];
                if (n0 + r < N) vw = W[(size_t)(n0 + r) * ldw + gk];
            }
            As[kk][r] = va;
            Ws[kk][r] = vw;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w};
            const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

MSTAR_API int mstar_sgemm_nt(const float* A, const float* W, float* C, int M, int N, int K,
                             int lda, int ldw, int ldc, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
    sgemm_nt_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, W, C, M, N, K, lda, ldw, ldc);
    return launch_status();
}
