// True fp32 GEMM on the CUDA cores: C[M,N] = A[M,K] * W[N,K]^T, fp32 FMA accumulation, no TF32.
//
// This is the matrix product of the 32-bit path of the whole model (the reference multiplies through
// nn.Linear, oxr_runtime/language.py:223-244; in fp32 only on the CPU in its tests). Every output element is
// the sum over k = 0, 1, 2, ... of a[m,k] * w[n,k] accumulated in that order with fused multiply-adds,
// whatever the tile shape and whatever else is in the batch: a row's result does not depend on M.
#include "common.cuh"

template <int BM>
__global__ void __launch_bounds__(256) gemm_f32_nt_kernel(float* __restrict__ C, const float* __restrict__ A,
                                                           const float* __restrict__ W, int M, int N, int K) {
    constexpr int BN = 64, BK = 16, TM = BM / 16, TN = 4;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = tid; i < BM * BK; i += 256) {
            const int r = i / BK, k = i % BK;
            const int gm = m0 + r, gk = k0 + k;
            As[k][r] = (gm < M && gk < K) ? A[(size_t)gm * K + gk] : 0.f;
        }
        for (int i = tid; i < BN * BK; i += 256) {
            const int r = i / BK, k = i % BK;
            const int gn = n0 + r, gk = k0 + k;
            Ws[k][r] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}

OXR_API int oxr_gemm_f32_nt(float* C, const float* A, const float* W, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return OXR_BAD_ARGUMENT;
    if (M <= 16) {
        dim3 grid((N + 63) / 64, (M + 15) / 16);
        gemm_f32_nt_kernel<16><<<grid, 256, 0, stream>>>(C, A, W, M, N, K);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        if (grid.y > 65535) return OXR_BAD_ARGUMENT;
        gemm_f32_nt_kernel<64><<<grid, 256, 0, stream>>>(C, A, W, M, N, K);
    }
    return oxr_launch_status();
}
