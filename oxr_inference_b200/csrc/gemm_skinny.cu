// Skinny bf16 GEMM for decode: C[M,N] = X[M,K] * W[N,K]^T with M <= 64, fp32 accumulation.
//
// At decode the projections (reference: nn.Linear / cuBLAS, oxr_runtime/language.py:223-244,261,268-269) read
// every weight once for a handful of rows, so the kernel is a weight stream. The product is computed
// transposed, C^T = W * X^T, so that 16 weight rows fill the M side of mma.m16n8k16 and the batch rows are
// its N side (8 per tile). Each lane loads 16 contiguous bytes of a weight row straight into the A fragment:
// within a chunk of 32 k-values lane (g, t) holds k = 8t..8t+7 of rows g and g+8 and feeds them to two MMAs
// as (8t, 8t+1 | 8t+2, 8t+3) and (8t+4, 8t+5 | 8t+6, 8t+7); the X fragment uses the same assignment, and a
// dot product does not care in which order k is visited. The 8 warps of a block share 16 weight rows and
// take the k-chunks round-robin; their partial tiles are summed through shared memory in warp order.
#include "common.cuh"

__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cached_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int SKINNY_WARPS = 8;

// TILES = number of 8-row groups of X (M <= 8 * TILES). TO = output type.
// GATED: W's rows alternate in groups of 8 between a gate and an up projection (rows 16j .. 16j+7 gate 8j .. 8j+7,
// rows 16j+8 .. 16j+15 the matching up rows), so a block's 16 rows are 8 gates and their 8 ups, and the epilogue
// writes silu(gate) * up (oxr_runtime/language.py:102-104) into C [M, N / 2]: the decode step's SiLU kernel and the
// round trip of the gate-up activations through memory are gone. SiLU is applied to the fp32 sums.
template <int TILES, typename TO, bool GATED = false>
__global__ void __launch_bounds__(SKINNY_WARPS * 32, TILES <= 2 ? 2 : 1)
gemm_skinny_kernel(TO* __restrict__ C, const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, int M,
                   int N, int K) {
    __shared__ float partial[SKINNY_WARPS][16][8 * TILES + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int row_a = n0 + g, row_b = n0 + g + 8;
    const bool ok_a = row_a < N, ok_b = row_b < N;
    const __nv_bfloat16* wa = W + (size_t)(ok_a ? row_a : 0) * K;
    const __nv_bfloat16* wb = W + (size_t)(ok_b ? row_b : 0) * K;

    float acc[TILES][4];
#pragma unroll
    for (int i = 0; i < TILES; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    constexpr int SKINNY_UNROLL = TILES <= 2 ? 8 : 4;   // 16-byte weight loads in flight per lane and row
    const int chunks = (K + 31) / 32;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 fa[SKINNY_UNROLL], fb[SKINNY_UNROLL];
    auto load_weights = [&](int c0) {
#pragma unroll
        for (int u = 0; u < SKINNY_UNROLL; ++u) {
            const int k = (c0 + u * SKINNY_WARPS) * 32 + 8 * t;
            const bool in = k < K;   // K is a multiple of 8, so a 16-byte word is inside or outside as a whole
            fa[u] = (in && ok_a) ? ld_stream_16(wa + k) : zero;
            fb[u] = (in && ok_b) ? ld_stream_16(wb + k) : zero;
        }
    };
    for (int c0 = warp; c0 < chunks; c0 += SKINNY_WARPS * SKINNY_UNROLL) {
        load_weights(c0);
#pragma unroll
        for (int u = 0; u < SKINNY_UNROLL; ++u) {
            const int k = (c0 + u * SKINNY_WARPS) * 32 + 8 * t;
            const bool in = k < K;
#pragma unroll
            for (int i = 0; i < TILES; ++i) {
                const int m = i * 8 + g;
                const uint4 x = (in && m < M) ? ld_cached_16(X + (size_t)m * K + k) : zero;
                mma_bf16_16816(acc[i], fa[u].x, fb[u].x, fa[u].y, fb[u].y, x.x, x.y);
                mma_bf16_16816(acc[i], fa[u].z, fb[u].z, fa[u].w, fb[u].w, x.z, x.w);
            }
        }
    }
    pdl_trigger();   // the weights are read: a chained kernel after this one may set itself up while the sums are gathered

    // C fragment: acc[i][0..1] = (weight row g, batch rows 8i + 2t, 2t+1); acc[i][2..3] = weight row g + 8.
#pragma unroll
    for (int i = 0; i < TILES; ++i) {
        partial[warp][g][8 * i + 2 * t] = acc[i][0];
        partial[warp][g][8 * i + 2 * t + 1] = acc[i][1];
        partial[warp][g + 8][8 * i + 2 * t] = acc[i][2];
        partial[warp][g + 8][8 * i + 2 * t + 1] = acc[i][3];
    }
    __syncthreads();
    if constexpr (GATED) {
        for (int idx = threadIdx.x; idx < 8 * 8 * TILES; idx += SKINNY_WARPS * 32) {
            const int r = idx % 8, m = idx / 8;
            if (m < M && n0 + r + 8 < N) {
                float gate = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < SKINNY_WARPS; ++w) { gate += partial[w][r][m]; up += partial[w][r + 8][m]; }
                C[(size_t)m * (N / 2) + n0 / 2 + r] = Num<TO>::from_f32(__fdividef(gate, 1.f + __expf(-gate)) * up);
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < 16 * 8 * TILES; idx += SKINNY_WARPS * 32) {
            const int r = idx % 16, m = idx / 16;   // consecutive threads -> consecutive n: coalesced stores
            if (m < M && n0 + r < N) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < SKINNY_WARPS; ++w) s += partial[w][r][m];
                C[(size_t)m * N + n0 + r] = Num<TO>::from_f32(s);
            }
        }
    }
}

// out_dtype: 0 = float32, 1 = bfloat16. Requires M <= 64, K % 8 == 0 and 16-byte aligned X and W.
OXR_API int oxr_gemm_skinny_bf16(void* C, const void* X, const void* W, int M, int N, int K, int out_dtype,
                                 cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0) return OXR_BAD_ARGUMENT;
    const unsigned blocks = (N + 15) / 16;
    const int tiles = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
#define LAUNCH(TL, TO) \
    gemm_skinny_kernel<TL, TO, false><<<blocks, SKINNY_WARPS * 32, 0, stream>>>((TO*)C, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, M, N, K)
#define BY_TILES(TO)                    \
    switch (tiles) {                    \
        case 1: LAUNCH(1, TO); break;   \
        case 2: LAUNCH(2, TO); break;   \
        case 4: LAUNCH(4, TO); break;   \
        default: LAUNCH(8, TO); break;  \
    }
    if (out_dtype == 0) { BY_TILES(float) }
    else if (out_dtype == 1) { BY_TILES(__nv_bfloat16) }
    else return OXR_BAD_ARGUMENT;
#undef BY_TILES
#undef LAUNCH
    return oxr_launch_status();
}

// C [M, N / 2] = silu(X Wg^T) * (X Wu^T) in bf16, for W [N, K] whose gate and up rows alternate in groups of 8
// (N a multiple of 16). Requires M <= 64, K % 8 == 0 and 16-byte aligned X and W.
OXR_API int oxr_gemm_skinny_gated_bf16(void* C, const void* X, const void* W, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || N % 16 != 0 || K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0) return OXR_BAD_ARGUMENT;
    const unsigned blocks = N / 16;
    using bf = __nv_bfloat16;
#define LAUNCH_GATED(TL) gemm_skinny_kernel<TL, bf, true><<<blocks, SKINNY_WARPS * 32, 0, stream>>>((bf*)C, (const bf*)X, (const bf*)W, M, N, K)
    if (M <= 8) LAUNCH_GATED(1);
    else if (M <= 16) LAUNCH_GATED(2);
    else if (M <= 32) LAUNCH_GATED(4);
    else LAUNCH_GATED(8);
#undef LAUNCH_GATED
    return oxr_launch_status();
}
