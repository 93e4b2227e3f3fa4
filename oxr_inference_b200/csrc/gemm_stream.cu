// Weight-streaming bf16 GEMM for decode: C[M,N] = X[M,K] * W[N,K]^T with M <= 16, fp32 accumulation.
//
// At decode a projection (reference: nn.Linear / cuBLAS, oxr_runtime/language.py:223-244,261,268-269) reads every weight
// once for a handful of rows: the product is a stream of W out of HBM.
//
//  * One block per SM, persistent; block b takes the 16-row groups b, b + gridDim.x, ... of W.
//  * A producer warp copies each group in slices of 2,048 k-values with cp.async.bulk, one 4 KB copy per weight row,
//    into a ring of two 65 KB shared-memory stages; an mbarrier per stage counts the bytes. Copies of 1 KB reached half
//    the bandwidth of 4 KB copies (3.2 against 6.6 TB/s over the GPU), 2 KB copies 5.8 TB/s.
//  * Eight consumer warps take a stage's k-values between them (256 each), read their fragments straight out of the
//    stage (rows are 4,160 bytes apart, so the 16-byte reads of a quarter-warp fall on different banks) and feed
//    mma.sync.m16n8k16 with the weight rows on the M side and the batch rows on the N side, as the register-fed skinny
//    kernel does; per group the warps' partial sums meet in shared memory in warp order (deterministic, and a row's
//    result does not depend on the rows beside it).
//  * X is read with ordinary cached loads. The ring leaves about 90 KB of the SM's 256 KB to L1, which holds the
//    64 KB of X of an 8 x 4,096 product, so after the first group X comes out of L1. (With a ring that fills the
//    SM and X from L2 for every group the kernel was slower than the skinny kernel, with three stages too.)
//  * The kernel is launched programmatically dependent on the kernel before it and lets its own dependents launch at
//    once: it is one round of blocks, so a dependent that arrives early takes no place from a block of this kernel that
//    has not started. The blocks are then resident, with barriers set up and the first copies issued, when the kernel
//    before completes; only the consumers wait (griddepcontrol.wait) before they touch X.
//
// Measured on a B200 (Qwen3-8B's products at 8 rows, isolated, in a CUDA graph): gate-up 30.3 us (6.6 TB/s; skinny
// kernel 32.7), o 6.1 (7.8), down 17.2 (17.8), qkv 8.7 (10.8); the batch-8 decode step 3.47 ms against 3.64 ms.
//
// What does not work, measured with %globaltimer stamps inside the kernel: fetching weights while the kernel before
// still runs. A grid launched programmatically dependent on another gets the bytes of its cp.async.bulk copies (and
// of cp.async copies) only after that grid has completed, however early they were issued: they land about half a
// microsecond after griddepcontrol.wait returns. Ordinary loads are served at once, and a variant in which the
// consumer warps fetched the first two stages that way above the wait did fill the ring early, but the step became
// slower (3.63 to 3.75 ms): the 20 MB that all SMs ask for at once queue up in front of the few loads of the small
// kernel that everybody is waiting for (RMSNorm took 8 instead of 5 us). Pacing the prefetch did not help.
//
// A product that follows another stream product directly (the fused forms below) starts later than one that follows a
// small kernel: a block needs a whole SM, so it becomes resident only when the block before it on that SM has left
// (0.35 us before its release instead of 4 to 5), and its first weights arrive that much later: qkv 10.1 instead of
// 8.4 us. The two norm kernels that the fused forms save are worth more (batch-8 step 3.46 against 3.50 ms).
//
// Every mbarrier wait is bounded; a wait that runs out records OXR_WAIT_EXPIRED, and the block goes on without
// waiting (its output is then meaningless, which the status word says) so that every thread still reaches the end.
#include "tma.cuh"

OXR_TL_DEFINE(oxr_tl_read_stream)
namespace {
constexpr int ST_WARPS = 8;                          // consumer warps
constexpr int ST_THREADS = (ST_WARPS + 1) * 32;      // + the producer warp
constexpr int ST_K = 2048;                           // k-values per stage
constexpr int ST_CH = ST_K / 32 / ST_WARPS;          // 32-wide k chunks per warp and stage
constexpr int ST_ROW_BYTES = ST_K * 2 + 64;          // 4,160: rows g and g + 1 of a quarter-warp's read hit different banks
constexpr int ST_STAGE_BYTES = 16 * ST_ROW_BYTES;    // 66,560
constexpr int ST_MAX_STAGES = 2;                     // more would take the L1 that X lives in
constexpr int ST_X_AHEAD = 1;                        // stages whose X words are in registers ahead of use

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ uint4 lds_16(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_addr(p)));
    return v;
}
__device__ __forceinline__ uint4 ldg_16(const void* p) {   // an ordinary cached load: X stays in what the ring leaves of L1
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(ST_WARPS * 32) : "memory"); }

// A bounded wait that, once any wait of the block has run out, stops waiting altogether.
__device__ __forceinline__ void wait_or_give_up(uint64_t* bar, uint32_t parity, volatile int* gave_up, int* status, int where) {
    if (*gave_up) return;
    if (!mbar_wait(bar, parity)) {
        *gave_up = 1;
        oxr_report(status, OXR_WAIT_EXPIRED, where);
    }
}

// The two fused forms that take the RMSNorm kernels out of a decode step (oxr_runtime/language.py:94-99,266-269).
// RMSNorm(r) W^T = inv * ((r * w_norm) W^T) with inv = rsqrt(mean(r^2) + eps) one number per batch row: the row's scale
// can be applied to the sums of the NEXT product instead of to its input, so nobody has to wait for a whole row's sum of
// squares before the next product starts. (Rounding r * w_norm to bf16 has the same relative error as rounding
// r * inv * w_norm; inv is applied to fp32 sums.)
//
//  ADD     (the last projection of a mixer or feed-forward): the epilogue rounds the product to bf16 (as the plain product
//          would be), adds it into the fp32 residual stream, writes the new residual r, y = bf16(r * w_norm) and, per
//          block, the sum of r^2 per batch row over the block's columns (16 floats per block): no block waits for another.
//  SCALED  (the first projection behind a norm): X is y; every block adds the blocks' sums of squares in block order
//          (while its first weights arrive) and its epilogue multiplies the sums of batch row m by inv[m].
struct FuseArgs {
    const float* res_in;       // ADD: residual stream [M, N] or null (none yet)
    float* res_out;            // ADD: new residual stream [M, N] (may be res_in)
    float* ss_out;             // ADD: [blocks of this launch][16]
    __nv_bfloat16* y_out;      // ADD: [M, N] bf16(residual * norm weight)
    const float* norm_weight;  // ADD: [N]
    const float* sc_ss;        // SCALED: [sc_blocks][16] sums of squares
    int sc_blocks;
    float eps;
};

// TILES: 8-row groups of X (M <= 8 * TILES). TO: output type. GATED: W's rows alternate in groups of 8 between a gate
// and an up projection and the epilogue writes silu(gate) * up into C [M, N / 2] (oxr_runtime/language.py:102-104).
template <int TILES, typename TO, bool GATED, bool ADD = false, bool SCALED = false>
__global__ void __launch_bounds__(ST_THREADS, 1)
gemm_stream_kernel(TO* __restrict__ C, const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, int M, int N, int K,
                   int stages, int* status, const FuseArgs fa) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;                                                     // stages x ST_STAGE_BYTES
    float* partial = reinterpret_cast<float*>(ring + (size_t)stages * ST_STAGE_BYTES);   // [ST_WARPS][16][8 * TILES + 1]
    uint64_t* full = reinterpret_cast<uint64_t*>(partial + ST_WARPS * 16 * (8 * TILES + 1) + 1);
    full = reinterpret_cast<uint64_t*>(((uintptr_t)full + 7) & ~(uintptr_t)7);
    uint64_t* empty = full + ST_MAX_STAGES;
    [[maybe_unused]] float* shares = reinterpret_cast<float*>(((uintptr_t)(empty + ST_MAX_STAGES) + 15) & ~(uintptr_t)15);   // SCALED: [sc_blocks][16]
    __shared__ int s_gave_up;
    __shared__ float s_inv[16];

    [[maybe_unused]] const unsigned long long tl_started = OXR_TL_NOW();
    pdl_trigger();   // dependents may be scheduled as soon as every block of this kernel is resident: they need a whole SM each
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, ST_WARPS); }
        s_gave_up = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const int groups = (N + 15) / 16, slices = (K + ST_K - 1) / ST_K;

    if (warp == ST_WARPS) {
        // ------------------------------------------------------------------------------ producer: never waits for X
        uint32_t n = 0;
        for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
            const int rows = min(16, N - grp * 16);
            for (int s = 0; s < slices; ++s, ++n) {
                const int st = n % stages;
                wait_or_give_up(empty + st, ((n / stages) & 1) ^ 1, &s_gave_up, status, 40);
                const uint32_t row_bytes = (uint32_t)min(ST_K, K - s * ST_K) * 2;
                if (lane == 0) mbar_expect_tx(full + st, row_bytes * rows);
                __syncwarp();
                if (lane < rows)
                    bulk_copy(ring + (size_t)st * ST_STAGE_BYTES + lane * ST_ROW_BYTES, W + (size_t)(grp * 16 + lane) * K + (size_t)s * ST_K,
                              row_bytes, full + st);
            }
        }
        return;
    }

    // ---------------------------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // this lane's X words of one stage: chunks 2 warp and 2 warp + 1 of the slice, rows 8 i + g
    auto load_x = [&](int s, uint4 (&x)[ST_CH][TILES]) {
#pragma unroll
        for (int c = 0; c < ST_CH; ++c) {
            const int k = s * ST_K + (ST_CH * warp + c) * 32 + 8 * t;
#pragma unroll
            for (int i = 0; i < TILES; ++i) {
                const int m = 8 * i + g;
                x[c][i] = (k < K && m < M) ? ldg_16(X + (size_t)m * K + k) : zero;
            }
        }
    };
    pdl_wait();   // X comes from the kernel before this one
    [[maybe_unused]] const unsigned long long tl_released = OXR_TL_NOW();
    [[maybe_unused]] float add_ss = 0.f;   // ADD: this thread's share of its batch row's sum of squares
    // The stages of this block in the order the producer fills them: q = (group index) * slices + slice. The X words of a
    // stage depend on its slice alone; those of stage q + X_AHEAD are asked for when stage q has been multiplied: a ring
    // of X_AHEAD register buffers, indexed by q % X_AHEAD (the loop is unrolled by it).
    constexpr int X_AHEAD = ST_X_AHEAD;
    const int my_groups = blockIdx.x < groups ? (groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int total = my_groups * slices;
    uint4 xr[X_AHEAD][ST_CH][TILES];
#pragma unroll
    for (int j = 0; j < X_AHEAD; ++j)
        if (j < total) load_x(j % slices, xr[j]);
    if constexpr (SCALED) {
        // The rows' scales, while the first weights are on their way. The blocks' shares of the sums of squares come through
        // shared memory (four 16-byte loads a thread in flight at a time: one round for up to 256 blocks); thread (j, m) adds
        // the shares of blocks j, j + 16, ... of batch row m, and thread m those sixteen sums: a fixed order.
        const int n4 = fa.sc_blocks * 4;
        for (int base = 0; base < n4; base += 4 * ST_WARPS * 32) {
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = base + j * ST_WARPS * 32 + (int)threadIdx.x;
                if (i < n4) v[j] = __ldcg(reinterpret_cast<const float4*>(fa.sc_ss) + i);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = base + j * ST_WARPS * 32 + (int)threadIdx.x;
                if (i < n4) reinterpret_cast<float4*>(shares)[i] = v[j];
            }
        }
        consumers_sync();
        {
            const int m = threadIdx.x & 15, j = threadIdx.x >> 4;
            float t = 0.f;
            for (int b = j; b < fa.sc_blocks; b += 16) t += shares[b * 16 + m];
            consumers_sync();            // everyone has read the shares: the sums take their place
            shares[j * 16 + m] = t;
        }
        consumers_sync();
        if (threadIdx.x < 16) {
            float t = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) t += shares[j * 16 + threadIdx.x];
            s_inv[threadIdx.x] = rsqrtf(t / (float)K + fa.eps);   // read after the barriers of the first group's epilogue
        }
    }
    // ADD: this thread's element (weight row r, batch row m) of the group's residual and norm weight, asked for when the
    // group starts
    [[maybe_unused]] float pre_res = 0.f, pre_nw = 0.f;
    [[maybe_unused]] auto prefetch_add = [&](int group) {
        const int r = threadIdx.x % 16, m = threadIdx.x / 16, n = group * 16 + r;
        if (group < groups && m < M && n < N) {
            pre_res = fa.res_in != nullptr ? __ldcg(fa.res_in + (size_t)m * N + n) : 0.f;
            pre_nw = __ldg(fa.norm_weight + n);
        }
    };
    if constexpr (ADD) prefetch_add(blockIdx.x);
    int grp = blockIdx.x, sl = 0;
    float acc[TILES][4];
#pragma unroll
    for (int i = 0; i < TILES; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int q0 = 0; q0 < total; q0 += X_AHEAD) {
#pragma unroll
        for (int j = 0; j < X_AHEAD; ++j) {
            const int q = q0 + j;
            if (q >= total) break;
            const int n0 = grp * 16;
            const bool ok_a = n0 + g < N, ok_b = n0 + g + 8 < N;
            const int st = q % stages;
            wait_or_give_up(full + st, (q / stages) & 1, &s_gave_up, status, 41);
            const unsigned char* stage = ring + (size_t)st * ST_STAGE_BYTES;
#pragma unroll
            for (int c = 0; c < ST_CH; ++c) {
                const int chunk = ST_CH * warp + c;
                const bool in = sl * ST_K + chunk * 32 + 8 * t < K;   // K is a multiple of 8: a 16-byte word is inside or outside as a whole
                const uint4 fa = (in && ok_a) ? lds_16(stage + g * ST_ROW_BYTES + chunk * 64 + 16 * t) : zero;
                const uint4 fb = (in && ok_b) ? lds_16(stage + (g + 8) * ST_ROW_BYTES + chunk * 64 + 16 * t) : zero;
#pragma unroll
                for (int i = 0; i < TILES; ++i) {
                    mma_16816(acc[i], fa.x, fb.x, fa.y, fb.y, xr[j][c][i].x, xr[j][c][i].y);
                    mma_16816(acc[i], fa.z, fb.z, fa.w, fb.w, xr[j][c][i].z, xr[j][c][i].w);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + st);
            if (q + X_AHEAD < total) load_x((sl + X_AHEAD) % slices, xr[j]);
            if (++sl < slices) continue;
            sl = 0;
            // ---- the group is complete: the warps' partial sums meet in shared memory
            // C fragment: acc[i][0..1] = (weight row g, batch rows 8 i + 2 t, 2 t + 1); acc[i][2..3] = weight row g + 8
            constexpr int PW = 8 * TILES + 1;
            consumers_sync();   // the epilogue of the group before has read `partial`
#pragma unroll
        for (int i = 0; i < TILES; ++i) {
            float* p = partial + (size_t)warp * 16 * PW;
            p[g * PW + 8 * i + 2 * t] = acc[i][0];
            p[g * PW + 8 * i + 2 * t + 1] = acc[i][1];
            p[(g + 8) * PW + 8 * i + 2 * t] = acc[i][2];
            p[(g + 8) * PW + 8 * i + 2 * t + 1] = acc[i][3];
        }
        consumers_sync();
        if constexpr (GATED) {
            for (int idx = threadIdx.x; idx < 8 * 8 * TILES; idx += ST_WARPS * 32) {
                const int r = idx % 8, m = idx / 8;
                if (m < M && n0 + r + 8 < N) {
                    float gate = 0.f, up = 0.f;
#pragma unroll
                    for (int w = 0; w < ST_WARPS; ++w) { gate += partial[(w * 16 + r) * PW + m]; up += partial[(w * 16 + r + 8) * PW + m]; }
                    if constexpr (SCALED) { gate *= s_inv[m]; up *= s_inv[m]; }
                    C[(size_t)m * (N / 2) + n0 / 2 + r] = Num<TO>::from_f32(__fdividef(gate, 1.f + __expf(-gate)) * up);
                }
            }
        } else if constexpr (ADD) {
            // one (weight row r, batch row m) per thread
            const int r = threadIdx.x % 16, m = threadIdx.x / 16;
            if (m < M && m < 8 * TILES && n0 + r < N) {
                const size_t at = (size_t)m * N + n0 + r;
                const float before = pre_res, nw = pre_nw;
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < ST_WARPS; ++w) sum += partial[(w * 16 + r) * PW + m];
                const float v = __bfloat162float(__float2bfloat16_rn(sum)) + before;
                fa.res_out[at] = v;
                fa.y_out[at] = __float2bfloat16_rn(v * nw);
                add_ss += v * v;
            }
        } else {
            for (int idx = threadIdx.x; idx < 16 * 8 * TILES; idx += ST_WARPS * 32) {
                const int r = idx % 16, m = idx / 16;   // consecutive threads -> consecutive n: coalesced stores
                if (m < M && n0 + r < N) {
                    float s = 0.f;
#pragma unroll
                    for (int w = 0; w < ST_WARPS; ++w) s += partial[(w * 16 + r) * PW + m];
                    if constexpr (SCALED) s *= s_inv[m];
                    C[(size_t)m * N + n0 + r] = Num<TO>::from_f32(s);
                }
            }
        }
            grp += gridDim.x;
            if constexpr (ADD) prefetch_add(grp);
#pragma unroll
            for (int i = 0; i < TILES; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        }
    }
    if constexpr (ADD) {
        // this block's share of each row's sum of squares: over the 16 weight rows of a half-warp, then over the groups
        // (already summed per thread), in a fixed order
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) add_ss += __shfl_xor_sync(0xffffffffu, add_ss, o);
        if (threadIdx.x % 16 == 0) fa.ss_out[(size_t)blockIdx.x * 16 + threadIdx.x / 16] = add_ss;
    }
#ifdef OXR_TIMELINE
    consumers_sync();
    if (threadIdx.x == 0) OXR_TL_PUT(1, tl_released, OXR_TL_NOW(), (unsigned long long)N, (unsigned long long)K, tl_started);
#endif
    // A block that gave up may still have copies in flight into its ring: give them time to land (a bounded sleep)
    // before the block's shared memory goes to someone else.
    if (s_gave_up) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        consumers_sync();
    }
}

template <int TILES, typename TO, bool GATED, bool ADD = false, bool SCALED = false>
int launch_stream(void* C, const void* X, const void* W, int M, int N, int K, int* status, cudaStream_t stream, FuseArgs fa = FuseArgs{}) {
    static int sms = 0, stages = 0;
    static size_t smem = 0;
    if (sms == 0) {
        int dev = 0, max_smem = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess || n <= 0)
            return OXR_BAD_ARGUMENT;
        // partial sums, two barriers a stage, and (SCALED) 16 floats for each block of the launch before: at most one block an SM
        const size_t fixed = (size_t)ST_WARPS * 16 * (8 * TILES + 1) * sizeof(float) + 16 + 2 * ST_MAX_STAGES * sizeof(uint64_t) + 128 +
                             (SCALED ? (size_t)(n < 16 ? 16 : n) * 16 * sizeof(float) : 0);
        int st = (int)(((size_t)max_smem - 1024 - fixed) / ST_STAGE_BYTES);   // 1 KB left for the kernel's static shared memory
        if (st > ST_MAX_STAGES) st = ST_MAX_STAGES;
        if (st < 2) return OXR_BAD_ARGUMENT;
        const size_t bytes = (size_t)st * ST_STAGE_BYTES + fixed;
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<TILES, TO, GATED, ADD, SCALED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return 1000 + (int)e;
        stages = st; smem = bytes; sms = n;
    }
    if (SCALED && fa.sc_blocks > sms) return OXR_BAD_ARGUMENT;
    const int groups = (N + 15) / 16;
    const int blocks = groups < sms ? groups : sms;
    oxr_launch(gemm_stream_kernel<TILES, TO, GATED, ADD, SCALED>, dim3(blocks), dim3(ST_THREADS), smem, stream, true,
               (TO*)C, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, M, N, K, stages, status, fa);
    return oxr_launch_status();
}
}  // namespace

// out_dtype: 0 = float32, 1 = bfloat16. Requires M <= 16, K % 8 == 0 and 16-byte aligned X and W.
OXR_API int oxr_gemm_stream_bf16(void* C, const void* X, const void* W, int M, int N, int K, int out_dtype, int* status,
                                 cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0) return OXR_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    if (out_dtype == 0) return M <= 8 ? launch_stream<1, float, false>(C, X, W, M, N, K, status, stream) : launch_stream<2, float, false>(C, X, W, M, N, K, status, stream);
    if (out_dtype == 1) return M <= 8 ? launch_stream<1, bf, false>(C, X, W, M, N, K, status, stream) : launch_stream<2, bf, false>(C, X, W, M, N, K, status, stream);
    return OXR_BAD_ARGUMENT;
}

// C [M, N / 2] = silu(X Wg^T) * (X Wu^T) in bf16, for W [N, K] whose gate and up rows alternate in groups of 8
// (N a multiple of 16). Requires M <= 16, K % 8 == 0 and 16-byte aligned X and W.
OXR_API int oxr_gemm_stream_gated_bf16(void* C, const void* X, const void* W, int M, int N, int K, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || N % 16 != 0 || K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0) return OXR_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    return M <= 8 ? launch_stream<1, bf, true>(C, X, W, M, N, K, status, stream) : launch_stream<2, bf, true>(C, X, W, M, N, K, status, stream);
}

// Blocks of a launch for N weight rows (ADD leaves 16 floats for each in `ss_out`).
OXR_API int oxr_gemm_stream_blocks(int N) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    const int groups = (N + 15) / 16;
    return groups < sms ? groups : sms;
}

// residual_out [M, N] fp32 = residual_in + bf16(X W^T) (residual_in may be null or equal residual_out), y_out [M, N] =
// bf16(residual_out * norm_weight), and ss_out [oxr_gemm_stream_blocks(N)][16]: per block and batch row the sum of squares
// of the block's columns of residual_out. Requires M <= 16, K % 8 == 0 and 16-byte aligned X and W.
OXR_API int oxr_gemm_stream_add_bf16(void* residual_out, const void* residual_in, void* y_out, float* ss_out, const float* norm_weight,
                                     const void* X, const void* W, int M, int N, int K, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0 || residual_out == nullptr || ss_out == nullptr ||
        y_out == nullptr || norm_weight == nullptr)
        return OXR_BAD_ARGUMENT;
    FuseArgs fa{};
    fa.res_in = (const float*)residual_in; fa.res_out = (float*)residual_out; fa.ss_out = ss_out;
    fa.y_out = (__nv_bfloat16*)y_out; fa.norm_weight = norm_weight;
    return M <= 8 ? launch_stream<1, __nv_bfloat16, false, true, false>(nullptr, X, W, M, N, K, status, stream, fa)
                  : launch_stream<2, __nv_bfloat16, false, true, false>(nullptr, X, W, M, N, K, status, stream, fa);
}

// C = (Y W^T) * rsqrt(sum / K + eps) row by row, in bf16 (gated != 0: silu(gate) * up of the scaled sums for a weight whose
// gate and up rows alternate in groups of 8, C [M, N / 2]): the product behind an RMSNorm whose input came from
// oxr_gemm_stream_add_bf16 as Y [M, K] = bf16(residual * norm weight) and `ss` [ss_blocks][16]. Requires M <= 16, K % 8 == 0,
// 16-byte aligned Y and W and ss_blocks <= the device's SMs.
OXR_API int oxr_gemm_stream_scaled_bf16(void* C, const void* Y, const float* ss, int ss_blocks, float eps, const void* W, int M, int N, int K,
                                        int gated, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || K % 8 != 0 || (uintptr_t)W % 16 != 0 || (uintptr_t)Y % 16 != 0 || ss == nullptr || ss_blocks <= 0 ||
        (gated && N % 16 != 0))
        return OXR_BAD_ARGUMENT;
    FuseArgs fa{};
    fa.sc_ss = ss; fa.sc_blocks = ss_blocks; fa.eps = eps;
    using bf = __nv_bfloat16;
    if (M <= 8)
        return gated ? launch_stream<1, bf, true, false, true>(C, Y, W, M, N, K, status, stream, fa)
                     : launch_stream<1, bf, false, false, true>(C, Y, W, M, N, K, status, stream, fa);
    return gated ? launch_stream<2, bf, true, false, true>(C, Y, W, M, N, K, status, stream, fa)
                 : launch_stream<2, bf, false, false, true>(C, Y, W, M, N, K, status, stream, fa);
}
