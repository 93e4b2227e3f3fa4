// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = X[M,K] * W[N,K]^T, fp32 accumulation in tensor memory.
//
// The reference multiplies through nn.Linear / cuBLAS (oxr_runtime/language.py:223-244,261,268-269). This is the
// engine's own kernel for the prefill-sized products (M > 64):
//   * operands are staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), STAGES deep, each stage
//     guarded by a pair of mbarriers (full: TMA -> MMA, empty: MMA -> TMA);
//   * one thread issues tcgen05.mma (M = 128 rows of X, N = BN rows of W, K = 16 per instruction) with shared-memory
//     matrix descriptors; the 128 x BN fp32 accumulator lives in tensor memory (TMEM), one column per output column;
//   * tcgen05.commit releases a stage when the MMAs that read it are done, and signals the epilogue at the end;
//   * four epilogue warps read the accumulator with tcgen05.ld (warp w owns TMEM lanes 32 (w % 4) .. +31, i.e. 32
//     rows of the tile), round to the output type and store.
// Blocks are persistent: one per SM, each walking over 128 x BN tiles, with two accumulators in TMEM so that the
// epilogue of one tile overlaps the MMAs of the next. Rows and columns beyond M, N and K are zero-filled by TMA on
// the way in and masked on the way out. Every wait on an mbarrier is bounded: if one runs out, the block records
// OXR_WAIT_EXPIRED in the status word, stops waiting, frees its tensor memory and returns.
#include "tma.cuh"

namespace {
constexpr int BM = 128;           // rows of X per tile = TMEM lanes
constexpr int BK = 64;            // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int TC_THREADS = 192;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..5: epilogue

template <int BN> struct Cfg {
    static constexpr int STAGES = BN >= 256 ? 4 : 6;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle: rows 128 B apart,
// groups of 8 rows 1024 B apart (stride byte offset), leading byte offset 1 (unused for swizzled K-major),
// descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: fp32 accumulator (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), both
// K-major (bits 15, 16 = 0), N / 8 at bits 17-22, M / 16 at bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// Tile order: blocks that run at the same time share few W tiles and GROUP_M consecutive X tiles, so that W is
// streamed from HBM once and the X tiles of a group stay in L2 (W can be far larger than L2, X of a group is not).
template <int BN>
__device__ __forceinline__ void tile_origin(int tile, int M, int N, int& m0, int& n0) {
    constexpr int GROUP_M = 32;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int per_group = GROUP_M * tiles_n;
    const int group = tile / per_group, within = tile % per_group;
    const int group_rows = min(GROUP_M, tiles_m - group * GROUP_M);
    m0 = (group * GROUP_M + within % group_rows) * BM;
    n0 = (within / group_rows) * BN;
}

// Persistent: block b computes tiles b, b + gridDim.x, ... The accumulator is double-buffered in tensor memory
// (2 x BN columns), so the epilogue warps drain tile i while the MMA warp already accumulates tile i + 1.
template <int BN, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_kernel(TO* __restrict__ C, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    int M, int N, int K, int num_tiles, int* status) {
    using C_ = Cfg<BN>;
    constexpr int STAGES = C_::STAGES;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms are 1024 B
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * C_::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum_full = empty + STAGES;    // [2] MMA -> epilogue
    uint64_t* accum_empty = accum_full + 2;   // [2] epilogue -> MMA (4 arrivals: one per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_empty + 2);
    uint32_t* gave_up = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(accum_full + i, 1); mbar_init(accum_empty + i, 4); }
        *gave_up = 0;
        mbar_fence_init();
    }
    if (warp == 1) {   // the whole warp allocates the tensor memory and gives up the permit to allocate more
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            uint32_t kb_all = 0;   // k-blocks issued so far, over all tiles: the stage ring does not restart per tile
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int m0, n0;
                tile_origin<BN>(tile, M, N, m0, n0);
                for (int kb = 0; kb < num_kb; ++kb, ++kb_all) {
                    const int s = kb_all % STAGES;
                    const uint32_t phase = (kb_all / STAGES) & 1;
                    if (!mbar_wait(empty + s, phase ^ 1)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 0); ok = false; break; }
                    unsigned char* a_dst = tiles + (size_t)s * C_::STAGE_BYTES;
                    mbar_expect_tx(full + s, C_::STAGE_BYTES);
                    tma_load_2d(a_dst, &map_x, kb * BK, m0, full + s);
                    tma_load_2d(a_dst + C_::A_BYTES, &map_w, kb * BK, n0, full + s);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc = umma_idesc(BM, BN);
            uint32_t kb_all = 0;
            bool ok = true;
            int it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait(accum_empty + acc, acc_phase ^ 1)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 3); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++kb_all) {
                    const int s = kb_all % STAGES;
                    const uint32_t phase = (kb_all / STAGES) & 1;
                    if (!mbar_wait(full + s, phase)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 1); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_addr(tiles + (size_t)s * C_::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + C_::A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // inside the 128-byte swizzle row, the next 16 k-values start 32 bytes further
                        umma_bf16(tmem_d, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc,
                                  (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty + s);   // the stage is free once these MMAs have read it
                }
                umma_commit(accum_full + acc);   // arrives when every MMA issued so far is complete (also after giving up)
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: TMEM -> registers -> global
        const int quarter = warp & 3;                     // this warp may touch TMEM lanes 32 * quarter .. + 31
        int it = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            int m0, n0;
            tile_origin<BN>(tile, M, N, m0, n0);
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int row = m0 + quarter * 32 + lane;
            bool ok = mbar_wait(accum_full + acc, acc_phase);
            if (!ok) { atomicExch(gave_up, 1u); if (lane == 0) oxr_report(status, OXR_WAIT_EXPIRED, 2); }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            ok = ok && (*reinterpret_cast<volatile uint32_t*>(gave_up) == 0);
            ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld is warp-wide: all lanes take the same path
            if (!ok) break;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + c * 32), v);
                const int col0 = n0 + c * 32;
                if (row < M && col0 < N) {
                    TO* dst = C + (size_t)row * N + col0;
                    const bool whole = col0 + 32 <= N && ((uintptr_t)dst % 16 == 0);
                    if (whole) {
                        if constexpr (sizeof(TO) == 2) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint4 o;
                                __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    op[e] = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
                                reinterpret_cast<uint4*>(dst)[j] = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        }
                    } else {
                        for (int j = 0; j < 32 && col0 + j < N; ++j) dst[j] = Num<TO>::from_f32(__uint_as_float(v[j]));
                    }
                }
            }
            // this warp has read its quarter of the accumulator: hand the buffer back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(accum_empty + acc);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------- host side
template <int BN, typename TO>
int launch(void* C, const void* X, const void* W, int M, int N, int K, int* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN>::SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    CUtensorMap map_x, map_w;
    if (!oxr_make_map_bf16(&map_x, X, M, K, BM) || !oxr_make_map_bf16(&map_w, W, N, K, BN)) return OXR_BAD_ARGUMENT;
    const long long tiles = (long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    if (tiles > 0x7fffffffLL) return OXR_BAD_ARGUMENT;
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
            num_sms = 148;
    }
    dim3 grid((unsigned)(tiles < num_sms ? tiles : num_sms));   // one block per SM (its shared memory fills the SM)
    gemm_tcgen05_kernel<BN, TO><<<grid, TC_THREADS, Cfg<BN>::SMEM, stream>>>((TO*)C, map_x, map_w, M, N, K, (int)tiles, status);
    return oxr_launch_status();
}
}  // namespace

// out_dtype: 0 = float32, 1 = bfloat16. Requires K % 8 == 0 (rows are whole 16-byte words) and 16-byte aligned X, W.
// tile_n: 128 or 256 columns of the output per block.
OXR_API int oxr_gemm_tcgen05_bf16(void* C, const void* X, const void* W, int M, int N, int K, int out_dtype, int tile_n, int* status,
                                  cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0) return OXR_BAD_ARGUMENT;
    if (tile_n == 256) {
        if (out_dtype == 1) return launch<256, __nv_bfloat16>(C, X, W, M, N, K, status, stream);
        if (out_dtype == 0) return launch<256, float>(C, X, W, M, N, K, status, stream);
    } else if (tile_n == 128) {
        if (out_dtype == 1) return launch<128, __nv_bfloat16>(C, X, W, M, N, K, status, stream);
        if (out_dtype == 0) return launch<128, float>(C, X, W, M, N, K, status, stream);
    }
    return OXR_BAD_ARGUMENT;
}
