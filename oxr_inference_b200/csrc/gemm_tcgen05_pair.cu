// bf16 GEMM on the 5th-generation tensor cores with two SMs per tile: C[M,N] = X[M,K] * W[N,K]^T for many rows.
//
// The reference multiplies through nn.Linear / cuBLAS (oxr_runtime/language.py:223-244,261,268-269). The one-SM
// kernel fills 16 KB of X and up to 32 KB of W into shared memory per 64-wide k step of a 128 x 256 tile; with a
// third less to fill per block the tensor pipe waits less (a k step measured 0.42 us per block instead of 0.45 us).
// Two blocks of a cluster share a 256 x bn tile (tcgen05 cta_group::2):
//   * block r of the pair stages rows 128 r .. + 127 of the X tile and rows bn/2 r .. of the W tile, by TMA, STAGES
//     deep: per k step half the W bytes of the one-SM kernel for the same 128 x bn of output per block;
//   * the pair's leader (rank 0) issues tcgen05.mma.cta_group::2 with M = 256, N = bn: the tensor cores of both SMs
//     read X from their own shared memory and the halves of W from both, and accumulate 128 x bn each in their own
//     tensor memory;
//   * the barriers that count TMA bytes live in the leader (both blocks' copies complete on them), tcgen05.commit
//     with a cluster mask frees a stage in both blocks and hands the accumulator to both blocks' epilogue warps,
//     which give it back by arriving on the leader's barrier;
//   * tiles are walked persistently by the pairs, two accumulators in tensor memory overlap epilogue and MMA.
// No TMA copy is multicast. Every wait on an mbarrier is bounded as in the one-SM kernel; both blocks meet at a
// cluster barrier before tensor memory is freed, so neither leaves while the other may still touch its memory.
#include "umma.cuh"

namespace {
constexpr int PAIR_THREADS = 192;   // warp 0: TMA, warp 1: MMA (leader) + TMEM owner, warps 2..5: epilogue

__host__ __device__ constexpr int pair_stage_bytes(int bn) { return A_BYTES + (bn / 2) * BK * 2; }

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of the same shared-memory location in block `rank` of the cluster.
__device__ __forceinline__ uint32_t in_block(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA tile load whose bytes are counted on a barrier that may live in the pair's other block (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void umma_pair_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this shared-memory offset in both blocks of the pair when the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_addr(bar)), "h"((uint16_t)3) : "memory");
}

// Tile order as in the one-SM kernel, with 256-row tiles: pairs that run at the same time share few W tiles.
__device__ __forceinline__ void pair_tile_origin(int tile, int M, int N, int bn, int& m0, int& n0) {
    constexpr int GROUP_M = 16;
    const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + bn - 1) / bn;
    const int per_group = GROUP_M * tiles_n;
    const int group = tile / per_group, within = tile % per_group;
    const int group_rows = min(GROUP_M, tiles_m - group * GROUP_M);
    m0 = (group * GROUP_M + within % group_rows) * 2 * BM;
    n0 = (within / group_rows) * bn;
}

template <typename TO, bool GATED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_tcgen05_pair_kernel(TO* __restrict__ C, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         int M, int N, int K, int bn, int stages, int tmem_cols, int num_tiles, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms are 1024 B
    const int stage_size = pair_stage_bytes(bn);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)stages * stage_size);   // used in the leader only
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* accum_full = empty + MAX_STAGES;   // [2] MMA -> epilogue, in each block
    uint64_t* accum_empty = accum_full + 2;      // [2] epilogue -> MMA, used in the leader only: 8 arrivals (4 warps x 2 blocks)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_empty + 2);
    uint32_t* gave_up = tmem_slot + 1;
    static_assert((2 * MAX_STAGES + 4) * 8 + 8 <= BARRIER_BYTES, "barriers outgrow their space");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = (K + BK - 1) / BK;
    const uint32_t acc_stride = (uint32_t)tmem_cols / 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(accum_full + i, 1); mbar_init(accum_empty + i, 8); }
        *gave_up = 0;
        mbar_fence_init();
    }
    if (warp == 1) {   // one warp of each block of the pair: the allocation is made in both blocks' tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"((uint32_t)tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();   // both blocks' barriers are initialised before either signals the other's
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (each block its halves)
        if (elect_one()) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            // No kernel writes the weights: this block's halves of W's tiles for the first ring of stages are requested
            // before the kernel (when it is launched dependent on the one before) waits for that one; the rows of X for
            // the same stages follow after the wait. The leader arms each of these stages for both blocks' bytes.
            int early = 0;
            for (int tile = pair; tile < num_tiles && early < stages; tile += num_pairs) {
                int m0, n0;
                pair_tile_origin(tile, M, N, bn, m0, n0);
                for (int kb = 0; kb < num_kb && early < stages; ++kb, ++early) {
                    if (rank == 0) mbar_expect_tx(full + early, 2u * (uint32_t)stage_size);
                    tma_load_2d_pair(tiles + (size_t)early * stage_size + A_BYTES, &map_w, kb * BK, n0 + (int)rank * (bn / 2),
                                     in_block(smem_addr(full + early), 0));
                }
            }
            pdl_wait();
            int step = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                int m0, n0;
                pair_tile_origin(tile, M, N, bn, m0, n0);
                for (int kb = 0; kb < num_kb; ++kb, ++step) {
                    unsigned char* a_dst = tiles + (size_t)s * stage_size;
                    const uint32_t leader_full = in_block(smem_addr(full + s), 0);
                    if (step < early) {   // first ring: the stage is free and armed, its half of W's tile is on its way
                        tma_load_2d_pair(a_dst, &map_x, kb * BK, m0 + (int)rank * BM, leader_full);
                    } else {
                        if (!mbar_wait(empty + s, phase ^ 1)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 10); ok = false; break; }
                        if (rank == 0) mbar_expect_tx(full + s, 2u * (uint32_t)stage_size);   // both blocks' bytes
                        tma_load_2d_pair(a_dst, &map_x, kb * BK, m0 + (int)rank * BM, leader_full);
                        tma_load_2d_pair(a_dst + A_BYTES, &map_w, kb * BK, n0 + (int)rank * (bn / 2), leader_full);
                    }
                    if (++s == stages) { s = 0; phase ^= 1; }
                }
            }
            pdl_trigger();   // every load of this block is issued: a chained kernel after this one may be scheduled
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (the leader's one thread)
        if (rank == 0 && elect_one()) {
            const uint32_t idesc = umma_idesc(2 * BM, bn);
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait(accum_empty + acc, acc_phase ^ 1)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 13); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)acc * acc_stride;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full + s, phase)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 11); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_addr(tiles + (size_t)s * stage_size);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_pair_bf16(tmem_d, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty + s);   // the stage is free in both blocks once these MMAs have read it
                    if (++s == stages) { s = 0; phase ^= 1; }
                }
                umma_commit_pair(accum_full + acc);   // both blocks' epilogues may read (also after giving up)
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: this block's 128 rows
        pdl_wait();   // C may still be read by the kernels before this one
        const int quarter = warp & 3;
        int it = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
            int m0, n0;
            pair_tile_origin(tile, M, N, bn, m0, n0);
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int row = m0 + (int)rank * BM + quarter * 32 + lane;
            bool ok = mbar_wait(accum_full + acc, acc_phase);
            if (!ok) { atomicExch(gave_up, 1u); if (lane == 0) oxr_report(status, OXR_WAIT_EXPIRED, 12); }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            ok = ok && (*reinterpret_cast<volatile uint32_t*>(gave_up) == 0);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * acc_stride;
#pragma unroll 1
            for (int c0 = 0; c0 < bn; c0 += 32) {
                uint32_t v[32];
                const int count = min(32, bn - c0);
                if (count == 32) tmem_ld_32x32(acc_addr + (uint32_t)c0, v);
                else tmem_ld_32x16(acc_addr + (uint32_t)c0, v);
                if (row < M && n0 + c0 < N) {
                    if constexpr (GATED) store_row_piece_gated<TO>(C + (size_t)row * (N / 2) + (n0 + c0) / 2, v, count, n0 + c0, N);
                    else store_row_piece<TO>(C + (size_t)row * N + n0 + c0, v, count, n0 + c0, N);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(in_block(smem_addr(accum_empty + acc), 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();   // neither block frees or leaves while the other may still read its shared or tensor memory
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
    }
}

template <typename TO, bool GATED = false>
int launch_pair(void* C, const void* X, const void* W, int M, int N, int K, int bn, int* status, cudaStream_t stream) {
    static int max_pairs = 0;   // per instantiation
    if (max_pairs == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<TO, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return 1000 + (int)e;
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) sms = 148;
        // how many pairs the device holds at once: ask, and fall back to one per two SMs
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sms / 2 * 2));
        cfg.blockDim = dim3(PAIR_THREADS);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_pair_kernel<TO, GATED>, &cfg) != cudaSuccess || clusters <= 0) {
            (void)cudaGetLastError();
            clusters = sms / 2;
        }
        max_pairs = clusters < sms / 2 ? clusters : sms / 2;
    }
    CUtensorMap map_x, map_w;
    if (!oxr_make_map_bf16(&map_x, X, M, K, BM) || !oxr_make_map_bf16(&map_w, W, N, K, bn / 2)) return OXR_BAD_ARGUMENT;
    const long long tiles = (long long)((N + bn - 1) / bn) * ((M + 2 * BM - 1) / (2 * BM));
    if (tiles > 0x7fffffffLL) return OXR_BAD_ARGUMENT;
    int stages = RING_BYTES / pair_stage_bytes(bn);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    int tmem_cols = 32;
    while (tmem_cols < 2 * bn) tmem_cols *= 2;
    const unsigned pairs = (unsigned)(tiles < max_pairs ? tiles : max_pairs);
    oxr_launch(gemm_tcgen05_pair_kernel<TO, GATED>, dim3(2 * pairs), dim3(PAIR_THREADS), SMEM_BYTES, stream, true, (TO*)C, map_x, map_w, M, N, K,
               bn, stages, tmem_cols, (int)tiles, status);
    return oxr_launch_status();
}
}  // namespace

// out_dtype: 0 = float32, 1 = bfloat16. Requires K % 8 == 0 and 16-byte aligned X, W. tile_n: columns of the output
// per pair of blocks, a multiple of 32 from 32 to 256 (each block stages half of them).
OXR_API int oxr_gemm_tcgen05_pair_bf16(void* C, const void* X, const void* W, int M, int N, int K, int out_dtype, int tile_n, int* status,
                                       cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0) return OXR_BAD_ARGUMENT;
    if (tile_n < 32 || tile_n > MAX_BN || tile_n % 32 != 0) return OXR_BAD_ARGUMENT;
    if (out_dtype == 1) return launch_pair<__nv_bfloat16>(C, X, W, M, N, K, tile_n, status, stream);
    if (out_dtype == 0) return launch_pair<float>(C, X, W, M, N, K, tile_n, status, stream);
    return OXR_BAD_ARGUMENT;
}

// C [M, N / 2] = silu(X Wg^T) * (X Wu^T) in bf16 for W [N, K] whose gate and up rows alternate in groups of 8 (N a
// multiple of 16): the pair kernel with the gated epilogue.
OXR_API int oxr_gemm_tcgen05_pair_gated_bf16(void* C, const void* X, const void* W, int M, int N, int K, int tile_n, int* status,
                                             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (N % 16 != 0 || K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0 || (uintptr_t)C % 16 != 0) return OXR_BAD_ARGUMENT;
    if (tile_n < 32 || tile_n > MAX_BN || tile_n % 32 != 0) return OXR_BAD_ARGUMENT;
    return launch_pair<__nv_bfloat16, true>(C, X, W, M, N, K, tile_n, status, stream);
}
