// bf16 product of FEW rows (a decode batch of tens to a few hundred requests) on the 5th-generation tensor cores:
// C[M,N] = X[M,K] * W[N,K]^T with M <= 256, fp32 accumulation in tensor memory.
//
// The reference multiplies through nn.Linear / cuBLAS (oxr_runtime/language.py:223-244,261,268-269). With few rows the
// product is a stream of W, and a narrow W (N / 128 tiles) gives far fewer tiles than the GPU has SMs. This kernel
// computes the transpose, C^T = W X^T: 128 rows of W are the 128-row side of a tile, the M rows of X (rounded up to 16)
// its width, so no shared memory is spent on padding rows. The 64-wide k steps of a tile are dealt out to `shares`
// blocks that form ONE THREAD-BLOCK CLUSTER: share r takes steps r, r + shares, ... Each block accumulates its partial
// tile in tensor memory, copies it to its own shared memory (the operand ring is free by then), and after a cluster
// barrier every block adds the partial tiles of all blocks for its own part of the tile's columns, reading the other
// blocks' shared memory directly (distributed shared memory), in the order of the shares, rounds and stores. No partial
// tile goes through global memory, there is no ticket and no block that works alone at the end; the sum does not
// depend on timing.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer and owner of the tensor memory, 2..5 = accumulator -> shared memory; all
// six warps add and store. Every wait on an mbarrier is bounded (OXR_WAIT_EXPIRED in the status word); every block
// reaches both cluster barriers whatever happened before, so no block of a cluster waits for one that has left.
#include "umma.cuh"

namespace {
constexpr int FR_THREADS = 192;
constexpr int FR_COLS_IN_FLIGHT = 4;   // columns of the tile a warp adds at a time (their loads are issued together)

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t peer_smem(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__host__ __device__ constexpr int fr_stage_bytes(int bn) { return A_BYTES + bn * BK * 2; }

// map_w: W [N, K] in boxes of 128 rows; map_x: X [M, K] in boxes of bn rows. C is [M, N].
template <typename TO>
__global__ void __launch_bounds__(FR_THREADS, 1)
gemm_few_rows_kernel(TO* __restrict__ C, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, int M, int N,
                     int K, int bn, int stages, int tmem_cols, int shares, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int stage_size = fr_stage_bytes(bn);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + RING_BYTES - (RING_BYTES % 1024));   // behind the ring and the partial tile
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* accum_full = empty + MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_full + 1);
    uint32_t* gave_up = tmem_slot + 1;
    static_assert((2 * MAX_STAGES + 1) * 8 + 8 <= BARRIER_BYTES, "barriers outgrow their space");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();
    const int n0 = (int)cluster_id_x() * BM;        // first row of W (column of C) of this cluster's tile
    const int num_kb = (K + BK - 1) / BK;
    const int my_steps = rank < num_kb ? (num_kb - rank + shares - 1) / shares : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(accum_full, 1);
        *gave_up = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"((uint32_t)tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            // No kernel writes the weights: their tiles of the first ring of stages are requested before this kernel
            // (when it is launched dependent on the one before) waits for that one; the rows of X follow the wait.
            const int early = min(my_steps, stages);
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(full + i, (uint32_t)stage_size);
                tma_load_2d(tiles + (size_t)i * stage_size, &map_w, (rank + i * shares) * BK, n0, full + i);
            }
            pdl_wait();
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < my_steps; ++i) {
                const int kb = rank + i * shares;
                unsigned char* dst = tiles + (size_t)s * stage_size;
                if (i >= early) {
                    if (!mbar_wait(empty + s, phase ^ 1)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 0); break; }
                    mbar_expect_tx(full + s, (uint32_t)stage_size);
                    tma_load_2d(dst, &map_w, kb * BK, n0, full + s);
                }
                tma_load_2d(dst + A_BYTES, &map_x, kb * BK, 0, full + s);
                if (++s == stages) { s = 0; phase ^= 1; }
            }
            pdl_trigger();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            const uint32_t idesc = umma_idesc(BM, bn);
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < my_steps; ++i) {
                if (!mbar_wait(full + s, phase)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 1); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_addr(tiles + (size_t)s * stage_size);
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_bf16(tmem_base, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty + s);
                if (++s == stages) { s = 0; phase ^= 1; }
            }
            umma_commit(accum_full);   // arrives when every MMA issued so far is complete (also after giving up)
        }
    } else {
        // ------------------------------------------------------------------ accumulator -> this block's shared memory
        // part[c][r], c < M a row of X, r < 128 a row of W: the ring is free once the last MMA is complete
        const int quarter = warp & 3;
        bool ok = mbar_wait(accum_full, 0);
        if (!ok) { atomicExch(gave_up, 1u); if (lane == 0) oxr_report(status, OXR_WAIT_EXPIRED, 2); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        ok = ok && (*reinterpret_cast<volatile uint32_t*>(gave_up) == 0);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            float* part = reinterpret_cast<float*>(tiles) + quarter * 32 + lane;
            const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < M; c0 += 32) {
                uint32_t v[32];
                const int count = min(32, bn - c0);
                if (my_steps == 0) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;   // more shares than k steps: this block adds nothing
                } else if (count == 32) {
                    tmem_ld_32x32(acc_addr + (uint32_t)c0, v);
                } else {
                    tmem_ld_32x16(acc_addr + (uint32_t)c0, v);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (j < count && c0 + j < M) part[(size_t)(c0 + j) * BM] = __uint_as_float(v[j]);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }

    // ---------------------------------------------------------------------- every block adds its part of the columns
    __syncwarp();
    pdl_wait();          // C may still be read by the kernels before this one
    cluster_barrier();   // the partial tiles of all shares are in place
    if (*reinterpret_cast<volatile uint32_t*>(gave_up) == 0) {
        const uint32_t part0 = smem_addr(tiles);
        const int r4 = lane * 4;
        const int rows = min(BM, N - n0);   // rows of W in this tile = columns of C
        // warp w of block `rank` takes columns rank + shares * (w + 6 j): FR_COLS_IN_FLIGHT of them per pass
        for (int j0 = warp; rank + shares * j0 < M; j0 += (FR_THREADS / 32) * FR_COLS_IN_FLIGHT) {
            float4 sum[FR_COLS_IN_FLIGHT];
#pragma unroll
            for (int i = 0; i < FR_COLS_IN_FLIGHT; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < shares; ++s) {
                const uint32_t base = peer_smem(part0, (uint32_t)s);
                float4 p[FR_COLS_IN_FLIGHT];
#pragma unroll
                for (int i = 0; i < FR_COLS_IN_FLIGHT; ++i) {
                    const int c = min(rank + shares * (j0 + i * (FR_THREADS / 32)), M - 1);
                    p[i] = ld_cluster_f4(base + (uint32_t)((c * BM + r4) * 4));
                }
#pragma unroll
                for (int i = 0; i < FR_COLS_IN_FLIGHT; ++i) { sum[i].x += p[i].x; sum[i].y += p[i].y; sum[i].z += p[i].z; sum[i].w += p[i].w; }
            }
#pragma unroll
            for (int i = 0; i < FR_COLS_IN_FLIGHT; ++i) {
                const int c = rank + shares * (j0 + i * (FR_THREADS / 32));
                if (c >= M || r4 >= rows) continue;
                TO* dst = C + (size_t)c * N + n0 + r4;
                if (r4 + 4 <= rows && (uintptr_t)dst % (4 * sizeof(TO)) == 0) {
                    if constexpr (sizeof(TO) == 2) {
                        uint2 o;
                        reinterpret_cast<__nv_bfloat162*>(&o)[0] = __floats2bfloat162_rn(sum[i].x, sum[i].y);
                        reinterpret_cast<__nv_bfloat162*>(&o)[1] = __floats2bfloat162_rn(sum[i].z, sum[i].w);
                        *reinterpret_cast<uint2*>(dst) = o;
                    } else {
                        *reinterpret_cast<float4*>(dst) = sum[i];
                    }
                } else {
                    const float e[4] = {sum[i].x, sum[i].y, sum[i].z, sum[i].w};
                    for (int j = 0; j < 4 && r4 + j < rows; ++j) dst[j] = Num<TO>::from_f32(e[j]);
                }
            }
        }
    }
    cluster_barrier();   // no block leaves while another may still read its shared memory
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
    }
}

template <typename TO>
int configure() {
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(gemm_few_rows_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return 1000 + (int)e;
        done = true;
    }
    return 0;
}

template <typename TO>
int launch_few_rows(void* C, const void* X, const void* W, int M, int N, int K, int shares, int* status, cudaStream_t stream) {
    if (int rc = configure<TO>()) return rc;
    const int bn = (M + 15) / 16 * 16;
    CUtensorMap map_w, map_x;
    if (!oxr_make_map_bf16(&map_w, W, N, K, BM) || !oxr_make_map_bf16(&map_x, X, M, K, bn)) return OXR_BAD_ARGUMENT;
    const int tiles = (N + BM - 1) / BM;
    int stages = (RING_BYTES - (RING_BYTES % 1024)) / fr_stage_bytes(bn);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    int tmem_cols = 32;
    while (tmem_cols < bn) tmem_cols *= 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * shares));
    cfg.blockDim = dim3(FR_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = (unsigned)shares;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = oxr_chain_kernels ? 2 : 1;
    cudaLaunchKernelEx(&cfg, gemm_few_rows_kernel<TO>, (TO*)C, map_w, map_x, M, N, K, bn, stages, tmem_cols, shares, status);
    return oxr_launch_status();
}
}  // namespace

// How many clusters of `shares` blocks of the few-rows kernel the GPU holds at a time (0 if such a cluster cannot be
// launched). The caller picks the shares so that all tiles of a product run at once.
OXR_API int oxr_gemm_few_rows_max_clusters(int shares) {
    if (shares < 1 || shares > 8) return 0;
    if (configure<__nv_bfloat16>() != 0) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(shares * 64));
    cfg.blockDim = dim3(FR_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)shares;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_few_rows_kernel<__nv_bfloat16>, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

// C [M, N] = X [M, K] W [N, K]^T for M <= 256; out_dtype: 0 = float32, 1 = bfloat16. `shares` (1 to 8) blocks of a
// cluster share the k steps of each 128-column tile of C. Requires K % 8 == 0 and 16-byte aligned X and W.
OXR_API int oxr_gemm_few_rows_cluster_bf16(void* C, const void* X, const void* W, int M, int N, int K, int out_dtype, int shares, int* status,
                                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > MAX_BN || K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0 || shares < 1 || shares > 8) return OXR_BAD_ARGUMENT;
    if (out_dtype == 1) return launch_few_rows<__nv_bfloat16>(C, X, W, M, N, K, shares, status, stream);
    if (out_dtype == 0) return launch_few_rows<float>(C, X, W, M, N, K, shares, status, stream);
    return OXR_BAD_ARGUMENT;
}
