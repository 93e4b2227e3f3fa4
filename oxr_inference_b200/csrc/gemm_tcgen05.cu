// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = X[M,K] * W[N,K]^T, fp32 accumulation in tensor memory.
//
// The reference multiplies through nn.Linear / cuBLAS (oxr_runtime/language.py:223-244,261,268-269). This is the
// engine's own kernel for every product of more rows than the skinny kernel takes:
//   * operands are staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), STAGES deep, each stage
//     guarded by a pair of mbarriers (full: TMA -> MMA, empty: MMA -> TMA);
//   * one thread issues tcgen05.mma (M = 128 rows of X, N = bn rows of W, K = 16 per instruction) with shared-memory
//     matrix descriptors; the 128 x bn fp32 accumulator lives in tensor memory (TMEM), one column per output column;
//     bn is any multiple of 16 up to 256, chosen per product by the caller so that the tiles fill the SMs evenly;
//   * tcgen05.commit releases a stage when the MMAs that read it are done, and signals the epilogue at the end;
//   * four epilogue warps read the accumulator with tcgen05.ld (warp w owns TMEM lanes 32 (w % 4) .. +31, i.e. 32
//     rows of the tile), round to the output type and store.
// Blocks are persistent: one per SM, each walking over 128 x bn tiles, with two accumulators in TMEM so that the
// epilogue of one tile overlaps the MMAs of the next. Rows and columns beyond M, N and K are zero-filled by TMA on
// the way in and masked on the way out. Every wait on an mbarrier is bounded: if one runs out, the block records
// OXR_WAIT_EXPIRED in the status word, stops waiting, frees its tensor memory and returns.
//
// A few hundred rows and a narrow W give few tiles, fewer than SMs, while the product is still bound by streaming W
// (fewer rows than that take the few-rows kernel of gemm_tcgen05_few_rows.cu). The SPLIT variant therefore deals the k steps of a tile out to `splits` shares and
// makes (tile, share) the unit of work, so that every SM streams a part of W. A unit writes its fp32 partial tile to
// a workspace and takes a ticket of its tile; the unit that draws the last ticket adds the partial tiles in the order
// of the shares (so the sum does not depend on who came last), rounds and stores. Nothing waits for another block.
#include "umma.cuh"

namespace {
constexpr int RED_ROWS = 8;       // rows per lane and pass when partial tiles are added
constexpr int TC_THREADS = 192;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..5: epilogue

__host__ __device__ constexpr int stage_bytes(int bn) { return A_BYTES + bn * BK * 2; }

// Barrier 1 is the epilogue warps' own (128 threads); the other warps never touch it.
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool epilogue_all(bool v) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"((uint32_t)v) : "memory");
    return r != 0;
}

// Tile order: blocks that run at the same time share few W tiles and GROUP_M consecutive X tiles, so that W is
// streamed from HBM once and the X tiles of a group stay in L2 (W can be far larger than L2, X of a group is not).
__device__ __forceinline__ void tile_origin(int tile, int M, int N, int bn, int& m0, int& n0) {
    constexpr int GROUP_M = 32;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + bn - 1) / bn;
    const int per_group = GROUP_M * tiles_n;
    const int group = tile / per_group, within = tile % per_group;
    const int group_rows = min(GROUP_M, tiles_m - group * GROUP_M);
    m0 = (group * GROUP_M + within % group_rows) * BM;
    n0 = (within / group_rows) * bn;
}

// GATED (never with SPLIT): W's rows alternate in groups of 8 between a gate and an up projection, and the epilogue
// writes silu(gate) * up into C [M, N / 2] instead of the product itself.
// Persistent: block b computes units b, b + gridDim.x, ... The accumulator is double-buffered in tensor memory
// (two buffers `acc_stride` columns apart), so the epilogue warps drain one unit while the MMA warp already
// accumulates the next. Without SPLIT a unit is a tile. With SPLIT it is (tile, share): unit u is share u % splits
// of tile u / splits, and share r takes the 64-wide k steps r, r + splits, ...: the shares of a tile run side by
// side, read neighbouring 128-byte pieces of W's rows, and finish together.
template <typename TO, bool SPLIT, bool GATED>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_kernel(TO* __restrict__ C, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    int M, int N, int K, int bn, int stages, int tmem_cols, int num_tiles, int splits, float* __restrict__ partial,
                    unsigned int* __restrict__ tickets, int* status) {
    static_assert(!(GATED && SPLIT), "the gated epilogue is the plain one's variant only");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms are 1024 B
    const int stage_size = stage_bytes(bn);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)stages * stage_size);
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* accum_full = empty + MAX_STAGES;   // [2] MMA -> epilogue
    uint64_t* accum_empty = accum_full + 2;      // [2] epilogue -> MMA (4 arrivals: one per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_empty + 2);
    uint32_t* gave_up = tmem_slot + 1;
    uint32_t* drew_last = gave_up + 1;
    static_assert((2 * MAX_STAGES + 4) * 8 + 12 <= BARRIER_BYTES, "barriers outgrow their space");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    const int kb_step = SPLIT ? splits : 1;
    const int num_units = SPLIT ? num_tiles * splits : num_tiles;
    const uint32_t acc_stride = (uint32_t)tmem_cols / 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(accum_full + i, 1); mbar_init(accum_empty + i, 4); }
        *gave_up = 0;
        mbar_fence_init();
    }
    if (warp == 1) {   // the whole warp allocates the tensor memory and gives up the permit to allocate more
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
            int s = 0;             // the stage ring does not restart per unit
            uint32_t phase = 0;
            bool ok = true;
            // No kernel writes the weights, so their tiles of the first ring of stages are requested before this kernel
            // (when it is launched dependent on the one before) waits for that one to finish; the activations' tiles
            // of the same stages follow after the wait.
            int early = 0;
            for (int unit = blockIdx.x; unit < num_units && early < stages; unit += gridDim.x) {
                const int tile = SPLIT ? unit / splits : unit;
                int m0, n0;
                tile_origin(tile, M, N, bn, m0, n0);
                for (int kb = SPLIT ? unit % splits : 0; kb < num_kb && early < stages; kb += kb_step, ++early) {
                    unsigned char* a_dst = tiles + (size_t)early * stage_size;
                    mbar_expect_tx(full + early, (uint32_t)stage_size);
                    tma_load_2d(a_dst + A_BYTES, &map_w, kb * BK, n0, full + early);
                }
            }
            pdl_wait();
            int step = 0;
            for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
                const int tile = SPLIT ? unit / splits : unit;
                int m0, n0;
                tile_origin(tile, M, N, bn, m0, n0);
                for (int kb = SPLIT ? unit % splits : 0; kb < num_kb; kb += kb_step, ++step) {
                    unsigned char* a_dst = tiles + (size_t)s * stage_size;
                    if (step < early) {   // first ring: the stage is free and armed, its weight tile is on its way
                        tma_load_2d(a_dst, &map_x, kb * BK, m0, full + s);
                    } else {
                        if (!mbar_wait(empty + s, phase ^ 1)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 0); ok = false; break; }
                        mbar_expect_tx(full + s, (uint32_t)stage_size);
                        tma_load_2d(a_dst, &map_x, kb * BK, m0, full + s);
                        tma_load_2d(a_dst + A_BYTES, &map_w, kb * BK, n0, full + s);
                    }
                    if (++s == stages) { s = 0; phase ^= 1; }
                }
            }
            pdl_trigger();   // every load of this block is issued: a chained kernel after this one may be scheduled
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            const uint32_t idesc = umma_idesc(BM, bn);
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++it) {
                const int kb0 = SPLIT ? unit % splits : 0;
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait(accum_empty + acc, acc_phase ^ 1)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 3); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)acc * acc_stride;
                for (int kb = kb0; kb < num_kb; kb += kb_step) {
                    if (!mbar_wait(full + s, phase)) { atomicExch(gave_up, 1u); oxr_report(status, OXR_WAIT_EXPIRED, 1); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_addr(tiles + (size_t)s * stage_size);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // inside the 128-byte swizzle row, the next 16 k-values start 32 bytes further
                        umma_bf16(tmem_d, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc,
                                  (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty + s);   // the stage is free once these MMAs have read it
                    if (++s == stages) { s = 0; phase ^= 1; }
                }
                umma_commit(accum_full + acc);   // arrives when every MMA issued so far is complete (also after giving up)
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: TMEM -> registers -> global
        pdl_wait();   // C and the workspace may still be read by the kernels before this one
        const int quarter = warp & 3;                     // this warp may touch TMEM lanes 32 * quarter .. + 31
        int it = 0;
        for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++it) {
            const int tile = SPLIT ? unit / splits : unit;
            int m0, n0;
            tile_origin(tile, M, N, bn, m0, n0);
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int row = m0 + quarter * 32 + lane;
            bool ok = mbar_wait(accum_full + acc, acc_phase);
            if (!ok) { atomicExch(gave_up, 1u); if (lane == 0) oxr_report(status, OXR_WAIT_EXPIRED, 2); }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            ok = ok && (*reinterpret_cast<volatile uint32_t*>(gave_up) == 0);
            if constexpr (SPLIT) ok = epilogue_all(ok);   // the four warps meet at barriers below: they leave together
            else ok = __all_sync(0xffffffffu, ok);        // tcgen05.ld is warp-wide: all lanes take the same path
            if (!ok) break;
            const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * acc_stride;
            const size_t tile_floats = (size_t)BM * bn;
            // SPLIT: this share's partial tile -> workspace [share][tile][BM][bn], rows of the matrix only
            float* mine = !SPLIT ? nullptr : partial + ((size_t)(unit % splits) * num_tiles + tile) * tile_floats + (size_t)(quarter * 32 + lane) * bn;
#pragma unroll 1
            for (int c0 = 0; c0 < bn; c0 += 32) {
                uint32_t v[32];
                const int count = min(32, bn - c0);   // 32, or 16 at the end of a tile whose width is an odd multiple of 16
                if (count == 32) tmem_ld_32x32(acc_addr + (uint32_t)c0, v);
                else tmem_ld_32x16(acc_addr + (uint32_t)c0, v);
                if (row < M) {
                    if constexpr (SPLIT) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (4 * j < count) reinterpret_cast<uint4*>(mine + c0)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else if (n0 + c0 < N) {
                        if constexpr (GATED) store_row_piece_gated<TO>(C + (size_t)row * (N / 2) + (n0 + c0) / 2, v, count, n0 + c0, N);
                        else store_row_piece<TO>(C + (size_t)row * N + n0 + c0, v, count, n0 + c0, N);
                    }
                }
            }
            // this warp has read its quarter of the accumulator: hand the buffer back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(accum_empty + acc);
            if constexpr (SPLIT) {
                // ticket: the partial tiles are published before it is drawn, and read only after the last one is
                __threadfence();
                epilogue_sync();
                if (threadIdx.x == 64) {
                    const unsigned int t = atomicAdd(tickets + tile, 1u);
                    const bool last = t + 1 == (unsigned int)splits;
                    if (last) tickets[tile] = 0;   // left zero for the next launch
                    *drew_last = last ? 1u : 0u;
                }
                epilogue_sync();
                if (*reinterpret_cast<volatile uint32_t*>(drew_last) != 0) {
                    __threadfence();
                    const int rows = min(BM, M - m0);
                    const float* first = partial + (size_t)tile * tile_floats;
                    const size_t share_stride = (size_t)num_tiles * tile_floats;
                    // eight rows per pass and lane, the loads of four shares in flight together: the loads' latency
                    // under a saturated memory system, not their number, is what this costs
                    for (int c = lane * 4; c < bn; c += 128) {
                        const int col = n0 + c;
                        for (int r0 = quarter; r0 < rows; r0 += 4 * RED_ROWS) {
                            float4 sum[RED_ROWS];
#pragma unroll
                            for (int i = 0; i < RED_ROWS; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                            for (int s = 0; s < splits; ++s) {
                                float4 p[RED_ROWS];
#pragma unroll
                                for (int i = 0; i < RED_ROWS; ++i) {
                                    const int r = min(r0 + 4 * i, rows - 1);
                                    p[i] = __ldcg(reinterpret_cast<const float4*>(first + (size_t)s * share_stride + (size_t)r * bn + c));
                                }
#pragma unroll
                                for (int i = 0; i < RED_ROWS; ++i) { sum[i].x += p[i].x; sum[i].y += p[i].y; sum[i].z += p[i].z; sum[i].w += p[i].w; }
                            }
#pragma unroll
                            for (int i = 0; i < RED_ROWS; ++i) {
                                const int r = r0 + 4 * i;
                                if (r >= rows) break;
                                TO* dst = C + (size_t)(m0 + r) * N + col;
                                if (col + 4 <= N && (uintptr_t)dst % (4 * sizeof(TO)) == 0) {
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
                                    for (int j = 0; j < 4 && col + j < N; ++j) dst[j] = Num<TO>::from_f32(e[j]);
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------- host side
template <typename TO, bool SPLIT, bool GATED = false>
int launch(void* C, const void* X, const void* W, int M, int N, int K, int bn, int splits, float* partial, unsigned int* tickets, int* status,
           cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<TO, SPLIT, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    CUtensorMap map_x, map_w;
    if (!oxr_make_map_bf16(&map_x, X, M, K, BM) || !oxr_make_map_bf16(&map_w, W, N, K, bn)) return OXR_BAD_ARGUMENT;
    const long long tiles = (long long)((N + bn - 1) / bn) * ((M + BM - 1) / BM);
    const long long units = tiles * (SPLIT ? splits : 1);
    if (units > 0x7fffffffLL) return OXR_BAD_ARGUMENT;
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
            num_sms = 148;
    }
    int stages = RING_BYTES / stage_bytes(bn);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    int tmem_cols = 32;                      // a power of two that holds both accumulators
    while (tmem_cols < 2 * bn) tmem_cols *= 2;
    dim3 grid((unsigned)(units < num_sms ? units : num_sms));   // one block per SM (its shared memory fills the SM)
    oxr_launch(gemm_tcgen05_kernel<TO, SPLIT, GATED>, grid, dim3(TC_THREADS), SMEM_BYTES, stream, true, (TO*)C, map_x, map_w, M, N, K, bn,
               stages, tmem_cols, (int)tiles, splits, partial, tickets, status);
    return oxr_launch_status();
}
}  // namespace

// out_dtype: 0 = float32, 1 = bfloat16. Requires K % 8 == 0 (rows are whole 16-byte words) and 16-byte aligned X, W.
// tile_n: columns of the output per tile, a multiple of 16 from 16 to 256.
// splits > 1 deals the 64-wide k steps out to that many shares per tile (at most as many as steps); `partial` then
// holds splits * tiles * 128 * tile_n floats (tiles = ceil(M / 128) * ceil(N / tile_n)) and `tickets` one zeroed
// counter per tile, which the kernel leaves zeroed.
OXR_API int oxr_gemm_tcgen05_bf16(void* C, const void* X, const void* W, int M, int N, int K, int out_dtype, int tile_n, int splits,
                                  float* partial, unsigned int* tickets, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0) return OXR_BAD_ARGUMENT;
    if (tile_n < 16 || tile_n > MAX_BN || tile_n % 16 != 0) return OXR_BAD_ARGUMENT;
    if (splits > 1) {
        if (partial == nullptr || tickets == nullptr || (uintptr_t)partial % 16 != 0 || splits > (K + BK - 1) / BK) return OXR_BAD_ARGUMENT;
        if (out_dtype == 1) return launch<__nv_bfloat16, true>(C, X, W, M, N, K, tile_n, splits, partial, tickets, status, stream);
        if (out_dtype == 0) return launch<float, true>(C, X, W, M, N, K, tile_n, splits, partial, tickets, status, stream);
        return OXR_BAD_ARGUMENT;
    }
    if (out_dtype == 1) return launch<__nv_bfloat16, false>(C, X, W, M, N, K, tile_n, 1, nullptr, nullptr, status, stream);
    if (out_dtype == 0) return launch<float, false>(C, X, W, M, N, K, tile_n, 1, nullptr, nullptr, status, stream);
    return OXR_BAD_ARGUMENT;
}

// C [M, N / 2] = silu(X Wg^T) * (X Wu^T) in bf16 for W [N, K] whose gate and up rows alternate in groups of 8 (N a
// multiple of 16); tile_n as above, no shares of k.
OXR_API int oxr_gemm_tcgen05_gated_bf16(void* C, const void* X, const void* W, int M, int N, int K, int tile_n, int* status,
                                        cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (N % 16 != 0 || K <= 0 || K % 8 != 0 || (uintptr_t)X % 16 != 0 || (uintptr_t)W % 16 != 0 || (uintptr_t)C % 16 != 0) return OXR_BAD_ARGUMENT;
    if (tile_n < 16 || tile_n > MAX_BN || tile_n % 16 != 0) return OXR_BAD_ARGUMENT;
    return launch<__nv_bfloat16, false, true>(C, X, W, M, N, K, tile_n, 1, nullptr, nullptr, status, stream);
}
