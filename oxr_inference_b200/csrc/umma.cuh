// What the tcgen05 matrix-product kernels share: tile constants, shared-memory matrix and instruction descriptors,
// the tcgen05.mma / commit / ld wrappers and the epilogue's store of a piece of an output row.
#pragma once

#include "tma.cuh"

namespace {
constexpr int BM = 128;           // rows of X per block and tile = TMEM lanes
constexpr int BK = 64;            // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int MAX_BN = 256;       // widest tile: one tcgen05.mma takes N <= 256, a TMA box 256 rows
constexpr int MAX_STAGES = 10;
constexpr int A_BYTES = BM * BK * 2;
constexpr int BARRIER_BYTES = 256;
constexpr int SMEM_BYTES = 227 * 1024;                                  // all a block may have
constexpr int RING_BYTES = SMEM_BYTES - 1024 /* alignment slack */ - BARRIER_BYTES;

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
// 32 lanes x 32 (or 16) consecutive columns of tensor memory: lane i of the warp gets row i's values.
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
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
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
// `count` (16 or 32) consecutive fp32 values of one output row -> C, rounded to TO; columns from `col0` on, N in all.
template <typename TO>
__device__ __forceinline__ void store_row_piece(TO* dst, const uint32_t (&v)[32], int count, int col0, int N) {
    if (col0 + count <= N && ((uintptr_t)dst % 16 == 0)) {
        if constexpr (sizeof(TO) == 2) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (8 * j >= count) break;
                uint4 o;
                __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    op[e] = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]), __uint_as_float(v[8 * j + 2 * e + 1]));
                reinterpret_cast<uint4*>(dst)[j] = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (4 * j >= count) break;
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < count && col0 + j < N) dst[j] = Num<TO>::from_f32(__uint_as_float(v[j]));
    }
}


// The same piece of a product whose columns alternate in groups of 8 between a gate and an up projection (columns
// 16j .. 16j+7 gate 8j .. 8j+7, 16j+8 .. 16j+15 the matching up values; col0 a multiple of 16): writes
// silu(gate) * up (oxr_runtime/language.py:102-104), `count / 2` values, into a row of N / 2 columns. `dst` points at
// column col0 / 2 of that row.
template <typename TO>
__device__ __forceinline__ void store_row_piece_gated(TO* dst, const uint32_t (&v)[32], int count, int col0, int N) {
    float o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float g = __uint_as_float(v[(j / 8) * 16 + j % 8]), u = __uint_as_float(v[(j / 8) * 16 + 8 + j % 8]);
        o[j] = __fdividef(g, 1.f + __expf(-g)) * u;   // the fast division: two ulp, far inside a bf16 step
    }
    const int outs = count / 2;
    if (col0 + count <= N && ((uintptr_t)dst % 16 == 0)) {
        if constexpr (sizeof(TO) == 2) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (8 * j >= outs) break;
                uint4 w;
                __nv_bfloat162* wp = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                for (int e = 0; e < 4; ++e) wp[e] = __floats2bfloat162_rn(o[8 * j + 2 * e], o[8 * j + 2 * e + 1]);
                reinterpret_cast<uint4*>(dst)[j] = w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (4 * j >= outs) break;
                reinterpret_cast<float4*>(dst)[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < outs && col0 + (j / 8) * 16 + 8 + j % 8 < N) dst[j] = Num<TO>::from_f32(o[j]);
    }
}
}  // namespace
