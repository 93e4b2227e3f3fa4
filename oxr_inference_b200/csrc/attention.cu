// Paged grouped-query attention over the KV cache for a mixed batch: each request brings q_len >= 1 new
// tokens (a prompt portion or one decoded token) whose K and V are already in the cache; a query at absolute
// position p sees the keys at positions <= p of its own request (and > p - window when the layer has a
// window). Compiled once per head size: -DHEAD_DIM=<multiple of 16, at most 256>.
//
// This is the engine's counterpart of the reference's three library calls `attention.varlen`,
// `attention.paged_decode` and `attention.paged_extend` (oxr_runtime/attention.py:47-109), with the masking
// rule of `paged_extend` ("queries aligned to the end of the context", attention.py:100-101) generalised to a
// different q_len per request. Scores, softmax and the weighted sum of V are computed in fp32.
//
// Work is cut into tiles of BM = 16 rows; a row is one (token, q head) pair, the q heads of one KV head being
// packed next to each other so that K and V are read once for the whole group. Keys are visited in blocks of
// BN = 32 that start at absolute positions 0, 32, 64, ...; because the blocks do not depend on where a portion
// starts or on the rest of the batch, a row's result is bit-identical however the work was cut.
#include "tma.cuh"
OXR_TL_DEFINE(oxr_tl_read_attn)

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size: a multiple of 16 up to 256");

namespace {
constexpr int D = HEAD_DIM;
constexpr int BM = 16;
constexpr int BN = 32;
constexpr int SIMT_WARPS = 4;
constexpr int ROWS_PER_WARP = BM / SIMT_WARPS;
constexpr int DCHUNKS = (D + 31) / 32;
constexpr int KS_STRIDE = D + 1;

struct AttnArgs {
    const int* tile_req;     // [tiles] request of each tile
    const int* tile_tok0;    // [tiles] first token (offset inside the request's new tokens) of each tile
    const int* cu_q;         // [n + 1] start of each request's new tokens in the packed token axis
    const int* ctx_lens;     // [n] tokens in the cache after this step (context before + q_len)
    const int* block_table;  // [n, table_width] page ids; entries of released pages may hold anything
    int table_width;
    int page_size;
    int page_shift;          // log2(page_size) when it is a power of two, else -1
    int num_pages;
    int H, KV;
    int heads_per_tile;      // q heads of one KV head handled by one tile: min(G, BM)
    int tokens_per_tile;     // BM / heads_per_tile
    int head_groups;         // ceil(G / heads_per_tile)
    float scale;
    int window;              // 0 = unlimited
    int* status;
};

template <typename T> struct Vec;   // 16-byte vectors of T
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            out[2 * i] = f.x; out[2 * i + 1] = f.y;
        }
    }
};

template <typename T>
__global__ void __launch_bounds__(SIMT_WARPS * 32)
attn_simt_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_cache,
                 const T* __restrict__ v_cache, const AttnArgs a) {
    extern __shared__ float smem[];
    float* Qs = smem;                       // [BM][D]
    float* Ks = Qs + BM * D;                // [BN][D + 1]
    float* Vs = Ks + BN * KS_STRIDE;        // [BN][D]
    float* Ps = Vs + BN * D;                // [BM][BN]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.x;
    const int kvh = blockIdx.y / a.head_groups, hg = blockIdx.y % a.head_groups;
    const int G = a.H / a.KV;
    const int req = a.tile_req[tile], tok0 = a.tile_tok0[tile];
    const int q_begin = a.cu_q[req], q_len = a.cu_q[req + 1] - q_begin;
    const int ctx = a.ctx_lens[req];
    const int pos0 = ctx - q_len;
    const int tok_end = min(tok0 + a.tokens_per_tile, q_len);   // exclusive
    if (tok0 >= tok_end) return;
    const int rows_used = a.tokens_per_tile * a.heads_per_tile;

    // ---- Q tile -> shared (fp32); rows without a (token, head) are zero
    for (int i = tid; i < BM * D; i += SIMT_WARPS * 32) {
        const int r = i / D, d = i % D;
        const int tok = tok0 + r / a.heads_per_tile, gh = hg * a.heads_per_tile + r % a.heads_per_tile;
        float v = 0.f;
        if (r < rows_used && tok < tok_end && gh < G)
            v = Num<T>::to_f32(q[((size_t)(q_begin + tok) * a.H + (size_t)kvh * G + gh) * D + d]);
        Qs[i] = v;
    }

    int row_pos[ROWS_PER_WARP];
    bool row_ok[ROWS_PER_WARP];
    float m[ROWS_PER_WARP], l[ROWS_PER_WARP], o[ROWS_PER_WARP][DCHUNKS];
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
        const int r = warp * ROWS_PER_WARP + i;
        const int tok = tok0 + r / a.heads_per_tile, gh = hg * a.heads_per_tile + r % a.heads_per_tile;
        row_ok[i] = r < rows_used && tok < tok_end && gh < G;
        row_pos[i] = pos0 + tok;
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < DCHUNKS; ++c) o[i][c] = 0.f;
    }

    const int k_end = pos0 + tok_end;                                                  // exclusive, causal bound
    const int k_lo = a.window > 0 ? max(0, pos0 + tok0 - a.window + 1) : 0;            // first key any row sees
    const int k_first = (k_lo / BN) * BN;
    constexpr int VE = Vec<T>::N, VPK = D / VE;                                       // vectors per key

    for (int kt = k_first; kt < k_end; kt += BN) {
        __syncthreads();   // previous tile fully consumed (also orders the Q store before the first use)
        for (int v = tid; v < BN * VPK; v += SIMT_WARPS * 32) {
            const int j = v / VPK, part = v % VPK;
            const int kp = kt + j;
            float kf[VE], vf[VE];
#pragma unroll
            for (int e = 0; e < VE; ++e) kf[e] = vf[e] = 0.f;
            if (kp >= k_lo && kp < k_end) {
                const int page = a.block_table[(size_t)req * a.table_width + kp / a.page_size];
                if (page < 0 || page >= a.num_pages) {
                    if (part == 0) oxr_report(a.status, OXR_BAD_PAGE, req);
                } else {
                    const size_t base = (((size_t)page * a.page_size + kp % a.page_size) * a.KV + kvh) * D + part * VE;
                    Vec<T>::load(k_cache + base, kf);
                    Vec<T>::load(v_cache + base, vf);
                }
            }
#pragma unroll
            for (int e = 0; e < VE; ++e) {
                Ks[j * KS_STRIDE + part * VE + e] = kf[e];
                Vs[j * D + part * VE + e] = vf[e];
            }
        }
        __syncthreads();

        // ---- scores: lane = key, this warp's rows
        float s[ROWS_PER_WARP];
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) s[i] = 0.f;
        const float* krow = Ks + lane * KS_STRIDE;
#pragma unroll 8
        for (int d = 0; d < D; ++d) {
            const float kv = krow[d];
#pragma unroll
            for (int i = 0; i < ROWS_PER_WARP; ++i) s[i] = fmaf(Qs[(warp * ROWS_PER_WARP + i) * D + d], kv, s[i]);
        }
        const int kp = kt + lane;
        float alpha[ROWS_PER_WARP];
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) {
            const bool seen = row_ok[i] && kp <= row_pos[i] && (a.window <= 0 || kp > row_pos[i] - a.window);
            const float sv = seen ? s[i] * a.scale : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(sv));
            float p = 0.f;
            alpha[i] = 1.f;
            if (m_new != -INFINITY) {
                alpha[i] = expf(m[i] - m_new);   // exp(-inf) = 0 for the first block with a visible key
                p = seen ? expf(sv - m_new) : 0.f;
            }
            l[i] = l[i] * alpha[i] + warp_sum(p);
            m[i] = m_new;
            Ps[(warp * ROWS_PER_WARP + i) * BN + lane] = p;
        }
        __syncwarp();

        // ---- O += P V: lane = column of V
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i)
#pragma unroll
            for (int c = 0; c < DCHUNKS; ++c) o[i][c] *= alpha[i];
        for (int j = 0; j < BN; ++j) {
            float pv[ROWS_PER_WARP];
#pragma unroll
            for (int i = 0; i < ROWS_PER_WARP; ++i) pv[i] = Ps[(warp * ROWS_PER_WARP + i) * BN + j];
#pragma unroll
            for (int c = 0; c < DCHUNKS; ++c) {
                const int d = lane + 32 * c;
                if (d < D) {
                    const float vv = Vs[j * D + d];
#pragma unroll
                    for (int i = 0; i < ROWS_PER_WARP; ++i) o[i][c] = fmaf(pv[i], vv, o[i][c]);
                }
            }
        }
        __syncwarp();
    }

#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
        if (!row_ok[i]) continue;
        const int r = warp * ROWS_PER_WARP + i;
        const int tok = tok0 + r / a.heads_per_tile, gh = hg * a.heads_per_tile + r % a.heads_per_tile;
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
        T* dst = out + ((size_t)(q_begin + tok) * a.H + (size_t)kvh * G + gh) * D;
#pragma unroll
        for (int c = 0; c < DCHUNKS; ++c) {
            const int d = lane + 32 * c;
            if (d < D) dst[d] = Num<T>::from_f32(o[i][c] * inv);
        }
    }
}

constexpr size_t SIMT_SMEM = (size_t)(BM * D + BN * KS_STRIDE + BN * D + BM * BN) * sizeof(float);

template <typename T>
int launch_simt(void* out, const void* q, const void* k_cache, const void* v_cache, const AttnArgs& a, int num_tiles,
                cudaStream_t stream) {
    static bool configured = false;   // one attribute call per process and dtype
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_simt_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SIMT_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    dim3 grid(num_tiles, a.KV * a.head_groups);
    attn_simt_kernel<T><<<grid, SIMT_WARPS * 32, SIMT_SMEM, stream>>>((T*)out, (const T*)q, (const T*)k_cache, (const T*)v_cache, a);
    return oxr_launch_status();
}
}  // namespace


// =====================================================================================================================
// bfloat16 on the tensor cores (mma.sync m16n8k16, fp32 accumulation): the same attention, two kernels.
//
//  * attn_mma_prefill_kernel: a tile is 64 rows; warp w owns rows 16w..16w+15 and visits every key block.
//  * attn_mma_decode_kernel: a tile is 16 rows (one decoded token's whole group of q heads, or a few tokens of a
//    short portion); the four warps share the rows and each takes a quarter of every 64-key block; the key range
//    is further split over gridDim.z blocks; the block that finishes last merges the partial (max, sum, output).
//
// K and V blocks are gathered page by page with cp.async (16 bytes per request, zero-filled outside the visible
// range) into padded shared-memory rows, two stages deep; fragments are read with ldmatrix.
// =====================================================================================================================
namespace {
typedef __nv_bfloat16 bf16;
constexpr int PADE = 8;                        // 16 bytes of padding per row: ldmatrix rows fall on different banks
constexpr int LDS = D + PADE;                  // shared-memory row stride in elements
constexpr int MMA_BN = 64;                     // keys per block
constexpr int MMA_THREADS = 128;
constexpr int KSTEPS = D / 16;                 // k16 steps over the head dimension
constexpr int DT8 = D / 8;                     // n8 tiles over the head dimension
constexpr bool Q_IN_REGS = D <= 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are zero-filled and gmem is not read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Gather keys [k0, k0 + MMA_BN) of one request into Ks / Vs (rows of LDS elements); keys outside [k_lo, k_end)
// become zeros. All MMA_THREADS threads take part: a thread keeps its 16-byte column and walks down the rows, so
// that per row it needs one block-table lookup, one multiply and two cp.async. page_shift >= 0 when the page size
// is a power of two.
__device__ __forceinline__ void load_kv_block(bf16* Ks, bf16* Vs, const bf16* __restrict__ k_cache,
                                              const bf16* __restrict__ v_cache, const int* __restrict__ table_row,
                                              const AttnArgs& a, int kvh, int k0, int k_lo, int k_end, int req) {
    constexpr int CPR = D / 8;                                    // 16-byte chunks per row
    constexpr int ROW_STEP = MMA_THREADS / CPR > 0 ? MMA_THREADS / CPR : 1;
    static_assert(CPR <= MMA_THREADS, "a row has at most as many 16-byte chunks as the block has threads");
    if (threadIdx.x >= ROW_STEP * CPR) return;                   // head sizes whose chunk count does not divide the block
    const int c = threadIdx.x % CPR;
    const size_t row_elems = (size_t)a.KV * D;
    const size_t col = (size_t)kvh * D + c * 8;
    const int smem_col = c * 8;
    for (int j = threadIdx.x / CPR; j < MMA_BN; j += ROW_STEP) {
        const int kp = k0 + j;
        bool ok = kp >= k_lo && kp < k_end;
        size_t base = 0;
        if (ok) {
            int page, slot;
            if (a.page_shift >= 0) {
                page = table_row[kp >> a.page_shift];
                slot = (page << a.page_shift) + (kp & (a.page_size - 1));
            } else {
                page = table_row[kp / a.page_size];
                slot = page * a.page_size + kp % a.page_size;
            }
            if (page < 0 || page >= a.num_pages) {
                if (c == 0) oxr_report(a.status, OXR_BAD_PAGE, req);
                ok = false;
            } else {
                base = (size_t)slot * row_elems + col;
            }
        }
        cp_async_16(Ks + j * LDS + smem_col, k_cache + base, ok);
        cp_async_16(Vs + j * LDS + smem_col, v_cache + base, ok);
    }
}

// Where element (row, d) of a K or V block lives in shared memory. Padded layout (cp.async gathers): rows of LDS
// elements. Swizzled layout (TMA gathers): panels of 64 keys x 64 d, 128 bytes per row, the 16-byte chunks of a row
// XOR-ed with the row number modulo 8 (the TMA 128-byte swizzle), 8 KB per panel.
template <bool SWZ>
__device__ __forceinline__ const bf16* kv_elem(const bf16* base, int row, int d) {
    if constexpr (SWZ) {
        return base + (d >> 6) * (MMA_BN * 64) + row * 64 + ((((d & 63) >> 3) ^ (row & 7)) << 3);
    } else {
        return base + row * LDS + d;
    }
}

// One warp: S = Q K^T for its 16 rows and NK keys starting at Kw, masked online softmax, O += P V.
// qf: Q fragments when Q_IN_REGS, else read from Qw (this warp's 16 rows in shared memory).
template <int NK, bool SWZ = false, bool QREG = Q_IN_REGS>
__device__ __forceinline__ void warp_block(const uint32_t (&qf)[QREG ? KSTEPS : 1][4], const bf16* Qw, const bf16* Kw,
                                           const bf16* Vw, int key0, const int (&row_pos)[2], const bool (&row_ok)[2],
                                           int window, bool full_block, float scale_log2, float (&m)[2], float (&l)[2],
                                           float (&o)[DT8][4]) {
    constexpr int NT = NK / 8;
    const int lane = threadIdx.x & 31, t = lane & 3;
    float s[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t aq[4];
        if constexpr (QREG) {
            aq[0] = qf[kk][0]; aq[1] = qf[kk][1]; aq[2] = qf[kk][2]; aq[3] = qf[kk][3];
        } else {
            ldsm_x4(aq, Qw + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));
        }
#pragma unroll
        for (int np = 0; np < NK / 16; ++np) {
            uint32_t bk[4];
            ldsm_x4(bk, kv_elem<SWZ>(Kw, np * 16 + (lane & 7) + 8 * (lane >> 4), kk * 16 + 8 * ((lane >> 3) & 1)));
            mma16816(s[2 * np], aq, bk[0], bk[1]);
            mma16816(s[2 * np + 1], aq, bk[2], bk[3]);
        }
    }
    // ---- mask, running maximum. A block that every row of the warp sees in full (no causal or window edge inside)
    // needs no per-element test.
    float mx[2] = {-INFINITY, -INFINITY};
    if (full_block) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[i][e] *= scale_log2;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[i][e]);
            }
    } else {
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const int kp = key0 + i * 8 + 2 * t + (e & 1);
                const bool seen = row_ok[r] && kp <= row_pos[r] && (window <= 0 || kp > row_pos[r] - window);
                s[i][e] = seen ? s[i][e] * scale_log2 : -INFINITY;
                mx[r] = fmaxf(mx[r], s[i][e]);
            }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        alpha[r] = (m_new == -INFINITY) ? 1.f : exp2f(m[r] - m_new);
        m[r] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const float p = (m[r] == -INFINITY) ? 0.f : exp2f(s[i][e] - m[r]);
            s[i][e] = p;
            psum[r] += p;
        }
    l[0] = l[0] * alpha[0] + psum[0];
    l[1] = l[1] * alpha[1] + psum[1];
    // the accumulator is rescaled only when some row's maximum moved (after the first blocks it rarely does)
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < DT8; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < NK / 16; ++kk) {
        uint32_t ap[4];
        ap[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        ap[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        ap[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        ap[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            uint32_t bv[4];
            ldsm_x4_trans(bv, kv_elem<SWZ>(Vw, kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dp * 16 + 8 * (lane >> 4)));
            mma16816(o[2 * dp], ap, bv[0], bv[1]);
            mma16816(o[2 * dp + 1], ap, bv[2], bv[3]);
        }
    }
}

// Row r of a tile of `rows` rows -> (token offset inside the request's new tokens, q head inside the group).
struct TileGeometry {
    int req, tok0, kvh, hg, G, q_begin, q_len, pos0, tok_end, heads_per_tile, rows_used;
    __device__ __forceinline__ bool row(int r, int& tok, int& gh) const {
        tok = tok0 + r / heads_per_tile;
        gh = hg * heads_per_tile + r % heads_per_tile;
        return r < rows_used && tok < tok_end && gh < G;
    }
};
// `tile`: index into the tile list (default: the block's x index); `y`: (KV head, head group) index (default: the
// block's y index).
__device__ __forceinline__ TileGeometry tile_geometry(const AttnArgs& a, int rows, int tile = -1, int y = -1) {
    if (tile < 0) tile = blockIdx.x;
    if (y < 0) y = blockIdx.y;
    TileGeometry g;
    g.G = a.H / a.KV;
    g.heads_per_tile = g.G < rows ? g.G : rows;
    const int tokens_per_tile = rows / g.heads_per_tile;
    const int head_groups = (g.G + g.heads_per_tile - 1) / g.heads_per_tile;
    g.kvh = y / head_groups;
    g.hg = y % head_groups;
    g.req = a.tile_req[tile];
    g.tok0 = a.tile_tok0[tile];
    g.q_begin = a.cu_q[g.req];
    g.q_len = a.cu_q[g.req + 1] - g.q_begin;
    g.pos0 = a.ctx_lens[g.req] - g.q_len;
    g.tok_end = min(g.tok0 + tokens_per_tile, g.q_len);
    g.rows_used = tokens_per_tile * g.heads_per_tile;
    return g;
}

// Q rows [row0, row0 + nrows) of the tile -> shared memory (zeros for rows without a token/head).
__device__ __forceinline__ void load_q_rows(bf16* Qs, const bf16* __restrict__ q, const AttnArgs& a, const TileGeometry& g,
                                            int nrows) {
    constexpr int CPR = D / 8;
    for (int idx = threadIdx.x; idx < nrows * CPR; idx += MMA_THREADS) {
        const int r = idx / CPR, c = idx % CPR;
        int tok, gh;
        const bool ok = g.row(r, tok, gh);
        const size_t src = ok ? ((size_t)(g.q_begin + tok) * a.H + (size_t)g.kvh * g.G + gh) * D + c * 8 : 0;
        cp_async_16(Qs + r * LDS + c * 8, q + src, ok);
    }
}

constexpr int PREFILL_ROWS = 64;
constexpr size_t PREFILL_SMEM = (size_t)(PREFILL_ROWS + 4 * MMA_BN) * LDS * sizeof(bf16);

__global__ void __launch_bounds__(MMA_THREADS)
attn_mma_prefill_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ k_cache,
                        const bf16* __restrict__ v_cache, int n_tiles, int n_y, const AttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + PREFILL_ROWS * LDS;          // 2 stages
    bf16* Vs = Ks + 2 * MMA_BN * LDS;            // 2 stages
    // the list is in token order and later tiles of a prompt see more keys: start the long ones first, and all (KV head,
    // head group) pairs of a tile side by side (a one-dimensional grid), so that no pair's long tiles wait behind another's short ones
    const TileGeometry g = tile_geometry(a, PREFILL_ROWS, n_tiles - 1 - (int)(blockIdx.x / (unsigned)n_y), (int)(blockIdx.x % (unsigned)n_y));
    if (g.tok0 >= g.tok_end) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int* table_row = a.block_table + (size_t)g.req * a.table_width;

    const int k_end = g.pos0 + g.tok_end;
    const int k_lo = a.window > 0 ? max(0, g.pos0 + g.tok0 - a.window + 1) : 0;
    const int k_first = (k_lo / MMA_BN) * MMA_BN;
    const int n_blocks = (k_end - k_first + MMA_BN - 1) / MMA_BN;

    load_q_rows(Qs, q, a, g, PREFILL_ROWS);
    load_kv_block(Ks, Vs, k_cache, v_cache, table_row, a, g.kvh, k_first, k_lo, k_end, g.req);
    cp_async_commit();

    int row_pos[2];
    bool row_ok[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        int tok, gh;
        row_ok[r] = g.row(warp * 16 + (lane >> 2) + 8 * r, tok, gh);
        row_pos[r] = g.pos0 + tok;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DT8][4];
#pragma unroll
    for (int i = 0; i < DT8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
    const bf16* Qw = Qs + warp * 16 * LDS;
    const float scale_log2 = a.scale * LOG2E;
    // the last key this warp's rows can see: blocks beyond it are skipped by this warp
    int warp_last_pos = -1, warp_first_pos = 0x7fffffff;
    bool warp_all_rows = true;
    {
        int tok, gh;
        for (int r = 15; r >= 0; --r) {
            if (g.row(warp * 16 + r, tok, gh)) {
                warp_last_pos = max(warp_last_pos, g.pos0 + tok);
                warp_first_pos = min(warp_first_pos, g.pos0 + tok);
            } else {
                warp_all_rows = false;
            }
        }
    }

    for (int b = 0; b < n_blocks; ++b) {
        const int stage = b & 1;
        if (b + 1 < n_blocks)
            load_kv_block(Ks + (stage ^ 1) * MMA_BN * LDS, Vs + (stage ^ 1) * MMA_BN * LDS, k_cache, v_cache, table_row, a, g.kvh,
                          k_first + (b + 1) * MMA_BN, k_lo, k_end, g.req);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (b == 0) {
            if constexpr (Q_IN_REGS) {
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk)
                    ldsm_x4(qf[kk], Qw + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));
            }
        }
        const int key0 = k_first + b * MMA_BN;
        if (key0 <= warp_last_pos) {
            // every row of the warp holds a (token, head), the block ends at or before the earliest row's position and
            // starts inside the latest row's window
            const bool full_block = warp_all_rows && key0 + MMA_BN - 1 <= warp_first_pos &&
                                    (a.window <= 0 || key0 > warp_last_pos - a.window);
            warp_block<MMA_BN>(qf, Qw, Ks + stage * MMA_BN * LDS, Vs + stage * MMA_BN * LDS, key0, row_pos, row_ok, a.window,
                               full_block, scale_log2, m, l, o);
        }
        __syncthreads();   // everyone is done with this stage before the next prefetch overwrites it
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        int tok, gh;
        if (!g.row(warp * 16 + (lane >> 2) + 8 * r, tok, gh)) continue;
        const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
        bf16* dst = out + ((size_t)(g.q_begin + tok) * a.H + (size_t)g.kvh * g.G + gh) * D + 2 * (lane & 3);
#pragma unroll
        for (int i = 0; i < DT8; ++i)
            *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
}

constexpr int DECODE_ROWS = 16;
constexpr int DECODE_STAGES = 3;
constexpr size_t DECODE_STAGE_SMEM = (size_t)(DECODE_ROWS + DECODE_STAGES * 2 * MMA_BN) * LDS * sizeof(bf16);
constexpr int MERGE_STRIDE = D + 4;             // floats per row of the warps' merge area: O, m, l, and 16-byte alignment
constexpr size_t DECODE_MERGE_SMEM = (size_t)4 * DECODE_ROWS * MERGE_STRIDE * sizeof(float);
constexpr size_t DECODE_SMEM = DECODE_STAGE_SMEM > DECODE_MERGE_SMEM ? DECODE_STAGE_SMEM : DECODE_MERGE_SMEM;

// The four warps of a block have each seen a quarter of the block's keys: their (O, m, l) per row stand in shared
// memory `mo` [warp][row][MERGE_STRIDE]. Merge them in the order of the warps; with one piece per unit that is the
// output, else it is this piece's partial result. Four d of one row per thread and pass.
// `mo` holds rows row0 .. row0 + nrows - 1 of the tile, `rows_stride` rows per warp.
__device__ __forceinline__ void merge_warps(const float* mo, int nrows, int splits, bf16* __restrict__ out, float* __restrict__ my_o,
                                            float* __restrict__ my_ml, const TileGeometry& g, const AttnArgs& a, int row0 = 0,
                                            int rows_stride = DECODE_ROWS) {
    constexpr int DV = D / 4, MS = MERGE_STRIDE;
    for (int idx = threadIdx.x; idx < nrows * DV; idx += MMA_THREADS) {
        const int r = row0 + idx / DV, d = (idx % DV) * 4;
        int tok, gh;
        if (!g.row(r, tok, gh)) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mo[((size_t)w * rows_stride + r - row0) * MS + D]);
        float L = 0.f;
        float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = mo + ((size_t)w * rows_stride + r - row0) * MS;
            const float f = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - M);
            const float4 v = *reinterpret_cast<const float4*>(src + d);
            L += src[D + 1] * f;
            O.x += v.x * f; O.y += v.y * f; O.z += v.z * f; O.w += v.w * f;
        }
        if (splits == 1) {
            const float inv = L > 0.f ? 1.f / L : 0.f;
            uint2 packed;
            packed.x = pack_bf16(O.x * inv, O.y * inv);
            packed.y = pack_bf16(O.z * inv, O.w * inv);
            *reinterpret_cast<uint2*>(out + ((size_t)(g.q_begin + tok) * a.H + (size_t)g.kvh * g.G + gh) * D + d) = packed;
        } else {
            *reinterpret_cast<float4*>(my_o + r * D + d) = O;
            if (d == 0) { my_ml[2 * r] = M; my_ml[2 * r + 1] = L; }
        }
    }
}

// The block that drew the last ticket of a unit merges the pieces' partial results (m, l, unnormalised O per row) in
// the order of the pieces and writes the output rows. Four d of one row per thread and pass; the loads of up to
// eight pieces are issued together and none depends on a value loaded before it, because what the merge costs is the
// latency of its loads from L2, not their number. An empty piece wrote (-inf, 0) and no O: its O is read (it is
// memory of the workspace) and dropped by a select, never multiplied.
__device__ __forceinline__ void merge_pieces(bf16* __restrict__ out, const float* __restrict__ all_ml, const float* __restrict__ all_o,
                                             int splits, int rows_live, const TileGeometry& g, const AttnArgs& a) {
    constexpr int CHUNK = 8, DV = D / 4;
    for (int idx = threadIdx.x; idx < rows_live * DV; idx += MMA_THREADS) {
        const int r = idx / DV, d = (idx % DV) * 4;
        int tok, gh;
        if (!g.row(r, tok, gh)) continue;
        float M = -INFINITY, L = 0.f;
        float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < splits; s0 += CHUNK) {
            float2 pml[CHUNK];
            float4 po[CHUNK];
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) {
                const int s2 = min(s0 + j, splits - 1);
                pml[j] = __ldcg(reinterpret_cast<const float2*>(all_ml + ((size_t)s2 * DECODE_ROWS + r) * 2));
                po[j] = __ldcg(reinterpret_cast<const float4*>(all_o + ((size_t)s2 * DECODE_ROWS + r) * D + d));
            }
            float m_new = M;
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) {
                if (s0 + j >= splits) pml[j].x = -INFINITY;   // a clamped repeat of the last piece
                m_new = fmaxf(m_new, pml[j].x);
            }
            const float keep = (M == -INFINITY) ? 0.f : exp2f(M - m_new);
            L *= keep;
            O.x *= keep; O.y *= keep; O.z *= keep; O.w *= keep;
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) {
                if (pml[j].x == -INFINITY) continue;          // compile-time unrolled: a select, no load depends on it
                const float f = exp2f(pml[j].x - m_new);
                L += pml[j].y * f;
                O.x += po[j].x * f; O.y += po[j].y * f; O.z += po[j].z * f; O.w += po[j].w * f;
            }
            M = m_new;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        uint2 packed;
        packed.x = pack_bf16(O.x * inv, O.y * inv);
        packed.y = pack_bf16(O.z * inv, O.w * inv);
        *reinterpret_cast<uint2*>(out + ((size_t)(g.q_begin + tok) * a.H + (size_t)g.kvh * g.G + gh) * D + d) = packed;
    }
}

// Split-KV attention for tiles of 16 rows. Grid (tiles, KV * head groups, splits). Each block handles one piece
// of the key range; its four warps each take a quarter of every 64-key block and are merged through shared
// memory. With one split the result goes straight to `out`. With several, each block writes its partial
//   part_o  [unit, split, 16, D] fp32 (unnormalised, relative to the partial maximum)
//   part_ml [unit, split, 16, 2] = (maximum in log2 units, sum)
// and takes a ticket from counters[unit]; the block that draws the last ticket merges all pieces and resets the
// counter to zero for the next launch. Nobody waits for anybody.
__global__ void __launch_bounds__(MMA_THREADS)
attn_mma_decode_kernel(bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                       int* __restrict__ counters, const bf16* __restrict__ q, const bf16* __restrict__ k_cache,
                       const bf16* __restrict__ v_cache, const AttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_ticket;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + DECODE_ROWS * LDS;                      // DECODE_STAGES stages
    bf16* Vs = Ks + DECODE_STAGES * MMA_BN * LDS;           // DECODE_STAGES stages
    const TileGeometry g = tile_geometry(a, DECODE_ROWS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int splits = gridDim.z, split = blockIdx.z;
    const size_t unit = (size_t)blockIdx.x * gridDim.y + blockIdx.y;
    float* my_ml = part_ml + (unit * splits + split) * DECODE_ROWS * 2;
    float* my_o = part_o + (unit * splits + split) * DECODE_ROWS * D;
    const int rows_live = g.tok0 < g.tok_end ? (g.tok_end - g.tok0) * g.heads_per_tile : 0;   // rows 0..rows_live-1 may hold a (token, head)

    int first = 0, count = 0, k_lo = 0, k_end = 0, k_first = 0;
    if (rows_live > 0) {
        k_end = g.pos0 + g.tok_end;
        k_lo = a.window > 0 ? max(0, g.pos0 + g.tok0 - a.window + 1) : 0;
        k_first = (k_lo / MMA_BN) * MMA_BN;
        const int n_blocks = (k_end - k_first + MMA_BN - 1) / MMA_BN;
        const int per = (n_blocks + splits - 1) / splits;
        first = split * per;
        count = max(0, min(per, n_blocks - first));
    }
    if (rows_live == 0) return;   // every split of this unit returns here: no tickets are drawn

    if (count > 0) {
        const int* table_row = a.block_table + (size_t)g.req * a.table_width;
        load_q_rows(Qs, q, a, g, DECODE_ROWS);
#pragma unroll
        for (int st = 0; st < DECODE_STAGES - 1; ++st) {
            if (st < count)
                load_kv_block(Ks + st * MMA_BN * LDS, Vs + st * MMA_BN * LDS, k_cache, v_cache, table_row, a, g.kvh,
                              k_first + (first + st) * MMA_BN, k_lo, k_end, g.req);
            cp_async_commit();
        }
        int row_pos[2];
        bool row_ok[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int tok, gh;
            row_ok[r] = g.row((lane >> 2) + 8 * r, tok, gh);
            row_pos[r] = g.pos0 + tok;
        }
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[DT8][4];
#pragma unroll
        for (int i = 0; i < DT8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
        const float scale_log2 = a.scale * LOG2E;
        const int tile_first_pos = g.pos0 + g.tok0, tile_last_pos = g.pos0 + g.tok_end - 1;

        for (int b = 0; b < count; ++b) {
            const int stage = b % DECODE_STAGES;
            // block b + STAGES - 1 goes into the stage that block b - 1 used; the barrier at the end of the previous
            // iteration made it free
            const int nb = b + DECODE_STAGES - 1;
            if (nb < count)
                load_kv_block(Ks + (nb % DECODE_STAGES) * MMA_BN * LDS, Vs + (nb % DECODE_STAGES) * MMA_BN * LDS, k_cache, v_cache,
                              table_row, a, g.kvh, k_first + (first + nb) * MMA_BN, k_lo, k_end, g.req);
            cp_async_commit();
            cp_async_wait<DECODE_STAGES - 1>();
            __syncthreads();
            if (b == 0) {
                if constexpr (Q_IN_REGS) {
#pragma unroll
                    for (int kk = 0; kk < KSTEPS; ++kk)
                        ldsm_x4(qf[kk], Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));
                }
            }
            const int key0 = k_first + (first + b) * MMA_BN + warp * 16;   // this warp's quarter of the block
            // rows without a (token, head) have zero queries: unmasked they give finite numbers that are never stored,
            // so the block counts as fully visible when the rows that do exist see all of it
            const bool full_block = key0 + 15 <= tile_first_pos && key0 >= k_lo && (a.window <= 0 || key0 > tile_last_pos - a.window);
            warp_block<16>(qf, Qs, Ks + (stage * MMA_BN + warp * 16) * LDS, Vs + (stage * MMA_BN + warp * 16) * LDS, key0, row_pos,
                           row_ok, a.window, full_block, scale_log2, m, l, o);
            __syncthreads();
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        }
        // ---- merge the four warps (the K/V stages are free now: the loop ended with a barrier)
        float* mo = reinterpret_cast<float*>(smem_raw);   // [4 warps][16 rows][D + 2]: O then (m, l)
        constexpr int MS = MERGE_STRIDE;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float* dst = mo + ((size_t)warp * DECODE_ROWS + (lane >> 2) + 8 * r) * MS;
#pragma unroll
            for (int i = 0; i < DT8; ++i) {
                dst[i * 8 + 2 * (lane & 3)] = o[i][2 * r];
                dst[i * 8 + 2 * (lane & 3) + 1] = o[i][2 * r + 1];
            }
            if ((lane & 3) == 0) { dst[D] = m[r]; dst[D + 1] = l[r]; }
        }
        __syncthreads();
        merge_warps(mo, rows_live, splits, out, my_o, my_ml, g, a);
    } else if (splits > 1) {   // nothing for this piece: an empty partial
        for (int i = threadIdx.x; i < rows_live; i += MMA_THREADS) { my_ml[2 * i] = -INFINITY; my_ml[2 * i + 1] = 0.f; }
    }
    if (splits == 1) return;

    // ---- ticket: the last piece to finish merges them all
    __threadfence();          // this block's partial is visible device-wide before its ticket is
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(&counters[unit], 1);
    __syncthreads();
    if (s_ticket != splits - 1) return;
    __threadfence();          // order the reads below after the tickets of the other pieces
    if (threadIdx.x == 0) counters[unit] = 0;   // ready for the next launch (nobody else touches it any more)
    const float* all_ml = part_ml + unit * splits * DECODE_ROWS * 2;
    const float* all_o = part_o + unit * splits * DECODE_ROWS * D;
    merge_pieces(out, all_ml, all_o, splits, rows_live, g, a);
}

// ---------------------------------------------------------------------------------------------------------------------
// The same split-KV kernel with the K/V blocks fetched by TMA instead of per-thread cp.async: a fifth warp is the
// producer; for every 64-key block each of its lanes issues one cp.async.bulk.tensor per (page piece, 64-wide panel
// of K or V), the hardware writes them 128-byte-swizzled, and an mbarrier per stage counts the bytes. The four
// consumer warps wait on that barrier, compute as before (ldmatrix with the swizzled addressing) and hand the stage
// back through a second mbarrier. Needs head sizes that are multiples of 64 and pages of 8 x 2^k tokens.
// The tensor maps cover a whole group's pool: rows = layers * pages * page_size, columns = KV * D.
// ---------------------------------------------------------------------------------------------------------------------
constexpr bool TMA_OK = (D % 64 == 0);
constexpr int PANELS = D / 64 > 0 ? D / 64 : 1;             // 64-wide panels of one head
constexpr int PANEL_BYTES = MMA_BN * 128;                    // 64 keys x 128 bytes
constexpr int KV_STAGE_BYTES = 2 * PANELS * PANEL_BYTES;     // K panels then V panels
constexpr int TMA_STAGES = 3;
constexpr int TMA_THREADS = 160;                             // 4 consumer warps + 1 producer warp
constexpr size_t TMA_DECODE_TILES = (size_t)TMA_STAGES * KV_STAGE_BYTES;
constexpr size_t NEW_KV_BYTES = 2 * (size_t)D * sizeof(bf16);   // the new token's k and v head (fused form), behind the barriers
constexpr size_t TMA_DECODE_SMEM = 1024 + (TMA_DECODE_TILES > DECODE_MERGE_SMEM ? TMA_DECODE_TILES : DECODE_MERGE_SMEM) +
                                   (size_t)DECODE_ROWS * LDS * sizeof(bf16) + 128 + NEW_KV_BYTES;

// ---------------------------------------------------------------------------------------------------------------------
// A decode step without the q/k norm + rotation + store kernel (qk_norm_rope.cu; oxr_runtime/kernels.py:66-99): when every
// request brings ONE token, the split-KV kernel with TMA gathers (a block per piece) can take the raw q|k|v projections itself. The
// consumer warps normalise and rotate the tile's q heads on their way into shared memory; the warp that owns the new
// token's key in the last key block does the same for the k head, copies the v head, writes both to the cache for the steps
// to come, and puts them over that row of the stage when the block has arrived (whatever the TMA copy found in the cache
// row of a token that nobody had stored yet). The arithmetic is that of the stand-alone kernel: fp32 from the bf16
// projections, one rounding.
// ---------------------------------------------------------------------------------------------------------------------
struct FuseQkv {
    const bf16* qkv;          // [requests, (H + 2 KV) * D]: null = q is given, the cache is complete
    bf16* k_cache;            // this layer's pool, written at the new token's row; null = the layer stores nothing and
    bf16* v_cache;            //   attends to what the cache holds (a layer that reads another layer's cache)
    const float* q_weight;    // [D] or null: no norm
    const float* k_weight;
    const float* cos_table;   // [max_positions, D / 2] or null: no rotation
    const float* sin_table;
    float eps;
    int max_positions;
};
constexpr int QK_STEPS = (D / 2 + 63) / 64;   // lane l holds elements 2 l, 2 l + 1 (+ 64 i) of a head's first half and their partners

struct HeadWords {
    float2 x1[QK_STEPS], x2[QK_STEPS];
};
__device__ __forceinline__ void load_head(HeadWords& w, const bf16* __restrict__ src, int lane) {
#pragma unroll
    for (int i = 0; i < QK_STEPS; ++i) {
        const int j = 2 * lane + 64 * i;
        w.x1[i] = w.x2[i] = make_float2(0.f, 0.f);
        if (j < D / 2) {
            w.x1[i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + j));
            w.x2[i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + j + D / 2));
        }
    }
}
// One warp, one head: RMSNorm over the head with `weight` (null: none), then the half-split rotation with the rows
// `cos_row`, `sin_row` of the tables (null: none). o1[i], o2[i]: the lane's elements as load_head holds them.
__device__ __forceinline__ void norm_rope_head(const HeadWords& w, const float* __restrict__ weight, const float* __restrict__ cos_row,
                                               const float* __restrict__ sin_row, float eps, int lane, __nv_bfloat162 (&o1)[QK_STEPS],
                                               __nv_bfloat162 (&o2)[QK_STEPS]) {
    constexpr int half = D / 2;
    float inv = 1.f;
    if (weight != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < QK_STEPS; ++i)
            ss += w.x1[i].x * w.x1[i].x + w.x1[i].y * w.x1[i].y + w.x2[i].x * w.x2[i].x + w.x2[i].y * w.x2[i].y;
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float)D + eps);
    }
#pragma unroll
    for (int i = 0; i < QK_STEPS; ++i) {
        const int j = 2 * lane + 64 * i;
        float2 y1 = w.x1[i], y2 = w.x2[i];
        if (j < half) {
            if (weight != nullptr) {
                const float2 w1 = *reinterpret_cast<const float2*>(weight + j), w2 = *reinterpret_cast<const float2*>(weight + j + half);
                y1.x = y1.x * inv * w1.x; y1.y = y1.y * inv * w1.y;
                y2.x = y2.x * inv * w2.x; y2.y = y2.y * inv * w2.y;
            }
            if (cos_row != nullptr) {
                const float2 c = *reinterpret_cast<const float2*>(cos_row + j), sn = *reinterpret_cast<const float2*>(sin_row + j);
                const float2 r1 = make_float2(y1.x * c.x - y2.x * sn.x, y1.y * c.y - y2.y * sn.y);
                const float2 r2 = make_float2(y1.x * sn.x + y2.x * c.x, y1.y * sn.y + y2.y * c.y);
                y1 = r1;
                y2 = r2;
            }
        }
        o1[i] = __float22bfloat162_rn(y1);
        o2[i] = __float22bfloat162_rn(y2);
    }
}
// The position of a request's one new token, checked against the rotary table.
__device__ __forceinline__ int checked_position(const FuseQkv& f, const AttnArgs& a, int pos, int req, int lane) {
    if (f.cos_table != nullptr && (pos < 0 || pos >= f.max_positions)) {
        if (lane == 0) oxr_report(a.status, OXR_BAD_POSITION, req);
        return 0;
    }
    return pos;
}
// The tile's q rows from the raw projections into shared memory, normalised and rotated (zeros for rows without a head):
// consumer warp w takes rows w, w + 4, ..., all their loads first.
__device__ __forceinline__ void fused_q_rows(bf16* Qs, const FuseQkv& f, const AttnArgs& a, const TileGeometry& g, int warp, int lane) {
    constexpr int RPW = DECODE_ROWS / 4;
    const int heads = a.H + 2 * a.KV;
    HeadWords w[RPW];
    bool ok[RPW];
    const int pos = checked_position(f, a, g.pos0 + g.tok0, g.req, lane);
    const bf16* token = f.qkv + (size_t)(g.q_begin + g.tok0) * heads * D;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        int tok, gh;
        ok[i] = g.row(warp + 4 * i, tok, gh) && tok == g.tok0;   // one token per request
        if (ok[i]) load_head(w[i], token + (size_t)(g.kvh * g.G + gh) * D, lane);
    }
    const float* cos_row = f.cos_table != nullptr ? f.cos_table + (size_t)pos * (D / 2) : nullptr;
    const float* sin_row = f.cos_table != nullptr ? f.sin_table + (size_t)pos * (D / 2) : nullptr;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        __nv_bfloat162 o1[QK_STEPS], o2[QK_STEPS];
        if (ok[i]) {
            norm_rope_head(w[i], f.q_weight, cos_row, sin_row, f.eps, lane, o1, o2);
        } else {
#pragma unroll
            for (int s = 0; s < QK_STEPS; ++s) o1[s] = o2[s] = __floats2bfloat162_rn(0.f, 0.f);
        }
        bf16* dst = Qs + (warp + 4 * i) * LDS;
#pragma unroll
        for (int s = 0; s < QK_STEPS; ++s) {
            const int j = 2 * lane + 64 * s;
            if (j < D / 2) {
                *reinterpret_cast<__nv_bfloat162*>(dst + j) = o1[s];
                *reinterpret_cast<__nv_bfloat162*>(dst + j + D / 2) = o2[s];
            }
        }
    }
}
// One warp: the new token's k head (normalised, rotated) and v head into `newkv` ([2][D] in shared memory) and into the
// cache row that the block table names for position `pos`.
__device__ __forceinline__ void fused_new_kv(bf16* newkv, const FuseQkv& f, const AttnArgs& a, const TileGeometry& g, int lane) {
    const int heads = a.H + 2 * a.KV;
    const int pos_raw = g.pos0 + g.tok0;
    const int pos = checked_position(f, a, pos_raw, g.req, lane);
    const bf16* token = f.qkv + (size_t)(g.q_begin + g.tok0) * heads * D;
    HeadWords w;
    load_head(w, token + (size_t)(a.H + g.kvh) * D, lane);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (lane < D / 8) v = *reinterpret_cast<const uint4*>(token + (size_t)(a.H + a.KV + g.kvh) * D + 8 * lane);
    const int page = a.block_table[(size_t)g.req * a.table_width + (a.page_shift >= 0 ? (pos_raw >> a.page_shift) : (pos_raw / a.page_size))];
    const bool page_ok = page >= 0 && page < a.num_pages;
    if (!page_ok && lane == 0) oxr_report(a.status, OXR_BAD_PAGE, g.req);
    const size_t row = (size_t)(page_ok ? page : 0) * a.page_size + (a.page_shift >= 0 ? (pos_raw & (a.page_size - 1)) : (pos_raw % a.page_size));
    __nv_bfloat162 o1[QK_STEPS], o2[QK_STEPS];
    norm_rope_head(w, f.k_weight, f.cos_table != nullptr ? f.cos_table + (size_t)pos * (D / 2) : nullptr,
                   f.cos_table != nullptr ? f.sin_table + (size_t)pos * (D / 2) : nullptr, f.eps, lane, o1, o2);
    bf16* k_row = f.k_cache + (row * a.KV + g.kvh) * D;
    bf16* v_row = f.v_cache + (row * a.KV + g.kvh) * D;
#pragma unroll
    for (int s = 0; s < QK_STEPS; ++s) {
        const int j = 2 * lane + 64 * s;
        if (j < D / 2) {
            *reinterpret_cast<__nv_bfloat162*>(newkv + j) = o1[s];
            *reinterpret_cast<__nv_bfloat162*>(newkv + j + D / 2) = o2[s];
            if (page_ok) {
                *reinterpret_cast<__nv_bfloat162*>(k_row + j) = o1[s];
                *reinterpret_cast<__nv_bfloat162*>(k_row + j + D / 2) = o2[s];
            }
        }
    }
    if (lane < D / 8) {
        *reinterpret_cast<uint4*>(newkv + D + 8 * lane) = v;
        if (page_ok) *reinterpret_cast<uint4*>(v_row + 8 * lane) = v;
    }
    __syncwarp();
}

// The same warp, once the key block with the new token's row has arrived: k and v over that row of the stage (16-byte
// words at their swizzled places). The fence orders these writes before the TMA copy that fills the stage next.
__device__ __forceinline__ void patch_new_kv(const bf16* Kst, const bf16* Vst, const bf16* newkv, int row, int lane) {
    if (lane < D / 8) {
        *reinterpret_cast<uint4*>(const_cast<bf16*>(kv_elem<true>(Kst, row, 8 * lane))) = *reinterpret_cast<const uint4*>(newkv + 8 * lane);
        *reinterpret_cast<uint4*>(const_cast<bf16*>(kv_elem<true>(Vst, row, 8 * lane))) = *reinterpret_cast<const uint4*>(newkv + D + 8 * lane);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
}

// First key of the page piece to fetch for the piece that starts at key `kp`: itself when any of its `box_rows` keys
// is visible (k_lo <= key < k_end), else the piece that holds the nearest visible key.
__device__ __forceinline__ int piece_to_fetch(int kp, int box_rows, int k_lo, int k_end) {
    if (kp >= k_end) return ((k_end - 1) / box_rows) * box_rows;
    if (kp + box_rows <= k_lo) return (k_lo / box_rows) * box_rows;
    return kp;
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <bool FUSED>
__global__ void __launch_bounds__(TMA_THREADS)
attn_tma_decode_kernel(bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                       const bf16* __restrict__ q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       int pool_row0, int box_rows, const AttnArgs a, const FuseQkv f) {
    extern __shared__ unsigned char smem_dyn[];
    __shared__ int s_ticket;
    __shared__ int s_gave_up;
    unsigned char* stages = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    constexpr size_t TILE_REGION = TMA_DECODE_TILES > DECODE_MERGE_SMEM ? TMA_DECODE_TILES : DECODE_MERGE_SMEM;
    bf16* Qs = reinterpret_cast<bf16*>(stages + TILE_REGION);
    uint64_t* full = reinterpret_cast<uint64_t*>(stages + TILE_REGION + (size_t)DECODE_ROWS * LDS * sizeof(bf16));
    uint64_t* empty = full + TMA_STAGES;
    [[maybe_unused]] bf16* newkv = reinterpret_cast<bf16*>(stages + TILE_REGION + (size_t)DECODE_ROWS * LDS * sizeof(bf16) + 128);

    [[maybe_unused]] unsigned long long tl_released = 0, tl_first = 0, tl_streamed = 0;   // timeline stamps of the consumer warps
    const TileGeometry g = tile_geometry(a, DECODE_ROWS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int splits = gridDim.z, split = blockIdx.z;
    const size_t unit = (size_t)blockIdx.x * gridDim.y + blockIdx.y;
    float* my_ml = part_ml + (unit * splits + split) * DECODE_ROWS * 2;
    float* my_o = part_o + (unit * splits + split) * DECODE_ROWS * D;
    const int rows_live = g.tok0 < g.tok_end ? (g.tok_end - g.tok0) * g.heads_per_tile : 0;
    if (rows_live == 0) return;   // every piece of this unit returns here: no tickets are drawn

    const int k_end = g.pos0 + g.tok_end;
    const int k_lo = a.window > 0 ? max(0, g.pos0 + g.tok0 - a.window + 1) : 0;
    const int k_first = (k_lo / MMA_BN) * MMA_BN;
    const int n_blocks = (k_end - k_first + MMA_BN - 1) / MMA_BN;
    const int per = (n_blocks + splits - 1) / splits;
    const int first = split * per;
    const int count = max(0, min(per, n_blocks - first));
    // fused form: the key block and the row in it of the request's new token, and whether this piece holds it
    [[maybe_unused]] const int new_blk = (g.pos0 + g.tok0 - k_first) / MMA_BN, new_row = (g.pos0 + g.tok0 - k_first) % MMA_BN;
    [[maybe_unused]] const bool has_new = FUSED && f.k_cache != nullptr && new_blk >= first && new_blk < first + count;

    if (count > 0) {
        if (threadIdx.x == 0) {
            for (int s2 = 0; s2 < TMA_STAGES; ++s2) { mbar_init(full + s2, 1); mbar_init(empty + s2, 4); }
            s_gave_up = 0;
            mbar_fence_init();
        }
        // Every page piece of a block is fetched, also one that lies wholly outside the visible range: its keys get a
        // probability of exactly zero, but what stands in the stage is multiplied by that zero and must be finite
        // numbers, which the pool's pages are and a fresh stage need not be. In place of such a piece (its page may
        // have been given back behind a window) the nearest visible piece is fetched once more.
        __syncthreads();

        if (warp == 4) {
            // ------------------------------------------------------------------ producer
            // The kernel before this one (when this one is launched dependent on it) writes q and the keys and values
            // of the NEW tokens; every older key is in the cache already. So the blocks of old keys are fetched at
            // once, while that kernel may still run, and the wait comes before the first block that reaches pos0.
            const int* table_row = a.block_table + (size_t)g.req * a.table_width;
            const int boxes = MMA_BN / box_rows;              // page pieces per block
            const int loads = boxes * 2 * PANELS;             // TMA instructions per block
            bool waited = false;
            for (int b = 0; b < count; ++b) {
                const int st = b % TMA_STAGES;
                const int k0 = k_first + (first + b) * MMA_BN;
                // where this lane's loads come from (at most two: a block has at most 8 pieces and 4 panels), looked up before
                // the wait for the stage so that the table's latency passes meanwhile
                int rows[2] = {-1, -1};
                int my_bytes = 0;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = lane + 32 * j;
                    if (i < loads) {
                        const int kp = piece_to_fetch(k0 + (i / (2 * PANELS)) * box_rows, box_rows, k_lo, k_end);
                        const int page = table_row[a.page_shift >= 0 ? (kp >> a.page_shift) : (kp / a.page_size)];
                        if (page >= 0 && page < a.num_pages) {
                            rows[j] = pool_row0 + page * a.page_size + (a.page_shift >= 0 ? (kp & (a.page_size - 1)) : (kp % a.page_size));
                            my_bytes += box_rows * 128;
                        } else oxr_report(a.status, OXR_BAD_PAGE, g.req);
                    }
                }
                if (!mbar_wait(empty + st, ((b / TMA_STAGES) & 1) ^ 1)) {
                    if (lane == 0) { atomicExch(&s_gave_up, 1); oxr_report(a.status, OXR_WAIT_EXPIRED, 10); }
                    break;
                }
                if (!FUSED && !waited && k0 + MMA_BN > g.pos0) {   // fused form: no kernel of the step wrote the cache before this one
                    pdl_wait();
                    waited = true;
                }
                unsigned char* dst = stages + (size_t)st * KV_STAGE_BYTES;
                const int total = __reduce_add_sync(0xffffffffu, my_bytes);
                if (lane == 0) {
                    if (total > 0) mbar_expect_tx(full + st, (uint32_t)total);
                    else mbar_arrive(full + st);
                }
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = lane + 32 * j;
                    if (rows[j] >= 0) {
                        const int box = i / (2 * PANELS), which = i % (2 * PANELS);     // which: K panels, then V panels
                        unsigned char* d2 = dst + (size_t)which * PANEL_BYTES + (size_t)box * box_rows * 128;
                        tma_load_2d(d2, which < PANELS ? &map_k : &map_v, g.kvh * D + (which % PANELS) * 64, rows[j], full + st);
                    }
                }
            }
            pdl_trigger();
            return;   // the producer takes no part in the merge
        }

        // ---------------------------------------------------------------------- consumers (warps 0..3)
        pdl_wait();   // q comes from the kernel before this one
        tl_released = OXR_TL_NOW();
        if constexpr (FUSED) {
            fused_q_rows(Qs, f, a, g, warp, lane);
            if (has_new && warp == new_row / 16) fused_new_kv(newkv, f, a, g, lane);
        } else {
            load_q_rows(Qs, q, a, g, DECODE_ROWS);   // strided over MMA_THREADS = the 128 consumer threads
        }
        cp_async_commit();
        int row_pos[2];
        bool row_ok[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int tok, gh;
            row_ok[r] = g.row((lane >> 2) + 8 * r, tok, gh);
            row_pos[r] = g.pos0 + tok;
        }
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[DT8][4];
#pragma unroll
        for (int i = 0; i < DT8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
        const float scale_log2 = a.scale * LOG2E;
        const int tile_first_pos = g.pos0 + g.tok0, tile_last_pos = g.pos0 + g.tok_end - 1;
        cp_async_wait<0>();
        consumer_sync();
        if constexpr (Q_IN_REGS) {
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk)
                ldsm_x4(qf[kk], Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));
        }
        for (int b = 0; b < count; ++b) {
            const int st = b % TMA_STAGES;
            if (!mbar_wait(full + st, (b / TMA_STAGES) & 1)) {
                if (lane == 0) { atomicExch(&s_gave_up, 1); oxr_report(a.status, OXR_WAIT_EXPIRED, 11); }
                break;
            }
            if (b == 0) tl_first = OXR_TL_NOW();
            const bf16* Kst = reinterpret_cast<const bf16*>(stages + (size_t)st * KV_STAGE_BYTES);
            const bf16* Vst = Kst + PANELS * (PANEL_BYTES / 2);
            if constexpr (FUSED) {
                if (has_new && first + b == new_blk && warp == new_row / 16) patch_new_kv(Kst, Vst, newkv, new_row, lane);
            }
            const int key0 = k_first + (first + b) * MMA_BN + warp * 16;
            const bool full_block = key0 + 15 <= tile_first_pos && key0 >= k_lo && (a.window <= 0 || key0 > tile_last_pos - a.window);
            warp_block<16, true>(qf, Qs, Kst + warp * 16 * 64, Vst + warp * 16 * 64, key0, row_pos, row_ok, a.window, full_block,
                                 scale_log2, m, l, o);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + st);   // this warp is done with the stage
        }
        tl_streamed = OXR_TL_NOW();
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        }
        pdl_trigger();     // the cache is read: the next kernel may set itself up during the merges
        consumer_sync();   // every consumer has left the loop: all fetched stages were read, the region is free
        float* mo = reinterpret_cast<float*>(stages);   // [4 warps][16 rows][D + 2]: O then (m, l)
        constexpr int MS = MERGE_STRIDE;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float* dst = mo + ((size_t)warp * DECODE_ROWS + (lane >> 2) + 8 * r) * MS;
#pragma unroll
            for (int i = 0; i < DT8; ++i) {
                dst[i * 8 + 2 * (lane & 3)] = o[i][2 * r];
                dst[i * 8 + 2 * (lane & 3) + 1] = o[i][2 * r + 1];
            }
            if ((lane & 3) == 0) { dst[D] = m[r]; dst[D + 1] = l[r]; }
        }
        consumer_sync();
        merge_warps(mo, rows_live, splits, out, my_o, my_ml, g, a);
    } else {
        pdl_wait();
        if (warp == 4) return;
        if (splits > 1)   // nothing for this piece: an empty partial
            for (int i = threadIdx.x; i < rows_live; i += MMA_THREADS) { my_ml[2 * i] = -INFINITY; my_ml[2 * i + 1] = 0.f; }
    }
    if (splits == 1) return;

    // ---- ticket (consumer warps only): the last piece to finish merges them all
    __threadfence();
    consumer_sync();
    if (threadIdx.x == 0) s_ticket = atomicAdd(&counters[unit], 1);
    consumer_sync();
    if (s_ticket != splits - 1) {
        if (threadIdx.x == 0) OXR_TL_PUT(4, tl_released, OXR_TL_NOW(), tl_first, tl_streamed, blockIdx.x);
        return;
    }
    __threadfence();
    if (threadIdx.x == 0) counters[unit] = 0;
    const float* all_ml = part_ml + unit * splits * DECODE_ROWS * 2;
    const float* all_o = part_o + unit * splits * DECODE_ROWS * D;
    merge_pieces(out, all_ml, all_o, splits, rows_live, g, a);
#ifdef OXR_TIMELINE
    consumer_sync();
    if (threadIdx.x == 0) OXR_TL_PUT(5, tl_released, OXR_TL_NOW(), tl_first, tl_streamed, blockIdx.x);   // id 5: the block that merged its unit
#endif
}

// ---------------------------------------------------------------------------------------------------------------------
// The split-KV kernel for more pieces than blocks fit on the GPU at once: the grid is one round of blocks, and block b
// walks over the pieces b, b + gridDim.x, ... (piece i = tile i / (Y S), KV-head group (i / S) % Y, split i % S). The
// producer warp does not stop between pieces: while the consumer warps merge their quarters of one piece, draw its
// ticket and perhaps merge a request's pieces, the ring already fills with the next piece's keys, so what a piece
// costs beside its streaming (the wait for its first block, the merges) is hidden after the first piece. Because of
// that the ring cannot lend its memory to the warps' merge, which has an area of its own and, to keep two blocks per
// SM, takes the tile's rows in rounds of four.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int WALK_ROWS = 4;                                         // rows per round of the warps' merge
constexpr int EVEN_MAX_UNITS = 16384;                                // most units for the even cut (32 of them then share a start)
constexpr int EVEN_STARTS = 512;                                     // starts kept in shared memory for the even cut (of every unit, or every n-th)
constexpr size_t WALK_MERGE_BYTES = (size_t)4 * WALK_ROWS * MERGE_STRIDE * sizeof(float);
constexpr size_t WALK_SMEM = 1024 + TMA_DECODE_TILES + WALK_MERGE_BYTES + (size_t)DECODE_ROWS * LDS * sizeof(bf16) + 128;

__device__ __forceinline__ bool consumer_any(bool v) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"((uint32_t)v) : "memory");
    return r != 0;
}

struct Piece {
    TileGeometry g;
    size_t unit;
    size_t slot;       // where this piece's partial goes; the partials of a unit are `parts` consecutive slots from slot - split on
    int split, parts, rows_live, k_end, k_lo, k_first, first, count;
};
// The unit's geometry and its key blocks; returns how many 64-key blocks it has (0 for a padding tile).
__device__ __forceinline__ int unit_of(const AttnArgs& a, int unit, int groups_y, Piece& p) {
    p.g = tile_geometry(a, DECODE_ROWS, unit / groups_y, unit % groups_y);
    p.unit = (size_t)unit;
    p.rows_live = p.g.tok0 < p.g.tok_end ? (p.g.tok_end - p.g.tok0) * p.g.heads_per_tile : 0;
    p.k_end = p.g.pos0 + p.g.tok_end;
    p.k_lo = a.window > 0 ? max(0, p.g.pos0 + p.g.tok0 - a.window + 1) : 0;
    p.k_first = (p.k_lo / MMA_BN) * MMA_BN;
    return p.rows_live > 0 ? (p.k_end - p.k_first + MMA_BN - 1) / MMA_BN : 0;
}
// Pieces by equal shares: every unit is cut into `splits` pieces of as many key blocks (the last may be shorter or empty).
__device__ __forceinline__ Piece piece_of(const AttnArgs& a, int item, int groups_y, int splits) {
    Piece p;
    p.split = item % splits;
    p.parts = splits;
    const int n_blocks = unit_of(a, item / splits, groups_y, p);
    p.slot = p.unit * splits + p.split;
    const int per = (n_blocks + splits - 1) / splits;
    p.first = p.split * per;
    p.count = p.rows_live > 0 ? max(0, min(per, n_blocks - p.first)) : 0;
    return p;
}
// Pieces by an even cut of ALL key blocks: the units' key blocks (with the slots of even_cost) laid end to end are dealt out to the `nb` blocks of the grid
// in runs of q or q + 1 (the first r blocks take q + 1); a block's run may cover the end of one unit and the beginning of
// the next, so requests of very different lengths still give every block the same share. The pieces of a unit are those of
// consecutive blocks; piece (u, block i) has slot u + i (each new unit and each new block moves the number on by one, so
// no two pieces share a slot). The units of one tile (its KV heads and head groups, `per_tile` of them, consecutive) have the
// same number of key blocks, so shared memory holds per TILE the key blocks of one unit of all tiles before it, and only of
// every `grp`-th tile, so that any number of tiles fits EVEN_STARTS entries (the tiles in between are counted again when a
// run is looked up).
// What is dealt out evenly are not the key blocks alone: a piece costs a block about as much as three key blocks beside its
// streaming (its Q, the warps' merge, perhaps a ticket and the merge of a request's pieces), and requests come longest first, so
// that a run of key blocks alone at the short end would be a hundred one-block pieces. Every unit therefore counts for its
// key blocks and EVEN_PIECE_COST slots before them that hold no work.
constexpr int EVEN_PIECE_COST = 3;
__device__ __forceinline__ int even_cost(int n_blocks) { return n_blocks > 0 ? n_blocks + EVEN_PIECE_COST : 0; }

struct EvenCut {
    const int* starts;   // [ceil(tiles / grp) + 1], in shared memory: starts[c] = key blocks of ONE unit each of the tiles before c * grp
    int tiles, per_tile, grp, q, r, nb;
    __device__ __forceinline__ int begin(int block) const { return block * q + min(block, r); }
    __device__ __forceinline__ int block_of(int x) const { const int big = r * (q + 1); return x < big ? x / (q + 1) : r + (x - big) / q; }
    // the unit that holds key block x of the step, and that unit's first key block
    __device__ __forceinline__ int unit_at(const AttnArgs& a, int x, int& start) const {
        int lo = 0, hi = (tiles - 1) / grp;
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (starts[mid] * per_tile <= x) lo = mid; else hi = mid - 1; }
        int t = lo * grp, n = 0;
        start = starts[lo] * per_tile;
        for (;; ++t) {
            Piece tmp;
            n = even_cost(unit_of(a, t * per_tile, per_tile, tmp));
            if (x < start + n * per_tile || t + 1 >= tiles) break;
            start += n * per_tile;
        }
        const int y = n > 0 ? min((x - start) / n, per_tile - 1) : 0;
        start += y * n;
        return t * per_tile + y;
    }
};
// The piece of `unit` (whose slots begin at number u0 of the step) that falls into `block`'s run; slots: how many the unit has.
__device__ __forceinline__ Piece piece_even(const AttnArgs& a, const EvenCut& f, int unit, int u0, int block, int groups_y, int& slots) {
    Piece p;
    const int n_blocks = unit_of(a, unit, groups_y, p);
    slots = even_cost(n_blocks);
    const int k0 = u0 + EVEN_PIECE_COST, k1 = k0 + n_blocks;      // the unit's key blocks among its slots
    const int lo = max(f.begin(block), k0), hi = min(f.begin(block + 1), k1);
    p.first = max(0, lo - k0);
    p.count = max(0, hi - lo);
    const int b0 = n_blocks > 0 ? f.block_of(k0) : block, b1 = n_blocks > 0 ? f.block_of(k1 - 1) : block;
    p.split = block - b0;
    p.parts = b1 - b0 + 1;
    p.slot = (size_t)unit + (size_t)block;
    return p;
}

__global__ void __launch_bounds__(TMA_THREADS, 2)   // two blocks an SM: the second bound keeps the registers within that
attn_tma_decode_walk_kernel(bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                            const bf16* __restrict__ q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            int pool_row0, int box_rows, int n_tiles, int groups_y, int splits, int cut, const AttnArgs a) {
    // cut 0: every unit in `splits` equal pieces, dealt out piece by piece. cut 1: the even cut of all key blocks (EvenCut),
    // which the host asks for when the requests' lengths differ much.
    extern __shared__ unsigned char smem_dyn[];
    __shared__ int s_ticket;
    __shared__ int s_gave_up;
    __shared__ int s_starts[EVEN_STARTS + 1];
    unsigned char* stages = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    float* mo = reinterpret_cast<float*>(stages + TMA_DECODE_TILES);        // [4 warps][WALK_ROWS][MERGE_STRIDE]
    bf16* Qs = reinterpret_cast<bf16*>(stages + TMA_DECODE_TILES + WALK_MERGE_BYTES);
    uint64_t* full = reinterpret_cast<uint64_t*>(stages + TMA_DECODE_TILES + WALK_MERGE_BYTES + (size_t)DECODE_ROWS * LDS * sizeof(bf16));
    uint64_t* empty = full + TMA_STAGES;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int items = n_tiles * groups_y * splits;
    const int units = n_tiles * groups_y;

    if (threadIdx.x == 0) {
        for (int s2 = 0; s2 < TMA_STAGES; ++s2) { mbar_init(full + s2, 1); mbar_init(empty + s2, 4); }
        s_gave_up = 0;
        mbar_fence_init();
    }
    __syncthreads();
    EvenCut even;
    even.starts = s_starts; even.tiles = n_tiles; even.per_tile = groups_y; even.q = even.r = 0; even.nb = 1;
    even.grp = (n_tiles + EVEN_STARTS - 1) / EVEN_STARTS;
    if (even.grp < 1) even.grp = 1;
    int u_first = 0, u_last = -1;      // even cut: the units this block's run touches
    int run_start = 0, run_n = 0;      // even cut: the first key block of the unit a walk stands at, and that unit's count
    const bool flat = cut != 0;
    if (flat) {
        // what no kernel of a step writes (lengths, tile lists) is read above the wait: every block counts every tile's key
        // blocks (a thread `grp` consecutive tiles at a time), warp 0 turns the counts into starts (each lane sixteen of them,
        // then a scan over the lanes)
        const int coarse = (n_tiles + even.grp - 1) / even.grp;
        for (int c = threadIdx.x; c < EVEN_STARTS; c += blockDim.x) {
            int sum = 0;
            if (c < coarse)
                for (int t = c * even.grp; t < min(n_tiles, (c + 1) * even.grp); ++t) {
                    Piece tmp;
                    sum += even_cost(unit_of(a, t * groups_y, groups_y, tmp));
                }
            s_starts[c + 1] = sum;
        }
        if (threadIdx.x == 0) s_starts[0] = 0;
        __syncthreads();
        if (warp == 0) {
            constexpr int PER = EVEN_STARTS / 32;
            int v[PER], sum = 0;
#pragma unroll
            for (int j = 0; j < PER; ++j) { v[j] = s_starts[1 + lane * PER + j]; sum += v[j]; }
            int before = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, before, o); if (lane >= o) before += t; }
            before -= sum;
#pragma unroll
            for (int j = 0; j < PER; ++j) { before += v[j]; s_starts[1 + lane * PER + j] = before; }
        }
        __syncthreads();
        const int total = s_starts[coarse] * groups_y;
        even.nb = min((int)gridDim.x, total);
        if (even.nb > 0) { even.q = total / even.nb; even.r = total % even.nb; }
        if ((int)blockIdx.x < even.nb) {
            int last_start;
            u_first = even.unit_at(a, even.begin(blockIdx.x), run_start);
            u_last = even.unit_at(a, even.begin(blockIdx.x + 1) - 1, last_start);
        }
    }
    // one walk for both forms: `it` is an item (equal shares) or a unit (even cut); in the even cut a walk carries the
    // start of the unit it stands at (run_start), moved on by the unit's count when the walk steps
    const int it_begin = flat ? u_first : (int)blockIdx.x, it_end = flat ? u_last + 1 : items, it_step = flat ? 1 : (int)gridDim.x;
    const int run_start0 = run_start;
    auto piece_at = [&](int it) { return flat ? piece_even(a, even, it, run_start, blockIdx.x, groups_y, run_n) : piece_of(a, it, groups_y, splits); };

    if (warp == 4) {
        // ---------------------------------------------------------------------- producer: piece after piece, one ring
        const int boxes = MMA_BN / box_rows;
        const int loads = boxes * 2 * PANELS;
        uint32_t n = 0;          // blocks requested so far: stage n % TMA_STAGES, use n / TMA_STAGES of that stage
        bool waited = false, ok = true;
        run_start = run_start0;
        for (int item = it_begin; item < it_end && ok; item += it_step, run_start += run_n) {
            const Piece p = piece_at(item);
            const int* table_row = a.block_table + (size_t)p.g.req * a.table_width;
            for (int b = 0; b < p.count; ++b, ++n) {
                const int st = n % TMA_STAGES;
                const int k0 = p.k_first + (p.first + b) * MMA_BN;
                // where this lane's loads come from (at most two), looked up before the wait for the stage
                int rows[2] = {-1, -1};
                int my_bytes = 0;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = lane + 32 * j;
                    if (i < loads) {
                        const int kp = piece_to_fetch(k0 + (i / (2 * PANELS)) * box_rows, box_rows, p.k_lo, p.k_end);
                        const int page = table_row[a.page_shift >= 0 ? (kp >> a.page_shift) : (kp / a.page_size)];
                        if (page >= 0 && page < a.num_pages) {
                            rows[j] = pool_row0 + page * a.page_size + (a.page_shift >= 0 ? (kp & (a.page_size - 1)) : (kp % a.page_size));
                            my_bytes += box_rows * 128;
                        } else oxr_report(a.status, OXR_BAD_PAGE, p.g.req);
                    }
                }
                if (!mbar_wait(empty + st, ((n / TMA_STAGES) & 1) ^ 1)) {
                    if (lane == 0) { atomicExch(&s_gave_up, 1); oxr_report(a.status, OXR_WAIT_EXPIRED, 20); }
                    ok = false;
                    break;
                }
                if (!waited && k0 + MMA_BN > p.g.pos0) {   // old keys are fetched while the kernel before this one may still run
                    pdl_wait();
                    waited = true;
                }
                unsigned char* dst = stages + (size_t)st * KV_STAGE_BYTES;
                const int total = __reduce_add_sync(0xffffffffu, my_bytes);
                if (lane == 0) {
                    if (total > 0) mbar_expect_tx(full + st, (uint32_t)total);
                    else mbar_arrive(full + st);
                }
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = lane + 32 * j;
                    if (rows[j] >= 0) {
                        const int box = i / (2 * PANELS), which = i % (2 * PANELS);
                        unsigned char* d2 = dst + (size_t)which * PANEL_BYTES + (size_t)box * box_rows * 128;
                        tma_load_2d(d2, which < PANELS ? &map_k : &map_v, p.g.kvh * D + (which % PANELS) * 64, rows[j], full + st);
                    }
                }
            }
        }
        pdl_trigger();
        return;
    }

    // -------------------------------------------------------------------------- consumers (warps 0..3)
    pdl_wait();   // q comes from the kernel before this one
    const float scale_log2 = a.scale * LOG2E;
    constexpr int MS = MERGE_STRIDE;
    uint32_t n = 0;
    run_start = run_start0;
    for (int item = it_begin; item < it_end; item += it_step, run_start += run_n) {
        // the barrier frees Qs, the merge area and s_ticket of the piece before; all warps leave together once a wait
        // has run out anywhere in the block
        if (consumer_any(*reinterpret_cast<volatile int*>(&s_gave_up) != 0)) return;
        const Piece p = piece_at(item);
        if (p.rows_live == 0) continue;   // every piece of this unit passes here: no tickets are drawn
        if (flat && p.count == 0) continue;   // the even cut gives a unit no empty pieces (and counts none)
        const TileGeometry& g = p.g;
        float* my_ml = part_ml + p.slot * DECODE_ROWS * 2;
        float* my_o = part_o + p.slot * DECODE_ROWS * D;
        if (p.count > 0) {
            load_q_rows(Qs, q, a, g, DECODE_ROWS);
            cp_async_commit();
            int row_pos[2];
            bool row_ok[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                int tok, gh;
                row_ok[r] = g.row((lane >> 2) + 8 * r, tok, gh);
                row_pos[r] = g.pos0 + tok;
            }
            float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
            float o[DT8][4];
#pragma unroll
            for (int i = 0; i < DT8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
            uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
            const int tile_first_pos = g.pos0 + g.tok0, tile_last_pos = g.pos0 + g.tok_end - 1;
            cp_async_wait<0>();
            consumer_sync();
            if constexpr (Q_IN_REGS) {
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk)
                    ldsm_x4(qf[kk], Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + kk * 16 + 8 * (lane >> 4));
            }
            for (int b = 0; b < p.count; ++b, ++n) {
                const int st = n % TMA_STAGES;
                if (!mbar_wait(full + st, (n / TMA_STAGES) & 1)) {
                    if (lane == 0) { atomicExch(&s_gave_up, 1); oxr_report(a.status, OXR_WAIT_EXPIRED, 21); }
                    break;
                }
                const bf16* Kst = reinterpret_cast<const bf16*>(stages + (size_t)st * KV_STAGE_BYTES);
                const bf16* Vst = Kst + PANELS * (PANEL_BYTES / 2);
                const int key0 = p.k_first + (p.first + b) * MMA_BN + warp * 16;
                const bool full_block = key0 + 15 <= tile_first_pos && key0 >= p.k_lo && (a.window <= 0 || key0 > tile_last_pos - a.window);
                warp_block<16, true>(qf, Qs, Kst + warp * 16 * 64, Vst + warp * 16 * 64, key0, row_pos, row_ok, a.window, full_block,
                                     scale_log2, m, l, o);
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + st);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
                l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
            }
            // the four warps' quarters meet in the merge area, WALK_ROWS rows of the tile per round
            for (int r0 = 0; r0 < p.rows_live; r0 += WALK_ROWS) {
                if (r0 > 0) consumer_sync();   // the round before is read
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int row = (lane >> 2) + 8 * r;
                    if (row >= r0 && row < r0 + WALK_ROWS) {
                        float* dst = mo + ((size_t)warp * WALK_ROWS + row - r0) * MS;
#pragma unroll
                        for (int i = 0; i < DT8; ++i) {
                            dst[i * 8 + 2 * (lane & 3)] = o[i][2 * r];
                            dst[i * 8 + 2 * (lane & 3) + 1] = o[i][2 * r + 1];
                        }
                        if ((lane & 3) == 0) { dst[D] = m[r]; dst[D + 1] = l[r]; }
                    }
                }
                consumer_sync();
                merge_warps(mo, min(WALK_ROWS, p.rows_live - r0), p.parts, out, my_o, my_ml, g, a, r0, WALK_ROWS);
            }
        } else if (p.parts > 1) {   // nothing for this piece: an empty partial
            for (int i = threadIdx.x; i < p.rows_live; i += MMA_THREADS) { my_ml[2 * i] = -INFINITY; my_ml[2 * i + 1] = 0.f; }
        }
        if (p.parts == 1) continue;
        // ---- ticket: the last piece of a unit to finish merges them all
        __threadfence();
        consumer_sync();
        if (threadIdx.x == 0) s_ticket = atomicAdd(&counters[p.unit], 1);
        consumer_sync();
        if (s_ticket == p.parts - 1) {
            __threadfence();
            if (threadIdx.x == 0) counters[p.unit] = 0;
            const size_t slot0 = p.slot - (size_t)p.split;
            merge_pieces(out, part_ml + slot0 * DECODE_ROWS * 2, part_o + slot0 * DECODE_ROWS * D, p.parts, p.rows_live, g, a);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Prefill attention on tcgen05: a tile is two halves of 128 rows (one TMEM lane per row); both halves use every 128-key
// block that arrives, so K and V are fetched once per 256 rows. Per block and half
//   S = Q K^T      tcgen05.mma 128 x 128 x 16, Q and K from shared memory (K-major, 128-byte swizzle), S (128 x 128 fp32) in TMEM;
//   softmax        four warps, ONE THREAD PER ROW: tcgen05.ld of its 128 scores (read once, kept in registers), the maximum,
//                  then P = exp2(S - m), which goes back INTO TENSOR MEMORY as bf16 pairs over the columns S came from
//                  (keys 2 j, 2 j + 1 in column j);
//   O += P V       tcgen05.mma with P as the A operand FROM TENSOR MEMORY and V from the TMA stage as an MN-major operand,
//                  O (128 x D fp32) in TMEM.
// The tensor pipe runs one thread's products in the order they were issued, so nothing but that order keeps S(b + 1) of a
// half off the columns that P(b) V(b) still reads: the issuing thread alternates PV0(b), S0(b + 1), PV1(b), S1(b + 1), and
// while one half's softmax runs the pipe works for the other half.
// Why 128 keys: measured with stamps inside the kernel, the form with 64-key blocks (S 128 x 64 x 16, P through shared
// memory) was bound by the tensor pipe at a third of its rate: a 128 x 64 x 16 product took about 120 cycles, hardly less
// than a 128 x 128 x 16 one, and reading P from shared memory cost the PV products another 4 KB each.
// The running maximum is only raised when a row's maximum grows by more than 8 (in log2 units): P then stays below
// 2^8, which bf16 and the fp32 accumulator take without loss, and the rescale of O (tcgen05.ld, multiply, tcgen05.st)
// becomes rare. K and V blocks arrive by TMA from a producer warp, Q as one 3-D box per half and panel.
// Warp roles: 0 = TMA producer, 1 = MMA issuer and owner of the TMEM allocation, 2..5 / 6..9 = softmax and epilogue of
// the first / second half.
// Every mbarrier wait is bounded.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int HALF_ROWS = 128;                                      // rows of one accumulator (TMEM lanes)
constexpr int BIG_ROWS = 2 * HALF_ROWS;                             // a tile is two such halves sharing every K/V block
constexpr int TC_BN = 128;                                          // keys per block
constexpr int TC_STAGES = 2;
constexpr int TC_THREADS = 320;                                     // warp 0 TMA, warp 1 MMA, warps 2..9 softmax (4 per half)
constexpr int Q_PANEL_BYTES = HALF_ROWS * 128;                      // 128 rows x 64 d
constexpr int TC_PANEL_BYTES = TC_BN * 128;                         // 128 keys x 64 d
constexpr int TC_HALF_STAGE = PANELS * TC_PANEL_BYTES;              // the K (or the V) panels of a block
constexpr size_t TC_SMEM = 2 * (size_t)PANELS * Q_PANEL_BYTES + 2 * (size_t)TC_STAGES * TC_HALF_STAGE + 512;
constexpr uint32_t TC_TMEM_COLS = 512;                              // S | P of half h at 128 h, O of half h at 256 + h * D
constexpr float RESCALE_THRESHOLD = 8.f;

// K-major operand tile with 128-byte rows, 128-byte swizzle (Q, K): see gemm_tcgen05.cu
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (V: rows are keys = K, 64 d contiguous per 128-byte row, panels of 64 d TC_PANEL_BYTES apart): 8 keys
// per swizzle atom, the next 8 keys 1024 bytes on (stride byte offset), the next 64 d one panel on (leading byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(TC_PANEL_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor: fp32 accumulator, bf16 operands, A K-major, B K-major or MN-major
__host__ __device__ constexpr uint32_t attn_idesc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// The same with the A operand in tensor memory (128 lanes x 8 columns of bf16 pairs per 16 k).
__device__ __forceinline__ void tc_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {   // the caller issues tcgen05.wait::ld before it uses r
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ bool elect_one_lane() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
// Two fp32 numbers in one 64-bit register pair, for the packed fp32 instructions of sm_100 (one issue slot for two results).
__device__ __forceinline__ uint64_t pair_of(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpair(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
attn_tc5_prefill_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_q, int q_by_tma,
                        int pool_row0, int box_rows, int n_tiles, int n_y, const AttnArgs a) {
    // The kernel has no static shared memory, so the dynamic part starts at the block's shared-memory origin, which
    // is 1024-byte aligned as the swizzled tiles need (checked below).
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char* base = smem_dyn;
    unsigned char* Qs = base;                                              // [half][PANELS] panels of [128 rows][128 B], swizzled
    unsigned char* k_ring = Qs + 2 * (size_t)PANELS * Q_PANEL_BYTES;       // TC_STAGES x K panels of [128 keys][128 B]
    unsigned char* v_ring = k_ring + (size_t)TC_STAGES * TC_HALF_STAGE;     // TC_STAGES x V panels
    uint64_t* k_full = reinterpret_cast<uint64_t*>(v_ring + (size_t)TC_STAGES * TC_HALF_STAGE);
    uint64_t* k_empty = k_full + TC_STAGES;      // K(b) is free once S(b) of both halves has completed: long before V(b) is
    uint64_t* v_full = k_empty + TC_STAGES;
    uint64_t* v_empty = v_full + TC_STAGES;
    uint64_t* s_full = v_empty + TC_STAGES;      // [half] S(b) is in TMEM
    uint64_t* p_full = s_full + 2;               // [half] P(b) is in TMEM and O is rescaled (4 arrivals)
    uint64_t* o_done = p_full + 2;               // [half] O += P(b) V(b) has completed
    uint64_t* q_ready = o_done + 2;              // Q is in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
#ifdef OXR_TIMELINE
    unsigned long long* tl = reinterpret_cast<unsigned long long*>(q_ready + 2);   // eight stamps in the spare bytes behind the barriers
    unsigned long long* tl2 = tl + 8;
    constexpr int TLB = 10;
#endif

    // the list is in token order and later tiles of a prompt see more keys: start the long ones first,
    [[maybe_unused]] const unsigned long long tl_started = OXR_TL_NOW();
    if (threadIdx.x == 0) {   // the tensor maps are on their way before anything else
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
        if (q_by_tma) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    }
    // and all (KV head, head group) pairs of a tile side by side, so that no pair's long tiles wait behind another pair's short ones
    const TileGeometry g = tile_geometry(a, BIG_ROWS, n_tiles - 1 - (int)(blockIdx.x / (unsigned)n_y), (int)(blockIdx.x % (unsigned)n_y));
    if (g.tok0 >= g.tok_end) return;
    if (smem_addr(base) & 1023u) {   // cannot happen without static shared memory; refuse rather than compute rubbish
        if (threadIdx.x == 0) oxr_report(a.status, OXR_BAD_ARGUMENT, 1024);
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int k_end = g.pos0 + g.tok_end;
    const int k_lo = a.window > 0 ? max(0, g.pos0 + g.tok0 - a.window + 1) : 0;
    const int k_first = (k_lo / TC_BN) * TC_BN;
    const int count = (k_end - k_first + TC_BN - 1) / TC_BN;
    // A lane of the producer warp fetches one page piece of a block's K and of its V (a block has at most 16 pieces of 8 keys
    // and 2 panels): the pool row of this lane's piece of block b, or -1 if it is not fetched. The first block's pages are
    // looked up here, before the set-up, and every later block's while the block before it waits for its place in the rings.
    const int* table_row = a.block_table + (size_t)g.req * a.table_width;
    const int pieces = (TC_BN / box_rows) * PANELS;
    const int my_box = lane / PANELS, my_pnl = lane % PANELS;
    auto lookup = [&](int b) -> int {
        const int kp = k_first + b * TC_BN + my_box * box_rows;
        if (lane < pieces && kp < k_end && kp + box_rows > k_lo) {
            const int page = table_row[a.page_shift >= 0 ? (kp >> a.page_shift) : (kp / a.page_size)];
            if (page >= 0 && page < a.num_pages)
                return pool_row0 + page * a.page_size + (a.page_shift >= 0 ? (kp & (a.page_size - 1)) : (kp % a.page_size));
            oxr_report(a.status, OXR_BAD_PAGE, g.req);
        }
        return -1;
    };
    const int row_first = warp == 0 ? lookup(0) : -1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TC_STAGES; ++i) { mbar_init(k_full + i, 1); mbar_init(k_empty + i, 1); mbar_init(v_full + i, 1); mbar_init(v_empty + i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(s_full + i, 1); mbar_init(p_full + i, 4); mbar_init(o_done + i, 1); }
        mbar_init(q_ready, q_by_tma ? 1 : TC_THREADS / 32 - 2);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Nothing else stands before the first loads: the producer warp goes ahead while Q comes in (the MMA warp waits for
    // `q_ready` before its first product).
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
#ifdef OXR_TIMELINE
    if (threadIdx.x == 0) tl[0] = OXR_TL_NOW();
#endif
    // Q without a tensor map (a number of heads per KV head that does not divide 128): every softmax thread copies its own row
    // (D bf16) into the swizzled panels; rows without a (token, head) are zero.
    if (warp >= 2 && !q_by_tma) {
        const int half = (warp - 2) >> 2, rr = (warp & 3) * 32 + lane;   // row inside the half = its TMEM lane
        int tok, gh;
        const bool ok = g.row(half * HALF_ROWS + rr, tok, gh);
        const uint4* src = reinterpret_cast<const uint4*>(q + ((size_t)(g.q_begin + (ok ? tok : 0)) * a.H + (size_t)g.kvh * g.G + (ok ? gh : 0)) * D);
        unsigned char* qh = Qs + (size_t)half * PANELS * Q_PANEL_BYTES;
        uint4 v[D / 8];
#pragma unroll
        for (int c = 0; c < D / 8; ++c) v[c] = ok ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int c = 0; c < D / 8; ++c)
            *reinterpret_cast<uint4*>(qh + (size_t)(c >> 3) * Q_PANEL_BYTES + (size_t)rr * 128 + (((c & 7) ^ (rr & 7)) << 4)) = v[c];
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_ready);
    }
    // TMEM columns: S (fp32) and then P (bf16 pairs) of half h at 128 h; O of half h at 256 + h * D
    // the second half of a tile may be empty (short portions): its products and softmax are then skipped
    const bool half1_live = g.tok0 + (HALF_ROWS / g.heads_per_tile) < g.tok_end || g.heads_per_tile > HALF_ROWS;

    if (warp == 0) {
        // ---------------------------------------------------------------------- TMA producer (all 32 lanes issue)
        if (q_by_tma && lane == 0) {
            // Q: one box per half and 64-wide panel, rows in the order (token, head) as the tile counts them. Rows behind the
            // request's last token are somebody else's (or zero behind the tensor): finite, and masked like the padding rows.
            const int halves = half1_live ? 2 : 1;
            mbar_expect_tx(q_ready, (uint32_t)(halves * PANELS * Q_PANEL_BYTES));
            for (int h = 0; h < halves; ++h)
                for (int pnl = 0; pnl < PANELS; ++pnl)
                    tma_load_3d(Qs + (size_t)(h * PANELS + pnl) * Q_PANEL_BYTES, &map_q, pnl * 64, g.kvh * g.G,
                                g.q_begin + g.tok0 + h * (HALF_ROWS / g.G), q_ready);
        }
        // K(0), V(0), K(1), V(1), ...: each into its own ring
        int row = row_first;
        for (int b = 0; b < count; ++b) {
            const int row_next = b + 1 < count ? lookup(b + 1) : -1;
            const int st = b % TC_STAGES;
            const int total = __reduce_add_sync(0xffffffffu, row >= 0 ? box_rows * 128 : 0);
            bool ok = true;
            for (int is_v = 0; is_v < 2; ++is_v) {
                uint64_t* full = (is_v ? v_full : k_full) + st;
                if (!mbar_wait((is_v ? v_empty : k_empty) + st, ((b / TC_STAGES) & 1) ^ 1)) { if (lane == 0) oxr_report(a.status, OXR_WAIT_EXPIRED, 30); ok = false; break; }
                unsigned char* dst = (is_v ? v_ring : k_ring) + (size_t)st * TC_HALF_STAGE;
#ifdef OXR_TIMELINE
                if (b == 0 && is_v == 0 && lane == 0) tl[5] = OXR_TL_NOW();
#endif
                if (total < pieces * box_rows * 128) {
                    // Page pieces that are not fetched (beyond the last key, before the window, a bad page) meet a probability of
                    // exactly zero, but must hold finite numbers: zero them (the ring may hold anything from an earlier kernel).
                    if (lane < pieces && row < 0) {
                        uint4* z = reinterpret_cast<uint4*>(dst + (size_t)my_pnl * TC_PANEL_BYTES + (size_t)my_box * box_rows * 128);
                        for (int j = 0; j < box_rows * 8; ++j) z[j] = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();
                    __syncwarp();
                }
                if (lane == 0) {
                    if (total > 0) mbar_expect_tx(full, (uint32_t)total);
                    else mbar_arrive(full);
                }
                __syncwarp();
                if (row >= 0)
                    tma_load_2d(dst + (size_t)my_pnl * TC_PANEL_BYTES + (size_t)my_box * box_rows * 128, is_v ? &map_v : &map_k,
                                g.kvh * D + my_pnl * 64, row, full);
#ifdef OXR_TIMELINE
                if (b == 0 && is_v == 0 && lane == 0) tl[1] = OXR_TL_NOW();
#endif
            }
            if (!ok) break;
            row = row_next;
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------------- MMA issuer
        if (elect_one_lane()) {
            constexpr uint32_t idesc_s = attn_idesc(HALF_ROWS, TC_BN, false);
            constexpr uint32_t idesc_o = attn_idesc(HALF_ROWS, D, true);
            const uint32_t q_addr = smem_addr(Qs);
            const int halves = half1_live ? 2 : 1;
            bool ok = true;
            auto issue_s = [&](int b, int h) {      // S_h(b) = Q_h K(b)^T into the half's 128 columns
                const uint32_t k_addr = smem_addr(k_ring + (size_t)(b % TC_STAGES) * TC_HALF_STAGE);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    tc_mma(tmem_base + (uint32_t)(h * TC_BN), desc_kmajor(q_addr + (h * PANELS + (kk >> 2)) * Q_PANEL_BYTES + (kk & 3) * 32),
                           desc_kmajor(k_addr + (kk >> 2) * TC_PANEL_BYTES + (kk & 3) * 32), idesc_s, kk > 0 ? 1u : 0u);
                tc_commit(s_full + h);
                if (h == halves - 1) tc_commit(k_empty + b % TC_STAGES);   // every product that reads K(b) has been issued
            };
            auto wait_for = [&](uint64_t* full, int b, int where) -> bool {
                if (!mbar_wait(full + b % TC_STAGES, (b / TC_STAGES) & 1)) { oxr_report(a.status, OXR_WAIT_EXPIRED, where); return false; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                return true;
            };
            if (!mbar_wait(q_ready, 0)) { oxr_report(a.status, OXR_WAIT_EXPIRED, 36); ok = false; }
            ok = ok && wait_for(k_full, 0, 31);
#ifdef OXR_TIMELINE
            tl[2] = OXR_TL_NOW();
#endif
            if (ok)
                for (int h = 0; h < halves; ++h) issue_s(0, h);
            // then, block by block and half by half: O_h += P_h(b) V(b), and at once S_h(b + 1) over the same columns
            for (int b = 0; b < count && ok; ++b) {
                const uint32_t v_addr = smem_addr(v_ring + (size_t)(b % TC_STAGES) * TC_HALF_STAGE);
#ifdef OXR_TIMELINE
                if (b == TLB) tl2[0] = OXR_TL_NOW();
#endif
                for (int h = 0; h < halves && ok; ++h) {
                    if (!mbar_wait(p_full + h, b & 1)) { oxr_report(a.status, OXR_WAIT_EXPIRED, 33); ok = false; break; }
#ifdef OXR_TIMELINE
                    if (b == TLB) tl2[2 + 3 * h] = OXR_TL_NOW();
#endif
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (h == 0 && !wait_for(v_full, b, 32)) { ok = false; break; }
#pragma unroll
                    for (int kk = 0; kk < TC_BN / 16; ++kk)
                        tc_mma_a_tmem(tmem_base + 256 + (uint32_t)(h * D), tmem_base + (uint32_t)(h * TC_BN + kk * 8),
                                      desc_mnmajor(v_addr + kk * 16 * 128), idesc_o, (b > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(o_done + h);
                    if (h == halves - 1) tc_commit(v_empty + b % TC_STAGES);   // every product that reads V(b) has been issued
#ifdef OXR_TIMELINE
                    if (b == TLB) tl2[3 + 3 * h] = OXR_TL_NOW();
#endif
                    if (b + 1 < count) {
                        if (h == 0 && !wait_for(k_full, b + 1, 31)) { ok = false; break; }
#ifdef OXR_TIMELINE
                        if (b == TLB && h == 0) tl2[1] = OXR_TL_NOW();
#endif
                        issue_s(b + 1, h);
                    }
#ifdef OXR_TIMELINE
                    if (b == TLB) tl2[4 + 3 * h] = OXR_TL_NOW();
#endif
                }
            }
        }
    } else if (warp - 2 < 4 || half1_live) {
        // ---------------------------------------------------------------------- softmax and epilogue: one thread per row
        const int half = (warp - 2) >> 2;
        const int quarter = warp & 3;                        // TMEM lanes 32 * quarter .. + 31 belong to this warp
        const int rr = quarter * 32 + lane;                  // row inside the half
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t tmem_s = tmem_base + lane_base + (uint32_t)(half * TC_BN);
        const uint32_t tmem_o = tmem_base + 256 + (uint32_t)(half * D);
        int tok, gh;
        const bool row_ok = g.row(half * HALF_ROWS + rr, tok, gh);
        const int row_pos = g.pos0 + tok;
        const float scale_log2 = a.scale * LOG2E;
        float m_used = -INFINITY, l = 0.f;                   // the maximum P is taken against, the running sum
        bool alive = true;
        for (int b = 0; b < count; ++b) {
            const int key0 = k_first + b * TC_BN;
            if (!mbar_wait(s_full + half, b & 1)) { if (lane == 0) oxr_report(a.status, OXR_WAIT_EXPIRED, 34); alive = false; break; }
#ifdef OXR_TIMELINE
            if (b == 0 && warp == 2 && lane == 0) tl[3] = OXR_TL_NOW();
            const bool tl_me = b == TLB && lane == 0 && quarter == 0;
            if (tl_me) tl2[8 + 4 * half] = OXR_TL_NOW();
#endif
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the row's 128 scores, read once
            uint32_t sv[TC_BN / 32][32];
#pragma unroll
            for (int c = 0; c < TC_BN / 32; ++c) tc_ld32_nowait(tmem_s + (uint32_t)(c * 32), sv[c]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#ifdef OXR_TIMELINE
            if (tl_me) tl2[9 + 4 * half] = OXR_TL_NOW();
#endif
            // Blocks that this row sees in full need no per-key test; on the others the hidden keys become -inf.
            const bool whole = row_ok && key0 + TC_BN - 1 <= row_pos && key0 >= k_lo && (a.window <= 0 || key0 > row_pos - a.window);
            if (!whole) {
                // the keys of this block that the row sees are those with index lo .. lo + span: one subtraction and one
                // unsigned comparison per key
                int lo = max(k_lo, a.window > 0 ? row_pos - a.window + 1 : 0) - key0;
                int span = row_pos - key0 - lo;
                if (!row_ok || span < 0) { lo = 1 << 30; span = 0; }
#pragma unroll
                for (int c = 0; c < TC_BN / 32; ++c)
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if ((unsigned)(c * 32 + j - lo) > (unsigned)span) sv[c][j] = __float_as_uint(-INFINITY);
            }
            // the row's maximum of the raw scores (four independent chains); the (positive) scale is applied once
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < TC_BN / 32; ++c)
#pragma unroll
                for (int j = 0; j < 16; ++j) mx4[j & 3] = max3(mx4[j & 3], __uint_as_float(sv[c][2 * j]), __uint_as_float(sv[c][2 * j + 1]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            // raise the maximum only when it grew by more than the threshold (or there was none yet)
            float alpha = 1.f;
            bool raise = mx > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && mx != -INFINITY);
            if (raise) {
                alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - mx);
                m_used = mx;
            }
            // S(b) complete means that O += P(b - 1) V(b - 1), issued before it, is complete: O may be rescaled
            if (__any_sync(0xffffffffu, raise && b > 0)) {
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t ov[32];
                    tc_ld32(tmem_o + lane_base + (uint32_t)(c * 32), ov);
#pragma unroll
                    for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
                    tc_st32(tmem_o + lane_base + (uint32_t)(c * 32), ov);
                }
            }
#ifdef OXR_TIMELINE
            if (tl_me) tl2[10 + 4 * half] = OXR_TL_NOW();
#endif
            // P = exp2(score * scale - m), one FMA and one ex2 per key, written back as bf16 pairs over the columns S came from:
            // keys 2 j and 2 j + 1 in column j
            const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;    // a row that has seen no key yet has only -inf scores
            // (the scale, the shift and the sums go two keys at a time through the packed fp32 instructions)
            const uint64_t scale2 = pair_of(scale_log2, scale_log2), neg_m2 = pair_of(neg_m, neg_m);
            uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
            for (int c = 0; c < TC_BN / 32; ++c) {
                uint32_t pv[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    float x0, x1;
                    unpair(fma2(pair_of(__uint_as_float(sv[c][2 * e]), __uint_as_float(sv[c][2 * e + 1])), scale2, neg_m2), x0, x1);
                    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                    sum2[e & 3] = add2(sum2[e & 3], pair_of(p0, p1));
                    const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                    pv[e] = *reinterpret_cast<const uint32_t*>(&pk);
                }
                tc_st16(tmem_s + (uint32_t)(c * 16), pv);
            }
            float sum4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { float lo, hi; unpair(sum2[i], lo, hi); sum4[i] = lo + hi; }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + half);
#ifdef OXR_TIMELINE
            if (tl_me) tl2[11 + 4 * half] = OXR_TL_NOW();
#endif
        }
        // ---- epilogue: O / l -> out
        if (alive && count > 0) {
            const int last = count - 1;
            if (!mbar_wait(o_done + half, last & 1)) { if (lane == 0) oxr_report(a.status, OXR_WAIT_EXPIRED, 37); alive = false; }
        }
        alive = __all_sync(0xffffffffu, alive);
#ifdef OXR_TIMELINE
        if (warp == 2 && lane == 0) tl[4] = OXR_TL_NOW();
        if (warp == 6 && lane == 0) tl[6] = OXR_TL_NOW();
#endif
        if (alive) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.f / l : 0.f;
            // The row goes, as bf16, into the place of this half's Q (every product that read Q has completed), 16-byte pieces
            // swizzled by the row; then the warp writes its 32 rows out two at a time, 256 contiguous bytes each.
            unsigned char* oh = Qs + (size_t)half * PANELS * Q_PANEL_BYTES;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t ov[32];
                tc_ld32(tmem_o + lane_base + (uint32_t)(c * 32), ov);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint4 o4;
                    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        op[e] = __floats2bfloat162_rn(__uint_as_float(ov[8 * j + 2 * e]) * inv, __uint_as_float(ov[8 * j + 2 * e + 1]) * inv);
                    *reinterpret_cast<uint4*>(oh + (size_t)rr * (D * 2) + (((c * 4 + j) ^ (rr & (D / 8 - 1))) << 4)) = o4;
                }
            }
            __syncwarp();
            constexpr int LPR = D / 8;                 // lanes per row
            constexpr int RPI = 32 / LPR;              // rows per instruction
            // where this thread's row goes (null: nowhere); the copying lanes ask the row's owner
            const unsigned long long my_dst = row_ok ? (unsigned long long)(out + ((size_t)(g.q_begin + tok) * a.H + (size_t)g.kvh * g.G + gh) * D) : 0ull;
#pragma unroll 4
            for (int it = 0; it < 32 / RPI; ++it) {
                const int owner = it * RPI + lane / LPR, c2 = lane % LPR;
                const int r2 = quarter * 32 + owner;
                const unsigned long long dst2 = __shfl_sync(0xffffffffu, my_dst, owner);
                if (dst2 != 0ull)
                    reinterpret_cast<uint4*>(dst2)[c2] = *reinterpret_cast<const uint4*>(oh + (size_t)r2 * (D * 2) + ((c2 ^ (r2 & (LPR - 1))) << 4));
            }
        }
#ifdef OXR_TIMELINE
        if (warp == 2 && lane == 0) tl[7] = OXR_TL_NOW();
#endif
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
#ifdef OXR_TIMELINE
    if (threadIdx.x == 0) {   // ids 6 to 8: a prefill tile (started, ended, set up, first S in tensor memory, epilogue begins; first loads issued, first keys landed, ...)
        OXR_TL_PUT(6ull | ((unsigned long long)count << 8), tl_started, OXR_TL_NOW(), tl[0], tl[3], tl[4]);
        OXR_TL_PUT(7ull | ((unsigned long long)count << 8), tl_started, tl[1], tl[2], tl[5], tl[6]);
        OXR_TL_PUT(8ull | ((unsigned long long)count << 8), tl_started, tl[7], 0, 0, 0);
        if (count > TLB + 2) {   // ids 9 to 12: inside block TLB: the MMA warp's loop, the first softmax warp of each half
            OXR_TL_PUT(9ull, tl2[0], tl2[1], tl2[2], tl2[3], tl2[4]);
            OXR_TL_PUT(10ull, tl2[0], tl2[5], tl2[6], tl2[7], tl2[8]);
            OXR_TL_PUT(11ull, tl2[0], tl2[9], tl2[10], tl2[11], tl2[12]);
            OXR_TL_PUT(12ull, tl2[0], tl2[13], tl2[14], tl2[15], 0);
        }
    }
#endif
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}
}  // namespace

// Blocks of the walking split-KV kernel that the GPU holds at once (0 if it cannot run here).
static int walk_slots() {
    static int slots = 0;
    if (slots == 0 && TMA_OK) {
        int dev = 0, sms = 0, per_sm = 0;
        if (cudaFuncSetAttribute(attn_tma_decode_walk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WALK_SMEM) != cudaSuccess ||
            cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_tma_decode_walk_kernel, TMA_THREADS, WALK_SMEM) != cudaSuccess ||
            sms <= 0 || per_sm <= 0)
            return 0;
        slots = sms * per_sm;
    }
    return slots;
}
// For `cut` 1 of oxr_paged_attention_bf16: how many partial slots the scratch must have for
// `units` = short tiles x KV heads x head groups (part_o: slots x 16 x D floats, part_ml: slots x 16 x 2): units + the
// blocks of one round, or 0 if the even cut cannot be used for so many units or on this head size.
OXR_API int oxr_attn_even_cut_slots(int units) {
    const int slots = walk_slots();
    return (slots > 0 && units > 0 && units <= EVEN_MAX_UNITS) ? units + slots : 0;
}

// Pieces that the split-KV kernel with TMA gathers runs with a block each (beyond it, one round of blocks walks over them).
OXR_API int oxr_attn_one_round_of_pieces() { return walk_slots(); }

OXR_API int oxr_attn_head_dim() { return D; }
// Which split-KV kernel the last call with short tiles launched: 0 none yet, 1 cp.async gathers, 2 TMA gathers with one
// block per piece, 3 TMA gathers with one round of blocks that walk over the pieces, 4 the same with the even cut of all key
// blocks. For tests and profiles.
static int oxr_last_short_kernel = 0;
OXR_API int oxr_attn_last_short_kernel() { return oxr_last_short_kernel; }

// The split-KV kernels with TMA gathers for the short tiles: kv_maps holds the group's two tensor maps (K, V) made by
// oxr_attn_make_kv_maps. FUSED: the tiles are single tokens and `f` names their raw projections (FuseQkv); only the form with
// a block per piece does that (a block that walks over many pieces would prepare q again for each, which at 64 requests of
// 2,048 keys cost more than the kernel it saves: 7.21 against 7.14 ms for a Qwen3-8B decode step), so more pieces than one
// round of blocks, or the even cut, are refused.
template <bool FUSED>
static int launch_tma_decode(void* out, const void* q, int n_short, int groups_y, int splits, float* part_o, float* part_ml, int* counters,
                             const void* kv_maps, int pool_row0, int cut, const AttnArgs& a, const FuseQkv& f, cudaStream_t stream) {
    static bool tma_configured = false;
    if (!tma_configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tma_decode_kernel<FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TMA_DECODE_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        tma_configured = true;
    }
    const CUtensorMap* maps = reinterpret_cast<const CUtensorMap*>(kv_maps);
    const int box_rows = a.page_size < MMA_BN ? a.page_size : MMA_BN;
    const long long pieces = (long long)n_short * groups_y * splits;
    if (pieces > 0x7fffffffLL) return OXR_BAD_ARGUMENT;
    const int slots = walk_slots();   // blocks of the walking kernel that the GPU holds at once
    if (slots <= 0) return OXR_BAD_ARGUMENT;
    if (FUSED && (cut != 0 || pieces > slots)) return OXR_BAD_ARGUMENT;
    if (cut != 0) {
        // one round of blocks and the even cut of all key blocks
        if (cut != 1 || (long long)n_short * groups_y > EVEN_MAX_UNITS) return OXR_BAD_ARGUMENT;
        oxr_last_short_kernel = 4;
        oxr_launch(attn_tma_decode_walk_kernel, dim3(slots), dim3(TMA_THREADS), WALK_SMEM, stream, true,
            (bf16*)out, part_o, part_ml, counters, (const bf16*)q, maps[0], maps[1], pool_row0, box_rows, n_short, groups_y, splits, cut, a);
        return oxr_launch_status();
    }
    if (pieces > slots) {
        // more pieces than fit at once: one round of blocks that walk over them
        oxr_last_short_kernel = 3;
        oxr_launch(attn_tma_decode_walk_kernel, dim3(slots), dim3(TMA_THREADS), WALK_SMEM, stream, true,
            (bf16*)out, part_o, part_ml, counters, (const bf16*)q, maps[0], maps[1], pool_row0, box_rows, n_short, groups_y, splits, 0, a);
        return oxr_launch_status();
    }
    oxr_last_short_kernel = 2;
    oxr_launch(attn_tma_decode_kernel<FUSED>, dim3(n_short, groups_y, splits), dim3(TMA_THREADS), TMA_DECODE_SMEM, stream, true,
        (bf16*)out, part_o, part_ml, counters, (const bf16*)q, maps[0], maps[1], pool_row0, box_rows, a, f);
    return oxr_launch_status();
}
// Rows of a tile for each kind of tile list that the host builds: 0 generic, 1 decode, 2 prefill (mma.sync), 3 prefill
// (tcgen05). The host keeps the same numbers and compares them when it loads the library.
OXR_API int oxr_attn_tile_rows(int kind) {
    switch (kind) {
        case 0: return BM;
        case 1: return DECODE_ROWS;
        case 2: return PREFILL_ROWS;
        case 3: return BIG_ROWS;
        default: return -1;
    }
}

// bfloat16 on the tensor cores. Two tile lists made by the host: `short` tiles (16 rows each; decoded tokens and
// portions of a few tokens) go to the split-KV kernel, `long` tiles (64 rows each) to the prefill kernel. With
// splits > 1 the caller provides scratch: part_o [n_short * KV * groups16 * splits * 16 * D] floats, part_ml
// [n_short * KV * groups16 * splits * 16 * 2] floats and counters [n_short * KV * groups16] ints that are zero
// before the first launch (the kernel leaves them zero), groups16 = ceil(G / min(G, 16)).
// kv_maps (optional): the two tensor maps of oxr_attn_make_kv_maps for the pool that k_cache / v_cache are a layer
// of, with pool_row0 = layer * num_pages * page_size; the split-KV kernel then fetches K and V by TMA.
// long_rows: rows per long tile the host cut the long list for: 64 (cp.async kernel) or 256 (tcgen05 kernel, needs kv_maps).
// q_tokens: tokens (rows) of q and out, or 0 if unknown (the tcgen05 kernel then reads Q with ordinary loads).
// cut (split-KV with TMA gathers only): 0 every request in `splits` equal pieces; 1 all key blocks of the step dealt out
// evenly to one round of blocks, for requests of very different lengths (the scratch must then have
// oxr_attn_even_cut_slots(units) slots, also with splits == 1).
OXR_API int oxr_paged_attention_bf16(void* out, const void* q, const void* k_cache, const void* v_cache,
                                     const int* short_req, const int* short_tok0, int n_short, const int* long_req,
                                     const int* long_tok0, int n_long, const int* cu_q, const int* ctx_lens,
                                     const int* block_table, int table_width, int page_size, int num_pages, int H, int KV,
                                     float scale, int window, int splits, float* part_o, float* part_ml, int* counters,
                                     const void* kv_maps, int pool_row0, int long_rows, int q_tokens, int cut, int* status, cudaStream_t stream) {
    if (n_short <= 0 && n_long <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV != 0 || page_size <= 0 || table_width <= 0 || window < 0 || splits < 1) return OXR_BAD_ARGUMENT;
    if ((splits > 1 || cut != 0) && n_short > 0 && (part_o == nullptr || part_ml == nullptr || counters == nullptr)) return OXR_BAD_ARGUMENT;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_mma_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREFILL_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_mma_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    const int G = H / KV;
    AttnArgs a;
    a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.block_table = block_table;
    a.table_width = table_width; a.page_size = page_size; a.num_pages = num_pages; a.H = H; a.KV = KV;
    a.page_shift = -1;
    for (int sh = 0; sh < 30; ++sh) if ((1 << sh) == page_size) a.page_shift = sh;
    a.heads_per_tile = a.tokens_per_tile = a.head_groups = 0;   // the tensor-core kernels derive these from their row count
    a.scale = scale; a.window = window; a.status = status;
    if (n_long > 0 && long_rows == BIG_ROWS) {
        // long tiles of 256 rows: the tcgen05 kernel (the host made the tile list for 256 rows)
        if (!TMA_OK || D > 128 || kv_maps == nullptr || a.page_shift < 3 || !(scale > 0.f)) return OXR_BAD_ARGUMENT;
        static bool big_configured = false;
        if (!big_configured) {
            cudaError_t e = cudaFuncSetAttribute(attn_tc5_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
            if (e != cudaSuccess) return 1000 + (int)e;
            big_configured = true;
        }
        const int hpt = G < BIG_ROWS ? G : BIG_ROWS;
        const int groups = (G + hpt - 1) / hpt;
        if ((size_t)KV * groups * (size_t)n_long > 0x7fffffffull) return OXR_BAD_ARGUMENT;
        a.tile_req = long_req; a.tile_tok0 = long_tok0;
        const CUtensorMap* maps = reinterpret_cast<const CUtensorMap*>(kv_maps);
        const int box_rows = page_size < MMA_BN ? page_size : MMA_BN;
        // Q by TMA when a half's 128 rows are whole tokens (a [tokens, H, D] map made for this call: q moves from call to call)
        CUtensorMap map_q = maps[0];
        const int q_by_tma = (q_tokens > 0 && HALF_ROWS % G == 0 &&
                              oxr_make_map_bf16_3d(&map_q, q, (unsigned long long)q_tokens, (unsigned long long)H, D, HALF_ROWS / G, G)) ? 1 : 0;
        attn_tc5_prefill_kernel<<<dim3((unsigned)(n_long * KV * groups)), TC_THREADS, TC_SMEM, stream>>>(
            (bf16*)out, (const bf16*)q, maps[0], maps[1], map_q, q_by_tma, pool_row0, box_rows, n_long, KV * groups, a);
        int rc = oxr_launch_status();
        if (rc) return rc;
    } else if (n_long > 0) {
        if (long_rows != PREFILL_ROWS) return OXR_BAD_ARGUMENT;
        const int hpt = G < PREFILL_ROWS ? G : PREFILL_ROWS;
        const int groups = (G + hpt - 1) / hpt;
        if ((size_t)KV * groups * (size_t)n_long > 0x7fffffffull) return OXR_BAD_ARGUMENT;
        a.tile_req = long_req; a.tile_tok0 = long_tok0;
        attn_mma_prefill_kernel<<<dim3((unsigned)(n_long * KV * groups)), MMA_THREADS, PREFILL_SMEM, stream>>>(
            (bf16*)out, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, n_long, KV * groups, a);
        int rc = oxr_launch_status();
        if (rc) return rc;
    }
    if (n_short > 0) {
        const int hpt = G < DECODE_ROWS ? G : DECODE_ROWS;
        const int groups = (G + hpt - 1) / hpt;
        if ((size_t)KV * groups > 65535 || splits > 65535) return OXR_BAD_ARGUMENT;
        a.tile_req = short_req; a.tile_tok0 = short_tok0;
        if (TMA_OK && kv_maps != nullptr && a.page_shift >= 3)
            return launch_tma_decode<false>(out, q, n_short, KV * groups, splits, part_o, part_ml, counters, kv_maps, pool_row0, cut, a, FuseQkv{}, stream);
        oxr_last_short_kernel = 1;
        attn_mma_decode_kernel<<<dim3(n_short, KV * groups, splits), MMA_THREADS, DECODE_SMEM, stream>>>(
            (bf16*)out, part_o, part_ml, counters, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, a);
        int rc = oxr_launch_status();
        if (rc) return rc;
    }
    return 0;
}

// A decode step's attention straight from the raw projections: every request brings ONE token (row r of qkv
// [n, (H + 2 KV) * D] is request r's; cu_q = 0, 1, 2, ...), `short_req` / `short_tok0` are the n tiles of the short list. The
// kernel normalises q and k per head (q_weight / k_weight [D] fp32, null: no norm), rotates them by the rows of the tables
// [max_positions, D / 2] at each request's last position (null tables: no rotation), writes k and v into the cache
// (store = 0: writes nothing and attends to what the cache holds) and attends, as oxr_qk_norm_rope_store followed by
// oxr_paged_attention_bf16 would. Needs kv_maps, a head size that is a multiple of 64 and pages of 8 * 2^k tokens
// and no more pieces (n_short * KV * head groups * splits) than oxr_attn_one_round_of_pieces(), cut 0 (OXR_BAD_ARGUMENT
// otherwise); splits and scratch as in oxr_paged_attention_bf16.
OXR_API int oxr_paged_attention_fused_decode_bf16(void* out, const void* qkv, void* k_cache, void* v_cache, const int* short_req,
                                                  const int* short_tok0, int n_short, const int* cu_q, const int* ctx_lens,
                                                  const int* block_table, int table_width, int page_size, int num_pages, int H, int KV,
                                                  float scale, int window, int splits, float* part_o, float* part_ml, int* counters,
                                                  const void* kv_maps, int pool_row0, int cut, const float* q_weight, const float* k_weight,
                                                  const float* cos_table, const float* sin_table, float eps, int max_positions, int store,
                                                  int* status, cudaStream_t stream) {
    if (n_short <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV != 0 || page_size <= 0 || table_width <= 0 || window < 0 || splits < 1) return OXR_BAD_ARGUMENT;
    if ((splits > 1 || cut != 0) && (part_o == nullptr || part_ml == nullptr || counters == nullptr)) return OXR_BAD_ARGUMENT;
    if (!TMA_OK || kv_maps == nullptr || qkv == nullptr || (uintptr_t)qkv % 16 != 0 || (cos_table == nullptr) != (sin_table == nullptr) ||
        (cos_table != nullptr && max_positions <= 0))
        return OXR_BAD_ARGUMENT;
    const int G = H / KV;
    AttnArgs a;
    a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.block_table = block_table;
    a.table_width = table_width; a.page_size = page_size; a.num_pages = num_pages; a.H = H; a.KV = KV;
    a.page_shift = -1;
    for (int sh = 0; sh < 30; ++sh) if ((1 << sh) == page_size) a.page_shift = sh;
    if (a.page_shift < 3) return OXR_BAD_ARGUMENT;
    a.heads_per_tile = a.tokens_per_tile = a.head_groups = 0;
    a.scale = scale; a.window = window; a.status = status;
    a.tile_req = short_req; a.tile_tok0 = short_tok0;
    const int hpt = G < DECODE_ROWS ? G : DECODE_ROWS;
    const int groups = (G + hpt - 1) / hpt;
    if ((size_t)KV * groups > 65535 || splits > 65535) return OXR_BAD_ARGUMENT;
    FuseQkv f;
    f.qkv = (const bf16*)qkv;
    f.k_cache = store ? (bf16*)k_cache : nullptr;
    f.v_cache = store ? (bf16*)v_cache : nullptr;
    f.q_weight = q_weight; f.k_weight = k_weight; f.cos_table = cos_table; f.sin_table = sin_table;
    f.eps = eps; f.max_positions = max_positions;
    return launch_tma_decode<true>(out, nullptr, n_short, KV * groups, splits, part_o, part_ml, counters, kv_maps, pool_row0, cut, a, f, stream);
}

// dtype: 0 = float32, 1 = bfloat16 (q, out and the cache). q, out: [tokens, H, D]. k_cache, v_cache: one layer's
// pool [num_pages, page_size, KV, D]. The tile list is made by the host with tokens_per_tile =
// tile_rows / min(G, tile_rows) tokens per tile.
OXR_API int oxr_paged_attention(void* out, const void* q, const void* k_cache, const void* v_cache, const int* tile_req,
                                const int* tile_tok0, int num_tiles, const int* cu_q, const int* ctx_lens,
                                const int* block_table, int table_width, int page_size, int num_pages, int H, int KV,
                                float scale, int window, int dtype, int* status, cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV != 0 || page_size <= 0 || table_width <= 0 || window < 0) return OXR_BAD_ARGUMENT;
    const int G = H / KV;
    AttnArgs a;
    a.tile_req = tile_req; a.tile_tok0 = tile_tok0; a.cu_q = cu_q; a.ctx_lens = ctx_lens; a.block_table = block_table;
    a.table_width = table_width; a.page_size = page_size; a.num_pages = num_pages; a.H = H; a.KV = KV;
    a.page_shift = -1;
    for (int sh = 0; sh < 30; ++sh) if ((1 << sh) == page_size) a.page_shift = sh;
    a.heads_per_tile = G < BM ? G : BM;
    a.tokens_per_tile = BM / a.heads_per_tile;
    a.head_groups = (G + a.heads_per_tile - 1) / a.heads_per_tile;
    a.scale = scale; a.window = window; a.status = status;
    if ((size_t)KV * a.head_groups > 65535) return OXR_BAD_ARGUMENT;
    if (dtype == 0) return launch_simt<float>(out, q, k_cache, v_cache, a, num_tiles, stream);
    if (dtype == 1) return launch_simt<__nv_bfloat16>(out, q, k_cache, v_cache, a, num_tiles, stream);
    return OXR_BAD_ARGUMENT;
}

// Two CUtensorMap (K then V, 128 bytes each, written to 64-byte aligned host memory at `out_maps`) over a whole
// group's pool [layers * pages * page_size rows, KV * D columns] bf16, in boxes of min(page_size, 64) rows x 64
// columns with the 128-byte swizzle. Returns 0, or OXR_BAD_ARGUMENT when the sizes do not allow TMA gathers (head size
// not a multiple of 64, page size not 8 * 2^k, misaligned pool).
OXR_API int oxr_attn_make_kv_maps(void* out_maps, const void* k_pool, const void* v_pool, unsigned long long total_rows, int row_elems,
                                  int page_size) {
    if (!TMA_OK || out_maps == nullptr || (uintptr_t)out_maps % 64 != 0 || row_elems % 8 != 0 || total_rows == 0) return OXR_BAD_ARGUMENT;
    if (page_size < 8 || (page_size & (page_size - 1)) != 0) return OXR_BAD_ARGUMENT;
    if ((uintptr_t)k_pool % 16 != 0 || (uintptr_t)v_pool % 16 != 0) return OXR_BAD_ARGUMENT;
    CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(out_maps);
    const int box_rows = page_size < MMA_BN ? page_size : MMA_BN;
    if (!oxr_make_map_bf16(&maps[0], k_pool, total_rows, (unsigned long long)row_elems, box_rows)) return OXR_BAD_ARGUMENT;
    if (!oxr_make_map_bf16(&maps[1], v_pool, total_rows, (unsigned long long)row_elems, box_rows)) return OXR_BAD_ARGUMENT;
    return 0;
}

// Whether this library's split-KV kernel is launched programmatically dependent on the kernel before it (common.cuh).
OXR_API void oxr_set_chain(int on) { oxr_chain_kernels = on ? 1 : 0; }
