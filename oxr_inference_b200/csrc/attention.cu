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
#include "common.cuh"

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

OXR_API int oxr_attn_head_dim() { return D; }
OXR_API int oxr_attn_tile_rows() { return BM; }

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
    a.heads_per_tile = G < BM ? G : BM;
    a.tokens_per_tile = BM / a.heads_per_tile;
    a.head_groups = (G + a.heads_per_tile - 1) / a.heads_per_tile;
    a.scale = scale; a.window = window; a.status = status;
    if ((size_t)KV * a.head_groups > 65535) return OXR_BAD_ARGUMENT;
    if (dtype == 0) return launch_simt<float>(out, q, k_cache, v_cache, a, num_tiles, stream);
    if (dtype == 1) return launch_simt<__nv_bfloat16>(out, q, k_cache, v_cache, a, num_tiles, stream);
    return OXR_BAD_ARGUMENT;
}
