// Fused per-head q/k RMSNorm + rotary position encoding + store of K and V into the paged cache.
//
// Takes the place of the reference's one hand-written GPU kernel, the Triton
// `_qk_norm_rope_store_kernel` (oxr_runtime/kernels.py:66-99): for each token, every q head and k head is
// RMS-normalised over head_dim with a weight shared by all heads (kernels.py:48-60), rotated by the
// half-split (GPT-NeoX) rule out = (y1*c - y2*s, y1*s + y2*c) (kernels.py:61-63), q is written out and k, v go
// to `cache + slot * KV * D` (kernels.py:84-99). Unlike the reference it takes any even head_dim, gathers
// cos/sin by position itself, keeps the whole computation in fp32 and rounds once.
#include "common.cuh"
OXR_TL_DEFINE(oxr_tl_read_rope)

// One warp per (token, head); heads 0..H-1 are q, H..H+KV-1 are k, H+KV..H+2KV-1 are v.
// Lane l handles the pairs (j, j + D/2) for j = l, l + 32, ...
template <typename T, int MAX_PAIRS_PER_LANE>
__global__ void qk_norm_rope_store_kernel(
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache, const T* __restrict__ qkv,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight, const float* __restrict__ cos_table,
    const float* __restrict__ sin_table, const int* __restrict__ positions, const int* __restrict__ slots,
    int n_tokens, int H, int KV, int D, float eps, int max_positions, long long num_slots, int norm_q, int norm_k,
    int rotate, int* status) {
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int heads = H + 2 * KV;
    if (unit >= (long long)n_tokens * heads) return;
    const int t = (int)(unit / heads), head = (int)(unit % heads);
    const int half = D >> 1;
    const T* src = qkv + (size_t)t * heads * D + (size_t)head * D;

    T* dst;
    if (head < H) {
        dst = q_out + (size_t)t * H * D + (size_t)head * D;
    } else {
        const long long slot = slots[t];
        if (slot < 0) return;  // a row that is not to be stored (padding)
        if (slot >= num_slots) {
            if (lane == 0) oxr_report(status, OXR_BAD_SLOT, t);
            return;
        }
        const bool is_k = head < H + KV;
        const int kvh = is_k ? head - H : head - H - KV;
        dst = (is_k ? k_cache : v_cache) + (size_t)slot * KV * D + (size_t)kvh * D;
        if (!is_k) {  // v: copied unchanged
            for (int j = lane; j < D; j += 32) dst[j] = src[j];
            return;
        }
    }

    const bool is_q = head < H;
    const bool do_norm = is_q ? norm_q : norm_k;
    const float* w = is_q ? q_weight : k_weight;

    float x1[MAX_PAIRS_PER_LANE], x2[MAX_PAIRS_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PAIRS_PER_LANE; ++i) {
        const int j = lane + 32 * i;
        x1[i] = x2[i] = 0.f;
        if (j < half) {
            x1[i] = Num<T>::to_f32(src[j]);
            x2[i] = Num<T>::to_f32(src[j + half]);
            ss += x1[i] * x1[i] + x2[i] * x2[i];
        }
    }
    float inv = 1.f;
    if (do_norm) {
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float)D + eps);
    }
    int pos = 0;
    if (rotate) {
        pos = positions[t];
        if (pos < 0 || pos >= max_positions) {
            if (lane == 0) oxr_report(status, OXR_BAD_POSITION, t);
            pos = 0;
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_PAIRS_PER_LANE; ++i) {
        const int j = lane + 32 * i;
        if (j < half) {
            float y1 = x1[i], y2 = x2[i];
            if (do_norm) {
                y1 = y1 * inv * w[j];
                y2 = y2 * inv * w[j + half];
            }
            if (rotate) {
                const float c = cos_table[(size_t)pos * half + j], s = sin_table[(size_t)pos * half + j];
                const float r1 = y1 * c - y2 * s, r2 = y1 * s + y2 * c;
                y1 = r1;
                y2 = r2;
            }
            dst[j] = Num<T>::from_f32(y1);
            dst[j + half] = Num<T>::from_f32(y2);
        }
    }
}

// bf16 with head sizes that are multiples of 64. One warp takes HPW consecutive heads of a token: lane l holds elements
// 2l, 2l+1 (+64 per step) of the first half of each head and their partners in the second half (4-byte loads and
// stores); the loads of all its heads are issued before anything is reduced, so that a warp has several cache lines in
// flight. v heads are copied with 16-byte words.
template <int STEPS, int HPW>
__global__ void qk_norm_rope_store_bf16x2_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, const int* __restrict__ positions,
    const int* __restrict__ slots, int n_tokens, int H, int KV, int D, float eps, int max_positions, long long num_slots,
    int norm_q, int norm_k, int rotate, int* status) {
    if (gridDim.x <= 296) pdl_trigger();   // a decode step's few blocks: the next kernel may set itself up beside them
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int heads = H + 2 * KV;
    const int groups = (heads + HPW - 1) / HPW;
    const bool live = unit < (long long)n_tokens * groups;
    const int t = live ? (int)(unit / groups) : 0, head0 = (int)(unit % groups) * HPW;
    const int half = D >> 1;
    // ---- above the wait: what no kernel of the step writes (the step's slots and positions, the rotary tables, the norm
    // weights); only qkv comes from the kernel before this one
    long long slot = -1;
    int pos = 0;
    bool bad_slot = false, bad_pos = false;
    float2 c[STEPS], sn[STEPS], wq1[STEPS], wq2[STEPS], wk1[STEPS], wk2[STEPS];
    if (live) {
        slot = slots[t];
        bad_slot = slot >= num_slots;
        if (rotate) {
            pos = positions[t];
            bad_pos = pos < 0 || pos >= max_positions;
            if (bad_pos) pos = 0;
        }
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            const int j = 2 * lane + 64 * i;
            c[i] = wq1[i] = wq2[i] = wk1[i] = wk2[i] = make_float2(1.f, 1.f);
            sn[i] = make_float2(0.f, 0.f);
            if (j < half) {
                if (rotate) {
                    c[i] = *reinterpret_cast<const float2*>(cos_table + (size_t)pos * half + j);
                    sn[i] = *reinterpret_cast<const float2*>(sin_table + (size_t)pos * half + j);
                }
                if (norm_q) { wq1[i] = *reinterpret_cast<const float2*>(q_weight + j); wq2[i] = *reinterpret_cast<const float2*>(q_weight + j + half); }
                if (norm_k) { wk1[i] = *reinterpret_cast<const float2*>(k_weight + j); wk2[i] = *reinterpret_cast<const float2*>(k_weight + j + half); }
            }
        }
    }
    pdl_wait();
    if (!live) return;
#ifdef OXR_TIMELINE
    struct TlEnd {   // this warp's record, written when the warp leaves the kernel
        unsigned long long released;
        __device__ ~TlEnd() { if ((threadIdx.x & 31) == 0) OXR_TL_PUT(3, released, OXR_TL_NOW(), 0, 0, blockIdx.x); }
    } tl_end{OXR_TL_NOW()};
#endif
    if (bad_slot && lane == 0) oxr_report(status, OXR_BAD_SLOT, t);
    if (bad_pos && lane == 0) oxr_report(status, OXR_BAD_POSITION, t);
    const bool can_store = slot >= 0 && slot < num_slots;
    const __nv_bfloat16* row = qkv + (size_t)t * heads * D;
    // ---- all loads first
    float2 x1[HPW][STEPS], x2[HPW][STEPS];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int head = head0 + hh;
        const bool normed = head < H + KV;   // q or k
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            const int j = 2 * lane + 64 * i;
            x1[hh][i] = x2[hh][i] = make_float2(0.f, 0.f);
            if (head < heads && normed && j < half) {
                x1[hh][i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + (size_t)head * D + j));
                x2[hh][i] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + (size_t)head * D + j + half));
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int head = head0 + hh;
        if (head >= heads) break;
        if (head >= H + KV) {   // v: copied unchanged
            if (can_store) {
                const uint4* src = reinterpret_cast<const uint4*>(row + (size_t)head * D);
                uint4* dst = reinterpret_cast<uint4*>(v_cache + (size_t)slot * KV * D + (size_t)(head - H - KV) * D);
                for (int j = lane; j < D / 8; j += 32) dst[j] = src[j];
            }
            continue;
        }
        const bool is_q = head < H;
        if (!is_q && !can_store) continue;
        __nv_bfloat16* dst = is_q ? q_out + (size_t)t * H * D + (size_t)head * D : k_cache + (size_t)slot * KV * D + (size_t)(head - H) * D;
        const bool do_norm = is_q ? norm_q : norm_k;
        float inv = 1.f;
        if (do_norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < STEPS; ++i)
                ss += x1[hh][i].x * x1[hh][i].x + x1[hh][i].y * x1[hh][i].y + x2[hh][i].x * x2[hh][i].x + x2[hh][i].y * x2[hh][i].y;
            ss = warp_sum(ss);
            inv = rsqrtf(ss / (float)D + eps);
        }
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
            const int j = 2 * lane + 64 * i;
            if (j < half) {
                float2 y1 = x1[hh][i], y2 = x2[hh][i];
                if (do_norm) {
                    const float2 w1 = is_q ? wq1[i] : wk1[i], w2 = is_q ? wq2[i] : wk2[i];
                    y1.x = y1.x * inv * w1.x; y1.y = y1.y * inv * w1.y;
                    y2.x = y2.x * inv * w2.x; y2.y = y2.y * inv * w2.y;
                }
                if (rotate) {
                    const float2 r1 = make_float2(y1.x * c[i].x - y2.x * sn[i].x, y1.y * c[i].y - y2.y * sn[i].y);
                    const float2 r2 = make_float2(y1.x * sn[i].x + y2.x * c[i].x, y1.y * sn[i].y + y2.y * c[i].y);
                    y1 = r1;
                    y2 = r2;
                }
                *reinterpret_cast<__nv_bfloat162*>(dst + j) = __float22bfloat162_rn(y1);
                *reinterpret_cast<__nv_bfloat162*>(dst + j + half) = __float22bfloat162_rn(y2);
            }
        }
    }
}

// bf16 with head size 16 * LPH (64, 128, 256) for steps of many tokens: LPH lanes share a head, lane j of them holds
// elements 8j .. 8j+7 of the head's first half and their rotation partners in the second half, one 16-byte word each,
// so that a warp reads and writes whole 32-byte sectors with two loads and two stores per lane and head; the sum of
// squares goes over the LPH lanes by shuffles. A warp takes WIDE_PASSES * 32 / LPH consecutive heads of a token and
// issues the loads of all of them before it works on any.
constexpr int WIDE_PASSES = 2;
template <int LPH>
__global__ void qk_norm_rope_store_bf16x8_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, const int* __restrict__ positions,
    const int* __restrict__ slots, int n_tokens, int H, int KV, float eps, int max_positions, long long num_slots,
    int norm_q, int norm_k, int rotate, int* status) {
    constexpr int D = 16 * LPH, HPW = 32 / LPH, half = D / 2;
    if (gridDim.x <= 296) pdl_trigger();
    pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int heads = H + 2 * KV;
    const int groups = (heads + WIDE_PASSES * HPW - 1) / (WIDE_PASSES * HPW);
    if (unit >= (long long)n_tokens * groups) return;
    const int t = (int)(unit / groups), head0 = (int)(unit % groups) * WIDE_PASSES * HPW + lane / LPH, j = lane % LPH;
    const long long slot = slots[t];
    if (slot >= num_slots && lane == 0) oxr_report(status, OXR_BAD_SLOT, t);
    const bool can_store = slot >= 0 && slot < num_slots;
    int pos = 0;
    if (rotate) {
        pos = positions[t];
        if (pos < 0 || pos >= max_positions) {
            if (lane == 0) oxr_report(status, OXR_BAD_POSITION, t);
            pos = 0;
        }
    }
    uint4 a[WIDE_PASSES], b[WIDE_PASSES];
#pragma unroll
    for (int p = 0; p < WIDE_PASSES; ++p) {
        const int head = head0 + p * HPW;
        a[p] = b[p] = make_uint4(0, 0, 0, 0);
        if (head < heads) {
            const __nv_bfloat16* src = qkv + ((size_t)t * heads + head) * D + 8 * j;
            a[p] = *reinterpret_cast<const uint4*>(src);
            b[p] = *reinterpret_cast<const uint4*>(src + half);
        }
    }
    float c[8], sn[8];
    if (rotate) {
        const float* cp = cos_table + (size_t)pos * half + 8 * j;
        const float* sp = sin_table + (size_t)pos * half + 8 * j;
        const float4 ca = *reinterpret_cast<const float4*>(cp), cb = *reinterpret_cast<const float4*>(cp + 4);
        const float4 sa = *reinterpret_cast<const float4*>(sp), sb = *reinterpret_cast<const float4*>(sp + 4);
        c[0] = ca.x; c[1] = ca.y; c[2] = ca.z; c[3] = ca.w; c[4] = cb.x; c[5] = cb.y; c[6] = cb.z; c[7] = cb.w;
        sn[0] = sa.x; sn[1] = sa.y; sn[2] = sa.z; sn[3] = sa.w; sn[4] = sb.x; sn[5] = sb.y; sn[6] = sb.z; sn[7] = sb.w;
    }
#pragma unroll
    for (int p = 0; p < WIDE_PASSES; ++p) {
        const int head = head0 + p * HPW;
        const bool live = head < heads, is_q = head < H, is_v = head >= H + KV;
        float x1[8], x2[8];
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a[p]);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b[p]);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f1 = __bfloat1622float2(ap[e]), f2 = __bfloat1622float2(bp[e]);
            x1[2 * e] = f1.x; x1[2 * e + 1] = f1.y; x2[2 * e] = f2.x; x2[2 * e + 1] = f2.y;
            ss += f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y;
        }
#pragma unroll
        for (int o = 1; o < LPH; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // every lane takes part
        if (!live) continue;
        if (is_v) {
            if (can_store) {
                __nv_bfloat16* dst = v_cache + ((size_t)slot * KV + (head - H - KV)) * D + 8 * j;
                *reinterpret_cast<uint4*>(dst) = a[p];
                *reinterpret_cast<uint4*>(dst + half) = b[p];
            }
            continue;
        }
        if (!is_q && !can_store) continue;
        if (is_q ? norm_q : norm_k) {
            const float* w = (is_q ? q_weight : k_weight) + 8 * j;
            const float inv = rsqrtf(ss / (float)D + eps);
            const float4 w1a = *reinterpret_cast<const float4*>(w), w1b = *reinterpret_cast<const float4*>(w + 4);
            const float4 w2a = *reinterpret_cast<const float4*>(w + half), w2b = *reinterpret_cast<const float4*>(w + half + 4);
            const float w1[8] = {w1a.x, w1a.y, w1a.z, w1a.w, w1b.x, w1b.y, w1b.z, w1b.w};
            const float w2[8] = {w2a.x, w2a.y, w2a.z, w2a.w, w2b.x, w2b.y, w2b.z, w2b.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) { x1[e] = x1[e] * inv * w1[e]; x2[e] = x2[e] * inv * w2[e]; }
        }
        if (rotate) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float r1 = x1[e] * c[e] - x2[e] * sn[e], r2 = x1[e] * sn[e] + x2[e] * c[e];
                x1[e] = r1;
                x2[e] = r2;
            }
        }
        uint4 o1, o2;
        __nv_bfloat162* p1 = reinterpret_cast<__nv_bfloat162*>(&o1);
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&o2);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p1[e] = __floats2bfloat162_rn(x1[2 * e], x1[2 * e + 1]);
            p2[e] = __floats2bfloat162_rn(x2[2 * e], x2[2 * e + 1]);
        }
        __nv_bfloat16* dst = (is_q ? q_out + ((size_t)t * H + head) * D : k_cache + ((size_t)slot * KV + (head - H)) * D) + 8 * j;
        *reinterpret_cast<uint4*>(dst) = o1;
        *reinterpret_cast<uint4*>(dst + half) = o2;
    }
}

// dtype: 0 = float32, 1 = bfloat16 (qkv, q_out and the cache). head_dim: even, at most 512.
// k_cache / v_cache: one layer's pool viewed as [num_slots, KV, D]. slots[t] < 0 skips the store.
OXR_API int oxr_qk_norm_rope_store(void* q_out, void* k_cache, void* v_cache, const void* qkv, const float* q_weight,
                                   const float* k_weight, const float* cos_table, const float* sin_table,
                                   const int* positions, const int* slots, int n_tokens, int H, int KV, int D, float eps,
                                   int max_positions, long long num_slots, int norm_q, int norm_k, int rotate, int dtype,
                                   int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || (D & 1) || D > 512) return OXR_BAD_ARGUMENT;
    const int warps = 4;
    const long long units = (long long)n_tokens * (H + 2 * KV);
    const unsigned blocks = (unsigned)((units + warps - 1) / warps);
    if (dtype == 1 && D % 64 == 0 && D <= 512 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_cache % 16 == 0 &&
        (uintptr_t)v_cache % 16 == 0 && (q_weight == nullptr || (uintptr_t)q_weight % 8 == 0) &&
        (k_weight == nullptr || (uintptr_t)k_weight % 8 == 0) && (cos_table == nullptr || ((uintptr_t)cos_table % 8 == 0 && (uintptr_t)sin_table % 8 == 0))) {
        typedef __nv_bfloat16 B;
        const bool wide_ok = (D == 64 || D == 128 || D == 256) && n_tokens >= 64 && (q_weight == nullptr || (uintptr_t)q_weight % 16 == 0) &&
                             (k_weight == nullptr || (uintptr_t)k_weight % 16 == 0) &&
                             (cos_table == nullptr || ((uintptr_t)cos_table % 16 == 0 && (uintptr_t)sin_table % 16 == 0));
        if (wide_ok) {   // steps of many tokens: 16-byte accesses, D / 16 lanes per head
            const int hpw = WIDE_PASSES * 32 / (D / 16);
            const long long wunits = (long long)n_tokens * ((H + 2 * KV + hpw - 1) / hpw);
            const unsigned wblocks = (unsigned)((wunits + warps - 1) / warps);
#define LAUNCH_W(L)                                                                                                     \
            oxr_launch(qk_norm_rope_store_bf16x8_kernel<L>, dim3(wblocks), dim3(warps * 32), 0, stream, true,             \
                (B*)q_out, (B*)k_cache, (B*)v_cache, (const B*)qkv, q_weight, k_weight, cos_table, sin_table, positions, slots, n_tokens, \
                H, KV, eps, max_positions, num_slots, norm_q, norm_k, rotate, status)
            if (D == 64) LAUNCH_W(4);
            else if (D == 128) LAUNCH_W(8);
            else LAUNCH_W(16);
#undef LAUNCH_W
            return oxr_launch_status();
        }
        const int steps = (D / 2 + 63) / 64;   // 1..4
        constexpr int HPW = 4;                  // heads per warp
        const long long vunits = (long long)n_tokens * ((H + 2 * KV + HPW - 1) / HPW);
        const unsigned vblocks = (unsigned)((vunits + warps - 1) / warps);
#define LAUNCH_V(S)                                                                                                     \
        oxr_launch(qk_norm_rope_store_bf16x2_kernel<S, HPW>, dim3(vblocks), dim3(warps * 32), 0, stream, true,           \
            (B*)q_out, (B*)k_cache, (B*)v_cache, (const B*)qkv, q_weight, k_weight, cos_table, sin_table, positions, slots, n_tokens, \
            H, KV, D, eps, max_positions, num_slots, norm_q, norm_k, rotate, status)
        if (steps <= 1) LAUNCH_V(1);
        else if (steps <= 2) LAUNCH_V(2);
        else LAUNCH_V(4);
#undef LAUNCH_V
        return oxr_launch_status();
    }
    const int pairs = (D / 2 + 31) / 32;  // 1..8
#define LAUNCH(T, P)                                                                                               \
    qk_norm_rope_store_kernel<T, P><<<blocks, warps * 32, 0, stream>>>(                                              \
        (T*)q_out, (T*)k_cache, (T*)v_cache, (const T*)qkv, q_weight, k_weight, cos_table, sin_table, positions, slots, \
        n_tokens, H, KV, D, eps, max_positions, num_slots, norm_q, norm_k, rotate, status)
#define DISPATCH(T)                                   \
    if (pairs <= 1) LAUNCH(T, 1);                     \
    else if (pairs <= 2) LAUNCH(T, 2);                \
    else if (pairs <= 4) LAUNCH(T, 4);                \
    else LAUNCH(T, 8)
    if (dtype == 0) { DISPATCH(float); }
    else if (dtype == 1) { DISPATCH(__nv_bfloat16); }
    else return OXR_BAD_ARGUMENT;
#undef DISPATCH
#undef LAUNCH
    return oxr_launch_status();
}
