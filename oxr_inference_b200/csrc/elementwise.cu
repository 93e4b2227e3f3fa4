// Embedding gather, RMSNorm with fused residual add, SiLU-gated product, dtype casts.
//
// What each computes follows the reference's language model: embedding lookup (oxr_runtime/decode_graph.py:75),
// `_rms_norm` / `_add_rms_norm` (oxr_runtime/language.py:69-72,94-99) and `_silu_mul`
// (oxr_runtime/language.py:102-104). Differences, all toward more exactness: the residual stream is carried
// in fp32 whatever the activation dtype, and each result is rounded to the activation dtype once.
#include "common.cuh"
OXR_TL_DEFINE(oxr_tl_read_elem)

// ---------------------------------------------------------------------------------------------- embedding
template <typename TT, typename TO>
__global__ void embedding_kernel(TO* __restrict__ out, const TT* __restrict__ table, const int* __restrict__ ids,
                                 int hidden, int vocab, int* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    TO* dst = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) oxr_report(status, OXR_BAD_TOKEN_ID, t);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = Num<TO>::from_f32(0.f);
        return;
    }
    const TT* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = Num<TO>::from_f32(Num<TT>::to_f32(src[i]));
}

// 16-byte copies when table and output share a dtype and a row is a whole number of 16-byte words.
template <typename T>
__global__ void embedding_vec_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                     int words_per_row, int vocab, int* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    uint4* dst = reinterpret_cast<uint4*>(out) + (size_t)t * words_per_row;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) oxr_report(status, OXR_BAD_TOKEN_ID, t);
        for (int i = threadIdx.x; i < words_per_row; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(table) + (size_t)id * words_per_row;
    for (int i = threadIdx.x; i < words_per_row; i += blockDim.x) dst[i] = __ldg(src + i);
}

// table_dtype / out_dtype: 0 = float32, 1 = bfloat16
OXR_API int oxr_embedding(void* out, const void* table, const int* ids, int n_tokens, int hidden, int vocab,
                          int table_dtype, int out_dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = 256;
    if (table_dtype == out_dtype) {
        const int esize = table_dtype == 0 ? 4 : 2;
        const bool aligned = ((size_t)hidden * esize) % 16 == 0 && ((uintptr_t)out % 16 == 0) && ((uintptr_t)table % 16 == 0);
        if (aligned) {
            const int words = hidden * esize / 16;
            if (table_dtype == 0)
                embedding_vec_kernel<float><<<n_tokens, threads, 0, stream>>>((float*)out, (const float*)table, ids, words, vocab, status);
            else
                embedding_vec_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)table, ids, words, vocab, status);
            return oxr_launch_status();
        }
    }
    if (table_dtype == 0 && out_dtype == 0)
        embedding_kernel<float, float><<<n_tokens, threads, 0, stream>>>((float*)out, (const float*)table, ids, hidden, vocab, status);
    else if (table_dtype == 1 && out_dtype == 1)
        embedding_kernel<__nv_bfloat16, __nv_bfloat16><<<n_tokens, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)table, ids, hidden, vocab, status);
    else if (table_dtype == 0 && out_dtype == 1)
        embedding_kernel<float, __nv_bfloat16><<<n_tokens, threads, 0, stream>>>((__nv_bfloat16*)out, (const float*)table, ids, hidden, vocab, status);
    else if (table_dtype == 1 && out_dtype == 0)
        embedding_kernel<__nv_bfloat16, float><<<n_tokens, threads, 0, stream>>>((float*)out, (const __nv_bfloat16*)table, ids, hidden, vocab, status);
    else
        return OXR_BAD_ARGUMENT;
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- RMSNorm
// One block per output row. Row r reads input row `rows ? rows[r] : r`.
//   sum      = x (+ residual_in)                  in fp32; written to residual_out (fp32) when given
//   out[r,:] = round( sum * rsqrt(mean(sum^2) + eps) * weight )
// The second pass re-reads `sum` from shared memory when the row fits there, else from residual_out, else
// recomputes it.
template <typename T>
__global__ void add_rms_norm_kernel(T* __restrict__ out, float* __restrict__ residual_out, const T* __restrict__ x,
                                    const float* __restrict__ residual_in, const float* __restrict__ weight,
                                    const int* __restrict__ rows, int hidden, float eps, int row_floats_in_smem) {
    extern __shared__ float smem[];
    float* red = smem;            // 32 floats
    float* rowbuf = smem + 32;    // row_floats_in_smem floats
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    const size_t dst = (size_t)r * hidden;
    const bool cached = row_floats_in_smem >= hidden;

    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = Num<T>::to_f32(x[src + i]);
        if (residual_in) v += residual_in[src + i];
        if (residual_out) residual_out[dst + i] = v;
        if (cached) rowbuf[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v;
        if (cached) {
            v = rowbuf[i];
        } else if (residual_out) {
            v = residual_out[dst + i];   // written by this same thread in the first pass
        } else {
            v = Num<T>::to_f32(x[src + i]);
            if (residual_in) v += residual_in[src + i];
        }
        out[dst + i] = Num<T>::from_f32(v * inv * weight[i]);
    }
}

// Fast path for bf16 rows that are a whole number of 16-byte words: a thread takes up to VEC_PER_THREAD words of 8
// elements, loads everything it needs up front (x as one 16-byte load, the residual as two), and writes from
// registers, so the row is read once and no load waits behind a store.
template <int VEC_PER_THREAD>
__global__ void add_rms_norm_bf16x8_kernel(__nv_bfloat16* __restrict__ out, float* residual_out, const __nv_bfloat16* __restrict__ x,
                                           const float* residual_in, const float* __restrict__ weight,
                                           const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float red[32];
    if (gridDim.x <= 296) pdl_trigger();   // a decode step's few blocks: the next kernel may set itself up beside them
    const int words = hidden >> 3;
    // the norm's weights are written by no kernel of a step: they are fetched while the kernel before still runs
    float4 wt[VEC_PER_THREAD][2];
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; ++i) {
        const int w = threadIdx.x + i * blockDim.x;
        if (w < words) {
            wt[i][0] = __ldg(reinterpret_cast<const float4*>(weight + (size_t)w * 8));
            wt[i][1] = __ldg(reinterpret_cast<const float4*>(weight + (size_t)w * 8 + 4));
        }
    }
    pdl_wait();
    [[maybe_unused]] const unsigned long long tl_released = OXR_TL_NOW();
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    const size_t dst = (size_t)r * hidden;
    float v[VEC_PER_THREAD][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; ++i) {
        const int w = threadIdx.x + i * blockDim.x;
        if (w < words) {
            const uint4 xv = *reinterpret_cast<const uint4*>(x + src + (size_t)w * 8);
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(xp[k]);
                v[i][2 * k] = f.x;
                v[i][2 * k + 1] = f.y;
            }
            if (residual_in) {
                const float4 r0 = *reinterpret_cast<const float4*>(residual_in + src + (size_t)w * 8);
                const float4 r1 = *reinterpret_cast<const float4*>(residual_in + src + (size_t)w * 8 + 4);
                v[i][0] += r0.x; v[i][1] += r0.y; v[i][2] += r0.z; v[i][3] += r0.w;
                v[i][4] += r1.x; v[i][5] += r1.y; v[i][6] += r1.z; v[i][7] += r1.w;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += v[i][k] * v[i][k];
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; ++i) {
        const int w = threadIdx.x + i * blockDim.x;
        if (w < words) {
            if (residual_out) {
                *reinterpret_cast<float4*>(residual_out + dst + (size_t)w * 8) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
                *reinterpret_cast<float4*>(residual_out + dst + (size_t)w * 8 + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
            }
            const float4 w0 = wt[i][0], w1 = wt[i][1];
            uint4 o;
            __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
            op[0] = __floats2bfloat162_rn(v[i][0] * inv * w0.x, v[i][1] * inv * w0.y);
            op[1] = __floats2bfloat162_rn(v[i][2] * inv * w0.z, v[i][3] * inv * w0.w);
            op[2] = __floats2bfloat162_rn(v[i][4] * inv * w1.x, v[i][5] * inv * w1.y);
            op[3] = __floats2bfloat162_rn(v[i][6] * inv * w1.z, v[i][7] * inv * w1.w);
            *reinterpret_cast<uint4*>(out + dst + (size_t)w * 8) = o;
        }
    }
#ifdef OXR_TIMELINE
    __syncthreads();
    if (threadIdx.x == 0) OXR_TL_PUT(2, tl_released, OXR_TL_NOW(), 0, 0, blockIdx.x);
#endif
}

// dtype: 0 = float32, 1 = bfloat16 (of x and out). residual_in / residual_out / rows may be null.
// residual_out may alias residual_in only when rows is null (each element is read before it is written by
// the same thread).
OXR_API int oxr_add_rms_norm(void* out, float* residual_out, const void* x, const float* residual_in,
                             const float* weight, const int* rows, int n_rows, int hidden, float eps, int dtype,
                             cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (rows != nullptr && residual_out != nullptr && residual_out == residual_in) return OXR_BAD_ARGUMENT;
    if (dtype == 1 && hidden % 8 == 0 && hidden <= 8 * 4 * 512 && (uintptr_t)out % 16 == 0 && (uintptr_t)x % 16 == 0 &&
        (uintptr_t)weight % 16 == 0 && (residual_in == nullptr || (uintptr_t)residual_in % 16 == 0) &&
        (residual_out == nullptr || (uintptr_t)residual_out % 16 == 0)) {
        const int words = hidden / 8;
        const int vt = words <= 128 ? 128 : (words <= 256 ? 256 : 512);
        const int per = (words + vt - 1) / vt;
#define NORM_VEC(P) oxr_launch(add_rms_norm_bf16x8_kernel<P>, dim3(n_rows), dim3(vt), 0, stream, true, (__nv_bfloat16*)out, residual_out, (const __nv_bfloat16*)x, residual_in, weight, rows, hidden, eps)
        if (per <= 1) NORM_VEC(1);
        else if (per <= 2) NORM_VEC(2);
        else NORM_VEC(4);
#undef NORM_VEC
        return oxr_launch_status();
    }
    int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int cache_floats = hidden <= 10240 ? hidden : 0;   // 40 KB of row cache at most
    const size_t smem = (32 + cache_floats) * sizeof(float);
    if (dtype == 0)
        add_rms_norm_kernel<float><<<n_rows, threads, smem, stream>>>((float*)out, residual_out, (const float*)x, residual_in, weight, rows, hidden, eps, cache_floats);
    else if (dtype == 1)
        add_rms_norm_kernel<__nv_bfloat16><<<n_rows, threads, smem, stream>>>((__nv_bfloat16*)out, residual_out, (const __nv_bfloat16*)x, residual_in, weight, rows, hidden, eps, cache_floats);
    else
        return OXR_BAD_ARGUMENT;
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- SiLU * up
// gate_up is [n, 2*inter]. Side by side (`interleave` 0): gate = first half, up = second half
// (oxr_runtime/language.py:102-104). Interleaved by 8: columns 16j .. 16j+7 are gate 8j .. 8j+7 and columns
// 16j+8 .. 16j+15 the matching up values, which is what a product with a weight whose gate and up rows alternate in
// groups of 8 writes (the decode kernel that applies SiLU in its epilogue needs both in one block).
__device__ __forceinline__ void gate_up_at(size_t row, size_t col, int inter, int interleave, size_t& g, size_t& u) {
    if (interleave) {
        g = row * 2 * inter + (col / 8) * 16 + col % 8;
        u = g + 8;
    } else {
        g = row * 2 * inter + col;
        u = g + inter;
    }
}
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, int interleave, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t gi, ui;
        gate_up_at(i / inter, i % inter, inter, interleave, gi, ui);
        const float g = Num<T>::to_f32(gate_up[gi]);
        const float u = Num<T>::to_f32(gate_up[ui]);
        out[i] = Num<T>::from_f32(g / (1.f + __expf(-g)) * u);
    }
}
template <>
__global__ void silu_mul_kernel<float>(float* __restrict__ out, const float* __restrict__ gate_up, int inter, int interleave, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t gi, ui;
        gate_up_at(i / inter, i % inter, inter, interleave, gi, ui);
        const float g = gate_up[gi];
        const float u = gate_up[ui];
        out[i] = g / (1.f + expf(-g)) * u;   // full-precision exp on the 32-bit path
    }
}

// bf16, inter a multiple of 8: 16-byte loads and stores. Grid (column chunks, rows): no division per element.
// With INTERLEAVED the gate word of output word `col` is word 2 col of the row and its up word the next one.
template <bool INTERLEAVED>
__global__ void silu_mul_bf16x8_kernel(uint4* __restrict__ out, const uint4* __restrict__ gate_up, int inter8) {
    const size_t row = blockIdx.y;
    const uint4* g_row = gate_up + row * 2 * inter8;
    uint4* o_row = out + row * inter8;
    for (int col = blockIdx.x * blockDim.x + threadIdx.x; col < inter8; col += gridDim.x * blockDim.x) {
        uint4 g = __ldg(g_row + (INTERLEAVED ? 2 * col : col));
        uint4 u = __ldg(g_row + (INTERLEAVED ? 2 * col + 1 : inter8 + col));
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
        uint4 o;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 gf = __bfloat1622float2(gp[k]), uf = __bfloat1622float2(up[k]);
            float2 r;
            r.x = gf.x / (1.f + __expf(-gf.x)) * uf.x;
            r.y = gf.y / (1.f + __expf(-gf.y)) * uf.y;
            op[k] = __float22bfloat162_rn(r);
        }
        o_row[col] = o;
    }
}

// interleave: 0 (gate | up side by side) or 8 (alternating groups of 8 columns; inter must then be a multiple of 8).
OXR_API int oxr_silu_mul(void* out, const void* gate_up, int n_rows, int inter, int interleave, int dtype, cudaStream_t stream) {
    const size_t total = (size_t)n_rows * inter;
    if (total == 0) return 0;
    if (interleave != 0 && (interleave != 8 || inter % 8 != 0)) return OXR_BAD_ARGUMENT;
    const int threads = 256;
    if (dtype == 1 && inter % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gate_up % 16 == 0) {
        const int inter8 = inter / 8;
        int rows_done = 0;
        while (rows_done < n_rows) {   // grid.y holds at most 65535 rows per launch
            const int rows = n_rows - rows_done < 65535 ? n_rows - rows_done : 65535;
            dim3 grid((inter8 + threads - 1) / threads, rows);
            uint4* o = (uint4*)out + (size_t)rows_done * inter8;
            const uint4* gu = (const uint4*)gate_up + (size_t)rows_done * 2 * inter8;
            if (interleave) silu_mul_bf16x8_kernel<true><<<grid, threads, 0, stream>>>(o, gu, inter8);
            else silu_mul_bf16x8_kernel<false><<<grid, threads, 0, stream>>>(o, gu, inter8);
            rows_done += rows;
        }
        return oxr_launch_status();
    }
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == 0)
        silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, (const float*)gate_up, inter, interleave, total);
    else if (dtype == 1)
        silu_mul_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, inter, interleave, total);
    else
        return OXR_BAD_ARGUMENT;
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------- casts
template <typename TS, typename TD>
__global__ void cast_kernel(TD* __restrict__ dst, const TS* __restrict__ src, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = Num<TD>::from_f32(Num<TS>::to_f32(src[i]));
}

OXR_API int oxr_cast(void* dst, const void* src, size_t n, int src_dtype, int dst_dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    if (src_dtype == 0 && dst_dtype == 1)
        cast_kernel<float, __nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)dst, (const float*)src, n);
    else if (src_dtype == 1 && dst_dtype == 0)
        cast_kernel<__nv_bfloat16, float><<<blocks, threads, 0, stream>>>((float*)dst, (const __nv_bfloat16*)src, n);
    else
        return OXR_BAD_ARGUMENT;
    return oxr_launch_status();
}

// Whether the kernels of this library that are written for it are launched programmatically dependent on the kernel
// before them (see common.cuh). Off until set.
OXR_API void oxr_set_chain(int on) { oxr_chain_kernels = on ? 1 : 0; }
