// Shared device helpers for the sm_100a kernels of this engine.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define OXR_API extern "C" __attribute__((visibility("default")))

// ---- an optional timeline of a step's kernels (compiled in with -DOXR_TIMELINE only; see ops/microbench.py `timeline`)
// Every block of an instrumented kernel leaves one record of six 64-bit words: a kernel id, the time its wait for the
// kernel before it returned, the time it ended, and three more stamps or sizes of the kernel's choosing. Times are
// %globaltimer nanoseconds, one clock for all SMs. Each source file has a buffer of its own and exports a reader.
#ifdef OXR_TIMELINE
#define OXR_TL_DEFINE(reader) \
    static __device__ unsigned long long oxr_tl_buf[1 << 15]; \
    static __device__ unsigned int oxr_tl_n; \
    OXR_API int reader(unsigned long long* out, int words) { /* copies the records out and clears them */ \
        if (words > (1 << 15)) words = 1 << 15; \
        cudaMemcpyFromSymbol(out, oxr_tl_buf, (size_t)words * 8); \
        void* p = nullptr; \
        if (cudaGetSymbolAddress(&p, oxr_tl_buf) == cudaSuccess) cudaMemset(p, 0, sizeof(unsigned long long) << 15); \
        if (cudaGetSymbolAddress(&p, oxr_tl_n) == cudaSuccess) cudaMemset(p, 0, 4); \
        return words; \
    }
static __device__ __forceinline__ unsigned long long oxr_tl_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define OXR_TL_NOW() oxr_tl_now()
#define OXR_TL_PUT(kid, a, b, c, d, e) do { \
        const unsigned int s_ = atomicAdd(&oxr_tl_n, 1u); \
        if (s_ < (1u << 15) / 6) { \
            unsigned long long* r_ = oxr_tl_buf + (size_t)s_ * 6; \
            r_[0] = (kid); r_[1] = (a); r_[2] = (b); r_[3] = (c); r_[4] = (d); r_[5] = (e); \
        } \
    } while (0)
#else
#define OXR_TL_DEFINE(reader)
#define OXR_TL_NOW() 0ull
#define OXR_TL_PUT(kid, a, b, c, d, e) do { } while (0)
#endif

// Error codes written to the engine's device status word (first error wins) and returned by launchers.
enum OxrStatus : int {
    OXR_OK = 0,
    OXR_BAD_TOKEN_ID = 1,     // embedding: id outside [0, vocab)
    OXR_BAD_SLOT = 2,         // cache store: slot outside the pool
    OXR_BAD_POSITION = 3,     // position outside the rotary table
    OXR_BAD_PAGE = 4,         // attention: block table names a page outside the pool
    OXR_WAIT_EXPIRED = 5,     // a bounded wait on an mbarrier ran out
    OXR_BAD_ARGUMENT = 100,   // launcher refused its arguments (host side)
};

__device__ __forceinline__ void oxr_report(int* status, int code, int detail) {
    if (status != nullptr && atomicCAS(status, 0, code) == 0) status[1] = detail;
}

template <typename T> struct Num;
template <> struct Num<float> {
    static __device__ __forceinline__ float to_f32(float v) { return v; }
    static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Num<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum in a fixed order (warp butterflies, then warp 0 over the per-warp partials), so that the
// result for a row does not depend on what else runs. `scratch` holds 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
    return warp_max(t);
}

// ---- programmatic dependent launch
// A kernel launched with `oxr_launch(..., chained = true)` may start while the kernel before it on the stream still
// runs: as soon as every block of that kernel has called `pdl_trigger()` (or left). It must call `pdl_wait()` before
// it reads anything an earlier kernel wrote and before it writes anything at all; `pdl_wait()` returns when the kernel
// before it is complete and its writes are visible (which, since that kernel waited in the same way, holds for all
// kernels before). What stands above the wait (barrier set-up, loads of weights, which no kernel of a step writes)
// overlaps the tail of the kernel before. Both calls do nothing in a kernel launched the ordinary way.
// Chained: RMSNorm, q/k norm + RoPE + store, split-KV attention (which fetches the old keys above its wait), the
// weight-streaming GEMM of decode steps (whose producer warp never waits) and the tcgen05 GEMMs (which request the
// weight tiles of their first ring of stages above their wait). The register-fed skinny GEMM triggers (so the small
// kernel after it starts early) but is itself launched the ordinary way: launched chained it made the step 4 % slower
// on a B200, with or without weight loads above its wait.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline int oxr_chain_kernels = 0;   // one per library: set through oxr_set_chain()

template <typename... KArgs, typename... Args>
static inline void oxr_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool chained, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = (chained && oxr_chain_kernels) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

static inline int oxr_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : 1000 + (int)e;
}
