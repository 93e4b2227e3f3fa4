// Next-token choice on the device: greedy argmax, temperature sampling, repetition penalty.
//
// The reference samples greedily with `logits.argmax(-1)` (oxr_runtime/decode_graph.py:82,
// oxr_runtime/engine.py:454,641) after an optional repetition penalty on the tokens seen so far, prompt
// included: a positive logit is divided by the penalty, any other multiplied (oxr_runtime/engine.py:632-639).
// Temperature sampling is this engine's addition: inverse-CDF over softmax(logits / T) in fp32 with a uniform
// number that depends only on (request seed, index of the output token), never on the row's place in the batch,
// so a request samples the same tokens alone, batched or after recomputation.
#include "common.cuh"

namespace {
constexpr int SAMPLE_THREADS = 256;

// splitmix64 of (seed, counter) -> 24 random bits -> [0, 1)
__device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned int counter) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * ((unsigned long long)counter + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

constexpr int SAMPLE_CHUNK = 2048;   // vocabulary entries per first-pass block

__device__ __forceinline__ float clean(float v) { return (v == v) ? v : -INFINITY; }   // NaN counts as -inf

// (value, index) maximum with the smaller index winning ties, over the block; result in every thread.
__device__ __forceinline__ void block_argmax(float& v, int& i, float* sval, int* sidx) {
    sval[threadIdx.x] = v;
    sidx[threadIdx.x] = i;
    __syncthreads();
    for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = sval[threadIdx.x + s], mv = sval[threadIdx.x];
            const int oi = sidx[threadIdx.x + s], mi = sidx[threadIdx.x];
            if (ov > mv || (ov == mv && oi < mi)) { sval[threadIdx.x] = ov; sidx[threadIdx.x] = oi; }
        }
        __syncthreads();
    }
    v = sval[0];
    i = sidx[0];
    __syncthreads();
}

// Pass 1, grid (chunks, rows): maximum, its first index and sum of exp((x - max) / T) of one chunk of one row.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_partial_kernel(float* __restrict__ part_max, int* __restrict__ part_idx, float* __restrict__ part_sum,
                      const float* __restrict__ logits, int vocab, const float* __restrict__ temperature) {
    __shared__ float sval[SAMPLE_THREADS];
    __shared__ int sidx[SAMPLE_THREADS];
    const int r = blockIdx.y, chunks = gridDim.x, c = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const int lo = c * SAMPLE_CHUNK, hi = min(vocab, lo + SAMPLE_CHUNK);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += SAMPLE_THREADS) {
        const float v = clean(row[i]);
        if (bi == 0x7fffffff || v > bv) { bv = v; bi = i; }
    }
    block_argmax(bv, bi, sval, sidx);
    const float temp = temperature ? temperature[r] : 0.f;
    float sum = 0.f;
    if (temp > 0.f && bv != -INFINITY) {
        const float inv_t = 1.f / temp;
        float part = 0.f;
        for (int i = lo + threadIdx.x; i < hi; i += SAMPLE_THREADS) part += expf((clean(row[i]) - bv) * inv_t);
        sum = block_sum(part, sval);
    }
    if (threadIdx.x == 0) {
        part_max[(size_t)r * chunks + c] = bv;
        part_idx[(size_t)r * chunks + c] = bi;
        part_sum[(size_t)r * chunks + c] = sum;
    }
}

// Pass 2, one block per row: the row's first maximum; with a temperature, the chunk and then the entry in which
// the cumulative probability (taken in index order) passes uniform(seed, counter) * total.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_final_kernel(int* __restrict__ out, const float* __restrict__ part_max, const int* __restrict__ part_idx,
                    const float* __restrict__ part_sum, int chunks, const float* __restrict__ logits, int vocab,
                    const float* __restrict__ temperature, const int* __restrict__ seed_lo, const int* __restrict__ seed_hi,
                    const int* __restrict__ counter) {
    __shared__ float sval[SAMPLE_THREADS];
    __shared__ int sidx[SAMPLE_THREADS];
    __shared__ float s_target;
    __shared__ int s_chunk;
    const int r = blockIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < chunks; c += SAMPLE_THREADS) {   // ascending chunks: ascending indices
        const float v = part_max[(size_t)r * chunks + c];
        const int i = part_idx[(size_t)r * chunks + c];
        if (bi == 0x7fffffff || v > bv) { bv = v; bi = i; }
    }
    block_argmax(bv, bi, sval, sidx);
    const int greedy = bi == 0x7fffffff ? 0 : bi;
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 0.f) || bv == -INFINITY) {
        if (threadIdx.x == 0) out[r] = greedy;
        return;
    }
    const float inv_t = 1.f / temp, M = bv;
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int c = 0; c < chunks; ++c) {
            const float cm = part_max[(size_t)r * chunks + c];
            if (cm != -INFINITY) total += part_sum[(size_t)r * chunks + c] * expf((cm - M) * inv_t);
        }
        const unsigned long long seed = ((unsigned long long)(unsigned int)seed_hi[r] << 32) | (unsigned int)seed_lo[r];
        const float target = uniform_from(seed, (unsigned int)counter[r]) * total;
        float run = 0.f;
        int pick = chunks - 1;
        for (int c = 0; c < chunks; ++c) {
            const float cm = part_max[(size_t)r * chunks + c];
            const float w = cm != -INFINITY ? part_sum[(size_t)r * chunks + c] * expf((cm - M) * inv_t) : 0.f;
            if (run + w > target) { pick = c; break; }
            run += w;
        }
        s_chunk = pick;
        s_target = target - run;   // what is left to pass inside the chosen chunk
    }
    __syncthreads();
    const float* row = logits + (size_t)r * vocab;
    const int lo = s_chunk * SAMPLE_CHUNK, hi = min(vocab, lo + SAMPLE_CHUNK);
    constexpr int PER = SAMPLE_CHUNK / SAMPLE_THREADS;   // contiguous entries per thread
    const int a = min(hi, lo + (int)threadIdx.x * PER), b = min(hi, a + PER);
    float mine = 0.f;
    for (int i = a; i < b; ++i) mine += expf((clean(row[i]) - M) * inv_t);
    sval[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float run = 0.f;
        int owner = -1;
        for (int t = 0; t < SAMPLE_THREADS; ++t) {
            if (run + sval[t] > s_target) { owner = t; break; }
            run += sval[t];
        }
        int pick = -1, last_pos = -1;
        if (owner >= 0) {
            const int oa = min(hi, lo + owner * PER), ob = min(hi, oa + PER);
            for (int i = oa; i < ob; ++i) {
                const float p = expf((clean(row[i]) - M) * inv_t);
                if (p > 0.f) last_pos = i;
                run += p;
                if (run > s_target) { pick = i; break; }
            }
        }
        if (pick < 0) {   // rounding left the target just beyond the sums: the last entry with any probability
            if (last_pos < 0)
                for (int i = hi - 1; i >= lo; --i)
                    if (expf((clean(row[i]) - M) * inv_t) > 0.f) { last_pos = i; break; }
            pick = last_pos >= 0 ? last_pos : greedy;
        }
        out[r] = pick;
    }
}

__global__ void repetition_penalty_kernel(float* __restrict__ logits, const unsigned char* __restrict__ seen,
                                          const int* __restrict__ row_slot, const float* __restrict__ penalty, int vocab) {
    const int r = blockIdx.y;
    const float p = penalty[r];
    if (p == 1.f) return;
    const unsigned char* mask = seen + (size_t)row_slot[r] * vocab;
    float* row = logits + (size_t)r * vocab;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        if (mask[i]) {
            const float v = row[i];
            row[i] = v > 0.f ? v / p : v * p;
        }
    }
}

__global__ void mark_seen_kernel(unsigned char* __restrict__ seen, const int* __restrict__ slots,
                                 const int* __restrict__ tokens, int n, int vocab) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const int tok = tokens[i];
        if (tok >= 0 && tok < vocab) seen[(size_t)slots[i] * vocab + tok] = 1;
    }
}
}  // namespace

OXR_API int oxr_sample_chunks(int vocab) { return (vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK; }

// logits: fp32 [rows, vocab]. temperature / seed_lo / seed_hi / counter: per row; temperature may be null (all
// greedy). scratch: 3 * rows * oxr_sample_chunks(vocab) 4-byte words, overwritten.
OXR_API int oxr_sample(int* out, const float* logits, int rows, int vocab, const float* temperature, const int* seed_lo,
                       const int* seed_hi, const int* counter, void* scratch, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || scratch == nullptr || rows > 65535) return OXR_BAD_ARGUMENT;
    const int chunks = (vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    float* part_max = (float*)scratch;
    int* part_idx = (int*)scratch + (size_t)rows * chunks;
    float* part_sum = (float*)scratch + 2 * (size_t)rows * chunks;
    sample_partial_kernel<<<dim3(chunks, rows), SAMPLE_THREADS, 0, stream>>>(part_max, part_idx, part_sum, logits, vocab, temperature);
    int rc = oxr_launch_status();
    if (rc) return rc;
    sample_final_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(out, part_max, part_idx, part_sum, chunks, logits, vocab, temperature,
                                                            seed_lo, seed_hi, counter);
    return oxr_launch_status();
}

OXR_API int oxr_repetition_penalty(float* logits, const unsigned char* seen, const int* row_slot, const float* penalty,
                                   int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return 0;
    dim3 grid((vocab + 1023) / 1024 < 64 ? (vocab + 1023) / 1024 : 64, rows);
    repetition_penalty_kernel<<<grid, 256, 0, stream>>>(logits, seen, row_slot, penalty, vocab);
    return oxr_launch_status();
}

OXR_API int oxr_mark_seen(unsigned char* seen, const int* slots, const int* tokens, int n, int vocab, cudaStream_t stream) {
    if (n <= 0) return 0;
    mark_seen_kernel<<<(n + 255) / 256, 256, 0, stream>>>(seen, slots, tokens, n, vocab);
    return oxr_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------------
// oxr_sample_static: the same two passes with the scratch in a static device array (see sampling_static.h).
// ---------------------------------------------------------------------------------------------------------------------
#include <stdio.h>

#include "sampling_static.h"

static_assert(OXR_SAMPLE_STATIC_CHUNK == SAMPLE_CHUNK, "the header states the chunk size of the first pass");

// Partial results of the first pass: [rows * chunks] maxima, then indices, then sums. Device memory of this
// library image; in host code the name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned int oxr_sample_static_scratch[OXR_SAMPLE_STATIC_WORDS];

namespace {
constexpr int MAX_DEVICES = 64;
void* g_static_scratch[MAX_DEVICES];   // device address of the array on each device, looked up at first use

int fail(int code, char* msg, int cap, const char* text) {
    if (msg != nullptr && cap > 0) snprintf(msg, (size_t)cap, "%s", text);
    return code;
}
}  // namespace

int oxr_sample_static(int* out_tokens, const float* logits, int rows, int vocab, const float* temperature, const int* seed_lo,
                      const int* seed_hi, const int* counter, cudaStream_t stream, char* error_message, int error_capacity) {
    char text[256];
    if (out_tokens == nullptr || logits == nullptr || rows <= 0 || vocab <= 0 || rows > 65535)
        return fail(OXR_SAMPLE_STATIC_BAD_ARGUMENT, error_message, error_capacity,
                    "oxr_sample_static: out_tokens and logits must be device pointers, 1 <= rows <= 65535, vocab >= 1");
    if (temperature != nullptr && (seed_lo == nullptr || seed_hi == nullptr || counter == nullptr))
        return fail(OXR_SAMPLE_STATIC_BAD_ARGUMENT, error_message, error_capacity,
                    "oxr_sample_static: seed_lo, seed_hi and counter are required when a temperature is given");
    const long long chunks = ((long long)vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    const long long words = 3LL * rows * chunks;
    if (words > OXR_SAMPLE_STATIC_WORDS) {
        snprintf(text, sizeof(text),
                 "oxr_sample_static: %d rows x %lld chunks of %d entries need %lld words of scratch, the static array holds %d "
                 "(rows * ceil(vocab / %d) must not exceed %d); use oxr_sample with caller-provided scratch",
                 rows, chunks, SAMPLE_CHUNK, words, OXR_SAMPLE_STATIC_WORDS, SAMPLE_CHUNK, OXR_SAMPLE_STATIC_WORDS / 3);
        return fail(OXR_SAMPLE_STATIC_TOO_LARGE, error_message, error_capacity, text);
    }
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
        snprintf(text, sizeof(text), "oxr_sample_static: cudaGetDevice gave device %d (%s)", device, cudaGetErrorString(e));
        return fail(OXR_SAMPLE_STATIC_SETUP_FAILED, error_message, error_capacity, text);
    }
    if (g_static_scratch[device] == nullptr) {
        // once per device, with that device current: the array's address there
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, oxr_sample_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            snprintf(text, sizeof(text), "oxr_sample_static: cudaGetSymbolAddress failed on device %d: %s", device,
                     cudaGetErrorString(e));
            return fail(OXR_SAMPLE_STATIC_SETUP_FAILED, error_message, error_capacity, text);
        }
        g_static_scratch[device] = ptr;
    }
    void* scratch = g_static_scratch[device];
    float* part_max = (float*)scratch;
    int* part_idx = (int*)scratch + (size_t)rows * chunks;
    float* part_sum = (float*)scratch + 2 * (size_t)rows * chunks;
    sample_partial_kernel<<<dim3((unsigned)chunks, rows), SAMPLE_THREADS, 0, stream>>>(part_max, part_idx, part_sum, logits, vocab,
                                                                                        temperature);
    e = cudaGetLastError();
    if (e == cudaSuccess) {
        sample_final_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(out_tokens, part_max, part_idx, part_sum, (int)chunks, logits, vocab,
                                                                temperature, seed_lo, seed_hi, counter);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        snprintf(text, sizeof(text), "oxr_sample_static: kernel launch failed: %s", cudaGetErrorString(e));
        return fail(1000 + (int)e, error_message, error_capacity, text);
    }
    return 0;
}
