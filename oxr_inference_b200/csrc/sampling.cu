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

// first index of the row maximum (NaN counts as -inf); every thread returns it
__device__ int block_argmax(const float* __restrict__ row, int vocab, float* best_val, int* smem_idx, float* smem_val) {
    constexpr int EMPTY = 0x7fffffff;
    float bv = -INFINITY;
    int bi = EMPTY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {   // ascending i: a strict '>' keeps the first index
        float v = row[i];
        if (!(v == v)) v = -INFINITY;
        if (bi == EMPTY || v > bv) { bv = v; bi = i; }
    }
    smem_val[threadIdx.x] = bv;
    smem_idx[threadIdx.x] = bi;
    __syncthreads();
    for (int s = blockDim.x >> 1; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = smem_val[threadIdx.x + s], mv = smem_val[threadIdx.x];
            const int oi = smem_idx[threadIdx.x + s], mi = smem_idx[threadIdx.x];
            if (ov > mv || (ov == mv && oi < mi)) {
                smem_val[threadIdx.x] = ov;
                smem_idx[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    const int idx = smem_idx[0];
    *best_val = smem_val[0];
    __syncthreads();
    return idx == EMPTY ? 0 : idx;
}

// One block per row. temperature[r] <= 0 -> greedy.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ seed_lo, const int* __restrict__ seed_hi, const int* __restrict__ counter) {
    __shared__ float sval[SAMPLE_THREADS];
    __shared__ int sidx[SAMPLE_THREADS];
    __shared__ int chosen;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    float vmax;
    const int greedy = block_argmax(row, vocab, &vmax, sidx, sval);
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 0.f)) {
        if (threadIdx.x == 0) out[r] = greedy;
        return;
    }
    const float inv_t = 1.f / temp;
    // contiguous segment per thread so that the cumulative sum runs in index order
    const int seg = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int lo = min(vocab, (int)threadIdx.x * seg), hi = min(vocab, lo + seg);
    float part = 0.f;
    for (int i = lo; i < hi; ++i) part += expf((row[i] - vmax) * inv_t);
    sval[threadIdx.x] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int k = 0; k < SAMPLE_THREADS; ++k) total += sval[k];
        const unsigned long long seed = ((unsigned long long)(unsigned int)seed_hi[r] << 32) | (unsigned int)seed_lo[r];
        const float target = uniform_from(seed, (unsigned int)counter[r]) * total;
        float run = 0.f;
        int k = 0;
        for (; k < SAMPLE_THREADS - 1; ++k) {
            if (run + sval[k] > target) break;
            run += sval[k];
        }
        const int a = min(vocab, k * seg), b = min(vocab, a + seg);
        int pick = -1, last_pos = -1;
        for (int i = a; i < b; ++i) {
            const float p = expf((row[i] - vmax) * inv_t);
            if (p > 0.f) last_pos = i;
            run += p;
            if (run > target) { pick = i; break; }
        }
        if (pick < 0) pick = last_pos >= 0 ? last_pos : greedy;   // rounding left the target just beyond the segment
        chosen = pick;
        out[r] = chosen;
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

// logits: fp32 [rows, vocab]. temperature / seed_lo / seed_hi / counter: per row; temperature may be null (all greedy).
OXR_API int oxr_sample(int* out, const float* logits, int rows, int vocab, const float* temperature, const int* seed_lo,
                       const int* seed_hi, const int* counter, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return OXR_BAD_ARGUMENT;
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(out, logits, vocab, temperature, seed_lo, seed_hi, counter);
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
