/* oxr_sample_static: next-token choice without any device-memory allocation.
 *
 * This entry point has no counterpart in the reference (NickWilde18/oxr-inference samples with torch's argmax on
 * tensors that torch allocates). It exists for callers that must not allocate device memory when they sample:
 *   - a host program that embeds this library through its C symbols and has handed all device memory to another
 *     runtime's pool at start-up, so that a cudaMalloc from here would fail or fragment that pool;
 *   - a serving loop with a hard latency bound that forbids allocator calls (and the implicit synchronisation a
 *     cudaMalloc / cudaFree can cause) after warm-up;
 *   - code that runs between other frameworks' kernels on a stream and may not touch their caching allocators.
 * The regular entry point, oxr_sample, takes its scratch memory from the caller (the Python wrapper gets it from
 * torch's allocator on every call); this one keeps the scratch inside the library.
 *
 * What it computes is exactly what oxr_sample computes: for each row of fp32 logits [rows, vocab], the first
 * maximum where temperature[row] <= 0 (or temperature == NULL), else a draw from softmax(logits / temperature)
 * decided by (seed, counter) of that row alone. The caller passes inputs and outputs as device pointers.
 *
 * Scratch: the per-(row, vocabulary chunk) partial results of the first pass live in a file-scope
 * `static __device__` array of OXR_SAMPLE_STATIC_WORDS 4-byte words (768 KiB), which every GPU that loads the
 * library holds until the process exits. A call needs 3 * rows * ceil(vocab / 2048) words; a call that needs more
 * is refused with OXR_SAMPLE_STATIC_TOO_LARGE and a message, and launches nothing.
 *
 * First call on a device: the entry point looks the array's device address up once per device (the device that is
 * current at the call) and remembers it. That first call on each device should be made before any stream capture
 * begins, since an address lookup is not a stream operation.
 *
 * Sharing: all calls on a device use the same array. The array keeps the previous call's contents; nothing in it
 * has to start at zero, because the second pass reads only words that the first pass of the same call wrote. Two
 * calls whose kernels can overlap on the GPU (different streams without an ordering between them, or two host
 * threads) race on the array and give wrong tokens: order such calls on one stream or with events.
 *
 * It calls no cudaMalloc, cudaFree, or any library routine that allocates (none of torch's either).
 *
 * Returns 0 on success. On failure returns a non-zero code and, when error_message != NULL, writes a
 * NUL-terminated explanation of at most error_capacity bytes there.
 */
#pragma once

#include <cuda_runtime.h>

#define OXR_SAMPLE_STATIC_WORDS (3 * 65536)      /* 4-byte words of scratch held per GPU: 768 KiB */
#define OXR_SAMPLE_STATIC_CHUNK 2048             /* vocabulary entries per chunk of the first pass */
#define OXR_SAMPLE_STATIC_TOO_LARGE 200          /* rows * chunks exceeds what the static scratch holds */
#define OXR_SAMPLE_STATIC_BAD_ARGUMENT 201       /* null pointer, non-positive sizes, more than 65535 rows */
#define OXR_SAMPLE_STATIC_SETUP_FAILED 202       /* the scratch array's address could not be looked up */

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default")))
int oxr_sample_static(int* out_tokens,            /* [rows] int32, device */
                      const float* logits,        /* [rows, vocab] fp32, device */
                      int rows, int vocab,
                      const float* temperature,   /* [rows] or NULL (all greedy), device */
                      const int* seed_lo,         /* [rows] low 32 bits of each row's seed (with a temperature) */
                      const int* seed_hi,         /* [rows] high 32 bits */
                      const int* counter,         /* [rows] index of the output token being drawn */
                      cudaStream_t stream,
                      char* error_message, int error_capacity);

#ifdef __cplusplus
}
#endif
