/* Allocation-free entry point of libprism_kernels.
 *
 * This entry point has no counterpart in andre-fu/prism.  It exists for
 * callers that are not allowed to allocate device memory at the moment they
 * need attention: code that runs while another component owns the whole
 * memory budget of the GPU, a real-time loop that must not enter the
 * driver's allocator, or a host program that holds no allocator at all and
 * only has the buffers it was handed.  Such a caller cannot provide the
 * scratch buffers that the split-KV decode attention needs for its partial
 * results, so this variant keeps them in a fixed array inside the library.
 *
 * What it computes is exactly prism_attention_decode_bf16 (attention_bf16.cu):
 * one new token per request over a paged bf16 K/V cache; see that file for
 * the meaning of every argument.  The caller still passes inputs and outputs.
 *
 * Limits and rules:
 *   - The scratch is PRISM_NOALLOC_SCRATCH_BYTES (4 MiB) of device memory that
 *     every GPU which loads the library holds until the process exits.  A call
 *     needs T * nh * nsplit * (hd + 2) floats; a larger call is refused with
 *     cudaErrorInvalidValue (1) and prism_noalloc_last_error() says why.
 *   - It calls no cudaMalloc, cudaFree or any library routine that allocates.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress) and remembers it; make that first call before any
 *     stream capture begins on that device.
 *   - All calls share the one array and it keeps the previous call's contents.
 *     Nothing in it has to start at zero: every partial result a call reads was
 *     written by that same call.  Two calls whose kernels overlap on the GPU
 *     (different streams, no ordering between them) race on the array; order
 *     them, or use the allocating entry point with buffers of your own.
 */
#ifndef PRISM_NOALLOC_H
#define PRISM_NOALLOC_H

#include <cuda_runtime.h>

#define PRISM_NOALLOC_SCRATCH_BYTES (4u << 20)

#ifdef __cplusplus
extern "C" {
#endif

/* Returns a cudaError_t as int (0 = launched). */
int prism_attention_decode_bf16_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                        const void* k_cache, const void* v_cache,
                                        const int* block_table, int bt_width, const int* positions,
                                        const int* tok_seg, int T, int nh, int nkv, int hd,
                                        int page_size, int num_pages, int window, float scale,
                                        int nsplit, int* err, cudaStream_t stream);

/* Text of the last refusal or set-up failure of the entry point above ("" if none). */
const char* prism_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
