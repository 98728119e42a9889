/* Allocation-free split-KV paged attention.
 *
 * This entry point has no counterpart in the reference project: it exists for callers of this library that are
 * not allowed to allocate device memory at the moment they need attention - for example code running inside a
 * stream capture or a latency-critical serving loop where cudaMalloc would synchronise the device, or a host
 * that hands this library a fixed memory budget and forbids it from growing.  The ordinary entry point
 * (`cuteafd_paged_attention`) makes its caller provide scratch buffers for the split-KV partial results; this
 * one keeps that scratch inside the library instead.
 *
 * How it works and what to know:
 *   - The partial outputs (per split: unnormalised O, running max, running sum) live in one file-scope
 *     `static __device__` array of CUTEAFD_NOALLOC_SCRATCH_FLOATS floats (8 MiB).  Every GPU that loads the
 *     library carries that array until the process exits, whether or not this function is ever called.
 *   - A call needs n_splits * T * Hq * (D + 2) floats; a larger request is refused with an argument error
 *     (nothing is launched).  The function never calls cudaMalloc, cudaFree or any allocating library routine.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress) and caches it.
 *     Make that first call outside of any stream capture.
 *   - All calls share the one array and it keeps whatever the previous call left there; the per-split
 *     (max, sum) pairs are re-initialised on every call before the attention kernel runs.  Two calls whose
 *     kernels can overlap on the GPU (different streams, no ordering between them) would race on the array:
 *     keep calls on one stream or order them with events.
 *   - Inputs, outputs and semantics are exactly those of `cuteafd_paged_attention` (same kernels); only the two
 *     scratch pointers are gone.
 */
#pragma once
#include <cuda_runtime.h>

#define CUTEAFD_NOALLOC_SCRATCH_FLOATS (2u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int cuteafd_paged_attention_noalloc(const void* q, const void* kv, const int* page_table, const int* kv_len,
                                    const int* q_start, const int* q_len, const float* sink, void* out, int T, int n_seq,
                                    int max_q_len, int q_stride, int Hq, int Hkv, int D, int max_pages, int n_splits,
                                    int window, float scale, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
