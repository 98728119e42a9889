// KV page movement between the paged device store and a slab pool, and L2 prefetch of a weight range.
//
// The device store is [layers][slots][row bytes]; a page is `page_bytes` contiguous bytes per layer.  A slab of the
// pool holds one page of every layer back to back ([layers][page_bytes]).  The pool is either device memory (a
// staging buffer for one bulk copy) or pinned host memory mapped into the device address space, in which case the
// kernel itself moves the bytes over PCIe: one launch per batch of pages instead of one strided copy per page.
//
// Reference counterparts: native/shared/cuda/kv_cache.cu (block read / write), paged_staging_gather_* used by
// cuteafd-engine/src/prefix/cuda_copy.rs, and native/shared/cuda/l2_prefetch.cu.
#include "common.cuh"

// pairs[i] = {device page, slab}; dir 0: page -> slab, 1: slab -> page.  grid = (pairs, layers).
__global__ void kv_pages_copy_kernel(uint8_t* __restrict__ kv, long long layer_stride, int page_bytes, const int2* __restrict__ pairs,
                                     uint8_t* __restrict__ pool, long long slab_stride, int dir) {
  const int2 pr = pairs[blockIdx.x];
  const int layer = blockIdx.y;
  uint4* dev = (uint4*)(kv + (size_t)layer * layer_stride + (size_t)pr.x * page_bytes);
  uint4* slab = (uint4*)(pool + (size_t)pr.y * slab_stride + (size_t)layer * page_bytes);
  const uint4* src = dir ? slab : dev;
  uint4* dst = dir ? dev : slab;
  const int n = page_bytes >> 4;
  // four independent 16-byte loads in flight per thread: the slab side may be on the far side of PCIe
  int i = threadIdx.x;
  for (; i + 3 * (int)blockDim.x < n; i += 4 * blockDim.x) {
    const uint4 a = src[i], b = src[i + blockDim.x], c = src[i + 2 * blockDim.x], d = src[i + 3 * blockDim.x];
    dst[i] = a; dst[i + blockDim.x] = b; dst[i + 2 * blockDim.x] = c; dst[i + 3 * blockDim.x] = d;
  }
  for (; i < n; i += blockDim.x) dst[i] = src[i];
}

extern "C" int cuteafd_kv_pages_copy(void* kv, long long layer_stride, int n_layers, int page_bytes, const int* pairs, int n_pairs, void* pool,
                                     long long slab_stride, int dir, cudaStream_t s) {
  CA_REQUIRE(page_bytes % 16 == 0 && layer_stride % 16 == 0 && slab_stride % 16 == 0, "kv_pages_copy: sizes must be multiples of 16 bytes");
  CA_REQUIRE(slab_stride >= (long long)n_layers * page_bytes, "kv_pages_copy: slab smaller than one page of every layer");
  CA_REQUIRE(n_layers > 0 && n_layers <= 65535, "kv_pages_copy: bad layer count");
  if (n_pairs <= 0) return CA_OK;
  kv_pages_copy_kernel<<<dim3(n_pairs, n_layers), 256, 0, s>>>((uint8_t*)kv, layer_stride, page_bytes, (const int2*)pairs, (uint8_t*)pool, slab_stride, dir);
  CA_CHECK_LAUNCH("kv_pages_copy");
  return CA_OK;
}

// Asks the memory system to bring [p, p + bytes) into L2 (no data reaches the SM).  One thread per 16 KB piece.
#define PF_CHUNK 16384
__global__ void l2_prefetch_kernel(const uint8_t* __restrict__ p, long long bytes) {
  const long long off = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * PF_CHUNK;
  if (off >= bytes) return;
  const uint32_t n = (uint32_t)min((long long)PF_CHUNK, bytes - off) & ~15u;
  if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + off), "r"(n) : "memory");
}

extern "C" int cuteafd_l2_prefetch(const void* p, long long bytes, cudaStream_t s) {
  CA_REQUIRE(((uintptr_t)p & 15) == 0, "l2_prefetch: pointer must be 16-byte aligned");
  if (bytes <= 0) return CA_OK;
  const long long chunks = (bytes + PF_CHUNK - 1) / PF_CHUNK;
  l2_prefetch_kernel<<<(int)((chunks + 127) / 128), 128, 0, s>>>((const uint8_t*)p, bytes);
  CA_CHECK_LAUNCH("l2_prefetch");
  return CA_OK;
}
