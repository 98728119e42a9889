// Split-KV partial merge shared by the SIMT and the tensor-core paged attention kernels.
#pragma once
#include "common.cuh"

// Merge split partials: out = sum_s o_s * exp(m_s - M) / sum_s l_s * exp(m_s - M)  (+ sink term).
// Splits that saw no key carry m = -inf, l = 0 and drop out.  Partials of rows a split never touched are
// ignored through the `valid` test on m.
static __global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ sink,
                                  bf16* __restrict__ out, int T, int Hq, int D, int n_splits) {
  pdl_launch(); pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  float M = sink ? sink[h] : -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(((size_t)s * T + t) * Hq + h) * 2]);
  float L = sink ? __expf(sink[h] - M) : 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float* ml = part_ml + (((size_t)s * T + t) * Hq + h) * 2;
    if (ml[0] != -INFINITY) L += ml[1] * __expf(ml[0] - M);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float m = part_ml[(((size_t)s * T + t) * Hq + h) * 2];
      if (m != -INFINITY) o += part_o[(((size_t)s * T + t) * Hq + h) * D + d] * __expf(m - M);
    }
    out[((size_t)t * Hq + h) * D + d] = __float2bfloat16(L > 0.f ? o / L : 0.f);
  }
}

static __global__ void attn_fill_ml_kernel(float* ml, long long n) {
  pdl_launch(); pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ml[i] = (i & 1) ? 0.f : -INFINITY;
}

