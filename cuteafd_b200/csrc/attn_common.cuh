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

// Same merge, eight output elements per thread, optionally also writing the merged row quantised to FP4 for the
// output projection that follows (qkind 1 NVFP4 / 2 MXFP4; needs Hq * D % 256 == 0).  grid (T, ceil(Hq * D / 8 / 128)).
static __global__ void attn_merge8_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ sink,
                                          bf16* __restrict__ out, int T, int Hq, int D, int n_splits, uint8_t* __restrict__ q,
                                          uint8_t* __restrict__ sf, int ldsf, const float* __restrict__ inv_gs_ptr, int qkind) {
  pdl_launch(); pdl_wait();
  const int t = blockIdx.x, vi = blockIdx.y * blockDim.x + threadIdx.x, vpr = D / 8;
  if (vi >= Hq * vpr) return;                     // whole warps leave together (Hq * D / 8 is a multiple of 32 with FP4 output)
  const int h = vi / vpr, d0 = (vi % vpr) * 8;
  // Up to eight splits at a time, every load issued before the first use: the (m, l) pairs and the partial rows of all splits are
  // in flight together (a loop that reads m, branches, then loads the row is one L2 round trip per split on a decode step's
  // critical path).  Partial rows of empty splits (m = -inf) are loaded but not used; the buffers always cover every split.
  const float sk = sink ? sink[h] : -INFINITY;
  float M = sk, L = 0.f;
  float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s0 = 0; s0 < n_splits; s0 += 8) {
    float2 ml[8]; float4 pa[8], pb[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = min(s0 + j, n_splits - 1);
      const size_t row = ((size_t)s * T + t) * Hq + h;
      ml[j] = *(const float2*)(part_ml + row * 2);
      const float4* po = (const float4*)(part_o + row * D + d0);
      pa[j] = po[0]; pb[j] = po[1];
    }
    float Mn = M;
#pragma unroll
    for (int j = 0; j < 8; ++j) if (s0 + j < n_splits) Mn = fmaxf(Mn, ml[j].x);
    if (s0 == 0) {
      if (sink) L = __expf(sk - Mn);                  // the sink's share first, as the one-pass form adds it
    } else if (Mn != M && M != -INFINITY) {           // a later batch raised the maximum: rescale what was accumulated
      const float r = __expf(M - Mn);
      L *= r;
#pragma unroll
      for (int q = 0; q < 8; ++q) o[q] *= r;
    }
    M = Mn;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s0 + j < n_splits && ml[j].x != -INFINITY) {
        const float e = __expf(ml[j].x - M);
        L += ml[j].y * e;
        o[0] += pa[j].x * e; o[1] += pa[j].y * e; o[2] += pa[j].z * e; o[3] += pa[j].w * e;
        o[4] += pb[j].x * e; o[5] += pb[j].y * e; o[6] += pb[j].z * e; o[7] += pb[j].w * e;
      }
    }
  }

  const float inv = L > 0.f ? 1.f / L : 0.f;
  bf16 ob[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16(o[j] * inv);
  *(uint4*)(out + ((size_t)t * Hq + h) * D + d0) = *(uint4*)ob;
  if (qkind) {
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(ob[j]);
    quant8_store(f, qkind, inv_gs_ptr ? *inv_gs_ptr : 1.f, q + (size_t)t * (Hq * D / 2), sf + (size_t)t * ldsf, h * D + d0);
  }
}

static __global__ void attn_fill_ml_kernel(float* ml, long long n) {
  pdl_launch(); pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ml[i] = (i & 1) ? 0.f : -INFINITY;
}

