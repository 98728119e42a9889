// Hyper-connections (mHC): the residual stream of a V4-style decoder is S = 4 parallel streams [T, 4, H].  At every sub-layer
// boundary the streams are
//   closed   res'[d] = post[d] * sub + sum_s comb[s][d] * res[s]          (sub: the sub-layer's output, post / comb from its opening)
//   opened   24 projections of the flattened, RMS-normalised 4H row (fn [24, 4H]) give, per token,
//              pre [4]  = sigmoid(p * scale0 + base) + 1e-6                (how the streams collapse into the sub-layer's input)
//              post[4]  = 2 sigmoid(p * scale1 + base)                     (how its output spreads back)
//              comb[16] = Sinkhorn(softmax rows of (p * scale2 + base))    (stream-to-stream mix, doubly stochastic after 20 sweeps)
//            y = sum_s pre[s] * res'[s], handed on as y and as rmsnorm(y) * w.
// One kernel does close + open + collapse + norm for a token: the CTA stages the token's 4H row in shared memory (57 KB at H = 7168),
// so the residual crosses HBM once in and once out per boundary, and the coefficients never leave the chip between the projections
// and their use.  The first boundary of a step spreads the embedding over the streams (`init`), the last one opens with 4
// projections only (the head's collapse).  Large steps put two rows in a CTA so that fn is fetched from L2 once per two tokens.
//
// Reference: native/families/deepseek_v41/cuda/v41_hc.cu (pre / post / mixes as separate kernels; `mhc_pre`, `mhc_post_pre`,
// `mhc_head` programs of the V4 families fuse them with RMSNorm).
#include "common.cuh"

#define MHC_S 4
#define MHC_THREADS 256

struct MhcArgs {
  bf16* res;             // [T, 4, H] residual streams, updated in place
  const bf16* sub;       // [T, H] sub-layer output to close with (or the embedding rows when init), null: nothing to close
  const float* coef_in;  // [T, 20] post[4], comb[16] of the boundary being closed
  const float* fn;       // [n_proj, 4H]
  const float* scale;    // [3]
  const float* base;     // [n_proj]
  const float* norm_w;   // [H]
  bf16* y_raw;           // [T, H] collapsed input (optional)
  bf16* y_norm;          // [T, H] rmsnorm(y) * norm_w
  float* coef_out;       // [T, 20] post, comb of this boundary (null when n_proj == 4)
  int T, H, n_proj, init, iters;
  float eps;
};

template <int R>
__global__ void __launch_bounds__(MHC_THREADS) mhc_boundary_kernel(const MhcArgs a) {
  pdl_launch(); pdl_wait();
  extern __shared__ __align__(16) unsigned char mhc_smem[];
  bf16* xs = (bf16*)mhc_smem;                                  // [R][4][H]
  __shared__ float red[8][R * 25];
  __shared__ float coef[R][28];                                // pre[4], post[4], comb[16], inv rms, 1 / rms(y)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, H = a.H, W = MHC_S * H;
  const int row0 = blockIdx.x * R;

  // ---- close the previous boundary (or spread the embedding), stage the row, sum of squares
  float sq[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    sq[r] = 0.f;
    const int t = row0 + r;
    if (t >= a.T) continue;
    bf16* g = a.res + (size_t)t * W;
    bf16* x = xs + (size_t)r * W;
    float post[4], comb[16];
    if (a.sub && !a.init) {
#pragma unroll
      for (int i = 0; i < 4; ++i) post[i] = a.coef_in[(size_t)t * 20 + i];
#pragma unroll
      for (int i = 0; i < 16; ++i) comb[i] = a.coef_in[(size_t)t * 20 + 4 + i];
    }
    for (int c = tid * 8; c < H; c += MHC_THREADS * 8) {
      uint4 v[4];
      if (a.sub) {
        const uint4 sv = *(const uint4*)(a.sub + (size_t)t * H + c);
        if (a.init) {
#pragma unroll
          for (int d = 0; d < 4; ++d) v[d] = sv;
        } else {
          uint4 rv[4];
#pragma unroll
          for (int s = 0; s < 4; ++s) rv[s] = *(const uint4*)(g + (size_t)s * H + c);
          const bf16* se = (const bf16*)&sv;
#pragma unroll
          for (int d = 0; d < 4; ++d) {
            bf16* o = (bf16*)&v[d];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float acc = post[d] * __bfloat162float(se[j]);
#pragma unroll
              for (int s = 0; s < 4; ++s) acc = fmaf(comb[s * 4 + d], __bfloat162float(((const bf16*)&rv[s])[j]), acc);
              o[j] = __float2bfloat16(acc);
            }
          }
        }
#pragma unroll
        for (int d = 0; d < 4; ++d) *(uint4*)(g + (size_t)d * H + c) = v[d];
      } else {
#pragma unroll
        for (int d = 0; d < 4; ++d) v[d] = *(const uint4*)(g + (size_t)d * H + c);
      }
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        *(uint4*)(x + (size_t)d * H + c) = v[d];
        const bf16* e = (const bf16*)&v[d];
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float f = __bfloat162float(e[j]); sq[r] = fmaf(f, f, sq[r]); }
      }
    }
  }
  __syncthreads();

  // ---- projections of the staged rows: every thread walks the 4H row in float4 steps, fn comes from L2
  const int P = a.n_proj;
  float dot[R][24];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int p = 0; p < 24; ++p) dot[r][p] = 0.f;
  for (int c = tid * 4; c < W; c += MHC_THREADS * 4) {
    float xv[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint2 q = *(const uint2*)(xs + (size_t)r * W + c);
      const bf16* e = (const bf16*)&q;
#pragma unroll
      for (int j = 0; j < 4; ++j) xv[r][j] = __bfloat162float(e[j]);
    }
#pragma unroll
    for (int p = 0; p < 24; ++p) {
      if (p < P) {
        const float4 f = *(const float4*)(a.fn + (size_t)p * W + c);
#pragma unroll
        for (int r = 0; r < R; ++r)
          dot[r][p] = fmaf(xv[r][3], f.w, fmaf(xv[r][2], f.z, fmaf(xv[r][1], f.y, fmaf(xv[r][0], f.x, dot[r][p]))));
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int p = 0; p < 24; ++p) {
      if (p < P) { const float v = warp_sum(dot[r][p]); if (lane == 0) red[warp][r * 25 + p] = v; }
    }
    const float v = warp_sum(sq[r]);
    if (lane == 0) red[warp][r * 25 + 24] = v;
  }
  __syncthreads();

  // ---- coefficients: warp r finishes row r (lanes 0..23 own one projection each; lanes 0..15 then own one comb entry)
  if (warp < R && row0 + warp < a.T) {
    const int r = warp, t = row0 + r;
    float ss = 0.f, pj = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { ss += red[w][r * 25 + 24]; if (lane < P) pj += red[w][r * 25 + lane]; }
    const float inv = rsqrtf(ss / (float)W + 1e-20f);
    pj *= inv;
    if (lane < 4) coef[r][lane] = 1.f / (1.f + __expf(-fmaf(pj, a.scale[0], a.base[lane]))) + 1e-6f;
    if (P == 24) {
      if (lane >= 4 && lane < 8) coef[r][lane] = 2.f / (1.f + __expf(-fmaf(pj, a.scale[1], a.base[lane])));
      // comb entry e = source * 4 + destination sits in lane e: fetch projection 8 + e from lane 8 + e
      const float raw = __shfl_sync(0xffffffffu, fmaf(pj, a.scale[2], lane < 24 ? a.base[lane] : 0.f), (lane + 8) & 31);
      float v = lane < 16 ? raw : 0.f;
      float m = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      v = __expf(v - m);
      float s = v + __shfl_xor_sync(0xffffffffu, v, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      v = v / s + 1e-6f;                                         // softmax over the destinations of one source
      for (int it = 0; it < a.iters; ++it) {
        if (it) {                                                // rows (over destinations)
          s = v + __shfl_xor_sync(0xffffffffu, v, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          v /= s + 1e-6f;
        }
        s = v + __shfl_xor_sync(0xffffffffu, v, 4);              // columns (over sources)
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        v /= s + 1e-6f;
      }
      if (lane < 16) coef[r][8 + lane] = v;
      __syncwarp();
      if (a.coef_out && lane < 20) a.coef_out[(size_t)t * 20 + lane] = coef[r][4 + lane];
    }
  }
  __syncthreads();

  // ---- collapse, RMSNorm
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int t = row0 + r;
    float ysq = 0.f;
    const bf16* x = xs + (size_t)r * W;
    const float p0 = coef[r][0], p1 = coef[r][1], p2 = coef[r][2], p3 = coef[r][3];
    if (t < a.T) {
      for (int c = tid * 8; c < H; c += MHC_THREADS * 8) {
        const uint4 v0 = *(const uint4*)(x + c), v1 = *(const uint4*)(x + H + c), v2 = *(const uint4*)(x + 2 * H + c), v3 = *(const uint4*)(x + 3 * H + c);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float y = p0 * __bfloat162float(((const bf16*)&v0)[j]) + p1 * __bfloat162float(((const bf16*)&v1)[j]) +
                          p2 * __bfloat162float(((const bf16*)&v2)[j]) + p3 * __bfloat162float(((const bf16*)&v3)[j]);
          ysq = fmaf(y, y, ysq);
        }
      }
    }
    const float tot = block_sum(ysq, &red[0][0]);
    if (t >= a.T) continue;
    const float inv = rsqrtf(tot / (float)H + a.eps);
    for (int c = tid * 8; c < H; c += MHC_THREADS * 8) {
      const uint4 v0 = *(const uint4*)(x + c), v1 = *(const uint4*)(x + H + c), v2 = *(const uint4*)(x + 2 * H + c), v3 = *(const uint4*)(x + 3 * H + c);
      uint4 raw, nrm;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float y = p0 * __bfloat162float(((const bf16*)&v0)[j]) + p1 * __bfloat162float(((const bf16*)&v1)[j]) +
                        p2 * __bfloat162float(((const bf16*)&v2)[j]) + p3 * __bfloat162float(((const bf16*)&v3)[j]);
        ((bf16*)&raw)[j] = __float2bfloat16(y);
        ((bf16*)&nrm)[j] = __float2bfloat16(y * inv * a.norm_w[c + j]);
      }
      if (a.y_raw) *(uint4*)(a.y_raw + (size_t)t * H + c) = raw;
      *(uint4*)(a.y_norm + (size_t)t * H + c) = nrm;
    }
  }
}

// ---------------------------------------------------------------- decode-sized steps: one 8-CTA cluster per token
// A token's boundary is a chain of two full-row reductions (projections + sum of squares, then the collapsed row's sum of squares), so
// one CTA per token leaves a few dozen CTAs walking 24 x 4H weights each: latency-bound.  Here a thread-block cluster of 8 CTAs owns the
// token: CTA q holds columns [q H/8, (q+1) H/8) of all four streams, the partial sums cross the cluster through distributed shared
// memory (every CTA adds the 8 partials in rank order, so all of them hold the same coefficients), and each CTA collapses and
// normalises its own columns.
#define MHC_CL 8

__device__ __forceinline__ uint32_t mhc_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void mhc_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float mhc_ld_peer(const float* p, uint32_t rank) {
  uint32_t local = (uint32_t)__cvta_generic_to_shared(p), remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__global__ void __launch_bounds__(MHC_THREADS) mhc_boundary_cluster_kernel(const MhcArgs a) {
  pdl_launch(); pdl_wait();
  extern __shared__ __align__(16) unsigned char mhc_smem[];
  bf16* xs = (bf16*)mhc_smem;                                  // [4][Hc]
  __shared__ float red[8][25];
  __shared__ float part[25], part2[1];
  __shared__ float coef[24];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, H = a.H, Hc = H / MHC_CL;
  const uint32_t q = mhc_cluster_rank();
  const int t = blockIdx.y, c0 = (int)q * Hc, P = a.n_proj;
  bf16* g = a.res + (size_t)t * MHC_S * H;

  float sq = 0.f;
  {
    float post[4], comb[16];
    if (a.sub && !a.init) {
#pragma unroll
      for (int i = 0; i < 4; ++i) post[i] = a.coef_in[(size_t)t * 20 + i];
#pragma unroll
      for (int i = 0; i < 16; ++i) comb[i] = a.coef_in[(size_t)t * 20 + 4 + i];
    }
    for (int c = tid * 8; c < Hc; c += MHC_THREADS * 8) {
      uint4 v[4];
      if (a.sub) {
        const uint4 sv = *(const uint4*)(a.sub + (size_t)t * H + c0 + c);
        if (a.init) {
#pragma unroll
          for (int d = 0; d < 4; ++d) v[d] = sv;
        } else {
          uint4 rv[4];
#pragma unroll
          for (int s = 0; s < 4; ++s) rv[s] = *(const uint4*)(g + (size_t)s * H + c0 + c);
          const bf16* se = (const bf16*)&sv;
#pragma unroll
          for (int d = 0; d < 4; ++d) {
            bf16* o = (bf16*)&v[d];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float acc = post[d] * __bfloat162float(se[j]);
#pragma unroll
              for (int s = 0; s < 4; ++s) acc = fmaf(comb[s * 4 + d], __bfloat162float(((const bf16*)&rv[s])[j]), acc);
              o[j] = __float2bfloat16(acc);
            }
          }
        }
#pragma unroll
        for (int d = 0; d < 4; ++d) *(uint4*)(g + (size_t)d * H + c0 + c) = v[d];
      } else {
#pragma unroll
        for (int d = 0; d < 4; ++d) v[d] = *(const uint4*)(g + (size_t)d * H + c0 + c);
      }
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        *(uint4*)(xs + (size_t)d * Hc + c) = v[d];
        const bf16* e = (const bf16*)&v[d];
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float f = __bfloat162float(e[j]); sq = fmaf(f, f, sq); }
      }
    }
  }
  __syncthreads();

  // partial projections over my columns: item i = (stream, 4 columns)
  float dot[24];
#pragma unroll
  for (int p = 0; p < 24; ++p) dot[p] = 0.f;
  const int per = Hc / 4;
  for (int i = tid; i < MHC_S * per; i += MHC_THREADS) {
    const int s = i / per, c = (i - s * per) * 4;
    const uint2 qv = *(const uint2*)(xs + (size_t)s * Hc + c);
    const bf16* e = (const bf16*)&qv;
    const float x0 = __bfloat162float(e[0]), x1 = __bfloat162float(e[1]), x2 = __bfloat162float(e[2]), x3 = __bfloat162float(e[3]);
    const float* f0 = a.fn + (size_t)s * H + c0 + c;
#pragma unroll
    for (int p = 0; p < 24; ++p) {
      if (p < P) {
        const float4 f = *(const float4*)(f0 + (size_t)p * MHC_S * H);
        dot[p] = fmaf(x3, f.w, fmaf(x2, f.z, fmaf(x1, f.y, fmaf(x0, f.x, dot[p]))));
      }
    }
  }
#pragma unroll
  for (int p = 0; p < 24; ++p) {
    if (p < P) { const float v = warp_sum(dot[p]); if (lane == 0) red[warp][p] = v; }
  }
  {
    const float v = warp_sum(sq);
    if (lane == 0) red[warp][24] = v;
  }
  __syncthreads();
  if (tid < 25) {
    float v = 0.f;
    if (tid < P || tid == 24) {
#pragma unroll
      for (int w = 0; w < 8; ++w) v += red[w][tid];
    }
    part[tid] = v;
  }
  mhc_cluster_sync();                                            // every CTA's partials are visible to the cluster

  if (warp == 0) {
    float ss = 0.f, pj = 0.f;
#pragma unroll
    for (uint32_t r = 0; r < MHC_CL; ++r) { ss += mhc_ld_peer(&part[24], r); if (lane < P) pj += mhc_ld_peer(&part[lane], r); }
    const float inv = rsqrtf(ss / (float)(MHC_S * H) + 1e-20f);
    pj *= inv;
    if (lane < 4) coef[lane] = 1.f / (1.f + __expf(-fmaf(pj, a.scale[0], a.base[lane]))) + 1e-6f;
    if (P == 24) {
      if (lane >= 4 && lane < 8) coef[lane] = 2.f / (1.f + __expf(-fmaf(pj, a.scale[1], a.base[lane])));
      const float raw = __shfl_sync(0xffffffffu, fmaf(pj, a.scale[2], lane < 24 ? a.base[lane] : 0.f), (lane + 8) & 31);
      float v = lane < 16 ? raw : 0.f;
      float m = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      v = __expf(v - m);
      float s = v + __shfl_xor_sync(0xffffffffu, v, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      v = v / s + 1e-6f;
      for (int it = 0; it < a.iters; ++it) {
        if (it) {
          s = v + __shfl_xor_sync(0xffffffffu, v, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          v /= s + 1e-6f;
        }
        s = v + __shfl_xor_sync(0xffffffffu, v, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        v /= s + 1e-6f;
      }
      if (lane < 16) coef[8 + lane] = v;
      __syncwarp();
      if (q == 0 && a.coef_out && lane < 20) a.coef_out[(size_t)t * 20 + lane] = coef[4 + lane];
    }
  }
  __syncthreads();

  // collapse my columns, exchange the sums of squares, normalise
  const float p0 = coef[0], p1 = coef[1], p2 = coef[2], p3 = coef[3];
  float ysq = 0.f;
  for (int c = tid * 8; c < Hc; c += MHC_THREADS * 8) {
    const uint4 v0 = *(const uint4*)(xs + c), v1 = *(const uint4*)(xs + Hc + c), v2 = *(const uint4*)(xs + 2 * Hc + c), v3 = *(const uint4*)(xs + 3 * Hc + c);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float y = p0 * __bfloat162float(((const bf16*)&v0)[j]) + p1 * __bfloat162float(((const bf16*)&v1)[j]) +
                      p2 * __bfloat162float(((const bf16*)&v2)[j]) + p3 * __bfloat162float(((const bf16*)&v3)[j]);
      ysq = fmaf(y, y, ysq);
    }
  }
  const float mine = block_sum(ysq, &red[0][0]);
  if (tid == 0) part2[0] = mine;
  mhc_cluster_sync();
  float tot = 0.f;
#pragma unroll
  for (uint32_t r = 0; r < MHC_CL; ++r) tot += mhc_ld_peer(&part2[0], r);
  const float inv = rsqrtf(tot / (float)H + a.eps);
  for (int c = tid * 8; c < Hc; c += MHC_THREADS * 8) {
    const uint4 v0 = *(const uint4*)(xs + c), v1 = *(const uint4*)(xs + Hc + c), v2 = *(const uint4*)(xs + 2 * Hc + c), v3 = *(const uint4*)(xs + 3 * Hc + c);
    uint4 raw, nrm;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float y = p0 * __bfloat162float(((const bf16*)&v0)[j]) + p1 * __bfloat162float(((const bf16*)&v1)[j]) +
                      p2 * __bfloat162float(((const bf16*)&v2)[j]) + p3 * __bfloat162float(((const bf16*)&v3)[j]);
      ((bf16*)&raw)[j] = __float2bfloat16(y);
      ((bf16*)&nrm)[j] = __float2bfloat16(y * inv * a.norm_w[c0 + c + j]);
    }
    if (a.y_raw) *(uint4*)(a.y_raw + (size_t)t * H + c0 + c) = raw;
    *(uint4*)(a.y_norm + (size_t)t * H + c0 + c) = nrm;
  }
  mhc_cluster_sync();                                            // nobody leaves while a peer may still read its partials
}

static int mhc_launch_cluster(const MhcArgs& a, cudaStream_t s) {
  const size_t smem = (size_t)MHC_S * (a.H / MHC_CL) * sizeof(bf16);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(MHC_CL, a.T); cfg.blockDim = dim3(MHC_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = MHC_CL; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = ca_pdl_enabled(CA_PDL_CLASS) ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, mhc_boundary_cluster_kernel, a);
  if (e != cudaSuccess) return ca_cuda(e, "mhc_boundary_cluster launch");
  return CA_OK;
}

extern "C" int cuteafd_mhc_boundary(void* res, const void* sub, const float* coef_in, const float* fn, const float* scale, const float* base,
                                    const float* norm_w, void* y_raw, void* y_norm, float* coef_out, int T, int H, int n_proj, int init, int iters,
                                    float eps, cudaStream_t s) {
  CA_REQUIRE(res && fn && scale && base && norm_w && y_norm, "mhc_boundary: null argument");
  CA_REQUIRE(H >= 8 && H % 8 == 0 && H <= 14336, "mhc_boundary: hidden size must be a multiple of 8, at most 14336");
  CA_REQUIRE(n_proj == 24 || n_proj == 4, "mhc_boundary: 24 projections (pre, post, comb) or 4 (pre only)");
  CA_REQUIRE(n_proj == 4 || coef_out, "mhc_boundary: an opening with post / comb needs coef_out");
  CA_REQUIRE(init || !sub || coef_in, "mhc_boundary: closing a boundary needs its coefficients");
  CA_REQUIRE(!init || sub, "mhc_boundary: init spreads `sub` over the streams");
  CA_REQUIRE(iters >= 1 && iters <= 64, "mhc_boundary: 1..64 Sinkhorn sweeps");
  if (T <= 0) return CA_OK;
  MhcArgs a;
  a.res = (bf16*)res; a.sub = (const bf16*)sub; a.coef_in = coef_in; a.fn = fn; a.scale = scale; a.base = base; a.norm_w = norm_w;
  a.y_raw = (bf16*)y_raw; a.y_norm = (bf16*)y_norm; a.coef_out = coef_out; a.T = T; a.H = H; a.n_proj = n_proj; a.init = init; a.iters = iters;
  a.eps = eps;
  if (T <= 256 && H % (MHC_CL * 8) == 0) {      // decode / verify sized steps: a cluster per token
    int rc = mhc_launch_cluster(a, s);
    if (rc != CA_OK) return rc;
    CA_CHECK_LAUNCH("mhc_boundary_cluster");
    return CA_OK;
  }
  const size_t row_bytes = (size_t)MHC_S * H * sizeof(bf16);
  const bool two = T > 512 && 2 * row_bytes <= 200 * 1024;
  const size_t smem = (two ? 2 : 1) * row_bytes;
  if (two) {
    cudaError_t e = cudaFuncSetAttribute(mhc_boundary_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ca_cuda(e, "mhc_boundary: shared memory size");
    CA_LAUNCH_PDL(mhc_boundary_kernel<2>, (T + 1) / 2, MHC_THREADS, smem, s, a);
  } else {
    cudaError_t e = cudaFuncSetAttribute(mhc_boundary_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ca_cuda(e, "mhc_boundary: shared memory size");
    CA_LAUNCH_PDL(mhc_boundary_kernel<1>, T, MHC_THREADS, smem, s, a);
  }
  CA_CHECK_LAUNCH("mhc_boundary");
  return CA_OK;
}
