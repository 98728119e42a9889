// Mixture-of-experts control kernels: router selection, route packing into expert order (with the
// tile table the grouped tcgen05 GEMM walks), and the ordered weighted combine (+ shared expert +
// residual) with fp32 accumulation in slot order and a single bf16 rounding.
// Reference counterparts: native/shared/cuda/expert_router.cu:73-171 (select kernels),
// route_reduce.cu:30-125 (ordered reduce), residual.cu:419-498 (scatter-add / combine + residual).
#include "common.cuh"

enum { SCORE_SIGMOID = 0, SCORE_SOFTMAX = 1, SCORE_SQRTSOFTPLUS = 2 };

// One block per token.  logits fp32 [T, E] (E <= 512).  Selection uses score + bias (bias may be null),
// optional group-limited routing (top `topk_group` of `n_group` groups ranked by the sum of their two
// best biased scores); gate weights come from the unbiased scores, normalised over the chosen k and
// multiplied by route_scale.  Ties resolve to the lowest expert id.
__global__ void router_select_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ idx,
                                     float* __restrict__ wts, int E, int k, int scoring, int normalize, float route_scale,
                                     int n_group, int topk_group) {
  pdl_launch(); pdl_wait();
  __shared__ float score[512], choice[512], red[32];
  __shared__ float gscore[32];
  __shared__ int sel[16];
  __shared__ float selw[16];
  const int t = blockIdx.x, tid = threadIdx.x;
  const float* lg = logits + (size_t)t * E;
  float mx = -INFINITY;
  for (int e = tid; e < E; e += blockDim.x) mx = fmaxf(mx, lg[e]);
  float denom = 1.f;
  if (scoring == SCORE_SOFTMAX) {
    mx = block_max(mx, red);
    float s = 0.f;
    for (int e = tid; e < E; e += blockDim.x) s += expf(lg[e] - mx);
    denom = block_sum(s, red);
  }
  for (int e = tid; e < E; e += blockDim.x) {
    const float x = lg[e];
    float sc;
    if (scoring == SCORE_SIGMOID) sc = 1.f / (1.f + expf(-x));
    else if (scoring == SCORE_SOFTMAX) sc = expf(x - mx) / denom;
    else sc = sqrtf(x > 20.f ? x : log1pf(expf(x)));
    score[e] = sc;
    choice[e] = sc + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (n_group > 1 && topk_group < n_group) {
    const int per = E / n_group;
    if (tid < n_group) {
      float a = -INFINITY, b = -INFINITY;
      for (int j = 0; j < per; ++j) { const float v = choice[tid * per + j]; if (v > a) { b = a; a = v; } else if (v > b) b = v; }
      gscore[tid] = a + b;
    }
    __syncthreads();
    if (tid == 0) {
      // keep the best topk_group groups (stable: lowest group id first among equals)
      unsigned keep = 0;
      for (int r = 0; r < topk_group; ++r) {
        int best = -1; float bv = -INFINITY;
        for (int g = 0; g < n_group; ++g) if (!(keep >> g & 1) && (best < 0 || gscore[g] > bv)) { best = g; bv = gscore[g]; }
        keep |= 1u << best;
      }
      for (int g = 0; g < n_group; ++g) if (!(keep >> g & 1)) gscore[g] = -INFINITY; else gscore[g] = 0.f;
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) if (gscore[e / per] != 0.f) choice[e] = -INFINITY;
    __syncthreads();
  }
  // k rounds of block-wide argmax (value desc, index asc)
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int e = tid; e < E; e += blockDim.x) { const float v = choice[e]; if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    __shared__ float wv[32]; __shared__ int wi[32];
    if ((tid & 31) == 0) { wv[tid >> 5] = bv; wi[tid >> 5] = bi; }
    __syncthreads();
    if (tid == 0) {
      const int nw = (blockDim.x + 31) >> 5;
      for (int j = 1; j < nw; ++j) if (wv[j] > bv || (wv[j] == bv && wi[j] < bi)) { bv = wv[j]; bi = wi[j]; }
      if (bi >= E) bi = 0;
      sel[r] = bi; selw[r] = score[bi]; choice[bi] = -INFINITY;
    }
    __syncthreads();
  }
  if (tid == 0) {
    float s = 0.f;
    for (int r = 0; r < k; ++r) s += selw[r];
    const float inv = normalize ? 1.f / fmaxf(s, 1e-12f) : 1.f;
    for (int r = 0; r < k; ++r) { idx[(size_t)t * k + r] = sel[r]; wts[(size_t)t * k + r] = selw[r] * inv * route_scale; }
  }
}

extern "C" int cuteafd_router_select(const float* logits, const float* bias, int* idx, float* wts, int T, int E, int k,
                                     int scoring, int normalize, float route_scale, int n_group, int topk_group, cudaStream_t s) {
  CA_REQUIRE(E >= k && E <= 512 && k >= 1 && k <= 16, "router_select: need k <= 16 and E <= 512 (E=%d k=%d)", E, k);
  CA_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0, "router_select: bad group count");
  if (T <= 0) return CA_OK;
  const int threads = E <= 64 ? 64 : (E <= 128 ? 128 : 256);
  CA_LAUNCH_PDL(router_select_kernel, T, threads, 0, s, logits, bias, idx, wts, E, k, scoring, normalize, route_scale, n_group, topk_group);
  CA_CHECK_LAUNCH("router_select");
  return CA_OK;
}

// ---------------------------------------------------------------- route packing
// Inputs: idx [T, k] (expert ids; ids outside [e_lo, e_hi) are skipped - they belong to another expert rank).
// Outputs: src_token [cap]  (token of each packed row, expert-major), slot_row [T, k] (packed row of each
// route, -1 when skipped), counts/offsets per local expert, a tile table {local expert, first row, rows, 0}
// with at most `tn` rows per entry, n_tiles and n_rows.  Single block; T*k up to ~64K routes.
__global__ void route_pack_kernel(const int* __restrict__ idx, int* __restrict__ src_token, int* __restrict__ slot_row,
                                  int* __restrict__ counts, int* __restrict__ offsets, int4* __restrict__ tiles,
                                  int* __restrict__ n_tiles, int* __restrict__ n_rows, int T, int k, int e_lo, int e_hi, int tn,
                                  int max_tiles, int* __restrict__ src_route) {
  pdl_launch(); pdl_wait();
  extern __shared__ int sh[];   // [E_local] counts, [E_local] offsets/cursors
  const int El = e_hi - e_lo;
  int* cnt = sh; int* cur = sh + El;
  for (int e = threadIdx.x; e < El; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int n = T * k;
  for (int i = threadIdx.x; i < n; i += blockDim.x) { const int e = idx[i] - e_lo; if (e >= 0 && e < El) atomicAdd(&cnt[e], 1); }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < El; ++e) {
      cur[e] = off; offsets[e] = off; counts[e] = cnt[e];
      for (int r = 0; r < cnt[e]; r += tn) { if (nt < max_tiles) tiles[nt] = make_int4(e, off + r, min(tn, cnt[e] - r), 0); ++nt; }
      off += cnt[e];
    }
    *n_tiles = min(nt, max_tiles); *n_rows = off;
  }
  __syncthreads();
  // Stable placement (token order inside each expert) so packed layouts are reproducible: one thread per expert
  // walks the routes in order when T*k is small; larger batches use atomics (row order inside an expert does
  // not change any result: rows are independent in the GEMM and the combine reads them by index).
  if (n <= 4096) {
    // rank of route i inside its expert = number of earlier routes to the same expert (ids staged in shared memory)
    int* sid = cur + El;
    for (int i = threadIdx.x; i < n; i += blockDim.x) sid[i] = idx[i] - e_lo;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int e = sid[i];
      if (e < 0 || e >= El) { slot_row[i] = -1; continue; }
      int rank = 0;
      for (int j = 0; j < i; ++j) rank += (sid[j] == e);
      const int c = cur[e] + rank;
      src_token[c] = i / k; slot_row[i] = c;
      if (src_route) src_route[c] = i;
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int e = idx[i] - e_lo;
      if (e >= 0 && e < El) { const int c = atomicAdd(&cur[e], 1); src_token[c] = i / k; slot_row[i] = c; if (src_route) src_route[c] = i; } else slot_row[i] = -1;
    }
  }
}

extern "C" int cuteafd_route_pack(const int* idx, int* src_token, int* slot_row, int* counts, int* offsets, void* tiles,
                                  int* n_tiles, int* n_rows, int T, int k, int e_lo, int e_hi, int tn, int max_tiles, int* src_route, cudaStream_t s) {
  CA_REQUIRE(e_hi > e_lo && e_hi - e_lo <= 4096, "route_pack: bad expert range");
  CA_REQUIRE(tn >= 1, "route_pack: bad tile rows");
  CA_LAUNCH_PDL(route_pack_kernel, 1, 1024, (2 * (e_hi - e_lo) + (T * k <= 4096 ? T * k : 0)) * sizeof(int), s, idx, src_token, slot_row, counts, offsets, (int4*)tiles,
                                                                    n_tiles, n_rows, T, k, e_lo, e_hi, tn, max_tiles, src_route);
  CA_CHECK_LAUNCH("route_pack");
  return CA_OK;
}

// ---------------------------------------------------------------- ordered weighted combine
// out[t] = residual[t] + shared[t] + sum_{slot} w[t,slot] * y[slot_row[t,slot]]   (fp32, slot order, one rounding).
// residual / shared may be null; routes with slot_row < 0 are skipped.
__global__ void moe_combine_kernel(const bf16* __restrict__ y, const int* __restrict__ slot_row, const float* __restrict__ wts,
                                   const bf16* __restrict__ shared, const bf16* __restrict__ residual, bf16* __restrict__ out,
                                   int H, int k) {
  pdl_launch(); pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int sl = 0; sl < k; ++sl) {
      const int r = slot_row[(size_t)t * k + sl];
      if (r < 0) continue;
      const float w = wts[(size_t)t * k + sl];
      uint4 q = *(const uint4*)(y + (size_t)r * H + i);
      const bf16* e = (const bf16*)&q;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += w * __bfloat162float(e[j]);
    }
    if (shared) { uint4 q = *(const uint4*)(shared + (size_t)t * H + i); const bf16* e = (const bf16*)&q;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(e[j]); }
    if (residual) { uint4 q = *(const uint4*)(residual + (size_t)t * H + i); const bf16* e = (const bf16*)&q;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(e[j]); }
    bf16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16(acc[j]);
    *(uint4*)(out + (size_t)t * H + i) = *(uint4*)o;
  }
}

extern "C" int cuteafd_moe_combine(const void* y, const int* slot_row, const float* wts, const void* shared, const void* residual,
                                   void* out, int T, int H, int k, cudaStream_t s) {
  CA_REQUIRE(H % 8 == 0, "moe_combine: hidden must be a multiple of 8");
  if (T <= 0) return CA_OK;
  const int threads = H / 8 >= 256 ? 256 : (H / 8 >= 128 ? 128 : 64);
  CA_LAUNCH_PDL(moe_combine_kernel, T, threads, 0, s, (const bf16*)y, slot_row, wts, (const bf16*)shared, (const bf16*)residual, (bf16*)out, H, k);
  CA_CHECK_LAUNCH("moe_combine");
  return CA_OK;
}
