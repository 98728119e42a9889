// Token selection on device: greedy argmax (lowest id wins ties, optional allowed-token bitmask, optional
// log-probability), the exact sampling chain  mask -> temperature -> min_p -> top_k -> top_p -> categorical
// with a counter-based uniform that depends only on (seed, position), and greedy speculative verification.
// Reference counterparts: native/shared/cuda/sampling_gpu.cu:238-1701 (exact sampler), token_io.cu:82
// (logits_greedy_f32), sampling.cu:548-903, rust/crates/cuteafd-core/src/dspark_verify.rs:21-69.
#include "common.cuh"

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16; return x;
}
__device__ __forceinline__ float uniform_from(uint64_t seed, uint64_t pos) {
  uint32_t h = mix32((uint32_t)seed ^ 0x9E3779B9u);
  h = mix32(h ^ (uint32_t)(seed >> 32) ^ 0x85EBCA6Bu);
  h = mix32(h ^ (uint32_t)pos ^ 0xC2B2AE35u);
  h = mix32(h ^ (uint32_t)(pos >> 32) ^ 0x27D4EB2Fu);
  return fminf((float)(h >> 8) * (1.0f / 16777216.0f), 0.99999994f);
}
__device__ __forceinline__ bool allowed(const uint32_t* mask, int i) { return !mask || ((mask[i >> 5] >> (i & 31)) & 1u); }

// ---------------------------------------------------------------- greedy
// status[t]: 0 ok, 1 = non-finite logit seen, 2 = mask allows nothing.
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int ld, int V, const uint32_t* __restrict__ masks, int mask_words,
                                   int* __restrict__ tok, float* __restrict__ logprob, int* __restrict__ status) {
  pdl_launch(); pdl_wait();
  __shared__ float sv[32]; __shared__ int si[32]; __shared__ float red[32];
  const int t = blockIdx.x;
  const float* x = logits + (size_t)t * ld;
  const uint32_t* m = masks ? masks + (size_t)t * mask_words : nullptr;
  float bv = -INFINITY; int bi = 0x7fffffff; int bad = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = x[i];
    if (!isfinite(v)) bad = 1;
    if (allowed(m, i) && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  bad = __syncthreads_or(bad);
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    bv = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY; bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) { sv[0] = bv; si[0] = bi; }
  }
  __syncthreads();
  bv = sv[0]; bi = si[0];
  if (threadIdx.x == 0) { tok[t] = bi < V ? bi : 0; if (status) status[t] = bad ? 1 : (bi >= V ? 2 : 0); }
  if (logprob) {
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(x[i] - bv);
    s = block_sum(s, red);
    if (threadIdx.x == 0) logprob[t] = -logf(s);
  }
}

// Large vocabularies with few rows (decode): one block per row leaves most SMs idle and takes ~70 us for 16 x 152k logits.
// Split variant: AM_SPLIT blocks per row scan a slice each and leave (value, index, non-finite) in a scratch slot; the block that
// arrives last on the row's counter reduces the slices (same tie rule: lowest index) and re-arms the counter.
#define AM_SPLIT 8
#define AM_MAX_ROWS 8192
static __device__ float am_val[AM_MAX_ROWS * AM_SPLIT];
static __device__ int am_idx[AM_MAX_ROWS * AM_SPLIT];
static __device__ int am_bad[AM_MAX_ROWS * AM_SPLIT];
static __device__ unsigned int am_cnt[AM_MAX_ROWS];

__global__ void __launch_bounds__(512) argmax_rows_split_kernel(const float* __restrict__ logits, int ld, int V, const uint32_t* __restrict__ masks,
                                                                int mask_words, int* __restrict__ tok, int* __restrict__ status) {
  pdl_launch(); pdl_wait();
  __shared__ float sv[16]; __shared__ int si[16]; __shared__ int is_last;
  const int t = blockIdx.x, part = blockIdx.y;
  const float* x = logits + (size_t)t * ld;
  const uint32_t* m = masks ? masks + (size_t)t * mask_words : nullptr;
  const int per = ((V + AM_SPLIT - 1) / AM_SPLIT + 3) & ~3, i0 = part * per, i1 = min(V, i0 + per);
  float bv = -INFINITY; int bi = 0x7fffffff; int bad = 0;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
    const float v = x[i];
    if (!isfinite(v)) bad = 1;
    if (allowed(m, i) && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  bad = __syncthreads_or(bad);
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    am_val[t * AM_SPLIT + part] = bv; am_idx[t * AM_SPLIT + part] = bi; am_bad[t * AM_SPLIT + part] = bad;
    __threadfence();
    is_last = atomicAdd(&am_cnt[t], 1u) == AM_SPLIT - 1;
  }
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    __threadfence();
    float fv = -INFINITY; int fi = 0x7fffffff, fb = 0;
    for (int p = 0; p < AM_SPLIT; ++p) {
      const float v = __ldcg(&am_val[t * AM_SPLIT + p]); const int i = __ldcg(&am_idx[t * AM_SPLIT + p]);
      fb |= __ldcg(&am_bad[t * AM_SPLIT + p]);
      if (v > fv || (v == fv && i < fi)) { fv = v; fi = i; }
    }
    tok[t] = fi < V ? fi : 0;
    if (status) status[t] = fb ? 1 : (fi >= V ? 2 : 0);
    am_cnt[t] = 0;
  }
}

extern "C" int cuteafd_argmax_rows(const float* logits, int ld, int T, int V, const uint32_t* masks, int mask_words, int* tok,
                                   float* logprob, int* status, cudaStream_t s) {
  if (T <= 0) return CA_OK;
  if (!logprob && V >= 32768 && T <= 256) {      // shares one scratch area: calls on different streams at the same time are not supported
    CA_LAUNCH_PDL(argmax_rows_split_kernel, dim3(T, AM_SPLIT), 512, 0, s, logits, ld, V, masks, mask_words, tok, status);
    CA_CHECK_LAUNCH("argmax_rows_split");
    return CA_OK;
  }
  CA_LAUNCH_PDL(argmax_rows_kernel, T, 1024, 0, s, logits, ld, V, masks, mask_words, tok, logprob, status);
  CA_CHECK_LAUNCH("argmax_rows");
  return CA_OK;
}

// ---------------------------------------------------------------- exact sampler (top_k in [1, 1024])
struct SampleParams {   // 32 bytes per row
  float temperature, top_p, min_p; int top_k;
  uint64_t seed, position;
};

__device__ __forceinline__ uint32_t fkey(float f) {   // monotonic: larger float -> larger key
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

#define KMAX 1024
__global__ void __launch_bounds__(1024) sample_rows_kernel(const float* __restrict__ logits, int ld, int V, const uint32_t* __restrict__ masks,
                                                           int mask_words, const SampleParams* __restrict__ params,
                                                           int* __restrict__ tok, int* __restrict__ status) {
  __shared__ uint32_t hist[256];
  __shared__ float cv[KMAX]; __shared__ int ci[KMAX];
  __shared__ uint32_t s_prefix, s_remaining; __shared__ int s_count, s_ties;
  __shared__ float red[32];
  const int t = blockIdx.x, tid = threadIdx.x;
  const SampleParams P = params[t];
  const float* x = logits + (size_t)t * ld;
  const uint32_t* m = masks ? masks + (size_t)t * mask_words : nullptr;
  const float inv_t = 1.f / fmaxf(P.temperature, 1e-5f);
  // pass 0: max of scaled allowed logits
  float mx = -INFINITY; int bad = 0, any = 0;
  for (int i = tid; i < V; i += blockDim.x) { const float v = x[i]; if (!isfinite(v)) bad = 1; if (allowed(m, i)) { any = 1; mx = fmaxf(mx, v * inv_t); } }
  mx = block_max(mx, red);
  bad = __syncthreads_or(bad); any = __syncthreads_or(any);
  if (!any || bad) { if (tid == 0) { tok[t] = 0; status[t] = bad ? 1 : 2; } return; }
  const float floor_v = P.min_p > 0.f ? mx + logf(P.min_p) : -INFINITY;
  int k = P.top_k; if (k <= 0 || k > KMAX) k = KMAX;
  // radix select of the k-th largest key among survivors (4 passes x 8 bits)
  if (tid == 0) { s_prefix = 0; s_remaining = (uint32_t)k; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int b = tid; b < 256; b += blockDim.x) hist[b] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, pmask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += blockDim.x) {
      const float v = x[i] * inv_t;
      if (!allowed(m, i) || v < floor_v) continue;
      const uint32_t key = fkey(v);
      if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t rem = s_remaining; int b = 255;
      for (; b > 0; --b) { if (hist[b] >= rem) break; rem -= hist[b]; }
      if (hist[b] < rem) rem = hist[b];    // fewer survivors than k: take all
      s_prefix = prefix | ((uint32_t)b << shift); s_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;       // key of the k-th largest survivor (or of the smallest when fewer than k)
  if (tid == 0) { s_count = 0; s_ties = 0; }
  __syncthreads();
  // collect strictly-greater candidates, then ties in ascending id order (block-ordered scan keeps ids sorted)
  for (int i = tid; i < V; i += blockDim.x) {
    const float v = x[i] * inv_t;
    if (!allowed(m, i) || v < floor_v) continue;
    if (fkey(v) > kth) { const int p = atomicAdd(&s_count, 1); if (p < KMAX) { cv[p] = v; ci[p] = i; } }
  }
  __syncthreads();
  const int n_gt = min(s_count, KMAX);
  const int need = min((int)s_remaining, KMAX - n_gt);
  // ties: lowest ids win; walk the vocabulary in chunks so order is by id
  for (int base = 0; base < V && s_ties < need; base += blockDim.x) {
    const int i = base + tid;
    int is_tie = 0;
    if (i < V) { const float v = x[i] * inv_t; is_tie = allowed(m, i) && v >= floor_v && fkey(v) == kth; }
    // rank within the chunk
    const unsigned bal = __ballot_sync(0xffffffffu, is_tie);
    __shared__ int wcount[32];
    if ((tid & 31) == 0) wcount[tid >> 5] = __popc(bal);
    __syncthreads();
    int before = 0;
    for (int w = 0; w < (tid >> 5); ++w) before += wcount[w];
    const int rank = s_ties + before + __popc(bal & ((1u << (tid & 31)) - 1));
    if (is_tie && rank < need) { cv[n_gt + rank] = x[i] * inv_t; ci[n_gt + rank] = i; }
    __syncthreads();
    if (tid == 0) { int tot = 0; for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += wcount[w]; s_ties += tot; }
    __syncthreads();
  }
  const int n = n_gt + min(s_ties, need);
  // bitonic sort of n candidates (padded to a power of two) by (value desc, id asc)
  int np2 = 1; while (np2 < n) np2 <<= 1;
  for (int i = tid; i < np2; i += blockDim.x) if (i >= n) { cv[i] = -INFINITY; ci[i] = 0x7fffffff; }
  __syncthreads();
  for (int sz = 2; sz <= np2; sz <<= 1) {
    for (int st = sz >> 1; st > 0; st >>= 1) {
      for (int i = tid; i < np2; i += blockDim.x) {
        const int j = i ^ st;
        if (j > i) {
          const bool up = (i & sz) == 0;     // first-before-second ordering in this run
          const float a = cv[i], b = cv[j]; const int ia = ci[i], ib = ci[j];
          const bool a_first = a > b || (a == b && ia < ib);
          if (a_first != up) { cv[i] = b; cv[j] = a; ci[i] = ib; ci[j] = ia; }
        }
      }
      __syncthreads();
    }
  }
  if (tid == 0) {
    // sequential fp32 arithmetic in candidate order (the oracle does the same)
    const float x0 = cv[0];
    float sum = 0.f;
    for (int i = 0; i < n; ++i) { cv[i] = expf(cv[i] - x0); sum += cv[i]; }
    int keep = n;
    if (P.top_p < 1.f) {
      float c = 0.f; keep = 0;
      for (int i = 0; i < n; ++i) { c += cv[i] / sum; ++keep; if (!(c < P.top_p)) break; }
      float s2 = 0.f;
      for (int i = 0; i < keep; ++i) s2 += cv[i] / sum;
      sum *= s2;
    }
    const float u = uniform_from(P.seed, P.position);
    float c = 0.f, total = 0.f;
    for (int i = 0; i < keep; ++i) total += cv[i] / sum;
    int pick = keep - 1;
    for (int i = 0; i < keep; ++i) { c += cv[i] / sum; if (c > u * total) { pick = i; break; } }
    tok[t] = ci[pick]; status[t] = 0;
  }
}

extern "C" int cuteafd_sample_rows(const float* logits, int ld, int T, int V, const uint32_t* masks, int mask_words,
                                   const void* params, int* tok, int* status, cudaStream_t s) {
  CA_REQUIRE(params && tok && status, "sample_rows: null argument");
  if (T <= 0) return CA_OK;
  sample_rows_kernel<<<T, 1024, 0, s>>>(logits, ld, V, masks, mask_words, (const SampleParams*)params, tok, status);
  CA_CHECK_LAUNCH("sample_rows");
  return CA_OK;
}

// ---------------------------------------------------------------- greedy speculative verification
// inputs [n_seq, width] = anchor followed by drafts; target [n_seq, width] = target choice after each input row.
// accepted[s] = number of input rows whose KV is kept (>= 1); n_emit[s] = tokens emitted this round
// (target[s, 0 .. n_emit-1]); n_drafts[s] = how many of the drafts are live for this sequence.
__global__ void verify_accept_kernel(const int* __restrict__ inputs, const int* __restrict__ target, const int* __restrict__ n_drafts,
                                     int* __restrict__ accepted, int* __restrict__ n_emit, int n_seq, int width, int eos) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_seq) return;
  const int live = 1 + (n_drafts ? n_drafts[s] : width - 1);
  int acc = 1, emit = 0;
  for (int i = 0; i < live; ++i) {
    const int tk = target[s * width + i];
    ++emit;
    const bool matched = i + 1 < live && inputs[s * width + i + 1] == tk;
    if (matched) ++acc;
    if (!matched || tk == eos) break;
  }
  accepted[s] = acc; n_emit[s] = emit;
}

extern "C" int cuteafd_verify_accept(const int* inputs, const int* target, const int* n_drafts, int* accepted, int* n_emit,
                                     int n_seq, int width, int eos, cudaStream_t s) {
  if (n_seq <= 0) return CA_OK;
  verify_accept_kernel<<<(n_seq + 127) / 128, 128, 0, s>>>(inputs, target, n_drafts, accepted, n_emit, n_seq, width, eos);
  CA_CHECK_LAUNCH("verify_accept");
  return CA_OK;
}
