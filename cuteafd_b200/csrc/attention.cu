// Paged GQA attention (decode, speculative verify and chunked prefill share one kernel) with split-KV
// partials and a log-sum-exp merge.  Queries of a sequence are its last q_len positions; each attends
// causally by absolute position to the sequence's paged K/V (page = 64 tokens).  Optional sliding window
// and per-head attention sink.
//
// Work decomposition: grid = (kv splits, kv heads, sequence x query tile).  A CTA owns up to 16 query rows
// (G heads of the KV group x 16/G tokens), walks its share of 64-key pages, and keeps running max / sum /
// output in shared memory + registers (online softmax).  With more than one split the partial (o, m, l)
// triples go to scratch memory and `attn_merge_kernel` combines them.
//
// Reference counterparts: native/shared/cuda/draft_attention.cu:41-340 (split + merge, window, sink),
// attention.cu:7-87 (causal attention), v41_sparse_attention.cu:304 (LSE merge).
#include "common.cuh"
#include "attn_common.cuh"

#define PAGE 64
#define ROWS 16

struct AttnArgs {
  const bf16* q;            // [T, q_stride] (q heads first)
  const bf16* kv;           // [n_slots, 2, Hkv, D]
  const int* page_table;    // [n_seq, max_pages]
  const int* kv_len;        // [n_seq] context length including the new tokens
  const int* q_start;       // [n_seq] first query row of the sequence
  const int* q_len;         // [n_seq]
  const float* sink;        // [Hq] or null
  bf16* out;                // [T, Hq * D]
  float* part_o;            // [splits, T, Hq, D]
  float* part_ml;           // [splits, T, Hq, 2]
  int q_stride, Hq, Hkv, max_pages, n_splits, window, max_q_tiles, T;
  float scale;
};

template <int D>
__global__ void __launch_bounds__(128) paged_attn_kernel(const AttnArgs a) {
  constexpr int KS = D + 8;                          // padded row stride (bf16) -> conflict-free 16-byte reads
  extern __shared__ uint8_t sm[];
  bf16* sK = (bf16*)sm;                              // [PAGE][KS]
  bf16* sV = sK + PAGE * KS;                         // [PAGE][KS]
  float* sQ = (float*)(sV + PAGE * KS);              // [ROWS][D]
  float* sS = sQ + ROWS * D;                         // [ROWS][PAGE]
  __shared__ float sM[ROWS], sL[ROWS], sAlpha[ROWS];
  __shared__ int sPos[ROWS];

  const int G = a.Hq / a.Hkv;
  const int tok_per_tile = ROWS / G > 0 ? ROWS / G : 1;
  const int split = blockIdx.x, kvh = blockIdx.y;
  const int seq = blockIdx.z / a.max_q_tiles, qt = blockIdx.z % a.max_q_tiles;
  const int qlen = a.q_len[seq], kvlen = a.kv_len[seq];
  const int tok0 = qt * tok_per_tile;
  if (tok0 >= qlen) return;
  const int ntok = min(tok_per_tile, qlen - tok0);
  const int R = ntok * G;                            // live rows: r = tok * G + g
  const int tid = threadIdx.x;
  const int row_base = a.q_start[seq] + tok0;

  for (int i = tid; i < ROWS * D; i += 128) {
    const int r = i / D, d = i % D;
    float v = 0.f;
    if (r < R) v = __bfloat162float(a.q[(size_t)(row_base + r / G) * a.q_stride + (size_t)(kvh * G + r % G) * D + d]) * a.scale;
    sQ[i] = v;
  }
  if (tid < ROWS) { sM[tid] = -INFINITY; sL[tid] = 0.f; sPos[tid] = tid < R ? kvlen - qlen + tok0 + tid / G : -1; }
  __syncthreads();

  // keys visible to this tile: [lo, hi)
  const int max_pos = kvlen - qlen + tok0 + ntok - 1;
  const int hi = max_pos + 1;
  int lo = 0;
  if (a.window > 0) lo = max(0, (kvlen - qlen + tok0) - a.window + 1);
  const int first_page = lo / PAGE, last_page = (hi + PAGE - 1) / PAGE;        // [first, last)
  const int n_pages = last_page - first_page;
  const int per = (n_pages + a.n_splits - 1) / a.n_splits;
  const int p0 = first_page + split * per, p1 = min(last_page, p0 + per);

  constexpr int ACC = ROWS * D / 128;               // accumulators per thread
  constexpr int RSTEP = 128 / D > 0 ? 128 / D : 1;  // rows advance by this between a thread's accumulators
  float acc[ACC];
#pragma unroll
  for (int j = 0; j < ACC; ++j) acc[j] = 0.f;
  const int d_own = tid % D, r_own = tid / D;       // D <= 128

  for (int p = p0; p < p1; ++p) {
    const int page = a.page_table[(size_t)seq * a.max_pages + p];
    const bf16* kbase = a.kv + ((size_t)page * PAGE * 2) * a.Hkv * D + (size_t)kvh * D;
    // load K and V page slices for this kv head: token stride = 2*Hkv*D
    for (int i = tid; i < PAGE * (D / 8); i += 128) {
      const int key = i / (D / 8), c = i % (D / 8);
      const bf16* src = kbase + (size_t)key * 2 * a.Hkv * D + c * 8;
      *(uint4*)(sK + key * KS + c * 8) = *(const uint4*)src;
      *(uint4*)(sV + key * KS + c * 8) = *(const uint4*)(src + (size_t)a.Hkv * D);
    }
    __syncthreads();
    // scores: thread = (key, half of the rows)
    {
      const int key = tid & 63, half = tid >> 6;
      const int kpos = p * PAGE + key;
      float s[ROWS / 2];
#pragma unroll
      for (int j = 0; j < ROWS / 2; ++j) s[j] = 0.f;
      for (int c = 0; c < D / 8; ++c) {
        uint4 kq = *(const uint4*)(sK + key * KS + c * 8);
        const bf16* ke = (const bf16*)&kq;
        float kf[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) kf[e] = __bfloat162float(ke[e]);
#pragma unroll
        for (int j = 0; j < ROWS / 2; ++j) {
          const float* qr = sQ + (half * (ROWS / 2) + j) * D + c * 8;
#pragma unroll
          for (int e = 0; e < 8; ++e) s[j] += qr[e] * kf[e];
        }
      }
#pragma unroll
      for (int j = 0; j < ROWS / 2; ++j) {
        const int r = half * (ROWS / 2) + j;
        const int qp = sPos[r];
        const bool ok = qp >= 0 && kpos <= qp && kpos < kvlen && (a.window <= 0 || kpos > qp - a.window);
        sS[r * PAGE + key] = ok ? s[j] : -INFINITY;
      }
    }
    __syncthreads();
    // online softmax per row: warp w handles rows w, w+4, ...
    {
      const int w = tid >> 5, lane = tid & 31;
      for (int r = w; r < ROWS; r += 4) {
        const float s0 = sS[r * PAGE + lane], s1 = sS[r * PAGE + lane + 32];
        const float mx = warp_max(fmaxf(s0, s1));
        const float m_old = sM[r], m_new = fmaxf(m_old, mx);
        const float p0v = (m_new == -INFINITY) ? 0.f : __expf(s0 - m_new), p1v = (m_new == -INFINITY) ? 0.f : __expf(s1 - m_new);
        const float ps = warp_sum(p0v + p1v);
        sS[r * PAGE + lane] = p0v; sS[r * PAGE + lane + 32] = p1v;
        if (lane == 0) {
          const float al = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
          sAlpha[r] = al; sL[r] = sL[r] * al + ps; sM[r] = m_new;
        }
      }
    }
    __syncthreads();
    // PV: thread owns column d_own for rows r_own + j*RSTEP
#pragma unroll
    for (int j = 0; j < ACC; ++j) acc[j] *= sAlpha[r_own + j * RSTEP];
    for (int key = 0; key < PAGE; ++key) {
      const float v = __bfloat162float(sV[key * KS + d_own]);
#pragma unroll
      for (int j = 0; j < ACC; ++j) acc[j] += sS[(r_own + j * RSTEP) * PAGE + key] * v;
    }
    __syncthreads();
  }

  // write out
#pragma unroll
  for (int j = 0; j < ACC; ++j) {
    const int r = r_own + j * RSTEP;
    if (r >= R) continue;
    const int t = row_base + r / G, h = kvh * G + r % G;
    if (a.n_splits == 1) {
      float l = sL[r], m = sM[r], o = acc[j];
      if (a.sink) {   // sink = one extra logit with zero value
        const float sk = a.sink[h];
        const float m2 = fmaxf(m, sk);
        const float e1 = (m == -INFINITY) ? 0.f : __expf(m - m2);
        l = l * e1 + __expf(sk - m2); o *= e1;
      }
      a.out[(size_t)t * a.Hq * D + (size_t)h * D + d_own] = __float2bfloat16(l > 0.f ? o / l : 0.f);
    } else {
      a.part_o[(((size_t)split * a.T + t) * a.Hq + h) * D + d_own] = acc[j];
      if (d_own == 0) {
        float* ml = a.part_ml + (((size_t)split * a.T + t) * a.Hq + h) * 2;
        ml[0] = sM[r]; ml[1] = sL[r];
      }
    }
  }
}

extern "C" int cuteafd_paged_attention(const void* q, const void* kv, const int* page_table, const int* kv_len, const int* q_start,
                                       const int* q_len, const float* sink, void* out, float* part_o, float* part_ml, int T,
                                       int n_seq, int max_q_len, int q_stride, int Hq, int Hkv, int D, int max_pages, int n_splits,
                                       int window, float scale, cudaStream_t s) {
  CA_REQUIRE(D == 32 || D == 64 || D == 128, "paged_attention: head_dim %d unsupported", D);
  CA_REQUIRE(Hq % Hkv == 0 && Hq / Hkv <= ROWS && ROWS % (Hq / Hkv) == 0, "paged_attention: group size %d unsupported", Hq / Hkv);
  CA_REQUIRE(n_splits >= 1 && (n_splits == 1 || (part_o && part_ml)), "paged_attention: split-KV needs scratch");
  if (T <= 0 || n_seq <= 0) return CA_OK;
  AttnArgs a;
  a.q = (const bf16*)q; a.kv = (const bf16*)kv; a.page_table = page_table; a.kv_len = kv_len; a.q_start = q_start; a.q_len = q_len;
  a.sink = sink; a.out = (bf16*)out; a.part_o = part_o; a.part_ml = part_ml; a.q_stride = q_stride; a.Hq = Hq; a.Hkv = Hkv;
  a.max_pages = max_pages; a.n_splits = n_splits; a.window = window; a.T = T; a.scale = scale;
  const int G = Hq / Hkv, tpt = ROWS / G;
  a.max_q_tiles = (max_q_len + tpt - 1) / tpt;
  dim3 grid(n_splits, Hkv, n_seq * a.max_q_tiles);
  const size_t smem = (size_t)2 * PAGE * (D + 8) * 2 + (size_t)ROWS * D * 4 + (size_t)ROWS * PAGE * 4;
  if (n_splits > 1) {
    const long long n = (long long)n_splits * T * Hq * 2;
    attn_fill_ml_kernel<<<(int)((n + 255) / 256), 256, 0, s>>>(part_ml, n);
  }
  if (D == 32) paged_attn_kernel<32><<<grid, 128, smem, s>>>(a);
  else if (D == 64) paged_attn_kernel<64><<<grid, 128, smem, s>>>(a);
  else paged_attn_kernel<128><<<grid, 128, smem, s>>>(a);
  CA_CHECK_LAUNCH("paged_attention");
  if (n_splits > 1) {
    attn_merge_kernel<<<dim3(T, Hq), D < 128 ? D : 128, 0, s>>>(part_o, part_ml, sink, (bf16*)out, T, Hq, D, n_splits);
    CA_CHECK_LAUNCH("attn_merge");
  }
  return CA_OK;
}

// ---------------------------------------------------------------- allocation-free variant (see no_alloc.h)
#include "no_alloc.h"

// Split-KV scratch owned by the library.  In host code this name is only a stand-in for the symbol, never a
// device address: the address is looked up once per device below and that pointer is what kernels receive.
static __device__ __align__(256) float g_noalloc_scratch[CUTEAFD_NOALLOC_SCRATCH_FLOATS];
static float* g_noalloc_ptr[64] = {nullptr};

extern "C" int cuteafd_paged_attention_noalloc(const void* q, const void* kv, const int* page_table, const int* kv_len,
                                               const int* q_start, const int* q_len, const float* sink, void* out, int T, int n_seq,
                                               int max_q_len, int q_stride, int Hq, int Hkv, int D, int max_pages, int n_splits,
                                               int window, float scale, cudaStream_t stream) {
  CA_REQUIRE(n_splits >= 1 && T >= 0 && Hq > 0 && D > 0, "paged_attention_noalloc: bad shape");
  const unsigned long long n_o = (unsigned long long)n_splits * T * Hq * D, n_ml = (unsigned long long)n_splits * T * Hq * 2;
  if (n_o + n_ml > CUTEAFD_NOALLOC_SCRATCH_FLOATS)
    return ca_fail(CA_ERR_ARG, "paged_attention_noalloc: %llu scratch floats needed (splits %d x rows %d x heads %d x (%d + 2)) but the "
                   "built-in scratch holds %u; use fewer splits or the entry point that takes caller scratch",
                   n_o + n_ml, n_splits, T, Hq, D, (unsigned)CUTEAFD_NOALLOC_SCRATCH_FLOATS);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return ca_cuda(e, "cudaGetDevice");
  CA_REQUIRE(dev >= 0 && dev < 64, "paged_attention_noalloc: device index %d out of range", dev);
  if (!g_noalloc_ptr[dev]) {
    // first call on this device (it is the current device): resolve the symbol to its device address
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return ca_cuda(e, "cudaGetSymbolAddress(scratch)");
    g_noalloc_ptr[dev] = p;
  }
  float* part_o = g_noalloc_ptr[dev];
  float* part_ml = part_o + n_o;
  return cuteafd_paged_attention(q, kv, page_table, kv_len, q_start, q_len, sink, out, part_o, part_ml, T, n_seq, max_q_len,
                                 q_stride, Hq, Hkv, D, max_pages, n_splits, window, scale, stream);
}
