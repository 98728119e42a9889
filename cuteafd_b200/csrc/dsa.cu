// Sparse-attention indexer ("lightning indexer" of the DSA models) and the pieces that turn its selection into an attention
// call: every query token scores every visible cached position with a small multi-head dot product,
//
//     score(t, s) = sum_h w[t, h] * relu(q_idx[t, h, :] . k_idx[s, :])          (Hi index heads of Di = 128 dimensions)
//
// keeps the `topk` best positions, and the latent attention then runs over those rows only.
//
//   dsa_index_scores   tcgen05: a CTA takes 128 cached index keys of one sequence as the M side (TMA from the paged index-key
//                      cache, two pages per tile) and the Hi x q index queries of up to four query tokens as the N side, so the
//                      accumulator holds [key][token, head] and one thread per key folds relu + head weights in registers;
//   dsa_topk           per query row: radix select (4 x 8 bits over order-preserving float keys) of the k-th best score, then an
//                      order-preserving compaction, so the selected positions come out ascending and ties at the threshold
//                      resolve to the lowest positions;
//   dsa_gather_rows    copies the selected rows of a paged cache (latent rows of 576 bf16) into per-query pseudo-pages, over
//                      which the ordinary absorbed attention kernel runs with one "sequence" per query row.
//
// Reference: native/families/deepseek_v41/cuda/v41_index_scores.cu:37 (score definition: relu, head weights, -inf outside the
// causal range), v41_index_topk.cu:25-57 (top-k over paged index keys), v41_sparse_attention.cu:89 (attention over the
// selected rows).  The reference scores one (query, candidate) pair per block with SIMT dot products over FP4 keys; here the
// score matrix is a tensor-core product over bf16 index keys.
#include <string.h>

#define CA_PDL_CLASS 2
#include "common.cuh"

#define DSA_DI 128              // index head dimension
#define DSA_KT 128              // keys per tile
#define DSA_PAGE 64
#define DSA_MAXN 256            // Hi * query tokens per CTA

struct DsaScoreArgs {
  const bf16* q_idx;            // [T, Hi, 128]
  const float* w;               // [T, Hi]
  const CUtensorMap* key_map;   // {128, slots, 1}, box {64, 64, 1}, 128-byte swizzle
  const int* page_table; const int* kv_len; const int* q_start; const int* q_len;
  float* scores;                // [T, ld]
  int* status;
  int Hi, ld, max_pages, tok_per_cta, max_q_blocks;
};

__device__ __forceinline__ uint32_t dsa_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// grid (key tiles, n_seq * max_q_blocks); 192 threads: warp 0 loads, warp 1 issues, warps 2-5 = one thread per key
__global__ void __launch_bounds__(192) dsa_index_scores_kernel(const __grid_constant__ DsaScoreArgs a) {
  pdl_launch(); pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;                    // 2 chunks (64 dims) x [128 keys x 128 B]
  uint8_t* sQ = smem + 32768;            // 2 chunks x [N rows x 128 B], N <= 256
  float* sW = (float*)(smem + 32768 + 65536);     // [N] head weights
  uint64_t* bars = (uint64_t*)(smem + 32768 + 65536 + 1024);
  uint64_t& k_full = bars[0]; uint64_t& s_full = bars[1];
  uint32_t& tmem_slot = *(uint32_t*)(bars + 2);
  int& abort_flag = *(int*)(bars + 3);
  if (smem_u32(smem) & 1023) { if (threadIdx.x == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, 0xD51); return; }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int seq = blockIdx.y / a.max_q_blocks, qb = blockIdx.y % a.max_q_blocks;
  const int qlen = a.q_len[seq], kvlen = a.kv_len[seq];
  const int tok0 = qb * a.tok_per_cta;
  if (tok0 >= qlen) return;
  const int ntok = min(a.tok_per_cta, qlen - tok0);
  const int row_base = a.q_start[seq] + tok0;
  const int first_pos = kvlen - qlen + tok0;                 // position of the first query token of this CTA
  const int key0 = blockIdx.x * DSA_KT;
  if (key0 > first_pos + ntok - 1) {                          // the whole tile lies in every token's future: -inf, no loads
    for (int i = tid; i < ntok * DSA_KT; i += blockDim.x) {
      const int j = i / DSA_KT, c = key0 + i % DSA_KT;
      if (c < a.ld) a.scores[(size_t)(row_base + j) * a.ld + c] = -INFINITY;
    }
    return;
  }
  const int N = ((ntok * a.Hi + 15) / 16) * 16;              // MMA N: a multiple of 16

  if (tid == 0) { mbar_init(&k_full, 1); mbar_init(&s_full, 1); abort_flag = 0; fence_barrier_init(); }
  if (warp == 1) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  // index queries -> two swizzled K-major chunks; rows past ntok * Hi are zero
  for (int i = tid; i < N * 16; i += 192) {
    const int r = i >> 4, c = i & 15;                         // 16-byte unit c (8 dims) of row r = token j, head h
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < ntok * a.Hi) v = *(const uint4*)(a.q_idx + ((size_t)(row_base + r / a.Hi) * a.Hi + r % a.Hi) * DSA_DI + c * 8);
    *(uint4*)(sQ + (c >> 3) * 32768 + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
  }
  for (int i = tid; i < N; i += 192) sW[i] = i < ntok * a.Hi ? a.w[(size_t)(row_base + i / a.Hi) * a.Hi + i % a.Hi] : 0.f;
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&k_full, 32768);
#pragma unroll
      for (int p = 0; p < DSA_KT / DSA_PAGE; ++p) {          // pages past the sequence's table entry hold page 0 (finite rows)
        const int pi = key0 / DSA_PAGE + p;
        const int page = pi < a.max_pages ? a.page_table[(size_t)seq * a.max_pages + pi] : 0;
        tma_load_3d(sK + p * 8192, a.key_map, &k_full, 0, page * DSA_PAGE, 0);
        tma_load_3d(sK + 16384 + p * 8192, a.key_map, &k_full, 64, page * DSA_PAGE, 0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (!mbar_wait_bounded(&k_full, 0, abortp)) ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, (int)blockIdx.x);
    else {
      tc_fence_after();
      if (lane == 0) {
        const uint32_t id = dsa_idesc(N);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16(tmem, umma_desc_sw128(smem_u32(sK) + kb * 16384) + 2 * k, umma_desc_sw128(smem_u32(sQ) + kb * 32768) + 2 * k, id, (kb | k) ? 1u : 0u);
        tc_commit(&s_full);
      }
      __syncwarp();
    }
  } else {
    const int q4 = warp & 3, key = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const bool ok = mbar_wait_bounded(&s_full, 0, abortp);
    if (!ok) ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, (int)blockIdx.x);
    tc_fence_after();
    if (__all_sync(0xffffffffu, ok)) {
      const int pos = key0 + key;
      for (int j = 0; j < ntok; ++j) {                        // token j: columns [j * Hi, (j + 1) * Hi)
        float s = 0.f;
        for (int c0 = 0; c0 < a.Hi; c0 += 16) {              // Hi is a multiple of 16 (checked on the host)
          uint32_t r[16];
          tmem_ld_x16(tmem + lane_addr + j * a.Hi + c0, r);
          tc_wait_ld();
#pragma unroll
          for (int q = 0; q < 16; ++q) s = fmaf(sW[j * a.Hi + c0 + q], fmaxf(__uint_as_float(r[q]), 0.f), s);
        }
        const bool vis = pos <= first_pos + j && pos < kvlen;
        if (pos < a.ld) a.scores[(size_t)(row_base + j) * a.ld + pos] = vis ? s : -INFINITY;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 256);
}

extern "C" int cuteafd_dsa_index_scores(const void* q_idx, const float* w, const void* key_map, const int* page_table, const int* kv_len,
                                        const int* q_start, const int* q_len, float* scores, int T, int n_seq, int max_q_len, int max_kv,
                                        int Hi, int ld, int max_pages, int* status, cudaStream_t s) {
  CA_REQUIRE(q_idx && w && key_map && page_table && kv_len && q_start && q_len && scores, "dsa_index_scores: null argument");
  CA_REQUIRE(Hi >= 16 && Hi % 16 == 0 && Hi <= DSA_MAXN, "dsa_index_scores: index heads must be a multiple of 16, at most %d", DSA_MAXN);
  CA_REQUIRE(ld % 4 == 0 && ld >= ((max_kv + DSA_KT - 1) / DSA_KT) * DSA_KT, "dsa_index_scores: score rows must hold whole key tiles");
  if (T <= 0 || n_seq <= 0 || max_kv <= 0) return CA_OK;
  DsaScoreArgs a;
  a.q_idx = (const bf16*)q_idx; a.w = w; a.key_map = (const CUtensorMap*)key_map; a.page_table = page_table; a.kv_len = kv_len;
  a.q_start = q_start; a.q_len = q_len; a.scores = scores; a.status = status; a.Hi = Hi; a.ld = ld; a.max_pages = max_pages;
  a.tok_per_cta = DSA_MAXN / Hi > 4 ? 4 : DSA_MAXN / Hi;
  a.max_q_blocks = (max_q_len + a.tok_per_cta - 1) / a.tok_per_cta;
  const int smem = 32768 + 65536 + 1024 + 64;
  static bool attr_set[64] = {false};
  int dev = 0; cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(dsa_index_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(dsa_index_scores)");
    attr_set[dev & 63] = true;
  }
  CA_LAUNCH_PDL(dsa_index_scores_kernel, dim3((max_kv + DSA_KT - 1) / DSA_KT, n_seq * a.max_q_blocks), 192, smem, s, a);
  CA_CHECK_LAUNCH("dsa_index_scores");
  return CA_OK;
}

// Descriptor of one layer's paged index-key cache [slots, 128] bf16.
extern "C" int cuteafd_tmap_encode_index_keys(void* out128, const void* base, uint64_t n_slots) {
  CUtensorMap m;
  int rc = ca_encode_tmap_3d(&m, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, DSA_DI, n_slots, 1, DSA_DI * 2, (uint64_t)DSA_DI * 2 * n_slots, 64, DSA_PAGE, 1,
                             CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  memcpy(out128, &m, sizeof(m));
  return CA_OK;
}

// ---------------------------------------------------------------- top-k positions per query row
__device__ __forceinline__ uint32_t dsa_fkey(float f) {     // larger float -> larger key; -inf -> smallest
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One block per query row.  n = n_valid[row] + n_bias leading positions are looked at (with the rows' positions as n_valid and
// n_bias = 1: everything up to and including the row's own position).
// Writes the selected positions ascending into sel[row, 0 .. count) and count into sel_count[row]; entries past count are -1.
__global__ void __launch_bounds__(1024) dsa_topk_kernel(const float* __restrict__ scores, int ld, const int* __restrict__ n_valid, int n_bias, int k,
                                                        int* __restrict__ sel, int* __restrict__ sel_count) {
  pdl_launch(); pdl_wait();
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_remaining;
  __shared__ int warp_gt[32], warp_eq[32];
  __shared__ int base_gt, base_eq;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const float* x = scores + (size_t)row * ld;
  const int n = min(n_valid[row] + n_bias, ld);
  int* out = sel + (size_t)row * k;
  if (n <= k) {                                               // everything visible is selected
    for (int i = tid; i < k; i += blockDim.x) out[i] = i < n ? i : -1;
    if (tid == 0) sel_count[row] = max(n, 0);
    return;
  }
  if (tid == 0) { s_prefix = 0; s_remaining = (uint32_t)k; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int b = tid; b < 256; b += blockDim.x) hist[b] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, pmask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < n; i += blockDim.x) {
      const uint32_t key = dsa_fkey(x[i]);
      if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t rem = s_remaining; int b = 255;
      for (; b > 0; --b) { if (hist[b] >= rem) break; rem -= hist[b]; }
      s_prefix = prefix | ((uint32_t)b << shift); s_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;          // key of the k-th best score
  const int need_eq = (int)s_remaining;   // how many entries equal to it are taken (the lowest positions)
  if (tid == 0) { base_gt = 0; base_eq = 0; }
  __syncthreads();
  // order-preserving compaction, 1024 positions per round: entries above the threshold keep their position order; entries equal to
  // it are numbered in position order and the first `need_eq` of them are taken.  Final order: merge by position is not needed
  // by the consumer, so the "greater" entries come first (ascending), then the "equal" ones (ascending).
  const int n_gt = k - need_eq;
  for (int i0 = 0; i0 < n; i0 += blockDim.x) {
    const int i = i0 + tid;
    const uint32_t key = i < n ? dsa_fkey(x[i]) : 0u;
    const bool gt = i < n && key > kth, eq = i < n && key == kth;
    const uint32_t mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) { warp_gt[wid] = __popc(mg); warp_eq[wid] = __popc(me); }
    __syncthreads();
    int og = base_gt, oe = base_eq;
    for (int wv = 0; wv < wid; ++wv) { og += warp_gt[wv]; oe += warp_eq[wv]; }
    og += __popc(mg & ((1u << lane) - 1u)); oe += __popc(me & ((1u << lane) - 1u));
    if (gt && og < n_gt) out[og] = i;
    if (eq && oe < need_eq) out[n_gt + oe] = i;
    __syncthreads();
    if (tid == 0) {
      int tg = 0, te = 0;
      for (int wv = 0; wv < (int)(blockDim.x >> 5); ++wv) { tg += warp_gt[wv]; te += warp_eq[wv]; }
      base_gt += tg; base_eq += te;
    }
    __syncthreads();
  }
  if (tid == 0) sel_count[row] = k;
}

extern "C" int cuteafd_dsa_topk(const float* scores, int ld, const int* n_valid, int rows, int k, int n_bias, int* sel, int* sel_count,
                                cudaStream_t s) {
  CA_REQUIRE(scores && n_valid && sel && sel_count && k >= 1, "dsa_topk: bad arguments");
  if (rows <= 0) return CA_OK;
  CA_LAUNCH_PDL(dsa_topk_kernel, rows, 1024, 0, s, scores, ld, n_valid, n_bias, k, sel, sel_count);
  CA_CHECK_LAUNCH("dsa_topk");
  return CA_OK;
}

// ---------------------------------------------------------------- gather of selected cache rows into per-query pseudo-pages
// dst[(row * kp + j), :] = cache[page_table[seq_of_row[row]][sel[row][j] / 64] * 64 + sel[row][j] % 64, :] for j < sel_count[row];
// row_bytes is a multiple of 16.  Entries of dst past sel_count[row] are left as they are (the attention masks them by length).
__global__ void dsa_gather_rows_kernel(const uint4* __restrict__ cache, const int* __restrict__ page_table, const int* __restrict__ seq_of_row,
                                       const int* __restrict__ sel, const int* __restrict__ sel_count, uint4* __restrict__ dst, int k, int kp,
                                       int max_pages, long long n_slots, int vec_per_row, int* status) {
  pdl_launch(); pdl_wait();
  const int row = blockIdx.y;
  const int per_block = blockDim.x / vec_per_row;
  const int j = blockIdx.x * per_block + threadIdx.x / vec_per_row, c = threadIdx.x % vec_per_row;
  if (threadIdx.x >= per_block * vec_per_row || j >= sel_count[row] || j >= k) return;
  const int pos = sel[(size_t)row * k + j];
  const long long slot = pos < 0 ? -1 : (long long)page_table[(size_t)seq_of_row[row] * max_pages + pos / DSA_PAGE] * DSA_PAGE + pos % DSA_PAGE;
  if (slot < 0 || slot >= n_slots) { if (c == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, 0xD52); return; }
  dst[((size_t)row * kp + j) * vec_per_row + c] = cache[slot * vec_per_row + c];
}

extern "C" int cuteafd_dsa_gather_rows(const void* cache, const int* page_table, const int* seq_of_row, const int* sel, const int* sel_count,
                                       void* dst, int rows, int k, int kp, int max_pages, long long n_slots, int row_bytes, int* status,
                                       cudaStream_t s) {
  CA_REQUIRE(cache && page_table && seq_of_row && sel && sel_count && dst, "dsa_gather_rows: null argument");
  CA_REQUIRE(row_bytes % 16 == 0 && row_bytes / 16 <= 256 && kp >= k, "dsa_gather_rows: rows must be 16-byte multiples of at most 4 KB, kp >= k");
  if (rows <= 0) return CA_OK;
  const int vec = row_bytes / 16, per_block = 288 / vec > 0 ? 288 / vec : 1;
  const int threads = per_block * vec;
  CA_LAUNCH_PDL(dsa_gather_rows_kernel, dim3((k + per_block - 1) / per_block, rows), threads, 0, s, (const uint4*)cache, page_table, seq_of_row, sel,
                sel_count, (uint4*)dst, k, kp, max_pages, n_slots, vec, status);
  CA_CHECK_LAUNCH("dsa_gather_rows");
  return CA_OK;
}

// Scatter of freshly computed rows into a paged cache by slot (index keys of the step's tokens): cache[slot_map[t], :] = src[t, :].
__global__ void dsa_scatter_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ slot_map, uint4* __restrict__ cache, int T,
                                        long long n_slots, int vec_per_row, int* status) {
  pdl_launch(); pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * vec_per_row) return;
  const int t = i / vec_per_row, c = i % vec_per_row;
  const long long slot = slot_map[t];
  if (slot < 0 || slot >= n_slots) { if (c == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, 0xD53); return; }
  cache[slot * vec_per_row + c] = src[(size_t)t * vec_per_row + c];
}

extern "C" int cuteafd_dsa_scatter_rows(const void* src, const int* slot_map, void* cache, int T, long long n_slots, int row_bytes, int* status,
                                        cudaStream_t s) {
  CA_REQUIRE(src && slot_map && cache && row_bytes % 16 == 0, "dsa_scatter_rows: bad arguments");
  if (T <= 0) return CA_OK;
  const int vec = row_bytes / 16, n = T * vec;
  CA_LAUNCH_PDL(dsa_scatter_rows_kernel, (n + 255) / 256, 256, 0, s, (const uint4*)src, slot_map, (uint4*)cache, T, n_slots, vec, status);
  CA_CHECK_LAUNCH("dsa_scatter_rows");
  return CA_OK;
}
