// Learned KV compressor of the compressed-attention families (the V4 line: CSA with a ratio of 4, HCA with 128; the V4.1 CED cache
// with 2): every token projects to a candidate row kv[t] and a score row s[t] (two GEMMs outside this file), and each block of
// `ratio` consecutive positions is pooled per channel with a softmax over its scores,
//     c[j][d] = sum_{t in block j} softmax_t(s[t][d]) * kv[t][d],
// rounded to bf16, RMS-normalised over the row and scaled by a weight: one cache entry per `ratio` tokens.
// A block that a step leaves unfinished is carried as an online-softmax state per sequence (running max, sum and weighted sum per
// channel), so chunked prefill and one-token decode steps give exactly the rows of a one-shot pass in the same arithmetic order.
//   grid (blocks a sequence touches in this step, sequences); thread = channel (D <= 1024).
// Reference: native/families/deepseek_v41/cuda/v41_compressor.cu (`pool_kernel`: softmax pooling of a row with its predecessor,
// RMSNorm, weight), `compressor_{decode,prefill,continuation}_c{4,128}` programs of the V4 families.
#include "common.cuh"

struct CompressArgs {
  const float* kv;         // [T, D] candidate rows of the step's tokens
  const float* scores;     // [T, D]
  float* state;            // [n_slots, 3, D]: running max, sum, weighted sum of each sequence's open block
  const int* state_slot;   // [n_seq]
  const int* q_start;      // [n_seq] first row of the sequence in this step
  const int* q_len;        // [n_seq]
  const int* pos0;         // [n_seq] position of that first row in the sequence
  const int* out_start;    // [n_seq] first output row of the sequence in this step
  const float* norm_w;     // [D]
  bf16* out;               // [n_out, D] rows of the blocks completed in this step, in order
  int D, ratio, n_seq;
  float eps;
};

__global__ void __launch_bounds__(1024) compress_pool_kernel(const CompressArgs a) {
  pdl_launch(); pdl_wait();
  __shared__ float red[32];
  const int s = blockIdx.y, d = threadIdx.x;
  const int qlen = a.q_len[s], p0 = a.pos0[s], m = a.ratio;
  if (qlen <= 0) return;
  const int first_block = p0 / m, last_block = (p0 + qlen - 1) / m;
  const int b = first_block + blockIdx.x;
  if (b > last_block) return;
  const int lo = max(b * m, p0), hi = min((b + 1) * m, p0 + qlen);       // positions of this block present in the step
  const bool live = d < a.D;
  float mx = -INFINITY, l = 0.f, acc = 0.f;
  float* st = a.state + (size_t)a.state_slot[s] * 3 * a.D;
  if (live && lo > b * m) { mx = st[d]; l = st[a.D + d]; acc = st[2 * a.D + d]; }           // the block was opened by an earlier step
  if (live) {
    for (int p = lo; p < hi; ++p) {
      const size_t row = (size_t)(a.q_start[s] + p - p0) * a.D + d;
      const float sc = a.scores[row], v = a.kv[row];
      const float nm = fmaxf(mx, sc);
      const float r = (mx == -INFINITY) ? 0.f : __expf(mx - nm), e = __expf(sc - nm);
      l = l * r + e;
      acc = acc * r + e * v;
      mx = nm;
    }
  }
  if (hi < (b + 1) * m) {            // still open: only the last block of a sequence's step can be
    if (live) { st[d] = mx; st[a.D + d] = l; st[2 * a.D + d] = acc; }
    return;
  }
  const float pooled = live ? __bfloat162float(__float2bfloat16(acc / l)) : 0.f;
  const float ss = block_sum(pooled * pooled, red);
  if (live) {
    const int orow = a.out_start[s] + (b - first_block);
    a.out[(size_t)orow * a.D + d] = __float2bfloat16(pooled * rsqrtf(ss / a.D + a.eps) * a.norm_w[d]);
  }
}

extern "C" int cuteafd_compress_pool(const float* kv, const float* scores, float* state, const int* state_slot, const int* q_start,
                                     const int* q_len, const int* pos0, const int* out_start, const float* norm_w, void* out, int n_seq,
                                     int max_blocks, int D, int ratio, float eps, cudaStream_t s) {
  CA_REQUIRE(kv && scores && state && state_slot && q_start && q_len && pos0 && out_start && norm_w && out, "compress_pool: null argument");
  CA_REQUIRE(D >= 32 && D <= 1024 && D % 32 == 0 && ratio >= 2 && ratio <= 1024, "compress_pool: 32 <= D <= 1024 (multiple of 32), 2 <= ratio <= 1024");
  if (n_seq <= 0 || max_blocks <= 0) return CA_OK;
  CompressArgs a{kv, scores, state, state_slot, q_start, q_len, pos0, out_start, norm_w, (bf16*)out, D, ratio, n_seq, eps};
  CA_LAUNCH_PDL(compress_pool_kernel, dim3(max_blocks, n_seq), D, 0, s, a);
  CA_CHECK_LAUNCH("compress_pool");
  return CA_OK;
}
