// Gated delta-rule linear attention (the recurrent layers of the GDN / KDA hybrid families): decode, verify and short prefill runs.
//
// Per (sequence, head) a state S [dk x dv] in fp32 is carried from token to token:
//     S   <- diag(g_t) S                       g_t: decay, one scalar per head (GDN) or one value per key channel (KDA), in (0, 1]
//     u   =  S^T k_t                           what the state currently returns for this key          [dv]
//     S   <- S + k_t (beta_t (v_t - u))^T      delta rule: move the stored value towards v_t
//     o_t =  S^T q_t                                                                                   [dv]
// q and k arrive L2-normalised (q also scaled by dk^-1/2) from the projection side.  One CTA per (sequence, head), one thread per
// value channel j: the thread keeps column S[:, j] (dk = 128 fp32 values) in registers for the whole run of tokens, so the state
// crosses HBM once in and once out per call, every load and store of a state row is one coalesced 512-byte line, and q / k / g of
// a token are broadcast from shared memory.  Tokens of a run are processed in order (the recurrence is sequential); long prefills
// are correct but not fast this way - a chunked formulation is not built.
//
// Reference: the `gdn*` / `kda*` programs of the Qwen 3.8 and GLM 5.3 Flash families (AOT-exported, sources absent:
// python/tools/aot/) and their per-slot recurrent state, rust/crates/cuteafd-daemon/src/families/qwen4/ (state slots per
// sequence, draft rows rolled back by restoring the state snapshot).
#include "common.cuh"

#define LA_DK 128
#define LA_DV 128

struct LinAttnArgs {
  const bf16* q; const bf16* k; const bf16* v;   // [T, H, 128]
  const float* g;                                 // [T, H] (per_channel = 0) or [T, H, 128]
  const float* beta;                              // [T, H]
  float* state;                                   // [slots, H, dk, dv]
  const int* slot_of_seq; const int* q_start; const int* q_len;
  bf16* out;                                      // [T, H, 128]
  float* snapshots;                               // optional [T, H, dk, dv]: the state AFTER each token (verify rollback), or null
  int H, per_channel, n_slots;
  int* status;
};

__global__ void __launch_bounds__(LA_DV) gated_delta_kernel(const LinAttnArgs a) {
  pdl_launch(); pdl_wait();
  __shared__ float sq[LA_DK], sk[LA_DK], sg[LA_DK];
  const int seq = blockIdx.y, h = blockIdx.x, j = threadIdx.x;
  const int slot = a.slot_of_seq[seq];
  if (slot < 0 || slot >= a.n_slots) { if (j == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, 0x6D1); return; }
  float* S = a.state + ((size_t)slot * a.H + h) * LA_DK * LA_DV;
  float col[LA_DK];
#pragma unroll
  for (int i = 0; i < LA_DK; ++i) col[i] = S[(size_t)i * LA_DV + j];
  const int t0 = a.q_start[seq], n = a.q_len[seq];
  for (int t = t0; t < t0 + n; ++t) {
    const size_t th = (size_t)t * a.H + h;
    __syncthreads();                                   // the previous token's readers are done with sq / sk / sg
    sq[j] = __bfloat162float(a.q[th * LA_DK + j]);
    sk[j] = __bfloat162float(a.k[th * LA_DK + j]);
    sg[j] = a.per_channel ? a.g[th * LA_DK + j] : a.g[th];
    __syncthreads();
    const float vj = __bfloat162float(a.v[th * LA_DV + j]), bt = a.beta[th];
    float u = 0.f;
#pragma unroll
    for (int i = 0; i < LA_DK; ++i) { col[i] *= sg[i]; u = fmaf(col[i], sk[i], u); }
    const float d = bt * (vj - u);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < LA_DK; ++i) { col[i] = fmaf(sk[i], d, col[i]); o = fmaf(col[i], sq[i], o); }
    a.out[th * LA_DV + j] = __float2bfloat16(o);
    if (a.snapshots) {
      float* snap = a.snapshots + th * LA_DK * LA_DV;
#pragma unroll
      for (int i = 0; i < LA_DK; ++i) snap[(size_t)i * LA_DV + j] = col[i];
    }
  }
#pragma unroll
  for (int i = 0; i < LA_DK; ++i) S[(size_t)i * LA_DV + j] = col[i];
}

extern "C" int cuteafd_gated_delta_step(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state,
                                        const int* slot_of_seq, const int* q_start, const int* q_len, void* out, float* snapshots, int n_seq,
                                        int H, int per_channel, int n_slots, int* status, cudaStream_t s) {
  CA_REQUIRE(q && k && v && g && beta && state && slot_of_seq && q_start && q_len && out, "gated_delta_step: null argument");
  CA_REQUIRE(H >= 1 && n_slots >= 1, "gated_delta_step: bad geometry");
  if (n_seq <= 0) return CA_OK;
  LinAttnArgs a;
  a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.g = g; a.beta = beta; a.state = state; a.slot_of_seq = slot_of_seq;
  a.q_start = q_start; a.q_len = q_len; a.out = (bf16*)out; a.snapshots = snapshots; a.H = H; a.per_channel = per_channel; a.n_slots = n_slots;
  a.status = status;
  CA_LAUNCH_PDL(gated_delta_kernel, dim3(H, n_seq), LA_DV, 0, s, a);
  CA_CHECK_LAUNCH("gated_delta_step");
  return CA_OK;
}

// Causal depthwise convolution of width 4 over the token axis with a per-sequence carry of the last three inputs (the short
// convolution in front of q / k / v in these layers), SiLU on the output.  x, y: [T, C] bf16; w: [C, 4] fp32; carry: [slots, 3, C]
// bf16, updated in place to the last three inputs of each sequence.
__global__ void short_conv4_kernel(const bf16* __restrict__ x, const float* __restrict__ w, bf16* __restrict__ carry, const int* __restrict__ slot_of_seq,
                                   const int* __restrict__ q_start, const int* __restrict__ q_len, bf16* __restrict__ y, int C, int n_slots, int* status) {
  pdl_launch(); pdl_wait();
  const int seq = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int slot = slot_of_seq[seq];
  if (slot < 0 || slot >= n_slots) { if (c == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, 0x6D2); return; }
  bf16* cr = carry + (size_t)slot * 3 * C;
  float h0 = __bfloat162float(cr[c]), h1 = __bfloat162float(cr[C + c]), h2 = __bfloat162float(cr[2 * C + c]);   // inputs t-3, t-2, t-1
  const float w0 = w[c * 4], w1 = w[c * 4 + 1], w2 = w[c * 4 + 2], w3 = w[c * 4 + 3];
  const int t0 = q_start[seq], n = q_len[seq];
  for (int t = t0; t < t0 + n; ++t) {
    const float xt = __bfloat162float(x[(size_t)t * C + c]);
    const float acc = w0 * h0 + w1 * h1 + w2 * h2 + w3 * xt;
    y[(size_t)t * C + c] = __float2bfloat16(acc / (1.f + __expf(-acc)));
    h0 = h1; h1 = h2; h2 = xt;
  }
  cr[c] = __float2bfloat16(h0); cr[C + c] = __float2bfloat16(h1); cr[2 * C + c] = __float2bfloat16(h2);
}

extern "C" int cuteafd_short_conv4(const void* x, const float* w, void* carry, const int* slot_of_seq, const int* q_start, const int* q_len, void* y,
                                   int n_seq, int C, int n_slots, int* status, cudaStream_t s) {
  CA_REQUIRE(x && w && carry && slot_of_seq && q_start && q_len && y && C >= 1, "short_conv4: bad arguments");
  if (n_seq <= 0) return CA_OK;
  CA_LAUNCH_PDL(short_conv4_kernel, dim3((C + 255) / 256, n_seq), 256, 0, s, (const bf16*)x, w, (bf16*)carry, slot_of_seq, q_start, q_len, (bf16*)y, C,
                n_slots, status);
  CA_CHECK_LAUNCH("short_conv4");
  return CA_OK;
}
