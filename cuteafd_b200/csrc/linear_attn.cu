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
  int H, per_channel, n_slots;             // per_channel: bit 0 = one decay per key channel, bit 1 = do not write the state back
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
    sg[j] = (a.per_channel & 1) ? a.g[th * LA_DK + j] : a.g[th];
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
  if (a.per_channel & 2) return;          // verify rows of a speculative step: outputs only, the state is committed later by a replay
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
// convolution in front of q / k / v in these layers), SiLU on the output.  x: [T, C] bf16 with row pitch ldx, y: [T, C]; w: [C, 4] fp32; carry: [slots, 3, C]
// bf16, updated in place to the last three inputs of each sequence.
template <bool UPDATE>
__global__ void short_conv4_kernel(const bf16* __restrict__ x, const float* __restrict__ w, bf16* __restrict__ carry, const int* __restrict__ slot_of_seq,
                                   const int* __restrict__ q_start, const int* __restrict__ q_len, bf16* __restrict__ y, int C, int ldx, int n_slots, int* status) {
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
    const float xt = __bfloat162float(x[(size_t)t * ldx + c]);
    const float acc = w0 * h0 + w1 * h1 + w2 * h2 + w3 * xt;
    y[(size_t)t * C + c] = __float2bfloat16(acc / (1.f + __expf(-acc)));
    h0 = h1; h1 = h2; h2 = xt;
  }
  if (UPDATE) { cr[c] = __float2bfloat16(h0); cr[C + c] = __float2bfloat16(h1); cr[2 * C + c] = __float2bfloat16(h2); }
}

extern "C" int cuteafd_short_conv4(const void* x, const float* w, void* carry, const int* slot_of_seq, const int* q_start, const int* q_len, void* y,
                                   int n_seq, int C, int ldx, int n_slots, int* status, cudaStream_t s) {
  CA_REQUIRE(x && w && carry && slot_of_seq && q_start && q_len && y && C >= 1 && ldx >= C, "short_conv4: bad arguments");
  if (n_seq <= 0) return CA_OK;
  CA_LAUNCH_PDL(short_conv4_kernel<true>, dim3((C + 255) / 256, n_seq), 256, 0, s, (const bf16*)x, w, (bf16*)carry, slot_of_seq, q_start, q_len, (bf16*)y, C,
                ldx, n_slots, status);
  CA_CHECK_LAUNCH("short_conv4");
  return CA_OK;
}

// The same convolution without touching the carry: the verify rows of a speculative step (the accepted prefix is replayed through
// `cuteafd_short_conv4` afterwards, which then moves the carry).
extern "C" int cuteafd_short_conv4_peek(const void* x, const float* w, const void* carry, const int* slot_of_seq, const int* q_start, const int* q_len,
                                        void* y, int n_seq, int C, int ldx, int n_slots, int* status, cudaStream_t s) {
  CA_REQUIRE(x && w && carry && slot_of_seq && q_start && q_len && y && C >= 1 && ldx >= C, "short_conv4_peek: bad arguments");
  if (n_seq <= 0) return CA_OK;
  CA_LAUNCH_PDL(short_conv4_kernel<false>, dim3((C + 255) / 256, n_seq), 256, 0, s, (const bf16*)x, w, (bf16*)carry, slot_of_seq, q_start, q_len, (bf16*)y,
                C, ldx, n_slots, status);
  CA_CHECK_LAUNCH("short_conv4_peek");
  return CA_OK;
}

// ---------------------------------------------------------------- glue of a gated delta-rule layer
// After the convolution: conv [T, (2 Hk + Hv) * 128] bf16 holds q (Hk heads), k (Hk heads), v (Hv heads); ba [T, ldb] fp32 holds
// b [Hv] then a [Hv] (or a per key channel [Hv * 128]).  One warp per (token, value head) writes what the recurrence consumes:
// q_e / k_e [T, Hv, 128] = the L2-normalised q (scaled by 128^-1/2) and k of key head hv / (Hv / Hk), v_e [T, Hv, 128] (contiguous
// copy), beta = sigmoid(b), g = exp(-exp(a_log[hv]) * softplus(a + dt_bias)) per head or per channel.
__global__ void linear_prepare_kernel(const bf16* __restrict__ conv, const float* __restrict__ ba, const float* __restrict__ a_log,
                                      const float* __restrict__ dt_bias, bf16* __restrict__ q_e, bf16* __restrict__ k_e, bf16* __restrict__ v_e,
                                      float* __restrict__ g, float* __restrict__ beta, int T, int Hk, int Hv, int ldb, int per_channel) {
  pdl_launch(); pdl_wait();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * Hv) return;
  const int t = w / Hv, hv = w % Hv, hk = hv / (Hv / Hk);
  const int C = (2 * Hk + Hv) * 128;
  const bf16* row = conv + (size_t)t * C;
  const uint2 qr = *(const uint2*)(row + hk * 128 + lane * 4), kr = *(const uint2*)(row + (Hk + hk) * 128 + lane * 4);
  const uint2 vr = *(const uint2*)(row + (2 * Hk + hv) * 128 + lane * 4);
  const bf16* qe = (const bf16*)&qr; const bf16* ke = (const bf16*)&kr;
  float q[4], k[4], sq = 0.f, sk = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { q[j] = __bfloat162float(qe[j]); k[j] = __bfloat162float(ke[j]); sq += q[j] * q[j]; sk += k[j] * k[j]; }
  sq = warp_sum(sq); sk = warp_sum(sk);
  const float iq = 0.08838834764831845f / fmaxf(sqrtf(sq), 1e-6f), ik = 1.f / fmaxf(sqrtf(sk), 1e-6f);     // 128^-1/2 folded into q
  bf16 qo[4], ko[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) { qo[j] = __float2bfloat16(q[j] * iq); ko[j] = __float2bfloat16(k[j] * ik); }
  const size_t o = ((size_t)t * Hv + hv) * 128 + lane * 4;
  *(uint2*)(q_e + o) = *(uint2*)qo; *(uint2*)(k_e + o) = *(uint2*)ko; *(uint2*)(v_e + o) = vr;
  const float* bar = ba + (size_t)t * ldb;
  const float al = __expf(a_log[hv]);
  if (per_channel) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = hv * 128 + lane * 4 + j;
      const float x = bar[Hv + c] + dt_bias[c];
      g[(size_t)t * Hv * 128 + c] = __expf(-al * (x > 20.f ? x : log1pf(__expf(x))));
    }
  } else if (lane == 0) {
    const float x = bar[Hv + hv] + dt_bias[hv];
    g[(size_t)t * Hv + hv] = __expf(-al * (x > 20.f ? x : log1pf(__expf(x))));
  }
  if (lane == 0) beta[(size_t)t * Hv + hv] = 1.f / (1.f + __expf(-bar[hv]));
}

extern "C" int cuteafd_linear_prepare(const void* conv, const float* ba, const float* a_log, const float* dt_bias, void* q_e, void* k_e, void* v_e,
                                      float* g, float* beta, int T, int Hk, int Hv, int ldb, int per_channel, cudaStream_t s) {
  CA_REQUIRE(conv && ba && a_log && dt_bias && q_e && k_e && v_e && g && beta && Hk >= 1 && Hv % Hk == 0, "linear_prepare: bad arguments");
  if (T <= 0) return CA_OK;
  const long long threads = (long long)T * Hv * 32;
  CA_LAUNCH_PDL(linear_prepare_kernel, (int)((threads + 255) / 256), 256, 0, s, (const bf16*)conv, ba, a_log, dt_bias, (bf16*)q_e, (bf16*)k_e, (bf16*)v_e, g,
                beta, T, Hk, Hv, ldb, per_channel);
  CA_CHECK_LAUNCH("linear_prepare");
  return CA_OK;
}

// out[t, h * 128 + :] = rmsnorm(o[t, h, :]) * w * silu(z[t, h, :]); z lives at column z_off of rows with pitch ldz (the z part of the
// fused input projection).  One warp per (token, head).
__global__ void gated_rmsnorm_kernel(const bf16* __restrict__ o, const bf16* __restrict__ z, const float* __restrict__ w, bf16* __restrict__ out, int T, int H,
                                     int ldz, int z_off, float eps) {
  pdl_launch(); pdl_wait();
  const int wi = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (wi >= T * H) return;
  const int t = wi / H, h = wi % H;
  const uint2 orw = *(const uint2*)(o + ((size_t)t * H + h) * 128 + lane * 4), zr = *(const uint2*)(z + (size_t)t * ldz + z_off + h * 128 + lane * 4);
  const bf16* oe = (const bf16*)&orw; const bf16* ze = (const bf16*)&zr;
  float v[4], ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = __bfloat162float(oe[j]); ss += v[j] * v[j]; }
  const float inv = rsqrtf(warp_sum(ss) / 128.f + eps);
  bf16 r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float zz = __bfloat162float(ze[j]);
    const float n = __bfloat162float(__float2bfloat16(v[j] * inv * w[lane * 4 + j]));        // the norm's bf16 output, as the stand-alone kernel rounds it
    r[j] = __float2bfloat16(n * (zz / (1.f + __expf(-zz))));
  }
  *(uint2*)(out + ((size_t)t * H + h) * 128 + lane * 4) = *(uint2*)r;
}

extern "C" int cuteafd_gated_rmsnorm(const void* o, const void* z, const float* w, void* out, int T, int H, int ldz, int z_off, float eps, cudaStream_t s) {
  CA_REQUIRE(o && z && w && out && ldz % 4 == 0 && z_off % 4 == 0, "gated_rmsnorm: bad arguments");
  if (T <= 0) return CA_OK;
  const long long threads = (long long)T * H * 32;
  CA_LAUNCH_PDL(gated_rmsnorm_kernel, (int)((threads + 255) / 256), 256, 0, s, (const bf16*)o, (const bf16*)z, w, (bf16*)out, T, H, ldz, z_off, eps);
  CA_CHECK_LAUNCH("gated_rmsnorm");
  return CA_OK;
}
