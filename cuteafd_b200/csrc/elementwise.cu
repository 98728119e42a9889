// Memory-bound glue kernels (one pass over the activations each, fused where one op feeds the next):
// embedding gather, (residual add +) RMSNorm, q/k head-norm + RoPE + paged KV write, activation
// quantisation to NVFP4 / MXFP4 / FP8 wire rows (optionally gathering rows into expert order), SiLU*up.
// Reference counterparts: native/shared/cuda/norm.cu:5-114, embedding.cu:6-105, attention.cu:88-135
// (rope), kv_cache.cu:142 (norm+RoPE+store), nvfp4_payload.cu:35-117, residual.cu:170-296 (gather +
// quantise on dispatch), mlp.cu:83 (silu_mul).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const bf16* __restrict__ table, bf16* __restrict__ out,
                                    int H, int vocab, int* status) {
  pdl_launch(); pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) { ca_dev_fail(status, CA_DEV_BAD_INDEX, t); tok = 0; }
  const uint4* src = (const uint4*)(table + (size_t)tok * H);
  uint4* dst = (uint4*)(out + (size_t)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

extern "C" int cuteafd_embed_gather(const int* tokens, const void* table, void* out, int T, int H, int vocab, int* status,
                                    cudaStream_t s) {
  CA_REQUIRE(H % 8 == 0, "embed_gather: hidden must be a multiple of 8");
  if (T <= 0) return CA_OK;
  CA_LAUNCH_PDL(embed_gather_kernel, T, 128, 0, s, tokens, (const bf16*)table, (bf16*)out, H, vocab, status);
  CA_CHECK_LAUNCH("embed_gather");
  return CA_OK;
}

// ---------------------------------------------------------------- (add +) rmsnorm
// x_out = x (+ delta)  [written back when delta != null];  y = rmsnorm(x_out) * w.
// One block per row; the row is kept in registers between the two passes (H <= 8 * 1024 elements at 1024 threads).
// Optional FP4 output (qkind 1 NVFP4 / 2 MXFP4): the normalised row is also written quantised (codes + block scales)
// for the GEMM that follows, saving the separate quantiser launch; y may then be null.
template <int VEC>
__global__ void add_rmsnorm_kernel(bf16* __restrict__ x, const bf16* __restrict__ delta, const float* __restrict__ w,
                                   bf16* __restrict__ y, int H, float eps, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                   int ldsf, const float* __restrict__ inv_gs_ptr, int qkind) {
  pdl_launch(); pdl_wait();
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * H;
  float v[VEC * 8];
  float4 nw[VEC * 2];                  // norm weights and the activation scale are fetched with the row, not after the reduction
  const float inv_gs_pre = (qkind == 1 && inv_gs_ptr) ? *inv_gs_ptr : 1.f;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    nw[2 * k] = nw[2 * k + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < H) {
      nw[2 * k] = *(const float4*)(w + i); nw[2 * k + 1] = *(const float4*)(w + i + 4);
      uint4 q = *(const uint4*)(x + base + i);
      const bf16* e = (const bf16*)&q;
      if (delta) {
        uint4 dq = *(const uint4*)(delta + base + i);
        const bf16* de = (const bf16*)&dq;
        bf16 o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { o[j] = __float2bfloat16(__bfloat162float(e[j]) + __bfloat162float(de[j])); v[k * 8 + j] = __bfloat162float(o[j]); }
        *(uint4*)(x + base + i) = *(uint4*)o;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[k * 8 + j] = __bfloat162float(e[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[k * 8 + j] * v[k * 8 + j];
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / H + eps);
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      bf16 o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16(v[k * 8 + j] * inv * ((const float*)&nw[2 * k])[j]);
      if (y) *(uint4*)(y + base + i) = *(uint4*)o;
      if (qkind) {      // H is a multiple of 256 here, so whole warps take this branch together
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(o[j]);
        if (qkind == 3) quant8_store_fp8b(f, q + (size_t)blockIdx.x * H, (float*)sf + (size_t)blockIdx.x * ldsf, i);
        else quant8_store(f, qkind, qkind == 1 ? inv_gs_pre : (inv_gs_ptr ? *inv_gs_ptr : 1.f), q + (size_t)blockIdx.x * (H / 2), sf + (size_t)blockIdx.x * ldsf, i);
      }
    }
  }
}

static int add_rmsnorm_launch(void* x, const void* delta, const float* w, void* y, int T, int H, float eps, void* q, void* sf, int ldsf,
                              const float* inv_gs, int qkind, cudaStream_t s);

extern "C" int cuteafd_add_rmsnorm(void* x, const void* delta, const float* w, void* y, int T, int H, float eps, cudaStream_t s) {
  return add_rmsnorm_launch(x, delta, w, y, T, H, eps, nullptr, nullptr, 0, nullptr, 0, s);
}

// add_rmsnorm that also (or only, y == null) writes the row quantised: qkind 1 = NVFP4, 2 = MXFP4, 3 = FP8 E4M3 with one fp32
// scale per 128 channels (sf then points at floats, ldsf counts floats).
extern "C" int cuteafd_add_rmsnorm_quant(void* x, const void* delta, const float* w, void* y, int T, int H, float eps, void* q, void* sf,
                                         int ldsf, const float* inv_gs, int qkind, cudaStream_t s) {
  CA_REQUIRE(qkind >= 1 && qkind <= 3 && q && sf && H % 256 == 0, "add_rmsnorm_quant: needs quantised outputs and hidden %% 256 == 0");
  return add_rmsnorm_launch(x, delta, w, y, T, H, eps, q, sf, ldsf, inv_gs, qkind, s);
}

static int add_rmsnorm_launch(void* x, const void* delta, const float* w, void* y, int T, int H, float eps, void* q, void* sf, int ldsf,
                              const float* inv_gs, int qkind, cudaStream_t s) {
  CA_REQUIRE(H % 8 == 0 && H <= 32768, "add_rmsnorm: hidden %d unsupported", H);
  CA_REQUIRE(((uintptr_t)w & 15) == 0, "add_rmsnorm: the norm weights must be 16-byte aligned");
  if (T <= 0) return CA_OK;
  const int vecs = H / 8;
  int threads = vecs >= 1024 ? 1024 : ((vecs + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  const int per = (vecs + threads - 1) / threads;
  if (per == 1) CA_LAUNCH_PDL(add_rmsnorm_kernel<1>, T, threads, 0, s, (bf16*)x, (const bf16*)delta, w, (bf16*)y, H, eps, (uint8_t*)q, (uint8_t*)sf, ldsf, inv_gs, qkind);
  else if (per == 2) CA_LAUNCH_PDL(add_rmsnorm_kernel<2>, T, threads, 0, s, (bf16*)x, (const bf16*)delta, w, (bf16*)y, H, eps, (uint8_t*)q, (uint8_t*)sf, ldsf, inv_gs, qkind);
  else CA_LAUNCH_PDL(add_rmsnorm_kernel<4>, T, threads, 0, s, (bf16*)x, (const bf16*)delta, w, (bf16*)y, H, eps, (uint8_t*)q, (uint8_t*)sf, ldsf, inv_gs, qkind);
  CA_CHECK_LAUNCH("add_rmsnorm");
  return CA_OK;
}

// ---------------------------------------------------------------- head-norm + RoPE + paged KV write (GQA)
// qkv: [T, (Hq + 2*Hkv) * D] bf16, q in place.  One warp per (token, head).  K and V rows go to
// kv_cache[slot] with slot = slot_map[t] (page * page_size + offset): layout [slots, 2, Hkv, D].
__global__ void qk_norm_rope_kvwrite_kernel(bf16* __restrict__ qkv, const int* __restrict__ positions,
                                            const int* __restrict__ slot_map, const float* __restrict__ q_norm,
                                            const float* __restrict__ k_norm, bf16* __restrict__ kv_cache, int T, int Hq,
                                            int Hkv, int D, float theta, int interleaved, float eps, int n_slots, int* status) {
  pdl_launch(); pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hkv;
  if (warp >= T * heads) return;
  const int t = warp / heads, h = warp % heads;
  bf16* row = qkv + (size_t)t * heads * D + (size_t)h * D;
  const bool is_q = h < Hq, is_k = !is_q && h < Hq + Hkv;
  // Each lane owns up to 4 rotation pairs.  Pair p is (2p, 2p+1) when interleaved, (p, p + D/2) otherwise.
  const int n_pairs = D / 2, ppl = (n_pairs + 31) / 32;
  float a[4], b[4], wa[4], wb[4];
  int ia[4], ib[4];
  // everything this warp reads from global memory is requested up front (row, norm weights, position, slot): one round trip to
  // L2 instead of four in a row on the decode step's critical path
  const float* nw = is_q ? q_norm : (is_k ? k_norm : nullptr);
  const int pos_i = positions[t];
  const int slot_pre = is_q ? 0 : slot_map[t];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = lane * ppl + j;
    const bool on = j < ppl && p < n_pairs;
    ia[j] = on ? (interleaved ? 2 * p : p) : -1;
    ib[j] = on ? (interleaved ? 2 * p + 1 : p + n_pairs) : -1;
    a[j] = on ? __bfloat162float(row[ia[j]]) : 0.f;
    b[j] = on ? __bfloat162float(row[ib[j]]) : 0.f;
    wa[j] = (on && nw) ? nw[ia[j]] : 1.f;
    wb[j] = (on && nw) ? nw[ib[j]] : 1.f;
  }
  if (is_q || is_k) {
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += a[j] * a[j] + b[j] * b[j];
      const float inv = rsqrtf(warp_sum(ss) / D + eps);
#pragma unroll
      for (int j = 0; j < 4; ++j) if (ia[j] >= 0) { a[j] *= inv * wa[j]; b[j] *= inv * wb[j]; }
    }
    const float pos = (float)pos_i;
#pragma unroll
    for (int j = 0; j < 4; ++j) if (ia[j] >= 0) {
      const int p = lane * ppl + j;
      const float ang = pos * powf(theta, -2.f * (float)p / (float)D);
      const float sn = sinf(ang), cs = cosf(ang);
      const float x0 = a[j], x1 = b[j];
      a[j] = x0 * cs - x1 * sn;
      b[j] = x0 * sn + x1 * cs;
    }
  }
  bf16* dst = row;
  if (!is_q) {
    const int slot = slot_pre;
    if (slot < 0 || slot >= n_slots) { if (lane == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, t); return; }
    dst = kv_cache + ((size_t)slot * 2 + (is_k ? 0 : 1)) * Hkv * D + (size_t)(h - Hq - (is_k ? 0 : Hkv)) * D;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) if (ia[j] >= 0) { dst[ia[j]] = __float2bfloat16(a[j]); dst[ib[j]] = __float2bfloat16(b[j]); }
}

extern "C" int cuteafd_qk_norm_rope_kvwrite(void* qkv, const int* positions, const int* slot_map, const float* q_norm,
                                            const float* k_norm, void* kv_cache, int T, int Hq, int Hkv, int D, float theta,
                                            int interleaved, float eps, int n_slots, int* status, cudaStream_t s) {
  CA_REQUIRE(D == 32 || D == 64 || D == 128 || D == 256, "qk_norm_rope_kvwrite: head_dim %d unsupported", D);
  if (T <= 0) return CA_OK;
  const long long warps = (long long)T * (Hq + 2 * Hkv);
  const int blocks = (int)((warps * 32 + 255) / 256);
  CA_LAUNCH_PDL(qk_norm_rope_kvwrite_kernel, blocks, 256, 0, s, (bf16*)qkv, positions, slot_map, q_norm, k_norm, (bf16*)kv_cache, T, Hq,
                                                     Hkv, D, theta, interleaved, eps, n_slots, status);
  CA_CHECK_LAUNCH("qk_norm_rope_kvwrite");
  return CA_OK;
}

// ---------------------------------------------------------------- FP4 activation quantisation (+ gather)
// One thread quantises 16 consecutive elements.  NVFP4: E4M3 scale per 16 with a static global scale
// (inv_gs = 1 / global_scale); MXFP4: UE8M0 scale per 32 (two threads cooperate through a shuffle).
// dst row i takes src row (src_rows ? src_rows[i] : i); rows with a negative source are zero-filled.
template <bool MX>
__global__ void quant_fp4_rows_kernel(const bf16* __restrict__ x, const int* __restrict__ src_rows, const int* __restrict__ n_rows_dev,
                                      uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int rows, int K, int ldx, int ldsf,
                                      const float* __restrict__ inv_gs_ptr) {
  pdl_launch(); pdl_wait();
  const int per_row = K / 16;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int r = (int)(gid / per_row), c = (int)(gid % per_row);
  // the row count, the row's source and the activation scale are independent loads: issue them together (a decode step's quantiser
  // is a chain of L2 round trips, not bandwidth)
  const int n_dev = n_rows_dev ? *n_rows_dev : rows;
  const int src_any = (r < rows) ? (src_rows ? src_rows[r] : r) : -1;
  const float inv_gs_pre = (!MX && inv_gs_ptr) ? *inv_gs_ptr : 1.f;
  const int n_rows = min(n_dev, rows);
  const bool active = r < n_rows;
  float v[16];
  int src = active ? src_any : -1;
  if (src >= 0) {
    const uint4* p = (const uint4*)(x + (size_t)src * ldx + c * 16);
    uint4 a = p[0], b = p[1];
    const bf16* ea = (const bf16*)&a; const bf16* eb = (const bf16*)&b;
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[j] = __bfloat162float(ea[j]); v[8 + j] = __bfloat162float(eb[j]); }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
  float eff;   // value of one FP4 unit
  uint8_t sb;
  if (MX) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    // OCP MX: shared exponent = floor(log2(amax)) - 2
    int e = amax > 0.f ? (int)((__float_as_uint(amax) >> 23) & 0xFF) - 2 : 0;
    e = max(e, 0); e = min(e, 254);
    sb = (uint8_t)e;
    eff = ue8m0_to_float(sb);
  } else {
    const float inv_gs = inv_gs_pre;
    const float target = fminf(amax * inv_gs / 6.f, 448.f);
    sb = float_to_e4m3(target);
    eff = e4m3_to_float(sb) / inv_gs;
  }
  if (!active) return;
  const float inv = eff > 0.f ? 1.f / eff : 0.f;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) { lo |= float_to_e2m1(v[j] * inv) << (4 * j); hi |= float_to_e2m1(v[8 + j] * inv) << (4 * j); }
  *(uint2*)(q + (size_t)r * (K / 2) + c * 8) = make_uint2(lo, hi);
  if (MX) { if (!(c & 1)) sf[(size_t)r * ldsf + (c >> 1)] = sb; }
  else sf[(size_t)r * ldsf + c] = sb;
}

extern "C" int cuteafd_quant_fp4_rows(int mx, const void* x, const int* src_rows, const int* n_rows_dev, void* q, void* sf,
                                      int rows, int K, int ldx, int ldsf, const float* inv_gs, cudaStream_t s) {
  CA_REQUIRE(K % 32 == 0 && ldx % 8 == 0, "quant_fp4_rows: K must be a multiple of 32");
  if (rows <= 0) return CA_OK;
  const long long n = (long long)rows * (K / 16);
  const int blocks = (int)((n + 255) / 256);
  if (mx) CA_LAUNCH_PDL(quant_fp4_rows_kernel<true>, blocks, 256, 0, s, (const bf16*)x, src_rows, n_rows_dev, (uint8_t*)q, (uint8_t*)sf, rows, K, ldx, ldsf, inv_gs);
  else CA_LAUNCH_PDL(quant_fp4_rows_kernel<false>, blocks, 256, 0, s, (const bf16*)x, src_rows, n_rows_dev, (uint8_t*)q, (uint8_t*)sf, rows, K, ldx, ldsf, inv_gs);
  CA_CHECK_LAUNCH("quant_fp4_rows");
  return CA_OK;
}

// Gather bf16 rows into expert order (BF16 expert path).
__global__ void gather_rows_kernel(const bf16* __restrict__ x, const int* __restrict__ src_rows, const int* __restrict__ n_rows_dev,
                                   bf16* __restrict__ out, int rows, int K) {
  pdl_launch(); pdl_wait();
  const int r = blockIdx.x;
  const int n_rows = n_rows_dev ? min(*n_rows_dev, rows) : rows;
  if (r >= n_rows) return;
  const int src = src_rows[r];
  uint4* dst = (uint4*)(out + (size_t)r * K);
  if (src < 0) { for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0); return; }
  const uint4* sp = (const uint4*)(x + (size_t)src * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = sp[i];
}

extern "C" int cuteafd_gather_rows(const void* x, const int* src_rows, const int* n_rows_dev, void* out, int rows, int K, cudaStream_t s) {
  CA_REQUIRE(K % 8 == 0, "gather_rows: K must be a multiple of 8");
  if (rows <= 0) return CA_OK;
  CA_LAUNCH_PDL(gather_rows_kernel, rows, 128, 0, s, (const bf16*)x, src_rows, n_rows_dev, (bf16*)out, rows, K);
  CA_CHECK_LAUNCH("gather_rows");
  return CA_OK;
}

// ---------------------------------------------------------------- FP8 wire rows (E4M3 + UE8M0 / 32)
// Activation hand-off format between attention ranks and expert ranks: BF16-rounded input, amax floor 1e-4,
// scale = 2^ceil(log2(amax / 448)).  One warp-lane group of 4 threads per 32 elements (8 each).
__global__ void act_quant_fp8_ue8m0_kernel(const bf16* __restrict__ x, const int* __restrict__ src_rows, const int* __restrict__ n_rows_dev,
                                           uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int rows, int H, int ldx, int ldsf) {
  pdl_launch(); pdl_wait();
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = H / 8;
  if (gid >= (long long)rows * per_row) return;
  const int r = (int)(gid / per_row), c = (int)(gid % per_row);
  if (n_rows_dev && r >= *n_rows_dev) return;           // whole groups of 4 lanes leave together (one row per group)
  const int sr = src_rows ? src_rows[r] : r;
  uint4 a = *(const uint4*)(x + (size_t)sr * ldx + c * 8);
  const bf16* e = (const bf16*)&a;
  float v[8], amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { v[j] = __bfloat162float(e[j]); amax = fmaxf(amax, fabsf(v[j])); }
  amax = fmaxf(amax, __shfl_xor_sync(__activemask(), amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(__activemask(), amax, 2));
  amax = fmaxf(amax, 1e-4f);
  const uint8_t sb = ue8m0_ceil(amax / 448.f);
  const float inv = 1.f / ue8m0_to_float(sb);
  uint32_t w0 = 0, w1 = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) { w0 |= (uint32_t)float_to_e4m3(v[j] * inv) << (8 * j); w1 |= (uint32_t)float_to_e4m3(v[4 + j] * inv) << (8 * j); }
  *(uint2*)(q + (size_t)r * H + c * 8) = make_uint2(w0, w1);
  if ((c & 3) == 0) sf[(size_t)r * ldsf + (c >> 2)] = sb;
}

// `src_rows` (optional) gathers: output row r quantises input row src_rows[r]; `n_rows_dev` (optional) bounds the live rows
// on the device; `ldx` is the input row pitch in elements, `ldsf` the scale row pitch in bytes (>= H / 32).
extern "C" int cuteafd_act_quant_fp8_ue8m0(const void* x, const int* src_rows, const int* n_rows_dev, void* q, void* sf, int rows, int H,
                                           int ldx, int ldsf, cudaStream_t s) {
  CA_REQUIRE(H % 32 == 0 && ldsf >= H / 32 && ldx >= H && ldx % 8 == 0, "act_quant_fp8_ue8m0: H %% 32 == 0, scale pitch >= H / 32");
  if (rows <= 0) return CA_OK;
  const long long n = (long long)rows * (H / 8);
  CA_LAUNCH_PDL(act_quant_fp8_ue8m0_kernel, (int)((n + 255) / 256), 256, 0, s, (const bf16*)x, src_rows, n_rows_dev, (uint8_t*)q, (uint8_t*)sf,
                rows, H, ldx, ldsf);
  return CA_OK;
}

// ---------------------------------------------------------------- silu(gate) * up  (unfused FC1 outputs)
__global__ void silu_mul_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u, bf16* __restrict__ o, long long n, float limit) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i >= n) return;
  float2 a = __bfloat1622float2(*(const bf162*)(g + i)), b = __bfloat1622float2(*(const bf162*)(u + i));
  if (limit > 0.f) { a.x = fminf(a.x, limit); a.y = fminf(a.y, limit); b.x = fminf(fmaxf(b.x, -limit), limit); b.y = fminf(fmaxf(b.y, -limit), limit); }
  float2 r = make_float2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
  *(bf162*)(o + i) = __float22bfloat162_rn(r);
}

extern "C" int cuteafd_silu_mul(const void* g, const void* u, void* o, long long n, float limit, cudaStream_t s) {
  CA_REQUIRE(n % 2 == 0, "silu_mul: element count must be even");
  if (n <= 0) return CA_OK;
  silu_mul_kernel<<<(int)((n / 2 + 255) / 256), 256, 0, s>>>((const bf16*)g, (const bf16*)u, (bf16*)o, n, limit);
  CA_CHECK_LAUNCH("silu_mul");
  return CA_OK;
}

// silu(gate) * up written as the FP8 operand of the GEMM that follows (E4M3 + one fp32 scale per 128 channels), with the same
// bf16 rounding of the product as the two-kernel form (silu_mul, then the quantiser).  g, u: [rows, N] bf16 (row pitch ld);
// q: [rows, N] bytes; sa: [rows, N / 128].  One warp per 256 channels of a row; N % 256 == 0.
__global__ void silu_mul_quant_fp8b_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u, uint8_t* __restrict__ q, float* __restrict__ sa,
                                           int rows, int N, int ld) {
  pdl_launch(); pdl_wait();
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31, per_row = N / 256;
  if (w >= (long long)rows * per_row) return;
  const int r = (int)(w / per_row), i = (int)(w % per_row) * 256 + lane * 8;
  const uint4 gq = *(const uint4*)(g + (size_t)r * ld + i), uq = *(const uint4*)(u + (size_t)r * ld + i);
  const bf16* ge = (const bf16*)&gq; const bf16* ue = (const bf16*)&uq;
  float f[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float a = __bfloat162float(ge[j]), b = __bfloat162float(ue[j]);
    f[j] = __bfloat162float(__float2bfloat16(a / (1.f + __expf(-a)) * b));
  }
  quant8_store_fp8b(f, q + (size_t)r * N, sa + (size_t)r * (N / 128), i);
}

extern "C" int cuteafd_silu_mul_quant_fp8b(const void* g, const void* u, void* q, float* sa, int rows, int N, int ld, cudaStream_t s) {
  CA_REQUIRE(g && u && q && sa && N % 256 == 0 && ld % 8 == 0, "silu_mul_quant_fp8b: N must be a multiple of 256");
  if (rows <= 0) return CA_OK;
  const long long warps = (long long)rows * (N / 256);
  CA_LAUNCH_PDL(silu_mul_quant_fp8b_kernel, (int)((warps * 32 + 255) / 256), 256, 0, s, (const bf16*)g, (const bf16*)u, (uint8_t*)q, sa, rows, N, ld);
  CA_CHECK_LAUNCH("silu_mul_quant_fp8b");
  return CA_OK;
}
