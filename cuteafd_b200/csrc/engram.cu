// N-gram memory ("engram"): per token and engram layer, 24 rows of a very large hashed table (FP8 E4M3 values, one UE8M0 scale per 32)
// are fetched, projected (a bf16 GEMM) to one key per residual stream and one value, and a gate mixes the value into the streams.
//   engram_gather   rows addressed by idx[T, 24] -> bf16 [T, 24 * D].  The table may live in device memory or in pinned host memory
//                   mapped into the device's address space: the tables of a full model (hundreds of millions of rows) do not fit
//                   beside the weights, a step touches 24 rows of 264 bytes per token and layer, and the kernel reads exactly those
//                   over the host link instead of staging copies through the host.  Masked rows (images) are written as zeros.
//   engram_gate     one CTA per (token, stream): the stream row stays in registers across the three reductions
//                   (|x|^2, |k|^2, <x wq wk, k>); out = x + sigmoid(ssqrt(dot / (rms x rms k sqrt(H)))) * value, in place.
// Reference: native/families/deepseek_v41/cuda/engram.cu (engram_gate, engram_dequant kernels),
// rust/crates/cuteafd-loader/src/families/deepseek_v41/engram_gather.rs (row gathers from mapped tables).
#include "common.cuh"

#define ENGRAM_COLS 24

// grid (T, 24 / cols_per_block); a row of D = 256 values is 16 threads x 16 bytes.
__global__ void __launch_bounds__(128) engram_gather_kernel(const uint8_t* __restrict__ tq, const uint8_t* __restrict__ te,
                                                            const long long* __restrict__ idx, const uint8_t* __restrict__ text_mask,
                                                            bf16* __restrict__ out, int D, long long n_rows, int* status) {
  pdl_launch(); pdl_wait();
  const int t = blockIdx.x, vec_per_row = D / 16, rows_per_block = 128 / vec_per_row;
  const int col = blockIdx.y * rows_per_block + threadIdx.x / vec_per_row, v = threadIdx.x % vec_per_row;
  if (col >= ENGRAM_COLS) return;
  bf16* dst = out + ((size_t)t * ENGRAM_COLS + col) * D + v * 16;
  uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
  const long long row = idx[(size_t)t * ENGRAM_COLS + col];
  const bool live = !text_mask || text_mask[t];
  if (live && (row < 0 || row >= n_rows)) { if (v == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, 0xE60); }
  else if (live) {
    const uint4 q = *(const uint4*)(tq + (size_t)row * D + v * 16);
    const float s = ue8m0_to_float(te[(size_t)row * (D / 32) + v / 2]);
    const uint8_t* b = (const uint8_t*)&q;
    bf16 o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = __float2bfloat16(e4m3_to_float(b[j]) * s);
    lo = *(const uint4*)&o[0]; hi = *(const uint4*)&o[8];
  }
  *(uint4*)dst = lo;
  *(uint4*)(dst + 8) = hi;
}

// grid (T, S), 256 threads; x [T, S, H] bf16 in place, kv [T, S + 1, H] bf16 (ld_kv elements per token), wq / wk fp32 [S, H].
template <int ITEMS>
__global__ void __launch_bounds__(256) engram_gate_kernel(bf16* __restrict__ x, const bf16* __restrict__ kv, int ld_kv,
                                                          const float* __restrict__ wq, const float* __restrict__ wk,
                                                          const uint8_t* __restrict__ text_mask, int S, int H) {
  pdl_launch(); pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x, s = blockIdx.y;
  if (text_mask && !text_mask[t]) return;
  bf16* xr = x + ((size_t)t * S + s) * H;
  const bf16* kr = kv + (size_t)t * ld_kv + (size_t)s * H;
  const bf16* vr = kv + (size_t)t * ld_kv + (size_t)S * H;
  float xv[ITEMS], xx = 0.f, kk = 0.f, dot = 0.f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int c = threadIdx.x + i * 256;
    xv[i] = 0.f;
    if (c < H) {
      const float h = __bfloat162float(xr[c]), k = __bfloat162float(kr[c]);
      xv[i] = h;
      xx += h * h; kk += k * k; dot += h * (wq[s * H + c] * wk[s * H + c]) * k;
    }
  }
  xx = block_sum(xx, red); kk = block_sum(kk, red); dot = block_sum(dot, red);
  const float d = dot * rsqrtf(xx / H + 1e-20f) * rsqrtf(kk / H + 1e-20f) * rsqrtf((float)H);
  const float g = 1.f / (1.f + __expf(-copysignf(sqrtf(fmaxf(fabsf(d), 1e-6f)), d)));
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < H) xr[c] = __float2bfloat16(xv[i] + g * __bfloat162float(vr[c]));
  }
}

extern "C" int cuteafd_engram_gather(const void* table_q, const void* table_e, const long long* idx, const uint8_t* text_mask, void* out,
                                     int T, int D, long long n_rows, int* status, cudaStream_t s) {
  CA_REQUIRE(table_q && table_e && idx && out && D >= 32 && D <= 2048 && D % 32 == 0 && 128 % (D / 16) == 0 && n_rows > 0,
             "engram_gather: row width %d must be a multiple of 32 whose 16-byte vectors divide 128", D);
  if (T <= 0) return CA_OK;
  const int rows_per_block = 128 / (D / 16);
  CA_LAUNCH_PDL(engram_gather_kernel, dim3(T, (ENGRAM_COLS + rows_per_block - 1) / rows_per_block), 128, 0, s, (const uint8_t*)table_q,
                (const uint8_t*)table_e, idx, text_mask, (bf16*)out, D, n_rows, status);
  CA_CHECK_LAUNCH("engram_gather");
  return CA_OK;
}

extern "C" int cuteafd_engram_gate(void* x, const void* kv, int ld_kv, const float* wq, const float* wk, const uint8_t* text_mask, int T,
                                   int S, int H, cudaStream_t s) {
  CA_REQUIRE(x && kv && wq && wk && S >= 1 && S <= 8 && H > 0 && H <= 8192 && ld_kv >= (S + 1) * H, "engram_gate: 1..8 streams, hidden <= 8192");
  if (T <= 0) return CA_OK;
  const int items = (H + 255) / 256;
  if (items <= 8) CA_LAUNCH_PDL(engram_gate_kernel<8>, dim3(T, S), 256, 0, s, (bf16*)x, (const bf16*)kv, ld_kv, wq, wk, text_mask, S, H);
  else if (items <= 16) CA_LAUNCH_PDL(engram_gate_kernel<16>, dim3(T, S), 256, 0, s, (bf16*)x, (const bf16*)kv, ld_kv, wq, wk, text_mask, S, H);
  else CA_LAUNCH_PDL(engram_gate_kernel<32>, dim3(T, S), 256, 0, s, (bf16*)x, (const bf16*)kv, ld_kv, wq, wk, text_mask, S, H);
  CA_CHECK_LAUNCH("engram_gate");
  return CA_OK;
}
