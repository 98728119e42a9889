// EXL3 (trellis-coded) weights: dequant-GEMM for decode-sized batches, reading the checkpoint's tensors as shipped.
//
//   W[K, N] = diag(suh) * H_K * inner * H_N * diag(svh)        (H: block-diagonal normalised 128-point Hadamard)
//   y = x W  =  H_N( ((H_K(x * suh)) @ inner) ) * svh
// so the weight-sized work is `x' @ inner` with `inner` decoded on the fly from the trellis, and the rotations are two
// small activation-sized kernels.
//
// Trellis: each 16 x 16 tile is 256 symbols of `bits` bits in a circular big-endian bit stream (the stored uint16
// pairs are swapped precisely so that the stream is a sequence of native 32-bit words); the value of symbol p is a
// hash of the 16 stream bits that END with symbol p (tail-biting: the first symbols wrap into the tile's end), so
// every value decodes independently.  The 256 values sit in the register order of the m16n8k16 tensor-core B
// fragment: lane l of a warp decodes symbols 8l .. 8l+7 and owns exactly the operands of two MMAs.  This kernel is
// bandwidth-bound on the trellis bits (2-8 bits per weight), which is why it uses the warp-level MMA with operands
// produced in registers rather than a shared-memory staged tcgen05 pipeline.
//
// Reference: the EXL3 GEMM/GEMV programs (native/shared/cuda/exl3_gemm.cu, exl3_kernel_map.cu) and the format oracle
// python/tools/lib/exl3_reference.py:13-96.
#include <cuda_fp16.h>

#include "common.cuh"

__device__ __forceinline__ float exl3_value(uint32_t state) {
  uint32_t r = state * 0xCBAC1FEDu;
  r = 0x3B603B60u ^ (r & 0x8FFF8FFFu);
  const __half2 h = *reinterpret_cast<const __half2*>(&r);
  return __low2float(h) + __high2float(h);
}

// 16 stream bits ending (exclusive) at bit `e` of a circular stream of `nw` 32-bit big-endian words held in shared memory.
__device__ __forceinline__ uint32_t exl3_window(const uint32_t* w, int nw, int e) {
  const int total = nw * 32;
  int s = e - 16;
  if (s < 0) s += total;
  const int wi = s >> 5, bo = s & 31;
  const uint32_t a = w[wi], b = w[(wi + 1) % nw];
  const uint64_t cat = ((uint64_t)a << 32) | b;
  return (uint32_t)(cat >> (48 - bo)) & 0xFFFFu;
}

__device__ __forceinline__ void mma_m16n8k16_f16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// part[split][T16 * 16][N] (fp32) = x'[rows, k-slice] @ inner[k-slice, N].  One warp per (16-column strip, K slice,
// 16-token tile); x' is fp16 [rows_pad16, K].  4 warps per block.
__global__ void exl3_gemm_kernel(const __half* __restrict__ xr, const uint32_t* __restrict__ trellis, float* __restrict__ part,
                                 int rows_pad, int K, int N, int bits, int k_splits) {
  pdl_launch(); pdl_wait();
  __shared__ uint32_t words[4][128];               // one tile's bit stream per warp (bits <= 8 -> <= 128 words)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int strip = blockIdx.x * 4 + warp, split = blockIdx.y, ttile = blockIdx.z;
  const int n_strips = N / 16;
  if (strip >= n_strips) return;
  const int kt_all = K / 16;
  const int kt0 = (int)(((long long)kt_all * split) / k_splits), kt1 = (int)(((long long)kt_all * (split + 1)) / k_splits);
  const int nw = 8 * bits;                         // 32-bit words per tile
  float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
  const __half* xa = xr + (size_t)(ttile * 16) * K;
  const int ar = lane >> 2, ak = (lane & 3) * 2;
  for (int kt = kt0; kt < kt1; ++kt) {
    const uint32_t* src = trellis + ((size_t)kt * n_strips + strip) * nw;
    __syncwarp();
    for (int i = lane; i < nw; i += 32) words[warp][i] = src[i];
    __syncwarp();
    // A fragment: x'[16 tokens, 16 k] row-major
    uint32_t a[4];
    const __half* xk = xa + (size_t)kt * 16 + ak;
    a[0] = *(const uint32_t*)(xk + (size_t)ar * K);
    a[1] = *(const uint32_t*)(xk + (size_t)(ar + 8) * K);
    a[2] = *(const uint32_t*)(xk + (size_t)ar * K + 8);
    a[3] = *(const uint32_t*)(xk + (size_t)(ar + 8) * K + 8);
    // B fragments: this lane's 8 symbols
    __half v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __float2half(exl3_value(exl3_window(words[warp], nw, (lane * 8 + j + 1) * bits)));
    const uint32_t* vb = reinterpret_cast<const uint32_t*>(v);
    mma_m16n8k16_f16(c0, a, vb[0], vb[1]);
    mma_m16n8k16_f16(c1, a, vb[2], vb[3]);
  }
  // C fragment: rows lane/4 (+8), columns (lane%4)*2 (+1) of each 8-column half
  float* out = part + ((size_t)split * rows_pad + ttile * 16) * N + strip * 16;
  const int cr = lane >> 2, cc = (lane & 3) * 2;
  *(float2*)(out + (size_t)cr * N + cc) = make_float2(c0[0], c0[1]);
  *(float2*)(out + (size_t)(cr + 8) * N + cc) = make_float2(c0[2], c0[3]);
  *(float2*)(out + (size_t)cr * N + 8 + cc) = make_float2(c1[0], c1[1]);
  *(float2*)(out + (size_t)(cr + 8) * N + 8 + cc) = make_float2(c1[2], c1[3]);
}

// 128-point normalised Walsh-Hadamard transform of one 128-block per warp (4 values per lane: elements 4l .. 4l+3).
__device__ __forceinline__ void wht128(float* v, int lane) {
  // strides 1 and 2 inside the lane
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = (lane & m) ? o - v[j] : v[j] + o;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] *= 0.08838834764831845f;     // 1 / sqrt(128)
}

// x'[r, :] = H_K(x[r, :] * suh) as fp16, rows >= rows zero-filled up to rows_pad.
__global__ void exl3_pre_kernel(const bf16* __restrict__ x, const __half* __restrict__ suh, __half* __restrict__ xr, int rows, int rows_pad, int K) {
  pdl_launch(); pdl_wait();
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31, nb = K / 128;
  if (w >= (long long)rows_pad * nb) return;
  const int r = (int)(w / nb), k0 = (int)(w % nb) * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (r < rows) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(x[(size_t)r * K + k0 + j]) * __half2float(suh[k0 + j]);
  }
  wht128(v, lane);
#pragma unroll
  for (int j = 0; j < 4; ++j) xr[(size_t)r * K + k0 + j] = __float2half(v[j]);
}

// y[r, :] = H_N(sum_splits part[s][r, :]) * svh  (+ residual), bf16.
__global__ void exl3_post_kernel(const float* __restrict__ part, const __half* __restrict__ svh, const bf16* __restrict__ residual,
                                 bf16* __restrict__ y, int rows, int rows_pad, int N, int k_splits, int ldy) {
  pdl_launch(); pdl_wait();
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31, nb = N / 128;
  if (w >= (long long)rows * nb) return;
  const int r = (int)(w / nb), n0 = (int)(w % nb) * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < k_splits; ++s) {
    const float4 p = *(const float4*)(part + ((size_t)s * rows_pad + r) * N + n0);
    v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
  }
  wht128(v, lane);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float o = v[j] * __half2float(svh[n0 + j]);
    if (residual) o += __bfloat162float(residual[(size_t)r * ldy + n0 + j]);
    y[(size_t)r * ldy + n0 + j] = __float2bfloat16(o);
  }
}

// y[rows, N] (bf16, + optional residual) = x[rows, K] (bf16) @ W, W given as EXL3 tensors: trellis uint16
// [K/16, N/16, 16*bits], suh fp16 [K], svh fp16 [N].  Scratch: xr fp16 [rows_pad16, K], part fp32 [k_splits, rows_pad16, N].
extern "C" int cuteafd_exl3_linear(const void* x, const void* trellis, const void* suh, const void* svh, const void* residual, void* y,
                                   void* xr, float* part, int rows, int K, int N, int bits, int k_splits, int ldy, cudaStream_t s) {
  CA_REQUIRE(K % 128 == 0 && N % 128 == 0, "exl3_linear: K and N must be multiples of 128 (K=%d N=%d)", K, N);
  CA_REQUIRE(bits >= 1 && bits <= 8, "exl3_linear: 1..8 bits per weight");
  CA_REQUIRE(k_splits >= 1 && k_splits <= K / 16, "exl3_linear: bad split count");
  if (rows <= 0) return CA_OK;
  const int rows_pad = (rows + 15) / 16 * 16;
  {
    const long long warps = (long long)rows_pad * (K / 128);
    CA_LAUNCH_PDL(exl3_pre_kernel, (int)((warps * 32 + 255) / 256), 256, 0, s, (const bf16*)x, (const __half*)suh, (__half*)xr, rows, rows_pad, K);
  }
  {
    dim3 grid((N / 16 + 3) / 4, k_splits, rows_pad / 16);
    CA_LAUNCH_PDL(exl3_gemm_kernel, grid, 128, 0, s, (const __half*)xr, (const uint32_t*)trellis, part, rows_pad, K, N, bits, k_splits);
  }
  {
    const long long warps = (long long)rows * (N / 128);
    CA_LAUNCH_PDL(exl3_post_kernel, (int)((warps * 32 + 255) / 256), 256, 0, s, (const float*)part, (const __half*)svh, (const bf16*)residual, (bf16*)y,
                  rows, rows_pad, N, k_splits, ldy);
  }
  return CA_OK;
}
