// Shared device/host helpers for the sm_100a kernels: status ABI, numeric-format decode/encode,
// and thin inline-PTX wrappers for mbarrier, TMA (cp.async.bulk[.tensor]), tcgen05 (alloc, mma,
// commit, cp, ld) and system-scope release/acquire flags.
//
// Conventions
//  * Every exported function is `extern "C"`, takes raw device pointers + a cudaStream_t and returns
//    an int status (0 = ok).  `cuteafd_last_error()` returns the message of the last failure on the
//    calling thread.  (Same shape as the reference's C ABI, native/shared/include/cuteafd_native.h.)
//  * Every device-side wait is bounded.  A wait that runs out records a code in a status word and the
//    kernel unwinds (frees tensor memory, returns); nothing traps or spins forever.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CA_OK 0
#define CA_ERR_ARG 1
#define CA_ERR_CUDA 2
#define CA_ERR_UNSUPPORTED 3
#define CA_ERR_TIMEOUT 4

extern "C" const char* cuteafd_last_error();
int ca_fail(int code, const char* fmt, ...);
int ca_cuda(cudaError_t e, const char* what);
#define CA_CHECK_LAUNCH(what) do { cudaError_t _e = cudaGetLastError(); if (_e != cudaSuccess) return ca_cuda(_e, what); } while (0)
#define CA_REQUIRE(cond, ...) do { if (!(cond)) return ca_fail(CA_ERR_ARG, __VA_ARGS__); } while (0)

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// ------------------------------------------------------------------ programmatic dependent launch
// Kernels launched with CA_LAUNCH_PDL may become resident before the previous kernel in the stream has
// finished; they run their prologue (barrier init, tensor-memory alloc, loads of STATIC data such as weights)
// and must execute pdl_wait() before touching anything an earlier kernel produced and before their first
// global write.  pdl_launch() lets the NEXT kernel in the stream start its own prologue.  Both are no-ops
// for a kernel launched the ordinary way, so a kernel may be launched either way.
#ifdef CA_PDL_AFTER_WAIT
// Variant: a kernel releases its dependents only once it has itself been released, so at most ONE later kernel of the stream is
// resident early (with the release at kernel entry a whole chain of later kernels can cascade onto the SMs and hold shared / tensor
// memory that the running kernel's remaining CTAs need).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n\tgriddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() {}
#else
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif
// Classes: bit 0 glue kernels (norm, quant, routing, sampling), bit 1 GEMM, bit 2 attention; a file names its class
// with CA_PDL_CLASS before including this header.
int ca_pdl_enabled(int cls);
#ifndef CA_PDL_CLASS
#define CA_PDL_CLASS 0
#endif
#define CA_LAUNCH_PDL(kern_, grid_, block_, smem_, stream_, ...)                                              \
  do {                                                                                                   \
    cudaLaunchConfig_t _cfg = {};                                                                        \
    _cfg.gridDim = dim3(grid_); _cfg.blockDim = dim3(block_); _cfg.dynamicSmemBytes = (smem_); _cfg.stream = (stream_); \
    cudaLaunchAttribute _at[1];                                                                          \
    _at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                      \
    _at[0].val.programmaticStreamSerializationAllowed = 1;                                               \
    _cfg.attrs = _at; _cfg.numAttrs = ca_pdl_enabled(CA_PDL_CLASS) ? 1 : 0;                                          \
    cudaError_t _le = cudaLaunchKernelEx(&_cfg, kern_, __VA_ARGS__);                                      \
    if (_le != cudaSuccess) return ca_cuda(_le, #kern_ " launch");                                        \
  } while (0)

// Device status word layout (one int per kernel family, owned by the caller):
// 0 = ok; otherwise (code << 24) | detail.  Written with atomicCAS so the first failure wins.
#define CA_DEV_TIMEOUT_PRODUCER 1
#define CA_DEV_TIMEOUT_MMA 2
#define CA_DEV_TIMEOUT_EPILOGUE 3
#define CA_DEV_TIMEOUT_FLAG 4
#define CA_DEV_BAD_INDEX 5

__device__ __forceinline__ void ca_dev_fail(int* status, int code, int detail) {
  if (status) atomicCAS(status, 0, (code << 24) | (detail & 0xFFFFFF));
}

// ------------------------------------------------------------------ math
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is >= 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}

// ------------------------------------------------------------------ formats
__device__ __forceinline__ float e2m1_to_float(uint32_t c) {
  // magnitudes 0,.5,1,1.5,2,3,4,6 ; bit3 = sign
  const float tab[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  float m = tab[c & 7];
  return (c & 8) ? -m : m;
}
// round-to-nearest, ties to even code, saturating; matches ref.quant.e2m1_encode
__device__ __forceinline__ uint32_t float_to_e2m1(float x) {
  float a = fabsf(x);
  uint32_t c;
  if (a <= 0.25f) c = 0; else if (a < 0.75f) c = 1; else if (a <= 1.25f) c = 2; else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4; else if (a < 3.5f) c = 5; else if (a <= 5.0f) c = 6; else c = 7;
  return (x < 0.f && c != 0) ? (c | 8u) : c;
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __nv_fp8_e4m3 v; v.__x = b; return float(v);
}
__device__ __forceinline__ uint8_t float_to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float ue8m0_to_float(uint8_t b) {
  return __uint_as_float(b == 0 ? 0x00400000u : ((uint32_t)b << 23));  // 2^(b-127); b=0 -> 2^-127 (denormal)
}
__device__ __forceinline__ uint8_t ue8m0_ceil(float s) {
  // smallest power of two >= s (s > 0)
  uint32_t u = __float_as_uint(s);
  uint32_t e = (u >> 23) & 0xFF;
  if (u & 0x7FFFFF) e += 1;
  return (uint8_t)min(e, 254u);
}

// FP4 block quantisation of 8 consecutive values held by this thread.  The block (16 values NVFP4, 32 values MXFP4)
// spans 2 or 4 adjacent lanes, which must call this together (full warp converged).  Returns the 8 packed E2M1
// codes; `sb` is the block's scale byte (E4M3 with the static global scale 1/inv_gs, or UE8M0).  Same arithmetic as
// the stand-alone quantiser kernel, so fused and unfused paths produce identical bytes.
template <bool MX>
__device__ __forceinline__ uint32_t quant8_fp4(const float* v, float inv_gs, uint8_t& sb) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  float eff;
  if (MX) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int e = amax > 0.f ? (int)((__float_as_uint(amax) >> 23) & 0xFF) - 2 : 0;   // OCP MX: floor(log2(amax)) - 2
    e = max(e, 0); e = min(e, 254);
    sb = (uint8_t)e;
    eff = ue8m0_to_float(sb);
  } else {
    sb = float_to_e4m3(fminf(amax * inv_gs / 6.f, 448.f));
    eff = e4m3_to_float(sb) / inv_gs;
  }
  const float inv = eff > 0.f ? 1.f / eff : 0.f;
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) w |= float_to_e2m1(v[j] * inv) << (4 * j);
  return w;
}
// Writes one thread's share of a quantised row: codes of elements [i, i+8) and, from the first lane of the block,
// the scale byte.  qkind 1 = NVFP4, 2 = MXFP4.
__device__ __forceinline__ void quant8_store(const float* v, int qkind, float inv_gs, uint8_t* q_row, uint8_t* sf_row, int i) {
  uint8_t sb;
  if (qkind == 2) {
    const uint32_t w = quant8_fp4<true>(v, 1.f, sb);
    *(uint32_t*)(q_row + i / 2) = w;
    if (((i >> 3) & 3) == 0) sf_row[i >> 5] = sb;
  } else {
    const uint32_t w = quant8_fp4<false>(v, inv_gs, sb);
    *(uint32_t*)(q_row + i / 2) = w;
    if (((i >> 3) & 1) == 0) sf_row[i >> 4] = sb;
  }
}

// FP8 activation rows for the 128 x 128 block-scaled GEMM (qkind 3): this thread holds 8 consecutive elements starting at
// column i, 16 consecutive lanes hold one 128-channel block; E4M3 bytes go to q_row[i .. i + 8), the block's fp32 scale
// (amax floored at 1e-4, / 448: the stand-alone quantiser's arithmetic) to sa_row[i / 128].  All 32 lanes must call it.
__device__ __forceinline__ void quant8_store_fp8b(const float* v, uint8_t* q_row, float* sa_row, int i) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1)); amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4)); amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
  const float scale = fmaxf(amax, 1e-4f) / 448.f;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) { lo |= (uint32_t)float_to_e4m3(v[j] / scale) << (8 * j); hi |= (uint32_t)float_to_e4m3(v[4 + j] / scale) << (8 * j); }
  *(uint2*)(q_row + i) = make_uint2(lo, hi);
  if (((i >> 3) & 15) == 0) sa_row[i >> 7] = scale;
}

// ------------------------------------------------------------------ PTX: smem / mbarrier
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Non-blocking probe of a phase (the try_wait form may suspend the thread for a while, which is wrong for a thread
// that polls several barriers).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait (about two seconds of wall time).  Returns false when the limit ran out or another role
// of the CTA already raised `*abort_flag`; the caller then unwinds instead of spinning.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  uint64_t timeout_ns = 2000000000ull) {
  // The SM cycle counter bounds the wait (cheap to read; ~2 cycles per ns is an upper bound on the clock,
  // so the wall-time limit is at least `timeout_ns`).
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64(), limit = (long long)timeout_ns * 2;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------ PTX: TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)m) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// Streamed operands (expert / projection weights, their scales, the KV pages of a decode step) are read once per step and are far
// larger than L2: loaded with an evict-first policy they pass through without pushing out what the step's small kernels keep
// re-reading from L2 between the big loads (activations, routing tables, norm weights - and the kernels' own instructions).
__device__ __forceinline__ uint64_t l2_policy_stream() {
  uint64_t p;
#ifndef CA_NO_STREAM_HINT
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
#else
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
#endif
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_3d_hint(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, uint64_t pol) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
               ::"r"(smem_u32(dst)), "l"((uint64_t)m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "l"(pol) : "memory");
}
__device__ __forceinline__ void bulk_load_1d_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_u32(dst)), "l"((uint64_t)src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol) : "memory");
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"((uint64_t)src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// ------------------------------------------------------------------ PTX: tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc];  kind::f16 (bf16/fp16 inputs, fp32 accumulate)
__device__ __forceinline__ void tc_mma_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Same with the A operand in tensor memory: lane = row, each 32-bit column holds two consecutive K elements
// (8 columns per K = 16 instruction).  A read from tensor memory costs no shared-memory bandwidth.
__device__ __forceinline__ void tc_mma_f16_ta(uint32_t d, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// kind::f8f6f4 (e4m3/e5m2/e2m1-padded inputs, fp32 accumulate), K = 32 per instruction
__device__ __forceinline__ void tc_mma_f8(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Block-scaled FP4: NVFP4 (E4M3 scale per 16, K = 64 per instruction)
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                            uint32_t sfa, uint32_t sfb) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
// Block-scaled FP4: MXFP4 (UE8M0 scale per 32, K = 64 per instruction)
__device__ __forceinline__ void tc_mma_mxf4(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                            uint32_t sfa, uint32_t sfb) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
// Block-scaled FP8/FP6/FP4 mix (UE8M0 scale per 32, K = 32 per instruction)
__device__ __forceinline__ void tc_mma_mxf8f6f4(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                                uint32_t sfa, uint32_t sfb) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
// Scale factors: 32 rows x 128 bits from shared memory into 4 TMEM columns, replicated to all 4 lane quarters.
__device__ __forceinline__ void tc_cp_sf(uint32_t tmem_dst, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(sdesc) : "memory");
}
// 32 lanes x 32-bit, N consecutive columns -> N registers per thread
__device__ __forceinline__ void tmem_ld_x8(uint32_t addr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t addr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(addr));
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes wide and
// stored with the 128-byte swizzle (what a TMA box of {128 B, rows} with SWIZZLE_128B writes):
// 8-row groups are 1024 B apart (stride byte offset), layout type 2, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address
  d |= (uint64_t)1 << 16;                           // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset
  d |= (uint64_t)1 << 46;                           // version = 1 (Blackwell)
  d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
  return d;
}
// Descriptor for a 32-row x 16-byte scale-factor chunk (no swizzle, 8-row groups 128 B apart).
__device__ __forceinline__ uint64_t umma_desc_sf(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// ------------------------------------------------------------------ PTX: system-scope flags (peer memory)
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait until *flag >= want (monotonic sequence numbers).  Gives up after `timeout_ns`; returns false.
__device__ __forceinline__ bool wait_flag_bounded(const uint32_t* flag, uint32_t want, uint64_t timeout_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
      __nanosleep(32);
    }
    if (globaltimer_ns() - t0 > timeout_ns) return false;
  }
}

// A flag wait folded into the kernel that consumes what the peer sent (instead of a wait-only launch in front of
// it): threads 0..n-1 of every block poll flags[i * stride] >= ctl[1] (the current step) with the usual time limit;
// on failure the status word and the abort word ctl[0] are set and the block learns it must not touch the data.
struct FlagWait {
  const uint32_t* flags; uint32_t* ctl; int* status; unsigned long long timeout_ns; int n, stride;
};
__device__ __forceinline__ bool flag_wait_block(const FlagWait& w) {
  if (!w.flags) return true;
  __shared__ int fw_ok;
  if (threadIdx.x == 0) fw_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < w.n) {
    if (w.ctl[0]) fw_ok = 0;
    else if (!wait_flag_bounded(w.flags + (size_t)threadIdx.x * w.stride, w.ctl[1], w.timeout_ns)) {
      ca_dev_fail(w.status, CA_DEV_TIMEOUT_FLAG, (int)threadIdx.x);
      atomicExch(&w.ctl[0], 1u);
      fw_ok = 0;
    }
  }
  __syncthreads();
  return fw_ok != 0;
}
// Optional arguments cross the C ABI as explicit host structs passed by pointer (null = absent): nothing is armed for "the
// next call of this thread".
struct CaFlagWaitArg {        // in-kernel wait in front of a consumer of peer data (route_pack, moe_combine[_norm])
  const void* flags; void* ctl; int* status; unsigned long long timeout_ns; int n, stride;
};
struct CaTcExtra {            // tc_linear: FP4 copy of the output and/or stores of the output tile into peers' memory
  void* q_out; void* sf_out; const float* inv_gs_out; int ldsf_out; int n_peer;
  void* peer_y[2]; void* peer_flag[2]; const int* peer_row_map; void* peer_ctl; void* peer_done; int peer_ld; int reserved;
};
static inline FlagWait ca_flag_wait_from(const CaFlagWaitArg* a) {
  FlagWait w = {nullptr, nullptr, nullptr, 0ull, 0, 0};
  if (a && a->flags && a->n > 0) {
    w.flags = (const uint32_t*)a->flags; w.ctl = (uint32_t*)a->ctl; w.status = a->status;
    w.timeout_ns = a->timeout_ns; w.n = a->n > 32 ? 32 : a->n; w.stride = a->stride;
  }
  return w;
}

// ------------------------------------------------------------------ host: TMA descriptor encode
// Resolved at run time from the driver so the library links without libcuda.
int ca_encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw);
int ca_encode_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                      CUtensorMapSwizzle sw);
int ca_sm_count();
