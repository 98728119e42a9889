// Host runtime for the native library: status/error ABI, device info, TMA descriptor encoding
// (driver entry point resolved at run time, so nothing links against libcuda), and a few
// stream-ordered utilities.  Counterpart of the reference's C ABI core
// (native/shared/src/cuteafd_native.cc: status/last-error, device info, copies).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_err[512] = "";

extern "C" const char* cuteafd_last_error() { return g_err; }

int ca_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int ca_cuda(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
  return CA_ERR_CUDA;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int ca_encode_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint64_t d0, uint64_t d1, uint64_t d2,
                      uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                      CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return ca_fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (((uintptr_t)base & 15) || (stride1_bytes & 15) || (stride2_bytes & 15))
    return ca_fail(CA_ERR_ARG, "TMA operand must be 16-byte aligned with 16-byte-multiple strides");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return ca_fail(CA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return CA_OK;
}

int ca_encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
  return ca_encode_tmap_3d(out, base, dt, inner, outer, 1, row_stride_bytes, row_stride_bytes * outer, box_inner,
                           box_outer, 1, sw);
}

int ca_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return sms[dev] > 0 ? sms[dev] : 148;
}

// Programmatic dependent launch switch: a bit mask over kernel classes (bit 0 glue, bit 1 GEMM, bit 2 attention);
// -1 = not decided yet (environment CUTEAFD_PDL=<mask>; default 2: measured on B200, GEMM-only is the one setting that pays - chains of
// early-resident kernels take shared memory from the attention kernel and cost more than they save).
static int g_pdl = -1;
int ca_pdl_enabled(int cls) {
  if (g_pdl < 0) {
    const char* e = getenv("CUTEAFD_PDL");
    g_pdl = e ? atoi(e) & 7 : 2;
  }
  return (g_pdl >> cls) & 1;
}

extern "C" {

// Sets the programmatic-dependent-launch class mask for later launches of this process; returns the old mask.
int cuteafd_set_pdl(int mask) {
  ca_pdl_enabled(0);
  int old = g_pdl;
  g_pdl = mask & 7;
  return old;
}

// Fills a 128-byte host buffer with a tiled TMA descriptor for a K-major operand whose box is
// {128 bytes of K, box_rows rows} with the 128-byte swizzle.  elem_bytes: 1 (fp8 / packed fp4 bytes) or 2 (bf16).
// dims: [groups, rows, k_elems]; strides in bytes.
int cuteafd_tmap_encode_kmajor(void* out128, const void* base, int elem_bytes, uint64_t k_elems, uint64_t rows,
                               uint64_t groups, uint64_t row_stride_bytes, uint64_t group_stride_bytes,
                               uint32_t box_rows) {
  // elem_bytes 0: packed 4-bit elements (two per byte in global memory) that TMA unpacks into 8-bit containers, 16 elements
  // per 16-byte chunk, as tcgen05 kind::f8f6f4 / mxf8f6f4 want their sub-byte operands; k_elems then counts 4-bit elements.
  CA_REQUIRE(elem_bytes == 0 || elem_bytes == 1 || elem_bytes == 2, "elem_bytes must be 0 (packed 4-bit), 1 or 2");
  CA_REQUIRE(box_rows >= 1 && box_rows <= 256, "box_rows out of range");
  CA_REQUIRE(elem_bytes != 0 || (k_elems % 128 == 0 && row_stride_bytes % 32 == 0 && ((uintptr_t)base & 31) == 0),
             "packed 4-bit operands need K %% 128 == 0, 32-byte aligned rows and base");
  CUtensorMap m;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : (elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B);
  uint64_t gs = groups > 1 ? group_stride_bytes : row_stride_bytes * rows;
  int rc = ca_encode_tmap_3d(&m, base, dt, k_elems, rows, groups ? groups : 1, row_stride_bytes, gs,
                             elem_bytes ? 128 / elem_bytes : 128, box_rows, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  memcpy(out128, &m, sizeof(m));
  return CA_OK;
}

int cuteafd_device_info(int* sms, int* cc_major, int* cc_minor, size_t* free_b, size_t* total_b) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return ca_cuda(e, "cudaGetDevice");
  cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(cc_major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
  e = cudaMemGetInfo(free_b, total_b);
  if (e != cudaSuccess) return ca_cuda(e, "cudaMemGetInfo");
  return CA_OK;
}

int cuteafd_abi_version() { return 1; }

}  // extern "C"
