// Pointwise kernels of the vision tower (a ViT encoder in front of the decoder: patch embedding, `depth` pre-norm blocks of
// bidirectional multi-head attention + MLP, a 2x2 spatial merger).  The GEMMs are `tc_linear` (bf16 tcgen05), the attention is
// `gqa_prefill_kernel` in its bidirectional mode over a scratch paged store whose heads are zero-padded to 128 dimensions; what is
// left is memory-bound glue, fused so that every activation crosses HBM once per block half:
//   rgb_patches      resized RGB8 image -> normalised bf16 patch rows in merge-group order (the order the merger concatenates)
//   add_norm         x (fp32 residual) += y + bias of the GEMM before, then LayerNorm / RMSNorm to the bf16 input of the next GEMM
//   qkv_rope_store   bias, optional per-head q/k RMSNorm, 2-D rotary embedding, q padded to 128 wide, k / v rows into the paged store
//   bias_act         bias + GELU (erf or tanh form) or SwiGLU between the two MLP GEMMs
//
// Reference: native/shared/cuda/vision.cu (rmsnorm / layernorm / add_bias_residual / swiglu_bias / gelu / rope_qkv kernels),
// native/shared/cuda/vision_qwen.cuh, native/shared/cuda/vision_glm.cuh (per-family glue), native/shared/include/cuteafd_vision.h
// (fp32 residual, bf16 dense inputs).
#include "common.cuh"

// One block per patch.  Row order: merge groups row-major over the (gh / m, gw / m) grid, the m x m patches of a group row-major
// inside it; columns (channel, py, px), zero-padded to Kp.
__global__ void vision_rgb_patches_kernel(const uint8_t* __restrict__ rgb, const float* __restrict__ lut, bf16* __restrict__ out,
                                          int gh, int gw, int P, int m, int Kp) {
  const int row = blockIdx.x;
  const int gpr = gw / m, grp = row / (m * m), in = row % (m * m);
  const int py0 = ((grp / gpr) * m + in / m) * P, px0 = ((grp % gpr) * m + in % m) * P;
  const int W = gw * P, K = 3 * P * P;
  for (int c = threadIdx.x; c < Kp; c += blockDim.x) {
    float v = 0.f;
    if (c < K) {
      const int ch = c / (P * P), py = (c / P) % P, px = c % P;
      v = lut[ch * 256 + rgb[((size_t)(py0 + py) * W + px0 + px) * 3 + ch]];
    }
    out[(size_t)row * Kp + c] = __float2bfloat16(v);
  }
}

// One block per row.  x = (init ? 0 : x) + y + ybias (when y), then out = norm(x) * w (+ b: LayerNorm, b null: RMSNorm).
__global__ void __launch_bounds__(256) vision_add_norm_kernel(float* __restrict__ x, const bf16* __restrict__ y, int ldy,
                                                              const float* __restrict__ ybias, const float* __restrict__ w,
                                                              const float* __restrict__ b, bf16* __restrict__ out, int H, float eps,
                                                              int init) {
  pdl_launch(); pdl_wait();
  __shared__ float red[32];
  float* xr = x + (size_t)blockIdx.x * H;
  float s = 0.f, ss = 0.f;
  for (int c = threadIdx.x; c < H; c += 256) {
    float v = init ? 0.f : xr[c];
    if (y) {
      v += __bfloat162float(y[(size_t)blockIdx.x * ldy + c]) + (ybias ? ybias[c] : 0.f);
      xr[c] = v;
    }
    s += v; ss += v * v;
  }
  if (!out) return;
  float mean = 0.f, var;
  if (b) {
    mean = block_sum(s, red) / H;
    float d2 = 0.f;
    for (int c = threadIdx.x; c < H; c += 256) { const float d = xr[c] - mean; d2 += d * d; }     // own writes: visible to this thread
    var = block_sum(d2, red) / H;
  } else {
    var = block_sum(ss, red) / H;
  }
  const float rstd = rsqrtf(var + eps);
  for (int c = threadIdx.x; c < H; c += 256) {
    const float v = (xr[c] - mean) * rstd * w[c] + (b ? b[c] : 0.f);
    out[(size_t)blockIdx.x * H + c] = __float2bfloat16(v);
  }
}

// grid (tokens, heads), 128 threads: thread d owns dimension d of the head (hd <= 128).  cs[t] = cos[hd / 2] | sin[hd / 2] of the
// token's (row, column) angles; rotation pairs (d, d + hd / 2).  q -> q_out[t, h, 128], k / v -> kv[slot[t], 0 / 1, h, 128].
__global__ void __launch_bounds__(128) vision_qkv_rope_store_kernel(const bf16* __restrict__ qkv, const float* __restrict__ bias,
                                                                    const float* __restrict__ cs, const float* __restrict__ qw,
                                                                    const float* __restrict__ kw, bf16* __restrict__ q_out,
                                                                    bf16* __restrict__ kv, const int* __restrict__ slot, int nh, int hd,
                                                                    float eps, int* status) {
  pdl_launch(); pdl_wait();
  __shared__ float sq[128], sk[128], red[32];
  const int t = blockIdx.x, h = blockIdx.y, d = threadIdx.x, HD = nh * hd, half = hd / 2;
  const bool live = d < hd;
  float q = 0.f, k = 0.f, v = 0.f;
  if (live) {
    const bf16* r = qkv + (size_t)t * 3 * HD + h * hd + d;
    q = __bfloat162float(r[0]) + (bias ? bias[h * hd + d] : 0.f);
    k = __bfloat162float(r[HD]) + (bias ? bias[HD + h * hd + d] : 0.f);
    v = __bfloat162float(r[2 * HD]) + (bias ? bias[2 * HD + h * hd + d] : 0.f);
  }
  if (qw) {                                   // per-head RMSNorm of q and k before the rotation
    const float nq = block_sum(q * q, red), nk = block_sum(k * k, red);
    if (live) { q *= rsqrtf(nq / hd + eps) * qw[d]; k *= rsqrtf(nk / hd + eps) * kw[d]; }
  }
  sq[d] = q; sk[d] = k;
  __syncthreads();
  if (live) {
    const int j = d < half ? d : d - half;
    const float c = cs[(size_t)t * hd + j], s = cs[(size_t)t * hd + half + j];
    const float pq = d < half ? -sq[d + half] : sq[d - half], pk = d < half ? -sk[d + half] : sk[d - half];
    q = q * c + pq * s;
    k = k * c + pk * s;
  }
  const int sl = slot[t];
  if (sl < 0) { if (d == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, 0xB10); return; }
  q_out[((size_t)t * nh + h) * 128 + d] = __float2bfloat16(q);
  bf16* dst = kv + ((size_t)sl * 2 * nh + h) * 128 + d;
  dst[0] = __float2bfloat16(k);
  dst[(size_t)nh * 128] = __float2bfloat16(v);
}

__device__ __forceinline__ float vision_gelu(float x, int tanh_form) {
  if (tanh_form) return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}

// act 0: y + bias; 1: GELU (erf); 2: GELU (tanh); 3: SwiGLU over y = [gate | up] (bias covers both halves).  out [rows, n_out].
__global__ void vision_bias_act_kernel(const bf16* __restrict__ y, int ldy, const float* __restrict__ bias, bf16* __restrict__ out,
                                       int ldo, int rows, int n_out, int act) {
  pdl_launch(); pdl_wait();
  const size_t n = (size_t)rows * n_out;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / n_out), c = (int)(i % n_out);
    float v = __bfloat162float(y[(size_t)r * ldy + c]) + (bias ? bias[c] : 0.f);
    if (act == 3) {
      const float u = __bfloat162float(y[(size_t)r * ldy + n_out + c]) + (bias ? bias[n_out + c] : 0.f);
      v = v / (1.f + __expf(-v)) * u;
    } else if (act) {
      v = vision_gelu(v, act == 2);
    }
    out[(size_t)r * ldo + c] = __float2bfloat16(v);
  }
}

// Width-3 convolution as a GEMM: dst[t, k * C + c] = src[t * stride + k - 1, c] (zero rows outside [0, T)); 16-byte vectors.
// The audio tower's two convolutions over the frame axis (stride 1, then stride 2) read their operand rows from this.
__global__ void audio_im2col3_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int T, int T_out, int C8, int stride) {
  pdl_launch(); pdl_wait();
  const size_t n = (size_t)T_out * 3 * C8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / (3 * C8)), r = (int)(i % (3 * C8)), k = r / C8, c = r % C8;
    const int ts = t * stride + k - 1;
    dst[i] = (ts >= 0 && ts < T) ? src[(size_t)ts * C8 + c] : make_uint4(0, 0, 0, 0);
  }
}

extern "C" int cuteafd_audio_im2col3(const void* src, void* dst, int T, int C, int stride, cudaStream_t s) {
  CA_REQUIRE(src && dst && C % 8 == 0 && (stride == 1 || stride == 2) && (stride == 1 || T % 2 == 0), "audio_im2col3: C %% 8 == 0, stride 1 or 2");
  if (T <= 0) return CA_OK;
  const int T_out = T / stride;
  const size_t n = (size_t)T_out * 3 * (C / 8);
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  CA_LAUNCH_PDL(audio_im2col3_kernel, blocks, 256, 0, s, (const uint4*)src, (uint4*)dst, T, T_out, C / 8, stride);
  CA_CHECK_LAUNCH("audio_im2col3");
  return CA_OK;
}

extern "C" int cuteafd_vision_rgb_patches(const uint8_t* rgb, const float* lut, void* out, int gh, int gw, int P, int merge, int Kp,
                                          cudaStream_t s) {
  CA_REQUIRE(rgb && lut && out && gh > 0 && gw > 0 && P > 0 && merge > 0 && gh % merge == 0 && gw % merge == 0 && Kp >= 3 * P * P,
             "vision_rgb_patches: grid %d x %d must be whole merge groups of %d and Kp >= 3 P^2", gh, gw, merge);
  vision_rgb_patches_kernel<<<gh * gw, 256, 0, s>>>(rgb, lut, (bf16*)out, gh, gw, P, merge, Kp);
  CA_CHECK_LAUNCH("vision_rgb_patches");
  return CA_OK;
}

extern "C" int cuteafd_vision_add_norm(float* x, const void* y, int ldy, const float* ybias, const float* w, const float* b, void* out,
                                       int rows, int H, float eps, int init, cudaStream_t s) {
  CA_REQUIRE(x && rows >= 0 && H > 0 && (!out || w) && (y || !init), "vision_add_norm: bad arguments");
  if (!rows) return CA_OK;
  CA_LAUNCH_PDL(vision_add_norm_kernel, rows, 256, 0, s, x, (const bf16*)y, ldy, ybias, w, b, (bf16*)out, H, eps, init);
  CA_CHECK_LAUNCH("vision_add_norm");
  return CA_OK;
}

extern "C" int cuteafd_vision_qkv_rope_store(const void* qkv, const float* bias, const float* cs, const float* qw, const float* kw,
                                             void* q_out, void* kv, const int* slot, int rows, int nh, int hd, float eps, int* status,
                                             cudaStream_t s) {
  CA_REQUIRE(qkv && cs && q_out && kv && slot && nh > 0 && hd > 0 && hd <= 128 && hd % 2 == 0 && (!qw == !kw),
             "vision_qkv_rope_store: head_dim %d must be even and <= 128", hd);
  if (rows <= 0) return CA_OK;
  CA_LAUNCH_PDL(vision_qkv_rope_store_kernel, dim3(rows, nh), 128, 0, s, (const bf16*)qkv, bias, cs, qw, kw, (bf16*)q_out, (bf16*)kv, slot,
                nh, hd, eps, status);
  CA_CHECK_LAUNCH("vision_qkv_rope_store");
  return CA_OK;
}

extern "C" int cuteafd_vision_bias_act(const void* y, int ldy, const float* bias, void* out, int ldo, int rows, int n_out, int act,
                                       cudaStream_t s) {
  CA_REQUIRE(y && out && n_out > 0 && act >= 0 && act <= 3, "vision_bias_act: bad arguments");
  if (rows <= 0) return CA_OK;
  const size_t n = (size_t)rows * n_out;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  CA_LAUNCH_PDL(vision_bias_act_kernel, blocks, 256, 0, s, (const bf16*)y, ldy, bias, (bf16*)out, ldo, rows, n_out, act);
  CA_CHECK_LAUNCH("vision_bias_act");
  return CA_OK;
}
