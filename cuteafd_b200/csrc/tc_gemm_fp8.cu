// FP8 (E4M3) linear layer with DeepSeek-style block scales for sm_100a:
//   Y[rows, N] = sum_kb  sa[row, kb] * sw[n / 128, kb] * ( Xq[rows, kb-th 128 of K] * Wq[N, same 128]^T )
// weights carry one fp32 scale per 128 x 128 block (the checkpoint's `weight_scale_inv`), activations one fp32 scale
// per token and 128 channels (quantised on the fly by `act_quant_fp8_block128`).
//
// tcgen05 has no 128-wide fp32 block scaling, so the scaling happens between the tensor core and the registers:
// one pipeline stage is exactly one scale block (128 bytes of K per row, four kind::f8f6f4 MMAs of K = 32), each
// stage accumulates into a FRESH tensor-memory buffer (ring of four), and the epilogue warps pull every finished
// buffer with tcgen05.ld and add it, scaled, to fp32 registers while the next stages run.  swap-AB as in the other
// GEMMs (weight rows = MMA M, tokens = MMA N = 16..128), one work unit (128 x TN tile, one K slice) per CTA, optional
// split-K over a thread-block cluster with the partial tiles reduced through distributed shared memory.
//
// Reference counterparts: the W8A8 FP8 GEMV/GEMM (native/shared/cuda/fp8_gemv.cu, fp8_block.cu) and the block-scale
// handling of the FP8 backbone (families/deepseek_v4/engine.rs:1320-1390).
#define CA_PDL_CLASS 1
#include "common.cuh"

enum { F8_EPI_BF16 = 0, F8_EPI_BF16_RESIDUAL = 1, F8_EPI_F32 = 3 };

struct Fp8Args {
  const CUtensorMap* tmA;   // weights [N, K] bytes, box {128, 128}
  const CUtensorMap* tmB;   // activations [rows, K] bytes, box {128, TN}
  const float* sw;          // [ceil(N / 128), ceil(K / 128)]
  const float* sa;          // [rows, ceil(K / 128)]
  void* Y;
  const bf16* R;
  int* status;
  int ldy, rows_total, N, K, epi, splits;
  int budget;               // bytes of shared memory for ring + staging + scale table: 200 KB (one CTA per SM) or 100 KB (two per SM)
};

template <int TN>
struct Fp8Cfg {
  static constexpr int A_BYTES = 128 * 128, B_BYTES = TN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int NACC = 4;
  static constexpr int TMEM_COLS = NACC * TN < 32 ? 32 : NACC * TN;       // 64 / 128 / 256 / 512
  static constexpr int BUDGET = 200 * 1024, MAX_RING = 8;
  static constexpr int SMEM_BYTES = BUDGET + 1024;
  // Shared memory = stage ring + staging area of the cluster reduction + the table of combined scales
  // sa[token, kb] * sw[n / 128, kb] of this CTA's K slice (one fp32 per token and stage; without the table every stage
  // exposed two dependent global loads, ~0.5 us, in the epilogue warps).
  __host__ __device__ static constexpr int table_bytes(int nk) { return nk * TN * 4 <= 64 * 1024 ? nk * TN * 4 : 0; }
  // decode-sized tiles keep one more staging tile: rank 0's own partial, so that the tile can be finished row-wise (16-byte stores)
  static constexpr int OWN = TN <= 32 ? 1 : 0;
  __host__ __device__ static constexpr int ring(int S, int nk, int budget = BUDGET) {
    return (budget - (S - 1 + OWN) * 128 * TN * 4 - table_bytes(nk)) / STAGE_BYTES > MAX_RING
               ? MAX_RING : (budget - (S - 1 + OWN) * 128 * TN * 4 - table_bytes(nk)) / STAGE_BYTES;
  }
};

__device__ __forceinline__ uint32_t f8_cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void f8_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int TN>
__global__ void __launch_bounds__(192, (TN <= 32 ? 2 : 1)) fp8_linear_kernel(const __grid_constant__ Fp8Args a) {
  using C = Fp8Cfg<TN>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[C::MAX_RING], empty_bar[C::MAX_RING], accf_bar[C::NACC], acce_bar[C::NACC];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.splits > 1 ? a.splits : 1;
  const int nk_max = ((a.K + 127) / 128 + S - 1) / S;                      // stages of the longest K slice
  const int ring = C::ring(S, nk_max, a.budget);
  float* staging = (float*)(smem + ring * C::STAGE_BYTES);                 // [S-1][TN][128] fp32 on cluster rank 0
  float* sc_tab = staging + (size_t)(S - 1 + C::OWN) * 128 * TN;           // [stages of my slice][TN] combined scales
  const bool use_tab = C::table_bytes(nk_max) > 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::MAX_RING; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < C::NACC; ++b) { mbar_init(&accf_bar[b], 1); mbar_init(&acce_bar[b], 128); }
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  pdl_launch();

  const int sp = (int)f8_cluster_ctarank();
  const int tile = (int)blockIdx.x / S;
  const int n_nt = (a.N + 127) / 128;
  const int item = tile / n_nt, nt = tile % n_nt;
  const int row0 = item * TN, nrows = min(TN, a.rows_total - row0);
  const int nkb_all = (a.K + 127) / 128;
  const int kb0 = (int)(((long long)nkb_all * sp) / S), kb1 = (int)(((long long)nkb_all * (sp + 1)) / S);
  volatile int* abortp = &abort_flag;

  float acc[TN];
#pragma unroll
  for (int j = 0; j < TN; ++j) acc[j] = 0.f;
  const int q4 = warp & 3, et = q4 * 32 + lane;
  constexpr bool RES_PRE = TN <= 32;
  float res_pre[RES_PRE ? TN : 1];
#pragma unroll
  for (int j = 0; j < (RES_PRE ? TN : 1); ++j) res_pre[j] = 0.f;
  // row-wise finish of a decode-sized tile by rank 0 (see the staging tile above): (token, 8 features) items, 16-byte accesses
  constexpr int ITEMS = RES_PRE ? TN / 8 : 1;
  const bool vec_ok = RES_PRE && a.N % 8 == 0 && a.ldy % 8 == 0 && ((uintptr_t)a.Y & 15) == 0 &&
                      (a.epi != F8_EPI_BF16_RESIDUAL || ((uintptr_t)a.R & 15) == 0);
  const int tid128 = warp >= 2 ? (warp - 2) * 32 + lane : 0;
  uint4 rv_pre[ITEMS];
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) rv_pre[j] = make_uint4(0u, 0u, 0u, 0u);

  if (warp == 0) {
    // ---- producer: weight tiles first (static data), then wait for the previous kernel, then activation tiles
    const uint64_t wpol = a.rows_total <= TN ? l2_policy_stream() : l2_policy_normal();    // one token tile: every weight byte is read once
    const int npre = min(ring, kb1 - kb0);
    if (lane == 0)
      for (int i = 0; i < npre; ++i) {
        mbar_expect_tx(&full_bar[i], C::STAGE_BYTES);
        tma_load_3d_hint(smem + i * C::STAGE_BYTES, a.tmA, &full_bar[i], (kb0 + i) * 128, nt * 128, 0, wpol);
      }
    pdl_wait();
    for (int kb = kb0, it = 0; kb < kb1 && !*abortp; ++kb, ++it) {
      const int s = it % ring;
      if (it >= ring) {
        if (!mbar_wait_bounded(&empty_bar[s], ((it / ring) & 1) ^ 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, (int)blockIdx.x); break; }
        if (lane == 0) {
          mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
          tma_load_3d_hint(smem + s * C::STAGE_BYTES, a.tmA, &full_bar[s], kb * 128, nt * 128, 0, wpol);
        }
      }
      if (lane == 0) tma_load_3d(smem + s * C::STAGE_BYTES + C::A_BYTES, a.tmB, &full_bar[s], kb * 128, row0, 0);
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one fresh accumulator buffer per stage (= per scale block)
    pdl_wait();
    if (lane == 0) {
      const uint32_t smem_base = smem_u32(smem);
      const uint32_t idesc = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);   // E4M3 x E4M3 -> fp32
      for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
        const int s = it % ring, b = it % C::NACC;
        if (!mbar_wait_bounded(&acce_bar[b], ((it / C::NACC) & 1) ^ 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, (int)blockIdx.x); break; }
        if (!mbar_wait_bounded(&full_bar[s], (it / ring) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, (int)blockIdx.x); break; }
        tc_fence_after();
        const uint32_t st = smem_base + s * C::STAGE_BYTES;
        const uint64_t adesc = umma_desc_sw128(st), bdesc = umma_desc_sw128(st + C::A_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) tc_mma_f8(tmem + b * TN, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
        tc_commit(&empty_bar[s]);
        tc_commit(&accf_bar[b]);
      }
    }
    __syncwarp();
  } else {
    // ---- epilogue warps: scaled accumulation of every finished stage into registers
    pdl_wait();
    if (vec_ok && sp == 0 && a.epi == F8_EPI_BF16_RESIDUAL) {
      // decode-sized tiles: the residual rows are fetched under the main loop (and ahead of every store: R may alias Y)
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const int i = tid128 + it * 128, c = i >> 4, nn = nt * 128 + (i & 15) * 8;
        if (c < nrows && nn < a.N) rv_pre[it] = *(const uint4*)(a.R + (size_t)(row0 + c) * a.ldy + nn);
      }
    } else if (RES_PRE && sp == 0 && a.epi == F8_EPI_BF16_RESIDUAL && nt * 128 + et < a.N) {
#pragma unroll
      for (int j = 0; j < (RES_PRE ? TN : 1); ++j)
        if (j < nrows) res_pre[j] = __bfloat162float(a.R[(size_t)(row0 + j) * a.ldy + nt * 128 + et]);
    }
    const uint32_t tbase = tmem + ((uint32_t)(q4 * 32) << 16);
    bool ok = true;
    if (use_tab) {
      const int et128 = (warp - 2) * 32 + lane;          // 0..127 over the four epilogue warps
      for (int i = et128; i < (kb1 - kb0) * TN; i += 128) {
        const int kk = i / TN, tcol = i % TN;
        sc_tab[i] = (tcol < nrows) ? a.sa[(size_t)(row0 + tcol) * nkb_all + kb0 + kk] * a.sw[(size_t)nt * nkb_all + kb0 + kk] : 0.f;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
    }
    for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
      const int b = it % C::NACC;
      float sav[(TN + 15) / 16];                 // lane j (< 16) of chunk c holds the scale of token c * 16 + j
      if (use_tab) {
#pragma unroll
        for (int c = 0; c < (TN + 15) / 16; ++c) sav[c] = sc_tab[it * TN + c * 16 + (lane & 15)];
      } else {
        const float swv = a.sw[(size_t)nt * nkb_all + kb];
#pragma unroll
        for (int c = 0; c < (TN + 15) / 16; ++c) {
          const int tcol = c * 16 + (lane & 15);
          sav[c] = (tcol < nrows) ? a.sa[(size_t)(row0 + tcol) * nkb_all + kb] * swv : 0.f;
        }
      }
      ok = mbar_wait_bounded(&accf_bar[b], (it / C::NACC) & 1, abortp);
      ok = __all_sync(0xffffffffu, ok);          // tensor-memory loads must stay warp-uniform
      if (!ok) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, (int)blockIdx.x); break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < (TN + 15) / 16; ++c) {
        uint32_t r[16];
        tmem_ld_x16(tbase + b * TN + c * 16, r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c * 16 + j] += __uint_as_float(r[j]) * __shfl_sync(0xffffffffu, sav[c], j);
      }
      tc_fence_before();
      mbar_arrive(&acce_bar[b]);
    }
    if (S > 1 && sp != 0) {
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(staging)), "r"(0));
      remote += (uint32_t)(sp - 1) * (128 * TN * 4);
#pragma unroll
      for (int j = 0; j < TN; ++j)
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)(j * 128 + et) * 4), "f"(acc[j]) : "memory");
    } else if (vec_ok) {
      float* own = staging + (size_t)(S - 1) * (128 * TN);
#pragma unroll
      for (int j = 0; j < TN; ++j) own[j * 128 + et] = acc[j];
      if (S == 1) asm volatile("bar.sync 2, 128;" ::: "memory");     // the four epilogue warps; clusters meet at the barrier below
    }
  }
  __syncwarp();
  if (S > 1) f8_cluster_sync();              // every thread of every CTA of the cluster, exactly once
  if (warp >= 2 && sp == 0 && vec_ok) {
    const float* own = staging + (size_t)(S - 1) * (128 * TN);
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int i = tid128 + it * 128, c = i >> 4, g8 = (i & 15) * 8, nn = nt * 128 + g8;
      if (c < nrows && nn < a.N) {
        const float4 o0 = *(const float4*)(own + c * 128 + g8), o1 = *(const float4*)(own + c * 128 + g8 + 4);
        float f[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll 1
        for (int p = 1; p < S; ++p) {                                  // rank order, as the scalar path adds them
          const float* pp = staging + (size_t)(p - 1) * (128 * TN) + c * 128 + g8;
          const float4 p0 = *(const float4*)pp, p1 = *(const float4*)(pp + 4);
          f[0] += p0.x; f[1] += p0.y; f[2] += p0.z; f[3] += p0.w; f[4] += p1.x; f[5] += p1.y; f[6] += p1.z; f[7] += p1.w;
        }
        const size_t o = (size_t)(row0 + c) * a.ldy + nn;
        if (a.epi == F8_EPI_F32) {
          *(float4*)((float*)a.Y + o) = make_float4(f[0], f[1], f[2], f[3]);
          *(float4*)((float*)a.Y + o + 4) = make_float4(f[4], f[5], f[6], f[7]);
        } else {
          const bf16* rb = (const bf16*)&rv_pre[it];
          uint32_t wv[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const bf162 hh = __floats2bfloat162_rn(f[2 * q] + __bfloat162float(rb[2 * q]), f[2 * q + 1] + __bfloat162float(rb[2 * q + 1]));
            wv[q] = *(const uint32_t*)&hh;
          }
          *(uint4*)((bf16*)a.Y + o) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
      }
    }
  } else if (warp >= 2 && sp == 0) {
    const int n = nt * 128 + et;
    if (n < a.N) {
      // residual rows first, all in flight together: R may alias Y (in-place residual stream), so loads issued after a store
      // would wait for it, one L2 round trip per token row
#pragma unroll
      for (int j0 = 0; j0 < TN; j0 += 16) {
      float res[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (RES_PRE) res[j] = res_pre[(j0 + j) < (RES_PRE ? TN : 1) ? (j0 + j) : 0];
        else res[j] = (a.epi == F8_EPI_BF16_RESIDUAL && j0 + j < nrows) ? __bfloat162float(a.R[(size_t)(row0 + j0 + j) * a.ldy + n]) : 0.f;
      }
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        const int j = j0 + jj;
        if (j < nrows) {
          float v = acc[j];
          for (int p = 1; p < S; ++p) v += staging[(size_t)(p - 1) * (128 * TN) + j * 128 + et];
          const size_t o = (size_t)(row0 + j) * a.ldy + n;
          if (a.epi == F8_EPI_F32) ((float*)a.Y)[o] = v;
          else {
            v += res[jj];
            ((bf16*)a.Y)[o] = __float2bfloat16(v);
          }
        }
      }
      }
    }
  }
  if (*abortp && warp == 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <int TN>
static int fp8_launch(const Fp8Args& a, int grid, cudaStream_t stream) {
  using C = Fp8Cfg<TN>;
  auto kern = fp8_linear_kernel<TN>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(fp8_linear)");
    attr_set[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = a.budget + 1024; cfg.stream = stream;
  cudaLaunchAttribute at[2];
  int n_at = 0;
  if (a.splits > 1) {
    at[n_at].id = cudaLaunchAttributeClusterDimension;
    at[n_at].val.clusterDim.x = a.splits; at[n_at].val.clusterDim.y = 1; at[n_at].val.clusterDim.z = 1;
    ++n_at;
  }
  if (ca_pdl_enabled(CA_PDL_CLASS)) {
    at[n_at].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n_at].val.programmaticStreamSerializationAllowed = 1;
    ++n_at;
  }
  cfg.attrs = at; cfg.numAttrs = n_at;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) return ca_cuda(e, "fp8_linear launch");
  return CA_OK;
}

static int fp8_budget(int tn, int splits, int K) {
  if (tn <= 32) {
    const int nk = ((K + 127) / 128 + splits - 1) / splits;
    const int r = tn == 16 ? Fp8Cfg<16>::ring(splits, nk, 100 * 1024) : Fp8Cfg<32>::ring(splits, nk, 100 * 1024);
    if (r >= 3) return 100 * 1024;
  }
  return 200 * 1024;
}

// Clusters of `splits` CTAs of the FP8 kernel that the device holds at once for this shape (a cluster needs its CTAs inside one GPC):
// a split whose tile count exceeds this runs in two waves.
template <int TN>
static int fp8_capacity(int splits, int budget, int* out) {
  auto kern = fp8_linear_kernel<TN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Fp8Cfg<TN>::SMEM_BYTES);
  if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(fp8_linear)");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits * 64); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = budget + 1024;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = splits; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  e = cudaOccupancyMaxActiveClusters(out, kern, &cfg);
  if (e != cudaSuccess) return ca_cuda(e, "cudaOccupancyMaxActiveClusters");
  return CA_OK;
}

extern "C" int cuteafd_fp8_cluster_capacity(int tn, int splits, int K, int* out) {
  CA_REQUIRE(out && splits >= 1 && splits <= 8 && (tn == 16 || tn == 32 || tn == 64), "fp8_cluster_capacity: bad arguments");
  const int budget = fp8_budget(tn, splits, K);
  if (tn == 16) return fp8_capacity<16>(splits, budget, out);
  if (tn == 32) return fp8_capacity<32>(splits, budget, out);
  return fp8_capacity<64>(splits, budget, out);
}

extern "C" int cuteafd_fp8_linear(int tn, const void* tmA, const void* tmB, const float* sw, const float* sa, void* Y, const void* R,
                                  int ldy, int rows_total, int N, int K, int epi, int splits, int* status, cudaStream_t stream) {
  CA_REQUIRE(tmA && tmB && sw && sa && Y, "fp8_linear: null operand");
  CA_REQUIRE(K % 16 == 0, "fp8_linear: K must be a multiple of 16 (K=%d)", K);
  CA_REQUIRE(epi == F8_EPI_BF16 || epi == F8_EPI_BF16_RESIDUAL || epi == F8_EPI_F32, "fp8_linear: bad epilogue %d", epi);
  CA_REQUIRE(epi != F8_EPI_BF16_RESIDUAL || R, "fp8_linear: residual epilogue needs R");
  if (splits < 1) splits = 1;
  CA_REQUIRE(splits == 1 || (splits >= 2 && splits <= (tn == 16 ? 8 : 4) && tn <= 64),
             "fp8_linear: split-K is up to 4-way for token tiles of up to 64 rows (up to 8-way for 16 rows)");
  if (rows_total <= 0 || N <= 0) return CA_OK;
  Fp8Args a;
  a.tmA = (const CUtensorMap*)tmA; a.tmB = (const CUtensorMap*)tmB; a.sw = sw; a.sa = sa; a.Y = Y; a.R = (const bf16*)R; a.status = status;
  a.ldy = ldy; a.rows_total = rows_total; a.N = N; a.K = K; a.epi = epi; a.splits = splits;
  // Decode-sized tiles: two CTAs per SM (half the shared memory each) when the split's staging area leaves a ring of >= 3 stages -
  // the kernel is bound by its chain of tcgen05.mma issues per stage, and two CTAs run two such chains per SM.
  a.budget = fp8_budget(tn, splits, K);
  const int grid = ((rows_total + tn - 1) / tn) * ((N + 127) / 128) * splits;
  switch (tn) {
    case 16: return fp8_launch<16>(a, grid, stream);
    case 32: return fp8_launch<32>(a, grid, stream);
    case 64: return fp8_launch<64>(a, grid, stream);
    case 128: return fp8_launch<128>(a, grid, stream);
    default: return ca_fail(CA_ERR_ARG, "fp8_linear: unsupported token tile %d", tn);
  }
}

// ---------------------------------------------------------------- activation quantisation: E4M3 + fp32 scale / 128
// One warp per (row, 128-channel group): scale = max(amax, 1e-4) / 448, q = e4m3(x / scale).
__global__ void act_quant_fp8_block128_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ sa, int rows, int K,
                                              int ldx, int nkb) {
  pdl_launch(); pdl_wait();
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)rows * nkb) return;
  const int r = (int)(w / nkb), g = (int)(w % nkb);
  const int k0 = g * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (k0 < K) {
    const uint2 raw = *(const uint2*)(x + (size_t)r * ldx + k0);
    const bf16* e = (const bf16*)&raw;
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(e[j]);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-4f) / 448.f;
  if (k0 < K) {
    uint32_t pk = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) pk |= (uint32_t)float_to_e4m3(v[j] / scale) << (8 * j);
    *(uint32_t*)(q + (size_t)r * K + k0) = pk;
  }
  if (lane == 0) sa[(size_t)r * nkb + g] = scale;
}

extern "C" int cuteafd_act_quant_fp8_block128(const void* x, void* q, float* sa, int rows, int K, int ldx, cudaStream_t s) {
  CA_REQUIRE(K % 4 == 0 && ldx % 4 == 0, "act_quant_fp8_block128: K must be a multiple of 4");
  if (rows <= 0) return CA_OK;
  const int nkb = (K + 127) / 128;
  const long long warps = (long long)rows * nkb;
  CA_LAUNCH_PDL(act_quant_fp8_block128_kernel, (int)((warps * 32 + 255) / 256), 256, 0, s, (const bf16*)x, (uint8_t*)q, sa, rows, K, ldx, nkb);
  return CA_OK;
}
