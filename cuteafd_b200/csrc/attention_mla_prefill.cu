// MLA prefill attention on the 5th-generation tensor cores: the NON-absorbed form for long query chunks.
//
// Decode multiplies the query into the 512-wide latent space and attends over the latent cache (attention_mla.cu): per key
// that is 576 + 512 multiply-adds per head, fine while the step is bound by reading the cache.  A prefill chunk is bound by
// arithmetic, and the per-head form needs 192 + 128 multiply-adds per key: the latent rows of the sequence's context are
// first expanded once per chunk into per-head keys and values (one GEMM with the kv_b projection, `kvb` below), then
//   S[128 x 128] = [q_nope | q_rope] [k_nope | k_rope]^T      three 64-wide chunks, tcgen05.mma kind::f16, N = 128 keys
//   O[128 x 128] += softmax(S) V
// (a tcgen05.mma of M = 128 costs ~130 cycles whatever its N up to 256, so key tiles are 128 wide: 12 score + 8 PV
// instructions per 128 keys instead of 24 + 8 with 64-key tiles)
// with a CTA owning 128 query tokens of ONE head.  k_rope is shared by all heads and comes straight from the gathered latent
// rows (columns 512..575); k_nope and V come from the expanded buffer [rows, Hl * 256] (per head: 128 key columns, then 128
// value columns).  Both buffers are contiguous per sequence (`ctx_start[seq]` + key index), so tiles need no page table.
//
// Structure (one CTA per SM, 192 threads): warp 0 streams K tiles (48 KB, two stages) and V tiles (32 KB, two stages) by TMA;
// the 128 x 192 query tile sits in tensor memory (96 columns) as the A operand of the score MMAs, which leaves the shared
// memory to the K / V rings; warp 1 issues the MMAs (scores double-buffered in tensor memory), warps 2-5
// run the softmax, one thread per row in two passes over the tile's 128 score columns (maximum, then exponentials, which
// are computed BEFORE the wait for the PV product of tile i - 1, so that product runs under them).
// Every wait is bounded and reports through the status word.
//
// Reference: the dedicated MLA prefill kernels of the GLM5 family (native/families/glm5/cuda/glm_mla_prefill.cu:123, 539),
// which also expand the latent cache per chunk and run per-head attention with mma.sync.
#include <string.h>

#define CA_PDL_CLASS 2
#include "common.cuh"

#define PF_KT 128                 // keys per tile
#define PF_NS 2                   // K stages
#define PF_NSV 2                  // V stages
#define PF_Q_BYTES 0              // the query tile lives in tensor memory (A operand of the score MMAs)
#define PF_P_BYTES 32768          // 2 chunks (64 keys each) x [128 rows x 128 B]
#define PF_K_STAGE 49152          // 3 chunks x [128 keys x 128 B]
#define PF_V_STAGE 32768          // 2 chunks (64 dims each) x [128 keys x 128 B]
#define PF_SMEM (PF_Q_BYTES + PF_P_BYTES + PF_NS * PF_K_STAGE + PF_NSV * PF_V_STAGE + 256)

struct MlaPrefillArgs {
  const bf16* q_nope;           // [Hl, T, 128] head-major
  const bf16* q_rope;           // [T, Hl, 64]
  CUtensorMap kvb_map;          // {Hl * 256, rows, 1}, box {64, 128, 1}, 128-byte swizzle (encoded with rank 3: loads pass z = 0)
  CUtensorMap lat_map;          // {576, rows, 1}, box {64, 128, 1}, 128-byte swizzle
  const int* ctx_start;         // [n_seq] first row of the sequence's context in the two buffers
  const int* kv_len;
  const int* q_start;
  const int* q_len;
  bf16* out;                    // [T, Hl * 128] token-major
  int* status;
  int T, Hl, max_q_tiles;
  float scale;
};

__device__ __forceinline__ uint64_t pf_desc_mn_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint32_t pf_idesc(int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void pf_tmem_st_x16(uint32_t addr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                 "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

__global__ void __launch_bounds__(192, 1) mla_prefill_kernel(const __grid_constant__ MlaPrefillArgs a) {
  pdl_launch(); pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sP = smem;
  uint8_t* sK = sP + PF_P_BYTES;
  uint8_t* sV = sK + PF_NS * PF_K_STAGE;
  uint64_t* bars = (uint64_t*)(sV + PF_NSV * PF_V_STAGE);
  uint64_t* k_full = bars; uint64_t* k_empty = bars + 2; uint64_t* v_full = bars + 4; uint64_t* v_empty = bars + 6;     // [<= 2] each
  uint64_t* s_full = bars + 8;          // [2]
  uint64_t* s_free = bars + 10;         // [2]: the softmax threads are done with the score buffer
  uint64_t& p_full = bars[12]; uint64_t& o_done = bars[13];
  uint32_t& tmem_slot = *(uint32_t*)(bars + 14);
  int& abort_flag = *(int*)(bars + 15);
  if (smem_u32(smem) & 1023) { if (threadIdx.x == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, 0xA13); return; }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

  // the heaviest query tiles (most visible keys) are scheduled first
  const int head = blockIdx.x;
  const int seq = blockIdx.y / a.max_q_tiles, qt = a.max_q_tiles - 1 - blockIdx.y % a.max_q_tiles;
  const int qlen = a.q_len[seq], kvlen = a.kv_len[seq];
  const int tok0 = qt * 128;
  if (tok0 >= qlen) return;
  const int R = min(128, qlen - tok0);
  const int row_base = a.q_start[seq] + tok0;
  const int first_pos = kvlen - qlen + tok0;
  const int hi = first_pos + R;
  const int n_tiles = (hi + PF_KT - 1) / PF_KT;
  const int ctx0 = a.ctx_start[seq];

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_free[s], 128); }
    mbar_init(&p_full, 128); mbar_init(&o_done, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;
  const uint32_t S0_COL = 0, O_COL = 128, S1_COL = 256, Q_COL = 384;
  // query rows -> tensor memory (row = lane, two bf16 per 32-bit column, 32 columns per 64-wide chunk: q_nope low / high, q_rope)
  if (warp >= 2) {
    const int r = (warp & 3) * 32 + lane;
    const uint32_t dst = tmem + ((uint32_t)((warp & 3) * 32) << 16) + Q_COL;
    const int t = row_base + (r < R ? r : 0);
    const bf16* src_nope = a.q_nope + ((size_t)head * a.T + t) * 128;
    const bf16* src_rope = a.q_rope + ((size_t)t * a.Hl + head) * 64;
#pragma unroll 1
    for (int g = 0; g < 6; ++g) {                  // 16 columns = 32 elements per store
      const bf16* src = g < 4 ? src_nope + g * 32 : src_rope + (g - 4) * 32;
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 v = r < R ? *(const uint4*)(src + j * 8) : make_uint4(0, 0, 0, 0);
        w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
      }
      pf_tmem_st_x16(dst + g * 16, w);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp == 0) {
    // ------------------------------------------------------------------ K / V producer
    // K runs one tile ahead of V in this warp's program order: the single V stage only frees when the previous PV product
    // retires, and the K tile of the NEXT score pass must not queue behind that wait.
    auto load_k = [&](int i) -> bool {
      const int s = i % PF_NS, ph = ((i / PF_NS) & 1) ^ 1;
      if (!mbar_wait_bounded(&k_empty[s], ph, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, i); return false; }
      if (lane == 0) {
        const int row = ctx0 + i * PF_KT;
        mbar_expect_tx(&k_full[s], PF_K_STAGE);
        tma_load_3d(sK + s * PF_K_STAGE, &a.kvb_map, &k_full[s], head * 256, row, 0);
        tma_load_3d(sK + s * PF_K_STAGE + 16384, &a.kvb_map, &k_full[s], head * 256 + 64, row, 0);
        tma_load_3d(sK + s * PF_K_STAGE + 32768, &a.lat_map, &k_full[s], 512, row, 0);
      }
      __syncwarp();
      return true;
    };
    bool okp = n_tiles > 0 ? load_k(0) : true;
    for (int i = 0; okp && i < n_tiles && !*abortp; ++i) {
      if (i + 1 < n_tiles && !load_k(i + 1)) break;
      const int sv = i % PF_NSV, phv = ((i / PF_NSV) & 1) ^ 1;
      if (!mbar_wait_bounded(&v_empty[sv], phv, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, 0x1000 + i); break; }
      if (lane == 0) {
        const int row = ctx0 + i * PF_KT;
        mbar_expect_tx(&v_full[sv], PF_V_STAGE);
        tma_load_3d(sV + sv * PF_V_STAGE, &a.kvb_map, &v_full[sv], head * 256 + 128, row, 0);
        tma_load_3d(sV + sv * PF_V_STAGE + 16384, &a.kvb_map, &v_full[sv], head * 256 + 192, row, 0);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t id_s = pf_idesc(PF_KT, 0), id_o = pf_idesc(128, 1);
    auto issue_scores = [&](int j) -> bool {     // S[j & 1] = Q K(j)^T once the softmax threads have copied tile j - 2 out of it
      const int s = j % PF_NS;
      if (j >= 2 && !mbar_wait_bounded(&s_free[j & 1], ((j - 2) >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, 0x2000 + j); return false; }
      if (!mbar_wait_bounded(&k_full[s], (j / PF_NS) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, j); return false; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k0 = smem_u32(sK + s * PF_K_STAGE), d = tmem + ((j & 1) ? S1_COL : S0_COL);
#pragma unroll
        for (int kb = 0; kb < 3; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16_ta(d, tmem + Q_COL + kb * 32 + k * 8, umma_desc_sw128(k0 + kb * 16384) + 2 * k, id_s, (kb | k) ? 1u : 0u);
        tc_commit(&s_full[j & 1]);
        tc_commit(&k_empty[s]);
      }
      __syncwarp();
      return true;
    };
    bool ok = true;
    for (int j = 0; ok && j < min(2, n_tiles); ++j) ok = issue_scores(j);
    for (int i = 0; ok && i < n_tiles; ++i) {
      const int sv = i % PF_NSV;
      if (!mbar_wait_bounded(&p_full, i & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, 0x3000 + i); break; }
      if (!mbar_wait_bounded(&v_full[sv], (i / PF_NSV) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, 0x4000 + i); break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v0 = smem_u32(sV + sv * PF_V_STAGE);
#pragma unroll
        for (int k = 0; k < PF_KT / 16; ++k)       // 16 keys per MMA: P chunk k / 4 (64 keys per 128-byte row), V rows 16 k .. 16 k + 15
          tc_mma_f16(tmem + O_COL, umma_desc_sw128(smem_u32(sP) + (k >> 2) * 16384) + 2 * (k & 3), pf_desc_mn_sw128(v0 + k * 2048, 16384, 1024), id_o,
                     (i | k) ? 1u : 0u);
        tc_commit(&v_empty[sv]);
        tc_commit(&o_done);
      }
      __syncwarp();
      if (i + 2 < n_tiles) ok = issue_scores(i + 2);
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: thread = query row
    const int q4 = warp & 3, r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const bool live = r < R;
    const int qpos = live ? first_pos + r : -1;
    const float sc2 = a.scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      if (!mbar_wait_bounded(&s_full[i & 1], (i >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_addr + ((i & 1) ? S1_COL : S0_COL);
      const int key0 = i * PF_KT;
      const bool all_visible = key0 + PF_KT - 1 <= first_pos;      // CTA-uniform: every key of the tile is visible to every live row
      // two passes over the tile's 128 score columns: row maximum, then exponentials packed to bf16 pairs (64 registers).
      // Tiles below the diagonal need no mask (CTA-uniform test), which is all but the last one or two of a long context.
      float mx = -INFINITY;
      uint32_t pk[PF_KT / 2];
      float psum = 0.f;
      float alpha = 1.f;
      if (all_visible) {           // CTA-uniform (the tensor-memory loads below are warp collectives); rows past R hold zero queries
#pragma unroll 1
        for (int c = 0; c < PF_KT / 32; ++c) {
          uint32_t sr[32];
          tmem_ld_x16(s_addr + c * 32, sr);
          tmem_ld_x16(s_addr + c * 32 + 16, sr + 16);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(sr[j]));
        }
        mx *= sc2;                                   // sc2 > 0: scaling commutes with the maximum
        if (mx > m_ref + 8.f) {
          if (m_ref != -INFINITY) { alpha = exp2f(m_ref - mx); l *= alpha; }
          m_ref = mx;
        }
#pragma unroll
        for (int c = 0; c < PF_KT / 32; ++c) {
          uint32_t sr[32];
          tmem_ld_x16(s_addr + c * 32, sr);
          tmem_ld_x16(s_addr + c * 32 + 16, sr + 16);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float e0 = exp2f(fmaf(__uint_as_float(sr[2 * j]), sc2, -m_ref)), e1 = exp2f(fmaf(__uint_as_float(sr[2 * j + 1]), sc2, -m_ref));
            psum += e0 + e1;
            bf162 h = __floats2bfloat162_rn(e0, e1);
            pk[c * 16 + j] = *(uint32_t*)&h;
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < PF_KT / 32; ++c) {
          uint32_t sr[32];
          tmem_ld_x16(s_addr + c * 32, sr);
          tmem_ld_x16(s_addr + c * 32 + 16, sr + 16);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int kp = key0 + c * 32 + j;
            if (live && kp <= qpos) mx = fmaxf(mx, __uint_as_float(sr[j]) * sc2);
          }
        }
        if (mx > m_ref + 8.f) {
          if (m_ref != -INFINITY) { alpha = exp2f(m_ref - mx); l *= alpha; }
          m_ref = mx;
        }
#pragma unroll
        for (int c = 0; c < PF_KT / 32; ++c) {
          uint32_t sr[32];
          tmem_ld_x16(s_addr + c * 32, sr);
          tmem_ld_x16(s_addr + c * 32 + 16, sr + 16);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int kp = key0 + c * 32 + 2 * j;
            const float e0 = (live && kp <= qpos) ? exp2f(fmaf(__uint_as_float(sr[2 * j]), sc2, -m_ref)) : 0.f;
            const float e1 = (live && kp + 1 <= qpos) ? exp2f(fmaf(__uint_as_float(sr[2 * j + 1]), sc2, -m_ref)) : 0.f;
            psum += e0 + e1;
            bf162 h = __floats2bfloat162_rn(e0, e1);
            pk[c * 16 + j] = *(uint32_t*)&h;
          }
        }
      }
      l += psum;
      tc_fence_before();
      mbar_arrive(&s_free[i & 1]);
      // the previous P V product must have finished before P is overwritten or O rescaled
      if (i > 0 && !mbar_wait_bounded(&o_done, (i - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 0x1000 + i); ok = false; break; }
      tc_fence_after();
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {      // warp-uniform: tcgen05.ld/st are warp collectives
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[16];
          tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          pf_tmem_st_x16(tmem + lane_addr + O_COL + c * 16, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      // P: two K-major chunks of 64 keys; 16-byte unit u of a row holds keys 8 u .. 8 u + 7
#pragma unroll
      for (int u = 0; u < PF_KT / 8; ++u)
        *(uint4*)(sP + (u >> 3) * 16384 + r * 128 + (((u & 7) ^ (r & 7)) << 4)) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    if (ok && n_tiles > 0 && !mbar_wait_bounded(&o_done, (n_tiles - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 999); ok = false; }
    tc_fence_after();
    if (__all_sync(0xffffffffu, ok)) {
      const int t = row_base + (live ? r : 0);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = a.out + ((size_t)t * a.Hl + head) * 128;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t o[16];
        if (n_tiles > 0) { tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o); tc_wait_ld(); }
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = 0;
        }
        if (!live) continue;
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { bf162 hh = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * inv, __uint_as_float(o[2 * j + 1]) * inv); w[j] = *(uint32_t*)&hh; }
        *(uint4*)(dst + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        *(uint4*)(dst + c * 16 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
  }
  if (*abortp && warp == 0) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 200000) __nanosleep(1000); }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------------------
// The same structure for paged GQA prefill (head_dim 128): a CTA owns 128 query rows of one KV head (row = token_in_tile * G +
// head_in_group) and walks the sequence's pages two at a time (128-key tiles), K and V straight from the paged store.  Causal
// mask, optional sliding window and sink logit as in the decode kernel (attention_tc.cu), no split-KV: a prefill chunk has
// enough query tiles to fill the GPU.  window < 0 drops the causal mask (bidirectional attention of a vision / audio encoder:
// every query row sees keys [0, kvlen)).  The 64-key decode kernel spends 8 + 4 tcgen05.mma per 64 keys; this one 8 + 8 per 128 keys.
#define GQ_K_STAGE 32768          // 2 chunks (64 dims each) x [128 keys x 128 B]
struct GqaPrefillArgs {
  const bf16* q;
  const CUtensorMap* kv_map;    // 3-D {128, 2 * Hkv, slots}, box {64, 1, 64}, 128-byte swizzle (the decode kernel's descriptor)
  const int* page_table; const int* kv_len; const int* q_start; const int* q_len;
  const float* sink;
  bf16* out;
  int* status;
  int q_stride, Hq, Hkv, max_pages, window, max_q_tiles;
  float scale;
};

__global__ void __launch_bounds__(192, 1) gqa_prefill_kernel(const __grid_constant__ GqaPrefillArgs a) {
  pdl_launch(); pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sP = smem;
  uint8_t* sK = sP + PF_P_BYTES;
  uint8_t* sV = sK + PF_NS * GQ_K_STAGE;
  uint64_t* bars = (uint64_t*)(sV + PF_NSV * PF_V_STAGE);
  uint64_t* k_full = bars; uint64_t* k_empty = bars + 2; uint64_t* v_full = bars + 4; uint64_t* v_empty = bars + 6;     // [<= 2] each
  uint64_t* s_full = bars + 8;          // [2]
  uint64_t* s_free = bars + 10;         // [2]: the softmax threads are done with the score buffer
  uint64_t& p_full = bars[12]; uint64_t& o_done = bars[13];
  uint32_t& tmem_slot = *(uint32_t*)(bars + 14);
  int& abort_flag = *(int*)(bars + 15);
  if (smem_u32(smem) & 1023) { if (threadIdx.x == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, 0xA14); return; }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

  // the heaviest query tiles (most visible keys) are scheduled first
  const int G = a.Hq / a.Hkv, tok_per_tile = 128 / G;
  const int kvh = blockIdx.x;
  const int seq = blockIdx.y / a.max_q_tiles, qt = a.max_q_tiles - 1 - blockIdx.y % a.max_q_tiles;
  const int qlen = a.q_len[seq], kvlen = a.kv_len[seq];
  const int tok0 = qt * tok_per_tile;
  if (tok0 >= qlen) return;
  const int ntok = min(tok_per_tile, qlen - tok0);
  const int R = ntok * G;                                   // row = token_in_tile * G + head_in_group
  const int row_base = a.q_start[seq] + tok0;
  const bool bidir = a.window < 0;                          // encoder towers: every row sees all kvlen keys
  const int first_pos = bidir ? kvlen - 1 : kvlen - qlen + tok0;
  const int hi = bidir ? kvlen : first_pos + ntok;
  const int lo = a.window > 0 ? max(0, first_pos - a.window + 1) : 0;
  const int tile0 = lo / PF_KT;
  const int n_tiles = max(0, (hi + PF_KT - 1) / PF_KT - tile0);

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_free[s], 128); }
    mbar_init(&p_full, 128); mbar_init(&o_done, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;
  const uint32_t S0_COL = 0, O_COL = 128, S1_COL = 256, Q_COL = 384;
  // query rows -> tensor memory (row = lane, two bf16 per 32-bit column, 64 columns for the 128-wide head)
  if (warp >= 2) {
    const int r = (warp & 3) * 32 + lane;
    const uint32_t dst = tmem + ((uint32_t)((warp & 3) * 32) << 16) + Q_COL;
    const int rr = r < R ? r : 0;
    const bf16* src = a.q + (size_t)(row_base + rr / G) * a.q_stride + (size_t)(kvh * G + rr % G) * 128;
#pragma unroll 1
    for (int g = 0; g < 4; ++g) {                  // 16 columns = 32 elements per store
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 v = r < R ? *(const uint4*)(src + g * 32 + j * 8) : make_uint4(0, 0, 0, 0);
        w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
      }
      pf_tmem_st_x16(dst + g * 16, w);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp == 0) {
    // ------------------------------------------------------------------ K / V producer
    // K runs one tile ahead of V in this warp's program order: the single V stage only frees when the previous PV product
    // retires, and the K tile of the NEXT score pass must not queue behind that wait.
    auto page_of = [&](int key) -> int {                   // pages past the sequence's table are read as page 0 (finite rows, masked keys)
      const int pi = key / 64;
      return pi < a.max_pages ? a.page_table[(size_t)seq * a.max_pages + pi] : 0;
    };
    auto load_k = [&](int i) -> bool {
      const int s = i % PF_NS, ph = ((i / PF_NS) & 1) ^ 1;
      if (!mbar_wait_bounded(&k_empty[s], ph, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, i); return false; }
      if (lane == 0) {
        const int key0 = (tile0 + i) * PF_KT;
        mbar_expect_tx(&k_full[s], GQ_K_STAGE);
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          const int slot0 = page_of(key0 + p * 64) * 64;
          tma_load_3d(sK + s * GQ_K_STAGE + p * 8192, a.kv_map, &k_full[s], 0, kvh, slot0);
          tma_load_3d(sK + s * GQ_K_STAGE + 16384 + p * 8192, a.kv_map, &k_full[s], 64, kvh, slot0);
        }
      }
      __syncwarp();
      return true;
    };
    bool okp = n_tiles > 0 ? load_k(0) : true;
    for (int i = 0; okp && i < n_tiles && !*abortp; ++i) {
      if (i + 1 < n_tiles && !load_k(i + 1)) break;
      const int sv = i % PF_NSV, phv = ((i / PF_NSV) & 1) ^ 1;
      if (!mbar_wait_bounded(&v_empty[sv], phv, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, 0x1000 + i); break; }
      if (lane == 0) {
        const int key0 = (tile0 + i) * PF_KT;
        mbar_expect_tx(&v_full[sv], PF_V_STAGE);
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          const int slot0 = page_of(key0 + p * 64) * 64;
          tma_load_3d(sV + sv * PF_V_STAGE + p * 8192, a.kv_map, &v_full[sv], 0, a.Hkv + kvh, slot0);
          tma_load_3d(sV + sv * PF_V_STAGE + 16384 + p * 8192, a.kv_map, &v_full[sv], 64, a.Hkv + kvh, slot0);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t id_s = pf_idesc(PF_KT, 0), id_o = pf_idesc(128, 1);
    auto issue_scores = [&](int j) -> bool {     // S[j & 1] = Q K(j)^T once the softmax threads have copied tile j - 2 out of it
      const int s = j % PF_NS;
      if (j >= 2 && !mbar_wait_bounded(&s_free[j & 1], ((j - 2) >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, 0x2000 + j); return false; }
      if (!mbar_wait_bounded(&k_full[s], (j / PF_NS) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, j); return false; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k0 = smem_u32(sK + s * GQ_K_STAGE), d = tmem + ((j & 1) ? S1_COL : S0_COL);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16_ta(d, tmem + Q_COL + kb * 32 + k * 8, umma_desc_sw128(k0 + kb * 16384) + 2 * k, id_s, (kb | k) ? 1u : 0u);
        tc_commit(&s_full[j & 1]);
        tc_commit(&k_empty[s]);
      }
      __syncwarp();
      return true;
    };
    bool ok = true;
    for (int j = 0; ok && j < min(2, n_tiles); ++j) ok = issue_scores(j);
    for (int i = 0; ok && i < n_tiles; ++i) {
      const int sv = i % PF_NSV;
      if (!mbar_wait_bounded(&p_full, i & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, 0x3000 + i); break; }
      if (!mbar_wait_bounded(&v_full[sv], (i / PF_NSV) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, 0x4000 + i); break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v0 = smem_u32(sV + sv * PF_V_STAGE);
#pragma unroll
        for (int k = 0; k < PF_KT / 16; ++k)       // 16 keys per MMA: P chunk k / 4 (64 keys per 128-byte row), V rows 16 k .. 16 k + 15
          tc_mma_f16(tmem + O_COL, umma_desc_sw128(smem_u32(sP) + (k >> 2) * 16384) + 2 * (k & 3), pf_desc_mn_sw128(v0 + k * 2048, 16384, 1024), id_o,
                     (i | k) ? 1u : 0u);
        tc_commit(&v_empty[sv]);
        tc_commit(&o_done);
      }
      __syncwarp();
      if (i + 2 < n_tiles) ok = issue_scores(i + 2);
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: thread = query row
    const int q4 = warp & 3, r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const bool live = r < R;
    const int qpos = live ? (bidir ? first_pos : first_pos + r / G) : -1;
    const int wlo = a.window > 0 ? qpos - a.window : -1;           // keys at or below this position are outside the row's window
    const float sc2 = a.scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      if (!mbar_wait_bounded(&s_full[i & 1], (i >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_addr + ((i & 1) ? S1_COL : S0_COL);
      const int key0 = (tile0 + i) * PF_KT;
      // CTA-uniform: every key of the tile is visible to every live row (below the diagonal and inside every row's window)
      const bool all_visible = key0 + PF_KT - 1 <= first_pos && (a.window <= 0 || key0 > first_pos + ntok - 1 - a.window);
      // two passes over the tile's 128 score columns: row maximum, then exponentials packed to bf16 pairs (64 registers).
      // Tiles below the diagonal need no mask (CTA-uniform test), which is all but the last one or two of a long context.
      float mx = -INFINITY;
      uint32_t pk[PF_KT / 2];
      float psum = 0.f;
      float alpha = 1.f;
      if (all_visible) {           // CTA-uniform (the tensor-memory loads below are warp collectives); rows past R hold zero queries
#pragma unroll 1
        for (int c = 0; c < PF_KT / 32; ++c) {
          uint32_t sr[32];
          tmem_ld_x16(s_addr + c * 32, sr);
          tmem_ld_x16(s_addr + c * 32 + 16, sr + 16);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(sr[j]));
        }
        mx *= sc2;                                   // sc2 > 0: scaling commutes with the maximum
        if (mx > m_ref + 8.f) {
          if (m_ref != -INFINITY) { alpha = exp2f(m_ref - mx); l *= alpha; }
          m_ref = mx;
        }
#pragma unroll
        for (int c = 0; c < PF_KT / 32; ++c) {
          uint32_t sr[32];
          tmem_ld_x16(s_addr + c * 32, sr);
          tmem_ld_x16(s_addr + c * 32 + 16, sr + 16);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float e0 = exp2f(fmaf(__uint_as_float(sr[2 * j]), sc2, -m_ref)), e1 = exp2f(fmaf(__uint_as_float(sr[2 * j + 1]), sc2, -m_ref));
            psum += e0 + e1;
            bf162 h = __floats2bfloat162_rn(e0, e1);
            pk[c * 16 + j] = *(uint32_t*)&h;
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < PF_KT / 32; ++c) {
          uint32_t sr[32];
          tmem_ld_x16(s_addr + c * 32, sr);
          tmem_ld_x16(s_addr + c * 32 + 16, sr + 16);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int kp = key0 + c * 32 + j;
            if (live && kp <= qpos && kp > wlo) mx = fmaxf(mx, __uint_as_float(sr[j]) * sc2);
          }
        }
        if (mx > m_ref + 8.f) {
          if (m_ref != -INFINITY) { alpha = exp2f(m_ref - mx); l *= alpha; }
          m_ref = mx;
        }
#pragma unroll
        for (int c = 0; c < PF_KT / 32; ++c) {
          uint32_t sr[32];
          tmem_ld_x16(s_addr + c * 32, sr);
          tmem_ld_x16(s_addr + c * 32 + 16, sr + 16);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int kp = key0 + c * 32 + 2 * j;
            const float e0 = (live && kp <= qpos && kp > wlo) ? exp2f(fmaf(__uint_as_float(sr[2 * j]), sc2, -m_ref)) : 0.f;
            const float e1 = (live && kp + 1 <= qpos && kp + 1 > wlo) ? exp2f(fmaf(__uint_as_float(sr[2 * j + 1]), sc2, -m_ref)) : 0.f;
            psum += e0 + e1;
            bf162 h = __floats2bfloat162_rn(e0, e1);
            pk[c * 16 + j] = *(uint32_t*)&h;
          }
        }
      }
      l += psum;
      tc_fence_before();
      mbar_arrive(&s_free[i & 1]);
      // the previous P V product must have finished before P is overwritten or O rescaled
      if (i > 0 && !mbar_wait_bounded(&o_done, (i - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 0x1000 + i); ok = false; break; }
      tc_fence_after();
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {      // warp-uniform: tcgen05.ld/st are warp collectives
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[16];
          tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          pf_tmem_st_x16(tmem + lane_addr + O_COL + c * 16, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      // P: two K-major chunks of 64 keys; 16-byte unit u of a row holds keys 8 u .. 8 u + 7
#pragma unroll
      for (int u = 0; u < PF_KT / 8; ++u)
        *(uint4*)(sP + (u >> 3) * 16384 + r * 128 + (((u & 7) ^ (r & 7)) << 4)) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    if (ok && n_tiles > 0 && !mbar_wait_bounded(&o_done, (n_tiles - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 999); ok = false; }
    tc_fence_after();
    if (__all_sync(0xffffffffu, ok)) {
      const int rr = live ? r : 0;
      const int t = row_base + rr / G, h = kvh * G + rr % G;
      float scale_o = 1.f, lt = l;
      if (a.sink) {                                     // learned sink logit: one more softmax term with a zero value
        const float m_nat = (m_ref == -INFINITY) ? -INFINITY : m_ref * 0.6931471805599453f;
        const float sk = a.sink[h], m2 = fmaxf(m_nat, sk);
        const float e1 = (m_nat == -INFINITY) ? 0.f : __expf(m_nat - m2);
        lt = l * e1 + __expf(sk - m2); scale_o = e1;
      }
      const float inv = lt > 0.f ? scale_o / lt : 0.f;
      bf16* dst = a.out + ((size_t)t * a.Hq + h) * 128;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t o[16];
        if (n_tiles > 0) { tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o); tc_wait_ld(); }
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = 0;
        }
        if (!live) continue;
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { bf162 hh = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * inv, __uint_as_float(o[2 * j + 1]) * inv); w[j] = *(uint32_t*)&hh; }
        *(uint4*)(dst + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        *(uint4*)(dst + c * 16 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
  }
  if (*abortp && warp == 0) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 200000) __nanosleep(1000); }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}


extern "C" int cuteafd_gqa_prefill_attention(const void* q, const void* kv_map, const int* page_table, const int* kv_len, const int* q_start,
                                             const int* q_len, const float* sink, void* out, int T, int n_seq, int max_q_len, int q_stride, int Hq,
                                             int Hkv, int max_pages, int window, float scale, int* status, cudaStream_t s) {
  CA_REQUIRE(q && kv_map && page_table && kv_len && q_start && q_len && out, "gqa_prefill_attention: null argument");
  CA_REQUIRE(Hq % Hkv == 0 && 128 % (Hq / Hkv) == 0 && q_stride % 8 == 0, "gqa_prefill_attention: group size %d unsupported", Hq / Hkv);
  if (T <= 0 || n_seq <= 0) return CA_OK;
  GqaPrefillArgs a;
  a.q = (const bf16*)q; a.kv_map = (const CUtensorMap*)kv_map; a.page_table = page_table; a.kv_len = kv_len; a.q_start = q_start; a.q_len = q_len;
  a.sink = sink; a.out = (bf16*)out; a.status = status; a.q_stride = q_stride; a.Hq = Hq; a.Hkv = Hkv; a.max_pages = max_pages; a.window = window;
  a.scale = scale;
  const int tpt = 128 / (Hq / Hkv);
  a.max_q_tiles = (max_q_len + tpt - 1) / tpt;
  const int smem = PF_P_BYTES + PF_NS * GQ_K_STAGE + PF_NSV * PF_V_STAGE + 256;
  static bool attr_set[64] = {false};
  int dev = 0; cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gqa_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(gqa_prefill)");
    attr_set[dev & 63] = true;
  }
  CA_LAUNCH_PDL(gqa_prefill_kernel, dim3(Hkv, n_seq * a.max_q_tiles), 192, smem, s, a);
  CA_CHECK_LAUNCH("gqa_prefill_attention");
  return CA_OK;
}

// Gathers the latent rows of every sequence's context out of the paged cache into one contiguous buffer:
// dst[ctx_start[s] + j] = cache[page_table[s][j / 64] * 64 + j % 64] for j < kv_len[s]; rows of 576 bf16 = 72 x 16 bytes.
__global__ void mla_gather_ctx_kernel(const uint4* __restrict__ cache, const int* __restrict__ page_table, const int* __restrict__ ctx_start,
                                      const int* __restrict__ kv_len, uint4* __restrict__ dst, int max_pages, long long n_slots, long long dst_rows, int* status) {
  pdl_launch(); pdl_wait();
  const int seq = blockIdx.y;
  const int j = blockIdx.x * 4 + threadIdx.x / 72, c = threadIdx.x % 72;
  if (j >= kv_len[seq]) return;
  const long long slot = (long long)page_table[(size_t)seq * max_pages + j / 64] * 64 + j % 64;
  const long long row = (long long)ctx_start[seq] + j;
  if (slot < 0 || slot >= n_slots || row < 0 || row >= dst_rows) { if (c == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, 0xB01); return; }
  dst[row * 72 + c] = cache[slot * 72 + c];
}

extern "C" int cuteafd_mla_gather_ctx(const void* cache, const int* page_table, const int* ctx_start, const int* kv_len, void* dst, int n_seq,
                                      int max_kv, int max_pages, long long n_slots, long long dst_rows, int* status, cudaStream_t s) {
  CA_REQUIRE(cache && page_table && ctx_start && kv_len && dst, "mla_gather_ctx: null argument");
  if (n_seq <= 0 || max_kv <= 0) return CA_OK;
  CA_LAUNCH_PDL(mla_gather_ctx_kernel, dim3((max_kv + 3) / 4, n_seq), 288, 0, s, (const uint4*)cache, page_table, ctx_start, kv_len, (uint4*)dst, max_pages,
                n_slots, dst_rows, status);
  CA_CHECK_LAUNCH("mla_gather_ctx");
  return CA_OK;
}

// q_nope [Hl, T, 128] (head-major), q_rope [T, Hl, 64], kvb [rows, Hl * 256], lat [rows, 576], out [T, Hl * 128].
extern "C" int cuteafd_mla_prefill_attention(const void* q_nope, const void* q_rope, const void* kvb, const void* lat, long long rows, const int* ctx_start,
                                             const int* kv_len, const int* q_start, const int* q_len, void* out, int T, int n_seq, int max_q_len, int Hl,
                                             float scale, int* status, cudaStream_t s) {
  CA_REQUIRE(q_nope && q_rope && kvb && lat && out && rows > 0, "mla_prefill_attention: null argument");
  CA_REQUIRE(Hl >= 1, "mla_prefill_attention: no heads");
  if (T <= 0 || n_seq <= 0) return CA_OK;
  MlaPrefillArgs a;
  int rc = ca_encode_tmap_2d(&a.kvb_map, kvb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)Hl * 256, (uint64_t)rows, (uint64_t)Hl * 512, 64, PF_KT,
                             CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = ca_encode_tmap_2d(&a.lat_map, lat, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 576, (uint64_t)rows, 1152, 64, PF_KT, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  a.q_nope = (const bf16*)q_nope; a.q_rope = (const bf16*)q_rope; a.ctx_start = ctx_start; a.kv_len = kv_len; a.q_start = q_start; a.q_len = q_len;
  a.out = (bf16*)out; a.status = status; a.T = T; a.Hl = Hl; a.max_q_tiles = (max_q_len + 127) / 128; a.scale = scale;
  static bool attr_set[64] = {false};
  int dev = 0; cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(mla_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(mla_prefill)");
    attr_set[dev & 63] = true;
  }
  CA_LAUNCH_PDL(mla_prefill_kernel, dim3(Hl, n_seq * a.max_q_tiles), 192, PF_SMEM, s, a);
  CA_CHECK_LAUNCH("mla_prefill_attention");
  return CA_OK;
}
