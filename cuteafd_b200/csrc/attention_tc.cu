// Paged GQA attention on the 5th-generation tensor cores (head_dim 128): decode, speculative verify and
// chunked prefill in one kernel.
//
// A CTA owns up to 128 query rows of one KV head of one sequence (row = token_in_tile * G + head_in_group)
// and a contiguous range of 64-key pages (split-KV).  Per page:
//   S[128 x 64]  = Q K^T          tcgen05.mma kind::f16, Q and K (TMA, 128-byte swizzle) from shared memory,
//                                 accumulator in tensor memory columns [0, 64)
//   softmax      one thread per row: tcgen05.ld of its S row, causal/window mask, running max with lazy
//                rescaling (the reference max only moves when the row max grows by more than 2^8), P in bf16
//                written to shared memory in the swizzled K-major operand layout
//   O[128 x 128] += P V           V consumed in place as an MN-major operand, accumulator in columns [64, 192)
// K/V pages stream through a TMA ring (warp 0), warp 1 issues the MMAs, warps 2-5 do the softmax and the
// epilogue.  Two CTAs fit per SM (112 KB shared memory, 256 tensor-memory columns each) so one CTA's softmax
// overlaps the other's MMAs and loads.  With several splits the unnormalised (O, m, l) partials go to scratch
// and `attn_merge_kernel` (attention.cu) combines them.
//
// Replaces the reference's sparse/GQA attention programs (AOT-exported, sources absent) and its wmma/mma.sync
// kernels (native/shared/cuda/draft_attention.cu:41-340, families/glm5/cuda/glm_mla_prefill.cu:123-960).
#include <string.h>

#define CA_PDL_CLASS 2
#include "common.cuh"
#include "attn_common.cuh"

#define APAGE 64
#define AD 128
#define NS 2   // K/V ring stages

struct AttnTcArgs {
  const bf16* q;
  const CUtensorMap* kv_map;    // 3-D: {D, 2*Hkv, slots}, box {64, 1, 64}, 128-byte swizzle
  const int* page_table;
  const int* kv_len;
  const int* q_start;
  const int* q_len;
  const float* sink;
  bf16* out;
  float* part_o;
  float* part_ml;
  int* status;
  int q_stride, Hq, Hkv, max_pages, n_splits, window, max_q_tiles, T;
  float scale;
};

__device__ __forceinline__ uint64_t desc_kmajor_sw128(uint32_t saddr) { return umma_desc_sw128(saddr); }
// MN-major operand, 128-byte swizzle: 64-element MN blocks `lbo` bytes apart, 8-row K groups `sbo` bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint32_t idesc_bf16(int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void tmem_st_x16(uint32_t addr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                 "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(192, 2) paged_attn_tc_kernel(const __grid_constant__ AttnTcArgs a) {
  pdl_launch(); pdl_wait();
  // All shared memory is dynamic and 1024-byte aligned (operand tiles first, barriers at the tail) so that two
  // CTAs fit on one SM.
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = (uint64_t*)(smem + 49152 + NS * 32768);
  uint64_t* k_full = bars; uint64_t* k_empty = bars + 2; uint64_t* v_full = bars + 4; uint64_t* v_empty = bars + 6;
  uint64_t* s_full = bars + 8;              // two score buffers
  uint64_t& p_full = bars[10]; uint64_t& o_done = bars[11];
  uint32_t& tmem_slot = *(uint32_t*)(bars + 12);
  int& abort_flag = *(int*)(bars + 13);
  uint64_t& x_bar = bars[14];               // column-split softmax: cross-warp exchange barrier
  if (smem_u32(smem) & 1023) { if (threadIdx.x == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, 0xA11); return; }
  uint8_t* sQ = smem;                       // 2 x [128 rows x 128 B]
  uint8_t* sP = smem + 32768;               // [128 rows x 128 B]
  uint8_t* sK = smem + 49152;               // 2 stages x {lo, hi} x 8 KB
  uint8_t* sV = smem + 49152 + 32768;       // 2 stages x {lo, hi} x 8 KB
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

  const int G = a.Hq / a.Hkv;
  const int tok_per_tile = 128 / G;
  const int split = blockIdx.x, kvh = blockIdx.y;
  const int seq = blockIdx.z / a.max_q_tiles, qt = blockIdx.z % a.max_q_tiles;
  const int qlen = a.q_len[seq], kvlen = a.kv_len[seq];
  const int tok0 = qt * tok_per_tile;
  if (tok0 >= qlen) return;
  const int ntok = min(tok_per_tile, qlen - tok0);
  const int R = ntok * G;
  const int row_base = a.q_start[seq] + tok0;
  const int first_pos = kvlen - qlen + tok0;
  const int hi = first_pos + ntok;                      // keys [lo, hi) can be visible
  const int lo = a.window > 0 ? max(0, first_pos - a.window + 1) : 0;
  const int first_page = lo / APAGE, last_page = (hi + APAGE - 1) / APAGE;
  const int per = (last_page - first_page + a.n_splits - 1) / a.n_splits;
  const int p0 = first_page + split * per, p1 = min(last_page, p0 + per);
  const int n_tiles = max(0, p1 - p0);

  // Decode-shaped tiles (<= 32 real rows) replicate the rows into every 32-lane quarter of the MMA tile so that
  // the four softmax warps each take 16 of the 64 score columns of the SAME rows (4x shorter per-tile chain).
  const bool rep4 = R <= 32;
  const int n_live_warps = rep4 ? 4 : (R + 31) / 32;    // softmax warps with work
  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(&p_full, 32 * n_live_warps); mbar_init(&o_done, 1); mbar_init(&x_bar, 128);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, 256); tmem_relinquish(); }
  // Q rows -> swizzled K-major operand tiles (two 64-element halves)
  for (int i = tid; i < 128 * 16; i += 192) {
    const int r = i >> 4, c = i & 15;                  // 16-byte chunk c of row r
    uint4 v = make_uint4(0, 0, 0, 0);
    const int qr = rep4 ? (r & 31) : r;                // decode tiles replicate their <= 32 rows into all four lane quarters
    if (qr < R) v = *(const uint4*)(a.q + (size_t)(row_base + qr / G) * a.q_stride + (size_t)(kvh * G + qr % G) * AD + c * 8);
    *(uint4*)(sQ + (c >> 3) * 16384 + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;
  const uint32_t S0_COL = 0, O_COL = 64, S1_COL = 192;

  if (warp == 0) {
    // ------------------------------------------------------------------ K/V producer (separate K and V rings:
    // a K stage is free as soon as its score MMA retires, long before the matching V stage)
    // a decode step reads every K/V byte once: stream it through L2; with several query tiles per sequence the pages are shared
    const uint64_t kvpol = a.max_q_tiles == 1 ? l2_policy_stream() : l2_policy_normal();
    for (int i = 0; i < n_tiles && !*abortp; ++i) {
      const int s = i & 1, ph = ((i >> 1) & 1) ^ 1;
      const int page = a.page_table[(size_t)seq * a.max_pages + p0 + i];
      if (!mbar_wait_bounded(&k_empty[s], ph, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, i); break; }
      if (lane == 0) {
        mbar_expect_tx(&k_full[s], 16384);
        tma_load_3d_hint(sK + s * 16384, a.kv_map, &k_full[s], 0, kvh, page * APAGE, kvpol);
        tma_load_3d_hint(sK + s * 16384 + 8192, a.kv_map, &k_full[s], 64, kvh, page * APAGE, kvpol);
      }
      if (!mbar_wait_bounded(&v_empty[s], ph, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, i); break; }
      if (lane == 0) {
        mbar_expect_tx(&v_full[s], 16384);
        tma_load_3d_hint(sV + s * 16384, a.kv_map, &v_full[s], 0, a.Hkv + kvh, page * APAGE, kvpol);
        tma_load_3d_hint(sV + s * 16384 + 8192, a.kv_map, &v_full[s], 64, a.Hkv + kvh, page * APAGE, kvpol);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Scores are double-buffered in tensor memory: S(i+1) is computed while the softmax of tile i runs.
    const uint32_t id_s = idesc_bf16(64, 0), id_o = idesc_bf16(128, 1);
    auto issue_scores = [&](int j) -> bool {     // S[j & 1] = Q K(j)^T
      const int s = j & 1;
      if (!mbar_wait_bounded(&k_full[s], (j >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, j); return false; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k0 = smem_u32(sK + s * 16384), d = tmem + (s ? S1_COL : S0_COL);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f16(d, desc_kmajor_sw128(smem_u32(sQ) + kb * 16384) + 2 * k, desc_kmajor_sw128(k0 + kb * 8192) + 2 * k, id_s, (kb | k) ? 1u : 0u);
        tc_commit(&s_full[s]);
        tc_commit(&k_empty[s]);
      }
      __syncwarp();
      return true;
    };
    bool ok = true;
    for (int j = 0; ok && j < min(2, n_tiles); ++j) ok = issue_scores(j);
    for (int i = 0; ok && i < n_tiles; ++i) {
      const int s = i & 1;
      if (!mbar_wait_bounded(&p_full, i & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, i); break; }
      if (!mbar_wait_bounded(&v_full[s], (i >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, i); break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v0 = smem_u32(sV + s * 16384);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_f16(tmem + O_COL, desc_kmajor_sw128(smem_u32(sP)) + 2 * k, desc_mnmajor_sw128(v0 + k * 2048, 8192, 1024), id_o, (i | k) ? 1u : 0u);
        tc_commit(&v_empty[s]);
        tc_commit(&o_done);
      }
      __syncwarp();
      if (i + 2 < n_tiles) ok = issue_scores(i + 2);   // S[i & 1] was consumed before p_full(i) completed
    }
  } else if ((warp & 3) >= n_live_warps) {
    // softmax warps whose 32 rows are all padding: nothing to do (their P rows only feed their own unused O rows)
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: thread = row
    const int q4 = warp & 3, r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const bool live = r < R;                  // in the replicated layout quarter 0 (r = lane) holds the real rows
    const int qpos = live ? first_pos + r / G : -1;
    const float sc2 = a.scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    if (rep4) {
      // ---- column-split path: thread (q4, lane) owns row `lane`, score columns [16*q4, 16*q4 + 16)
      const bool rlive = lane < R;
      const int rq = rlive ? first_pos + lane / G : -1;
      float* xchg = (float*)(sP + 8192);                 // [2][4][32] row maxima (P rows >= 64 are never read back)
      float* lsum = xchg + 256;                          // [4][32]
      const int col0 = 16 * q4;
      for (int i = 0; i < n_tiles; ++i) {
        if (!mbar_wait_bounded(&s_full[i & 1], (i >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
        tc_fence_after();
        uint32_t sr[16];
        tmem_ld_x16(tmem + lane_addr + ((i & 1) ? S1_COL : S0_COL) + col0, sr);
        tc_wait_ld();
        const int key0 = (p0 + i) * APAGE + col0;
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int kp = key0 + j;
          const bool vis = rlive && kp <= rq && kp < kvlen && (a.window <= 0 || kp > rq - a.window);
          const float v = vis ? __uint_as_float(sr[j]) * sc2 : -INFINITY;
          sr[j] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
        float* xb = xchg + (i & 1) * 128;
        xb[q4 * 32 + lane] = mx;
        mbar_arrive(&x_bar);
        if (!mbar_wait_bounded(&x_bar, i & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
        mx = fmaxf(fmaxf(xb[lane], xb[32 + lane]), fmaxf(xb[64 + lane], xb[96 + lane]));
        if (i > 0 && !mbar_wait_bounded(&o_done, (i - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
        tc_fence_after();
        float alpha = 1.f;
        if (mx > m_ref + 8.f) {
          if (m_ref != -INFINITY) { alpha = exp2f(m_ref - mx); l *= alpha; }
          m_ref = mx;
        }
        if (q4 == 0 && i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {     // the real O rows live in lane quarter 0
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t o[16];
            tmem_ld_x16(tmem + O_COL + c * 16, o);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st_x16(tmem + O_COL + c * 16, o);
          }
          tc_wait_st();
        }
        uint32_t pk[8];
        float psum = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float a0 = __uint_as_float(sr[2 * j]), a1 = __uint_as_float(sr[2 * j + 1]);
          const float e0 = (m_ref == -INFINITY) ? 0.f : exp2f(a0 - m_ref), e1 = (m_ref == -INFINITY) ? 0.f : exp2f(a1 - m_ref);
          psum += e0 + e1;
          bf162 h = __floats2bfloat162_rn(e0, e1);
          pk[j] = *(uint32_t*)&h;
        }
        l += psum;
        *(uint4*)(sP + lane * 128 + (((2 * q4) ^ (lane & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        *(uint4*)(sP + lane * 128 + (((2 * q4 + 1) ^ (lane & 7)) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&p_full);
      }
      // total row sums: every warp contributes the sum over its 16 columns
      lsum[q4 * 32 + lane] = l;
      mbar_arrive(&x_bar);
      if (ok && !mbar_wait_bounded(&x_bar, n_tiles & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 998); ok = false; }
      l = lsum[lane] + lsum[32 + lane] + lsum[64 + lane] + lsum[96 + lane];
    } else
    for (int i = 0; i < n_tiles; ++i) {
      if (!mbar_wait_bounded(&s_full[i & 1], (i >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
      tc_fence_after();
      uint32_t sr[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_x16(tmem + lane_addr + ((i & 1) ? S1_COL : S0_COL) + c * 16, sr + c * 16);
      tc_wait_ld();
      const int key0 = (p0 + i) * APAGE;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const int kp = key0 + j;
        const bool vis = live && kp <= qpos && kp < kvlen && (a.window <= 0 || kp > qpos - a.window);
        const float v = vis ? __uint_as_float(sr[j]) * sc2 : -INFINITY;
        sr[j] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
      // the previous P V product must have finished before P is overwritten or O rescaled
      if (i > 0 && !mbar_wait_bounded(&o_done, (i - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
      tc_fence_after();
      // Lazy rescale.  tcgen05.ld/st are warp-collective (.sync.aligned), so the decision is made per warp:
      // if any lane must move its reference max, every lane runs the read-scale-write (alpha = 1 where not needed).
      const bool grow = mx > m_ref + 8.f;   // also true the first time a key becomes visible (m_ref = -inf)
      float alpha = 1.f;
      if (grow) {
        if (m_ref != -INFINITY) { alpha = exp2f(m_ref - mx); l *= alpha; }
        m_ref = mx;
      }
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[16];
          tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st_x16(tmem + lane_addr + O_COL + c * 16, o);
        }
        tc_wait_st();
      }
      float psum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float a0 = __uint_as_float(sr[2 * j]), a1 = __uint_as_float(sr[2 * j + 1]);
        const float e0 = (m_ref == -INFINITY) ? 0.f : exp2f(a0 - m_ref), e1 = (m_ref == -INFINITY) ? 0.f : exp2f(a1 - m_ref);
        psum += e0 + e1;
        bf162 h = __floats2bfloat162_rn(e0, e1);
        pk[j] = *(uint32_t*)&h;
      }
      l += psum;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *(uint4*)(sP + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    if (ok && n_tiles > 0 && !mbar_wait_bounded(&o_done, (n_tiles - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 999); ok = false; }
    tc_fence_after();
    // Epilogue.  The tensor-memory reads are warp-collective: every lane of a warp executes them (rows past
    // R read zeros or stale columns and simply do not store).
    if (__all_sync(0xffffffffu, ok) && (!rep4 || q4 == 0)) {
      const int rr = live ? r : 0;
      const int t = row_base + rr / G, h = kvh * G + rr % G;
      const float m_nat = (m_ref == -INFINITY) ? -INFINITY : m_ref * 0.6931471805599453f;
      float scale_o = 1.f, lt = l;
      if (a.n_splits == 1 && a.sink) {
        const float sk = a.sink[h], m2 = fmaxf(m_nat, sk);
        const float e1 = (m_nat == -INFINITY) ? 0.f : __expf(m_nat - m2);
        lt = l * e1 + __expf(sk - m2); scale_o = e1;
      }
      const float inv = lt > 0.f ? scale_o / lt : 0.f;
      bf16* dst = a.out + (size_t)t * a.Hq * AD + (size_t)h * AD;
      float* po = a.n_splits > 1 ? a.part_o + (((size_t)split * a.T + t) * a.Hq + h) * AD : nullptr;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t o[16];
        if (n_tiles > 0) { tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o); tc_wait_ld(); }   // n_tiles is CTA-uniform
        else {
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = 0;
        }
        if (!live) continue;
        if (a.n_splits == 1) {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) { bf162 hh = __floats2bfloat162_rn(__uint_as_float(o[2 * j]) * inv, __uint_as_float(o[2 * j + 1]) * inv); w[j] = *(uint32_t*)&hh; }
          *(uint4*)(dst + c * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          *(uint4*)(dst + c * 16 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) *(uint4*)(po + c * 16 + j * 4) = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        }
      }
      if (live && a.n_splits > 1) {
        float* ml = a.part_ml + (((size_t)split * a.T + t) * a.Hq + h) * 2;
        ml[0] = m_nat; ml[1] = l;
      }
    }
  }
  if (*abortp && warp == 0) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 200000) __nanosleep(1000); }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 256);
}

// Context split (a long context whose KV pages live on several GPUs): every owner runs the attention over ITS pages
// with "partials only" armed, which leaves the unnormalised outputs and (max, sum) pairs of its splits in the scratch
// buffers instead of merging them; the partials of all owners are then laid side by side ([owner 0 splits | owner 1
// splits | ...], moved with the ordinary peer copy) and merged once by `cuteafd_attn_merge`.  For decode rows
// (one query token per sequence) every cached key is visible to the query, so each owner simply passes the length of
// its own part.  Reference: the token-split attention exchange of the two-GPU coordinator split
// (shared/peer_split/context.rs) and its `lse_combine2` primitive.
static thread_local bool g_partials_only = false;
extern "C" int cuteafd_attn_partials_only() { g_partials_only = true; return CA_OK; }   // arms the next attention call of this thread

extern "C" int cuteafd_attn_merge(const float* part_o, const float* part_ml, const float* sink, void* out, int T, int Hq, int n_parts,
                                  cudaStream_t s) {
  CA_REQUIRE(part_o && part_ml && out && n_parts >= 1, "attn_merge: needs partials");
  if (T <= 0) return CA_OK;
  CA_LAUNCH_PDL(attn_merge8_kernel, dim3(T, (Hq * AD / 8 + 127) / 128), 128, 0, s, part_o, part_ml, sink, (bf16*)out, T, Hq, (int)AD, n_parts,
                (uint8_t*)nullptr, (uint8_t*)nullptr, 0, (const float*)nullptr, 0);
  CA_CHECK_LAUNCH("attn_merge");
  return CA_OK;
}

extern "C" int cuteafd_paged_attention_tc(const void* q, const void* kv_map, const int* page_table, const int* kv_len,
                                          const int* q_start, const int* q_len, const float* sink, void* out, float* part_o,
                                          float* part_ml, int T, int n_seq, int max_q_len, int q_stride, int Hq, int Hkv,
                                          int max_pages, int n_splits, int window, float scale, int* status, void* q_out, void* sf_out,
                                          int ldsf, const float* inv_gs, int qkind, cudaStream_t s) {
  // q_out/sf_out (qkind 1 NVFP4 / 2 MXFP4): with split-KV the merge also writes the output rows quantised for the
  // projection that follows; ignored (the caller quantises) when n_splits == 1.
  CA_REQUIRE(qkind == 0 || (q_out && sf_out && (Hq * AD) % 256 == 0), "paged_attention_tc: FP4 output needs buffers and Hq*128 %% 256 == 0");
  CA_REQUIRE(Hq % Hkv == 0 && 128 % (Hq / Hkv) == 0, "paged_attention_tc: group size %d unsupported", Hq / Hkv);
  CA_REQUIRE(n_splits >= 1 && (n_splits == 1 || (part_o && part_ml)), "paged_attention_tc: split-KV needs scratch");
  CA_REQUIRE(q_stride % 8 == 0, "paged_attention_tc: q rows must be 16-byte aligned");
  const bool partials_only = g_partials_only;
  g_partials_only = false;
  CA_REQUIRE(!partials_only || n_splits >= 2, "paged_attention_tc: partials-only needs at least two splits");
  if (T <= 0 || n_seq <= 0) return CA_OK;
  AttnTcArgs a;
  a.q = (const bf16*)q; a.kv_map = (const CUtensorMap*)kv_map; a.page_table = page_table; a.kv_len = kv_len; a.q_start = q_start;
  a.q_len = q_len; a.sink = sink; a.out = (bf16*)out; a.part_o = part_o; a.part_ml = part_ml; a.status = status;
  a.q_stride = q_stride; a.Hq = Hq; a.Hkv = Hkv; a.max_pages = max_pages; a.n_splits = n_splits; a.window = window; a.T = T; a.scale = scale;
  const int tpt = 128 / (Hq / Hkv);
  a.max_q_tiles = (max_q_len + tpt - 1) / tpt;
  const int smem = 49152 + NS * 32768 + 128;
  static bool attr_set[64] = {false};
  int dev = 0; cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(paged_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(paged_attn_tc)");
    attr_set[dev & 63] = true;
  }
  // No pre-fill of the (m, l) partials: every CTA writes them for all of its live rows, also when its split
  // holds no key (m = -inf, l = 0), and a CTA that gives up reports through the status word.
  dim3 grid(n_splits, Hkv, n_seq * a.max_q_tiles);
  CA_LAUNCH_PDL(paged_attn_tc_kernel, grid, 192, smem, s, a);
  CA_CHECK_LAUNCH("paged_attention_tc");
  if (n_splits > 1 && !partials_only) {
    CA_LAUNCH_PDL(attn_merge8_kernel, dim3(T, (Hq * AD / 8 + 127) / 128), 128, 0, s, part_o, part_ml, sink, (bf16*)out, T, Hq, (int)AD, n_splits,
                  (uint8_t*)q_out, (uint8_t*)sf_out, ldsf, inv_gs, qkind);
    CA_CHECK_LAUNCH("attn_merge");
  }
  return CA_OK;
}

// Descriptor for one layer's paged K/V store [slots, 2, Hkv, 128] bf16: dims {128, 2*Hkv, slots}, box {64, 1, 64}.
extern "C" int cuteafd_tmap_encode_kv(void* out128, const void* base, int Hkv, uint64_t n_slots) {
  CUtensorMap m;
  int rc = ca_encode_tmap_3d(&m, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, AD, 2 * (uint64_t)Hkv, n_slots, AD * 2,
                             (uint64_t)2 * Hkv * AD * 2, 64, 1, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  memcpy(out128, &m, sizeof(m));
  return CA_OK;
}
