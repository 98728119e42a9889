// Multi-head latent attention (DeepSeek-V3 style), absorbed form, on the 5th-generation tensor cores.
//
// Every head of a token attends to the same per-token latent: cache row = [c_kv (512, RMS-normed) | k_rope (64)] in
// bf16.  With W_UK folded into the query (q_lat = W_UK^T q_nope) the score of head h is q_full[h] . row, q_full =
// [q_lat (512) | q_rope (64)], and the value is the latent itself (W_UV is applied afterwards), so the kernel is an
// MQA with a 576-wide QK and a 512-wide V that share one cache row.
//
// CTA = (KV split, V half, sequence x query tile); rows of the MMA tile = local heads x tokens (128 rows).
//   S[128 x 64]   = Q K^T over nine 64-wide chunks (tcgen05.mma kind::f16; Q is resident: chunks 0..5 in tensor
//                   memory as the A operand, chunks 6..8 in shared memory; K tiles of 64 keys x 576 = one page
//                   through a two-stage TMA ring).  A score MMA costs ~130 cycles here whether it covers 32 or 64
//                   keys and wherever its A operand lives, so wide tiles are what makes the scores cheaper.
//   softmax       thread per row, lazy rescale (as in the GQA kernel), P in bf16 to shared memory
//   O[128 x 256] += P V_half, V_half read in place from the K tile as an MN-major operand (chunks 4*vh .. 4*vh+3)
// The 512-wide fp32 output of 128 rows would fill all of tensor memory, so the V dimension is split over two CTAs
// that both compute the (cheap) scores; adjacent CTAs run together, so the second reads the latent from L2.
// Outputs are head-major [heads, T, 512] for the grouped W_UV GEMM that follows; with several KV splits the
// unnormalised partials go to scratch and `mla_merge_kernel` combines them.
//
// Reference counterparts: native/shared/cuda/attention.cu:385 (mla_compressed_attention_bf16), :986 (merge),
// families/glm5/cuda/glm_mla_prefill.cu:123-960 (mma.sync MLA prefill), kv_cache.cu:142 (mla_kv_prepare).
#include <stdlib.h>
#include <string.h>
#include <cuda_fp16.h>

#define CA_PDL_CLASS 2
#include "common.cuh"

#define MKEYS 64            // keys per tile = one page
#define MPAGE 64
#define DQK 576
#define DV 512
#define NCH 9            // 64-wide chunks of the QK dimension

struct MlaArgs {
  const bf16* q_lat;        // [Hl * T, 512] head-major
  const bf16* q_rope;       // [T, Hl, 64]
  const CUtensorMap* kv_map;    // 2-D (as 3-D): {576, slots, 1}, box {64, 32, 1}, 128-byte swizzle
  const int* page_table; const int* kv_len; const int* q_start; const int* q_len;
  bf16* out;                // [Hl, T, 512] head-major
  float* part_o;            // [splits, T, Hl, 512]
  float* part_ml;           // [splits, T, Hl, 2]
  int* status;
  int Hl, max_pages, n_splits, max_q_tiles, T;
  float scale;
};

__device__ __forceinline__ uint64_t mla_desc_k_sw128(uint32_t saddr) { return umma_desc_sw128(saddr); }
__device__ __forceinline__ uint64_t mla_desc_mn_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// K-major operand without swizzle: 8-row x 16-byte core matrices, `lbo` bytes between core matrices along K,
// `sbo` bytes between 8-row groups.
__device__ __forceinline__ uint64_t mla_desc_k_plain(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ uint32_t mla_idesc(int n, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void mla_tmem_st_x16(uint32_t addr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                 "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

#define QT_CH 6                             // Q chunks 0..5 live in tensor memory (192 columns), chunks 6..8 in shared memory
#define NST 2                               // latent tile stages
#define SQ_BYTES ((NCH - QT_CH) * 16384)    // 3 chunks x [128 rows x 128 B]
#define SK_CHUNK (MKEYS * 128)              // one 64-wide chunk of a tile: [64 keys x 128 B]
#define SK_STAGE (NCH * SK_CHUNK)           // 9 chunks
#define SP_BYTES (128 * MKEYS * 2)          // [128 rows x 64 keys] bf16, core-matrix layout
#define MLA_SMEM (SQ_BYTES + NST * SK_STAGE + SP_BYTES + 128)

__global__ void __launch_bounds__(192, 1) mla_attn_kernel(const __grid_constant__ MlaArgs a) {
  pdl_launch(); pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = smem + SQ_BYTES;
  uint8_t* sP = sK + NST * SK_STAGE;
  uint64_t* bars = (uint64_t*)(sP + SP_BYTES);
  uint64_t* k_full = bars; uint64_t* k_empty = bars + NST;
  uint64_t& s_full = bars[2 * NST]; uint64_t& s_free = bars[2 * NST + 1];
  uint64_t& p_full = bars[2 * NST + 2]; uint64_t& o_done = bars[2 * NST + 3];
  uint32_t& tmem_slot = *(uint32_t*)(bars + 2 * NST + 4);
  int& abort_flag = *(int*)(bars + 2 * NST + 5);
  if (smem_u32(smem) & 1023) { if (threadIdx.x == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, 0xA12); return; }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

  const int tok_per_tile = 128 / a.Hl;
  const int split = blockIdx.x, vh = blockIdx.y;
  const int seq = blockIdx.z / a.max_q_tiles, qt = blockIdx.z % a.max_q_tiles;
  const int qlen = a.q_len[seq], kvlen = a.kv_len[seq];
  const int tok0 = qt * tok_per_tile;
  if (tok0 >= qlen) return;
  const int ntok = min(tok_per_tile, qlen - tok0);
  const int R = ntok * a.Hl;
  const int row_base = a.q_start[seq] + tok0;
  const int first_pos = kvlen - qlen + tok0;
  const int hi = first_pos + ntok;
  const int last_tile = (hi + MKEYS - 1) / MKEYS;                     // key tiles [0, last_tile)
  const int per = (last_tile + a.n_splits - 1) / a.n_splits;
  const int t0 = split * per, t1 = min(last_tile, t0 + per);
  const int n_tiles = max(0, t1 - t0);

  if (tid == 0) {
    for (int s = 0; s < NST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    mbar_init(&s_full, 1); mbar_init(&s_free, 128);
    mbar_init(&p_full, 128); mbar_init(&o_done, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  // Q rows: the 64-wide chunks 6, 7 (q_lat) and 8 (q_rope) become swizzled K-major tiles in shared memory ...
  for (int i = tid; i < 128 * 24; i += 192) {
    const int r = i / 24, c = 8 * QT_CH + i % 24;        // 16-byte chunk c (8 elements) of row r
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < R) {
      const int t = row_base + r / a.Hl, h = r % a.Hl;
      v = (c < 64) ? *(const uint4*)(a.q_lat + ((size_t)h * a.T + t) * DV + c * 8)
                   : *(const uint4*)(a.q_rope + ((size_t)t * a.Hl + h) * 64 + (c - 64) * 8);
    }
    *(uint4*)(sQ + ((c >> 3) - QT_CH) * 16384 + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;
  const uint32_t S_COL = 0, O_COL = 64, QT_COL = 320;
  // ... and chunks 0..5 go to tensor memory (row = lane, two elements per 32-bit column), where the score MMAs
  // read them as the A operand without touching shared memory; that leaves room there for two 64-key stages, and Q is
  // the same for every tile.
  if (warp >= 2) {
    const int r = (warp & 3) * 32 + lane;
    const uint32_t dst = tmem + ((uint32_t)((warp & 3) * 32) << 16) + QT_COL;
    const bf16* src = a.q_lat + ((size_t)((r < R ? r : 0) % a.Hl) * a.T + row_base + (r < R ? r : 0) / a.Hl) * DV;
#pragma unroll 1
    for (int g = 0; g < QT_CH * 2; ++g) {                // 16 columns = 32 elements per store
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 v = r < R ? *(const uint4*)(src + g * 32 + j * 8) : make_uint4(0, 0, 0, 0);
        w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
      }
      mla_tmem_st_x16(dst + g * 16, w);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp == 0) {
    // ------------------------------------------------------------------ latent tile producer
    for (int i = 0; i < n_tiles && !*abortp; ++i) {
      const int s = i % NST;
      if (!mbar_wait_bounded(&k_empty[s], ((i / NST) & 1) ^ 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, i); break; }
      if (lane == 0) {
        const int key0 = (t0 + i) * MKEYS;
        const int page = a.page_table[(size_t)seq * a.max_pages + key0 / MPAGE];
        const int slot0 = page * MPAGE + key0 % MPAGE;
        mbar_expect_tx(&k_full[s], SK_STAGE);
#pragma unroll
        for (int c = 0; c < NCH; ++c) tma_load_3d(sK + s * SK_STAGE + c * SK_CHUNK, a.kv_map, &k_full[s], c * 64, slot0, 0);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t id_s = mla_idesc(MKEYS, 0), id_o = mla_idesc(256, 1);
    // One thread issues everything.  It polls two conditions and serves whichever is ready: "the latent tile qk has
    // landed and the score buffer is free" (issue its scores) and "the probabilities of tile pv are in shared memory"
    // (issue its PV product, which also releases the tile's stage to the producer).  The 36 score MMAs of a tile
    // keep the issuing thread busy for as long as they execute (~130 cycles each whatever their operands, so a tile
    // is 64 keys wide to halve the count per key), and the PV probe is repeated between the 64-wide chunks:
    // otherwise a PV product that became ready just after the scores started would wait a whole score pass, and with
    // it the stage release and the next load.
    // There is one score buffer: the softmax threads copy it to registers first thing and release it (s_free).
    if (lane == 0) {
      int qk = 0, pv = 0, idle = 0;
      long long idle_t0 = 0;
      auto try_pv = [&]() -> bool {
        if (pv >= qk || !mbar_test(&p_full, pv & 1)) return false;
        tc_fence_after();
        const int s = pv % NST;
        const uint32_t v0 = smem_u32(sK + s * SK_STAGE) + (4 * vh) * SK_CHUNK;
#pragma unroll
        for (int k = 0; k < MKEYS / 16; ++k)       // 16 keys per MMA: two 8-key groups = 2048 B along K
          tc_mma_f16(tmem + O_COL, mla_desc_k_plain(smem_u32(sP) + k * 256, 128, MKEYS * 16), mla_desc_mn_sw128(v0 + k * 2048, SK_CHUNK, 1024), id_o,
                     (pv | k) ? 1u : 0u);
        tc_commit(&k_empty[s]);
        tc_commit(&o_done);
        ++pv;
        return true;
      };
      while (pv < n_tiles) {
        bool did = try_pv();
        if (qk < n_tiles && (qk == 0 || mbar_test(&s_free, (qk - 1) & 1)) && mbar_test(&k_full[qk % NST], (qk / NST) & 1)) {
          tc_fence_after();
          const uint32_t k0 = smem_u32(sK + (qk % NST) * SK_STAGE), d = tmem + S_COL;
#pragma unroll 1
          for (int c = 0; c < NCH; ++c) {
            if (c < QT_CH) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                tc_mma_f16_ta(d, tmem + QT_COL + c * 32 + k * 8, mla_desc_k_sw128(k0 + c * SK_CHUNK) + 2 * k, id_s, (c | k) ? 1u : 0u);
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                tc_mma_f16(d, mla_desc_k_sw128(smem_u32(sQ) + (c - QT_CH) * 16384) + 2 * k, mla_desc_k_sw128(k0 + c * SK_CHUNK) + 2 * k, id_s, 1u);
            }
            if (c + 1 < NCH) try_pv();
          }
          tc_commit(&s_full);
          ++qk;
          did = true;
        }
        if (did) { idle = 0; continue; }
        if (idle++ == 0) idle_t0 = clock64();
        if ((idle & 255) == 0) {
          if (*abortp) break;
          if (clock64() - idle_t0 > 4000000000LL) { *abortp = 1; ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, pv); break; }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: thread = row
    const int q4 = warp & 3, r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const bool live = r < R;
    const int qpos = live ? first_pos + r / a.Hl : -1;
    const float sc2 = a.scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      if (!mbar_wait_bounded(&s_full, i & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
      tc_fence_after();
      uint32_t sr[MKEYS];
#pragma unroll
      for (int j = 0; j < MKEYS / 16; ++j) tmem_ld_x16(tmem + lane_addr + S_COL + 16 * j, sr + 16 * j);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&s_free);                                // the scores are in registers: the next tile may overwrite them
      const int key0 = (t0 + i) * MKEYS;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < MKEYS; ++j) {
        const int kp = key0 + j;
        const float v = (live && kp <= qpos && kp < kvlen) ? __uint_as_float(sr[j]) * sc2 : -INFINITY;
        sr[j] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
      float alpha = 1.f;
      if (mx > m_ref + 8.f) {
        if (m_ref != -INFINITY) { alpha = exp2f(m_ref - mx); l *= alpha; }
        m_ref = mx;
      }
      // the probabilities only need the reference maximum, so they are computed while PV(i - 1) still runs; the
      // wait below guards the accumulator rescale and the P buffer, both of which PV(i - 1) uses
      uint32_t pk[MKEYS / 2];
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < MKEYS / 2; ++j) {
        const float a0 = __uint_as_float(sr[2 * j]), a1 = __uint_as_float(sr[2 * j + 1]);
        const float e0 = (m_ref == -INFINITY) ? 0.f : exp2f(a0 - m_ref), e1 = (m_ref == -INFINITY) ? 0.f : exp2f(a1 - m_ref);
        psum += e0 + e1;
        bf162 h = __floats2bfloat162_rn(e0, e1);
        pk[j] = *(uint32_t*)&h;
      }
      l += psum;
      if (i > 0 && !mbar_wait_bounded(&o_done, (i - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
      tc_fence_after();
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {       // warp-uniform: tcgen05.ld/st are warp collectives
#pragma unroll 1
        for (int c = 0; c < 16; ++c) {
          uint32_t o[16];
          tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          mla_tmem_st_x16(tmem + lane_addr + O_COL + c * 16, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      // core-matrix layout: 8-row groups 1024 B apart, the eight 8-key columns 128 B apart, 16 B per row inside
#pragma unroll
      for (int c = 0; c < MKEYS / 8; ++c)
        *(uint4*)(sP + (r >> 3) * (MKEYS * 16) + c * 128 + (r & 7) * 16) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    if (ok && n_tiles > 0 && !mbar_wait_bounded(&o_done, (n_tiles - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 999); ok = false; }
    tc_fence_after();
    if (__all_sync(0xffffffffu, ok)) {
      const int rr = live ? r : 0;
      const int t = row_base + rr / a.Hl, h = rr % a.Hl;
      const float m_nat = (m_ref == -INFINITY) ? -INFINITY : m_ref * 0.6931471805599453f;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = a.out + ((size_t)h * a.T + t) * DV + vh * 256;
      float* po = a.n_splits > 1 ? a.part_o + (((size_t)split * a.T + t) * a.Hl + h) * DV + vh * 256 : nullptr;
#pragma unroll 1
      for (int c = 0; c < 16; ++c) {
        uint32_t o[16];
        if (n_tiles > 0) { tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o); tc_wait_ld(); }
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
      if (live && a.n_splits > 1 && vh == 0) {
        float* ml = a.part_ml + (((size_t)split * a.T + t) * a.Hl + h) * 2;
        ml[0] = m_nat; ml[1] = l;
      }
    }
  }
  if (*abortp && warp == 0) { const long long c0 = clock64(); while (clock64() - c0 < 400000) __nanosleep(1000); }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------------------
// Paired variant: the two V-half CTAs of a (split, sequence x query tile) form a thread-block cluster and SHARE the score
// work instead of both computing all of it.  CTA 0 owns the score chunks 0..4 of the 576-wide QK dimension, CTA 1 the chunks
// 5..8; each issues only its own score MMAs into a partial S tile, its softmax threads read that partial from tensor memory,
// store it as fp16 into the partner's shared memory over the cluster network (st.shared::cluster) and release a
// cluster-scope mbarrier there, then add the partner's partial to their own fp32 one: both CTAs hold the full scores after
// one 16 KB exchange per 64-key tile, at 20 / 16 score MMAs per tile instead of 36.  The exchange is software-pipelined: the
// partial of tile i + 1 is sent BEFORE the softmax of tile i is computed, so it travels under that computation.
// A CTA needs only five of the nine 64-wide chunks of a key tile (its score chunks and its V half overlap in all but one),
// so stages shrink from 72 KB to 40 KB, three fit, and the whole query lives in tensor memory.  No multicast anywhere: each
// CTA issues its own TMA loads from local memory.  (The partner's half of a raw score is rounded to fp16, relative error
// 2^-11, before the 1/sqrt(d) scaling: below the bf16 rounding of the probabilities.)
#define PNST 3                                  // latent tile stages (five chunks each)
#define PCH 5                                   // chunks a CTA loads per tile
#define PK_STAGE (PCH * SK_CHUNK)
#define PX_BYTES (128 * MKEYS * 2)              // one partial score tile, fp16, [16-byte column group][row]
#define MLA_PAIR_SMEM (PNST * PK_STAGE + SP_BYTES + 2 * PX_BYTES + 256)

__device__ __forceinline__ uint32_t mla_mapa(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mla_st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void mla_arrive_cluster(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mla_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait on a barrier the PARTNER CTA arrives on (cluster-scope acquire).
__device__ __forceinline__ bool mla_wait_cluster_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mla_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64(), limit = 4000000000LL;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mla_try_wait_cluster(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) { *abort_flag = 1; return false; }
  }
}

__global__ void __launch_bounds__(192, 1) mla_attn_pair_kernel(const __grid_constant__ MlaArgs a) {
  pdl_launch(); pdl_wait();
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sP = sK + PNST * PK_STAGE;
  uint8_t* sX = sP + SP_BYTES;
  uint64_t* bars = (uint64_t*)(sX + 2 * PX_BYTES);
  uint64_t* k_full = bars; uint64_t* k_empty = bars + PNST;
  uint64_t& s_full = bars[2 * PNST]; uint64_t& s_free = bars[2 * PNST + 1];
  uint64_t& p_full = bars[2 * PNST + 2]; uint64_t& o_done = bars[2 * PNST + 3];
  uint64_t* x_full = bars + 2 * PNST + 4;                 // [2]: the partner's partial scores of tile i landed in sX[i & 1]
  uint32_t& tmem_slot = *(uint32_t*)(bars + 2 * PNST + 6);
  int& abort_flag = *(int*)(bars + 2 * PNST + 7);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const bool aligned = (smem_u32(smem) & 1023) == 0;       // same answer in both CTAs of the pair (same kernel, same layout)

  const int tok_per_tile = 128 / a.Hl;
  const int split = blockIdx.x, vh = blockIdx.y;           // vh = rank in the cluster (cluster shape 1 x 2 x 1)
  const int seq = blockIdx.z / a.max_q_tiles, qt = blockIdx.z % a.max_q_tiles;
  const int qlen = a.q_len[seq], kvlen = a.kv_len[seq];
  const int tok0 = qt * tok_per_tile;
  if (tok0 >= qlen || !aligned) {                         // both CTAs of a pair take this exit together
    if (!aligned && tid == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, 0xA12);
    return;
  }
  const int ntok = min(tok_per_tile, qlen - tok0);
  const int R = ntok * a.Hl;
  const int row_base = a.q_start[seq] + tok0;
  const int first_pos = kvlen - qlen + tok0;
  const int hi = first_pos + ntok;
  const int last_tile = (hi + MKEYS - 1) / MKEYS;
  const int per = (last_tile + a.n_splits - 1) / a.n_splits;
  const int t0 = split * per, t1 = min(last_tile, t0 + per);
  const int n_tiles = max(0, t1 - t0);
  const int c_lo = vh ? 5 : 0, c_hi = vh ? NCH : 5;        // score chunks of this CTA
  const int l_lo = vh ? 4 : 0;                             // first of the five chunks it loads (score chunks + V half 4 * vh .. 4 * vh + 3)

  if (tid == 0) {
    for (int s = 0; s < PNST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    mbar_init(&s_full, 1); mbar_init(&s_free, 128);
    mbar_init(&p_full, 128); mbar_init(&o_done, 1);
    mbar_init(&x_full[0], 128); mbar_init(&x_full[1], 128);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // the partner must have initialised its barriers before anyone arrives on them remotely
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;
  const uint32_t S_COL = 0, O_COL = 64, QT_COL = 320;
  // this CTA's query chunks -> tensor memory (row = lane, two elements per 32-bit column, 32 columns per 64-wide chunk)
  if (warp >= 2) {
    const int r = (warp & 3) * 32 + lane;
    const uint32_t dst = tmem + ((uint32_t)((warp & 3) * 32) << 16) + QT_COL;
    const int rr = r < R ? r : 0;
    const int t = row_base + rr / a.Hl, h = rr % a.Hl;
    const bf16* src_lat = a.q_lat + ((size_t)h * a.T + t) * DV;
    const bf16* src_rope = a.q_rope + ((size_t)t * a.Hl + h) * 64;
#pragma unroll 1
    for (int c = c_lo; c < c_hi; ++c) {
      const bf16* src = c < 8 ? src_lat + c * 64 : src_rope;
#pragma unroll
      for (int half = 0; half < 2; ++half) {             // 16 columns = 32 elements per store
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 v = r < R ? *(const uint4*)(src + half * 32 + j * 8) : make_uint4(0, 0, 0, 0);
          w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
        }
        mla_tmem_st_x16(dst + (c - c_lo) * 32 + half * 16, w);
      }
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp == 0) {
    // ------------------------------------------------------------------ latent tile producer (five chunks per tile)
    for (int i = 0; i < n_tiles && !*abortp; ++i) {
      const int s = i % PNST;
      if (!mbar_wait_bounded(&k_empty[s], ((i / PNST) & 1) ^ 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, i); break; }
      if (lane == 0) {
        const int key0 = (t0 + i) * MKEYS;
        const int page = a.page_table[(size_t)seq * a.max_pages + key0 / MPAGE];
        const int slot0 = page * MPAGE + key0 % MPAGE;
        mbar_expect_tx(&k_full[s], PK_STAGE);
#pragma unroll
        for (int j = 0; j < PCH; ++j) tma_load_3d(sK + s * PK_STAGE + j * SK_CHUNK, a.kv_map, &k_full[s], (l_lo + j) * 64, slot0, 0);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one thread; see mla_attn_kernel)
    const uint32_t id_s = mla_idesc(MKEYS, 0), id_o = mla_idesc(256, 1);
    if (lane == 0) {
      int qk = 0, pv = 0, idle = 0;
      long long idle_t0 = 0;
      auto try_pv = [&]() -> bool {
        if (pv >= qk || !mbar_test(&p_full, pv & 1)) return false;
        tc_fence_after();
        const int s = pv % PNST;
        const uint32_t v0 = smem_u32(sK + s * PK_STAGE);           // the V half is the first four chunks of the stage in both CTAs
#pragma unroll
        for (int k = 0; k < MKEYS / 16; ++k)
          tc_mma_f16(tmem + O_COL, mla_desc_k_plain(smem_u32(sP) + k * 256, 128, MKEYS * 16), mla_desc_mn_sw128(v0 + k * 2048, SK_CHUNK, 1024), id_o,
                     (pv | k) ? 1u : 0u);
        tc_commit(&k_empty[s]);
        tc_commit(&o_done);
        ++pv;
        return true;
      };
      while (pv < n_tiles) {
        bool did = try_pv();
        if (qk < n_tiles && (qk == 0 || mbar_test(&s_free, (qk - 1) & 1)) && mbar_test(&k_full[qk % PNST], (qk / PNST) & 1)) {
          tc_fence_after();
          const uint32_t k0 = smem_u32(sK + (qk % PNST) * PK_STAGE), d = tmem + S_COL;
#pragma unroll 1
          for (int c = c_lo; c < c_hi; ++c) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc_mma_f16_ta(d, tmem + QT_COL + (c - c_lo) * 32 + k * 8, mla_desc_k_sw128(k0 + (c - l_lo) * SK_CHUNK) + 2 * k, id_s, ((c - c_lo) | k) ? 1u : 0u);
            if (c + 1 < c_hi) try_pv();
          }
          tc_commit(&s_full);
          ++qk;
          did = true;
        }
        if (did) { idle = 0; continue; }
        if (idle++ == 0) idle_t0 = clock64();
        if ((idle & 255) == 0) {
          if (*abortp) break;
          if (clock64() - idle_t0 > 4000000000LL) { *abortp = 1; ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, pv); break; }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: thread = row
    const int q4 = warp & 3, r = q4 * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    const bool live = r < R;
    const int qpos = live ? first_pos + r / a.Hl : -1;
    const float sc2 = a.scale * 1.4426950408889634f;
    const uint32_t peer_x = mla_mapa(smem_u32(sX), (uint32_t)(vh ^ 1));
    const uint32_t peer_bar0 = mla_mapa(smem_u32(&x_full[0]), (uint32_t)(vh ^ 1)), peer_bar1 = mla_mapa(smem_u32(&x_full[1]), (uint32_t)(vh ^ 1));
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // fetch_send(j, dst): my partial scores of tile j -> registers (fp32) and, as fp16, into the partner's buffer j & 1
    // ([16-byte column group][row]: conflict-free on both sides); the release-arrive on its barrier publishes the stores.
    auto fetch_send = [&](int j, uint32_t* dst) -> bool {
      if (!mbar_wait_bounded(&s_full, j & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, j); return false; }
      tc_fence_after();
#pragma unroll
      for (int q = 0; q < MKEYS / 16; ++q) tmem_ld_x16(tmem + lane_addr + S_COL + 16 * q, dst + 16 * q);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&s_free);                                // the partial is in registers: the next tile may overwrite it
      const int b = j & 1;
#pragma unroll
      for (int g = 0; g < MKEYS / 8; ++g) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          __half2 h = __floats2half2_rn(__uint_as_float(dst[8 * g + 2 * q]), __uint_as_float(dst[8 * g + 2 * q + 1]));
          w[q] = *(uint32_t*)&h;
        }
        mla_st_cluster_v4(peer_x + b * PX_BYTES + (g * 128 + r) * 16, w[0], w[1], w[2], w[3]);
      }
      mla_arrive_cluster(b ? peer_bar1 : peer_bar0);
      return true;
    };
    uint32_t sr[MKEYS], nx[MKEYS];
    if (n_tiles > 0) ok = fetch_send(0, sr);
    for (int i = 0; ok && i < n_tiles; ++i) {
      // The partner's partial of tile i.  Order matters for the two-buffer scheme: I read buffer i & 1 BEFORE I send tile
      // i + 1, and the partner only overwrites buffer i & 1 (with its tile i + 2) after it has seen my tile i + 1.
      const int b = i & 1;
      if (!mla_wait_cluster_bounded(&x_full[b], (i >> 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 0x500 + i); ok = false; break; }
#pragma unroll
      for (int g = 0; g < MKEYS / 8; ++g) {
        const uint4 o = *(const uint4*)(sX + b * PX_BYTES + (g * 128 + r) * 16);
        const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __half22float2(*(const __half2*)&ow[q]);
          sr[8 * g + 2 * q] = __float_as_uint(__uint_as_float(sr[8 * g + 2 * q]) + f.x);
          sr[8 * g + 2 * q + 1] = __float_as_uint(__uint_as_float(sr[8 * g + 2 * q + 1]) + f.y);
        }
      }
      if (i + 1 < n_tiles && !fetch_send(i + 1, nx)) { ok = false; break; }     // travels under the softmax below
      const int key0 = (t0 + i) * MKEYS;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < MKEYS; ++j) {
        const int kp = key0 + j;
        const float v = (live && kp <= qpos && kp < kvlen) ? __uint_as_float(sr[j]) * sc2 : -INFINITY;
        sr[j] = __float_as_uint(v);
        mx = fmaxf(mx, v);
      }
      float alpha = 1.f;
      if (mx > m_ref + 8.f) {
        if (m_ref != -INFINITY) { alpha = exp2f(m_ref - mx); l *= alpha; }
        m_ref = mx;
      }
      uint32_t pk[MKEYS / 2];
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < MKEYS / 2; ++j) {
        const float a0 = __uint_as_float(sr[2 * j]), a1 = __uint_as_float(sr[2 * j + 1]);
        const float e0 = (m_ref == -INFINITY) ? 0.f : exp2f(a0 - m_ref), e1 = (m_ref == -INFINITY) ? 0.f : exp2f(a1 - m_ref);
        psum += e0 + e1;
        bf162 h = __floats2bfloat162_rn(e0, e1);
        pk[j] = *(uint32_t*)&h;
      }
      l += psum;
      if (i > 0 && !mbar_wait_bounded(&o_done, (i - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, i); ok = false; break; }
      tc_fence_after();
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {       // warp-uniform: tcgen05.ld/st are warp collectives
#pragma unroll 1
        for (int c = 0; c < 16; ++c) {
          uint32_t o[16];
          tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          mla_tmem_st_x16(tmem + lane_addr + O_COL + c * 16, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
#pragma unroll
      for (int c = 0; c < MKEYS / 8; ++c)
        *(uint4*)(sP + (r >> 3) * (MKEYS * 16) + c * 128 + (r & 7) * 16) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full);
#pragma unroll
      for (int j = 0; j < MKEYS; ++j) sr[j] = nx[j];
    }
    if (ok && n_tiles > 0 && !mbar_wait_bounded(&o_done, (n_tiles - 1) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 999); ok = false; }
    tc_fence_after();
    if (__all_sync(0xffffffffu, ok)) {
      const int rr = live ? r : 0;
      const int t = row_base + rr / a.Hl, h = rr % a.Hl;
      const float m_nat = (m_ref == -INFINITY) ? -INFINITY : m_ref * 0.6931471805599453f;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = a.out + ((size_t)h * a.T + t) * DV + vh * 256;
      float* po = a.n_splits > 1 ? a.part_o + (((size_t)split * a.T + t) * a.Hl + h) * DV + vh * 256 : nullptr;
#pragma unroll 1
      for (int c = 0; c < 16; ++c) {
        uint32_t o[16];
        if (n_tiles > 0) { tmem_ld_x16(tmem + lane_addr + O_COL + c * 16, o); tc_wait_ld(); }
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
      if (live && a.n_splits > 1 && vh == 0) {
        float* ml = a.part_ml + (((size_t)split * a.T + t) * a.Hl + h) * 2;
        ml[0] = m_nat; ml[1] = l;
      }
    }
  }
  if (*abortp && warp == 0) { const long long c0 = clock64(); while (clock64() - c0 < 400000) __nanosleep(1000); }
  // nobody leaves while the partner may still store into this CTA's shared memory or arrive on its barriers
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// out[h, t, :] = sum_s o_s * exp(m_s - M) / sum_s l_s * exp(m_s - M); partials are token-major, the output head-major.
__global__ void __launch_bounds__(128) mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out, int T, int Hl,
                                                        int n_splits) {
  // One block of 128 threads per (token, head), four output columns per thread.  The (m, l) pairs of all splits are read at once by
  // one warp (weights exp(m - M) and the denominator land in shared memory); the partial rows then come eight splits at a time,
  // every load issued before the first use.  (Reading m, branching, then loading the row made the merge a chain of one L2 round
  // trip per split: 21 us at 32 splits on a batch-1 step.)
  pdl_launch(); pdl_wait();
  __shared__ float wsh[64];
  __shared__ float Lsh;
  const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    float2 v[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int sidx = lane + 32 * j;
      v[j] = sidx < n_splits ? *(const float2*)(part_ml + (((size_t)sidx * T + t) * Hl + h) * 2) : make_float2(-INFINITY, 0.f);
    }
    const float M = warp_max(fmaxf(v[0].x, v[1].x));
    float l = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float w = (v[j].x != -INFINITY) ? __expf(v[j].x - M) : 0.f;
      wsh[lane + 32 * j] = w;
      l += v[j].y * w;
    }
    l = warp_sum(l);
    if (lane == 0) Lsh = l;
  }
  __syncthreads();
  const int d0 = threadIdx.x * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < n_splits; s0 += 8) {
    float4 pv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int sidx = min(s0 + j, n_splits - 1);
      pv[j] = *(const float4*)(part_o + (((size_t)sidx * T + t) * Hl + h) * DV + d0);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float w = (s0 + j < n_splits) ? wsh[s0 + j] : 0.f;
      if (w != 0.f) { acc.x += pv[j].x * w; acc.y += pv[j].y * w; acc.z += pv[j].z * w; acc.w += pv[j].w * w; }
    }
  }
  const float L = Lsh, inv = L > 0.f ? 1.f / L : 0.f;
  bf16 ob[4] = {__float2bfloat16(acc.x * inv), __float2bfloat16(acc.y * inv), __float2bfloat16(acc.z * inv), __float2bfloat16(acc.w * inv)};
  *(uint2*)(out + ((size_t)h * T + t) * DV + d0) = *(const uint2*)ob;
}

__global__ void mla_fill_ml_kernel(float* ml, long long n) {
  pdl_launch(); pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) ml[i] = (i & 1) ? 0.f : -INFINITY;
}

extern "C" int cuteafd_mla_attention(const void* q_lat, const void* q_rope, const void* kv_map, const int* page_table, const int* kv_len,
                                     const int* q_start, const int* q_len, void* out, float* part_o, float* part_ml, int T, int n_seq,
                                     int max_q_len, int Hl, int max_pages, int n_splits, float scale, int* status, cudaStream_t s) {
  CA_REQUIRE(Hl >= 1 && Hl <= 128 && 128 % Hl == 0, "mla_attention: local head count %d must divide 128", Hl);
  CA_REQUIRE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || (part_o && part_ml)), "mla_attention: 1..64 KV splits, and split-KV needs scratch");
  if (T <= 0 || n_seq <= 0) return CA_OK;
  MlaArgs a;
  a.q_lat = (const bf16*)q_lat; a.q_rope = (const bf16*)q_rope; a.kv_map = (const CUtensorMap*)kv_map; a.page_table = page_table;
  a.kv_len = kv_len; a.q_start = q_start; a.q_len = q_len; a.out = (bf16*)out; a.part_o = part_o; a.part_ml = part_ml; a.status = status;
  a.Hl = Hl; a.max_pages = max_pages; a.n_splits = n_splits; a.T = T; a.scale = scale;
  const int tpt = 128 / Hl;
  a.max_q_tiles = (max_q_len + tpt - 1) / tpt;
  static bool attr_set[64] = {false};
  int dev = 0; cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(mla_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MLA_SMEM);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(mla_attn)");
    attr_set[dev & 63] = true;
  }
  if (n_splits > 1) {
    const long long n = (long long)n_splits * T * Hl * 2;
    CA_LAUNCH_PDL(mla_fill_ml_kernel, (int)((n + 255) / 256), 256, 0, s, part_ml, n);
  }
  dim3 grid(n_splits, 2, n_seq * a.max_q_tiles);
  // CUTEAFD_MLA_PAIR=1 pairs the two V-half CTAs in a cluster that splits the score chunks and exchanges partial scores;
  // measured slower than the independent CTAs (10.7 against 10.3 ms per 7-layer step at batch 64 @ 8k: the exchange costs
  // more than the 16-20 saved score instructions per tile), so it is off by default.
  static int pair = -1;
  if (pair < 0) { const char* e = getenv("CUTEAFD_MLA_PAIR"); pair = e ? atoi(e) : 0; }
  if (pair) {
    static bool pair_attr[64] = {false};
    if (!pair_attr[dev & 63]) {
      cudaError_t e = cudaFuncSetAttribute(mla_attn_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MLA_PAIR_SMEM);
      if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(mla_attn_pair)");
      pair_attr[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = MLA_PAIR_SMEM; cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = 2; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = ca_pdl_enabled(CA_PDL_CLASS) ? 2 : 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, mla_attn_pair_kernel, a);
    if (le != cudaSuccess) return ca_cuda(le, "mla_attn_pair launch");
  } else {
    CA_LAUNCH_PDL(mla_attn_kernel, grid, 192, MLA_SMEM, s, a);
  }
  CA_CHECK_LAUNCH("mla_attention");
  if (n_splits > 1) {
    CA_LAUNCH_PDL(mla_merge_kernel, dim3(T, Hl), 128, 0, s, part_o, part_ml, (bf16*)out, T, Hl, n_splits);
    CA_CHECK_LAUNCH("mla_merge");
  }
  return CA_OK;
}

// Descriptor of one layer's latent cache [slots, 576] bf16: box {64 elements, 64 slots} (one page).
extern "C" int cuteafd_tmap_encode_latent(void* out128, const void* base, uint64_t n_slots) {
  CUtensorMap m;
  int rc = ca_encode_tmap_3d(&m, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, DQK, n_slots, 1, DQK * 2, (uint64_t)DQK * 2 * n_slots, 64, MKEYS, 1,
                             CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  memcpy(out128, &m, sizeof(m));
  return CA_OK;
}

// ---------------------------------------------------------------- MLA glue
// kv_a [T, 576] -> cache row: RMSNorm(c_kv) * w over the first 512, interleaved RoPE over the last 64.
__global__ void mla_kv_prepare_kernel(const bf16* __restrict__ kv_a, const float* __restrict__ w, const int* __restrict__ positions,
                                      const int* __restrict__ slot_map, bf16* __restrict__ cache, int n_slots, float theta, float eps,
                                      int interleaved, int* status) {
  pdl_launch(); pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x, tid = threadIdx.x;       // 128 threads
  const int slot = slot_map[t];
  if (slot < 0 || slot >= n_slots) { if (tid == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, t); return; }
  const bf16* src = kv_a + (size_t)t * DQK;
  bf16* dst = cache + (size_t)slot * DQK;
  float v[4], ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = __bfloat162float(src[tid * 4 + j]); ss += v[j] * v[j]; }
  const float inv = rsqrtf(block_sum(ss, red) / 512.f + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j) dst[tid * 4 + j] = __float2bfloat16(v[j] * inv * w[tid * 4 + j]);
  if (tid < 32) {
    const int i0 = interleaved ? 2 * tid : tid, i1 = interleaved ? 2 * tid + 1 : tid + 32;
    const float x0 = __bfloat162float(src[512 + i0]), x1 = __bfloat162float(src[512 + i1]);
    const float ang = (float)positions[t] * powf(theta, -2.f * (float)tid / 64.f);
    const float sn = sinf(ang), cs = cosf(ang);
    dst[512 + i0] = __float2bfloat16(x0 * cs - x1 * sn);
    dst[512 + i1] = __float2bfloat16(x0 * sn + x1 * cs);
  }
}

extern "C" int cuteafd_mla_kv_prepare(const void* kv_a, const float* w, const int* positions, const int* slot_map, void* cache, int T,
                                      int n_slots, float theta, float eps, int interleaved, int* status, cudaStream_t s) {
  if (T <= 0) return CA_OK;
  CA_LAUNCH_PDL(mla_kv_prepare_kernel, T, 128, 0, s, (const bf16*)kv_a, w, positions, slot_map, (bf16*)cache, n_slots, theta, eps, interleaved, status);
  CA_CHECK_LAUNCH("mla_kv_prepare");
  return CA_OK;
}

// q [T, Hl * 192] -> q_nope head-major [Hl, T, 128] and q_rope [T, Hl, 64] (RoPE applied).  One warp per (t, h).
__global__ void mla_q_split_kernel(const bf16* __restrict__ q, const int* __restrict__ positions, bf16* __restrict__ q_nope,
                                   bf16* __restrict__ q_rope, int T, int Hl, float theta, int interleaved) {
  pdl_launch(); pdl_wait();
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * Hl) return;
  const int t = w / Hl, h = w % Hl;
  const bf16* src = q + ((size_t)t * Hl + h) * 192;
  bf16* dn = q_nope + ((size_t)h * T + t) * 128;
  *(uint2*)(dn + lane * 4) = *(const uint2*)(src + lane * 4);
  const int i0 = interleaved ? 2 * lane : lane, i1 = interleaved ? 2 * lane + 1 : lane + 32;
  const float x0 = __bfloat162float(src[128 + i0]), x1 = __bfloat162float(src[128 + i1]);
  const float ang = (float)positions[t] * powf(theta, -2.f * (float)lane / 64.f);
  const float sn = sinf(ang), cs = cosf(ang);
  bf16* dr = q_rope + ((size_t)t * Hl + h) * 64;
  dr[i0] = __float2bfloat16(x0 * cs - x1 * sn);
  dr[i1] = __float2bfloat16(x0 * sn + x1 * cs);
}

extern "C" int cuteafd_mla_q_split(const void* q, const int* positions, void* q_nope, void* q_rope, int T, int Hl, float theta,
                                   int interleaved, cudaStream_t s) {
  if (T <= 0) return CA_OK;
  const long long warps = (long long)T * Hl;
  CA_LAUNCH_PDL(mla_q_split_kernel, (int)((warps * 32 + 255) / 256), 256, 0, s, (const bf16*)q, positions, (bf16*)q_nope, (bf16*)q_rope, T, Hl, theta, interleaved);
  CA_CHECK_LAUNCH("mla_q_split");
  return CA_OK;
}

// head-major [Hl, T, D] -> token-major [T, Hl * D]
__global__ void head_to_token_major_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int T, int Hl, int D) {
  pdl_launch(); pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const uint4* src = (const uint4*)(in + ((size_t)h * T + t) * D);
  uint4* dst = (uint4*)(out + ((size_t)t * Hl + h) * D);
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
}

extern "C" int cuteafd_head_to_token_major(const void* in, void* out, int T, int Hl, int D, cudaStream_t s) {
  CA_REQUIRE(D % 8 == 0, "head_to_token_major: D must be a multiple of 8");
  if (T <= 0) return CA_OK;
  CA_LAUNCH_PDL(head_to_token_major_kernel, dim3(T, Hl), 32, 0, s, (const bf16*)in, (bf16*)out, T, Hl, D);
  CA_CHECK_LAUNCH("head_to_token_major");
  return CA_OK;
}

// The same transpose writing the token-major row ALSO as the FP8 operand of the output projection (E4M3 + one fp32 scale per
// 128 channels = one head's 128 values): one warp per (token, head), 4 elements per lane as in the stand-alone quantiser.
__global__ void head_to_token_major_fp8b_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, uint8_t* __restrict__ q, float* __restrict__ sa,
                                                int T, int Hl) {
  pdl_launch(); pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
  const uint2 raw = *(const uint2*)(in + ((size_t)h * T + t) * 128 + lane * 4);
  if (out) *(uint2*)(out + ((size_t)t * Hl + h) * 128 + lane * 4) = raw;
  const bf16* e = (const bf16*)&raw;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(e[j]);
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-4f) / 448.f;
  uint32_t pk = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) pk |= (uint32_t)float_to_e4m3(v[j] / scale) << (8 * j);
  *(uint32_t*)(q + ((size_t)t * Hl + h) * 128 + lane * 4) = pk;
  if (lane == 0) sa[(size_t)t * Hl + h] = scale;
}

extern "C" int cuteafd_head_to_token_major_fp8b(const void* in, void* out, void* q, float* sa, int T, int Hl, int D, cudaStream_t s) {
  CA_REQUIRE(in && q && sa && D == 128, "head_to_token_major_fp8b: heads of 128 values");
  if (T <= 0) return CA_OK;
  CA_LAUNCH_PDL(head_to_token_major_fp8b_kernel, dim3(T, Hl), 32, 0, s, (const bf16*)in, (bf16*)out, (uint8_t*)q, sa, T, Hl);
  CA_CHECK_LAUNCH("head_to_token_major_fp8b");
  return CA_OK;
}
