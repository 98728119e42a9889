// tcgen05 linear layer family for sm_100a:  Y[rows, N] = X[rows, K] * W[N, K]^T  (dense or grouped per expert).
//
// One persistent, warp-specialised kernel covers every GEMM-shaped op of the engine:
//   * operand kinds: BF16 (kind::f16), NVFP4 (kind::mxf4nvf4, E4M3 scale / 16, scale_vec::4X) and
//     MXFP4 (kind::mxf4, UE8M0 scale / 32, scale_vec::2X), fp32 accumulation in tensor memory;
//   * "swap-AB": the 128 weight rows of a tile are the MMA M dimension and the tokens are the MMA N
//     dimension (TN = 16..256), so decode batches of 1..64 rows still fill the tensor core and the kernel
//     streams each weight byte from HBM exactly once;
//   * grouped mode walks a device-side tile table {expert, first row, row count} built by the route
//     packer, so one fixed-size launch (CUDA-graph friendly) serves any routing;
//   * SWIGLU mode multiplies two weight tiles (gate, up) against the same activation tile into two
//     accumulators and writes silu(g) * u, which is FC1 of an expert without materialising g and u.
//   * split-K for skinny dense layers: partial tiles go to fp32 scratch, the last CTA to arrive (a
//     per-tile counter) sums them in split order, so results are deterministic.
//
// Pipeline per CTA (192 threads): warp 0 = TMA producer (+ activation scale staging), warp 1 = MMA issuer and
// tensor-memory owner, warps 2-5 = epilogue (tcgen05.ld -> registers -> global).  Shared-memory stages
// are handed over with mbarriers (full/empty); accumulators are double-buffered in tensor memory when they
// fit so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Replaces, in the reference, the AOT-exported expert/FP8/FFN programs whose sources are absent
// (native/shared/include/cuteafd_experts.h:13-44, cuteafd_fp8_moe.h:1-51) and the cuBLAS linears
// (native/shared/cuda/linear.cu:865-1350).
#define CA_PDL_CLASS 1
#include <stdlib.h>
#include "common.cuh"

// KIND_W4A8: MXFP4 weights (E2M1 + UE8M0 / 32, unpacked by TMA into 8-bit containers) x FP8 E4M3 activations with UE8M0 / 32
// scales, kind::mxf8f6f4 (K = 32 per instruction) - the reference's default expert arithmetic
// (python/tools/aot/export_b12x_v41_experts_aot.py:21-93).  3 is the separate FP8 128x128 block-scaled kernel's kind.
enum { KIND_BF16 = 0, KIND_NVFP4 = 1, KIND_MXFP4 = 2, KIND_W4A8 = 4 };
enum { EPI_BF16 = 0, EPI_BF16_RESIDUAL = 1, EPI_F32 = 3 };

struct TcArgs {
  const CUtensorMap* tmA;     // [G] weight descriptors (gate weights in SWIGLU mode)
  const CUtensorMap* tmA2;    // [G] up-weight descriptors (SWIGLU)
  const CUtensorMap* tmB;     // activation descriptor
  const uint8_t* const* sfa;  // [G] weight scales in the 128x4 atom layout
  const uint8_t* const* sfa2;
  const uint8_t* sfb;         // activation scales, row-major [rows, K / vec]
  const float* alpha;         // [G] output scale (weight global scale x activation global scale) or null
  const float* alpha2;
  const int4* tiles;          // grouped: {group, first row, rows, 0}; null = dense
  const int* n_tiles;         // grouped: number of entries in `tiles` (device)
  void* Y;
  const bf16* R;              // residual (EPI_BF16_RESIDUAL)
  float* splitk_ws;           // [splits, rows_pad, N] partials (dense split-K)
  int* splitk_cnt;            // [items * n_tiles * 4] arrival counters, zero on entry, left zero on exit
  int* status;
  uint8_t* q_out;             // optional FP4 copy of the output (same kind as the operands): codes [rows, N / 2] ...
  uint8_t* sf_out;            // ... and block scales [rows, ldsf_out], for the GEMM that consumes this one's output
  const float* inv_gs_out;    // NVFP4: 1 / activation global scale of that consumer
  int ldsf_out;
  // Fused hand-off to peer GPUs: the bf16 output tile is also stored straight into peers' memory over NVLink from
  // the epilogue (row r of this GEMM lands in row peer_row_map[r], or r), and once every CTA has finished, the last
  // one releases the peers' flags with the current step number - GEMM and transfer are one kernel, tile by tile.
  void* peer_y0; void* peer_y1;
  uint32_t* peer_flag0; uint32_t* peer_flag1;
  const int* peer_row_map;
  uint32_t* peer_ctl;         // [0] abort word, [1] step number
  uint32_t* peer_done;        // arrival counter: zero on entry, left zero
  int peer_ld, n_peer;
  long long* trace;           // optional per-unit time stamps [grid, trace_units, 8] (see cuteafd_tc_trace)
  int ldsfb, ldy, rows_total, N, K, epi, splits, trace_units;
  int w4_tx;                  // KIND_W4A8: bytes one weight tile adds to the stage barrier's transaction count
};

// Per-unit device trace: slot 0/1 producer first/last load issued, 2 MMA thread owns the accumulator, 4 last MMA
// issued, 5/6 epilogue (first epilogue warp) begin/end - SM cycle counter - 7 the global nanosecond timer at
// the producer's unit start, 3 the same timer at the epilogue's end.
#define TC_TRACE(slot, val)                                                                        \
  do {                                                                                              \
    if (a.trace && lane == 0 && (w - w_begin) < a.trace_units)                                      \
      a.trace[((size_t)blockIdx.x * a.trace_units + (w - w_begin)) * 8 + (slot)] = (long long)(val); \
  } while (0)

template <int KIND, int TN, bool SWIGLU>
struct TcCfg {
  static constexpr int NA = SWIGLU ? 2 : 1;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = TN * 128;
  static constexpr int NBLK = TN > 128 ? 2 : 1;                      // 128-token scale blocks
  static constexpr int SF_CHUNKS = KIND == KIND_NVFP4 ? 4 : (KIND == KIND_MXFP4 ? 2 : (KIND == KIND_W4A8 ? 1 : 0));  // 512 B chunks / stage
  static constexpr int SFA_BYTES = SF_CHUNKS * 512;
  static constexpr int SFB_BYTES = SF_CHUNKS * 512 * NBLK;
  static constexpr int STAGE_BYTES = NA * A_BYTES + B_BYTES + NA * SFA_BYTES + SFB_BYTES;
  // Decode-sized token tiles run two CTAs per SM (half the shared memory and half the tensor memory each): the
  // per-stage chain of one CTA (barrier wait -> scale copies -> MMAs -> commit) is latency-bound, two
  // independent chains per SM keep the memory system busy.
  static constexpr int OCC = TN <= 32 ? 2 : 1;
  static constexpr int NSTAGE_RAW = ((OCC == 2 ? 104 : 200) * 1024) / STAGE_BYTES;
  static constexpr int NSTAGE = NSTAGE_RAW > 8 ? 8 : NSTAGE_RAW;
  static constexpr int ACC_COLS = NA * TN;
  // two accumulators let the next unit's MMAs run under this unit's epilogue; bf16 operands have no scale columns, so a
  // 256-token tile can still double-buffer (2 x 256 = all 512 columns)
  static constexpr int NACC = (2 * ACC_COLS <= (KIND == KIND_BF16 ? 512 : 384)) ? 2 : 1;
  static constexpr int TMEM_COLS = OCC == 2 ? 256 : 512;
  static constexpr int SFA_COL = TMEM_COLS - 64, SFA2_COL = TMEM_COLS - 48, SFB_COL = TMEM_COLS - 32;   // tensor-memory columns of the scales
  static constexpr int K_ELEMS = KIND == KIND_BF16 ? 64 : (KIND == KIND_W4A8 ? 128 : 256);   // K elements per stage (128 bytes of shared memory per row)
  // Staging for the transposed epilogue store of 64+-token tiles: two buffers of [16 tokens][128 features] fp32.  In the
  // swap-AB tile a lane owns ONE output feature, so direct stores are 2-byte elements, 64 contiguous bytes per warp
  // instruction; through the staging buffer the four epilogue warps write whole 256-byte rows with 16-byte stores.
  static constexpr int STG_BYTES = TN >= 64 ? 2 * 16 * 128 * 4 : 0;
  static constexpr int SMEM_BYTES = NSTAGE * STAGE_BYTES + STG_BYTES + 1024;
  static_assert(NSTAGE >= 2, "tile too large for shared memory");
  static_assert(KIND == KIND_BF16 ? ACC_COLS * NACC <= TMEM_COLS : ACC_COLS * NACC <= SFA_COL, "accumulators overlap the scale columns");
};

__device__ __forceinline__ uint32_t make_idesc(int kind, int n, uint32_t sf_id) {
  uint32_t d = 0;
  if (kind == KIND_BF16) {
    d |= 1u << 4;            // fp32 accumulator
    d |= 1u << 7;            // A = bf16
    d |= 1u << 10;           // B = bf16
  } else if (kind == KIND_W4A8) {
    d |= sf_id << 4;         // B scale-factor id: which byte of the 32-bit scale column this K = 32 step uses
    d |= 5u << 7;            // A = E2M1 (kind::mxf8f6f4 numbering: E4M3 0, E5M2 1, E2M3 3, E3M2 4, E2M1 5)
    d |= 0u << 10;           // B = E4M3
    d |= 1u << 23;           // UE8M0 scales
    d |= sf_id << 29;        // A scale-factor id
  } else {
    d |= sf_id << 4;         // B scale-factor id
    d |= 1u << 7;            // A = E2M1
    d |= 1u << 10;           // B = E2M1
    if (kind == KIND_MXFP4) d |= 1u << 23;   // UE8M0 scales (0 = UE4M3)
    d |= sf_id << 29;        // A scale-factor id
  }
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(128 >> 4) << 24;
  return d;
}

// Tail of a kernel whose epilogue stored to peers: the 128 epilogue threads fence their stores, one of them counts the
// CTA in, and the CTA that arrives last publishes the flags (system-scope release) and re-arms the counter.
__device__ __forceinline__ void peer_publish(const TcArgs& a, int warp, int lane) {
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (warp == 2 && lane == 0) {
    __threadfence();                            // GPU scope: orders the stores the barrier put before this thread ahead of the count
    const uint32_t prev = atomicAdd(a.peer_done, 1u);
    if (prev == gridDim.x - 1) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");        // one system-scope fence, cumulative over all CTAs' stores
      const uint32_t step = a.peer_ctl[1];
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.peer_flag0), "r"(step) : "memory");
      if (a.n_peer > 1) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.peer_flag1), "r"(step) : "memory");
      *a.peer_done = 0;
    }
  }
}
__device__ __forceinline__ void peer_store(const TcArgs& a, int row, int n, bf16 v) {
  const size_t prow = a.peer_row_map ? (size_t)a.peer_row_map[row] : (size_t)row;
  ((bf16*)a.peer_y0)[prow * a.peer_ld + n] = v;
  if (a.n_peer > 1) ((bf16*)a.peer_y1)[prow * a.peer_ld + n] = v;
}

// PEER instantiations carry the peer-store epilogue; the others are the plain local kernels (the extra code costs
// ~1.5 us per launch even when switched off at run time, so it is compiled in only where it is used).
template <int KIND, int TN, bool SWIGLU, bool PEER, bool QOUT>
__global__ void __launch_bounds__(192, TcCfg<KIND, TN, SWIGLU>::OCC) tc_linear_kernel(const __grid_constant__ TcArgs a) {
  using C = TcCfg<KIND, TN, SWIGLU>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[C::NSTAGE], empty_bar[C::NSTAGE], accf_bar[2], acce_bar[2], stg_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::NSTAGE; ++s) { mbar_init(&full_bar[s], 33); mbar_init(&empty_bar[s], 1); }   // 1 expect_tx + 32 lanes
    for (int i = 0; i < 2; ++i) { mbar_init(&accf_bar[i], 1); mbar_init(&acce_bar[i], 128); }
    mbar_init(&stg_bar, 128);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  // The next kernel of the stream may start its prologue now.  Grouped launches read the tile table an earlier
  // kernel wrote, so every thread waits for the previous kernel here; a dense launch lets its producer warp
  // stream the first weight stages (static data) before it waits.
  pdl_launch();
  const bool dense = a.tiles == nullptr;
  if (!(dense && warp == 0)) pdl_wait();
  const int n_items = dense ? (a.rows_total + TN - 1) / TN : *a.n_tiles;
  const int n_nt = (a.N + 127) / 128;
  const int nkb_all = (a.K + C::K_ELEMS - 1) / C::K_ELEMS;
  const int splits = a.splits > 1 ? a.splits : 1;
  const int total = n_items * n_nt * splits;
  // Each CTA takes one contiguous run of work units: consecutive units share the expert (TMA descriptor,
  // activation rows, scale rows) and walk the weight matrix in address order.
  const int chunk = (total + (int)gridDim.x - 1) / (int)gridDim.x;
  const int w_begin = min(total, (int)blockIdx.x * chunk), w_end = min(total, w_begin + chunk);
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    uint32_t it = 0, npre = 0;
    // decode-sized steps read every weight byte once: stream it through L2 without displacing the step's small data; larger steps
    // re-read a weight tile for every token tile and want it kept
    const uint64_t wpol = (dense ? a.rows_total <= TN : a.rows_total <= 1024) ? l2_policy_stream() : l2_policy_normal();
    // weight-side loads of one stage (static data: legal before the previous kernel has finished)
    auto load_weights = [&](int s, int g, int nt, int kb) {
      uint8_t* st = smem + s * C::STAGE_BYTES;
      uint8_t* sA = st, *sSFA = st + C::NA * C::A_BYTES + C::B_BYTES;
      mbar_expect_tx(&full_bar[s], C::NA * (KIND == KIND_W4A8 ? a.w4_tx : C::A_BYTES) + C::B_BYTES + C::NA * C::SFA_BYTES);
      const int kx = kb * (KIND == KIND_BF16 ? 64 : 128);      // elements of the descriptor's type
      tma_load_3d_hint(sA, a.tmA + g, &full_bar[s], kx, nt * 128, 0, wpol);
      if (SWIGLU) tma_load_3d_hint(sA + C::A_BYTES, a.tmA2 + g, &full_bar[s], kx, nt * 128, 0, wpol);
      if (KIND != KIND_BF16) {
        const size_t off = ((size_t)nt * nkb_all + (size_t)kb) * C::SF_CHUNKS * 512;   // scales are padded to whole stages
        bulk_load_1d_hint(sSFA, a.sfa[g] + off, C::SFA_BYTES, &full_bar[s], wpol);
        if (SWIGLU) bulk_load_1d_hint(sSFA + C::SFA_BYTES, a.sfa2[g] + off, C::SFA_BYTES, &full_bar[s], wpol);
      }
    };
    if (dense) {
      if (w_begin < w_end) {
        const int sp = w_begin % splits, nt = (w_begin / splits) % n_nt;
        const int kb0 = (int)(((long long)nkb_all * sp) / splits), kb1 = (int)(((long long)nkb_all * (sp + 1)) / splits);
        npre = (uint32_t)min(C::NSTAGE, kb1 - kb0);
        if (lane == 0)
          for (uint32_t i = 0; i < npre; ++i) load_weights((int)i, 0, nt, kb0 + (int)i);
      }
      pdl_wait();
    }
    for (int w = w_begin; w < w_end && !*abortp; ++w) {
      const int sp = w % splits, tile = w / splits, item = tile / n_nt, nt = tile % n_nt;
      int g = 0, row0 = item * TN, nrows = min(TN, a.rows_total - row0);
      if (a.tiles) { int4 t = a.tiles[item]; g = t.x; row0 = t.y; nrows = t.z; }
      const int kb0 = (int)(((long long)nkb_all * sp) / splits), kb1 = (int)(((long long)nkb_all * (sp + 1)) / splits);
      TC_TRACE(0, clock64()); TC_TRACE(7, globaltimer_ns());
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % C::NSTAGE;
        if (!mbar_wait_bounded(&empty_bar[s], ((it / C::NSTAGE) & 1) ^ 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, w); break; }
        uint8_t* st = smem + s * C::STAGE_BYTES;
        uint8_t* sB = st + C::NA * C::A_BYTES, *sSFB = sB + C::B_BYTES + C::NA * C::SFA_BYTES;
        if (lane == 0) {
          if (it >= npre) load_weights(s, g, nt, kb);          // the first `npre` stages already hold their weights
          tma_load_3d(sB, a.tmB, &full_bar[s], kb * (KIND == KIND_BF16 ? 64 : 128), row0, 0);
        }
        if (KIND != KIND_BF16) {
          // Activation scales: each token owns SF_CHUNKS*4 consecutive bytes per stage in the row-major array;
          // cp.async moves them 4 bytes at a time straight into the 32x16-byte chunk layout tcgen05.cp expects
          // (zero-filling rows past the tile), so the producer never waits on a global load.
          constexpr int SFB_PER_STAGE = C::SF_CHUNKS * 4;
          for (int c = lane; c < TN; c += 32) {
            const int row = row0 + c;
            const bool live = c < nrows && row < a.rows_total;
            const uint8_t* src = live ? a.sfb + (size_t)row * a.ldsfb + (size_t)kb * SFB_PER_STAGE : a.sfb;
            const uint32_t dst = smem_u32(sSFB + (c >> 7) * (C::SF_CHUNKS * 512) + (c & 31) * 16 + ((c & 127) >> 5) * 4);
            const uint32_t nbytes = live ? 4u : 0u;
#pragma unroll
            for (int q = 0; q < C::SF_CHUNKS; ++q)
              asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + q * 512), "l"(src + q * 4), "r"(nbytes) : "memory");
          }
          // counts as this lane's arrival once its copies have landed
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full_bar[s])) : "memory");
        } else {
          mbar_arrive(&full_bar[s]);
        }
      }
      TC_TRACE(1, clock64());
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // One elected thread waits and issues (the other lanes park at the warp barrier below): no per-stage
    // divergence or reconvergence on the chain that bounds a decode-sized tile.
    if (lane == 0) {
      uint32_t it = 0, tc = 0;
      const uint32_t smem_base = smem_u32(smem);
      for (int w = w_begin; w < w_end && !*abortp; ++w, ++tc) {
        const int sp = w % splits;
        const int kb0 = (int)(((long long)nkb_all * sp) / splits), kb1 = (int)(((long long)nkb_all * (sp + 1)) / splits);
        const int acc = tc % C::NACC;
        if (!mbar_wait_bounded(&acce_bar[acc], ((tc / C::NACC) & 1) ^ 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, w); break; }
        tc_fence_after();
        TC_TRACE(2, clock64());
        const uint32_t d0 = tmem + acc * C::ACC_COLS;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % C::NSTAGE;
          if (!mbar_wait_bounded(&full_bar[s], (it / C::NSTAGE) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, w); ok = false; break; }
          tc_fence_after();
          if (KIND != KIND_BF16) fence_proxy_async_smem();   // scale bytes arrived through the generic proxy (cp.async)
          const uint32_t st = smem_base + s * C::STAGE_BYTES;
          const uint32_t sA = st, sB = st + C::NA * C::A_BYTES, sSFA = sB + C::B_BYTES, sSFB = sSFA + C::NA * C::SFA_BYTES;
          if (KIND != KIND_BF16) {
#pragma unroll
            for (int q = 0; q < C::SF_CHUNKS; ++q) {
              tc_cp_sf(tmem + C::SFA_COL + 4 * q, umma_desc_sf(sSFA + q * 512));
              if (SWIGLU) tc_cp_sf(tmem + C::SFA2_COL + 4 * q, umma_desc_sf(sSFA + C::SFA_BYTES + q * 512));
#pragma unroll
              for (int b = 0; b < C::NBLK; ++b)
                tc_cp_sf(tmem + C::SFB_COL + (4 * C::NBLK) * q + 4 * b, umma_desc_sf(sSFB + b * (C::SF_CHUNKS * 512) + q * 512));
            }
          }
          const uint64_t adesc = umma_desc_sw128(sA), a2desc = umma_desc_sw128(sA + C::A_BYTES), bdesc = umma_desc_sw128(sB);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
            if (KIND == KIND_BF16) {
              const uint32_t id = make_idesc(KIND_BF16, TN, 0);
              tc_mma_f16(d0, adesc + 2 * k, bdesc + 2 * k, id, accum);
              if (SWIGLU) tc_mma_f16(d0 + TN, a2desc + 2 * k, bdesc + 2 * k, id, accum);
            } else if (KIND == KIND_NVFP4) {
              const uint32_t id = make_idesc(KIND_NVFP4, TN, 0);
              tc_mma_nvf4(d0, adesc + 2 * k, bdesc + 2 * k, id, accum, tmem + C::SFA_COL + 4 * k, tmem + C::SFB_COL + 4 * C::NBLK * k);
              if (SWIGLU) tc_mma_nvf4(d0 + TN, a2desc + 2 * k, bdesc + 2 * k, id, accum, tmem + C::SFA2_COL + 4 * k, tmem + C::SFB_COL + 4 * C::NBLK * k);
            } else if (KIND == KIND_W4A8) {
              const uint32_t id = make_idesc(KIND_W4A8, TN, k);       // one scale column per stage, byte k of it per K = 32 step
              tc_mma_mxf8f6f4(d0, adesc + 2 * k, bdesc + 2 * k, id, accum, tmem + C::SFA_COL, tmem + C::SFB_COL);
              if (SWIGLU) tc_mma_mxf8f6f4(d0 + TN, a2desc + 2 * k, bdesc + 2 * k, id, accum, tmem + C::SFA2_COL, tmem + C::SFB_COL);
            } else {
              const uint32_t id = make_idesc(KIND_MXFP4, TN, (k & 1) * 2);
              const int q = k >> 1;
              tc_mma_mxf4(d0, adesc + 2 * k, bdesc + 2 * k, id, accum, tmem + C::SFA_COL + 4 * q, tmem + C::SFB_COL + 4 * C::NBLK * q);
              if (SWIGLU) tc_mma_mxf4(d0 + TN, a2desc + 2 * k, bdesc + 2 * k, id, accum, tmem + C::SFA2_COL + 4 * q, tmem + C::SFB_COL + 4 * C::NBLK * q);
            }
          }
          tc_commit(&empty_bar[s]);
        }
        if (!ok) break;
        tc_commit(&accf_bar[acc]);
        TC_TRACE(4, clock64());
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q4 = warp & 3;                 // tensor-memory lane quarter this warp may read
    const int et = q4 * 32 + lane;           // 0..127: weight row inside the tile
    uint32_t tc = 0, stg_uses = 0;
    // staged (transposed) store: plain bf16 output of a 64+-token tile, 16-byte aligned rows
    const bool stage_ok = C::STG_BYTES > 0 && splits == 1 && a.epi != EPI_F32 && a.Y != nullptr && !(QOUT && a.q_out) && !(PEER && a.n_peer) &&
                          a.ldy % 8 == 0 && a.N % 8 == 0 && ((uintptr_t)a.Y & 15) == 0 && (a.epi != EPI_BF16_RESIDUAL || ((uintptr_t)a.R & 15) == 0);
    float* stg = (float*)(smem + C::NSTAGE * C::STAGE_BYTES);
    bool stg_fail = false;
    for (int w = w_begin; w < w_end && !*abortp; ++w, ++tc) {
      const int sp = w % splits, tile = w / splits, item = tile / n_nt, nt = tile % n_nt;
      int g = 0, row0 = item * TN, nrows = min(TN, a.rows_total - row0);
      if (a.tiles) { int4 t = a.tiles[item]; g = t.x; row0 = t.y; nrows = t.z; }
      nrows = min(nrows, a.rows_total - row0);
      const int acc = tc % C::NACC;
      if (!mbar_wait_bounded(&accf_bar[acc], (tc / C::NACC) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, w); break; }
      tc_fence_after();
      if (warp == 2) TC_TRACE(5, clock64());
      const int n = nt * 128 + et;
      const bool n_ok = n < a.N;
      const float al = a.alpha ? a.alpha[g] : 1.f;
      const float al2 = (SWIGLU && a.alpha2) ? a.alpha2[g] : al;
      const uint32_t tbase = tmem + ((uint32_t)(q4 * 32) << 16) + acc * C::ACC_COLS;
      float* ws = (splits > 1) ? a.splitk_ws + ((size_t)sp * a.rows_total) * a.N : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 16) {
        uint32_t r[16], r2[16];
        tmem_ld_x16(tbase + c0, r);
        if (SWIGLU) tmem_ld_x16(tbase + TN + c0, r2);
        tc_wait_ld();
        if (QOUT && KIND == KIND_W4A8 && a.q_out) {
          // FP8 output for the next GEMM (E4M3 + one UE8M0 scale per 32 features): this lane holds output feature n of 16
          // tokens and the 32 lanes of the warp are exactly one scale block, so amax is a warp reduction.  Same arithmetic
          // as the stand-alone quantiser on the bf16-rounded value (amax floor 1e-4, scale 2^ceil(log2(amax / 448))).
          if (c0 < nrows) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int c = c0 + j;
              if (c < nrows) {                       // warp-uniform
                float v = __uint_as_float(r[j]) * al;
                if (SWIGLU) {
                  const float u = __uint_as_float(r2[j]) * al2;
                  v = v / (1.f + __expf(-v)) * u;
                }
                const bf16 vb = __float2bfloat16(n_ok ? v : 0.f);
                v = __bfloat162float(vb);
                const float am = fmaxf(warp_max(fabsf(v)), 1e-4f);
                const uint8_t sb = ue8m0_ceil(am / 448.f);
                const uint8_t qb = float_to_e4m3(v / ue8m0_to_float(sb));
                const size_t row = (size_t)(row0 + c);
                if (n_ok) a.q_out[row * a.N + n] = qb;
                if (n_ok && lane == 0) a.sf_out[row * a.ldsf_out + n / 32] = sb;
                if (a.Y && n_ok) ((bf16*)a.Y)[row * a.ldy + n] = vb;
              }
            }
          }
        } else if (QOUT && KIND != KIND_BF16 && a.q_out) {
          // FP4 output for the next GEMM: this lane holds output feature n of 16 tokens; a quantisation block is 16
          // (NVFP4) or 32 (MXFP4) consecutive features = adjacent lanes, so amax and the nibble packing are shuffles.
          // Same arithmetic as the stand-alone quantiser on the bf16-rounded value.
          if (c0 < nrows) {
            const float inv_gs = (KIND == KIND_NVFP4 && a.inv_gs_out) ? *a.inv_gs_out : 1.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int c = c0 + j;
              if (c < nrows) {                       // warp-uniform
                float v = __uint_as_float(r[j]) * al;
                if (SWIGLU) {
                  const float u = __uint_as_float(r2[j]) * al2;
                  v = v / (1.f + __expf(-v)) * u;
                }
                const bf16 vb = __float2bfloat16(n_ok ? v : 0.f);
                v = __bfloat162float(vb);
                float am = fabsf(v);
                am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1)); am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
                am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4)); am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 8));
                float eff; uint8_t sb;
                if (KIND == KIND_MXFP4) {
                  am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 16));
                  int e = am > 0.f ? (int)((__float_as_uint(am) >> 23) & 0xFF) - 2 : 0;
                  e = max(e, 0); e = min(e, 254); sb = (uint8_t)e; eff = ue8m0_to_float(sb);
                } else {
                  sb = float_to_e4m3(fminf(am * inv_gs / 6.f, 448.f)); eff = e4m3_to_float(sb) / inv_gs;
                }
                uint32_t wv = float_to_e2m1(v * (eff > 0.f ? 1.f / eff : 0.f)) << (4 * (lane & 7));
                wv |= __shfl_xor_sync(0xffffffffu, wv, 1); wv |= __shfl_xor_sync(0xffffffffu, wv, 2); wv |= __shfl_xor_sync(0xffffffffu, wv, 4);
                const size_t row = (size_t)(row0 + c);
                if (n_ok && (lane & 7) == 0) *(uint32_t*)(a.q_out + row * (a.N / 2) + n / 2) = wv;
                if (n_ok && (lane & (KIND == KIND_MXFP4 ? 31 : 15)) == 0) a.sf_out[row * a.ldsf_out + n / (KIND == KIND_MXFP4 ? 32 : 16)] = sb;
                if (a.Y && n_ok) ((bf16*)a.Y)[row * a.ldy + n] = vb;
              }
            }
          }
        } else if (stage_ok) {
          if (c0 < nrows) {                            // the same for all four epilogue warps: they meet at the barrier below
            float* buf = stg + ((c0 >> 4) & 1) * (16 * 128);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float v = __uint_as_float(r[j]) * al;
              if (SWIGLU) {
                const float u = __uint_as_float(r2[j]) * al2;
                v = v / (1.f + __expf(-v)) * u;
              }
              buf[j * 128 + et] = v;
            }
            mbar_arrive(&stg_bar);
            if (!mbar_wait_bounded(&stg_bar, stg_uses & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, 0x7000 + w); stg_fail = true; break; }
            ++stg_uses;
            // 16 rows x 16 groups of 8 features; thread -> (row, group), two per thread.  A buffer is rewritten two chunks
            // later, after every warp has passed the NEXT chunk's barrier, i.e. finished these reads.
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int idx = (warp - 2) * 32 + lane + h * 128, row = idx >> 4, grp = idx & 15;
              const int c = c0 + row, nn = nt * 128 + grp * 8;
              if (c < nrows && nn < a.N) {
                const float4 f0 = *(const float4*)(buf + row * 128 + grp * 8), f1 = *(const float4*)(buf + row * 128 + grp * 8 + 4);
                float f[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
                const size_t o = (size_t)(row0 + c) * a.ldy + nn;
                if (a.epi == EPI_BF16_RESIDUAL) {
                  const uint4 rv = *(const uint4*)(a.R + o);
                  const bf16* rb = (const bf16*)&rv;
#pragma unroll
                  for (int q = 0; q < 8; ++q) f[q] += __bfloat162float(rb[q]);
                }
                uint32_t wv[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) { bf162 hh = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]); wv[q] = *(uint32_t*)&hh; }
                *(uint4*)((bf16*)a.Y + o) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
              }
            }
          }
        } else if (c0 < nrows && n_ok) {
          float res[16];        // residual rows ahead of the stores (R may alias Y: loads after a store would serialise)
#pragma unroll
          for (int j = 0; j < 16; ++j)
            res[j] = (a.epi == EPI_BF16_RESIDUAL && splits <= 1 && c0 + j < nrows) ? __bfloat162float(a.R[(size_t)(row0 + c0 + j) * a.ldy + n]) : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int c = c0 + j;
            if (c < nrows) {
              float v = __uint_as_float(r[j]) * al;
              if (SWIGLU) {
                const float u = __uint_as_float(r2[j]) * al2;
                v = v / (1.f + __expf(-v)) * u;
              }
              const size_t o = (size_t)(row0 + c) * a.ldy + n;
              if (splits > 1) ws[(size_t)(row0 + c) * a.N + n] = v;
              else if (a.epi == EPI_F32) ((float*)a.Y)[o] = v;
              else {
                v += res[j];
                const bf16 vb = __float2bfloat16(v);
                if (a.Y) ((bf16*)a.Y)[o] = vb;
                if (PEER && a.n_peer) peer_store(a, row0 + c, n, vb);
              }
            }
          }
        }
      }
      if (stg_fail) break;
      tc_fence_before();
      mbar_arrive(&acce_bar[acc]);
      if (warp == 2) { TC_TRACE(6, clock64()); TC_TRACE(3, globaltimer_ns()); }
      if (splits > 1) {
        // Deterministic split-K fix-up, warp by warp (no cross-warp barrier, so an aborting warp can never
        // strand another): each warp owns 32 weight rows of the tile and a counter; the last split to
        // arrive sums all partials in split order.
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = (atomicAdd(&a.splitk_cnt[tile * 4 + q4], 1) == splits - 1);
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          if (n_ok) {
            // loads are issued in batches (4 rows x up to 8 splits in flight) and summed in split order
            for (int c = 0; c < nrows; c += 4) {
              float v[4] = {0.f, 0.f, 0.f, 0.f};
              for (int p0 = 0; p0 < splits; p0 += 8) {
                float t[4][8];
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                  for (int p = 0; p < 8; ++p)
                    t[j][p] = (c + j < nrows && p0 + p < splits)
                                  ? __ldcg(a.splitk_ws + ((size_t)(p0 + p) * a.rows_total + row0 + c + j) * a.N + n) : 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                  for (int p = 0; p < 8; ++p) v[j] += t[j][p];
              }
              float res4[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                res4[j] = (a.epi == EPI_BF16_RESIDUAL && c + j < nrows) ? __bfloat162float(a.R[(size_t)(row0 + c + j) * a.ldy + n]) : 0.f;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (c + j >= nrows) break;
                const size_t o = (size_t)(row0 + c + j) * a.ldy + n;
                float r = v[j];
                if (a.epi == EPI_F32) ((float*)a.Y)[o] = r;
                else {
                  r += res4[j];
                  const bf16 rb = __float2bfloat16(r);
                  if (a.Y) ((bf16*)a.Y)[o] = rb;
                  if (PEER && a.n_peer) peer_store(a, row0 + c + j, n, rb);
                }
              }
            }
          }
          __syncwarp();
          if (lane == 0) a.splitk_cnt[tile * 4 + q4] = 0;
        }
      }
    }
    if (PEER && a.n_peer) peer_publish(a, warp, lane);
  }

  // ------------------------------------------------------------------ teardown
  if (*abortp && warp == 0) {
    // give copies already in flight time to land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <int KIND, int TN, bool SWIGLU, bool PEER, bool QOUT>
static int launch_p(const TcArgs& a, int grid, cudaStream_t stream) {
  using C = TcCfg<KIND, TN, SWIGLU>;
  auto kern = tc_linear_kernel<KIND, TN, SWIGLU, PEER, QOUT>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(tc_linear)");
    attr_set[dev & 63] = true;
  }
  CA_LAUNCH_PDL(kern, grid, 192, C::SMEM_BYTES, stream, a);
  return CA_OK;
}

template <int KIND, int TN, bool SWIGLU>
static int launch(const TcArgs& a, int grid, cudaStream_t stream) {
  if constexpr (!SWIGLU) { if (a.n_peer) return launch_p<KIND, TN, false, true, false>(a, grid, stream); }
  if constexpr (SWIGLU && KIND != KIND_BF16) { if (a.q_out) return launch_p<KIND, TN, true, false, true>(a, grid, stream); }
  return launch_p<KIND, TN, SWIGLU, false, false>(a, grid, stream);
}

template <int KIND, bool SWIGLU>
static int launch_tn(int tn, const TcArgs& a, int grid, cudaStream_t stream) {
  switch (tn) {
    case 16: return launch<KIND, 16, SWIGLU>(a, grid, stream);
    case 32: return launch<KIND, 32, SWIGLU>(a, grid, stream);
    case 64: return launch<KIND, 64, SWIGLU>(a, grid, stream);
    case 128: return launch<KIND, 128, SWIGLU>(a, grid, stream);
    case 256: if constexpr (!SWIGLU) return launch<KIND, 256, false>(a, grid, stream);
    default: return ca_fail(CA_ERR_ARG, "tc_linear: unsupported token tile %d (swiglu=%d)", tn, (int)SWIGLU);
  }
}

// ------------------------------------------------------------------------------------------------------------
// Split-K across a thread-block cluster for skinny dense layers (decode-time projections whose tile count is far
// below the SM count).  A cluster of S CTAs shares one 128 x TN output tile; CTA r streams the r-th slice of K into
// its own tensor-memory accumulator, then ranks 1..S-1 store their fp32 partial tile into rank 0's shared memory
// over the cluster network (st.shared::cluster), one cluster barrier later rank 0 adds the partials in rank order
// (deterministic) and runs the epilogue.  Compared with the global-memory fix-up above this removes the fences, the
// arrival counter and the reload from L2 - about 5 us per launch on B200.  Every CTA owns exactly one work unit.
template <int KIND, int TN>
struct ClCfg {
  using B = TcCfg<KIND, TN, false>;
  static constexpr int MAX_S = TN == 16 ? 8 : 4;
  static constexpr int BUDGET = 200 * 1024;                                  // ring + staging
  static constexpr int MAX_RING = 8;
  static constexpr int TMEM_COLS = 128;
  static constexpr int SFA_COL = 64, SFB_COL = 96;
  static constexpr int SMEM_BYTES = BUDGET + 1024;
  // Pipeline stages left beside the staging area of an S-way split (S partial tiles of 128 x TN fp32: ranks 1..S-1, then rank 0's own).
  __host__ __device__ static constexpr int ring(int S) {
    return (BUDGET - S * 128 * TN * 4) / B::STAGE_BYTES > MAX_RING ? MAX_RING : (BUDGET - S * 128 * TN * 4) / B::STAGE_BYTES;
  }
  static_assert(TN <= 32, "cluster split-K is for decode-sized token tiles");
};

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// Device trace of the cluster kernel (cuteafd_tc_trace(buf, -N): launches with this N record, per CTA, eight global-timer stamps:
// 0 entry, 1 rank 0: accumulator read back after the barrier, 2 producer released by the previous kernel, 3 first stage landed, 4 last MMA committed,
// 5 accumulator complete, 6 cluster barrier passed, 7 epilogue done).
#define CL_TRACE(slot) do { if (a.trace && a.trace_units == -a.N) a.trace[(size_t)blockIdx.x * 8 + (slot)] = (long long)globaltimer_ns(); } while (0)

template <int KIND, int TN, bool PEER>
__global__ void __launch_bounds__(192, 1) tc_linear_cluster_kernel(const __grid_constant__ TcArgs a) {
  using C = TcCfg<KIND, TN, false>;
  using L = ClCfg<KIND, TN>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[L::MAX_RING], empty_bar[L::MAX_RING], accf_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int S = a.splits;
  float* staging = (float*)(smem + L::ring(S) * C::STAGE_BYTES);         // [S-1][TN][128] fp32, rank 0's copy is the one used
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    CL_TRACE(0);
    for (int s = 0; s < L::MAX_RING; ++s) { mbar_init(&full_bar[s], 33); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accf_bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_slot, L::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  pdl_launch();

  const int sp = (int)cluster_ctarank();
  const int tile = (int)blockIdx.x / S;
  const int n_nt = (a.N + 127) / 128;
  const int item = tile / n_nt, nt = tile % n_nt;
  const int row0 = item * TN, nrows = min(TN, a.rows_total - row0);
  const int nkb_all = (a.K + C::K_ELEMS - 1) / C::K_ELEMS;
  const int kb0 = (int)(((long long)nkb_all * sp) / S), kb1 = (int)(((long long)nkb_all * (sp + 1)) / S);
  volatile int* abortp = &abort_flag;
  // Slices that fit the ring (the usual case: the split is chosen that way) have all their loads in flight from the
  // start; longer slices recycle stages through the empty barriers.
  const int ring = L::ring(S);

  if (warp == 0) {
    // ---- producer: weights first (static), then wait for the previous kernel, then activations
    const uint64_t wpol = a.rows_total <= TN ? l2_policy_stream() : l2_policy_normal();
    auto load_weights = [&](int s, int kb) {
      uint8_t* st = smem + s * C::STAGE_BYTES;
      uint8_t* sA = st, *sSFA = st + C::A_BYTES + C::B_BYTES;
      mbar_expect_tx(&full_bar[s], C::A_BYTES + C::B_BYTES + C::SFA_BYTES);
      tma_load_3d_hint(sA, a.tmA, &full_bar[s], kb * (KIND == KIND_BF16 ? 64 : 128), nt * 128, 0, wpol);
      if (KIND != KIND_BF16)
        bulk_load_1d_hint(sSFA, a.sfa[0] + ((size_t)nt * nkb_all + (size_t)kb) * C::SF_CHUNKS * 512, C::SFA_BYTES, &full_bar[s], wpol);
    };
    const int npre = min(ring, kb1 - kb0);
    if (lane == 0)
      for (int i = 0; i < npre; ++i) load_weights(i, kb0 + i);
    pdl_wait();
    if (lane == 0) CL_TRACE(2);
    for (int kb = kb0, it = 0; kb < kb1 && !*abortp; ++kb, ++it) {
      const int s = it % ring;
      if (it >= ring) {
        if (!mbar_wait_bounded(&empty_bar[s], ((it / ring) & 1) ^ 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_PRODUCER, (int)blockIdx.x); break; }
        if (lane == 0) load_weights(s, kb);
      }
      uint8_t* st = smem + s * C::STAGE_BYTES;
      uint8_t* sB = st + C::A_BYTES, *sSFB = sB + C::B_BYTES + C::SFA_BYTES;
      if (lane == 0) tma_load_3d(sB, a.tmB, &full_bar[s], kb * (KIND == KIND_BF16 ? 64 : 128), row0, 0);
      if (KIND != KIND_BF16) {
        constexpr int SFB_PER_STAGE = C::SF_CHUNKS * 4;
        for (int c = lane; c < TN; c += 32) {
          const int row = row0 + c;
          const bool live = c < nrows && row < a.rows_total;
          const uint8_t* src = live ? a.sfb + (size_t)row * a.ldsfb + (size_t)kb * SFB_PER_STAGE : a.sfb;
          const uint32_t dst = smem_u32(sSFB + (c & 31) * 16 + ((c & 127) >> 5) * 4);
          const uint32_t nbytes = live ? 4u : 0u;
#pragma unroll
          for (int q = 0; q < C::SF_CHUNKS; ++q)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + q * 512), "l"(src + q * 4), "r"(nbytes) : "memory");
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full_bar[s])) : "memory");
      } else {
        mbar_arrive(&full_bar[s]);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (one elected thread)
    pdl_wait();
    if (lane == 0) {
      const uint32_t smem_base = smem_u32(smem);
      bool ok = true;
      for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
        const int s = it % ring;
        if (!mbar_wait_bounded(&full_bar[s], (it / ring) & 1, abortp)) { ca_dev_fail(a.status, CA_DEV_TIMEOUT_MMA, (int)blockIdx.x); ok = false; break; }
        if (it == 0) CL_TRACE(3);
        tc_fence_after();
        if (KIND != KIND_BF16) fence_proxy_async_smem();
        const uint32_t st = smem_base + s * C::STAGE_BYTES;
        const uint32_t sA = st, sB = st + C::A_BYTES, sSFA = sB + C::B_BYTES, sSFB = sSFA + C::SFA_BYTES;
        if (KIND != KIND_BF16) {
#pragma unroll
          for (int q = 0; q < C::SF_CHUNKS; ++q) {
            tc_cp_sf(tmem + L::SFA_COL + 4 * q, umma_desc_sf(sSFA + q * 512));
            tc_cp_sf(tmem + L::SFB_COL + 4 * q, umma_desc_sf(sSFB + q * 512));
          }
        }
        const uint64_t adesc = umma_desc_sw128(sA), bdesc = umma_desc_sw128(sB);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
          if (KIND == KIND_BF16) tc_mma_f16(tmem, adesc + 2 * k, bdesc + 2 * k, make_idesc(KIND_BF16, TN, 0), accum);
          else if (KIND == KIND_NVFP4)
            tc_mma_nvf4(tmem, adesc + 2 * k, bdesc + 2 * k, make_idesc(KIND_NVFP4, TN, 0), accum, tmem + L::SFA_COL + 4 * k, tmem + L::SFB_COL + 4 * k);
          else
            tc_mma_mxf4(tmem, adesc + 2 * k, bdesc + 2 * k, make_idesc(KIND_MXFP4, TN, (k & 1) * 2), accum, tmem + L::SFA_COL + 4 * (k >> 1),
                        tmem + L::SFB_COL + 4 * (k >> 1));
        }
        tc_commit(&empty_bar[s]);
      }
      if (ok) tc_commit(&accf_bar);
      CL_TRACE(4);
    }
    __syncwarp();
  } else {
    pdl_wait();
  }

  // ---- partial tiles of ranks 1..S-1 travel to rank 0's staging area
  const int q4 = warp & 3, et = q4 * 32 + lane;
  const uint32_t tbase = tmem + ((uint32_t)(q4 * 32) << 16);
  // Everything the last step of the chain reads from global memory is fetched NOW, under the main loop: the output scale and the
  // residual rows of rank 0's tile (R may alias Y, so these loads must also come before the stores).  After the cluster barrier
  // only tensor-memory loads, shared-memory adds and the stores remain.
  // Rank 0 finishes the tile row-wise when the output allows 16-byte accesses: its own partial goes to the staging area too, and
  // after the barrier every thread owns (token, 8 consecutive features) items - two float4 reads per partial, one 16-byte store -
  // instead of sixteen 2-byte stores behind sixteen unrolled copies of the adds (short code: this tail runs once per launch, from a
  // cold instruction cache).
  const bool vec_ok = !(PEER && a.n_peer) && a.Y && a.N % 8 == 0 && a.ldy % 8 == 0 && ((uintptr_t)a.Y & 15) == 0 &&
                      (a.epi != EPI_BF16_RESIDUAL || ((uintptr_t)a.R & 15) == 0);
  constexpr int ITEMS = TN / 8;                              // items of one thread: TN rows x 16 feature groups / 128 threads
  const int tid128 = (warp >= 2) ? (warp - 2) * 32 + lane : 0;
  float al_pre = 1.f, res_pre[TN];
  uint4 rv_pre[ITEMS];
#pragma unroll
  for (int j = 0; j < TN; ++j) res_pre[j] = 0.f;
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) rv_pre[j] = make_uint4(0u, 0u, 0u, 0u);
  if (warp >= 2) {
    if (a.alpha) al_pre = a.alpha[0];
    const int n_pre = nt * 128 + et;
    if (sp == 0 && a.epi == EPI_BF16_RESIDUAL) {
      if (vec_ok) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
          const int i = tid128 + it * 128, c = i >> 4, nn = nt * 128 + (i & 15) * 8;
          if (c < nrows && nn < a.N) rv_pre[it] = *(const uint4*)(a.R + (size_t)(row0 + c) * a.ldy + nn);
        }
      } else if (n_pre < a.N) {
#pragma unroll
        for (int j = 0; j < TN; ++j)
          if (j < nrows) res_pre[j] = __bfloat162float(a.R[(size_t)(row0 + j) * a.ldy + n_pre]);
      }
    }
  }
  bool have_acc = false;
  if (warp >= 2) {
    have_acc = (kb1 > kb0) && mbar_wait_bounded(&accf_bar, 0, abortp);
    have_acc = __all_sync(0xffffffffu, have_acc);      // tensor-memory loads below must be warp-uniform
    if (!have_acc && kb1 > kb0) ca_dev_fail(a.status, CA_DEV_TIMEOUT_EPILOGUE, (int)blockIdx.x);
    tc_fence_after();
    if (warp == 2 && lane == 0) CL_TRACE(5);
    if (sp != 0) {
      const uint32_t remote = map_to_rank(smem_u32(staging), 0) + (uint32_t)(sp - 1) * (128 * TN * 4);
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 16) {
        uint32_t r[16];
        if (have_acc) { tmem_ld_x16(tbase + c0, r); tc_wait_ld(); }
#pragma unroll
        for (int j = 0; j < 16; ++j) st_cluster_f32(remote + (uint32_t)((c0 + j) * 128 + et) * 4, have_acc ? __uint_as_float(r[j]) : 0.f);
      }
    } else if (vec_ok) {
      float* own = staging + (size_t)(S - 1) * (128 * TN);
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 16) {
        uint32_t r[16];
        if (have_acc) { tmem_ld_x16(tbase + c0, r); tc_wait_ld(); }
#pragma unroll
        for (int j = 0; j < 16; ++j) own[(c0 + j) * 128 + et] = have_acc ? __uint_as_float(r[j]) : 0.f;
      }
    }
  }
  __syncwarp();
  cluster_sync_all();                      // every thread of every CTA of the cluster, exactly once
  if (warp == 2 && lane == 0) CL_TRACE(6);
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
          const float* sp_ = staging + (size_t)(p - 1) * (128 * TN) + c * 128 + g8;
          const float4 p0 = *(const float4*)sp_, p1 = *(const float4*)(sp_ + 4);
          f[0] += p0.x; f[1] += p0.y; f[2] += p0.z; f[3] += p0.w; f[4] += p1.x; f[5] += p1.y; f[6] += p1.z; f[7] += p1.w;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) f[q] *= al_pre;
        const size_t o = (size_t)(row0 + c) * a.ldy + nn;
        if (a.epi == EPI_F32) {
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
    const bool n_ok = n < a.N;
    const float al = al_pre;
#pragma unroll
    for (int c0 = 0; c0 < TN; c0 += 16) {
      uint32_t r[16];
      if (have_acc) { tmem_ld_x16(tbase + c0, r); tc_wait_ld(); }
      if (c0 == 0 && warp == 2 && lane == 0) CL_TRACE(1);
      if (c0 < nrows && n_ok) {
        const float* res = res_pre + c0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int c = c0 + j;
          if (c < nrows) {
            float v = have_acc ? __uint_as_float(r[j]) : 0.f;
            for (int p = 1; p < S; ++p) v += staging[(size_t)(p - 1) * (128 * TN) + c * 128 + et];
            v *= al;
            const size_t o = (size_t)(row0 + c) * a.ldy + n;
            if (a.epi == EPI_F32) ((float*)a.Y)[o] = v;
            else {
              v += res[j];
              const bf16 vb = __float2bfloat16(v);
              if (a.Y) ((bf16*)a.Y)[o] = vb;
              if (PEER && a.n_peer) peer_store(a, row0 + c, n, vb);
            }
          }
        }
      }
    }
  }
  if (warp == 2 && lane == 0) CL_TRACE(7);
  if (PEER && warp >= 2 && a.n_peer) peer_publish(a, warp, lane);      // every CTA counts in; only rank 0 of a cluster stored
  if (*abortp && warp == 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, L::TMEM_COLS);
}

template <int KIND, int TN, bool PEER>
static int launch_cluster_p(const TcArgs& a, int grid, cudaStream_t stream) {
  using L = ClCfg<KIND, TN>;
  auto kern = tc_linear_cluster_kernel<KIND, TN, PEER>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(tc_linear_cluster)");
    attr_set[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = L::SMEM_BYTES; cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = a.splits; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = ca_pdl_enabled(CA_PDL_CLASS) ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) return ca_cuda(e, "tc_linear_cluster launch");
  return CA_OK;
}

// How many clusters of `splits` CTAs of the split-K kernel the device can hold at once (a cluster needs `splits` free SMs inside
// ONE GPC, so the answer is well below SMs / splits for sizes that do not divide the GPCs evenly): a split whose cluster count
// exceeds this runs in two waves.
template <int KIND, int TN>
static int cluster_capacity(int splits, int* out) {
  using L = ClCfg<KIND, TN>;
  auto kern = tc_linear_cluster_kernel<KIND, TN, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
  if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(tc_linear_cluster)");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits * 64); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = L::SMEM_BYTES;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = splits; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  e = cudaOccupancyMaxActiveClusters(out, kern, &cfg);
  if (e != cudaSuccess) return ca_cuda(e, "cudaOccupancyMaxActiveClusters");
  return CA_OK;
}

extern "C" int cuteafd_tc_cluster_capacity(int kind, int tn, int splits, int* out) {
  CA_REQUIRE(out && (tn == 16 || tn == 32) && splits >= 1 && splits <= (tn == 16 ? 8 : 4), "tc_cluster_capacity: bad arguments");
  if (kind == KIND_BF16) return tn == 16 ? cluster_capacity<KIND_BF16, 16>(splits, out) : cluster_capacity<KIND_BF16, 32>(splits, out);
  if (kind == KIND_NVFP4) return tn == 16 ? cluster_capacity<KIND_NVFP4, 16>(splits, out) : cluster_capacity<KIND_NVFP4, 32>(splits, out);
  if (kind == KIND_MXFP4) return tn == 16 ? cluster_capacity<KIND_MXFP4, 16>(splits, out) : cluster_capacity<KIND_MXFP4, 32>(splits, out);
  return ca_fail(CA_ERR_UNSUPPORTED, "tc_cluster_capacity: no cluster kernel for this kind");
}

template <int KIND, int TN>
static int launch_cluster(const TcArgs& a, int grid, cudaStream_t stream) {
  return a.n_peer ? launch_cluster_p<KIND, TN, true>(a, grid, stream) : launch_cluster_p<KIND, TN, false>(a, grid, stream);
}

// Device trace buffer for later launches on the calling thread's device: [grid, units, 8] 64-bit stamps, or
// null to switch tracing off.  (No counterpart in the reference, whose GEMM programs are opaque AOT exports.)
static long long* g_trace = nullptr;
static int g_trace_units = 0;
extern "C" int cuteafd_tc_trace(void* buf, int units) {
  g_trace = (long long*)buf;
  g_trace_units = buf ? units : 0;         // units < 0: the cluster split-K kernel's launches with N == -units record instead
  return CA_OK;
}

extern "C" int cuteafd_tc_linear(int kind, int swiglu, int tn, const void* tmA, const void* tmA2, const void* tmB,
                                 const void* sfa, const void* sfa2, const void* sfb, int ldsfb, const float* alpha,
                                 const float* alpha2, const void* tiles, const int* n_tiles, int max_tiles, void* Y,
                                 const void* R, int ldy, int rows_total, int N, int K, int epi, int splits,
                                 float* splitk_ws, int* splitk_cnt, int* status, int max_ctas, const CaTcExtra* extra,
                                 cudaStream_t stream) {
  // `extra` (optional): an FP4 copy of the output for the GEMM that consumes it (an option of the fused SwiGLU GEMM: codes
  // [rows, N / 2], scales [rows, ldsf_out]; Y may then be null), and/or stores of the bf16 output tiles into 1-2 peers'
  // buffers (row r -> row peer_row_map[r] when a map is given) with the peers' flags released with step number peer_ctl[1]
  // once the whole GEMM has been written (`peer_done`: a zeroed device counter).
  CA_REQUIRE((kind >= 0 && kind <= 2) || kind == KIND_W4A8, "tc_linear: bad kind %d", kind);
  void* q_out = extra ? extra->q_out : nullptr; void* sf_out = extra ? extra->sf_out : nullptr;
  const float* inv_gs_out = extra ? extra->inv_gs_out : nullptr; const int ldsf_out = extra ? extra->ldsf_out : 0;
  struct { void* y[2]; void* flags[2]; const int* row_map; void* ctl; void* done; int ld, n; } peer = {};
  if (extra && extra->n_peer) {
    peer.n = extra->n_peer; peer.ld = extra->peer_ld; peer.row_map = extra->peer_row_map; peer.ctl = extra->peer_ctl; peer.done = extra->peer_done;
    for (int i = 0; i < 2; ++i) { peer.y[i] = extra->peer_y[i]; peer.flags[i] = extra->peer_flag[i]; }
    CA_REQUIRE(peer.n >= 1 && peer.n <= 2 && peer.y[0] && peer.flags[0] && peer.ctl && peer.done && (peer.n == 1 || (peer.y[1] && peer.flags[1])),
               "tc_linear: peer output takes 1 or 2 peers with buffers and flags");
  }
  CA_REQUIRE(tmA && tmB && (Y || q_out || peer.n), "tc_linear: null operand");
  CA_REQUIRE(!peer.n || (epi != EPI_F32 && !q_out && !swiglu), "tc_linear: peer output is a plain bf16 epilogue (no SwiGLU, no FP4 output)");
  CA_REQUIRE(!q_out || (kind != KIND_BF16 && swiglu && sf_out && splits <= 1 && N % 32 == 0 && epi == EPI_BF16),
             "tc_linear: FP4 output is an option of the fused SwiGLU GEMM of an FP4 kind (no split-K, N %% 32 == 0, bf16 epilogue)");
  CA_REQUIRE(!swiglu || tmA2, "tc_linear: swiglu needs the up-projection descriptor");
  CA_REQUIRE(kind == KIND_BF16 || (sfa && sfb && K % 32 == 0), "tc_linear: fp4 kinds need scales and K %% 32 == 0 (K=%d)", K);
  CA_REQUIRE(kind == KIND_BF16 ? (K % 8 == 0) : true, "tc_linear: K must be a multiple of 8");
  CA_REQUIRE(splits <= 1 || (!tiles && !swiglu && splitk_ws && splitk_cnt), "tc_linear: split-K is dense, non-swiglu only and needs scratch");
  CA_REQUIRE(epi == EPI_BF16 || epi == EPI_BF16_RESIDUAL || epi == EPI_F32, "tc_linear: bad epilogue %d", epi);
  CA_REQUIRE(epi != EPI_BF16_RESIDUAL || R, "tc_linear: residual epilogue needs R");
  if (rows_total <= 0 || N <= 0) return CA_OK;
  TcArgs a;
  a.tmA = (const CUtensorMap*)tmA; a.tmA2 = (const CUtensorMap*)tmA2; a.tmB = (const CUtensorMap*)tmB;
  a.sfa = (const uint8_t* const*)sfa; a.sfa2 = (const uint8_t* const*)sfa2; a.sfb = (const uint8_t*)sfb;
  a.alpha = alpha; a.alpha2 = alpha2; a.tiles = (const int4*)tiles; a.n_tiles = n_tiles;
  a.Y = Y; a.R = (const bf16*)R; a.splitk_ws = splitk_ws; a.splitk_cnt = splitk_cnt; a.status = status;
  a.trace = g_trace; a.trace_units = g_trace_units;
  a.peer_y0 = peer.y[0]; a.peer_y1 = peer.y[1]; a.peer_flag0 = (uint32_t*)peer.flags[0]; a.peer_flag1 = (uint32_t*)peer.flags[1];
  a.peer_row_map = peer.row_map; a.peer_ctl = (uint32_t*)peer.ctl; a.peer_done = (uint32_t*)peer.done; a.peer_ld = peer.ld; a.n_peer = peer.n;
  a.q_out = (uint8_t*)q_out; a.sf_out = (uint8_t*)sf_out; a.inv_gs_out = inv_gs_out; a.ldsf_out = ldsf_out;
  a.ldsfb = ldsfb; a.ldy = ldy; a.rows_total = rows_total; a.N = N; a.K = K; a.epi = epi; a.splits = splits > 1 ? splits : 1;
  // A 128 x 128 tile of packed 4-bit weights that TMA expands into 16-byte groups of 16 elements (8 data bytes + 8 bytes of
  // padding) occupies 16 KB of shared memory, but the barrier's transaction count receives the 8 KB of data that were copied
  // (measured: with 16 KB expected the stage never completes).
  a.w4_tx = 128 * 128 / 2;
  const int n_nt = (N + 127) / 128;
  if (kind == KIND_W4A8 && !tiles && !swiglu && a.splits > 1 && tn <= 32) a.splits = 1;       // no cluster split-K variant of this kind: one CTA per tile
  if (!tiles && !swiglu && (tn == 16 || tn == 32) && a.splits >= 2 && a.splits <= (tn == 16 ? 8 : 4)) {
    {
      const int grid_c = ((rows_total + tn - 1) / tn) * n_nt * a.splits;
      if (kind == KIND_BF16) return tn == 16 ? launch_cluster<KIND_BF16, 16>(a, grid_c, stream) : launch_cluster<KIND_BF16, 32>(a, grid_c, stream);
      if (kind == KIND_NVFP4) return tn == 16 ? launch_cluster<KIND_NVFP4, 16>(a, grid_c, stream) : launch_cluster<KIND_NVFP4, 32>(a, grid_c, stream);
      return tn == 16 ? launch_cluster<KIND_MXFP4, 16>(a, grid_c, stream) : launch_cluster<KIND_MXFP4, 32>(a, grid_c, stream);
    }
  }
  long long work = tiles ? (long long)max_tiles * n_nt : (long long)((rows_total + tn - 1) / tn) * n_nt * a.splits;
  int cap = max_ctas > 0 ? max_ctas : ca_sm_count() * (tn <= 32 ? 2 : 1);
  int grid = (int)(work < cap ? work : cap);
  if (grid < 1) grid = 1;
  if (kind == KIND_BF16) return swiglu ? launch_tn<KIND_BF16, true>(tn, a, grid, stream) : launch_tn<KIND_BF16, false>(tn, a, grid, stream);
  if (kind == KIND_NVFP4) return swiglu ? launch_tn<KIND_NVFP4, true>(tn, a, grid, stream) : launch_tn<KIND_NVFP4, false>(tn, a, grid, stream);
  if (kind == KIND_W4A8) return swiglu ? launch_tn<KIND_W4A8, true>(tn, a, grid, stream) : launch_tn<KIND_W4A8, false>(tn, a, grid, stream);
  return swiglu ? launch_tn<KIND_MXFP4, true>(tn, a, grid, stream) : launch_tn<KIND_MXFP4, false>(tn, a, grid, stream);
}
