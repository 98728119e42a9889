// Mixture-of-experts control kernels: router selection, route packing into expert order (with the
// tile table the grouped tcgen05 GEMM walks), and the ordered weighted combine (+ shared expert +
// residual) with fp32 accumulation in slot order and a single bf16 rounding.
// Reference counterparts: native/shared/cuda/expert_router.cu:73-171 (select kernels),
// route_reduce.cu:30-125 (ordered reduce), residual.cu:419-498 (scatter-add / combine + residual).
#include "common.cuh"

enum { SCORE_SIGMOID = 0, SCORE_SOFTMAX = 1, SCORE_SQRTSOFTPLUS = 2 };

// ---------------------------------------------------------------- route packing
// Inputs: idx [T, k] (expert ids; ids outside [e_lo, e_hi) are skipped - they belong to another expert rank).
// Outputs: src_token [cap]  (token of each packed row, expert-major), slot_row [T, k] (packed row of each
// route, -1 when skipped), counts/offsets per local expert, a tile table {local expert, first row, rows, 0}
// with at most `tn` rows per entry, n_tiles and n_rows.  Runs in ONE block (any size); T*k up to ~64K routes.
struct RoutePack {
  const int* idx; int* src_token; int* slot_row; int* counts; int* offsets; int4* tiles; int* n_tiles; int* n_rows; int* src_route;
  int T, k, e_lo, e_hi, tn, max_tiles;
  int* ticket;      // fused with the router: arrival counter of the select blocks (zero on entry, left zero)
  FlagWait wait;    // expert ranks: the routing table and the rows arrive from peers; wait for their flags first
  // Several senders ("lanes") share one routing table laid out [lane][t_cap][k]; lane l delivered lane_T[l] tokens this step
  // (written by the sender next to its rows).  Token index = l * t_cap + t; rows t >= lane_T[l] are stale and skipped.
  const int* lane_T; int t_cap;
};

__device__ __forceinline__ bool route_live(const RoutePack& p, int i) {
  if (!p.lane_T) return true;
  const int tok = i / p.k;
  return (tok % p.t_cap) < __ldcg(p.lane_T + tok / p.t_cap);
}

// `ids_sh`: the routing table idx [T * k] when the calling block holds it in shared memory (it then need not come back from L2).
__device__ __forceinline__ void route_pack_body(const RoutePack& p, int* sh, const int* ids_sh = nullptr) {
  // sh: [E_local] counts, [E_local] offsets/cursors, [T*k] staged ids (small batches)
  const int El = p.e_hi - p.e_lo;
  int* cnt = sh; int* cur = sh + El;
  for (int e = threadIdx.x; e < El; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int n = p.T * p.k;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    if (!route_live(p, i)) continue;
    const int e = (ids_sh ? ids_sh[i] : __ldcg(p.idx + i)) - p.e_lo;
    if (e >= 0 && e < El) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  // Row offsets and the tile table in expert order: warp 0 scans, each lane owning a run of consecutive experts
  // (a single thread walking all experts with its global stores was several microseconds of every MoE layer).
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x, per = (El + 31) / 32, e0 = min(El, lane * per), e1 = min(El, e0 + per);
    int rows = 0, tiles = 0;
    for (int e = e0; e < e1; ++e) { rows += cnt[e]; tiles += (cnt[e] + p.tn - 1) / p.tn; }
    int rsum = rows, tsum = tiles;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, rsum, o), b = __shfl_up_sync(0xffffffffu, tsum, o);
      if (lane >= o) { rsum += a; tsum += b; }
    }
    int off = rsum - rows, nt = tsum - tiles;                 // exclusive prefix of this lane's run
    for (int e = e0; e < e1; ++e) {
      const int c = cnt[e];
      cur[e] = off; p.offsets[e] = off; p.counts[e] = c;
      for (int r = 0; r < c; r += p.tn) { if (nt < p.max_tiles) p.tiles[nt] = make_int4(e, off + r, min(p.tn, c - r), 0); ++nt; }
      off += c;
    }
    if (lane == 31) { *p.n_tiles = min(tsum, p.max_tiles); *p.n_rows = rsum; }
  }
  __syncthreads();
  // Stable placement (token order inside each expert) so packed layouts are reproducible: each route counts the
  // earlier routes to its expert when T*k is small; larger batches use atomics (row order inside an expert does
  // not change any result: rows are independent in the GEMM and the combine reads them by index).
  // (multi-lane tables need no agreement with the senders on row positions, so their larger cases take the atomic path)
  if (n <= 256 && blockDim.x >= 256 && (blockDim.x & 31) == 0) {
    // Decode-sized tables: stable ranks without the quadratic walk.  Each warp owns 32 consecutive routes; a route's rank inside its
    // expert = routes to that expert in earlier warps (a per-warp histogram, summed) + lanes below it in its own warp with the same
    // expert (match + population count).  The walk below costs ~2.5 us at 128 routes, this a few hundred cycles.
    int* hist = cur + El;                                    // [8][El] routes per (warp chunk, expert); sized with the ids scratch
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nch = (n + 31) >> 5;
    for (int i = threadIdx.x; i < nch * El; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    int e_mine = -1, below = 0;
    if (warp < nch) {
      const int i = warp * 32 + lane;
      if (i < n && route_live(p, i)) e_mine = (ids_sh ? ids_sh[i] : __ldcg(p.idx + i)) - p.e_lo;
      if (e_mine < 0 || e_mine >= El) e_mine = -1;
      const unsigned same = __match_any_sync(0xffffffffu, e_mine);
      below = __popc(same & ((1u << lane) - 1u));
      if (e_mine >= 0 && below == 0) hist[warp * El + e_mine] = __popc(same);      // the lowest lane of each expert's group records it
    }
    __syncthreads();
    if (warp < nch) {
      const int i = warp * 32 + lane;
      if (i < n) {
        if (e_mine < 0) p.slot_row[i] = -1;
        else {
          int rank = below;
          for (int w = 0; w < warp; ++w) rank += hist[w * El + e_mine];
          const int c = cur[e_mine] + rank;
          p.src_token[c] = i / p.k; p.slot_row[i] = c;
          if (p.src_route) p.src_route[c] = i;
        }
      }
    }
  } else if (n <= (p.lane_T ? 256 : 4096)) {        // the quadratic ranking costs ~17 us at 1024 routes: lane tables switch to atomics early
    int* sid = cur + El;
    for (int i = threadIdx.x; i < n; i += blockDim.x) sid[i] = route_live(p, i) ? (ids_sh ? ids_sh[i] : __ldcg(p.idx + i)) - p.e_lo : -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int e = sid[i];
      if (e < 0 || e >= El) { p.slot_row[i] = -1; continue; }
      int rank = 0;
      for (int j = 0; j < i; ++j) rank += (sid[j] == e);
      const int c = cur[e] + rank;
      p.src_token[c] = i / p.k; p.slot_row[i] = c;
      if (p.src_route) p.src_route[c] = i;
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int e = route_live(p, i) ? (ids_sh ? ids_sh[i] : __ldcg(p.idx + i)) - p.e_lo : -1;
      if (e >= 0 && e < El) { const int c = atomicAdd(&cur[e], 1); p.src_token[c] = i / p.k; p.slot_row[i] = c; if (p.src_route) p.src_route[c] = i; } else p.slot_row[i] = -1;
    }
  }
}

__global__ void route_pack_kernel(const RoutePack p) {
  pdl_launch(); pdl_wait();
  extern __shared__ int sh[];
  if (!flag_wait_block(p.wait)) {      // the peer never delivered: publish an empty work list
    if (threadIdx.x == 0) { *p.n_tiles = 0; *p.n_rows = 0; }
    return;
  }
  route_pack_body(p, sh);
}

static size_t route_pack_smem(int T, int k, int e_lo, int e_hi) {
  const int El = e_hi - e_lo, n = T * k;
  int extra = n <= 4096 ? n : 0;                               // staged ids of the quadratic ranking
  if (n <= 256 && 8 * El > extra) extra = 8 * El;              // per-warp histograms of the decode-sized ranking
  return (size_t)(2 * El + extra) * sizeof(int);
}


// One block per token.  logits fp32 [T, E] (E <= 512).  Selection uses score + bias (bias may be null),
// optional group-limited routing (top `topk_group` of `n_group` groups ranked by the sum of their two
// best biased scores); gate weights come from the unbiased scores, normalised over the chosen k and
// multiplied by route_scale.  Ties resolve to the lowest expert id.
__global__ void router_select_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ idx,
                                     float* __restrict__ wts, int E, int k, int scoring, int normalize, float route_scale,
                                     int n_group, int topk_group, const RoutePack pack) {
  pdl_launch(); pdl_wait();
  extern __shared__ int pack_sh[];
  __shared__ int is_last;
  __shared__ float score[512], choice[512], red[32];
  __shared__ float gscore[32];
  __shared__ int sel[16];
  __shared__ float selw[16];
  const int t = blockIdx.x, tid = threadIdx.x;
  const float* lg = logits + (size_t)t * E;
  float mx = -INFINITY;
  for (int e = tid; e < E; e += blockDim.x) mx = fmaxf(mx, lg[e]);
  float denom = 1.f;
  if (scoring == SCORE_SOFTMAX) {
    mx = block_max(mx, red);
    float s = 0.f;
    for (int e = tid; e < E; e += blockDim.x) s += expf(lg[e] - mx);
    denom = block_sum(s, red);
  }
  for (int e = tid; e < E; e += blockDim.x) {
    const float x = lg[e];
    float sc;
    if (scoring == SCORE_SIGMOID) sc = 1.f / (1.f + expf(-x));
    else if (scoring == SCORE_SOFTMAX) sc = expf(x - mx) / denom;
    else sc = sqrtf(x > 20.f ? x : log1pf(expf(x)));
    score[e] = sc;
    choice[e] = sc + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (n_group > 1 && topk_group < n_group) {
    const int per = E / n_group;
    if (tid < n_group) {
      float a = -INFINITY, b = -INFINITY;
      for (int j = 0; j < per; ++j) { const float v = choice[tid * per + j]; if (v > a) { b = a; a = v; } else if (v > b) b = v; }
      gscore[tid] = a + b;
    }
    __syncthreads();
    if (tid == 0) {
      // keep the best topk_group groups (stable: lowest group id first among equals)
      unsigned keep = 0;
      for (int r = 0; r < topk_group; ++r) {
        int best = -1; float bv = -INFINITY;
        for (int g = 0; g < n_group; ++g) if (!(keep >> g & 1) && (best < 0 || gscore[g] > bv)) { best = g; bv = gscore[g]; }
        keep |= 1u << best;
      }
      for (int g = 0; g < n_group; ++g) if (!(keep >> g & 1)) gscore[g] = -INFINITY; else gscore[g] = 0.f;
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) if (gscore[e / per] != 0.f) choice[e] = -INFINITY;
    __syncthreads();
  }
  // k rounds of argmax (value desc, index asc) by warp 0 alone: the scores are in shared memory, so the rounds need
  // no block barrier (two per round cost more than the scan itself at 128 experts)
  if (tid < 32) {
    for (int r = 0; r < k; ++r) {
      float bv = -INFINITY; int bi = 0x7fffffff;
      for (int e = tid; e < E; e += 32) { const float v = choice[e]; if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; } }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (bi >= E) bi = 0;
      if (tid == 0) { sel[r] = bi; selw[r] = score[bi]; choice[bi] = -INFINITY; }
      __syncwarp();
    }
  }
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int r = 0; r < k; ++r) s += selw[r];
    const float inv = normalize ? 1.f / fmaxf(s, 1e-12f) : 1.f;
    for (int r = 0; r < k; ++r) { idx[(size_t)t * k + r] = sel[r]; wts[(size_t)t * k + r] = selw[r] * inv * route_scale; }
  }
  if (pack.ticket) {
    // the block that finishes last sees every token's routes and packs them (one launch instead of two)
    if (tid == 0) {
      __threadfence();
      is_last = (atomicAdd(pack.ticket, 1) == (int)gridDim.x - 1);
      __threadfence();
    }
    __syncthreads();
    if (is_last) {
      route_pack_body(pack, pack_sh);
      if (tid == 0) *pack.ticket = 0;
    }
  }
}

// Router logits for decode-sized batches: logits[t][e] = x[t] . w[e] in fp32, one block per expert.  The tensor-core
// path needs an 8-CTA cluster split-K to spread this 1 MB weight and still spends most of its ~14 us in launch and
// cluster overheads; here 128 blocks read 8 KB of weights each and the token rows from L2.
#define RL_TOK 16
__global__ void __launch_bounds__(512) router_logits_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, float* __restrict__ logits,
                                                             int T, int E, int H) {
  pdl_launch(); pdl_wait();
  __shared__ float red[RL_TOK][16];
  const int nw = blockDim.x >> 5;
  const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bf16* wr = w + (size_t)e * H;
  for (int t0 = 0; t0 < T; t0 += RL_TOK) {
    float acc[RL_TOK];
#pragma unroll
    for (int j = 0; j < RL_TOK; ++j) acc[j] = 0.f;
    for (int c = tid; c < H / 8; c += blockDim.x) {
      const uint4 wv = *(const uint4*)(wr + c * 8);
      const bf162* wp = (const bf162*)&wv;
      float wf[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(wp[q]); wf[2 * q] = f.x; wf[2 * q + 1] = f.y; }
#pragma unroll
      for (int j = 0; j < RL_TOK; ++j) {
        if (t0 + j < T) {
          const uint4 xv = *(const uint4*)(x + (size_t)(t0 + j) * H + c * 8);
          const bf162* xp = (const bf162*)&xv;
#pragma unroll
          for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(xp[q]); acc[j] = fmaf(f.x, wf[2 * q], acc[j]); acc[j] = fmaf(f.y, wf[2 * q + 1], acc[j]); }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < RL_TOK; ++j) {
      float v = acc[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) red[j][warp] = v;
    }
    __syncthreads();
    if (tid < RL_TOK && t0 + tid < T) {
      float v = 0.f;
      for (int q = 0; q < nw; ++q) v += red[tid][q];
      logits[(size_t)(t0 + tid) * E + e] = v;
    }
    __syncthreads();
  }
}

extern "C" int cuteafd_router_logits(const void* x, const void* w, float* logits, int T, int E, int H, cudaStream_t s) {
  CA_REQUIRE(H % 8 == 0 && E >= 1, "router_logits: hidden size must be a multiple of 8");
  if (T <= 0) return CA_OK;
  // one 16-byte weight chunk per thread where the row allows it: every load of a token row is in flight at once
  const int threads = H / 8 >= 512 ? 512 : (H / 8 >= 256 ? 256 : 128);
  CA_LAUNCH_PDL(router_logits_kernel, E, threads, 0, s, (const bf16*)x, (const bf16*)w, logits, T, E, H);
  CA_CHECK_LAUNCH("router_logits");
  return CA_OK;
}

static int launch_router_select_warps(const float* logits, const float* bias, int* idx, float* wts, int T, int E, int k, int scoring, int normalize,
                                      float route_scale, int n_group, int topk_group, cudaStream_t s);

extern "C" int cuteafd_router_select(const float* logits, const float* bias, int* idx, float* wts, int T, int E, int k,
                                     int scoring, int normalize, float route_scale, int n_group, int topk_group, cudaStream_t s) {
  CA_REQUIRE(E >= k && E <= 512 && k >= 1 && k <= 16, "router_select: need k <= 16 and E <= 512 (E=%d k=%d)", E, k);
  CA_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0, "router_select: bad group count");
  if (T <= 0) return CA_OK;
  // decode / verify steps: the warp-per-token selection that the one-block select + pack kernel uses (identical picks and weights)
  if (T <= 64) return launch_router_select_warps(logits, bias, idx, wts, T, E, k, scoring, normalize, route_scale, n_group, topk_group, s);
  const int threads = E <= 64 ? 64 : (E <= 128 ? 128 : 256);
  RoutePack none{};
  none.wait = FlagWait{nullptr, nullptr, nullptr, 0ull, 0, 0};
  none.lane_T = nullptr; none.t_cap = 0;
  CA_LAUNCH_PDL(router_select_kernel, T, threads, 0, s, logits, bias, idx, wts, E, k, scoring, normalize, route_scale, n_group, topk_group, none);
  return CA_OK;
}

extern "C" int cuteafd_route_pack(const int* idx, int* src_token, int* slot_row, int* counts, int* offsets, void* tiles,
                                  int* n_tiles, int* n_rows, int T, int k, int e_lo, int e_hi, int tn, int max_tiles, int* src_route,
                                  const CaFlagWaitArg* wait, const int* lane_T, int t_cap, cudaStream_t s) {
  const FlagWait fw = ca_flag_wait_from(wait);
  CA_REQUIRE(e_hi > e_lo && e_hi - e_lo <= 4096, "route_pack: bad expert range");
  CA_REQUIRE(tn >= 1, "route_pack: bad tile rows");
  CA_REQUIRE(!lane_T || (t_cap >= 1 && T % t_cap == 0), "route_pack: a lane table needs T = lanes * t_cap");
  RoutePack p{idx, src_token, slot_row, counts, offsets, (int4*)tiles, n_tiles, n_rows, src_route, T, k, e_lo, e_hi, tn, max_tiles, nullptr,
              fw, lane_T, t_cap};
  CA_LAUNCH_PDL(route_pack_kernel, 1, 1024, route_pack_smem(T, k, e_lo, e_hi), s, p);
  return CA_OK;
}

// Rows of a token-major slab (FP4 / bf16 payload + block scales, as the dispatch kernel delivered them) gathered into the
// expert-major order of the route pack: dst row c = src row src_token[c] for c < *n_rows.  One block per packed row.
__global__ void route_gather_kernel(const uint8_t* __restrict__ src_q, const uint8_t* __restrict__ src_sf, const int* __restrict__ src_token,
                                    const int* __restrict__ n_rows, uint8_t* __restrict__ dst_q, uint8_t* __restrict__ dst_sf,
                                    int row_bytes, int sf_bytes, int src_sf_ld, int dst_sf_ld, int src_rows, int* status) {
  pdl_launch(); pdl_wait();
  const int n = *n_rows;
  for (int c = blockIdx.x; c < n; c += gridDim.x) {
    const int t = src_token[c];
    if (t < 0 || t >= src_rows) { if (threadIdx.x == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, c); continue; }
    const uint4* sq = (const uint4*)(src_q + (size_t)t * row_bytes);
    uint4* dq = (uint4*)(dst_q + (size_t)c * row_bytes);
    for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) dq[i] = __ldcg(sq + i);
    if (sf_bytes) {
      const uint8_t* ss = src_sf + (size_t)t * src_sf_ld; uint8_t* ds = dst_sf + (size_t)c * dst_sf_ld;
      for (int i = threadIdx.x; i < sf_bytes / 4; i += blockDim.x) ((uint32_t*)ds)[i] = __ldcg((const uint32_t*)ss + i);
    }
  }
}

extern "C" int cuteafd_route_gather(const void* src_q, const void* src_sf, const int* src_token, const int* n_rows, void* dst_q, void* dst_sf,
                                    int row_bytes, int sf_bytes, int src_sf_ld, int dst_sf_ld, int src_rows, int rows_cap, int* status,
                                    cudaStream_t s) {
  CA_REQUIRE(row_bytes % 16 == 0 && sf_bytes % 4 == 0 && src_sf_ld % 4 == 0 && dst_sf_ld % 4 == 0, "route_gather: rows are 16-byte, scales 4-byte multiples");
  CA_REQUIRE(((uintptr_t)src_q & 15) == 0 && ((uintptr_t)dst_q & 15) == 0, "route_gather: 16-byte aligned payloads");
  if (rows_cap <= 0) return CA_OK;
  const int blocks = rows_cap < 592 ? rows_cap : 592;
  CA_LAUNCH_PDL(route_gather_kernel, blocks, 128, 0, s, (const uint8_t*)src_q, (const uint8_t*)src_sf, src_token, n_rows, (uint8_t*)dst_q,
                (uint8_t*)dst_sf, row_bytes, sf_bytes, src_sf_ld, dst_sf_ld, src_rows, status);
  return CA_OK;
}

// Hash routing (layers whose experts are a fixed function of the token id): expert ids come from tid2eid[token][0..k), gate
// weights are the sqrt-softplus scores of the logits at those experts, normalised over the k and scaled.  One warp per token.
__global__ void router_hash_select_kernel(const float* __restrict__ logits, const int* __restrict__ tid2eid, const int* __restrict__ tokens,
                                          int* __restrict__ idx, float* __restrict__ wts, int T, int E, int k, int vocab, float route_scale,
                                          int* status) {
  pdl_launch(); pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) { if (lane == 0) ca_dev_fail(status, CA_DEV_BAD_INDEX, t); tok = 0; }
  int e = 0; float sc = 0.f;
  if (lane < k) {
    e = tid2eid[(size_t)tok * k + lane];
    if (e < 0 || e >= E) { ca_dev_fail(status, CA_DEV_BAD_INDEX, t); e = 0; }
    const float x = logits[(size_t)t * E + e];
    sc = sqrtf(x > 20.f ? x : log1pf(expf(x)));
  }
  float tot = sc;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
  if (lane < k) { idx[(size_t)t * k + lane] = e; wts[(size_t)t * k + lane] = sc / (tot + 1e-20f) * route_scale; }
}

extern "C" int cuteafd_router_hash_select(const float* logits, const int* tid2eid, const int* tokens, int* idx, float* wts, int T, int E, int k,
                                          int vocab, float route_scale, int* status, cudaStream_t s) {
  CA_REQUIRE(k >= 1 && k <= 32 && E >= k && vocab >= 1, "router_hash_select: 1 <= k <= 32 <= E");
  if (T <= 0) return CA_OK;
  CA_LAUNCH_PDL(router_hash_select_kernel, (T + 3) / 4, 128, 0, s, logits, tid2eid, tokens, idx, wts, T, E, k, vocab, route_scale, status);
  return CA_OK;
}

// ---------------------------------------------------------------- whole router in one launch (decode / verify steps)
// logits -> selection -> route packing used to be two launches around a [T, E] fp32 round trip; on a decode step both are
// launch-latency sized.  Here one block per expert (512 threads: one 16-byte weight chunk per thread at H = 4096) computes that
// expert's logit for every token; the block that arrives last at the ticket then selects with one warp per token (scores in that
// warp's slice of shared memory) and packs the routes with the whole block.
#define RF_THREADS 512
#define RF_WARPS (RF_THREADS / 32)

// One warp, one token: scores, optional group-limited routing, k rounds of argmax (value desc, expert id asc), gate weights.
template <int NQ>       // logits per lane: E <= 32 * NQ (short, straight code: this runs once per launch from a cold instruction cache)
__device__ __forceinline__ void router_select_warp(const float* lg, const float* __restrict__ bias, float* score, float* choice, int E, int k,
                                                   int scoring, int normalize, float route_scale, int n_group, int topk_group,
                                                   int* idx_out, float* wts_out, int* sel_sh = nullptr) {
  const int lane = threadIdx.x & 31;
  float lv[NQ];                                 // this lane's logits, one trip to L2 for all of them
#pragma unroll
  for (int q = 0; q < NQ; ++q) lv[q] = (lane + 32 * q < E) ? __ldcg(lg + lane + 32 * q) : -INFINITY;
  float mx = -INFINITY;
#pragma unroll
  for (int q = 0; q < NQ; ++q) mx = fmaxf(mx, lv[q]);
  float denom = 1.f;
  if (scoring == SCORE_SOFTMAX) {
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < NQ; ++q) if (lane + 32 * q < E) s += expf(lv[q] - mx);
    denom = warp_sum(s);
  }
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    const int e = lane + 32 * q;
    if (e >= E) continue;
    const float x = lv[q];
    float sc;
    if (scoring == SCORE_SIGMOID) sc = 1.f / (1.f + expf(-x));
    else if (scoring == SCORE_SOFTMAX) sc = expf(x - mx) / denom;
    else sc = sqrtf(x > 20.f ? x : log1pf(expf(x)));
    score[e] = sc;
    choice[e] = sc + (bias ? bias[e] : 0.f);
  }
  __syncwarp();
  if (n_group > 1 && topk_group < n_group) {
    const int per = E / n_group;
    float gs = -INFINITY;                       // lane g: sum of the two best biased scores of group g
    if (lane < n_group) {
      float a = -INFINITY, b = -INFINITY;
      for (int j = 0; j < per; ++j) { const float v = choice[lane * per + j]; if (v > a) { b = a; a = v; } else if (v > b) b = v; }
      gs = a + b;
    }
    unsigned keep = 0;
    for (int r = 0; r < topk_group; ++r) {      // best groups first, lowest group id among equals
      float bv = (lane < n_group && !(keep >> lane & 1)) ? gs : -INFINITY;
      int bi = (lane < n_group && !(keep >> lane & 1)) ? lane : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
      }
      if (bi != 0x7fffffff) keep |= 1u << bi;
    }
    for (int e = lane; e < E; e += 32) if (!(keep >> (e / per) & 1)) choice[e] = -INFINITY;
    __syncwarp();
  }
  float wsum = 0.f, myw = 0.f; int mye = 0;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) { const float v = choice[e]; if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi >= E) bi = 0;
    const float w = score[bi];
    wsum += w;
    if (lane == r) { mye = bi; myw = w; }
    __syncwarp();
    if (lane == 0) choice[bi] = -INFINITY;
    __syncwarp();
  }
  const float inv = normalize ? 1.f / fmaxf(wsum, 1e-12f) : 1.f;
  if (lane < k) { idx_out[lane] = mye; wts_out[lane] = myw * inv * route_scale; if (sel_sh) sel_sh[lane] = mye; }
}

__global__ void __launch_bounds__(RF_THREADS) router_fused_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, float* __restrict__ logits,
                                                                  const float* __restrict__ bias, int* __restrict__ idx, float* __restrict__ wts,
                                                                  int T, int E, int H, int k, int scoring, int normalize, float route_scale,
                                                                  int n_group, int topk_group, const RoutePack pack, int do_pack) {
  pdl_launch(); pdl_wait();
  extern __shared__ int rf_sh[];                       // select: [warps][2][E] floats; pack: route_pack_smem ints (the larger of the two)
  __shared__ float red[RL_TOK][RF_WARPS];
  __shared__ int is_last;
  const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bf16* wr = w + (size_t)e * H;
  for (int t0 = 0; t0 < T; t0 += RL_TOK) {
    float acc[RL_TOK];
#pragma unroll
    for (int j = 0; j < RL_TOK; ++j) acc[j] = 0.f;
    for (int c = tid; c < H / 8; c += RF_THREADS) {
      const uint4 wv = *(const uint4*)(wr + c * 8);
      const bf162* wp = (const bf162*)&wv;
      float wf[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(wp[q]); wf[2 * q] = f.x; wf[2 * q + 1] = f.y; }
#pragma unroll
      for (int j = 0; j < RL_TOK; ++j) {
        if (t0 + j < T) {
          const uint4 xv = *(const uint4*)(x + (size_t)(t0 + j) * H + c * 8);
          const bf162* xp = (const bf162*)&xv;
#pragma unroll
          for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(xp[q]); acc[j] = fmaf(f.x, wf[2 * q], acc[j]); acc[j] = fmaf(f.y, wf[2 * q + 1], acc[j]); }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < RL_TOK; ++j) {
      const float v = warp_sum(acc[j]);
      if (lane == 0) red[j][warp] = v;
    }
    __syncthreads();
    if (tid < RL_TOK && t0 + tid < T) {
      float v = 0.f;
#pragma unroll
      for (int q = 0; q < RF_WARPS; ++q) v += red[tid][q];
      logits[(size_t)(t0 + tid) * E + e] = v;
    }
    __syncthreads();
  }
  // the block that arrives last sees every expert's logits
  if (tid == 0) {
    __threadfence();
    is_last = (atomicAdd(pack.ticket, 1) == (int)gridDim.x - 1);
    __threadfence();
  }
  __syncthreads();
  if (!is_last) return;
  float* sc = (float*)rf_sh + (size_t)warp * 2 * E;
  for (int t = warp; t < T; t += RF_WARPS)
    router_select_warp<16>(logits + (size_t)t * E, bias, sc, sc + E, E, k, scoring, normalize, route_scale, n_group, topk_group, idx + (size_t)t * k,
                           wts + (size_t)t * k);
  __syncthreads();                                     // idx is complete (block-scope visibility is enough: the same block packs)
  if (do_pack) route_pack_body(pack, rf_sh);
  if (tid == 0) *pack.ticket = 0;
}

// logits [T, E] fp32 are still written (tracing, tests).  `src_token == null` skips the packing (attention ranks of a multi-GPU
// layout select only: their experts live elsewhere).
extern "C" int cuteafd_router_fused(const void* x, const void* w, float* logits, const float* bias, int* idx, float* wts, int T, int E, int H, int k,
                                    int scoring, int normalize, float route_scale, int n_group, int topk_group, int* src_token, int* slot_row,
                                    int* counts, int* offsets, void* tiles, int* n_tiles, int* n_rows, int e_lo, int e_hi, int tn, int max_tiles,
                                    int* src_route, int* ticket, cudaStream_t s) {
  CA_REQUIRE(x && w && logits && idx && wts && ticket, "router_fused: null argument");
  CA_REQUIRE(H % 8 == 0 && E >= k && E <= 512 && k >= 1 && k <= 16, "router_fused: need hidden %% 8 == 0, k <= 16 and E <= 512 (E=%d k=%d)", E, k);
  CA_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0, "router_fused: bad group count");
  const int do_pack = src_token != nullptr;
  CA_REQUIRE(!do_pack || (e_hi > e_lo && e_hi - e_lo <= 512 && tn >= 1 && T * k <= 4096), "router_fused: bad pack arguments");
  if (T <= 0) return CA_OK;
  RoutePack p{idx, src_token, slot_row, counts, offsets, (int4*)tiles, n_tiles, n_rows, src_route, T, k, e_lo, e_hi, tn, max_tiles, ticket,
              FlagWait{nullptr, nullptr, nullptr, 0ull, 0, 0}, nullptr, 0};
  size_t smem = (size_t)RF_WARPS * 2 * E * sizeof(float);
  if (do_pack && route_pack_smem(T, k, e_lo, e_hi) > smem) smem = route_pack_smem(T, k, e_lo, e_hi);
  CA_REQUIRE(smem <= 96 * 1024, "router_fused: too many routes for one block");
  if (smem > 48 * 1024) {
    cudaError_t ce = cudaFuncSetAttribute(router_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (ce != cudaSuccess) return ca_cuda(ce, "router_fused: shared memory size");
  }
  CA_LAUNCH_PDL(router_fused_kernel, E, RF_THREADS, smem, s, (const bf16*)x, (const bf16*)w, logits, bias, idx, wts, T, E, H, k, scoring, normalize,
                route_scale, n_group, topk_group, p, do_pack);
  CA_CHECK_LAUNCH("router_fused");
  return CA_OK;
}

// Selection and packing of a decode-sized step by ONE block: a warp per token selects from the logits (no block barriers, no
// arrival counter, no fences), the chosen experts stay in shared memory and the same block packs them - the chain is one round
// trip to L2 for the logits instead of logits -> selections -> counter -> selections read back twice.
template <int NQ>
__global__ void __launch_bounds__(RF_THREADS) router_select_block_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                                         int* __restrict__ idx, float* __restrict__ wts, int T, int E, int k,
                                                                         int scoring, int normalize, float route_scale, int n_group,
                                                                         int topk_group, const RoutePack pack) {
  pdl_launch(); pdl_wait();
  extern __shared__ int rs_sh[];                       // [T * k] chosen experts | [warps][2][E] scores | route-pack scratch
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* ids = rs_sh;
  float* sc = (float*)(rs_sh + T * k) + (size_t)warp * 2 * E;
  for (int t = warp; t < T; t += RF_WARPS) {
    router_select_warp<NQ>(logits + (size_t)t * E, bias, sc, sc + E, E, k, scoring, normalize, route_scale, n_group, topk_group, idx + (size_t)t * k,
                           wts + (size_t)t * k, ids + t * k);
    __syncwarp();
  }
  __syncthreads();
  route_pack_body(pack, rs_sh + T * k + RF_WARPS * 2 * E, ids);
}

// Selection only, the same warp-per-token arithmetic (ranks of a multi-GPU layout whose experts live elsewhere must pick exactly
// what the single-GPU engine picks): four tokens per block.
template <int NQ>
__global__ void __launch_bounds__(128) router_select_warps_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ idx,
                                                                  float* __restrict__ wts, int T, int E, int k, int scoring, int normalize,
                                                                  float route_scale, int n_group, int topk_group) {
  pdl_launch(); pdl_wait();
  extern __shared__ int rs_sh[];
  const int warp = threadIdx.x >> 5, t = blockIdx.x * 4 + warp;
  if (t >= T) return;
  float* sc = (float*)rs_sh + (size_t)warp * 2 * E;
  router_select_warp<NQ>(logits + (size_t)t * E, bias, sc, sc + E, E, k, scoring, normalize, route_scale, n_group, topk_group, idx + (size_t)t * k,
                         wts + (size_t)t * k);
}

static int launch_router_select_warps(const float* logits, const float* bias, int* idx, float* wts, int T, int E, int k, int scoring, int normalize,
                                      float route_scale, int n_group, int topk_group, cudaStream_t s) {
#define CA_RSW(NQ) CA_LAUNCH_PDL(router_select_warps_kernel<NQ>, (T + 3) / 4, 128, (size_t)4 * 2 * E * sizeof(float), s, logits, bias, idx, wts, T, E, k, \
                                 scoring, normalize, route_scale, n_group, topk_group)
  if (E <= 128) CA_RSW(4); else if (E <= 256) CA_RSW(8); else CA_RSW(16);
#undef CA_RSW
  CA_CHECK_LAUNCH("router_select_warps");
  return CA_OK;
}

// Router selection and route packing in one launch: the select block that finishes last packs the routes.
extern "C" int cuteafd_router_select_pack(const float* logits, const float* bias, int* idx, float* wts, int T, int E, int k,
                                          int scoring, int normalize, float route_scale, int n_group, int topk_group,
                                          int* src_token, int* slot_row, int* counts, int* offsets, void* tiles, int* n_tiles,
                                          int* n_rows, int e_lo, int e_hi, int tn, int max_tiles, int* src_route, int* ticket,
                                          cudaStream_t s) {
  CA_REQUIRE(E >= k && E <= 512 && k >= 1 && k <= 16, "router_select: need k <= 16 and E <= 512 (E=%d k=%d)", E, k);
  CA_REQUIRE(n_group >= 1 && n_group <= 32 && E % n_group == 0, "router_select: bad group count");
  CA_REQUIRE(e_hi > e_lo && e_hi - e_lo <= 512 && tn >= 1 && ticket, "router_select_pack: bad pack arguments");
  if (T <= 0) return CA_OK;
  const int threads = E <= 64 ? 64 : (E <= 128 ? 128 : 256);
  RoutePack p{idx, src_token, slot_row, counts, offsets, (int4*)tiles, n_tiles, n_rows, src_route, T, k, e_lo, e_hi, tn, max_tiles, ticket,
              FlagWait{nullptr, nullptr, nullptr, 0ull, 0, 0}, nullptr, 0};
  if (T <= 64) {      // decode / verify steps: one block selects (a warp per token) and packs from shared memory
    const size_t smem = ((size_t)T * k + (size_t)RF_WARPS * 2 * E) * 4 + route_pack_smem(T, k, e_lo, e_hi);
    if (smem <= 96 * 1024) {
      p.ticket = nullptr;
#define CA_RSB(NQ) do {                                                                                                                              \
        if (smem > 48 * 1024) {                                                                                                                      \
          cudaError_t ce = cudaFuncSetAttribute(router_select_block_kernel<NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);             \
          if (ce != cudaSuccess) return ca_cuda(ce, "router_select_pack: shared memory size");                                                       \
        }                                                                                                                                            \
        CA_LAUNCH_PDL(router_select_block_kernel<NQ>, 1, RF_THREADS, smem, s, logits, bias, idx, wts, T, E, k, scoring, normalize, route_scale,      \
                      n_group, topk_group, p);                                                                                                       \
      } while (0)
      if (E <= 128) CA_RSB(4); else if (E <= 256) CA_RSB(8); else CA_RSB(16);
#undef CA_RSB
      CA_CHECK_LAUNCH("router_select_block");
      return CA_OK;
    }
  }
  CA_LAUNCH_PDL(router_select_kernel, T, threads, route_pack_smem(T, k, e_lo, e_hi), s, logits, bias, idx, wts, E, k, scoring, normalize, route_scale,
                n_group, topk_group, p);
  return CA_OK;
}

// acc[0..8) += sum over the token's routes (slot order) of w * y[row][i .. i+8).  The routes are taken eight at a time: their row
// numbers and weights first, then all eight rows in flight together - a loop that looks up one route, then loads its row, is a
// chain of 2 k dependent round trips to L2 (about 10 us of the decode step's combine at k = 8).
__device__ __forceinline__ void combine_routes8(const bf16* __restrict__ y, const int* __restrict__ rows, const float* __restrict__ wts, int k, int H,
                                                int i, float* acc) {
  for (int s0 = 0; s0 < k; s0 += 8) {
    int r[8]; float w[8]; uint4 qv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { r[j] = (s0 + j < k) ? rows[s0 + j] : -1; w[j] = (s0 + j < k) ? wts[s0 + j] : 0.f; }
#pragma unroll
    for (int j = 0; j < 8; ++j) qv[j] = (r[j] >= 0) ? *(const uint4*)(y + (size_t)r[j] * H + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (r[j] >= 0) {
        const bf16* e = (const bf16*)&qv[j];
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += w[j] * __bfloat162float(e[q]);
      }
    }
  }
}

// ---------------------------------------------------------------- ordered weighted combine
// out[t] = residual[t] + shared[t] + sum_{slot} w[t,slot] * y[slot_row[t,slot]]   (fp32, slot order, one rounding).
// residual / shared may be null; routes with slot_row < 0 are skipped.
__global__ void moe_combine_kernel(const bf16* __restrict__ y, const int* __restrict__ slot_row, const float* __restrict__ wts,
                                   const bf16* __restrict__ shared, const bf16* __restrict__ residual, bf16* __restrict__ out,
                                   int H, int k, const FlagWait fw) {
  pdl_launch(); pdl_wait();
  if (!flag_wait_block(fw)) return;
  const int t = blockIdx.x;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < H; i += gridDim.y * blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    combine_routes8(y, slot_row + (size_t)t * k, wts + (size_t)t * k, k, H, i, acc);
    if (shared) { uint4 q = *(const uint4*)(shared + (size_t)t * H + i); const bf16* e = (const bf16*)&q;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(e[j]); }
    if (residual) { uint4 q = *(const uint4*)(residual + (size_t)t * H + i); const bf16* e = (const bf16*)&q;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(e[j]); }
    bf16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16(acc[j]);
    *(uint4*)(out + (size_t)t * H + i) = *(uint4*)o;
  }
}

// Combine fused with the NEXT layer's input norm: one block per token holds the whole row in registers, writes
// the new residual stream `out`, then rmsnorm(out) * norm_w as bf16 (`xn`, optional) and/or quantised to FP4
// (`q`/`sf`, optional) - three launches (combine, norm, quantise) in one for decode-sized steps.
template <int VEC>
__global__ void moe_combine_norm_kernel(const bf16* __restrict__ y, const int* __restrict__ slot_row, const float* __restrict__ wts,
                                        const bf16* __restrict__ shared, const bf16* __restrict__ residual, bf16* __restrict__ out,
                                        int H, int k, const float* __restrict__ norm_w, float eps, bf16* __restrict__ xn,
                                        uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int ldsf,
                                        const float* __restrict__ inv_gs_ptr, int qkind, const FlagWait fw) {
  pdl_launch(); pdl_wait();
  __shared__ float red[32];
  if (!flag_wait_block(fw)) return;
  const int t = blockIdx.x;
  float v[VEC * 8];
  float4 nw[VEC * 2];                 // the norm weights of this thread's elements, fetched with the rows (not after the reduction)
  float ss = 0.f;
  const float inv_gs = (qkind == 1 && inv_gs_ptr) ? *inv_gs_ptr : 1.f;
#pragma unroll
  for (int kk = 0; kk < VEC; ++kk) {
    const int i = (threadIdx.x + kk * blockDim.x) * 8;
    nw[2 * kk] = nw[2 * kk + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < H) {
      nw[2 * kk] = *(const float4*)(norm_w + i); nw[2 * kk + 1] = *(const float4*)(norm_w + i + 4);
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      combine_routes8(y, slot_row + (size_t)t * k, wts + (size_t)t * k, k, H, i, acc);
      if (shared) { uint4 qv = *(const uint4*)(shared + (size_t)t * H + i); const bf16* e = (const bf16*)&qv;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(e[j]); }
      if (residual) { uint4 qv = *(const uint4*)(residual + (size_t)t * H + i); const bf16* e = (const bf16*)&qv;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(e[j]); }
      bf16 o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = __float2bfloat16(acc[j]); v[kk * 8 + j] = __bfloat162float(o[j]); ss += v[kk * 8 + j] * v[kk * 8 + j]; }
      *(uint4*)(out + (size_t)t * H + i) = *(uint4*)o;
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / H + eps);
#pragma unroll
  for (int kk = 0; kk < VEC; ++kk) {
    const int i = (threadIdx.x + kk * blockDim.x) * 8;
    if (i < H) {
      bf16 o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16(v[kk * 8 + j] * inv * ((const float*)&nw[2 * kk])[j]);
      if (xn) *(uint4*)(xn + (size_t)t * H + i) = *(uint4*)o;
      if (qkind) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(o[j]);
        if (qkind == 3) quant8_store_fp8b(f, q + (size_t)t * H, (float*)sf + (size_t)t * ldsf, i);
        else quant8_store(f, qkind, qkind == 1 ? inv_gs : (inv_gs_ptr ? *inv_gs_ptr : 1.f), q + (size_t)t * (H / 2), sf + (size_t)t * ldsf, i);
      }
    }
  }
}

extern "C" int cuteafd_moe_combine_norm(const void* y, const int* slot_row, const float* wts, const void* shared, const void* residual,
                                        void* out, int T, int H, int k, const float* norm_w, float eps, void* xn, void* q, void* sf,
                                        int ldsf, const float* inv_gs, int qkind, const CaFlagWaitArg* wait, cudaStream_t s) {
  const FlagWait fw = ca_flag_wait_from(wait);
  CA_REQUIRE(H % 8 == 0 && H <= 32768 && norm_w && ((uintptr_t)norm_w & 15) == 0, "moe_combine_norm: bad arguments (hidden %% 8, 16-byte aligned norm weights)");
  CA_REQUIRE(qkind == 0 || (qkind >= 1 && qkind <= 3 && q && sf && H % 256 == 0), "moe_combine_norm: quantised output needs buffers and hidden %% 256 == 0");
  if (T <= 0) return CA_OK;
  const int vecs = H / 8;
  int threads = vecs >= 1024 ? 1024 : ((vecs + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  const int per = (vecs + threads - 1) / threads;
#define CA_CN(V) CA_LAUNCH_PDL(moe_combine_norm_kernel<V>, T, threads, 0, s, (const bf16*)y, slot_row, wts, (const bf16*)shared, (const bf16*)residual, \
                               (bf16*)out, H, k, norm_w, eps, (bf16*)xn, (uint8_t*)q, (uint8_t*)sf, ldsf, inv_gs, qkind, fw)
  if (per == 1) CA_CN(1); else if (per == 2) CA_CN(2); else CA_CN(4);
#undef CA_CN
  return CA_OK;
}

extern "C" int cuteafd_moe_combine(const void* y, const int* slot_row, const float* wts, const void* shared, const void* residual,
                                   void* out, int T, int H, int k, const CaFlagWaitArg* wait, cudaStream_t s) {
  const FlagWait fw = ca_flag_wait_from(wait);
  CA_REQUIRE(H % 8 == 0, "moe_combine: hidden must be a multiple of 8");
  if (T <= 0) return CA_OK;
  const int threads = H / 8 >= 256 ? 256 : (H / 8 >= 128 ? 128 : 64);
  // few tokens: split the row over several blocks so more SMs pull the k routed rows
  const int ysplit = T >= 64 ? 1 : (H / 8 + threads - 1) / threads;
  CA_LAUNCH_PDL(moe_combine_kernel, dim3(T, ysplit), threads, 0, s, (const bf16*)y, slot_row, wts, (const bf16*)shared, (const bf16*)residual, (bf16*)out, H, k, fw);
  CA_CHECK_LAUNCH("moe_combine");
  return CA_OK;
}
