// NVLink peer-memory primitives and the fused communication kernels of the attention/expert split.
//
// Ranks of one node exchange device pointers to "symmetric" buffers (CUDA IPC); kernels then read and write
// peer memory directly with ordinary loads/stores (NVLink through NVSwitch) and signal with 32-bit sequence
// flags: the writer stores its payload, fences at system scope, then `st.release.sys` the step number; the
// reader spins on `ld.acquire.sys` until the flag reaches the step it expects.  Every spin is bounded: when the
// limit runs out the kernel records CA_DEV_TIMEOUT_FLAG in a status word, publishes an abort word so later
// kernels of the step fall through, and returns.  Nothing traps.
//
//   dispatch_push   attention rank -> expert ranks: quantise each token row once (NVFP4 / MXFP4 / bf16) and store it
//                   into the slab of every expert rank that owns one of its top-k experts, at the row the (replicated,
//                   deterministic) route packing assigned; then release one flag per destination.
//   combine_push    expert rank -> attention ranks: store each expert-output row into [token][slot] of every attention
//                   rank's receive buffer; release one flag per destination.
//   wait_flags      bounded wait for a set of flags (used in front of the grouped GEMM and of the ordered combine).
//   push_add        TP2 all-reduce for attention / shared-expert partials: push my partial to the peer, wait for the
//                   peer's, add in rank order (bit-identical on both ranks).
//
// Reference counterparts: native/shared/cuda/peer_exchange.cu:66-259 (push_signal, wait_flag, abortable waits,
// add_bf16), residual.cu:170-296 + 419-498 (quantise-on-dispatch, scatter-add on combine),
// rust/crates/cuteafd-daemon/src/shared/peer_split.rs:30-84 (slots, sequence numbers, terminal state).
#include <string.h>

#include "common.cuh"

#define MAX_PEERS 8

struct PeerPtrs { void* p[MAX_PEERS]; };

// ---------------------------------------------------------------- IPC plumbing (host)
extern "C" int cuteafd_ipc_export(const void* ptr, void* handle64, unsigned long long* offset) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (e != cudaSuccess) return ca_cuda(e, "cudaIpcGetMemHandle");
  memcpy(handle64, &h, sizeof(h));
  // offset of ptr inside its allocation: cudaIpcOpenMemHandle returns the allocation base on the peer
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (RangeFn)p;
  }
  if (!fn) return ca_fail(CA_ERR_CUDA, "cuMemGetAddressRange unavailable");
  CUdeviceptr base = 0; size_t size = 0;
  CUresult r = fn(&base, &size, (CUdeviceptr)ptr);
  if (r != CUDA_SUCCESS) return ca_fail(CA_ERR_CUDA, "cuMemGetAddressRange failed (%d)", (int)r);
  *offset = (unsigned long long)((CUdeviceptr)ptr - base);
  return CA_OK;
}

extern "C" int cuteafd_ipc_open(const void* handle64, unsigned long long offset, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* base = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return ca_cuda(e, "cudaIpcOpenMemHandle");
  *out = (char*)base + offset;
  return CA_OK;
}

extern "C" int cuteafd_ipc_close(void* ptr, unsigned long long offset) {
  cudaError_t e = cudaIpcCloseMemHandle((char*)ptr - offset);
  if (e != cudaSuccess) return ca_cuda(e, "cudaIpcCloseMemHandle");
  return CA_OK;
}

// ---------------------------------------------------------------- flags
// ctl[0] = abort word (non-zero: a wait of this step already gave up), ctl[1] = current step number (device-side
// counter so captured graphs see a fresh value each replay).
__global__ void step_begin_kernel(uint32_t* ctl) { ctl[1] += 1; ctl[0] = 0; }

extern "C" int cuteafd_step_begin(void* ctl, cudaStream_t s) {
  step_begin_kernel<<<1, 1, 0, s>>>((uint32_t*)ctl);
  CA_CHECK_LAUNCH("step_begin");
  return CA_OK;
}

// Wait until flags[i * stride] >= step for every i in [0, n).  One thread per flag.
__global__ void wait_flags_kernel(const uint32_t* flags, int n, int stride, uint32_t* ctl, uint32_t step_offset,
                                  unsigned long long timeout_ns, int* status) {
  const int i = threadIdx.x;
  if (i >= n) return;
  if (ctl[0]) return;
  const uint32_t want = ctl[1] + step_offset;
  if (!wait_flag_bounded(flags + (size_t)i * stride, want, timeout_ns)) {
    ca_dev_fail(status, CA_DEV_TIMEOUT_FLAG, i);
    atomicExch(&ctl[0], 1u);
  }
}

extern "C" int cuteafd_wait_flags(const void* flags, int n, int stride, void* ctl, unsigned step_offset,
                                  unsigned long long timeout_ns, int* status, cudaStream_t s) {
  CA_REQUIRE(n >= 1 && n <= 32, "wait_flags: 1..32 flags");
  wait_flags_kernel<<<1, 32, 0, s>>>((const uint32_t*)flags, n, stride, (uint32_t*)ctl, step_offset, timeout_ns, status);
  CA_CHECK_LAUNCH("wait_flags");
  return CA_OK;
}

// Last-block-publishes helper: every block calls it after its stores; the last one to arrive releases `n_dst`
// flags (flag pointers are peer addresses) with the current step number, then resets the counter.
__device__ __forceinline__ void publish_when_last(uint32_t* done_counter, uint32_t* const* flag_ptrs, int n_dst,
                                                  uint32_t value) {
  // Every block: barrier (orders the block's stores before thread 0), a GPU-scope fence, then the arrival count.  The LAST
  // block: one system-scope fence, which is cumulative over everything it observed through the counter (all blocks'
  // stores), then relaxed system-scope stores of the flags.  Measured on B200 with 148 blocks and eight flags: 4 us, against
  // 22 us for a system-scope fence per block plus a release store per flag (each release repeats the fence, in series) and
  // 8 us with per-block system-scope fences.  The same shape as a block barrier followed by one thread's fence + flag
  // store, with the counter in the barrier's place.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x * gridDim.y - 1) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      for (int d = 0; d < n_dst; ++d) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flag_ptrs[d]), "r"(value) : "memory");
      *done_counter = 0;
    }
  }
}

struct FlagPtrs { uint32_t* p[MAX_PEERS]; };

// ---------------------------------------------------------------- generic push (+ flag)
__global__ void push_bytes_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16, FlagPtrs flags, int n_dst,
                                  uint32_t* ctl, uint32_t step_offset, uint32_t* done_counter) {
  if (!ctl[0])
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
  publish_when_last(done_counter, flags.p, n_dst, ctl[1] + step_offset);
}

extern "C" int cuteafd_push_bytes(const void* src, void* peer_dst, size_t bytes, void* peer_flag, void* ctl, unsigned step_offset,
                                  void* done_counter, cudaStream_t s) {
  CA_REQUIRE(bytes % 16 == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)peer_dst & 15) == 0, "push_bytes: 16-byte alignment");
  FlagPtrs f; f.p[0] = (uint32_t*)peer_flag;
  const size_t n16 = bytes / 16;
  int blocks = (int)((n16 + 255) / 256); if (blocks > 32) blocks = 32; if (blocks < 1) blocks = 1;
  push_bytes_kernel<<<blocks, 256, 0, s>>>((const uint4*)src, (uint4*)peer_dst, n16, f, 1, (uint32_t*)ctl, step_offset, (uint32_t*)done_counter);
  CA_CHECK_LAUNCH("push_bytes");
  return CA_OK;
}

// ---------------------------------------------------------------- TP2 all-reduce: push partial, wait, add in rank order
// out = (residual) + partial[rank 0] + partial[rank 1]; `mine` is this rank's partial (local), `theirs` the landing
// buffer the peer pushes into.  Launch order per rank: push_bytes(mine -> peer.theirs) ; this kernel.
__global__ void wait_add_kernel(const bf16* __restrict__ mine, const bf16* __restrict__ theirs, const bf16* __restrict__ residual,
                                bf16* __restrict__ out, size_t n8, int my_rank, const uint32_t* flag, uint32_t* ctl,
                                uint32_t step_offset, unsigned long long timeout_ns, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    if (ctl[0]) ok = 0;
    else if (!wait_flag_bounded(flag, ctl[1] + step_offset, timeout_ns)) { ca_dev_fail(status, CA_DEV_TIMEOUT_FLAG, 100 + my_rank); atomicExch(&ctl[0], 1u); ok = 0; }
  }
  __syncthreads();
  if (!ok) return;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    uint4 a = ((const uint4*)mine)[i], b = __ldcv(((const uint4*)theirs) + i);
    const bf16* first = (const bf16*)(my_rank == 0 ? &a : &b);
    const bf16* second = (const bf16*)(my_rank == 0 ? &b : &a);
    uint4 r = make_uint4(0, 0, 0, 0);
    if (residual) r = ((const uint4*)residual)[i];
    const bf16* re = (const bf16*)&r;
    bf16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = __bfloat162float(first[j]) + __bfloat162float(second[j]);   // same operand order on both ranks
      if (residual) v += __bfloat162float(re[j]);
      o[j] = __float2bfloat16(v);
    }
    ((uint4*)out)[i] = *(uint4*)o;
  }
}

extern "C" int cuteafd_wait_add(const void* mine, const void* theirs, const void* residual, void* out, size_t elems, int my_rank,
                                const void* flag, void* ctl, unsigned step_offset, unsigned long long timeout_ns, int* status,
                                cudaStream_t s) {
  CA_REQUIRE(elems % 8 == 0, "wait_add: element count must be a multiple of 8");
  const size_t n8 = elems / 8;
  int blocks = (int)((n8 + 255) / 256); if (blocks > 296) blocks = 296; if (blocks < 1) blocks = 1;
  wait_add_kernel<<<blocks, 256, 0, s>>>((const bf16*)mine, (const bf16*)theirs, (const bf16*)residual, (bf16*)out, n8, my_rank,
                                          (const uint32_t*)flag, (uint32_t*)ctl, step_offset, timeout_ns, status);
  CA_CHECK_LAUNCH("wait_add");
  return CA_OK;
}

// ---------------------------------------------------------------- vocabulary-parallel LM head on a TP pair
// Each rank multiplies the logit rows by ITS share of the vocabulary into a contiguous staging buffer and pushes it to the partner
// (push_bytes); this kernel waits for the partner's share and writes the full rows out[r] = [share of rank 0 | share of rank 1],
// so selection and sampling run on complete rows and both ranks hold the same bits.  Widths in float4 units.
__global__ void wait_concat_kernel(const float4* __restrict__ mine, const float4* __restrict__ theirs, float4* __restrict__ out, int n_rows,
                                   int w0, int w1, int my_rank, const uint32_t* flag, uint32_t* ctl, uint32_t step_offset,
                                   unsigned long long timeout_ns, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    if (ctl[0]) ok = 0;
    else if (!wait_flag_bounded(flag, ctl[1] + step_offset, timeout_ns)) { ca_dev_fail(status, CA_DEV_TIMEOUT_FLAG, 200 + my_rank); atomicExch(&ctl[0], 1u); ok = 0; }
  }
  __syncthreads();
  if (!ok) return;
  const int W = w0 + w1;
  const float4* first = my_rank == 0 ? mine : theirs;
  const float4* second = my_rank == 0 ? theirs : mine;
  const size_t n = (size_t)n_rows * W;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / W), c = (int)(i % W);
    const float4* src = c < w0 ? first + (size_t)r * w0 + c : second + (size_t)r * w1 + (c - w0);
    const bool remote = (c < w0) != (my_rank == 0);
    out[i] = remote ? __ldcv(src) : *src;
  }
}

extern "C" int cuteafd_wait_concat(const void* mine, const void* theirs, void* out, int n_rows, int w0, int w1, int my_rank, const void* flag,
                                   void* ctl, unsigned step_offset, unsigned long long timeout_ns, int* status, cudaStream_t s) {
  CA_REQUIRE(mine && theirs && out && flag && ctl && w0 > 0 && w1 > 0 && w0 % 4 == 0 && w1 % 4 == 0 && (my_rank == 0 || my_rank == 1),
             "wait_concat: widths must be multiples of 4 floats");
  if (n_rows <= 0) return CA_OK;
  const size_t n = (size_t)n_rows * ((w0 + w1) / 4);
  int blocks = (int)((n + 255) / 256); if (blocks > 296) blocks = 296; if (blocks < 1) blocks = 1;
  wait_concat_kernel<<<blocks, 256, 0, s>>>((const float4*)mine, (const float4*)theirs, (float4*)out, n_rows, w0 / 4, w1 / 4, my_rank,
                                             (const uint32_t*)flag, (uint32_t*)ctl, step_offset, timeout_ns, status);
  CA_CHECK_LAUNCH("wait_concat");
  return CA_OK;
}

// ---------------------------------------------------------------- dispatch: quantise + scatter rows to expert ranks
// One block per (token of my share, route slot): the row is quantised into shared memory (FP4 payload + block scales,
// or kept bf16) and copied to the slab of the rank that owns this slot's expert, at row (slot_row - base of that
// rank's first expert).  Quantising per slot repeats a few KB of arithmetic k times but gives k times more blocks in
// flight, which is what bounds a decode-sized dispatch (one block per token took ~24 us for 64 tokens).
// kind: 0 bf16, 1 NVFP4, 2 MXFP4.
struct DispatchArgs {
  const bf16* x;            // [T, H] normalised activations (replicated on the attention ranks)
  const int* idx;           // [T, k] expert ids
  const int* slot_row;      // [T, k] packed row of each route in the GLOBAL expert-major order
  const int* offsets;       // [E] first packed row of each expert (global order)
  PeerPtrs slab_q;          // per expert rank: payload slab [rows_cap, row_bytes]
  PeerPtrs slab_sf;         // per expert rank: scale slab [rows_cap, sf_ld]
  PeerPtrs idx_dst;         // per expert rank: copy of the routing table [T, k] (each sender fills its tokens' rows)
  FlagPtrs flags;           // per expert rank: flag this attention rank releases
  const float* inv_gs;
  uint32_t* ctl; uint32_t* done_counter;
  int T0, T1, H, k, E_local /* total routed experts */, n_ep, kind, sf_ld, rows_cap;
  uint32_t step_offset;
  int* status;
};

__global__ void dispatch_push_kernel(const DispatchArgs a) {
  extern __shared__ uint8_t sh[];           // payload then scales
  const int t = a.T0 + blockIdx.x;
  const bool live = t < a.T1 && !a.ctl[0];
  const int H = a.H;
  const int row_bytes = a.kind == 0 ? H * 2 : H / 2;
  const int n_sf = a.kind == 0 ? 0 : (a.kind == 1 ? H / 16 : H / 32);
  uint8_t* pay = sh; uint8_t* sfs = sh + row_bytes;
  if (live) {
    const bf16* xr = a.x + (size_t)t * H;
    if (a.kind == 0) {
      for (int i = threadIdx.x; i < H / 8; i += blockDim.x) ((uint4*)pay)[i] = ((const uint4*)xr)[i];
    } else {
      const float inv_gs = (a.kind == 1 && a.inv_gs) ? *a.inv_gs : 1.f;
      for (int c = threadIdx.x; c < H / 16; c += blockDim.x) {
        uint4 q0 = ((const uint4*)xr)[2 * c], q1 = ((const uint4*)xr)[2 * c + 1];
        const bf16* e0 = (const bf16*)&q0; const bf16* e1 = (const bf16*)&q1;
        float v[16], amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[j] = __bfloat162float(e0[j]); v[8 + j] = __bfloat162float(e1[j]); }
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
        float eff; uint8_t sb;
        if (a.kind == 2) {
          amax = fmaxf(amax, __shfl_xor_sync(__activemask(), amax, 1));
          int e = amax > 0.f ? (int)((__float_as_uint(amax) >> 23) & 0xFF) - 2 : 0;
          e = max(e, 0); e = min(e, 254); sb = (uint8_t)e; eff = ue8m0_to_float(sb);
          if (!(c & 1)) sfs[c >> 1] = sb;
        } else {
          sb = float_to_e4m3(fminf(amax * inv_gs / 6.f, 448.f)); eff = e4m3_to_float(sb) / inv_gs;
          sfs[c] = sb;
        }
        const float inv = eff > 0.f ? 1.f / eff : 0.f;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) { lo |= float_to_e2m1(v[j] * inv) << (4 * j); hi |= float_to_e2m1(v[8 + j] * inv) << (4 * j); }
        ((uint2*)pay)[c] = make_uint2(lo, hi);
      }
    }
  }
  __syncthreads();
  if (live) {
    if (blockIdx.y == 0 && threadIdx.x < a.k)
      for (int d = 0; d < a.n_ep; ++d) ((int*)a.idx_dst.p[d])[(size_t)t * a.k + threadIdx.x] = a.idx[(size_t)t * a.k + threadIdx.x];
    for (int sl = blockIdx.y; sl < a.k; sl += gridDim.y) {
      const int e = a.idx[(size_t)t * a.k + sl];
      // expert ranks own contiguous, nearly equal ranges: rank o holds experts [o*E/n_ep, (o+1)*E/n_ep)
      int owner = -1;
      for (int o = 0; o < a.n_ep; ++o) if (e >= (o * a.E_local) / a.n_ep && e < ((o + 1) * a.E_local) / a.n_ep) owner = o;
      if (owner < 0 || owner >= a.n_ep) { if (threadIdx.x == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, t); continue; }
      const int row = a.slot_row[(size_t)t * a.k + sl] - a.offsets[(owner * a.E_local) / a.n_ep];
      if (row < 0 || row >= a.rows_cap) { if (threadIdx.x == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, t); continue; }
      uint4* dq = (uint4*)((uint8_t*)a.slab_q.p[owner] + (size_t)row * row_bytes);
      for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) dq[i] = ((const uint4*)pay)[i];
      if (n_sf) {
        uint8_t* ds = (uint8_t*)a.slab_sf.p[owner] + (size_t)row * a.sf_ld;
        for (int i = threadIdx.x; i < n_sf / 16; i += blockDim.x) ((uint4*)ds)[i] = ((const uint4*)sfs)[i];
        for (int i = (n_sf / 16) * 16 + threadIdx.x; i < n_sf; i += blockDim.x) ds[i] = sfs[i];
      }
    }
  }
  publish_when_last(a.done_counter, a.flags.p, a.n_ep, a.ctl[1] + a.step_offset);
}

extern "C" int cuteafd_dispatch_push(const void* x, const int* idx, const int* slot_row, const int* offsets, const void* const* slab_q,
                                     const void* const* slab_sf, const void* const* idx_dst, const void* const* flags, const float* inv_gs, void* ctl,
                                     void* done_counter, int T0, int T1, int H, int k, int E_local, int n_ep, int kind, int sf_ld,
                                     int rows_cap, unsigned step_offset, int* status, cudaStream_t s) {
  CA_REQUIRE(n_ep >= 1 && n_ep <= MAX_PEERS, "dispatch_push: 1..8 expert ranks");
  CA_REQUIRE(H % 256 == 0, "dispatch_push: hidden must be a multiple of 256");
  DispatchArgs a;
  a.x = (const bf16*)x; a.idx = idx; a.slot_row = slot_row; a.offsets = offsets; a.inv_gs = inv_gs;
  for (int i = 0; i < n_ep; ++i) { a.slab_q.p[i] = const_cast<void*>(slab_q[i]); a.slab_sf.p[i] = slab_sf ? const_cast<void*>(slab_sf[i]) : nullptr; a.idx_dst.p[i] = const_cast<void*>(idx_dst[i]); a.flags.p[i] = (uint32_t*)flags[i]; }
  a.ctl = (uint32_t*)ctl; a.done_counter = (uint32_t*)done_counter; a.T0 = T0; a.T1 = T1; a.H = H; a.k = k; a.E_local = E_local;
  a.n_ep = n_ep; a.kind = kind; a.sf_ld = sf_ld; a.rows_cap = rows_cap; a.step_offset = step_offset; a.status = status;
  const int blocks = T1 > T0 ? T1 - T0 : 1;
  const size_t smem = (kind == 0 ? (size_t)H * 2 : (size_t)H / 2 + H / 16);
  // few tokens: one block per route; many tokens (prefill): one block per token walks its k routes
  dispatch_push_kernel<<<dim3(blocks, blocks <= 512 ? k : 1), 128, smem, s>>>(a);
  CA_CHECK_LAUNCH("dispatch_push");
  return CA_OK;
}

// ---------------------------------------------------------------- token-major dispatch
// One block per token of my share: the row is quantised ONCE into shared memory and stored, with its block scales, into row
// (lane base + t) of the slab of every expert rank that owns at least one of the token's top-k experts - a token crosses
// NVLink once per destination rank, not once per route.  The token's k expert ids go to EVERY rank's routing table (a rank
// must see that a stale row is not for it), and the lane's token count goes next to it, so the expert side needs no host
// message to learn the step's shape.  The expert rank gathers rows into expert order itself (`route_gather`).
struct DispatchTokArgs {
  const bf16* x; const int* idx;
  PeerPtrs slab_q, slab_sf, idx_dst, lane_t_dst;   // per expert rank, already offset to this lane
  FlagPtrs flags;
  const float* inv_gs;
  uint32_t* ctl; uint32_t* done_counter;
  int T0, T1, T, H, k, E, n_ep, kind, sf_ld, broadcast;
  uint32_t step_offset;
  int* status;
};

__device__ __forceinline__ void quant_row_to_smem(const bf16* xr, int H, int kind, float inv_gs, uint8_t* pay, uint8_t* sfs) {
  if (kind == 0) {
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) ((uint4*)pay)[i] = ((const uint4*)xr)[i];
    return;
  }
  if (kind == 4) {      // FP8 E4M3 + one UE8M0 scale per 32 elements (amax floor 1e-4, scale 2^ceil(log2(amax / 448)))
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
      uint4 a = ((const uint4*)xr)[c];
      const bf16* e = (const bf16*)&a;
      float v[8], amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[j] = __bfloat162float(e[j]); amax = fmaxf(amax, fabsf(v[j])); }
      amax = fmaxf(amax, __shfl_xor_sync(__activemask(), amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(__activemask(), amax, 2));
      amax = fmaxf(amax, 1e-4f);
      const uint8_t sb = ue8m0_ceil(amax / 448.f);
      const float inv = 1.f / ue8m0_to_float(sb);
      uint32_t w0 = 0, w1 = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) { w0 |= (uint32_t)float_to_e4m3(v[j] * inv) << (8 * j); w1 |= (uint32_t)float_to_e4m3(v[4 + j] * inv) << (8 * j); }
      ((uint2*)pay)[c] = make_uint2(w0, w1);
      if ((c & 3) == 0) sfs[c >> 2] = sb;
    }
    return;
  }
  for (int c = threadIdx.x; c < H / 16; c += blockDim.x) {
    uint4 q0 = ((const uint4*)xr)[2 * c], q1 = ((const uint4*)xr)[2 * c + 1];
    const bf16* e0 = (const bf16*)&q0; const bf16* e1 = (const bf16*)&q1;
    float v[16], amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[j] = __bfloat162float(e0[j]); v[8 + j] = __bfloat162float(e1[j]); }
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    float eff; uint8_t sb;
    if (kind == 2) {
      amax = fmaxf(amax, __shfl_xor_sync(__activemask(), amax, 1));
      int e = amax > 0.f ? (int)((__float_as_uint(amax) >> 23) & 0xFF) - 2 : 0;
      e = max(e, 0); e = min(e, 254); sb = (uint8_t)e; eff = ue8m0_to_float(sb);
      if (!(c & 1)) sfs[c >> 1] = sb;
    } else {
      sb = float_to_e4m3(fminf(amax * inv_gs / 6.f, 448.f)); eff = e4m3_to_float(sb) / inv_gs;
      sfs[c] = sb;
    }
    const float inv = eff > 0.f ? 1.f / eff : 0.f;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { lo |= float_to_e2m1(v[j] * inv) << (4 * j); hi |= float_to_e2m1(v[8 + j] * inv) << (4 * j); }
    ((uint2*)pay)[c] = make_uint2(lo, hi);
  }
}

__global__ void dispatch_tok_push_kernel(const DispatchTokArgs a) {
  extern __shared__ uint8_t sh[];
  __shared__ unsigned owners;
  const int t = a.T0 + blockIdx.x;
  // the abort word, the activation scale and this token's routes are independent reads: requested together, ahead of the row
  const uint32_t abort_w = a.ctl[0];
  const float inv_gs_pre = (a.kind == 1 && a.inv_gs) ? *a.inv_gs : 1.f;
  const int e_pre = (t < a.T1 && (int)threadIdx.x < a.k) ? a.idx[(size_t)t * a.k + threadIdx.x] : -1;
  const bool live = t < a.T1 && !abort_w;
  const int H = a.H;
  const int row_bytes = a.kind == 0 ? H * 2 : (a.kind == 4 ? H : H / 2);
  const int n_sf = a.kind == 0 ? 0 : (a.kind == 1 ? H / 16 : H / 32);
  uint8_t* pay = sh; uint8_t* sfs = sh + row_bytes;
  if (threadIdx.x == 0) owners = 0u;
  __syncthreads();
  if (live) {
    quant_row_to_smem(a.x + (size_t)t * H, H, a.kind, inv_gs_pre, pay, sfs);
    if ((int)threadIdx.x < a.k) {
      const int e = e_pre;
      int owner = -1;
      for (int o = 0; o < a.n_ep; ++o) if (e >= (o * a.E) / a.n_ep && e < ((o + 1) * a.E) / a.n_ep) owner = o;
      if (owner < 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, t);
      else atomicOr(&owners, a.broadcast ? ((1u << a.n_ep) - 1u) : (1u << owner));   // expert TP: every rank holds a slice of every expert
      for (int d = 0; d < a.n_ep; ++d) ((int*)a.idx_dst.p[d])[(size_t)t * a.k + threadIdx.x] = e;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 32 && !abort_w)
    for (int d = 0; d < a.n_ep; ++d) *(int*)a.lane_t_dst.p[d] = a.T;
  __syncthreads();
  if (live) {
    const unsigned m = owners;
    for (int d = 0; d < a.n_ep; ++d) {
      if (!(m >> d & 1)) continue;
      uint4* dq = (uint4*)((uint8_t*)a.slab_q.p[d] + (size_t)t * row_bytes);
      for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) dq[i] = ((const uint4*)pay)[i];
      if (n_sf) {
        uint32_t* ds = (uint32_t*)((uint8_t*)a.slab_sf.p[d] + (size_t)t * a.sf_ld);
        for (int i = threadIdx.x; i < n_sf / 4; i += blockDim.x) ds[i] = ((const uint32_t*)sfs)[i];
      }
    }
  }
  publish_when_last(a.done_counter, a.flags.p, a.n_ep, a.ctl[1] + a.step_offset);
}

extern "C" int cuteafd_dispatch_tok_push(const void* x, const int* idx, const void* const* slab_q, const void* const* slab_sf,
                                         const void* const* idx_dst, const void* const* lane_t_dst, const void* const* flags,
                                         const float* inv_gs, void* ctl, void* done_counter, int T0, int T1, int T, int H, int k, int E,
                                         int n_ep, int kind, int sf_ld, int broadcast, unsigned step_offset, int* status, cudaStream_t s) {
  CA_REQUIRE(n_ep >= 1 && n_ep <= MAX_PEERS, "dispatch_tok_push: 1..8 expert ranks");
  CA_REQUIRE(H % 256 == 0 && k >= 1 && k <= 32, "dispatch_tok_push: hidden must be a multiple of 256 and k <= 32");
  CA_REQUIRE(((kind >= 0 && kind <= 2) || kind == 4) && (kind == 0 || (slab_sf && sf_ld % 4 == 0)), "dispatch_tok_push: quantised rows need a scale slab");
  CA_REQUIRE(T0 >= 0 && T1 >= T0 && T1 <= T, "dispatch_tok_push: my share [T0, T1) must lie inside the lane's T tokens");
  DispatchTokArgs a;
  a.x = (const bf16*)x; a.idx = idx; a.inv_gs = inv_gs;
  for (int i = 0; i < n_ep; ++i) {
    a.slab_q.p[i] = const_cast<void*>(slab_q[i]); a.slab_sf.p[i] = slab_sf ? const_cast<void*>(slab_sf[i]) : nullptr;
    a.idx_dst.p[i] = const_cast<void*>(idx_dst[i]); a.lane_t_dst.p[i] = const_cast<void*>(lane_t_dst[i]); a.flags.p[i] = (uint32_t*)flags[i];
  }
  a.ctl = (uint32_t*)ctl; a.done_counter = (uint32_t*)done_counter; a.T0 = T0; a.T1 = T1; a.T = T; a.H = H; a.k = k; a.E = E;
  a.n_ep = n_ep; a.kind = kind; a.sf_ld = sf_ld; a.broadcast = broadcast; a.step_offset = step_offset; a.status = status;
  const int blocks = T1 > T0 ? T1 - T0 : 1;
  const size_t smem = (kind == 0 ? (size_t)H * 2 : (kind == 4 ? (size_t)H + H / 32 : (size_t)H / 2 + H / 16));
  static bool attr_set[64] = {false};
  int dev = 0; cudaGetDevice(&dev);
  if (smem > 48 * 1024 && !attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(dispatch_tok_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return ca_cuda(e, "cudaFuncSetAttribute(dispatch_tok_push)");
    attr_set[dev & 63] = true;
  }
  CA_REQUIRE(smem <= 64 * 1024, "dispatch_tok_push: row does not fit shared memory");
  dispatch_tok_push_kernel<<<blocks, 256, smem, s>>>(a);      // one 16-element group per thread at hidden 4096: the row is one round of loads
  CA_CHECK_LAUNCH("dispatch_tok_push");
  return CA_OK;
}

// ---------------------------------------------------------------- combine: expert rank -> attention ranks
// Row i of y (local packed order) belongs to route src_route[i] = token * k + slot; it is stored to
// recv[token][slot][:] on every attention rank.  Rows >= *n_rows are skipped.
struct CombineArgs {
  const bf16* y; const int* src_route; const int* n_rows;
  PeerPtrs recv; FlagPtrs flags;
  uint32_t* ctl; uint32_t* done_counter;
  int H, n_attn, rows_cap;
  uint32_t step_offset;
};

__global__ void combine_push_kernel(const CombineArgs a) {
  const int n = min(*a.n_rows, a.rows_cap);
  if (!a.ctl[0]) {
    for (int r = blockIdx.x; r < n; r += gridDim.x) {
      const int route = a.src_route[r];
      const uint4* src = (const uint4*)(a.y + (size_t)r * a.H);
      for (int d = 0; d < a.n_attn; ++d) {
        uint4* dst = (uint4*)((bf16*)a.recv.p[d] + (size_t)route * a.H);
        for (int i = threadIdx.x; i < a.H / 8; i += blockDim.x) dst[i] = src[i];
      }
    }
  }
  publish_when_last(a.done_counter, a.flags.p, a.n_attn, a.ctl[1] + a.step_offset);
}

extern "C" int cuteafd_combine_push(const void* y, const int* src_route, const int* n_rows, const void* const* recv,
                                    const void* const* flags, void* ctl, void* done_counter, int H, int n_attn, int rows_cap,
                                    unsigned step_offset, cudaStream_t s) {
  CA_REQUIRE(n_attn >= 1 && n_attn <= MAX_PEERS && H % 8 == 0, "combine_push: bad arguments");
  CombineArgs a;
  a.y = (const bf16*)y; a.src_route = src_route; a.n_rows = n_rows;
  for (int i = 0; i < n_attn; ++i) { a.recv.p[i] = const_cast<void*>(recv[i]); a.flags.p[i] = (uint32_t*)flags[i]; }
  a.ctl = (uint32_t*)ctl; a.done_counter = (uint32_t*)done_counter; a.H = H; a.n_attn = n_attn; a.rows_cap = rows_cap; a.step_offset = step_offset;
  int blocks = rows_cap < 296 ? (rows_cap > 0 ? rows_cap : 1) : 296;
  combine_push_kernel<<<blocks, 128, 0, s>>>(a);
  CA_CHECK_LAUNCH("combine_push");
  return CA_OK;
}

// ---------------------------------------------------------------- combine for a lane table
// As combine_push, for rows that came from several lanes: route = (lane * t_cap + t) * k + slot; the row goes to
// recv[lane * tp + j][(t * k + slot)] for the tp attention ranks j of that lane (their buffers hold only their own lane),
// and every destination's flag is released once all rows are out.
struct CombineLanesArgs {
  const bf16* y; const int* src_route; const int* n_rows;
  PeerPtrs recv; FlagPtrs flags;
  uint32_t* ctl; uint32_t* done_counter;
  int H, k, t_cap, tp, n_dst, rows_cap;
  uint32_t step_offset;
  int* status;
};

__global__ void combine_push_lanes_kernel(const CombineLanesArgs a) {
  // row count, abort word and this block's first route are independent reads (the first route's slot is always inside the buffer)
  const int n_dev = *a.n_rows;
  const uint32_t abort_w = a.ctl[0];
  const int route0 = ((int)blockIdx.x < a.rows_cap) ? a.src_route[blockIdx.x] : -1;
  const int n = min(n_dev, a.rows_cap);
  if (!abort_w) {
    for (int r = blockIdx.x; r < n; r += gridDim.x) {
      const int route = (r == (int)blockIdx.x) ? route0 : a.src_route[r];
      const int tok = route / a.k, slot = route - tok * a.k;
      const int lane = tok / a.t_cap, t = tok - lane * a.t_cap;
      if (route < 0 || (lane + 1) * a.tp > a.n_dst) { if (threadIdx.x == 0) ca_dev_fail(a.status, CA_DEV_BAD_INDEX, r); continue; }
      const uint4* src = (const uint4*)(a.y + (size_t)r * a.H);
      for (int j = 0; j < a.tp; ++j) {
        uint4* dst = (uint4*)((bf16*)a.recv.p[lane * a.tp + j] + ((size_t)t * a.k + slot) * a.H);
        for (int i = threadIdx.x; i < a.H / 8; i += blockDim.x) dst[i] = src[i];
      }
    }
  }
  publish_when_last(a.done_counter, a.flags.p, a.n_dst, a.ctl[1] + a.step_offset);
}

extern "C" int cuteafd_combine_push_lanes(const void* y, const int* src_route, const int* n_rows, const void* const* recv,
                                          const void* const* flags, void* ctl, void* done_counter, int H, int k, int t_cap, int tp,
                                          int n_dst, int rows_cap, unsigned step_offset, int* status, cudaStream_t s) {
  CA_REQUIRE(n_dst >= 1 && n_dst <= MAX_PEERS && tp >= 1 && n_dst % tp == 0 && H % 8 == 0 && k >= 1 && t_cap >= 1,
             "combine_push_lanes: bad arguments");
  CombineLanesArgs a;
  a.y = (const bf16*)y; a.src_route = src_route; a.n_rows = n_rows;
  for (int i = 0; i < n_dst; ++i) { a.recv.p[i] = const_cast<void*>(recv[i]); a.flags.p[i] = (uint32_t*)flags[i]; }
  a.ctl = (uint32_t*)ctl; a.done_counter = (uint32_t*)done_counter; a.H = H; a.k = k; a.t_cap = t_cap; a.tp = tp; a.n_dst = n_dst;
  a.rows_cap = rows_cap; a.step_offset = step_offset; a.status = status;
  int blocks = rows_cap < 296 ? (rows_cap > 0 ? rows_cap : 1) : 296;
  combine_push_lanes_kernel<<<blocks, 128, 0, s>>>(a);
  CA_CHECK_LAUNCH("combine_push_lanes");
  return CA_OK;
}

// ---------------------------------------------------------------- link probes
// SM-issued copy between any two addresses (either may be peer memory): 16-byte loads and stores, grid chosen by the caller.
// dst = peer, src = local is an SM push; dst = local, src = peer an SM pull.  (Reference: the p2p probe modes of
// native/shared/include/cuteafd_peer_exchange.h:121-138, 353-371.)
__global__ void peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}

extern "C" int cuteafd_peer_copy(void* dst, const void* src, size_t bytes, int blocks, cudaStream_t s) {
  CA_REQUIRE(bytes % 16 == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0, "peer_copy: 16-byte alignment");
  if (!bytes) return CA_OK;
  const size_t n16 = bytes / 16;
  if (blocks < 1) { size_t b = (n16 + 255) / 256; blocks = (int)(b < 1184 ? b : 1184); }
  peer_copy_kernel<<<blocks, 256, 0, s>>>((const uint4*)src, (uint4*)dst, n16);
  CA_CHECK_LAUNCH("peer_copy");
  return CA_OK;
}

// Copy-engine copy between two device addresses (peer addresses included): no SM involved.
extern "C" int cuteafd_copy_engine(void* dst, const void* src, size_t bytes, cudaStream_t s) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s);
  if (e != cudaSuccess) return ca_cuda(e, "cudaMemcpyAsync(peer)");
  return CA_OK;
}

// Flag ping-pong between two GPUs (one launch on each, at the same time, one thread): the initiator releases i into the
// peer's flag and waits for i in its own; the responder waits, then answers.  `out_ns[0]` = nanoseconds for `iters` round
// trips on this side.  Every wait is bounded; a wait that runs out sets the status word and ends the loop.
__global__ void flag_pingpong_kernel(uint32_t* my_flag, uint32_t* peer_flag, uint32_t base, int iters, int initiator,
                                     unsigned long long timeout_ns, int* status, unsigned long long* out_ns) {
  const uint64_t t0 = globaltimer_ns();
  for (int i = 1; i <= iters; ++i) {
    const uint32_t v = base + (uint32_t)i;
    if (initiator) {
      st_release_sys(peer_flag, v);
      if (!wait_flag_bounded(my_flag, v, timeout_ns)) { ca_dev_fail(status, CA_DEV_TIMEOUT_FLAG, i); break; }
    } else {
      if (!wait_flag_bounded(my_flag, v, timeout_ns)) { ca_dev_fail(status, CA_DEV_TIMEOUT_FLAG, i); break; }
      st_release_sys(peer_flag, v);
    }
  }
  out_ns[0] = globaltimer_ns() - t0;
}

extern "C" int cuteafd_flag_pingpong(void* my_flag, void* peer_flag, unsigned base, int iters, int initiator, unsigned long long timeout_ns,
                                     int* status, void* out_ns, cudaStream_t s) {
  CA_REQUIRE(my_flag && peer_flag && iters >= 1 && out_ns, "flag_pingpong: flags, iterations and an output word");
  flag_pingpong_kernel<<<1, 1, 0, s>>>((uint32_t*)my_flag, (uint32_t*)peer_flag, base, iters, initiator, timeout_ns, status, (unsigned long long*)out_ns);
  CA_CHECK_LAUNCH("flag_pingpong");
  return CA_OK;
}
