// Device code of the variable all-gather (dispatch): flat multicast / peer copies, the
// low-latency packet mode, and the kernel body as a function so that other kernels can run the
// dispatch as their first phase.
#pragma once
#include "mcb_barrier.cuh"

namespace mcb {

__device__ __forceinline__ int ceil_div_i(long long a, long long b) { return (int)((a + b - 1) / b); }

// ------------------------------------------------------------------------------------------
// Flat copy helpers.  VEC = bytes per access (16, 8 or 4).
// ------------------------------------------------------------------------------------------
template <int VEC> struct Pack;
template <> struct Pack<16> {
  using T = uint4;
  static __device__ __forceinline__ T ld(const void* p) { return ld_v4_stream(p); }
  static __device__ __forceinline__ void st(void* p, T v) { st_v4(p, v); }
  static __device__ __forceinline__ void mm_st(void* p, T v) { mm_st_v4(p, v); }
};
template <> struct Pack<8> {
  using T = uint2;
  static __device__ __forceinline__ T ld(const void* p) { return ld_v2(p); }
  static __device__ __forceinline__ void st(void* p, T v) { st_v2(p, v); }
  static __device__ __forceinline__ void mm_st(void* p, T v) { mm_st_v2(p, v); }
};
template <> struct Pack<4> {
  using T = uint32_t;
  static __device__ __forceinline__ T ld(const void* p) { return ld_b32(p); }
  static __device__ __forceinline__ void st(void* p, T v) { st_b32(p, v); }
  static __device__ __forceinline__ void mm_st(void* p, T v) { mm_st_b32(p, v); }
};

constexpr int kUnroll = 4;

// Broadcast `nbytes` from local `src` to heap offset `dst_off` on every rank.
template <int VEC>
__device__ __forceinline__ void broadcast_flat(const McbCtx& c, const uint8_t* src, uint64_t dst_off,
                                               long long nbytes, long long start, long long stride) {
  using P = Pack<VEC>;
  const long long nvec = nbytes / VEC;
  if (c.transport == MCB_TRANSPORT_MULTIMEM) {
    uint8_t* dst = c.heap_mc + dst_off;
    for (long long i = start; i < nvec; i += stride * kUnroll) {
      typename P::T v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < nvec) v[u] = P::ld(src + (i + u * stride) * VEC);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < nvec) P::mm_st(dst + (i + u * stride) * VEC, v[u]);
    }
  } else {
    for (long long i = start; i < nvec; i += stride * kUnroll) {
      typename P::T v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < nvec) v[u] = P::ld(src + (i + u * stride) * VEC);
      // Start with the next rank so that all ranks do not hit the same peer at once.
      for (int k = 0; k < c.world; ++k) {
        int p = c.rank + 1 + k;
        if (p >= c.world) p -= c.world;
        uint8_t* dst = c.heap_peer[p] + dst_off;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (i + u * stride < nvec) P::st(dst + (i + u * stride) * VEC, v[u]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Flat cross-rank reduction: out[i] = sum over ranks of heap[base + 16 * i], 16 bytes at a time.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], uint4 v) {
  acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x);
  acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
  acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z);
  acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
}

// Sum of one 16-byte pack over every rank's heap with plain peer loads.
template <bool F32>
__device__ __forceinline__ uint4 p2p_reduce_pack(const McbCtx& c, uint64_t off) {
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int k = 0;
  for (; k + 4 <= c.world; k += 4) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int p = c.rank + k + u;
      if (p >= c.world) p -= c.world;
      v[u] = ld_v4_stream(c.heap_peer[p] + off);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (F32) {
        acc[0] += __uint_as_float(v[u].x); acc[1] += __uint_as_float(v[u].y);
        acc[2] += __uint_as_float(v[u].z); acc[3] += __uint_as_float(v[u].w);
      } else {
        acc_bf16x8(acc, v[u]);
      }
    }
  }
  for (; k < c.world; ++k) {
    int p = c.rank + k;
    if (p >= c.world) p -= c.world;
    const uint4 v = ld_v4_stream(c.heap_peer[p] + off);
    if (F32) {
      acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
      acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
    } else {
      acc_bf16x8(acc, v);
    }
  }
  if (F32)
    return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]),
                      __float_as_uint(acc[3]));
  return make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                    pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
}

// dtype 0: bf16 operands summed in fp32 (inside the switch with multimem), 1: fp32.
__device__ __forceinline__ void reduce_flat(const McbCtx& c, uint8_t* out, uint64_t base, long long nvec,
                                            long long start, long long stride, int dtype) {
  if (c.transport == MCB_TRANSPORT_MULTIMEM) {
    const uint8_t* src = c.heap_mc + base;
    for (long long i = start; i < nvec; i += stride * kUnroll) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < nvec)
          v[u] = dtype == 1 ? mm_ld_reduce_f32x4(src + (i + u * stride) * 16)
                            : mm_ld_reduce_bf16x8(src + (i + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < nvec) st_v4(out + (i + u * stride) * 16, v[u]);
    }
  } else {
    for (long long i = start; i < nvec; i += stride * kUnroll) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < nvec)
          v[u] = dtype == 1 ? p2p_reduce_pack<true>(c, base + (i + u * stride) * 16)
                            : p2p_reduce_pack<false>(c, base + (i + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (i + u * stride < nvec) st_v4(out + (i + u * stride) * 16, v[u]);
    }
  }
}

// Number of blocks that take part in a variable collective.  Depends only on values that
// are identical on every rank (grid size, largest per-rank count, bytes per row), so block b
// either runs on all ranks or on none.
__device__ __forceinline__ int active_blocks(int grid, int ep_max, long long bytes_per_row, int threads) {
  if (ep_max <= 0) return 0;
  const long long vecs = ((long long)ep_max * bytes_per_row + 15) / 16;
  int nb = ceil_div_i(vecs, threads);
  if (nb < 1) nb = 1;
  return nb < grid ? nb : grid;
}


// ------------------------------------------------------------------------------------------
// Low-latency packets.  A packet is 16 bytes {data.lo, flag, data.hi, flag}: 8 bytes of payload
// and the launch's flag value twice, so each 8-byte half carries its own flag and the packet is
// valid as soon as both flags match (the scheme of NCCL's LL protocol).  The flag changes with
// every launch, so a packet left over from an earlier launch is never mistaken for a new one.
// ------------------------------------------------------------------------------------------
constexpr int kLLBlocks = 128;

__device__ __forceinline__ uint4 ll_pack(uint2 d, uint32_t flag) { return make_uint4(d.x, flag, d.y, flag); }

// Poll one packet in local memory until it carries `flag`.  Bounded; on timeout records the
// error and returns zeros.
__device__ __forceinline__ uint2 ll_wait(const McbCtx& c, const uint8_t* slot, uint32_t flag, int site) {
  uint4 v = ld_v4_volatile(slot);
  if (v.y == flag && v.w == flag) return make_uint2(v.x, v.z);
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      v = ld_v4_volatile(slot);
      if (v.y == flag && v.w == flag) return make_uint2(v.x, v.z);
    }
    const bool poisoned = *reinterpret_cast<volatile uint32_t*>(c.status) != 0u;
    if (poisoned || globaltimer_ns() - t0 > c.timeout_ns) {
      report_error(c, MCB_ERR_TIMEOUT, (uint32_t)site, blockIdx.x, v.y, flag);
      return make_uint2(0u, 0u);
    }
  }
}

__device__ __forceinline__ bool agv_ll_eligible(const McbCtx& c, const McbAgvArgs& a, int valid) {
  if (c.world == 1 || a.ll_rows <= 0 || valid <= 0 || valid > a.ll_rows) return false;
  bool ok = true;
#pragma unroll
  for (int t = 0; t < MCB_MAX_TENSORS; ++t)
    if (t < a.num_tensors && (a.row_bytes[t] & 7u)) ok = false;
  return ok;
}

// Low-latency all-gather-V: send my rows as packets to every rank's staging area, then poll my
// own staging area for all `valid` rows and unpack them into the gathered tensors.
__device__ __forceinline__ void agv_ll(const McbCtx& c, const McbAgvArgs& a, int n, int offset, int valid,
                                       uint32_t flag) {
  int w[MCB_MAX_TENSORS];
  int wpr = 0;
#pragma unroll
  for (int t = 0; t < MCB_MAX_TENSORS; ++t) {
    w[t] = t < a.num_tensors ? (int)(a.row_bytes[t] >> 3) : 0;
    wpr += w[t];
  }
  const uint64_t stage = a.ll_off + (uint64_t)(flag & 1u) * a.ll_rows * wpr * 16;
  // Blocks poll for packets that other ranks' blocks send, so every taking-part block must be
  // resident at the same time: at most kLLBlocks of them (one per SM always fits).
  const int nb = (int)gridDim.x < kLLBlocks ? (int)gridDim.x : kLLBlocks;
  if ((int)blockIdx.x >= nb) return;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)nb * blockDim.x;
  // send: 4 independent packets per thread in flight
  const long long nsend = (long long)n * wpr;
  for (long long i0 = tid; i0 < nsend; i0 += nthreads * 4) {
    uint2 d[4];
    uint64_t off[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * nthreads;
      off[u] = ~0ull;
      if (i < nsend) {
        const int row = (int)(i / wpr);
        int j = (int)(i - (long long)row * wpr);
        const int jj = j;
        int t = 0;
#pragma unroll
        for (int k = 0; k < MCB_MAX_TENSORS - 1; ++k)
          if (t == k && j >= w[k]) { j -= w[k]; t = k + 1; }
        d[u] = ld_v2(reinterpret_cast<const uint8_t*>(a.src[t]) + (uint64_t)row * a.row_bytes[t] + (uint64_t)j * 8);
        off[u] = stage + ((uint64_t)(offset + row) * wpr + jj) * 16;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (off[u] == ~0ull) continue;
      const uint4 pkt = ll_pack(d[u], flag);
      if (c.transport == MCB_TRANSPORT_MULTIMEM) {
        mm_st_v4(c.heap_mc + off[u], pkt);
      } else {
        for (int k = 0; k < c.world; ++k) {
          int p = c.rank + 1 + k;
          if (p >= c.world) p -= c.world;
          st_v4(c.heap_peer[p] + off[u], pkt);
        }
      }
    }
  }
  // receive: poll 4 packets at a time, wait only for those not there yet
  const long long nrecv = (long long)valid * wpr;
  for (long long i0 = tid; i0 < nrecv; i0 += nthreads * 4) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * nthreads;
      if (i < nrecv) v[u] = ld_v4_volatile(c.heap_local + stage + (uint64_t)i * 16);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * nthreads;
      if (i >= nrecv) break;
      uint2 d = make_uint2(v[u].x, v[u].z);
      if (v[u].y != flag || v[u].w != flag) d = ll_wait(c, c.heap_local + stage + (uint64_t)i * 16, flag, a.site);
      const int row = (int)(i / wpr);
      int j = (int)(i - (long long)row * wpr);
      int t = 0;
#pragma unroll
      for (int k = 0; k < MCB_MAX_TENSORS - 1; ++k)
        if (t == k && j >= w[k]) { j -= w[k]; t = k + 1; }
      st_v2(c.heap_local + a.dst_off[t] + (uint64_t)row * a.row_bytes[t] + (uint64_t)j * 8, d);
    }
  }
}

// Body of the variable all-gather, shared by the stand-alone kernel and the fused
// dispatch + routing + FC1 kernel.  Call from all threads of the block.  The launch number (the
// packet flag) is returned in `ll_launch`: FUSED_SITE < 0 takes it from the per-block counters of
// MCB_SITE_AGV_LL; otherwise from launch_begin(FUSED_SITE), and the calling kernel must end with
// launch_end(FUSED_SITE, ll_launch).
template <int FUSED_SITE>
__device__ __forceinline__ void agv_device(const McbCtx& c, const McbAgvArgs& a, uint32_t& ll_launch) {
  const int bid = blockIdx.x;
  int n = 0, valid_pre = 0, offset = 0, ep_max = 0;
  if (a.meta_stable) {
    n = *a.n_local;
    valid_pre = a.step_meta[0]; offset = a.step_meta[1]; ep_max = a.step_meta[2];
  }
  pdl_wait();
  ll_launch = FUSED_SITE < 0 ? next_launch_count(c, MCB_SITE_AGV_LL) : launch_begin(c, FUSED_SITE);
  if (!a.meta_stable) {
    n = *a.n_local;
    valid_pre = a.step_meta[0]; offset = a.step_meta[1]; ep_max = a.step_meta[2];
  }
  long long bytes_per_row = 0;
#pragma unroll
  for (int t = 0; t < MCB_MAX_TENSORS; ++t)
    if (t < a.num_tensors) bytes_per_row += a.row_bytes[t];
  const int nact = active_blocks((int)gridDim.x, ep_max, bytes_per_row, (int)blockDim.x);
  pdl_launch_dependents();
  const bool bad = n < 0 || n > a.cap || offset < 0 || (long long)offset + n > (long long)a.cap * c.world;
  if (a.ll_rows > 0 && c.world > 1) {
    const uint32_t flag = ll_launch;      // changes with every launch, in either mode
    if (agv_ll_eligible(c, a, valid_pre)) {
      const int valid = valid_pre;
      if (bad) {
        if (threadIdx.x == 0) report_error(c, MCB_ERR_BOUNDS, (uint32_t)a.site, (uint32_t)bid, (uint32_t)n, (uint32_t)valid);
        return;
      }
      agv_ll(c, a, n, offset, valid, flag);
      return;
    }
  }
  if (bid >= nact) return;
  const uint32_t ep = *epoch_ptr(c, a.site, bid);
  if (n < 0) n = 0;
  if (bad) {
    if (threadIdx.x == 0)
      report_error(c, n > a.cap ? MCB_ERR_CAPACITY : MCB_ERR_BOUNDS, (uint32_t)a.site, (uint32_t)bid,
                   (uint32_t)n, (uint32_t)offset);
    n = 0;  // skip the copy, still meet the barrier
  }
  const long long start = (long long)bid * blockDim.x + threadIdx.x;
  const long long stride = (long long)nact * blockDim.x;
#pragma unroll
  for (int t = 0; t < MCB_MAX_TENSORS; ++t) {
    if (t >= a.num_tensors) break;
    const uint32_t rb = a.row_bytes[t];
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.src[t]);
    const uint64_t dst_off = a.dst_off[t] + (uint64_t)offset * rb;
    const long long nbytes = (long long)n * rb;
    if ((rb & 15u) == 0) broadcast_flat<16>(c, src, dst_off, nbytes, start, stride);
    else if ((rb & 7u) == 0) broadcast_flat<8>(c, src, dst_off, nbytes, start, stride);
    else broadcast_flat<4>(c, src, dst_off, nbytes, start, stride);
  }
  // Trailing barrier: when this kernel has finished on a rank, every peer's rows are there.
  block_barrier_all(c, a.site, bid, ep);
}

}  // namespace mcb
