// One whole decode step of the dense dispatcher as ONE persistent kernel for sm_100a.
//
// The reference issues a step as 1 + 2 * 88 kernels (bench_nvls.py:114-121: metadata once, then
// per layer an all-gather-V with a trailing cross-GPU barrier and a reduce-scatter-V with a leading
// one, variable_collectives.py:142-150, 209-219).  Here the whole step is one launch:
//
//   count exchange      block 0 publishes this rank's row count to every rank; every block of
//                       every rank waits for all counts.  Because a rank only publishes after its
//                       previous kernel has finished, passing this point also proves that every
//                       rank has left the previous step: nothing written now can race with it.
//   barrier mode        per layer: push my share of the local rows into the gathered buffers of
//                       every rank (multimem.st, or peer stores), ONE block-matched release barrier,
//                       then the switch-side reduction (multimem.ld_reduce, or peer loads) of the
//                       rows this rank owns.  The gathered buffers are double-buffered by layer
//                       parity, so the barrier of layer l is also the write-after-read fence that
//                       protects the readers of layer l - 1.
//   pipeline groups     optionally the blocks are split into G groups, each owning 1/G of every
//                       rank's rows.  A group's chain push -> barrier -> reduce is unchanged, but
//                       the groups take turns on the push, so one group's reduction (which loads
//                       the outbound direction of every link) runs while the next group's push
//                       fills the inbound direction.  Dependencies are per row: a row is reduced
//                       only after it was gathered everywhere, and pushed for the next layer only
//                       after it was reduced.
//   packet mode         small steps: rows travel as 16-byte {data, flag, data, flag} packets that
//                       the receiver polls, so a layer needs no barrier and no fence.  A packet is
//                       written and read by the same block index on every rank, and after each
//                       layer a block publishes "I have finished reading layer l" in a word of its
//                       own on every rank (one word per (block, source rank): a sum over ranks
//                       could not tell a slow rank from fast ones that ran ahead); a block re-uses
//                       a staging area (two parities) only when every rank's word has reached the
//                       layer that used it last.
//
// All per-step sizes are read from device memory, so one captured launch serves every batch.
// Every wait is bounded and reports through the status words.
//
// FP8 = true dispatches the hidden rows as 1 x 128 block-scaled e4m3 (BASELINE configuration of the
// DeepSeek-V3 shape): tensor 0's source is bf16 [cap, hidden], its gathered form is one byte per value,
// and tensor 3 is the gathered fp32 scales [rows, hidden / 128], produced here; quantisation happens
// inside the push (barrier mode: 16 neighbouring threads share a block and agree on its largest
// magnitude with shuffles; packet mode: every thread scans the 256 bytes of its block itself).
//
// CHECK = true is the self-checking build used by the race tests: the pushed payload is not the
// input rows but a hash of (layer sequence number, position), every receiver verifies the words
// it is entitled to read right after its barrier (or packet poll) and counts mismatches, and a
// rank can be slowed down by a bounded sleep per layer chosen on the host.  A write that
// arrives too early (a broken write-after-read fence) or too late then shows up as a mismatch
// instead of being invisible because consecutive layers carry identical bytes.
#include <cuda_runtime.h>

#include "mcb_barrier.cuh"
#include "mcb_dense.cuh"
#include "mcb_fp8.cuh"
#include "mcb_launch.h"
#include "mcb_step.cuh"

namespace mcb {

struct StepShape {
  int w[MCB_MAX_TENSORS];   // 8-byte words per row of each gathered tensor
  int wpr;                  // their sum
};

// Which tensor and which word of its row is word `jj` of a gathered row.
__device__ __forceinline__ void split_word(const StepShape& s, int jj, int& t, int& j) {
  t = 0;
  j = jj;
#pragma unroll
  for (int k = 0; k < MCB_MAX_TENSORS - 1; ++k)
    if (t == k && j >= s.w[k]) { j -= s.w[k]; t = k + 1; }
}

__device__ __forceinline__ uint32_t check_word(uint32_t seq, uint32_t tensor, uint32_t index) {
  uint32_t h = (seq + 1u) * 0x9E3779B1u ^ (index + 0x7F4A7C15u) * 0x85EBCA77u ^ (tensor + 1u) * 0xC2B2AE3Du;
  h ^= h >> 15;
  h *= 0x2C1B3C6Du;
  return h ^ (h >> 13);
}

__device__ __forceinline__ void check_fail(const McbDenseStepArgs& a) {
  if (a.check_errors) atomicAdd(a.check_errors, 1u);
}

// Packet all-gather of one layer.  Slot i = (global row) * wpr + word is sent by thread
// (i mod nthreads) of the row's owner and read by the same thread index on every rank.
// The 8 payload bytes of word j of gathered tensor t of local row `row` when the hidden rows are
// quantised on the way out: 8 e4m3 values (t == 0) or two fp32 scales (t == 3).
__device__ __forceinline__ uint2 fp8_word(const McbDenseStepArgs& a, int row, int t, int j) {
  const uint8_t* src = reinterpret_cast<const uint8_t*>(a.src[0]) + (uint64_t)row * a.fp8_hidden * 2;
  if (t == 0) {
    const float scale = e4m3_scale(block_absmax_serial(src + (uint64_t)(j >> 4) * 256));
    return quant_pack_e4m3(ld_v4(src + (uint64_t)j * 16), scale);
  }
  return make_uint2(__float_as_uint(e4m3_scale(block_absmax_serial(src + (uint64_t)(2 * j) * 256))),
                    __float_as_uint(e4m3_scale(block_absmax_serial(src + (uint64_t)(2 * j + 1) * 256))));
}

template <bool CHECK, bool FP8>
__device__ __forceinline__ void step_agv_ll(const McbCtx& c, const McbDenseStepArgs& a, const StepShape& s,
                                            int n, int offset, int valid, uint32_t flag, uint32_t par,
                                            uint32_t seq, long long gtid, long long nthreads) {
  const uint64_t stage = a.agv_ll_off + (uint64_t)(flag & 1u) * a.ll_rows * s.wpr * 16;
  const long long lo = (long long)offset * s.wpr, hi = (long long)(offset + n) * s.wpr;
  long long first = lo + ((gtid - lo) % nthreads + nthreads) % nthreads;
  for (long long i0 = first; i0 < hi; i0 += nthreads * 4) {
    uint2 d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * nthreads;
      if (i < hi) {
        const int row = (int)(i / s.wpr);
        int t, j;
        split_word(s, (int)(i - (long long)row * s.wpr), t, j);
        if (FP8 && (t == 0 || t == 3)) d[u] = fp8_word(a, row - offset, t, j);
        else
        d[u] = CHECK ? make_uint2(check_word(seq, 0u, (uint32_t)i * 2u), check_word(seq, 0u, (uint32_t)i * 2u + 1u))
                     : ld_v2(reinterpret_cast<const uint8_t*>(a.src[t]) + (uint64_t)(row - offset) * a.row_bytes[t] +
                             (uint64_t)j * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * nthreads;
      if (i >= hi) break;
      const uint4 pkt = ll_pack(d[u], flag);
      const uint64_t off = stage + (uint64_t)i * 16;
      if (c.transport == MCB_TRANSPORT_MULTIMEM) {
        mm_st_v4(c.heap_mc + off, pkt);
      } else {
        for (int k = 0; k < c.world; ++k) {
          int p = c.rank + 1 + k;
          if (p >= c.world) p -= c.world;
          st_v4(c.heap_peer[p] + off, pkt);
        }
      }
    }
  }
  const long long nrecv = (long long)valid * s.wpr;
  for (long long i0 = gtid; i0 < nrecv; i0 += nthreads * 4) {
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
      if (v[u].y != flag || v[u].w != flag)
        d = ll_wait(c, c.heap_local + stage + (uint64_t)i * 16, flag, MCB_SITE_STEP);
      if (CHECK && (d.x != check_word(seq, 0u, (uint32_t)i * 2u) || d.y != check_word(seq, 0u, (uint32_t)i * 2u + 1u)))
        check_fail(a);
      const int row = (int)(i / s.wpr);
      int t, j;
      split_word(s, (int)(i - (long long)row * s.wpr), t, j);
      st_v2(c.heap_local + a.dst_off[t] + (uint64_t)par * a.dst_par_stride[t] + (uint64_t)row * a.row_bytes[t] +
                (uint64_t)j * 8, d);
    }
  }
}

// Packet reduce-scatter of one layer (bf16).  Word i of owner o's rows is sent by thread
// (i mod nthreads) of every rank and summed, in rank order in fp32, by the same thread index of o.
__device__ __forceinline__ void step_rsv_ll(const McbCtx& c, const McbDenseStepArgs& a, const int* s_prefix,
                                            int n, int ep_max, uint32_t flag, long long gtid, long long nthreads) {
  const int wpr = (int)(a.rsv_row_bytes >> 3);
  const uint64_t per_src = (uint64_t)a.ll_src_rows * wpr * 16;
  const uint64_t stage = a.rsv_ll_off + (uint64_t)(flag & 1u) * c.world * per_src;
  const uint8_t* mine = c.heap_local + a.rsv_off;
  const uint64_t my_region = stage + (uint64_t)c.rank * per_src;
  for (long long i = gtid; i < (long long)ep_max * wpr; i += nthreads) {
    for (int o0 = 0; o0 < c.world; o0 += 4) {
      uint2 d[4];
      bool live[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int o = o0 + u;
        live[u] = o < c.world && i < (long long)(s_prefix[o + 1] - s_prefix[o]) * wpr;
        if (live[u]) d[u] = ld_v2(mine + ((uint64_t)s_prefix[o] * wpr + (uint64_t)i) * 8);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (live[u]) st_v4(c.heap_peer[o0 + u] + my_region + (uint64_t)i * 16, ll_pack(d[u], flag));
    }
  }
  uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
  for (long long i = gtid; i < (long long)n * wpr; i += nthreads) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint8_t* slot0 = c.heap_local + stage + (uint64_t)i * 16;
    for (int s0 = 0; s0 < c.world; s0 += 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (s0 + u < c.world) v[u] = ld_v4_volatile(slot0 + (uint64_t)(s0 + u) * per_src);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u >= c.world) break;
        uint2 d = make_uint2(v[u].x, v[u].z);
        if (v[u].y != flag || v[u].w != flag)
          d = ll_wait(c, slot0 + (uint64_t)(s0 + u) * per_src, flag, MCB_SITE_STEP);
        acc[0] += bf16_lo(d.x); acc[1] += bf16_hi(d.x);
        acc[2] += bf16_lo(d.y); acc[3] += bf16_hi(d.y);
      }
    }
    st_v2(out + (uint64_t)i * 8, make_uint2(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3])));
  }
}

// Self-checking push of one tensor's share (4-byte words) and its verification after the barrier.
__device__ __forceinline__ void check_push(const McbCtx& c, uint64_t dst_off, uint32_t tensor, uint32_t seq,
                                           long long first_word, long long nwords, long long start, long long stride) {
  for (long long i = start; i < nwords; i += stride) {
    const uint32_t v = check_word(seq, tensor, (uint32_t)(first_word + i));
    const uint64_t off = dst_off + (uint64_t)(first_word + i) * 4;
    if (c.transport == MCB_TRANSPORT_MULTIMEM) {
      mm_st_b32(c.heap_mc + off, v);
    } else {
      for (int k = 0; k < c.world; ++k) {
        int p = c.rank + 1 + k;
        if (p >= c.world) p -= c.world;
        st_b32(c.heap_peer[p] + off, v);
      }
    }
  }
}
__device__ __forceinline__ void check_verify(const McbCtx& c, const McbDenseStepArgs& a, uint64_t dst_off,
                                             uint32_t tensor, uint32_t seq, long long first_word, long long nwords,
                                             long long start, long long stride) {
  for (long long i = start; i < nwords; i += stride)
    if (ld_relaxed_sys(c.heap_local + dst_off + (uint64_t)(first_word + i) * 4) !=
        check_word(seq, tensor, (uint32_t)(first_word + i)))
      check_fail(a);
}

// A world of one: dispatch and combine are local copies.  Eight independent 16-byte accesses per
// thread keep one block per SM close to the copy bandwidth of the on-chip memory.
__device__ __forceinline__ void copy_flat_local(uint8_t* dst, const uint8_t* src, long long nbytes, long long start,
                                                long long stride) {
  const long long nvec = nbytes / 16;
  constexpr int U = 8;
  for (long long i = start; i < nvec; i += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < nvec) v[u] = ld_v4_stream(src + (i + u * stride) * 16);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < nvec) st_v4(dst + (i + u * stride) * 16, v[u]);
  }
}

// Barrier-mode push of the quantised hidden rows [r0, r1) of this rank and of their scales.  Packs
// (16 bytes of bf16 = 8 values) are dealt to threads in order, so the 16 lanes of a half warp hold one
// 128-value block.  Call from all threads of the block (whole warps take part in the shuffles).
__device__ __forceinline__ void fp8_push(const McbCtx& c, const McbDenseStepArgs& a, uint32_t par, int offset, int r0,
                                         int r1, long long start, long long stride) {
  const int H = (int)a.fp8_hidden, ppr = H / 8, nblk = H / 128;
  const long long total = (long long)(r1 - r0) * ppr;              // a multiple of 16
  const uint8_t* src = reinterpret_cast<const uint8_t*>(a.src[0]) + (uint64_t)r0 * H * 2;
  const uint64_t q_off = a.dst_off[0] + (uint64_t)par * a.dst_par_stride[0] + (uint64_t)(offset + r0) * H;
  const uint64_t s_off = a.dst_off[3] + (uint64_t)par * a.dst_par_stride[3] + (uint64_t)(offset + r0) * nblk * 4;
  const long long warp_start = start - (threadIdx.x & 31);
  for (long long base = warp_start; base < total; base += stride) {
    const long long i = base + (threadIdx.x & 31);
    const bool live = i < total;
    const uint4 v = live ? ld_v4_stream(src + i * 16) : make_uint4(0, 0, 0, 0);
    float amax = pack_absmax(v);
#pragma unroll
    for (int sh = 8; sh >= 1; sh >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
    if (!live) continue;
    const float scale = e4m3_scale(amax);
    const uint2 q = quant_pack_e4m3(v, scale);
    const long long row = i / ppr;
    const int pk = (int)(i - row * ppr);
    const uint64_t qo = q_off + (uint64_t)row * H + (uint64_t)pk * 8;
    const uint64_t so = s_off + ((uint64_t)row * nblk + (pk >> 4)) * 4;
    if (c.transport == MCB_TRANSPORT_MULTIMEM) {
      mm_st_v2(c.heap_mc + qo, q);
      if ((pk & 15) == 0) mm_st_b32(c.heap_mc + so, __float_as_uint(scale));
    } else {
      for (int k = 0; k < c.world; ++k) {
        int p = c.rank + 1 + k;
        if (p >= c.world) p -= c.world;
        st_v2(c.heap_peer[p] + qo, q);
        if ((pk & 15) == 0) st_b32(c.heap_peer[p] + so, __float_as_uint(scale));
      }
    }
  }
}

template <bool EMU, bool CHECK, bool FP8>
__global__ void __launch_bounds__(512) dense_step_kernel(const __grid_constant__ McbCtx ctx_p,
                                                         const __grid_constant__ McbDenseStepArgs args_p,
                                                         const McbCtx* ectx, const McbDenseStepArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbDenseStepArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  __shared__ int s_prefix[MCB_MAX_RANKS + 1];
  __shared__ int s_cnt[MCB_MAX_RANKS];
  __shared__ int s_max;
  const int tid = threadIdx.x, bid = blockIdx.x;
  const int W = c.world, L = a.num_layers;
  pdl_wait();                 // the previous kernel of this rank (the previous step) has finished
  pdl_launch_dependents();
  volatile uint32_t* state = a.state;
  const uint32_t step_seq = state[MCB_STATE_STEP_SEQ], layer_base = state[MCB_STATE_LAYER_BASE],
                 ll_base = state[MCB_STATE_LL_BASE];

  // ---- count exchange -------------------------------------------------------------------------
  const int n = step_count_exchange(c, MCB_SITE_STEP_META, a.counts_off, step_seq, *a.n_local, a.cap, s_cnt, s_prefix,
                                    &s_max);
  const int valid = s_prefix[W], offset = s_prefix[c.rank], ep_max = s_max;

  StepShape shp;
  long long bytes_per_row = 0;
  bool words_ok = (a.rsv_row_bytes & 7u) == 0;
  shp.wpr = 0;
#pragma unroll
  for (int t = 0; t < MCB_MAX_TENSORS; ++t) {
    const uint32_t rb = t < a.num_tensors ? a.row_bytes[t] : 0u;
    shp.w[t] = (int)(rb >> 3);
    shp.wpr += shp.w[t];
    bytes_per_row += rb;
    if (rb & 7u) words_ok = false;
  }
  const bool ll = W > 1 && a.ll_rows > 0 && valid > 0 && valid <= a.ll_rows && a.rsv_dtype == 0 && words_ok;

  // ---- pipeline groups of the barrier mode (identical decision on every rank) ---------------------
  int G = a.groups < 1 ? 1 : (a.groups > MCB_MAX_GROUPS ? MCB_MAX_GROUPS : a.groups);
  if (W == 1 || ll) G = 1;
  while (G > 1 && ((long long)ep_max * bytes_per_row < (long long)G * (long long)a.group_min_bytes ||
                   (int)gridDim.x < 2 * G))
    --G;
  const int bpg = (int)gridDim.x / G;                   // blocks per group (left-over blocks idle)
  const int grp = bid / bpg < G ? bid / bpg : -1;
  const int lb = bid - (grp < 0 ? 0 : grp) * bpg;       // block index inside its group
  const int ep_max_g = (ep_max + G - 1) / G;
  const int nact = active_blocks(bpg, ep_max_g, bytes_per_row, (int)blockDim.x);

  if (bid == 0 && tid == 0) {
    a.step_meta[0] = valid;
    a.step_meta[1] = offset;
    a.step_meta[2] = ep_max;
    a.step_meta[4] = (int)(step_seq + 1u);
    a.step_meta[5] = L > 0 ? (int)((layer_base + (uint32_t)L - 1u) & 1u) : 0;
    a.step_meta[6] = ll ? 1 : 0;
    a.step_meta[7] = G;
  }

  if (ll) {
    // ---- packet mode ---------------------------------------------------------------------------
    int nb = ceil_div_i((long long)valid * shp.wpr, blockDim.x);
    if (nb > (int)gridDim.x) nb = (int)gridDim.x;
    if (bid < nb) {
      const long long gtid = (long long)bid * blockDim.x + tid;
      const long long nthreads = (long long)nb * blockDim.x;
      const uint32_t cb = *epoch_ptr(c, MCB_SITE_STEP_CREDIT, bid);
      for (int l = 0; l < L; ++l) {
        const uint32_t flag = ll_base + (uint32_t)l + 1u;
        const uint32_t par = (layer_base + (uint32_t)l) & 1u;
        // The staging area of this parity was read last in layer l - 2 (every rank has left the
        // previous step: nothing to wait for in the first two layers).
        if (l >= 2) credit_wait(c, a.credit_off, cb + (uint32_t)l - 1u, MCB_SITE_STEP_CREDIT);
        if (CHECK && a.delay_ns && (l + c.rank) % (a.delay_every < 1 ? 1 : a.delay_every) == 0)
          __nanosleep(a.delay_ns > 1000000u ? 1000000u : a.delay_ns);
        step_agv_ll<CHECK, FP8>(c, a, shp, n, offset, valid, flag, par, layer_base + (uint32_t)l, gtid, nthreads);
        __syncthreads();      // the block holds all its gathered words before it starts the combine
        step_rsv_ll(c, a, s_prefix, n, ep_max, flag, gtid, nthreads);
        __syncthreads();
        credit_publish(c, a.credit_off, cb + (uint32_t)l + 1u);
      }
      if (tid == 0) *epoch_ptr(c, MCB_SITE_STEP_CREDIT, bid) = cb + (uint32_t)L;
    }
  } else if (grp >= 0 && lb < nact) {
    // ---- barrier mode ----------------------------------------------------------------------------
    uint32_t ep = *epoch_ptr(c, MCB_SITE_STEP, bid);
    // Rows of this group: an equal share of this rank's rows, and of the rows it owns.
    const int r0 = (int)((long long)n * grp / G), r1 = (int)((long long)n * (grp + 1) / G);
    const long long start = (long long)lb * blockDim.x + tid;
    const long long stride = (long long)nact * blockDim.x;
    const int prev = (grp + G - 1) % G;
    uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
    for (int l = 0; l < L; ++l) {
      const uint32_t par = (layer_base + (uint32_t)l) & 1u;
      if (CHECK && a.delay_ns && (l + c.rank + grp) % (a.delay_every < 1 ? 1 : a.delay_every) == 0)
        __nanosleep(a.delay_ns > 1000000u ? 1000000u : a.delay_ns);
      if (G > 1) {
        // Pushes take turns: group g of layer l goes after group g - 1 of layer l, group 0 after
        // the last group of layer l - 1.
        const uint32_t need = (uint32_t)nact * (uint32_t)(grp == 0 ? l : l + 1);
        if (tid == 0 && need) wait_local(c, a.state + MCB_STATE_GATE0 + prev, need, MCB_SITE_STEP);
        __syncthreads();
      }
      if (FP8) fp8_push(c, a, par, offset, r0, r1, start, stride);
#pragma unroll
      for (int t = 0; t < MCB_MAX_TENSORS; ++t) {
        if (t >= a.num_tensors) break;
        if (FP8 && (t == 0 || t == 3)) continue;      // quantised values and scales: pushed above
        const uint32_t rb = a.row_bytes[t];
        const uint8_t* src = reinterpret_cast<const uint8_t*>(a.src[t]) + (uint64_t)r0 * rb;
        const uint64_t dst_off = a.dst_off[t] + (uint64_t)par * a.dst_par_stride[t] + (uint64_t)(offset + r0) * rb;
        const long long nbytes = (long long)(r1 - r0) * rb;
        if (CHECK) {
          check_push(c, a.dst_off[t] + (uint64_t)par * a.dst_par_stride[t], (uint32_t)t, layer_base + (uint32_t)l,
                     (long long)(offset + r0) * (rb >> 2), nbytes >> 2, start, stride);
          continue;
        }
        if (W == 1 && (rb & 15u) == 0) copy_flat_local(c.heap_local + dst_off, src, nbytes, start, stride);
        else if ((rb & 15u) == 0) broadcast_flat<16>(c, src, dst_off, nbytes, start, stride);
        else if ((rb & 7u) == 0) broadcast_flat<8>(c, src, dst_off, nbytes, start, stride);
        else broadcast_flat<4>(c, src, dst_off, nbytes, start, stride);
      }
      if (W > 1) {
        __syncthreads();
        signal_all<true>(c, MCB_SITE_STEP, bid);
        if (tid == 0) {
          // The release above returns once this block's stores have left: the next group may push.
          if (G > 1) atomicAdd(a.state + MCB_STATE_GATE0 + grp, 1u);
          wait_flag(c, MCB_SITE_STEP, bid, (ep + 1u) * (uint32_t)W);
        }
        ++ep;
        __syncthreads();
      }
      if (CHECK) {
        // Words pushed by the matching block of every rank (this group's share of that rank's rows).
        for (int p = 0; p < W; ++p) {
          const int cnt = s_prefix[p + 1] - s_prefix[p];
          const int q0 = (int)((long long)cnt * grp / G), q1 = (int)((long long)cnt * (grp + 1) / G);
#pragma unroll
          for (int t = 0; t < MCB_MAX_TENSORS; ++t) {
            if (t >= a.num_tensors) break;
            const uint32_t rb = a.row_bytes[t];
            check_verify(c, a, a.dst_off[t] + (uint64_t)par * a.dst_par_stride[t], (uint32_t)t,
                         layer_base + (uint32_t)l, (long long)(s_prefix[p] + q0) * (rb >> 2),
                         (long long)(q1 - q0) * (rb >> 2), start, stride);
          }
        }
      }
      const long long nvec = (long long)(r1 - r0) * a.rsv_row_bytes / 16;
      if (W == 1)   // the sum over one rank is a copy (bit-exact for bf16 and fp32 alike)
        copy_flat_local(out + (uint64_t)r0 * a.rsv_row_bytes,
                        c.heap_local + a.rsv_off + (uint64_t)(offset + r0) * a.rsv_row_bytes, nvec * 16, start, stride);
      else
        reduce_flat(c, out + (uint64_t)r0 * a.rsv_row_bytes, a.rsv_off + (uint64_t)(offset + r0) * a.rsv_row_bytes,
                    nvec, start, stride, a.rsv_dtype);
    }
    if (tid == 0) *epoch_ptr(c, MCB_SITE_STEP, bid) = ep;
  }

  // ---- the last block out advances the sequence words ---------------------------------------------
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(a.state + MCB_STATE_FINISHED, 1u) == gridDim.x - 1u) {
      state[MCB_STATE_STEP_SEQ] = step_seq + 1u;
      state[MCB_STATE_LAYER_BASE] = layer_base + (uint32_t)L;
      state[MCB_STATE_LL_BASE] = ll_base + (ll ? (uint32_t)L : 0u);
      for (int g = 0; g < MCB_MAX_GROUPS; ++g) state[MCB_STATE_GATE0 + g] = 0u;
      state[MCB_STATE_FINISHED] = 0u;
      __threadfence();
    }
  }
}

}  // namespace mcb

using namespace mcb;

extern "C" {

int mcb_sizeof_dense_step_args() { return (int)sizeof(McbDenseStepArgs); }

static int check_step_args(const McbDenseStepArgs* a, int grid, int threads) {
  if (!a || grid < 1 || grid > MCB_MAX_BLOCKS || threads < 32 || threads > 512 || (threads & 31)) return 1;
  if (a->num_tensors < 1 || a->num_tensors > MCB_MAX_TENSORS || a->num_layers < 0 || a->cap < 1) return 1;
  if ((a->rsv_row_bytes & 15u) || !a->state || !a->step_meta || !a->n_local || !a->out) return 1;
  if (a->ll_rows > 0 && (a->credit_off == 0 || (a->credit_off & 3u))) return 1;
  for (int t = 0; t < a->num_tensors; ++t)
    if ((a->row_bytes[t] & 3u) || (!a->src[t] && !(a->fp8_hidden && t == 3))) return 1;
  if (a->fp8_hidden) {
    // quantised dispatch: tensor 0 = one byte per value, tensor 3 = one fp32 scale per 128 values
    if (a->check || a->num_tensors != 4 || a->fp8_hidden % 128u || a->row_bytes[0] != a->fp8_hidden ||
        a->row_bytes[3] != a->fp8_hidden / 128u * 4u)
      return 1;
  }
  return 0;
}

// The pipeline groups wait on one another inside the launch, so with groups > 1 all blocks must be
// resident at once: the launch is cooperative.
int mcb_launch_dense_step(const McbCtx* ctx, const McbDenseStepArgs* args, int grid, int threads, int pdl,
                          cudaStream_t stream) {
  if (!ctx || check_step_args(args, grid, threads)) return cudaErrorInvalidValue;
  const bool coop = args->groups > 1;
  if (args->check)
    return launch_kernel(dense_step_kernel<false, true, false>, dim3(grid), dim3(threads), 0, stream, pdl, coop, *ctx,
                         *args, (const McbCtx*)nullptr, (const McbDenseStepArgs*)nullptr);
  if (args->fp8_hidden)
    return launch_kernel(dense_step_kernel<false, false, true>, dim3(grid), dim3(threads), 0, stream, pdl, coop, *ctx,
                         *args, (const McbCtx*)nullptr, (const McbDenseStepArgs*)nullptr);
  return launch_kernel(dense_step_kernel<false, false, false>, dim3(grid), dim3(threads), 0, stream, pdl, coop, *ctx,
                       *args, (const McbCtx*)nullptr, (const McbDenseStepArgs*)nullptr);
}

int mcb_emu_dense_step(const McbCtx* d_ctx, const McbDenseStepArgs* d_args, const McbDenseStepArgs* h_args0,
                       int world, int grid, int threads, cudaStream_t stream) {
  if (!d_ctx || !d_args || world < 1 || check_step_args(h_args0, grid, threads)) return cudaErrorInvalidValue;
  McbCtx dummy{};
  McbDenseStepArgs dargs{};
  if (h_args0->check)
    return launch_kernel(dense_step_kernel<true, true, false>, dim3(grid, world), dim3(threads), 0, stream, 0, true,
                         dummy, dargs, d_ctx, d_args);
  if (h_args0->fp8_hidden)
    return launch_kernel(dense_step_kernel<true, false, true>, dim3(grid, world), dim3(threads), 0, stream, 0, true,
                         dummy, dargs, d_ctx, d_args);
  return launch_kernel(dense_step_kernel<true, false, false>, dim3(grid, world), dim3(threads), 0, stream, 0, true,
                       dummy, dargs, d_ctx, d_args);
}

}  // extern "C"
