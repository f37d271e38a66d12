// One whole decode step of the all-to-all dispatcher as ONE persistent kernel for sm_100a.
//
// Contract of the path the reference wraps (bench_deepep.py:68-115): a token travels once to every
// DISTINCT destination rank, routing travels with it, nothing synchronises with the host, and the
// combine returns, per source token, the sum of one row per destination rank.  The two-kernel form
// (a2a.cu) hands out compacted receive slots with atomic counters and publishes row counts; that
// costs two launches, a "last block" hand-over and a pull through a slot map per layer.  Here
//   * a token's slot on every destination is its own index (receive layout [parity][source][cap]):
//     no counters, no slot map, no hand-over; a destination tells valid rows by the stamp in the
//     row's metadata (the layer's sequence number), so stale rows of earlier layers never match;
//   * routing ids, weights, stamp and source index are one packed metadata row written with
//     16-byte stores ({stamp, token, (id, weight) x topk});
//   * a layer is: push -> ONE block-matched release barrier -> pull + fp32 sum, with the receive
//     buffers double buffered by layer parity (the barrier of layer l is the write-after-read fence
//     for the readers of layer l - 1), and the 88 layers run inside one launch after one count
//     exchange that also proves every rank has left the previous step;
//   * optional 1 x 128 block-scaled e4m3 dispatch, quantised on the way out;
//   * packet mode for small steps: rows travel as 16-byte flagged packets, so a layer needs no fence
//     and no barrier.  Every rank receives a one-packet header per token (routed to you or not), so a
//     destination knows which rows to wait for; the destination's warp for that token unpacks the row
//     into the ordinary receive buffers and sends the expert output straight back as packets, and the
//     source sums them as they arrive.  A token is served by a whole block (one 8-byte word per thread), all
//     traffic of a token runs between the same block index on the ranks involved, and the staging areas
//     (two parities) are recycled on per-source credit words.
// Every wait is bounded and reports through the status words.
#include <cuda_runtime.h>

#include "mcb_barrier.cuh"
#include "mcb_dense.cuh"
#include "mcb_fp8.cuh"
#include "mcb_launch.h"
#include "mcb_step.cuh"

namespace mcb {

struct DestMask { uint32_t w[3]; };    // 96 bits cover MCB_MAX_RANKS = 72

// Destination ranks of one token (all lanes of the warp get the same mask).
__device__ __forceinline__ DestMask dest_mask(const McbCtx& c, const McbA2AStepArgs& a, int t, int epr, int lane) {
  DestMask m = {{0u, 0u, 0u}};
  for (int k = lane; k < a.topk; k += 32) {
    const long long e = a.topk_idx[(long long)t * a.topk + k];
    if (e < 0 || e >= a.num_experts) {
      report_error(c, MCB_ERR_ROUTING, MCB_SITE_A2A_STEP, blockIdx.x, (uint32_t)t, (uint32_t)e);
      continue;
    }
    const int d = (int)(e / epr);
    m.w[d >> 5] |= 1u << (d & 31);
  }
#pragma unroll
  for (int i = 0; i < 3; ++i) m.w[i] = __reduce_or_sync(0xffffffffu, m.w[i]);
  return m;
}

// ---- packet mode ------------------------------------------------------------------------------------
struct LLShape {
  int xdata;      // 8-byte words of a dispatched row (bf16: hidden / 4, e4m3: hidden / 8)
  int scales;     // words of fp32 scales (e4m3 only: hidden / 256)
  int meta;       // words of the packed metadata row
  int xw;         // 1 header + xdata + scales + meta
  int yw;         // words of an expert-output row (hidden / 4)
};

__device__ __forceinline__ uint64_t ll_x_slot(const McbA2AStepArgs& a, const LLShape& s, int world, uint32_t par, int src,
                                              int t, int word) {
  return a.ll_x_off + ((((uint64_t)par * world + src) * a.ll_src_rows + t) * s.xw + word) * 16;
}
__device__ __forceinline__ uint64_t ll_y_slot(const McbA2AStepArgs& a, const LLShape& s, int world, uint32_t par, int dst,
                                              int t, int word) {
  return a.ll_y_off + ((((uint64_t)par * world + dst) * a.ll_src_rows + t) * s.yw + word) * 16;
}

// Send one 8-byte word of token t's row to every destination in the mask.
__device__ __forceinline__ void ll_send_x(const McbCtx& c, const McbA2AStepArgs& a, const LLShape& s, const DestMask& m,
                                          uint32_t par, int t, int word, uint2 d, uint32_t flag) {
  const uint4 pkt = ll_pack(d, flag);
#pragma unroll 1
  for (int wi = 0; wi < 3; ++wi) {
    uint32_t bits = m.w[wi];
    while (bits) {
      const int dst = wi * 32 + __ffs(bits) - 1;
      bits &= bits - 1;
      st_v4(c.heap_peer[dst] + ll_x_slot(a, s, c.world, par, c.rank, t, word), pkt);
    }
  }
}

// In packet mode a token is served by a whole BLOCK (steps are small, so blocks are plentiful, and a layer's
// latency is a chain of dependent loads: with one 8-byte word per thread the chain is one load deep).

// Source side of a layer: header to every rank, row / scales / metadata to the routed destinations.
__device__ __forceinline__ void ll_dispatch_token(const McbCtx& c, const McbA2AStepArgs& a, const LLShape& s, int t,
                                                  int epr, uint32_t par, uint32_t flag) {
  const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31;
  const DestMask m = dest_mask(c, a, t, epr, lane);
  for (int p = tid; p < c.world; p += nthreads) {
    const uint32_t routed = (m.w[p >> 5] >> (p & 31)) & 1u;
    st_v4(c.heap_peer[p] + ll_x_slot(a, s, c.world, par, c.rank, t, 0), ll_pack(make_uint2(routed, (uint32_t)t), flag));
  }
  const uint8_t* xrow = reinterpret_cast<const uint8_t*>(a.x) + (uint64_t)t * a.hidden * 2;
  if (!a.fp8) {
    for (int j = tid; j < s.xdata; j += nthreads) ll_send_x(c, a, s, m, par, t, 1 + j, ld_v2(xrow + (uint64_t)j * 8), flag);
  } else {
    const int row_packs = a.hidden / 8;               // a multiple of 32 (hidden % 256 == 0): warps are all in or all out
    for (int p = tid; p < row_packs; p += nthreads) {
      const uint4 v = ld_v4(xrow + (uint64_t)p * 16);
      float amax = pack_absmax(v);                     // 16 lanes hold one 128-value block
#pragma unroll
      for (int sh = 8; sh >= 1; sh >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
      const float scale = e4m3_scale(amax);
      ll_send_x(c, a, s, m, par, t, 1 + p, quant_pack_e4m3(v, scale), flag);
      // lanes 0-15 hold one block, lanes 16-31 the next one: one word carries both scales
      const float other = __shfl_sync(0xffffffffu, scale, 16);
      if (lane == 0)
        ll_send_x(c, a, s, m, par, t, 1 + s.xdata + (p >> 5), make_uint2(__float_as_uint(scale), __float_as_uint(other)), flag);
    }
  }
  // metadata row: chunk 0 = {stamp, token, id 0, weight 0}, chunk j = {id 2j-1, weight 2j-1, id 2j, weight 2j};
  // taken from the top of the block so that it does not queue behind the row words of the low threads
  for (int j = nthreads - 1 - tid; j < s.meta / 2; j += nthreads) {
    const int k0 = j == 0 ? 0 : 2 * j - 1, k1 = 2 * j;
    const long long tb = (long long)t * a.topk;
    const uint32_t id0 = k0 < a.topk ? (uint32_t)a.topk_idx[tb + k0] : 0xffffffffu;
    const uint32_t w0 = k0 < a.topk ? __float_as_uint(a.topk_w ? a.topk_w[tb + k0] : 1.0f) : 0u;
    uint2 lo, hi;
    if (j == 0) {
      lo = make_uint2(flag, (uint32_t)t);
      hi = make_uint2(id0, w0);
    } else {
      const uint32_t id1 = k1 < a.topk ? (uint32_t)a.topk_idx[tb + k1] : 0xffffffffu;
      const uint32_t w1 = k1 < a.topk ? __float_as_uint(a.topk_w ? a.topk_w[tb + k1] : 1.0f) : 0u;
      lo = make_uint2(id0, w0);
      hi = make_uint2(id1, w1);
    }
    ll_send_x(c, a, s, m, par, t, 1 + s.xdata + s.scales + 2 * j, lo, flag);
    ll_send_x(c, a, s, m, par, t, 1 + s.xdata + s.scales + 2 * j + 1, hi, flag);
  }
}

// Destination side: wait for the header of (source, token); if the token is routed here, unpack its row
// into the ordinary receive buffers and send the expert output (the row itself for the identity expert
// in bf16, the y buffer otherwise) back to the source.
__device__ __forceinline__ void ll_serve_token(const McbCtx& c, const McbA2AStepArgs& a, const LLShape& s, int src, int t,
                                               uint32_t par, uint32_t flag) {
  const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31;
  uint32_t routed = 0;
  if (lane == 0) routed = ll_wait(c, c.heap_local + ll_x_slot(a, s, c.world, par, src, t, 0), flag, MCB_SITE_A2A_STEP).x;
  routed = __shfl_sync(0xffffffffu, routed, 0);
  if (!routed) return;
  const uint64_t row = (uint64_t)src * a.cap + t;
  const uint64_t xrow_bytes = a.fp8 ? (uint64_t)a.hidden : (uint64_t)a.hidden * 2;
  uint8_t* rx = c.heap_local + a.recv_x_off + (uint64_t)par * a.x_par_stride + row * xrow_bytes;
  uint8_t* rs = c.heap_local + a.recv_scale_off + (uint64_t)par * a.scale_par_stride + row * (uint64_t)(a.hidden / 128) * 4;
  uint8_t* rm = c.heap_local + a.recv_meta_off + (uint64_t)par * a.meta_par_stride + row * a.meta_row_bytes;
  const uint8_t* yrow = c.heap_local + a.y_off + (uint64_t)par * a.y_par_stride + row * (uint64_t)a.hidden * 2;
  const int body = s.xdata + s.scales + s.meta;
  const bool echo = !a.fp8 && a.y_off == a.recv_x_off;     // identity expert on bf16 rows: the row is its own output
  if (!echo)     // the expert output is a bf16 row of its own: it can leave before the row has arrived
    for (int j = tid; j < s.yw; j += nthreads)
      st_v4(c.heap_peer[src] + ll_y_slot(a, s, c.world, par, c.rank, t, j), ll_pack(ld_v2(yrow + (uint64_t)j * 8), flag));
  for (int j = tid; j < body; j += nthreads) {
    const uint2 d = ll_wait(c, c.heap_local + ll_x_slot(a, s, c.world, par, src, t, 1 + j), flag, MCB_SITE_A2A_STEP);
    if (j < s.xdata) {
      if (echo) st_v4(c.heap_peer[src] + ll_y_slot(a, s, c.world, par, c.rank, t, j), ll_pack(d, flag));
      st_v2(rx + (uint64_t)j * 8, d);
    } else if (j < s.xdata + s.scales) {
      st_v2(rs + (uint64_t)(j - s.xdata) * 8, d);
    } else {
      st_v2(rm + (uint64_t)(j - s.xdata - s.scales) * 8, d);
    }
  }
}

__device__ __forceinline__ int pop_dest(DestMask& m) {
#pragma unroll
  for (int wi = 0; wi < 3; ++wi)
    if (m.w[wi]) {
      const int b = __ffs(m.w[wi]) - 1;
      m.w[wi] &= m.w[wi] - 1;
      return wi * 32 + b;
    }
  return -1;
}

// Source side again: sum the expert outputs of every destination as their packets arrive (four
// destinations' packets in flight per thread).
__device__ __forceinline__ void ll_combine_token(const McbCtx& c, const McbA2AStepArgs& a, const LLShape& s, int t,
                                                 int epr, uint32_t par, uint32_t flag) {
  const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31;
  const DestMask m = dest_mask(c, a, t, epr, lane);
  uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) + (uint64_t)t * a.hidden * 2;
  for (int j = tid; j < s.yw; j += nthreads) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    DestMask rest = m;
    for (;;) {
      int d[4];
      d[0] = pop_dest(rest);
      if (d[0] < 0) break;
#pragma unroll
      for (int u = 1; u < 4; ++u) d[u] = pop_dest(rest);
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (d[u] >= 0) v[u] = ld_v4_volatile(c.heap_local + ll_y_slot(a, s, c.world, par, d[u], t, j));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (d[u] < 0) continue;
        uint2 w = make_uint2(v[u].x, v[u].z);
        if (v[u].y != flag || v[u].w != flag)
          w = ll_wait(c, c.heap_local + ll_y_slot(a, s, c.world, par, d[u], t, j), flag, MCB_SITE_A2A_STEP);
        acc[0] += bf16_lo(w.x); acc[1] += bf16_hi(w.x);
        acc[2] += bf16_lo(w.y); acc[3] += bf16_hi(w.y);
      }
    }
    st_v2(orow + (uint64_t)j * 8, make_uint2(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3])));
  }
}

// Packet-mode layers of a step: global token g belongs to block g % blocks on every rank.  Kept out of line
// so that the two modes do not share one register allocation.
__device__ __noinline__ void packet_layers(const McbCtx& c, const McbA2AStepArgs& a, const LLShape& shp, const int* s_prefix,
                                           int n, int valid, uint32_t layer_base) {
  const int tid = threadIdx.x, bid = blockIdx.x;
  const int W = c.world, L = a.num_layers;
  const int nb = valid < (int)gridDim.x ? valid : (int)gridDim.x;
  if (bid >= nb) return;
  const int epr_ll = a.num_experts / W;
  const int offset = s_prefix[c.rank];
  const uint32_t cb = *epoch_ptr(c, MCB_SITE_A2A_STEP_CREDIT, bid);
  const int t0 = ((bid - offset) % nb + nb) % nb;      // first own token with (offset + t) % nb == bid
  for (int l = 0; l < L; ++l) {
    const uint32_t par = (layer_base + (uint32_t)l) & 1u;
    const uint32_t flag = layer_base + (uint32_t)l + 1u;
    // the staging areas of this parity were read last in layer l - 2
    if (l >= 2) credit_wait(c, a.credit_off, cb + (uint32_t)l - 1u, MCB_SITE_A2A_STEP_CREDIT);
    for (int t = t0; t < n; t += nb) ll_dispatch_token(c, a, shp, t, epr_ll, par, flag);
    for (int g = bid; g < valid; g += nb) {
      int src = 0;
      while (src + 1 < W && s_prefix[src + 1] <= g) ++src;
      ll_serve_token(c, a, shp, src, g - s_prefix[src], par, flag);
    }
    for (int t = t0; t < n; t += nb) ll_combine_token(c, a, shp, t, epr_ll, par, flag);
    __syncthreads();
    credit_publish(c, a.credit_off, cb + (uint32_t)l + 1u);
  }
  if (tid == 0) *epoch_ptr(c, MCB_SITE_A2A_STEP_CREDIT, bid) = cb + (uint32_t)L;
}

// Barrier-mode layers of a step: push -> one block-matched barrier -> pull + fp32 sum.  Out of line, as above.
__device__ __noinline__ void barrier_layers(const McbCtx& c, const McbA2AStepArgs& a, int n, int ep_max, uint32_t layer_base) {
  const int tid = threadIdx.x, bid = blockIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int W = c.world, L = a.num_layers;
  // One warp per token; as many blocks as the largest rank needs, the same on every rank.
  int nact = (ep_max + nwarps - 1) / nwarps;
  nact = nact > (int)gridDim.x ? (int)gridDim.x : nact;
  const int epr = a.num_experts / W;
  const int row_packs = a.hidden / 8;
  const uint64_t row_bytes = (uint64_t)a.hidden * 2;
  const uint64_t xrow_bytes = a.fp8 ? (uint64_t)a.hidden : row_bytes;     // bytes of a dispatched row
  const int nblk = a.hidden / 128;
  const int meta_chunks = (int)(a.meta_row_bytes >> 4);
  const uint8_t* x = reinterpret_cast<const uint8_t*>(a.x);
  uint8_t* out = reinterpret_cast<uint8_t*>(a.out);

  if (bid < nact) {
    uint32_t ep = *epoch_ptr(c, MCB_SITE_A2A_STEP, bid);
    for (int l = 0; l < L; ++l) {
      const uint32_t par = (layer_base + (uint32_t)l) & 1u;
      const uint32_t stamp = layer_base + (uint32_t)l + 1u;
      const uint64_t slot0 = (uint64_t)c.rank * a.cap;            // first row of this source on a destination
      // ---- push: row (+ scales) and metadata to every distinct destination rank ----
      for (int t = bid * nwarps + warp; t < n; t += nact * nwarps) {
        const DestMask m = dest_mask(c, a, t, epr, lane);
        const uint8_t* xrow = x + (uint64_t)t * row_bytes;
        const uint64_t row = slot0 + t;
        for (int p0 = 0; p0 < row_packs; p0 += 128) {
          uint4 v[4];
          uint2 q[4];
          float scale[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int p = p0 + u * 32 + lane;
            v[u] = p < row_packs ? ld_v4(xrow + (uint64_t)p * 16) : make_uint4(0, 0, 0, 0);
          }
          if (a.fp8) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              float amax = pack_absmax(v[u]);          // 16 lanes hold one 128-value block
#pragma unroll
              for (int sh = 8; sh >= 1; sh >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
              scale[u] = e4m3_scale(amax);
              q[u] = quant_pack_e4m3(v[u], scale[u]);
            }
          }
#pragma unroll 1
          for (int wi = 0; wi < 3; ++wi) {
            uint32_t bits = m.w[wi];
            while (bits) {
              const int d = wi * 32 + __ffs(bits) - 1;
              bits &= bits - 1;
              uint8_t* peer = c.heap_peer[d];
              uint8_t* dst = peer + a.recv_x_off + (uint64_t)par * a.x_par_stride + row * xrow_bytes;
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int p = p0 + u * 32 + lane;
                if (p >= row_packs) continue;
                if (a.fp8) {
                  st_v2(dst + (uint64_t)p * 8, q[u]);
                  if ((lane & 15) == 0)
                    st_b32(peer + a.recv_scale_off + (uint64_t)par * a.scale_par_stride + (row * nblk + (p >> 4)) * 4,
                           __float_as_uint(scale[u]));
                } else {
                  st_v4(dst + (uint64_t)p * 16, v[u]);
                }
              }
            }
          }
        }
        // metadata row: chunk 0 = {stamp, token, id 0, weight 0}, chunk j = {id 2j-1, weight 2j-1, id 2j, weight 2j}
        for (int j = lane; j < meta_chunks; j += 32) {
          uint4 ch;
          const int k0 = j == 0 ? 0 : 2 * j - 1, k1 = 2 * j;
          const long long tb = (long long)t * a.topk;
          const uint32_t id0 = k0 < a.topk ? (uint32_t)a.topk_idx[tb + k0] : 0xffffffffu;
          const uint32_t w0 = k0 < a.topk ? __float_as_uint(a.topk_w ? a.topk_w[tb + k0] : 1.0f) : 0u;
          if (j == 0) {
            ch = make_uint4(stamp, (uint32_t)t, id0, w0);
          } else {
            const uint32_t id1 = k1 < a.topk ? (uint32_t)a.topk_idx[tb + k1] : 0xffffffffu;
            const uint32_t w1 = k1 < a.topk ? __float_as_uint(a.topk_w ? a.topk_w[tb + k1] : 1.0f) : 0u;
            ch = make_uint4(id0, w0, id1, w1);
          }
#pragma unroll 1
          for (int wi = 0; wi < 3; ++wi) {
            uint32_t bits = m.w[wi];
            while (bits) {
              const int d = wi * 32 + __ffs(bits) - 1;
              bits &= bits - 1;
              st_v4(c.heap_peer[d] + a.recv_meta_off + (uint64_t)par * a.meta_par_stride + row * a.meta_row_bytes +
                        (uint64_t)j * 16, ch);
            }
          }
        }
      }
      // ---- one barrier: the matching block of every rank has pushed its tokens of this layer ----
      if (W > 1) {
        __syncthreads();
        signal_all<true>(c, MCB_SITE_A2A_STEP, bid);
        if (tid == 0) wait_flag(c, MCB_SITE_A2A_STEP, bid, (ep + 1u) * (uint32_t)W);
        ++ep;
        __syncthreads();
      }
      // ---- pull: one expert-output row per destination rank, summed in fp32 ----
      for (int t = bid * nwarps + warp; t < n; t += nact * nwarps) {
        const DestMask m = dest_mask(c, a, t, epr, lane);
        const uint64_t yoff = a.y_off + (uint64_t)par * a.y_par_stride + (slot0 + t) * row_bytes;
        for (int p0 = 0; p0 < row_packs; p0 += 128) {
          float acc[4][8];
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
#pragma unroll 1
          for (int wi = 0; wi < 3; ++wi) {
            uint32_t bits = m.w[wi];
            while (bits) {
              // two destinations per round: 8 independent 16-byte peer loads in flight per lane
              const int d0 = wi * 32 + __ffs(bits) - 1;
              bits &= bits - 1;
              int d1 = -1;
              if (bits) { d1 = wi * 32 + __ffs(bits) - 1; bits &= bits - 1; }
              uint4 v0[4], v1[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int p = p0 + u * 32 + lane;
                const bool in = p < row_packs;
                v0[u] = in ? ld_v4_stream(c.heap_peer[d0] + yoff + (uint64_t)p * 16) : make_uint4(0, 0, 0, 0);
                v1[u] = in && d1 >= 0 ? ld_v4_stream(c.heap_peer[d1] + yoff + (uint64_t)p * 16) : make_uint4(0, 0, 0, 0);
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                acc[u][0] += bf16_lo(v0[u].x) + bf16_lo(v1[u].x); acc[u][1] += bf16_hi(v0[u].x) + bf16_hi(v1[u].x);
                acc[u][2] += bf16_lo(v0[u].y) + bf16_lo(v1[u].y); acc[u][3] += bf16_hi(v0[u].y) + bf16_hi(v1[u].y);
                acc[u][4] += bf16_lo(v0[u].z) + bf16_lo(v1[u].z); acc[u][5] += bf16_hi(v0[u].z) + bf16_hi(v1[u].z);
                acc[u][6] += bf16_lo(v0[u].w) + bf16_lo(v1[u].w); acc[u][7] += bf16_hi(v0[u].w) + bf16_hi(v1[u].w);
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int p = p0 + u * 32 + lane;
            if (p < row_packs)
              st_v4(out + (uint64_t)t * row_bytes + (uint64_t)p * 16,
                    make_uint4(pack_bf16x2(acc[u][0], acc[u][1]), pack_bf16x2(acc[u][2], acc[u][3]),
                               pack_bf16x2(acc[u][4], acc[u][5]), pack_bf16x2(acc[u][6], acc[u][7])));
          }
        }
      }
    }
    if (tid == 0) *epoch_ptr(c, MCB_SITE_A2A_STEP, bid) = ep;
  }

}

template <bool EMU>
__global__ void __launch_bounds__(512) a2a_step_kernel(const __grid_constant__ McbCtx ctx_p,
                                                       const __grid_constant__ McbA2AStepArgs args_p,
                                                       const McbCtx* ectx, const McbA2AStepArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbA2AStepArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  __shared__ int s_prefix[MCB_MAX_RANKS + 1];
  __shared__ int s_cnt[MCB_MAX_RANKS];
  __shared__ int s_max;
  const int tid = threadIdx.x, bid = blockIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int W = c.world, L = a.num_layers;
  pdl_wait();
  pdl_launch_dependents();
  volatile uint32_t* state = a.state;
  const uint32_t step_seq = state[MCB_STATE_STEP_SEQ], layer_base = state[MCB_STATE_LAYER_BASE];
  const int n = step_count_exchange(c, MCB_SITE_A2A_STEP_META, a.counts_off, step_seq, *a.n_local, a.cap, s_cnt,
                                    s_prefix, &s_max);
  const int ep_max = s_max;
  if (bid == 0 && tid == 0) {
    a.step_meta[0] = s_prefix[W];
    a.step_meta[1] = s_prefix[c.rank];
    a.step_meta[2] = ep_max;
    a.step_meta[4] = (int)(step_seq + 1u);
    a.step_meta[5] = L > 0 ? (int)((layer_base + (uint32_t)L - 1u) & 1u) : 0;
    a.step_meta[7] = (int)(layer_base + (uint32_t)L);     // stamp of the last layer's rows
  }
  const int valid = s_prefix[W];
  LLShape shp;
  shp.xdata = a.fp8 ? a.hidden / 8 : a.hidden / 4;
  shp.scales = a.fp8 ? a.hidden / 256 : 0;
  shp.meta = (int)(a.meta_row_bytes >> 3);
  shp.xw = 1 + shp.xdata + shp.scales + shp.meta;
  shp.yw = a.hidden / 4;
  const bool ll = W > 1 && a.ll_rows > 0 && valid > 0 && valid <= a.ll_rows && (!a.fp8 || a.hidden % 256 == 0);
  if (bid == 0 && tid == 0) a.step_meta[6] = ll ? 1 : 0;
  if (ll) {
    packet_layers(c, a, shp, s_prefix, n, valid, layer_base);
  } else {
    barrier_layers(c, a, n, ep_max, layer_base);
  }
  // ---- the last block out advances the sequence words ----
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(a.state + MCB_STATE_FINISHED, 1u) == gridDim.x - 1u) {
      state[MCB_STATE_STEP_SEQ] = step_seq + 1u;
      state[MCB_STATE_LAYER_BASE] = layer_base + (uint32_t)L;
      state[MCB_STATE_FINISHED] = 0u;
      __threadfence();
    }
  }
}

}  // namespace mcb

using namespace mcb;

extern "C" {

int mcb_sizeof_a2a_step_args() { return (int)sizeof(McbA2AStepArgs); }

static int check_a2a_step(const McbCtx* ctx, const McbA2AStepArgs* a, int grid, int threads) {
  if (!ctx || !a || grid < 1 || grid > MCB_MAX_BLOCKS || threads < 32 || threads > 512 || (threads & 31)) return 1;
  if (!a->x || !a->topk_idx || !a->out || !a->n_local || !a->state || !a->step_meta) return 1;
  if (a->hidden < 8 || a->hidden % 8 || (a->fp8 && a->hidden % 128) || a->topk < 1 || a->cap < 1 || a->num_layers < 0) return 1;
  if (ctx->world < 1 || a->num_experts % ctx->world) return 1;
  if ((a->meta_row_bytes & 15u) || a->meta_row_bytes < 8u + 8u * (uint32_t)a->topk) return 1;
  if (a->ll_rows > 0 && (!a->ll_x_off || !a->ll_y_off || !a->credit_off || a->ll_src_rows < 1 || a->hidden % 4)) return 1;
  return 0;
}

int mcb_launch_a2a_step(const McbCtx* ctx, const McbA2AStepArgs* args, int grid, int threads, int pdl,
                        cudaStream_t stream) {
  if (check_a2a_step(ctx, args, grid, threads)) return cudaErrorInvalidValue;
  return launch_kernel(a2a_step_kernel<false>, dim3(grid), dim3(threads), 0, stream, pdl, false, *ctx, *args,
                       (const McbCtx*)nullptr, (const McbA2AStepArgs*)nullptr);
}

int mcb_emu_a2a_step(const McbCtx* d_ctx, const McbA2AStepArgs* d_args, const McbCtx* h_ctx0,
                     const McbA2AStepArgs* h_args0, int world, int grid, int threads, cudaStream_t stream) {
  if (!d_ctx || !d_args || world < 1 || check_a2a_step(h_ctx0, h_args0, grid, threads)) return cudaErrorInvalidValue;
  McbCtx dummy{};
  McbA2AStepArgs dargs{};
  return launch_kernel(a2a_step_kernel<true>, dim3(grid, world), dim3(threads), 0, stream, 0, true, dummy, dargs,
                       d_ctx, d_args);
}

}  // extern "C"
