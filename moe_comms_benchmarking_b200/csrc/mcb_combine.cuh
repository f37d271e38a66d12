// Combine body shared by the stand-alone combine kernel and the fused FC2 + combine kernel.
//
// Block b owns the gathered tokens t with t % nact == b on EVERY rank.
//   phase A  partial[t] = sum over the local (token, k) pairs of y[pair]       (this rank's heap)
//   barrier  block b of every rank has written its tokens' partial sums
//   phase B  for the tokens of block b that this rank owns: out = sum over ranks of partial[t]
//            (multimem.ld_reduce in the switch, or peer loads).
// While there are no more tokens than blocks a block serves ONE token and spreads the row's 16-byte
// packs over its warps, so each phase is a chain of one or two dependent loads; with more tokens a
// warp serves a token (throughput form).
// Call from all threads of the block; works for any block size that is a multiple of 32.
#pragma once
#include "mcb_barrier.cuh"
#include "mcb_gemm.h"

namespace mcb {

// Sum over ranks of one 16-byte pack of the partial buffers (phase B).
__device__ __forceinline__ uint4 combine_reduce_pack(const McbCtx& c, uint64_t off) {
  if (c.transport == MCB_TRANSPORT_MULTIMEM) return mm_ld_reduce_bf16x8(c.heap_mc + off);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < c.world; k0 += 8) {       // eight peers' loads in flight
    uint4 w[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      int q = c.rank + k0 + u;
      if (q >= c.world) q -= c.world;
      w[u] = k0 + u < c.world ? ld_v4_stream(c.heap_peer[q] + off) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      acc[0] += bf16_lo(w[u].x); acc[1] += bf16_hi(w[u].x);
      acc[2] += bf16_lo(w[u].y); acc[3] += bf16_hi(w[u].y);
      acc[4] += bf16_lo(w[u].z); acc[5] += bf16_hi(w[u].z);
      acc[6] += bf16_lo(w[u].w); acc[7] += bf16_hi(w[u].w);
    }
  }
  return make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                    pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
}

__device__ __forceinline__ void combine_body(const McbCtx& c, const McbCombineArgs& a, uint32_t parity = 0u) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int T = a.step_meta[0], offset = a.step_meta[1];
  int n = *a.n_local;
  if (n < 0) n = 0;
  if (n > a.cap) n = a.cap;
  if (T <= 0) return;
  // One token per block while there are fewer tokens than blocks (shortest critical path), the
  // whole grid otherwise; identical on every rank.
  int nact = T < (int)gridDim.x ? T : (int)gridDim.x;
  const int bid = blockIdx.x;
  if (bid >= nact) return;
  const uint32_t ep = *epoch_ptr(c, a.site, bid);
  const int packs = a.hidden / 8;
  const uint64_t row_bytes = (uint64_t)a.hidden * 2;
  const uint8_t* y = reinterpret_cast<const uint8_t*>(a.y);
  const uint64_t partial_off = a.partial_off + (uint64_t)(parity & 1u) * a.partial_par_stride;
  uint8_t* partial = c.heap_local + partial_off;

  if (T <= (int)gridDim.x) {
    // ---- one token per block (nact == T): warp w takes packs w*32 .. w*32+31 of the row ----
    const int t = bid;
    for (int p0 = warp * 32; p0 < packs; p0 += nwarps * 32) {
      const int p = p0 + lane;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k0 = 0; k0 < a.topk; k0 += 32) {
        const int k = k0 + lane;
        const int my_pos = k < a.topk ? a.pair_pos[(long long)t * a.topk + k] : -1;
        uint32_t have = __ballot_sync(0xffffffffu, my_pos >= 0);
        while (have) {          // two local pair rows in flight
          const int l0 = __ffs(have) - 1;
          have &= have - 1;
          const int l1 = have ? __ffs(have) - 1 : -1;
          if (have) have &= have - 1;
          const int pos0 = __shfl_sync(0xffffffffu, my_pos, l0);
          const int pos1 = __shfl_sync(0xffffffffu, my_pos, l1 < 0 ? l0 : l1);
          uint4 v0 = make_uint4(0, 0, 0, 0), v1 = make_uint4(0, 0, 0, 0);
          if (p < packs) {
            v0 = ld_v4(y + (uint64_t)pos0 * row_bytes + (uint64_t)p * 16);
            if (l1 >= 0) v1 = ld_v4(y + (uint64_t)pos1 * row_bytes + (uint64_t)p * 16);
          }
          acc[0] += bf16_lo(v0.x) + bf16_lo(v1.x); acc[1] += bf16_hi(v0.x) + bf16_hi(v1.x);
          acc[2] += bf16_lo(v0.y) + bf16_lo(v1.y); acc[3] += bf16_hi(v0.y) + bf16_hi(v1.y);
          acc[4] += bf16_lo(v0.z) + bf16_lo(v1.z); acc[5] += bf16_hi(v0.z) + bf16_hi(v1.z);
          acc[6] += bf16_lo(v0.w) + bf16_lo(v1.w); acc[7] += bf16_hi(v0.w) + bf16_hi(v1.w);
        }
      }
      if (p < packs)
        st_v4(partial + (uint64_t)t * row_bytes + (uint64_t)p * 16,
              make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                         pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7])));
    }
    block_barrier_all(c, a.site, bid, ep);
    if (t >= offset && t < offset + n) {
      uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) + (uint64_t)(t - offset) * row_bytes;
      for (int p = threadIdx.x; p < packs; p += blockDim.x)
        st_v4(orow + (uint64_t)p * 16, combine_reduce_pack(c, partial_off + (uint64_t)t * row_bytes + (uint64_t)p * 16));
    }
    return;
  }

  for (int t = bid + warp * nact; t < T; t += nact * nwarps) {
    // Pair rows of this token on this rank: lanes read the token's routing slots in parallel,
    // then the warp walks only the local ones.
    for (int p0 = 0; p0 < packs; p0 += 128) {
      float acc[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
      for (int k0 = 0; k0 < a.topk; k0 += 32) {
        const int k = k0 + lane;
        const int my_pos = k < a.topk ? a.pair_pos[(long long)t * a.topk + k] : -1;
        uint32_t have = __ballot_sync(0xffffffffu, my_pos >= 0);
        while (have) {
          const int src_lane = __ffs(have) - 1;
          have &= have - 1;
          const int pos = __shfl_sync(0xffffffffu, my_pos, src_lane);
          const uint8_t* row = y + (uint64_t)pos * row_bytes;
          uint4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int p = p0 + u * 32 + lane;
            v[u] = p < packs ? ld_v4(row + (uint64_t)p * 16) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            acc[u][0] += bf16_lo(v[u].x); acc[u][1] += bf16_hi(v[u].x);
            acc[u][2] += bf16_lo(v[u].y); acc[u][3] += bf16_hi(v[u].y);
            acc[u][4] += bf16_lo(v[u].z); acc[u][5] += bf16_hi(v[u].z);
            acc[u][6] += bf16_lo(v[u].w); acc[u][7] += bf16_hi(v[u].w);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int p = p0 + u * 32 + lane;
        if (p < packs)
          st_v4(partial + (uint64_t)t * row_bytes + (uint64_t)p * 16,
                make_uint4(pack_bf16x2(acc[u][0], acc[u][1]), pack_bf16x2(acc[u][2], acc[u][3]),
                           pack_bf16x2(acc[u][4], acc[u][5]), pack_bf16x2(acc[u][6], acc[u][7])));
      }
    }
  }
  block_barrier_all(c, a.site, bid, ep);

  uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
  for (int t = bid + warp * nact; t < T; t += nact * nwarps) {
    if (t < offset || t >= offset + n) continue;
    for (int p0 = lane; p0 < packs; p0 += 128) {       // four packs in flight per lane
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (p0 + u * 32 < packs) v[u] = combine_reduce_pack(c, partial_off + (uint64_t)t * row_bytes + (uint64_t)(p0 + u * 32) * 16);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (p0 + u * 32 < packs) st_v4(out + (uint64_t)(t - offset) * row_bytes + (uint64_t)(p0 + u * 32) * 16, v[u]);
    }
  }
}

}  // namespace mcb
