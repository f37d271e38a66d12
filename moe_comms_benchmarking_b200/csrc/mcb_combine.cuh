// Combine body shared by the stand-alone combine kernel and the fused FC2 + combine kernel.
//
// Block b owns the gathered tokens t with t % nact == b on EVERY rank.
//   phase A  partial[t] = sum over the local (token, k) pairs of y[pair]       (this rank's heap)
//   barrier  block b of every rank has written its tokens' partial sums
//   phase B  for the tokens of block b that this rank owns: out = sum over ranks of partial[t]
//            (multimem.ld_reduce in the switch, or peer loads).
// Call from all threads of the block; works for any block size that is a multiple of 32.
#pragma once
#include "mcb_barrier.cuh"
#include "mcb_gemm.h"

namespace mcb {

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
    for (int p = lane; p < packs; p += 32) {
      const uint64_t off = partial_off + (uint64_t)t * row_bytes + (uint64_t)p * 16;
      uint4 v;
      if (c.transport == MCB_TRANSPORT_MULTIMEM) {
        v = mm_ld_reduce_bf16x8(c.heap_mc + off);
      } else {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < c.world; ++k) {
          int q = c.rank + k;
          if (q >= c.world) q -= c.world;
          const uint4 w = ld_v4_stream(c.heap_peer[q] + off);
          acc[0] += bf16_lo(w.x); acc[1] += bf16_hi(w.x);
          acc[2] += bf16_lo(w.y); acc[3] += bf16_hi(w.y);
          acc[4] += bf16_lo(w.z); acc[5] += bf16_hi(w.z);
          acc[6] += bf16_lo(w.w); acc[7] += bf16_hi(w.w);
        }
        v = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                       pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
      }
      st_v4(out + (uint64_t)(t - offset) * row_bytes + (uint64_t)p * 16, v);
    }
  }
}

}  // namespace mcb
