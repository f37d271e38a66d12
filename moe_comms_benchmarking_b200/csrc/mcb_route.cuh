// Routing of the gathered tokens to this rank's experts as a device function (histogram ->
// offsets -> pair lists -> row-tile table), shared by the stand-alone routing kernel and the
// fused dispatch + routing + FC1 kernel.
#pragma once
#include "mcb_barrier.cuh"
#include "mcb_gemm.h"

namespace mcb {

constexpr int kRouteThreads = 1024;
constexpr int kMaxLocalExperts = 1024;
constexpr int kSingleBlockPerThread = 20;    // (token, k) entries per thread up to which ONE block routes alone

__device__ __forceinline__ bool spin_until_ge(const volatile int* p, int target, uint64_t timeout_ns) {
  if (*p - target >= 0) return true;
  uint64_t t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (*p - target >= 0) return true;
    if (globaltimer_ns() - t0 > timeout_ns) return false;
  }
}

// Exclusive prefix of the per-expert pair counts s_cnt[0..E) into a.expert_offset[0..E], the
// 128-row tile table of the tokens-as-rows GEMMs, the largest count, and the per-expert "gate/up
// blocks done" counters of the fused FFN back at zero.  One warp: every lane owns a contiguous
// run of experts, the runs are joined with a shuffle scan (E <= 1024 means at most 32 experts per
// lane, instead of a serial walk over all of them on one thread).  Call from the 32 threads of
// ONE warp; s_cnt must be visible to them.  Returns the total in every lane.
__device__ __forceinline__ int route_offsets(const McbRouteArgs& a, const int* s_cnt, int* s_off, int E) {
  const int lane = threadIdx.x & 31;
  const int per = (E + 31) / 32;
  const int e0 = lane * per, e1 = e0 + per < E ? e0 + per : E;
  int rows = 0, tiles = 0, mx = 0;
  for (int e = e0; e < e1; ++e) {
    const int c = s_cnt[e];
    rows += c;
    tiles += (c + 127) >> 7;
    mx = c > mx ? c : mx;
  }
  int row_pre = rows, tile_pre = tiles;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int r = __shfl_up_sync(0xffffffffu, row_pre, o), t = __shfl_up_sync(0xffffffffu, tile_pre, o);
    if (lane >= o) { row_pre += r; tile_pre += t; }
  }
  const int total = __shfl_sync(0xffffffffu, row_pre, 31), total_tiles = __shfl_sync(0xffffffffu, tile_pre, 31);
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  int run = row_pre - rows, tile = tile_pre - tiles;
  for (int e = e0; e < e1; ++e) {
    const int c = s_cnt[e];
    if (s_off) s_off[e] = run;
    a.expert_offset[e] = run;
    if (a.ffn_done) a.ffn_done[e] = 0;
    for (int r0 = 0; r0 < c; r0 += 128, ++tile) {
      if (tile < a.max_tiles) {
        a.tile_expert[tile] = e;
        a.tile_row0[tile] = run + r0;
        a.tile_rows[tile] = c - r0 < 128 ? c - r0 : 128;
      }
    }
    run += c;
  }
  if (lane == 0) {
    a.expert_offset[E] = total;
    if (a.max_rows) *a.max_rows = mx;
    if (total_tiles > a.max_tiles || total > a.max_pairs) {
      if (a.status && atomicCAS(a.status, 0u, (uint32_t)MCB_ERR_CAPACITY) == 0u) {
        a.status[1] = 100; a.status[2] = (uint32_t)total_tiles; a.status[3] = (uint32_t)total;
      }
    }
    *a.num_m_tiles = total_tiles < a.max_tiles ? total_tiles : a.max_tiles;
  }
  return total;
}

// One launch, two phases separated by a "last block computes the offsets" hand-over; blocks of
// the same launch wait for it on a local counter, so the grid must be co-resident (<= #SMs).
// Call from all threads of every block of the grid.
__device__ __forceinline__ void route_device(const McbRouteArgs& a) {
  __shared__ int s_hist[kMaxLocalExperts];
  __shared__ int s_flag;
  const int tid = threadIdx.x;
  const int E = a.num_local_experts;
  int T = *a.num_tokens;
  if (T < 0) T = 0;
  if (T > a.max_tokens) T = a.max_tokens;
  const int ready_base = *reinterpret_cast<volatile int*>(&a.sync[2]);   // stable until this launch's hand-over
  const long long entries = (long long)T * a.topk;
  if (entries <= (long long)kSingleBlockPerThread * blockDim.x) {
    // Small step: block 0 does everything in shared memory (no hand-over between blocks, no
    // global atomics), the other blocks leave at once.  Two passes of dependent loads, four entries
    // per thread and round.  On a 320-thread block: 3.7 us for 352 entries, 7.6 us for 2816 (the
    // multi-block form with its hand-over takes 11.7 us there), 21 us for 11264 (multi-block: about 13).
    if (blockIdx.x != 0) return;
    __shared__ int s_cursor[kMaxLocalExperts];
    for (int e = tid; e < E; e += blockDim.x) { s_hist[e] = 0; s_cursor[e] = 0; }
    __syncthreads();
    for (int i0 = tid; i0 < (int)entries; i0 += blockDim.x * 4) {
      long long e[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        e[u] = i < (int)entries ? a.topk_idx[i] - a.expert_begin : -1;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (e[u] >= 0 && e[u] < E) atomicAdd(&s_hist[(int)e[u]], 1);
    }
    __syncthreads();
    if (tid < 32) route_offsets(a, s_hist, s_cursor, E);     // offsets land in s_cursor ...
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) { s_hist[e] = s_cursor[e]; s_cursor[e] = 0; }   // ... and move over
    __syncthreads();
    for (int i0 = tid; i0 < (int)entries; i0 += blockDim.x * 4) {
      long long e[4];
      float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        const bool in = i < (int)entries;
        e[u] = in ? a.topk_idx[i] - a.expert_begin : -1;
        w[u] = in && a.topk_w ? a.topk_w[i] : 1.0f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i >= (int)entries) break;
        int pos = -1;
        if (e[u] >= 0 && e[u] < E) {
          pos = s_hist[(int)e[u]] + atomicAdd(&s_cursor[(int)e[u]], 1);
          if (pos < a.max_pairs) {
            a.pair_token[pos] = i / a.topk;
            a.pair_prob[pos] = w[u];
          } else {
            pos = -1;
          }
        }
        a.pair_pos[i] = pos;
      }
    }
    return;
  }
  const long long per_block = (entries + gridDim.x - 1) / gridDim.x;
  const long long lo = per_block * blockIdx.x;
  const long long hi = lo + per_block < entries ? lo + per_block : entries;

  // ---- phase 1: histogram of the entries owned by this block ----
  for (int e = tid; e < E; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  for (long long i0 = lo + tid; i0 < hi; i0 += blockDim.x * 4) {
    long long e[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * blockDim.x;
      e[u] = i < hi ? a.topk_idx[i] - a.expert_begin : -1;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (e[u] >= 0 && e[u] < E) atomicAdd(&s_hist[(int)e[u]], 1);
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x)
    if (s_hist[e]) atomicAdd(&a.expert_count[e], s_hist[e]);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_flag = (atomicAdd(&a.sync[0], 1) == (int)gridDim.x - 1);
    __threadfence();
  }
  __syncthreads();
  if (s_flag) {
    // Last block: exclusive prefix over experts, row-tile table, then release the others.
    for (int e = tid; e < E; e += blockDim.x) s_hist[e] = *reinterpret_cast<volatile int*>(&a.expert_count[e]);
    __syncthreads();
    if (tid < 32) {
      route_offsets(a, s_hist, nullptr, E);
      __threadfence();                   // every lane's table entries before the hand-over below
      __syncwarp();
      if (tid == 0) {
        a.sync[0] = 0;
        __threadfence();
        atomicAdd(&a.sync[2], 1);
      }
    }
  }
  if (tid == 0) {
    if (!spin_until_ge(reinterpret_cast<volatile int*>(&a.sync[2]), ready_base + 1, a.timeout_ns)) {
      if (a.status && atomicCAS(a.status, 0u, (uint32_t)MCB_ERR_TIMEOUT) == 0u) { a.status[1] = 101; a.status[2] = blockIdx.x; }
    }
    __threadfence();
  }
  __syncthreads();

  // ---- phase 2: place every local (token, k) entry into its expert's segment ----
  for (int e = tid; e < E; e += blockDim.x) s_hist[e] = *reinterpret_cast<volatile int*>(&a.expert_offset[e]);
  __syncthreads();
  for (long long i0 = lo + tid; i0 < hi; i0 += blockDim.x * 4) {
    long long e[4];
    float w[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * blockDim.x;
      e[u] = i < hi ? a.topk_idx[i] - a.expert_begin : -1;
      w[u] = i < hi && a.topk_w ? a.topk_w[i] : 1.0f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * blockDim.x;
      if (i >= hi) break;
      int pos = -1;
      if (e[u] >= 0 && e[u] < E) {
        pos = s_hist[(int)e[u]] + atomicAdd(&a.expert_cursor[(int)e[u]], 1);
        if (pos < a.max_pairs) {
          a.pair_token[pos] = (int)(i / a.topk);
          a.pair_prob[pos] = w[u];
        } else {
          pos = -1;
        }
      }
      a.pair_pos[i] = pos;
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_flag = (atomicAdd(&a.sync[1], 1) == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (s_flag) {
    // Last block out: scratch back to zero for the next launch.
    for (int e = tid; e < E; e += blockDim.x) { a.expert_count[e] = 0; a.expert_cursor[e] = 0; }
    if (tid == 0) a.sync[1] = 0;
  }
}

}  // namespace mcb
