// The count exchange that opens a persistent decode step (dense and all-to-all alike).
#pragma once
#include "mcb_barrier.cuh"

namespace mcb {

// Block 0 publishes this rank's row count to every rank; every block of every rank waits for all
// counts.  Because a rank only publishes after its previous kernel has finished (the caller has
// executed griddepcontrol.wait), passing this point also proves that every rank has left the
// previous step.  `step_seq` = steps completed so far (the same on every rank and in every block);
// counts are double buffered by its parity in heap[counts_off] (int32 [2][MCB_MAX_RANKS]).
// Fills s_prefix[0..W] (exclusive prefix of the clamped counts) and *s_max; returns this rank's
// clamped count.  Call from all threads of every block.
__device__ __forceinline__ int step_count_exchange(const McbCtx& c, int site, uint64_t counts_off, uint32_t step_seq,
                                                   int n, int cap, int* s_cnt, int* s_prefix, int* s_max) {
  const int tid = threadIdx.x, bid = blockIdx.x, W = c.world;
  if (n < 0) n = 0;
  if (n > cap) {
    if (tid == 0 && bid == 0) report_error(c, MCB_ERR_CAPACITY, (uint32_t)site, 0, (uint32_t)n, (uint32_t)cap);
    n = cap;
  }
  if (W > 1) {
    const uint32_t par_m = step_seq & 1u;
    if (bid == 0) {
      const uint64_t slot_off = counts_off + (uint64_t)(par_m * MCB_MAX_RANKS + c.rank) * sizeof(int32_t);
      if (c.transport == MCB_TRANSPORT_MULTIMEM) {
        if (tid == 0) mm_st_b32(c.heap_mc + slot_off, (uint32_t)n);
      } else {
        for (int p = tid; p < W; p += blockDim.x) st_relaxed_sys(c.heap_peer[p] + slot_off, (uint32_t)n);
      }
      __syncthreads();
      signal_all<true>(c, site, 0);   // the signalling thread is the one that stored
    }
    if (tid == 0) wait_flag(c, site, 0, (step_seq + 1u) * (uint32_t)W);
    __syncthreads();
    const uint8_t* counts = c.heap_local + counts_off + (uint64_t)par_m * MCB_MAX_RANKS * sizeof(int32_t);
    for (int p = tid; p < W; p += blockDim.x) s_cnt[p] = (int)ld_relaxed_sys(counts + p * 4);
  } else if (tid == 0) {
    s_cnt[0] = n;
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0, mx = 0;
    for (int p = 0; p < W; ++p) {
      int v = s_cnt[p];
      if (v < 0) v = 0;
      if (v > cap) v = cap;
      s_prefix[p] = run;
      run += v;
      mx = v > mx ? v : mx;
    }
    s_prefix[W] = run;
    *s_max = mx;
  }
  __syncthreads();
  return n;
}

// Credits of the packet modes: credit[block][source rank] = number of packet layers whose packets the
// source's block has finished reading (monotonic; written by that rank only, on every rank).  A sum over
// ranks could not tell a slow rank from fast ones that ran ahead, hence one word per source.
__device__ __forceinline__ uint64_t credit_word_off(uint64_t credit_off, int block, int rank) {
  return credit_off + ((uint64_t)block * MCB_MAX_RANKS + (uint64_t)rank) * 4;
}
// All threads: the first `world` threads publish (or wait for) one word each.
__device__ __forceinline__ void credit_publish(const McbCtx& c, uint64_t credit_off, uint32_t value) {
  const uint64_t off = credit_word_off(credit_off, blockIdx.x, c.rank);
  if (c.transport == MCB_TRANSPORT_MULTIMEM) {
    if (threadIdx.x == 0) mm_st_b32(c.heap_mc + off, value);
  } else {
    for (int p = threadIdx.x; p < c.world; p += blockDim.x) st_relaxed_sys(c.heap_peer[p] + off, value);
  }
}
__device__ __forceinline__ void credit_wait(const McbCtx& c, uint64_t credit_off, uint32_t target, int site) {
  for (int p = threadIdx.x; p < c.world; p += blockDim.x) {
    const uint8_t* w = c.heap_local + credit_word_off(credit_off, blockIdx.x, p);
    uint32_t v = ld_relaxed_sys(w);
    if ((int32_t)(v - target) >= 0) continue;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
      for (int i = 0; i < 64 && (int32_t)(v - target) < 0; ++i) v = ld_relaxed_sys(w);
      if ((int32_t)(v - target) >= 0) break;
      const bool poisoned = *reinterpret_cast<volatile uint32_t*>(c.status) != 0u;
      if (poisoned || globaltimer_ns() - t0 > c.timeout_ns) {
        report_error(c, MCB_ERR_TIMEOUT, (uint32_t)site, blockIdx.x, v, target);
        break;
      }
    }
  }
  __syncthreads();
}

}  // namespace mcb
