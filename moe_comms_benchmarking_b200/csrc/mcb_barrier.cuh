// Cross-GPU barrier with bounded waits and an error status word.
//
// Role of the reference's signal-pad barrier (nvls/torch_symm_triton/barrier.py:20-115),
// redesigned for latency and for shared GPUs:
//   * arrival is a one-way fire-and-forget add (multimem.red through the switch, or one
//     red.release.sys per peer) instead of a CAS that needs the old value back;
//   * slots are never reset: slot value after its k-th use is k * world, and each block
//     keeps its own k ("epoch") in local memory, so a CUDA graph can be replayed without
//     any host-side counter;
//   * every wait has a time budget; when it runs out the kernel records
//     {code, site, block, seen, wanted, rank} in the status words and carries on to its
//     exit, so the context stays usable and the host raises the error.
// The barrier is block-matched: block b of rank r meets block b of every other rank.
#pragma once
#include "mcb_ctx.h"
#include "mcb_ptx.cuh"

namespace mcb {

__device__ __forceinline__ void report_error(const McbCtx& c, uint32_t code, uint32_t site,
                                             uint32_t block, uint32_t seen, uint32_t wanted) {
  if (atomicCAS(c.status, 0u, code) == 0u) {
    c.status[1] = site;
    c.status[2] = block;
    c.status[3] = seen;
    c.status[4] = wanted;
    c.status[5] = (uint32_t)c.rank;
  }
}

__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* heap, const McbCtx& c, int site, int slot) {
  return reinterpret_cast<uint32_t*>(heap + c.flags_off) + site * MCB_MAX_BLOCKS + slot;
}
__device__ __forceinline__ uint32_t* epoch_ptr(const McbCtx& c, int site, int slot) {
  return c.epochs + site * MCB_MAX_BLOCKS + slot;
}

// Called by every thread of the block after a __syncthreads() that follows the block's
// data writes.  Adds 1 to flag[site][slot] on every rank (self included).
// RELEASE = false is for a barrier that only announces "the kernels before this one have
// finished" (their writes were completed at the kernel boundary), so no fence is needed.
template <bool RELEASE = true>
__device__ __forceinline__ void signal_all(const McbCtx& c, int site, int slot) {
  if (c.transport == MCB_TRANSPORT_MULTIMEM) {
    if (threadIdx.x == 0) {
      if (RELEASE) mm_red_add_release(flag_ptr(c.heap_mc, c, site, slot), 1u);
      else mm_red_add_relaxed(flag_ptr(c.heap_mc, c, site, slot), 1u);
    }
  } else {
    for (int p = threadIdx.x; p < c.world; p += blockDim.x) {
      if (RELEASE) red_add_release_sys(flag_ptr(c.heap_peer[p], c, site, slot), 1u);
      else red_add_relaxed_sys(flag_ptr(c.heap_peer[p], c, site, slot), 1u);
    }
  }
}

// Called by ONE thread.  Spins until flag[site][slot] reached `target` (wrap-safe) or the
// time budget ran out.  Returns false on timeout after recording the error.
__device__ __forceinline__ bool wait_flag(const McbCtx& c, int site, int slot, uint32_t target) {
  const uint32_t* f = flag_ptr(c.heap_local, c, site, slot);
  uint32_t v = ld_acquire_sys(f);
  if ((int32_t)(v - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      v = ld_acquire_sys(f);
      if ((int32_t)(v - target) >= 0) return true;
    }
    // Once any wait on this rank has failed, later waits give up at once so that the rest of
    // a captured multi-layer graph drains quickly instead of timing out kernel by kernel.
    const bool poisoned = *reinterpret_cast<volatile uint32_t*>(c.status) != 0u;
    if (poisoned || globaltimer_ns() - t0 > c.timeout_ns) {
      report_error(c, MCB_ERR_TIMEOUT, (uint32_t)site, (uint32_t)slot, v, target);
      return false;
    }
  }
}

// Whole-block barrier with every other rank's block `slot`.  `ep` is the block's epoch
// read earlier from epoch_ptr(); the epoch is advanced here.  Ends with __syncthreads().
template <bool RELEASE = true>
__device__ __forceinline__ void block_barrier_all(const McbCtx& c, int site, int slot, uint32_t ep) {
  __syncthreads();
  if (c.world == 1) return;  // nobody to meet: stream order alone orders a single rank's kernels
  signal_all<RELEASE>(c, site, slot);
  if (threadIdx.x == 0) {
    wait_flag(c, site, slot, (ep + 1u) * (uint32_t)c.world);
    *epoch_ptr(c, site, slot) = ep + 1u;
  }
  __syncthreads();
}

// Per-block launch counter: every block of every launch advances its own counter, whether it has
// work or not, so the value is the same in all blocks and on all ranks AS LONG AS every launch on
// the site uses the same grid; when the grid of a site changes the host levels the whole counter
// row first (SymmetricHeap.level_launch_counters).  Costs nothing at the end of the kernel, which
// matters for kernels of a few microseconds.  Call from all threads; returns 1, 2, ...
__device__ __forceinline__ uint32_t next_launch_count(const McbCtx& c, int site) {
  uint32_t* ctr = epoch_ptr(c, site, blockIdx.x);
  const uint32_t v = *ctr + 1u;
  __syncthreads();
  if (threadIdx.x == 0) *ctr = v;
  return v;
}

// Launch sequence number of a site (1, 2, ...), the same in every block of a launch and on every
// rank whatever the grid sizes of this and of earlier launches: word 0 of the site's epoch row counts
// the launches that have completed and changes only when the LAST block of a launch leaves (word 1
// counts the blocks that have left).  launch_begin(): all threads, after pdl_wait().  launch_end():
// all threads of every block, on the way out of the kernel (blocks without work included).  The
// atomic at the end costs about a microsecond of kernel tail: for long kernels only.
__device__ __forceinline__ uint32_t launch_begin(const McbCtx& c, int site) {
  return *reinterpret_cast<volatile uint32_t*>(epoch_ptr(c, site, 0)) + 1u;
}
// `also_zero`: a local word (the arrival counter of a grid-wide barrier) that the last block resets too.
__device__ __forceinline__ void launch_end(const McbCtx& c, int site, uint32_t launch, uint32_t* also_zero = nullptr) {
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = epoch_ptr(c, site, 1);
    __threadfence();
    if (atomicAdd(done, 1u) == gridDim.x - 1u) {
      *reinterpret_cast<volatile uint32_t*>(done) = 0u;
      if (also_zero) *reinterpret_cast<volatile uint32_t*>(also_zero) = 0u;
      *reinterpret_cast<volatile uint32_t*>(epoch_ptr(c, site, 0)) = launch;
      __threadfence();
    }
  }
}

// Bounded spin on a LOCAL word until it reached `target` (wrap-safe).  One thread.
__device__ __forceinline__ bool wait_local(const McbCtx& c, const uint32_t* word, uint32_t target, int site) {
  const volatile uint32_t* w = word;
  if ((int32_t)(*w - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if ((int32_t)(*w - target) >= 0) return true;
    const bool poisoned = *reinterpret_cast<volatile uint32_t*>(c.status) != 0u;
    if (poisoned || globaltimer_ns() - t0 > c.timeout_ns) {
      report_error(c, MCB_ERR_TIMEOUT, (uint32_t)site, blockIdx.x, *w, target);
      return false;
    }
  }
}

// Grid-wide barrier of a cooperative launch: `arrivals` only ever grows; the caller passes
// the total it must reach (a multiple of the grid size derived from its launch counter).
__device__ __forceinline__ void grid_sync(const McbCtx& c, uint32_t* arrivals, uint32_t target) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(arrivals, 1u);
    wait_local(c, arrivals, target, MCB_SITE_LAYER);
    __threadfence();
  }
  __syncthreads();
}

}  // namespace mcb
