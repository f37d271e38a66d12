// Dense expert-parallel transport for sm_100a: token-count metadata, variable all-gather
// (dispatch) and variable reduce-scatter (combine) over NVSwitch.
//
// Same capabilities as the reference's Triton kernels
//   nvls/metadata.py:46-139                          (count exchange -> [sum, prefix, max])
//   nvls/torch_symm_triton/variable_collectives.py:40-150, 366-544   (AllGather-V, 1 and 3 tensors)
//   nvls/torch_symm_triton/variable_collectives.py:153-258           (ReduceScatter-V)
// with a different design:
//   * every size that changes between steps (local token count, prefix offset, max) is read
//     from device memory, so one captured CUDA graph serves any batch up to the capacity;
//   * tensors are copied as flat byte ranges (rows are packed), 4 independent 16-byte
//     accesses per thread in flight, with a block count that grows with the largest rank's
//     token count and is the same on every rank;
//   * the barrier is the one-way epoch barrier of mcb_barrier.cuh (no CAS round trip), and
//     every kernel issues griddepcontrol so consecutive layers can overlap launch latency;
//   * each kernel runs with either transport: NVSwitch multicast (multimem.*) or plain peer
//     loads/stores (also the path used for world == 1 and for single-GPU emulation).
//
// Emulation (EMU = true): one cooperative launch with gridDim.y = world runs all ranks of a
// collective on one GPU, each y-slice using its own context; used to test the multi-rank
// protocol where only one GPU is available.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "mcb_barrier.cuh"
#include "mcb_dense.cuh"
#include "mcb_launch.h"

namespace mcb {

// ------------------------------------------------------------------------------------------
// Metadata: publish this rank's count to every rank, barrier, reduce to [sum, prefix, max].
// ------------------------------------------------------------------------------------------
template <bool EMU>
__global__ void __launch_bounds__(128) metadata_kernel(const __grid_constant__ McbCtx ctx_p,
                                                       const __grid_constant__ McbMetaArgs args_p,
                                                       const McbCtx* ectx, const McbMetaArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbMetaArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  __shared__ int s_counts[MCB_MAX_RANKS];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  const uint32_t ep = *epoch_ptr(c, MCB_SITE_META, 0);
  const uint32_t par = ep & 1u;
  int n = *a.n_local;
  if (n < 0) n = 0;
  if (n > a.cap) {
    if (tid == 0) report_error(c, MCB_ERR_CAPACITY, MCB_SITE_META, 0, (uint32_t)n, (uint32_t)a.cap);
    n = a.cap;
  }
  const uint64_t slot_off = a.counts_off + (uint64_t)(par * MCB_MAX_RANKS + c.rank) * sizeof(int32_t);
  if (c.transport == MCB_TRANSPORT_MULTIMEM) {
    if (tid == 0) mm_st_b32(c.heap_mc + slot_off, (uint32_t)n);
  } else {
    for (int p = tid; p < c.world; p += blockDim.x) st_relaxed_sys(c.heap_peer[p] + slot_off, (uint32_t)n);
  }
  // The signalling thread is the one that stored, so its release covers the store.
  block_barrier_all(c, MCB_SITE_META, 0, ep);
  const uint8_t* counts = c.heap_local + a.counts_off + (uint64_t)par * MCB_MAX_RANKS * sizeof(int32_t);
  for (int p = tid; p < c.world; p += blockDim.x) s_counts[p] = (int)ld_relaxed_sys(counts + p * 4);
  __syncthreads();
  if (tid == 0) {
    int sum = 0, prefix = 0, mx = 0;
    for (int p = 0; p < c.world; ++p) {
      const int v = s_counts[p];
      sum += v;
      if (p < c.rank) prefix += v;
      mx = v > mx ? v : mx;
    }
    a.step_meta[0] = sum;
    a.step_meta[1] = prefix;
    a.step_meta[2] = mx;
    a.step_meta[3] = (int)(ep + 1u);
  }
}

template <bool EMU>
__global__ void __launch_bounds__(512) agv_kernel(const __grid_constant__ McbCtx ctx_p,
                                                   const __grid_constant__ McbAgvArgs args_p,
                                                   const McbCtx* ectx, const McbAgvArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbAgvArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  uint32_t launch = 0;
  agv_device<-1>(c, a, launch);
}

// ------------------------------------------------------------------------------------------
// Reduce-scatter-V
// ------------------------------------------------------------------------------------------
// Low-latency reduce-scatter-V (bf16): push every valid row of my partial sums to its owner as
// packets, then sum, for each of my own rows, the packets of all ranks in rank order (fp32).
__device__ __forceinline__ void rsv_ll(const McbCtx& c, const McbRsvArgs& a, int n, int offset, int valid,
                                       uint32_t flag, const int* s_prefix) {
  const int wpr = (int)(a.row_bytes >> 3);
  const uint64_t per_src = (uint64_t)a.ll_src_rows * wpr * 16;
  const uint64_t stage = a.ll_off + (uint64_t)(flag & 1u) * c.world * per_src;
  const int nb = (int)gridDim.x < kLLBlocks ? (int)gridDim.x : kLLBlocks;
  if ((int)blockIdx.x >= nb) return;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)nb * blockDim.x;
  const uint8_t* mine = c.heap_local + a.src_off;
  // send: 4 independent packets per thread in flight
  const long long nsend = (long long)valid * wpr;
  for (long long i0 = tid; i0 < nsend; i0 += nthreads * 4) {
    uint2 d[4];
    uint8_t* dst[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * nthreads;
      dst[u] = nullptr;
      if (i < nsend) {
        const int g = (int)(i / wpr);
        const int j = (int)(i - (long long)g * wpr);
        int owner = 0;
        while (owner + 1 < c.world && s_prefix[owner + 1] <= g) ++owner;
        d[u] = ld_v2(mine + (uint64_t)g * a.row_bytes + (uint64_t)j * 8);
        dst[u] = c.heap_peer[owner] + stage + (uint64_t)c.rank * per_src +
                 ((uint64_t)(g - s_prefix[owner]) * wpr + j) * 16;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (dst[u]) st_v4(dst[u], ll_pack(d[u], flag));
  }
  // receive: read the packets of four sources at a time, wait only for those not there yet
  uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
  for (long long i = tid; i < (long long)n * wpr; i += nthreads) {
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
        if (v[u].y != flag || v[u].w != flag) d = ll_wait(c, slot0 + (uint64_t)(s0 + u) * per_src, flag, a.site);
        acc[0] += bf16_lo(d.x); acc[1] += bf16_hi(d.x);
        acc[2] += bf16_lo(d.y); acc[3] += bf16_hi(d.y);
      }
    }
    st_v2(out + (uint64_t)i * 8, make_uint2(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3])));
  }
}

__device__ __forceinline__ void rsv_device(const McbCtx& c, const McbRsvArgs& a, uint32_t& ll_launch) {
  const int bid = blockIdx.x;
  int n = 0, valid_pre = 0, offset = 0, ep_max = 0, meta_epoch = 0;
  if (a.meta_stable) {
    n = *a.n_local;
    valid_pre = a.step_meta[0]; offset = a.step_meta[1]; ep_max = a.step_meta[2]; meta_epoch = a.step_meta[3];
  }
  pdl_wait();
  ll_launch = next_launch_count(c, MCB_SITE_RSV_LL);
  if (!a.meta_stable) {
    n = *a.n_local;
    valid_pre = a.step_meta[0]; offset = a.step_meta[1]; ep_max = a.step_meta[2]; meta_epoch = a.step_meta[3];
  }
  const int nact = active_blocks((int)gridDim.x, ep_max, a.row_bytes, (int)blockDim.x);
  pdl_launch_dependents();
  const bool bad = n < 0 || n > a.cap || offset < 0 || (long long)offset + n > (long long)a.cap * c.world;
  if (a.ll_rows > 0 && c.world > 1) {
    __shared__ int s_prefix[MCB_MAX_RANKS + 1];
    const uint32_t flag = ll_launch;
    if (a.dtype == 0 && valid_pre > 0 && valid_pre <= a.ll_rows) {
      const int valid = valid_pre;
      if (bad || n > a.ll_src_rows) {
        if (threadIdx.x == 0) report_error(c, MCB_ERR_BOUNDS, (uint32_t)a.site, (uint32_t)bid, (uint32_t)n, (uint32_t)valid);
        return;
      }
      // Row ownership: prefix sums of the per-rank counts published by the metadata kernel.  The
      // counts are read by one thread each (independent loads), then summed from shared memory.
      {
        const uint32_t par = ((uint32_t)meta_epoch - 1u) & 1u;
        const uint8_t* counts = c.heap_local + a.counts_off + (uint64_t)par * MCB_MAX_RANKS * 4;
        for (int p = threadIdx.x; p < c.world; p += blockDim.x) s_prefix[p + 1] = (int)ld_relaxed_sys(counts + p * 4);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int run = 0;
        for (int p = 0; p < c.world; ++p) {
          const int cnt = s_prefix[p + 1];
          s_prefix[p] = run;
          run += cnt;
        }
        s_prefix[c.world] = run;
      }
      __syncthreads();
      rsv_ll(c, a, n, offset, valid, flag, s_prefix);
      return;
    }
    if (ep_max <= 0) return;
  }
  if (bid >= nact) return;
  const uint32_t ep = *epoch_ptr(c, a.site, bid);
  if (n < 0) n = 0;
  if (bad) {
    if (threadIdx.x == 0)
      report_error(c, n > a.cap ? MCB_ERR_CAPACITY : MCB_ERR_BOUNDS, (uint32_t)a.site, (uint32_t)bid,
                   (uint32_t)n, (uint32_t)offset);
    n = 0;
  }
  // Leading barrier: every rank's partial sums were written by kernels that finished before
  // that rank's block arrived here, so the arrival needs no release fence.
  block_barrier_all<false>(c, a.site, bid, ep);

  const long long nvec = (long long)n * a.row_bytes / 16;
  const long long start = (long long)bid * blockDim.x + threadIdx.x;
  const long long stride = (long long)nact * blockDim.x;
  reduce_flat(c, reinterpret_cast<uint8_t*>(a.out), a.src_off + (uint64_t)offset * a.row_bytes, nvec, start, stride,
              a.dtype);
}

template <bool EMU>
__global__ void __launch_bounds__(512) rsv_kernel(const __grid_constant__ McbCtx ctx_p,
                                                   const __grid_constant__ McbRsvArgs args_p,
                                                   const McbCtx* ectx, const McbRsvArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbRsvArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  uint32_t launch = 0;
  rsv_device(c, a, launch);
}

// ------------------------------------------------------------------------------------------
// Self-test of the barrier: `rounds` barriers on MCB_SITE_TEST.  With a context whose world
// counts a rank that never signals, the bounded wait runs out and the status is set.
// ------------------------------------------------------------------------------------------
template <bool EMU>
__global__ void barrier_test_kernel(const __grid_constant__ McbCtx ctx_p, const McbCtx* ectx, int rounds) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  for (int r = 0; r < rounds; ++r) {
    const uint32_t ep = *epoch_ptr(c, MCB_SITE_TEST, blockIdx.x);
    block_barrier_all(c, MCB_SITE_TEST, blockIdx.x, ep);
  }
}

}  // namespace mcb

// ------------------------------------------------------------------------------------------
// Launchers
// ------------------------------------------------------------------------------------------
using namespace mcb;

extern "C" {

int mcb_launch_metadata(const McbCtx* ctx, const McbMetaArgs* args, int pdl, cudaStream_t stream) {
  return launch_kernel(metadata_kernel<false>, dim3(1), dim3(128), 0, stream, pdl, false, *ctx, *args,
                       (const McbCtx*)nullptr, (const McbMetaArgs*)nullptr);
}

int mcb_launch_agv(const McbCtx* ctx, const McbAgvArgs* args, int grid, int threads, int pdl,
                   cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS || threads < 32 || threads > 512) return cudaErrorInvalidValue;
  return launch_kernel(agv_kernel<false>, dim3(grid), dim3(threads), 0, stream, pdl, false, *ctx, *args,
                       (const McbCtx*)nullptr, (const McbAgvArgs*)nullptr);
}

int mcb_launch_rsv(const McbCtx* ctx, const McbRsvArgs* args, int grid, int threads, int pdl,
                   cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS || threads < 32 || threads > 512) return cudaErrorInvalidValue;
  return launch_kernel(rsv_kernel<false>, dim3(grid), dim3(threads), 0, stream, pdl, false, *ctx, *args,
                       (const McbCtx*)nullptr, (const McbRsvArgs*)nullptr);
}

// One decode step of the dense dispatcher, issued natively: metadata once, then
// num_layers x (all-gather-V, reduce-scatter-V).  Mirrors NVLSBencher.decode_step
// (bench_nvls.py:114-121) without a Python loop.
int mcb_dense_decode_step(const McbCtx* ctx, const McbMetaArgs* meta, const McbAgvArgs* agv,
                          const McbRsvArgs* rsv, int num_layers, int grid, int threads, int pdl,
                          cudaStream_t stream) {
  int err = mcb_launch_metadata(ctx, meta, pdl, stream);
  // Only the first all-gather follows the kernel that writes the step metadata; every later
  // launch may read the metadata before waiting on its predecessor.
  McbAgvArgs agv_first = *agv, agv_rest = *agv;
  McbRsvArgs rsv_all = *rsv;
  agv_first.meta_stable = 0;
  agv_rest.meta_stable = pdl ? 1 : 0;
  rsv_all.meta_stable = pdl ? 1 : 0;
  for (int l = 0; l < num_layers && err == 0; ++l) {
    err = mcb_launch_agv(ctx, l == 0 ? &agv_first : &agv_rest, grid, threads, pdl, stream);
    if (err == 0) err = mcb_launch_rsv(ctx, &rsv_all, grid, threads, pdl, stream);
  }
  return err;
}

int mcb_launch_barrier_test(const McbCtx* ctx, int grid, int rounds, cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS) return cudaErrorInvalidValue;
  return launch_kernel(barrier_test_kernel<false>, dim3(grid), dim3(128), 0, stream, 0, false, *ctx,
                       (const McbCtx*)nullptr, rounds);
}

// ---- single-GPU emulation of `world` ranks (contexts and arguments live in device memory) ----
int mcb_emu_metadata(const McbCtx* d_ctx, const McbMetaArgs* d_args, int world, cudaStream_t stream) {
  McbCtx dummy{};
  McbMetaArgs dargs{};
  return launch_kernel(metadata_kernel<true>, dim3(1, world), dim3(128), 0, stream, 0, true, dummy, dargs,
                       d_ctx, d_args);
}
int mcb_emu_agv(const McbCtx* d_ctx, const McbAgvArgs* d_args, int world, int grid, int threads,
                cudaStream_t stream) {
  McbCtx dummy{};
  McbAgvArgs dargs{};
  return launch_kernel(agv_kernel<true>, dim3(grid, world), dim3(threads), 0, stream, 0, true, dummy, dargs,
                       d_ctx, d_args);
}
int mcb_emu_rsv(const McbCtx* d_ctx, const McbRsvArgs* d_args, int world, int grid, int threads,
                cudaStream_t stream) {
  McbCtx dummy{};
  McbRsvArgs dargs{};
  return launch_kernel(rsv_kernel<true>, dim3(grid, world), dim3(threads), 0, stream, 0, true, dummy, dargs,
                       d_ctx, d_args);
}
int mcb_emu_barrier_test(const McbCtx* d_ctx, int world, int grid, int rounds, cudaStream_t stream) {
  McbCtx dummy{};
  return launch_kernel(barrier_test_kernel<true>, dim3(grid, world), dim3(128), 0, stream, 0, true, dummy,
                       d_ctx, rounds);
}

}  // extern "C"
