// All-to-all-V dispatch / combine for sm_100a with direct peer stores and loads.
//
// Behavioural contract of the DeepEP ElasticBuffer path the reference wraps
// (bench_deepep.py:68-115): a token travels once to every *distinct* destination rank
// (not once per expert), the count exchange happens inside dispatch on the device, nothing
// synchronises with the host, and the combine returns, for each source token, the sum of
// one row per destination rank (m * x for the identity expert).
//
// Design:
//   * receive buffers are laid out [source rank][capacity][...]: a sender owns its region on
//     every destination, so it can pick slots with a local atomic counter and push rows with
//     plain peer stores before any count is known to the receiver;
//   * the last block to finish publishes the per-destination row counts and arrives at a
//     one-slot cross-GPU barrier; when the kernel has finished, every row sent to this rank
//     is in place and recv_count[] says how many rows each source sent;
//   * the sender remembers, per token and destination, the slot it used (slot_map); combine
//     is a pull: after a leading barrier each warp loads its token's rows straight from the
//     destinations' expert-output buffers, accumulates in fp32 and writes bf16;
//   * optional 1x128 block-scaled e4m3 dispatch: amax over each 128-element block, scale =
//     amax / 448, saturating convert, fp32 scales shipped next to the rows.
#include <cstdio>
#include <cuda_runtime.h>

#include "mcb_barrier.cuh"
#include "mcb_fp8.cuh"
#include "mcb_launch.h"
#include "mcb_noalloc.h"

namespace mcb {

constexpr int kMaxWarps = 16;

struct DestList {
  int dst[MCB_MAX_RANKS];
  int slot[MCB_MAX_RANKS];
};

__device__ __forceinline__ uint32_t warp_or(uint32_t v) { return __reduce_or_sync(0xffffffffu, v); }

template <bool EMU>
__global__ void __launch_bounds__(512) a2a_dispatch_kernel(const __grid_constant__ McbCtx ctx_p,
                                                           const __grid_constant__ McbA2ADispatchArgs args_p,
                                                           const McbCtx* ectx, const McbA2ADispatchArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbA2ADispatchArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  __shared__ DestList s_list[kMaxWarps];
  __shared__ int s_last;
  __shared__ int s_m;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int W = c.world;
  const int epr = a.num_experts / W;
  int n = *a.n_local;
  if (n < 0) n = 0;
  if (n > a.cap) {
    if (tid == 0) report_error(c, MCB_ERR_CAPACITY, MCB_SITE_A2A_DISPATCH, blockIdx.x, (uint32_t)n, (uint32_t)a.cap);
    n = a.cap;
  }
  const int row_packs = a.hidden / 8;  // 16-byte packs of bf16 per row
  const uint8_t* x = reinterpret_cast<const uint8_t*>(a.x);
  // With no more tokens than blocks, one block serves one token and its warps share the row
  // (short critical path for wide rows); otherwise one warp serves one token.  Only as many
  // blocks as that needs take part (at least one, which also publishes the counts of a rank
  // without tokens); the others leave at once.
  const bool bmode = n <= (int)gridDim.x;
  int nwork = bmode ? n : (n + nwarps - 1) / nwarps;
  nwork = nwork < 1 ? 1 : (nwork > (int)gridDim.x ? (int)gridDim.x : nwork);
  if ((int)blockIdx.x >= nwork) return;
  DestList& L = s_list[bmode ? 0 : warp];
  const int p_begin = bmode ? warp * 128 : 0;
  const int p_step = bmode ? nwarps * 128 : 128;

  for (int t = bmode ? (int)blockIdx.x : (int)blockIdx.x * nwarps + warp; t < n;
       t += bmode ? (int)gridDim.x : nwork * nwarps) {
    int m = 0;
    if (!bmode || warp == 0) {
    // Destination ranks of this token as a bitmask (3 words cover MCB_MAX_RANKS = 72).
    uint32_t m0 = 0, m1 = 0, m2 = 0;
    for (int k = lane; k < a.topk; k += 32) {
      const long long e = a.topk_idx[(long long)t * a.topk + k];
      if (e < 0 || e >= a.num_experts) {
        report_error(c, MCB_ERR_ROUTING, MCB_SITE_A2A_DISPATCH, blockIdx.x, (uint32_t)t, (uint32_t)e);
        continue;
      }
      const int d = (int)(e / epr);
      if (d < 32) m0 |= 1u << d; else if (d < 64) m1 |= 1u << (d - 32); else m2 |= 1u << (d - 64);
    }
    m0 = warp_or(m0); m1 = warp_or(m1); m2 = warp_or(m2);
    // One slot per destination from the local counters; remember it for the combine.
    for (int d0 = 0; d0 < W; d0 += 32) {
      const uint32_t word = d0 == 0 ? m0 : (d0 == 32 ? m1 : m2);
      const int d = d0 + lane;
      int slot = -1;
      if (d < W && ((word >> lane) & 1u)) slot = atomicAdd(&a.send_count[d], 1);
      if (d < W) a.slot_map[(long long)t * W + d] = slot;
      const uint32_t have = __ballot_sync(0xffffffffu, slot >= 0);
      if (slot >= 0) {
        const int pos = m + __popc(have & ((1u << lane) - 1u));
        L.dst[pos] = d;
        L.slot[pos] = slot;
      }
      m += __popc(have);
    }
    if (bmode && lane == 0) s_m = m;
    }
    if (bmode) { __syncthreads(); m = s_m; } else { __syncwarp(); }
    const uint8_t* xrow = x + (long long)t * a.hidden * 2;
    if (!a.fp8) {
      const uint64_t row_bytes = (uint64_t)a.hidden * 2;
      for (int p0 = p_begin; p0 < row_packs; p0 += p_step) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int p = p0 + u * 32 + lane;
          if (p < row_packs) v[u] = ld_v4(xrow + p * 16);
        }
        for (int j = 0; j < m; ++j) {
          uint8_t* dst = c.heap_peer[L.dst[j]] + a.recv_x_off +
                         ((uint64_t)c.rank * a.cap + L.slot[j]) * row_bytes;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int p = p0 + u * 32 + lane;
            if (p < row_packs) st_v4(dst + p * 16, v[u]);
          }
        }
      }
    } else {
      const int nblk = a.hidden / 128;
      for (int p0 = p_begin; p0 < row_packs; p0 += p_step) {
        uint4 v[4];
        uint2 q[4];
        float scale[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int p = p0 + u * 32 + lane;
          v[u] = p < row_packs ? ld_v4(xrow + p * 16) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          // amax over the 16 lanes that hold one 128-element block
          float amax = pack_absmax(v[u]);
#pragma unroll
          for (int sh = 8; sh >= 1; sh >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
          scale[u] = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
          q[u] = quant_pack_e4m3(v[u], scale[u]);
        }
        for (int j = 0; j < m; ++j) {
          const uint64_t row = (uint64_t)c.rank * a.cap + L.slot[j];
          uint8_t* peer = c.heap_peer[L.dst[j]];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int p = p0 + u * 32 + lane;
            if (p < row_packs) {
              st_v2(peer + a.recv_x_off + row * a.hidden + (uint64_t)p * 8, q[u]);
              if ((lane & 15) == 0)
                st_b32(peer + a.recv_scale_off + (row * nblk + (p >> 4)) * 4, __float_as_uint(scale[u]));
            }
          }
        }
      }
    }
    // Routing rows (ids, weights) and the source token index travel with the token.
    for (int k = lane; k < a.topk && (!bmode || warp == 0); k += 32) {
      const long long e = a.topk_idx[(long long)t * a.topk + k];
      const float w = a.topk_w ? a.topk_w[(long long)t * a.topk + k] : 1.0f;
      for (int j = 0; j < m; ++j) {
        const uint64_t row = (uint64_t)c.rank * a.cap + L.slot[j];
        uint8_t* peer = c.heap_peer[L.dst[j]];
        *reinterpret_cast<long long*>(peer + a.recv_idx_off + (row * a.topk + k) * 8) = e;
        *reinterpret_cast<float*>(peer + a.recv_w_off + (row * a.topk + k) * 4) = w;
      }
    }
    if (lane == 0 && (!bmode || warp == 0)) {
      for (int j = 0; j < m; ++j) {
        const uint64_t row = (uint64_t)c.rank * a.cap + L.slot[j];
        *reinterpret_cast<int*>(c.heap_peer[L.dst[j]] + a.recv_src_off + row * 4) = t;
      }
    }
    if (bmode) __syncthreads(); else __syncwarp();
  }

  // Grid-wide completion: the last block publishes counts and meets the other ranks.
  __syncthreads();
  if (tid == 0) {
    if (nwork > 1) {
      fence_sys();                      // this block's peer stores are performed before it counts itself done
      const int prev = atomicAdd(&a.send_count[MCB_MAX_RANKS], 1);
      __threadfence();                  // the other blocks are on this GPU: device scope is enough here
      s_last = (prev == nwork - 1);
    } else {
      s_last = 1;                       // single block: the release on the flag below covers its stores
    }
  }
  __syncthreads();
  if (!s_last) return;
  const uint32_t ep = *epoch_ptr(c, MCB_SITE_A2A_DISPATCH, 0);
  for (int d = tid; d < W; d += blockDim.x) {
    const int cnt = atomicExch(&a.send_count[d], 0);
    st_relaxed_sys(c.heap_peer[d] + a.recv_count_off + (uint64_t)c.rank * 4, (uint32_t)cnt);
  }
  if (tid == 0) a.send_count[MCB_MAX_RANKS] = 0;
  block_barrier_all(c, MCB_SITE_A2A_DISPATCH, 0, ep);
}

__device__ __forceinline__ void a2a_combine_device(const McbCtx& c, const McbA2ACombineArgs& a, uint32_t launch) {
  __shared__ DestList s_list[kMaxWarps];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int W = c.world;
  int n = *a.n_local;
  if (n < 0) n = 0;
  if (n > a.cap) n = a.cap;
  const bool bmode = n <= (int)gridDim.x;      // one block per token, its warps share the row
  int nwork = bmode ? n : (n + nwarps - 1) / nwarps;
  nwork = nwork < 1 ? 1 : (nwork > (int)gridDim.x ? (int)gridDim.x : nwork);
  if ((int)blockIdx.x >= nwork) return;
  if (W > 1) {
    // Leading barrier: every destination's expert outputs were written by kernels that finished
    // before it arrived here, so the arrival needs no release fence.  Block 0 alone meets the
    // other ranks (one flag slot) and then releases this rank's other working blocks through a
    // local word; blocks without tokens have left already.
    uint32_t* go = epoch_ptr(c, MCB_SITE_A2A_GO, 0);
    if (blockIdx.x == 0) {
      signal_all<false>(c, MCB_SITE_A2A_COMBINE, 0);
      if (tid == 0) {
        wait_flag(c, MCB_SITE_A2A_COMBINE, 0, launch * (uint32_t)W);
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(go) = launch;
      }
    } else if (tid == 0) {
      wait_local(c, go, launch, MCB_SITE_A2A_COMBINE);
      __threadfence();
    }
    __syncthreads();
  }

  const int row_packs = a.hidden / 8;
  const uint64_t row_bytes = (uint64_t)a.hidden * 2;
  uint8_t* out = reinterpret_cast<uint8_t*>(a.out);
  DestList& L = s_list[warp];            // in block mode every warp lists the destinations itself
  const int p_begin = bmode ? warp * 128 : 0;
  const int p_step = bmode ? nwarps * 128 : 128;
  for (int t = bmode ? (int)blockIdx.x : (int)blockIdx.x * nwarps + warp; t < n;
       t += bmode ? (int)gridDim.x : nwork * nwarps) {
    int m = 0;
    for (int d0 = 0; d0 < W; d0 += 32) {
      const int d = d0 + lane;
      const int slot = d < W ? a.slot_map[(long long)t * W + d] : -1;
      const uint32_t have = __ballot_sync(0xffffffffu, slot >= 0);
      if (slot >= 0) {
        const int pos = m + __popc(have & ((1u << lane) - 1u));
        L.dst[pos] = d;
        L.slot[pos] = slot;
      }
      m += __popc(have);
    }
    __syncwarp();
    // 4 packs per lane x up to 4 destinations = 16 independent peer loads in flight
    for (int p0 = p_begin; p0 < row_packs; p0 += p_step) {
      float acc[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
      for (int j = 0; j < m; j += 4) {
        uint4 v[4][4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          if (j + jj < m) {
            const uint8_t* row = c.heap_peer[L.dst[j + jj]] + a.y_off +
                                 ((uint64_t)c.rank * a.cap + L.slot[j + jj]) * row_bytes;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int p = p0 + u * 32 + lane;
              v[jj][u] = p < row_packs ? ld_v4_stream(row + (uint64_t)p * 16) : make_uint4(0, 0, 0, 0);
            }
          }
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          if (j + jj < m) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              acc[u][0] += bf16_lo(v[jj][u].x); acc[u][1] += bf16_hi(v[jj][u].x);
              acc[u][2] += bf16_lo(v[jj][u].y); acc[u][3] += bf16_hi(v[jj][u].y);
              acc[u][4] += bf16_lo(v[jj][u].z); acc[u][5] += bf16_hi(v[jj][u].z);
              acc[u][6] += bf16_lo(v[jj][u].w); acc[u][7] += bf16_hi(v[jj][u].w);
            }
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
    __syncwarp();
  }
}

template <bool EMU>
__global__ void __launch_bounds__(512) a2a_combine_kernel(const __grid_constant__ McbCtx ctx_p,
                                                          const __grid_constant__ McbA2ACombineArgs args_p,
                                                          const McbCtx* ectx, const McbA2ACombineArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbA2ACombineArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  pdl_wait();
  pdl_launch_dependents();
  // Block 0 meets the other ranks at launch * world and hands `launch` to the other blocks: the
  // number must be the same in every block (per-block counters, levelled by the host when the grid
  // of the site changes).
  const uint32_t launch = next_launch_count(c, MCB_SITE_A2A_COMBINE);
  a2a_combine_device(c, a, launch);
}

}  // namespace mcb

using namespace mcb;

extern "C" {

static int check_a2a_launch(int grid, int threads) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS || threads < 32 || threads > 512 || (threads & 31)) return 1;
  return 0;
}

int mcb_launch_a2a_dispatch(const McbCtx* ctx, const McbA2ADispatchArgs* args, int grid, int threads,
                            int pdl, cudaStream_t stream) {
  if (check_a2a_launch(grid, threads)) return cudaErrorInvalidValue;
  if (args->hidden % 8 || (args->fp8 && args->hidden % 128) || args->num_experts % ctx->world)
    return cudaErrorInvalidValue;
  return launch_kernel(a2a_dispatch_kernel<false>, dim3(grid), dim3(threads), 0, stream, pdl, false, *ctx,
                       *args, (const McbCtx*)nullptr, (const McbA2ADispatchArgs*)nullptr);
}

int mcb_launch_a2a_combine(const McbCtx* ctx, const McbA2ACombineArgs* args, int grid, int threads, int pdl,
                           cudaStream_t stream) {
  if (check_a2a_launch(grid, threads)) return cudaErrorInvalidValue;
  if (args->hidden % 8) return cudaErrorInvalidValue;
  return launch_kernel(a2a_combine_kernel<false>, dim3(grid), dim3(threads), 0, stream, pdl, false, *ctx,
                       *args, (const McbCtx*)nullptr, (const McbA2ACombineArgs*)nullptr);
}

// One decode step of the all-to-all dispatcher: num_layers x (dispatch, combine), issued
// natively (role of DeepEPBencher.decode_step, bench_deepep.py:96-101).
int mcb_a2a_decode_step(const McbCtx* ctx, const McbA2ADispatchArgs* d, const McbA2ACombineArgs* cmb,
                        int num_layers, int grid, int threads, int pdl, cudaStream_t stream) {
  int err = 0;
  for (int l = 0; l < num_layers && err == 0; ++l) {
    err = mcb_launch_a2a_dispatch(ctx, d, grid, threads, pdl, stream);
    if (err == 0) err = mcb_launch_a2a_combine(ctx, cmb, grid, threads, pdl, stream);
  }
  return err;
}

int mcb_emu_a2a_dispatch(const McbCtx* d_ctx, const McbA2ADispatchArgs* d_args, int world, int grid,
                         int threads, cudaStream_t stream) {
  if (check_a2a_launch(grid, threads)) return cudaErrorInvalidValue;
  McbCtx dummy{};
  McbA2ADispatchArgs dargs{};
  return launch_kernel(a2a_dispatch_kernel<true>, dim3(grid, world), dim3(threads), 0, stream, 0, true, dummy,
                       dargs, d_ctx, d_args);
}

int mcb_emu_a2a_combine(const McbCtx* d_ctx, const McbA2ACombineArgs* d_args, int world, int grid,
                        int threads, cudaStream_t stream) {
  if (check_a2a_launch(grid, threads)) return cudaErrorInvalidValue;
  McbCtx dummy{};
  McbA2ACombineArgs dargs{};
  return launch_kernel(a2a_combine_kernel<true>, dim3(grid, world), dim3(threads), 0, stream, 0, true, dummy,
                       dargs, d_ctx, d_args);
}

// ------------------------------------------------------------------------------------------
// Dispatch for callers that cannot allocate (see mcb_noalloc.h).
//
// The per-destination slot counters and the "blocks done" word, which the ordinary entry
// point expects the caller to provide in `send_count`, live here in a fixed array that is
// part of the loaded library image: every GPU that loads the library holds these
// MCB_NOALLOC_SCRATCH_BYTES bytes until the process exits.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) int32_t g_noalloc_send_count[MCB_NOALLOC_MAX_RANKS + 1];

#define MCB_NOALLOC_MAX_DEVICES 64
static int32_t* g_noalloc_scratch_addr[MCB_NOALLOC_MAX_DEVICES];   // device address, per device
static char g_noalloc_error[256] = "";

const char* mcb_noalloc_last_error() { return g_noalloc_error; }
int mcb_noalloc_max_ranks() { return MCB_NOALLOC_MAX_RANKS; }
int mcb_noalloc_scratch_bytes() { return MCB_NOALLOC_SCRATCH_BYTES; }

int mcb_a2a_dispatch_noalloc(const McbCtx* ctx, const McbA2ADispatchArgs* args, int grid, int threads,
                             cudaStream_t stream) {
  g_noalloc_error[0] = 0;
  if (ctx == nullptr || args == nullptr) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "mcb_a2a_dispatch_noalloc: null context or arguments");
    return cudaErrorInvalidValue;
  }
  if (ctx->world < 1 || ctx->world > MCB_NOALLOC_MAX_RANKS) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error),
             "mcb_a2a_dispatch_noalloc: world size %d is outside [1, %d], the number of destination "
             "counters the built-in scratch array holds", ctx->world, MCB_NOALLOC_MAX_RANKS);
    return cudaErrorInvalidValue;
  }
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return (int)err;
  if (dev < 0 || dev >= MCB_NOALLOC_MAX_DEVICES) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), "mcb_a2a_dispatch_noalloc: device ordinal %d is beyond %d",
             dev, MCB_NOALLOC_MAX_DEVICES);
    return cudaErrorInvalidDevice;
  }
  if (g_noalloc_scratch_addr[dev] == nullptr) {
    // In host code the array's name is only a stand-in; the kernel needs the address the
    // symbol has on the current device.  Looked up once per device, on this first call.
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, g_noalloc_send_count);
    if (err != cudaSuccess) {
      snprintf(g_noalloc_error, sizeof(g_noalloc_error), "mcb_a2a_dispatch_noalloc: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(err));
      return (int)err;
    }
    g_noalloc_scratch_addr[dev] = static_cast<int32_t*>(p);
  }
  McbA2ADispatchArgs a = *args;
  a.send_count = g_noalloc_scratch_addr[dev];
  // The counters must start at zero; an earlier call that was cut short may have left them dirty.
  err = cudaMemsetAsync(a.send_count, 0, sizeof(int32_t) * (MCB_NOALLOC_MAX_RANKS + 1), stream);
  if (err != cudaSuccess) return (int)err;
  return mcb_launch_a2a_dispatch(ctx, &a, grid, threads, 0, stream);
}

}  // extern "C"
