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
//   * optional 1 x 128 block-scaled e4m3 dispatch, quantised on the way out.
// Every wait is bounded and reports through the status words.
#include <cuda_runtime.h>

#include "mcb_barrier.cuh"
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
