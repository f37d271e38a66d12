// Reduce-scatter + residual add + RMSNorm + all-gather in one kernel, in place in a
// symmetric heap buffer (the tensor-parallel decode primitive).
//
// Same capability as the reference's fused_multimem_rs_add_norm_ag
// (nvls/torch_symm_triton/fused_collectives.py:114-280): every rank holds partial sums of
// all rows; rank r owns rows [r*T/W, (r+1)*T/W).  For each owned row: cross-rank sum
// (fp32 accumulate, bf16 result), add the local residual in bf16 and store it back,
// compute 1/rms of the new residual, scale by the norm weight and write the normalised row
// to every rank's buffer.  Unlike the reference, the row stays in registers between the
// two passes (no second residual load), the barriers are the bounded one-way epoch
// barriers, and the kernel also runs over plain peer loads/stores.
#include <cuda_runtime.h>

#include "mcb_barrier.cuh"
#include "mcb_launch.h"

namespace mcb {

__device__ __forceinline__ uint4 p2p_sum_bf16x8(const McbCtx& c, uint64_t off) {
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < c.world; ++k) {
    int p = c.rank + k;
    if (p >= c.world) p -= c.world;
    const uint4 v = ld_v4_stream(c.heap_peer[p] + off);
    acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x);
    acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
    acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z);
    acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
  }
  return make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                    pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
}

template <bool EMU>
__global__ void __launch_bounds__(1024) rs_add_norm_ag_kernel(const __grid_constant__ McbCtx ctx_p,
                                                              const __grid_constant__ McbNormArgs args_p,
                                                              const McbCtx* ectx, const McbNormArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbNormArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  __shared__ float s_part[32];
  __shared__ float s_rrms;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, bid = blockIdx.x;
  const int tpr = a.tokens / c.world;  // rows owned by each rank
  const int nact = tpr < (int)gridDim.x ? tpr : (int)gridDim.x;
  if (bid >= nact) return;
  const uint32_t ep_in = *epoch_ptr(c, MCB_SITE_NORM_IN, bid);
  const uint32_t ep_out = *epoch_ptr(c, MCB_SITE_NORM_OUT, bid);
  // Every rank's partial sums are in place once its block has arrived.
  block_barrier_all(c, MCB_SITE_NORM_IN, bid, ep_in);

  const int packs = a.hidden / 8;
  const bool live = tid < packs;
  const uint64_t row_bytes = (uint64_t)a.hidden * 2;
  uint8_t* residual = reinterpret_cast<uint8_t*>(a.residual);
  const uint8_t* weight = reinterpret_cast<const uint8_t*>(a.weight);
  uint4 wv = make_uint4(0, 0, 0, 0);
  if (live) wv = ld_v4(weight + tid * 16);

  for (int t = bid; t < tpr; t += nact) {
    const uint64_t off = a.buf_off + ((uint64_t)c.rank * tpr + t) * row_bytes + (uint64_t)tid * 16;
    uint4 s = make_uint4(0, 0, 0, 0);
    float sq = 0.f;
    if (live) {
      const uint4 v = c.transport == MCB_TRANSPORT_MULTIMEM ? mm_ld_reduce_bf16x8(c.heap_mc + off)
                                                            : p2p_sum_bf16x8(c, off);
      const uint4 r = ld_v4(residual + t * row_bytes + tid * 16);
      s = add_bf16x8(v, r);
      st_v4(residual + t * row_bytes + tid * 16, s);
      const uint32_t w4[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) sq += bf16_lo(w4[i]) * bf16_lo(w4[i]) + bf16_hi(w4[i]) * bf16_hi(w4[i]);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((tid & 31) == 0) s_part[tid >> 5] = sq;
    __syncthreads();
    if (tid < 32) {
      float v = tid < (int)(blockDim.x >> 5) ? s_part[tid] : 0.f;
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (tid == 0) s_rrms = rsqrt_approx(v / (float)a.hidden + a.eps);
    }
    __syncthreads();
    const float rrms = s_rrms;
    if (live) {
      const uint32_t s4[4] = {s.x, s.y, s.z, s.w};
      const uint32_t g4[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        o4[i] = pack_bf16x2(bf16_lo(s4[i]) * rrms * bf16_lo(g4[i]), bf16_hi(s4[i]) * rrms * bf16_hi(g4[i]));
      const uint4 y = make_uint4(o4[0], o4[1], o4[2], o4[3]);
      if (c.transport == MCB_TRANSPORT_MULTIMEM) {
        mm_st_v4(c.heap_mc + off, y);
      } else {
        for (int k = 0; k < c.world; ++k) {
          int p = c.rank + 1 + k;
          if (p >= c.world) p -= c.world;
          st_v4(c.heap_peer[p] + off, y);
        }
      }
    }
    __syncthreads();  // s_part / s_rrms are reused by the next row
  }
  // When this kernel has finished, the normalised rows of every rank are in the local buffer.
  block_barrier_all(c, MCB_SITE_NORM_OUT, bid, ep_out);
}

}  // namespace mcb

using namespace mcb;

extern "C" {

static int norm_threads(int hidden) {
  int t = (hidden / 8 + 31) / 32 * 32;
  return t < 32 ? 32 : t;
}

int mcb_launch_rs_add_norm_ag(const McbCtx* ctx, const McbNormArgs* args, int grid, int pdl,
                              cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS) return cudaErrorInvalidValue;
  if (args->hidden % 8 || args->hidden > 8192 || args->tokens % ctx->world) return cudaErrorInvalidValue;
  return launch_kernel(rs_add_norm_ag_kernel<false>, dim3(grid), dim3(norm_threads(args->hidden)), 0, stream,
                       pdl, false, *ctx, *args, (const McbCtx*)nullptr, (const McbNormArgs*)nullptr);
}

int mcb_emu_rs_add_norm_ag(const McbCtx* d_ctx, const McbNormArgs* d_args, int world, int hidden, int grid,
                           cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS || hidden % 8 || hidden > 8192) return cudaErrorInvalidValue;
  McbCtx dummy{};
  McbNormArgs dargs{};
  return launch_kernel(rs_add_norm_ag_kernel<true>, dim3(grid, world), dim3(norm_threads(hidden)), 0, stream,
                       0, true, dummy, dargs, d_ctx, d_args);
}

}  // extern "C"
