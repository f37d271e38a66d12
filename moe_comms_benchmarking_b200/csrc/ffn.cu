// The expert path of a MoE layer for sm_100a: the grouped SwiGLU FFN with the weights as the M
// operand (mcb_ffn.cuh) as a kernel of its own, and the WHOLE layer as one cooperative kernel:
//
//   dispatch    every CTA pushes its share of the local tokens to all ranks (multimem.st + cross-GPU
//               barrier, or flagged packets for small steps)                          mcb_dense.cuh
//   routing     histogram -> offsets -> pair lists for this rank's experts               mcb_route.cuh
//   experts     gate/up blocks, then down blocks, one persistent weight stream            mcb_ffn.cuh
//   combine     per-token pre-sum of the local expert outputs into the symmetric buffer, block-matched
//               cross-GPU barrier, multimem.ld_reduce of the rows this rank owns       mcb_combine.cuh
//
// separated by grid-wide barriers (the launch is cooperative: all CTAs are resident).  The reference
// stops at the identity expert (bench_nvls.py:109-121); its dispatch and combine are the first and the
// last phase here.  EMU = true runs several ranks inside one launch (gridDim.y = world, each y-slice
// with its own argument block in device memory), which is how the cross-rank protocol of this kernel
// is tested on a single GPU.
#include <cuda.h>
#include <cuda_runtime.h>

#define MCB_WITH_LAYER_ARGS
#include "mcb_combine.cuh"
#include "mcb_dense.cuh"
#include "mcb_ffn.cuh"
#include "mcb_gemm.h"
#include "mcb_launch.h"
#include "mcb_route.cuh"

namespace mcb {

__global__ void __launch_bounds__(kFfnThreads, 1) expert_ffn_kernel(const __grid_constant__ McbFfnArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  ffn_device(a);
}

template <bool EMU>
__global__ void __launch_bounds__(kFfnThreads, 1)
moe_layer_kernel(const __grid_constant__ McbLayerArgs p_, const McbLayerArgs* eargs) {
  const McbLayerArgs& p = EMU ? eargs[blockIdx.y] : p_;
  const McbCtx& c = p.ctx;
  uint32_t ll_launch = 0;
  const bool tracing = p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
  if (tracing) p.trace[0] = globaltimer_ns();
  agv_device<MCB_SITE_FC1_FUSED>(c, p.agv, ll_launch);      // waits for the previous kernel first
  if (tracing) p.trace[1] = globaltimer_ns();
  // The arrival counter is back at zero whenever a launch has ended (its last block resets it).
  uint32_t* arrivals = epoch_ptr(c, MCB_SITE_LAYER, 1);
  grid_sync(c, arrivals, gridDim.x);
  if (tracing) p.trace[2] = globaltimer_ns();
  route_device(p.route);
  if (tracing) p.trace[3] = globaltimer_ns();
  grid_sync(c, arrivals, 2u * gridDim.x);
  if (tracing) p.trace[4] = globaltimer_ns();
  ffn_device(p.ffn);
  if (tracing) p.trace[5] = globaltimer_ns();
  grid_sync(c, arrivals, 3u * gridDim.x);                   // every y row is written before any is summed
  if (tracing) p.trace[6] = globaltimer_ns();
  combine_body(c, p.cmb, ll_launch);      // partial sums alternate between two buffers, layer by layer
  if (tracing) p.trace[7] = globaltimer_ns();
  launch_end(c, MCB_SITE_FC1_FUSED, ll_launch, arrivals);
}

}  // namespace mcb

using namespace mcb;

extern "C" {

int mcb_sizeof_ffn_args() { return (int)sizeof(McbFfnArgs); }
int mcb_sizeof_layer_args() { return (int)sizeof(McbLayerArgs); }
int mcb_ffn_smem_bytes() { return kFfnSmemBytes; }
int mcb_ffn_threads() { return kFfnThreads; }

static bool configure_ffn_kernels() {
  static int state = 0;   // 0 = not tried, 1 = ok, -1 = failed
  if (state == 0) {
    cudaError_t e1 = cudaFuncSetAttribute(expert_ffn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFfnSmemBytes);
    cudaError_t e2 = cudaFuncSetAttribute(moe_layer_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFfnSmemBytes);
    cudaError_t e3 = cudaFuncSetAttribute(moe_layer_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFfnSmemBytes);
    state = (e1 == cudaSuccess && e2 == cudaSuccess && e3 == cudaSuccess) ? 1 : -1;
  }
  return state == 1;
}

static int check_ffn_args(const McbFfnArgs* a) {
  if (!a || !a->x || !a->pair_token || !a->expert_offset || !a->max_rows || !a->act || !a->y || !a->ffn_done) return 1;
  if (!a->w1 || !a->w2 || (reinterpret_cast<uintptr_t>(a->w1) & 15) || (reinterpret_cast<uintptr_t>(a->w2) & 15)) return 1;
  if (a->num_local_experts < 1 || a->num_local_experts > kFfnMaxExperts || a->hidden < 128 || a->hidden % 128 || a->intermediate < 128 || a->intermediate % 128) return 1;
  if (a->x_row_bytes & 15) return 1;
  return 0;
}

// Gate/up + SwiGLU + down over the pair lists of a routing, as one persistent launch.
int mcb_launch_expert_ffn(const McbFfnArgs* args, int grid, int pdl, cudaStream_t stream) {
  if (grid < 1 || check_ffn_args(args)) return cudaErrorInvalidValue;
  if (!configure_ffn_kernels()) return cudaErrorUnknown;
  // A down block waits for gate/up blocks that other CTAs compute: all CTAs must be resident.
  return launch_kernel(expert_ffn_kernel, dim3(grid), dim3(kFfnThreads), kFfnSmemBytes, stream, pdl, true, *args);
}

static int check_layer_args(const McbLayerArgs* p, int grid) {
  if (!p || grid < 1 || grid > MCB_MAX_BLOCKS || check_ffn_args(&p->ffn)) return 1;
  if (p->route.num_local_experts < 1 || p->route.num_local_experts > kMaxLocalExperts) return 1;
  if (p->cmb.hidden % 8) return 1;
  return 0;
}

// One whole MoE layer (dispatch, routing, experts, combine) as one cooperative launch.
int mcb_launch_moe_layer(const McbLayerArgs* p, int grid, int pdl, cudaStream_t stream) {
  if (check_layer_args(p, grid)) return cudaErrorInvalidValue;
  if (!configure_ffn_kernels()) return cudaErrorUnknown;
  return launch_kernel(moe_layer_kernel<false>, dim3(grid), dim3(kFfnThreads), kFfnSmemBytes, stream, pdl, true, *p,
                       (const McbLayerArgs*)nullptr);
}

// One decode step with real experts, issued natively: the count exchange, then num_layers layer
// kernels; layer l uses the argument block (weight set) l % num_sets.
int mcb_launch_metadata(const McbCtx* ctx, const McbMetaArgs* args, int pdl, cudaStream_t stream);   // dense.cu

int mcb_moe_decode_step(const McbCtx* ctx, const McbMetaArgs* meta, const McbLayerArgs* layers, int num_sets,
                        int num_layers, int grid, int pdl, cudaStream_t stream) {
  if (!ctx || !meta || !layers || num_sets < 1 || num_layers < 0) return cudaErrorInvalidValue;
  int err = mcb_launch_metadata(ctx, meta, pdl, stream);
  for (int l = 0; l < num_layers && err == 0; ++l) err = mcb_launch_moe_layer(&layers[l % num_sets], grid, pdl, stream);
  return err;
}

int mcb_emu_moe_layer(const McbLayerArgs* d_args, const McbLayerArgs* h_args0, int world, int grid,
                      cudaStream_t stream) {
  if (!d_args || world < 1 || check_layer_args(h_args0, grid)) return cudaErrorInvalidValue;
  if (!configure_ffn_kernels()) return cudaErrorUnknown;
  McbLayerArgs dummy{};
  return launch_kernel(moe_layer_kernel<true>, dim3(grid, world), dim3(kFfnThreads), kFfnSmemBytes, stream, 0, true,
                       dummy, d_args);
}

}  // extern "C"
