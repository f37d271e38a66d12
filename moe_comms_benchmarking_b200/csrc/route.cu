// Expert path glue for sm_100a: (1) routing of the gathered tokens to this rank's experts
// (histogram -> offsets -> pair lists -> row-tile table for the grouped GEMMs), and (2) the
// combine that sums each token's local expert outputs and reduce-scatters the partial sums
// across ranks in the same kernel.
//
// The reference defers the permute "to the GEMM" and never performs it (its expert is the
// identity; the only trace is the routing mask in bench_nvls.py:195).  Here the permute is an
// index list: the FC1 kernel gathers token rows through pair_token[], so no token is copied.
#include <cuda_runtime.h>

#include "mcb_barrier.cuh"
#include "mcb_combine.cuh"
#include "mcb_gemm.h"
#include "mcb_route.cuh"
#include "mcb_launch.h"

namespace mcb {

__global__ void __launch_bounds__(kRouteThreads, 1) route_kernel(const __grid_constant__ McbRouteArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  route_device(a);
}

// ------------------------------------------------------------------------------------------------
// Combine: block b owns the gathered tokens t with t % nact == b on EVERY rank.
//   phase A  partial[t] = sum over the local (token, k) pairs of y[pair]       (this rank's heap)
//   barrier  block b of every rank has written its tokens' partial sums
//   phase B  for the tokens of block b that this rank owns: out = sum over ranks of partial[t]
//            (multimem.ld_reduce in the switch, or peer loads).
// ------------------------------------------------------------------------------------------------
template <bool EMU>
__global__ void __launch_bounds__(512) combine_kernel(const __grid_constant__ McbCtx ctx_p,
                                                      const __grid_constant__ McbCombineArgs args_p,
                                                      const McbCtx* ectx, const McbCombineArgs* eargs) {
  const McbCtx& c = EMU ? ectx[blockIdx.y] : ctx_p;
  const McbCombineArgs& a = EMU ? eargs[blockIdx.y] : args_p;
  pdl_wait();
  pdl_launch_dependents();
  combine_body(c, a);
}

}  // namespace mcb

using namespace mcb;

extern "C" {

int mcb_sizeof_route_args() { return (int)sizeof(McbRouteArgs); }
int mcb_sizeof_combine_args() { return (int)sizeof(McbCombineArgs); }

int mcb_launch_route(const McbRouteArgs* args, int grid, int pdl, cudaStream_t stream) {
  if (grid < 1 || grid > 128 || args->num_local_experts > kMaxLocalExperts || args->num_local_experts < 1)
    return cudaErrorInvalidValue;
  return launch_kernel(route_kernel, dim3(grid), dim3(kRouteThreads), 0, stream, pdl, false, *args);
}

int mcb_launch_combine(const McbCtx* ctx, const McbCombineArgs* args, int grid, int threads, int pdl,
                       cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS || threads < 32 || threads > 512 || (threads & 31) || args->hidden % 8)
    return cudaErrorInvalidValue;
  return launch_kernel(combine_kernel<false>, dim3(grid), dim3(threads), 0, stream, pdl, false, *ctx, *args,
                       (const McbCtx*)nullptr, (const McbCombineArgs*)nullptr);
}

int mcb_emu_combine(const McbCtx* d_ctx, const McbCombineArgs* d_args, int world, int grid, int threads,
                    cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS || threads < 32 || threads > 512 || (threads & 31)) return cudaErrorInvalidValue;
  McbCtx dummy{};
  McbCombineArgs dargs{};
  return launch_kernel(combine_kernel<true>, dim3(grid, world), dim3(threads), 0, stream, 0, true, dummy, dargs,
                       d_ctx, d_args);
}

}  // extern "C"
