// Entry point for callers that must not allocate GPU memory.
//
// This has no counterpart in the reference benchmark; it exists for users of this library
// whose launch site cannot call cudaMalloc: code running inside a serving loop whose memory
// was handed out once at start-up by its own pool, plug-ins that are given a stream and
// buffers but no allocator, and code on a latency path where an allocation (which can
// synchronise the whole device) is not acceptable.
//
// mcb_a2a_dispatch_noalloc() is mcb_launch_a2a_dispatch() with one difference: the small
// scratch area of the kernel (one slot counter per destination rank plus the "blocks done"
// word, McbA2ADispatchArgs::send_count) is not taken from the caller.  It is a fixed array
// inside the library, MCB_NOALLOC_SCRATCH_BYTES bytes, present on every GPU that loads the
// library until the process exits.  The `send_count` field of `args` is ignored; every other
// field (inputs, receive buffers, slot_map, the context) is passed by the caller as usual.
//
// Rules:
//   * World sizes above MCB_NOALLOC_MAX_RANKS are refused with cudaErrorInvalidValue;
//     mcb_noalloc_last_error() then returns a sentence that says why.
//   * The call allocates nothing: no cudaMalloc / cudaFree, no allocating library routine.
//     It issues one cudaMemsetAsync on the scratch array (the counters must start at zero)
//     and one kernel launch, both on `stream`.
//   * The first call on each device looks up the device address of the scratch array
//     (cudaGetSymbolAddress, with that device current).  Make that first call before any
//     stream capture begins on that device.
//   * All calls on a device share the one array.  Calls that can overlap on the GPU (two
//     streams, or two host threads) race on it: serialise them, or use the ordinary entry
//     point with a send_count buffer per call site.
#pragma once
#include <cuda_runtime.h>

#include "mcb_ctx.h"

#define MCB_NOALLOC_MAX_RANKS MCB_MAX_RANKS
#define MCB_NOALLOC_SCRATCH_BYTES ((MCB_NOALLOC_MAX_RANKS + 1) * 4)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 (cudaSuccess) or a cudaError_t value.
int mcb_a2a_dispatch_noalloc(const McbCtx* ctx, const McbA2ADispatchArgs* args, int grid, int threads,
                             cudaStream_t stream);
// Human-readable reason why the most recent call was refused ("" if it was not).
const char* mcb_noalloc_last_error(void);
int mcb_noalloc_max_ranks(void);
int mcb_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
