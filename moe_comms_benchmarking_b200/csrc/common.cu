// Library-wide exports: struct sizes (checked by the Python binding), error strings and
// small device-memory utilities.
#include <cuda_runtime.h>

#include "mcb_ctx.h"

extern "C" {

int mcb_sizeof_ctx() { return (int)sizeof(McbCtx); }
int mcb_sizeof_meta_args() { return (int)sizeof(McbMetaArgs); }
int mcb_sizeof_agv_args() { return (int)sizeof(McbAgvArgs); }
int mcb_sizeof_rsv_args() { return (int)sizeof(McbRsvArgs); }
int mcb_sizeof_a2a_dispatch_args() { return (int)sizeof(McbA2ADispatchArgs); }
int mcb_sizeof_a2a_combine_args() { return (int)sizeof(McbA2ACombineArgs); }
int mcb_sizeof_norm_args() { return (int)sizeof(McbNormArgs); }

const char* mcb_error_string(int err) { return cudaGetErrorString((cudaError_t)err); }

int mcb_max_ranks() { return MCB_MAX_RANKS; }
int mcb_max_blocks() { return MCB_MAX_BLOCKS; }
int mcb_num_sites() { return MCB_NUM_SITES; }

}  // extern "C"
