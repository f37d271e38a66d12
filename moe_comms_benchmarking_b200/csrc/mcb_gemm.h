// Argument blocks of the expert path: routing (pair lists, row tiles) and grouped GEMMs.
// Mirrored with ctypes in ops/_ext.py.
#pragma once
#include <stdint.h>

#include "mcb_ctx.h"

#define MCB_GEMM_FC1 0          // gate/up projection + SwiGLU epilogue
#define MCB_GEMM_FC2 1          // down projection + per-row scale epilogue
#define MCB_GEMM_ERR_TIMEOUT 5  // status code: a bounded mbarrier wait ran out

#ifdef __cplusplus
extern "C" {
#endif

// One grouped GEMM: out[row, :] = epilogue(A[row_index[row], :] . W[expert(row)]^T).
typedef struct {
  const void* a_base;          // A rows, bf16, K contiguous
  uint64_t a_row_bytes;
  const int32_t* row_index;    // pair row -> A row (NULL: identity)
  const float* row_scale;      // FC2: factor per pair row (NULL: 1)
  void* out;                   // bf16 [pair rows, n_out]
  uint64_t out_row_bytes;
  const int32_t* tile_expert;  // per row tile: local expert
  const int32_t* tile_row0;    //               first pair row
  const int32_t* tile_rows;    //               rows in the tile (1..128)
  const int32_t* num_m_tiles;  // device scalar
  int32_t n_total;             // weight rows per expert (FC1: 2*I, gate rows then up rows; FC2: H)
  int32_t k_total;             // reduction length (FC1: H; FC2: I)
  uint32_t* status;            // status words (may be NULL)
  uint64_t timeout_ns;
} McbGemmArgs;

// Grouped SwiGLU FFN with the weights as the M operand (mcb_ffn.cuh): both projections in one
// persistent kernel over the pair lists written by the routing.
typedef struct {
  const void* x;               // gathered tokens [T, hidden] bf16
  uint64_t x_row_bytes;
  const int32_t* pair_token;   // [P] pair row -> gathered token
  const float* pair_prob;      // [P] routing weight of each pair row (NULL: 1)
  const int32_t* expert_offset;  // [E_loc + 1] first pair row of each local expert
  const int32_t* max_rows;     // device scalar: largest pair count of one expert
  void* act;                   // [P, intermediate] bf16 (written by the gate/up blocks, read by the down blocks)
  void* y;                     // [P, hidden] bf16 = prob * (act . Wd^T)
  int32_t* ffn_done;           // [E_loc] quarter-blocks of gate/up finished (zeroed by the routing)
  int32_t num_local_experts;
  int32_t hidden;              // multiple of 128
  int32_t intermediate;        // multiple of 128
  int32_t reserved0;
  uint32_t* status;
  uint64_t timeout_ns;
  const void* w1;              // packed interleaved gate/up matrix (E * 2I rows, hidden columns), see mcb_ffn.cuh
  const void* w2;              // packed down matrix (E * hidden rows, I columns)
} McbFfnArgs;

// Routing of the gathered tokens to this rank's experts.
typedef struct {
  const int64_t* topk_idx;     // gathered [T, topk]
  const float* topk_w;         // gathered [T, topk]
  const int32_t* num_tokens;   // device scalar T (step_meta[0])
  int32_t topk;
  int32_t expert_begin;        // first expert owned by this rank
  int32_t num_local_experts;
  int32_t max_tokens;          // capacity of the gathered buffers (bounds check)
  int32_t* expert_count;       // [E_loc]        (scratch, zero between launches)
  int32_t* expert_cursor;      // [E_loc]        (scratch, zero between launches)
  int32_t* expert_offset;      // [E_loc + 1]    first pair row of each expert
  int32_t* pair_token;         // [P] gathered-token index of each pair row
  float* pair_prob;            // [P] routing weight of each pair row
  int32_t* pair_pos;           // [T, topk] pair row of (token, k), -1 if the expert is not local
  int32_t* tile_expert;        // row-tile table consumed by the grouped GEMMs
  int32_t* tile_row0;
  int32_t* tile_rows;
  int32_t* num_m_tiles;        // device scalar
  int32_t* sync;               // [4] scratch: blocks-done (2 phases), ready counter, spare
  int32_t max_pairs;           // capacity of the pair arrays
  int32_t max_tiles;           // capacity of the tile table
  uint32_t* status;
  uint64_t timeout_ns;
  int32_t* max_rows;           // device scalar: largest number of pair rows of one expert (may be NULL)
  int32_t* ffn_done;           // [E_loc] gate/up blocks finished per expert, set to zero here (may be NULL)
} McbRouteArgs;

// Local pre-sum of each token's expert outputs + cross-rank reduce-scatter.
typedef struct {
  const void* y;               // [P, hidden] bf16, already scaled by the routing weight
  const int32_t* pair_pos;     // [T, topk]
  uint64_t partial_off;        // heap: [T_cap, hidden] bf16 per-rank partial sums
  void* out;                   // local [cap, hidden] bf16
  const int32_t* n_local;
  const int32_t* step_meta;    // [valid, offset, max, epoch]
  int32_t hidden;
  int32_t topk;
  int32_t cap;                 // per-rank capacity
  int32_t site;
  // Bytes between two copies of the partial-sum buffer (0 = one copy).  With two, a caller that runs
  // layers back to back alternates between them, so a rank that is already writing the partial sums of
  // the next layer cannot disturb a peer that is still reducing this one (the barrier inside every
  // combine keeps ranks within one layer of each other).
  uint64_t partial_par_stride;
} McbCombineArgs;

#ifdef __cplusplus
}
#endif

#ifdef MCB_WITH_LAYER_ARGS
// Everything one MoE layer needs, as ONE kernel parameter (or one element of a device array when
// several ranks are emulated inside one launch): the context and the argument blocks of the four phases.
typedef struct alignas(64) {
  McbCtx ctx;
  McbAgvArgs agv;
  McbRouteArgs route;
  McbFfnArgs ffn;
  McbCombineArgs cmb;
  // Optional phase trace (null = off): block 0 stores the global timer (ns) at kernel entry and after
  // dispatch, grid barrier, routing, grid barrier, experts, grid barrier, combine (8 words).
  unsigned long long* trace;
  unsigned long long reserved0;
} McbLayerArgs;
#endif
