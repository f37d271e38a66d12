// Host/device shared plain-C structures of the MoE comms kernels.
//
// Every struct here is mirrored field by field with ctypes in ops/_ext.py; the
// library exports mcb_sizeof_* so the Python side can assert the layouts agree.
//
// Memory model: each rank owns one *symmetric heap* (same size, same internal
// offsets on every rank).  A buffer is named by its byte offset into the heap;
// the same offset is valid against the local base, any peer's mapped base, and
// (when an NVSwitch multicast object is bound) the multicast base.
#pragma once
#include <stdint.h>

#define MCB_MAX_RANKS 72      // one NVL72 NVLink domain
#define MCB_MAX_BLOCKS 512    // flag slots per barrier site
#define MCB_NUM_SITES 24      // independent barrier sites / counter rows
#define MCB_STATUS_WORDS 8

// Transports for the cross-GPU part of a kernel.
#define MCB_TRANSPORT_P2P 0        // plain peer ld/st/red through NVLink mappings
#define MCB_TRANSPORT_MULTIMEM 1   // NVSwitch multicast: multimem.st / multimem.ld_reduce / multimem.red

// Barrier sites (one flag row each) so that different kernel families never share slots.
#define MCB_SITE_META 0
#define MCB_SITE_AGV 1
#define MCB_SITE_RSV 2
#define MCB_SITE_A2A_DISPATCH 3
#define MCB_SITE_A2A_COMBINE 4
#define MCB_SITE_UNIFORM_AG 5
#define MCB_SITE_UNIFORM_RS 6
#define MCB_SITE_NORM_IN 7
#define MCB_SITE_NORM_OUT 8
#define MCB_SITE_FUSED_FC1 9
#define MCB_SITE_FUSED_FC2 10
#define MCB_SITE_LAYER 11
#define MCB_SITE_AGV_LL 12       // launch counters of the low-latency paths (no flags used)
#define MCB_SITE_RSV_LL 13
#define MCB_SITE_A2A_GO 14       // local hand-over word of the all-to-all combine
#define MCB_SITE_TEST 15
#define MCB_SITE_FC1_FUSED 16     // per-block launch counters of the fused dispatch + routing + FC1 kernel
#define MCB_SITE_STEP_META 17     // count exchange at the start of a persistent decode step (slot 0)
#define MCB_SITE_STEP 18          // block-matched barrier of each layer of a persistent decode step
#define MCB_SITE_A2A_STEP_META 20 // count exchange at the start of a persistent all-to-all step (slot 0)
#define MCB_SITE_A2A_STEP 21      // block-matched barrier of each layer of a persistent all-to-all step
#define MCB_SITE_A2A_STEP_CREDIT 22  // per-block count of packet-mode layers of the all-to-all step (epochs only)
#define MCB_SITE_STEP_CREDIT 19   // per-block count of packet-mode layers (epochs only; the credit words are
                                  // in a heap region of their own, McbDenseStepArgs::credit_off)

// Status codes written to status[0] (first error wins; 0 = healthy).
#define MCB_OK 0
#define MCB_ERR_TIMEOUT 1        // a bounded cross-GPU wait ran out
#define MCB_ERR_CAPACITY 2       // a token count exceeded the buffer capacity
#define MCB_ERR_BOUNDS 3         // an offset fell outside its buffer
#define MCB_ERR_ROUTING 4        // an expert id outside [0, num_experts)

#ifdef __cplusplus
extern "C" {
#endif

// Per-rank communication context, passed by value to every kernel.
typedef struct {
  int32_t rank;
  int32_t world;
  int32_t transport;           // MCB_TRANSPORT_*
  int32_t reserved0;
  uint64_t timeout_ns;         // budget of each bounded wait
  uint8_t* heap_local;         // this rank's heap
  uint8_t* heap_mc;            // multicast alias of the heap (NULL without NVLS)
  uint64_t flags_off;          // heap offset of uint32 flags[MCB_NUM_SITES][MCB_MAX_BLOCKS]
  uint32_t* epochs;            // local (not symmetric) uint32 epochs[MCB_NUM_SITES][MCB_MAX_BLOCKS]
  uint32_t* status;            // local uint32 status[MCB_STATUS_WORDS]
  uint8_t* heap_peer[MCB_MAX_RANKS];  // every rank's heap as mapped here (heap_peer[rank] == heap_local)
} McbCtx;

// Token-count exchange: counts -> step_meta = [valid(sum), offset(prefix), max, 0].
typedef struct {
  const int32_t* n_local;      // device scalar: this rank's token count
  uint64_t counts_off;         // heap offset of int32 counts[2][MCB_MAX_RANKS] (parity double buffer)
  int32_t* step_meta;          // local int32[4]
  int32_t cap;                 // per-rank capacity (n_local > cap raises MCB_ERR_CAPACITY)
  int32_t reserved0;
} McbMetaArgs;

#define MCB_MAX_TENSORS 4

// Variable all-gather of up to MCB_MAX_TENSORS row-major tensors into packed
// [sum(n), row_bytes] heap buffers at row offset step_meta[1].
typedef struct {
  const void* src[MCB_MAX_TENSORS];
  uint64_t dst_off[MCB_MAX_TENSORS];
  uint32_t row_bytes[MCB_MAX_TENSORS];
  int32_t num_tensors;
  int32_t cap;                 // per-rank row capacity
  int32_t site;
  // Non-zero when the kernel launched just before this one does not write n_local / step_meta
  // (true for every launch of a step but the first after the metadata kernel): the kernel then
  // reads them before waiting on its predecessor, hiding one memory round trip.
  int32_t meta_stable;
  const int32_t* n_local;
  const int32_t* step_meta;
  // Low-latency mode (0 rows = off): when the step holds at most ll_rows rows over all ranks,
  // rows travel as 16-byte {data, flag, data, flag} packets through a staging area and the
  // receiver polls the packets themselves, so no fence and no separate barrier are needed.
  uint64_t ll_off;             // heap: [2][ll_rows][8-byte words per row] packets of 16 bytes
  int32_t ll_rows;
  int32_t reserved1;
} McbAgvArgs;

// Variable reduce-scatter: out[t,:] = sum over ranks of heap[src_off][(offset+t),:].
typedef struct {
  void* out;
  uint64_t src_off;
  uint32_t row_bytes;
  int32_t dtype;               // 0 = bf16 operands with fp32 accumulation, 1 = fp32
  int32_t cap;
  int32_t site;
  const int32_t* n_local;
  const int32_t* step_meta;
  // Low-latency mode (bf16 only): every rank pushes its partial rows to their owner as
  // flagged packets; the owner sums the world's packets in rank order in fp32.
  uint64_t ll_off;             // heap: [2][world][ll_src_rows][row_bytes / 8] packets of 16 bytes
  uint64_t counts_off;         // heap: int32 counts[2][MCB_MAX_RANKS] written by the metadata kernel
  int32_t ll_rows;             // low-latency mode when the step holds at most this many rows in total
  int32_t meta_stable;         // as in McbAgvArgs
  int32_t ll_src_rows;         // rows per source region = min(cap, ll_rows)
  int32_t reserved2;
} McbRsvArgs;

// Words of McbDenseStepArgs::state (local uint32[MCB_STEP_STATE_WORDS], zero at start).  They change
// only when the last block of a step leaves, so every block of a step reads the same values,
// whatever the grid size of this or of earlier launches.
#define MCB_STEP_STATE_WORDS 16
#define MCB_STATE_STEP_SEQ 0      // steps completed
#define MCB_STATE_LAYER_BASE 1    // layers completed (its low bit picks the gathered-buffer parity)
#define MCB_STATE_LL_BASE 2       // packet-mode layers completed (packet flag = this + layer + 1)
#define MCB_STATE_FINISHED 3      // blocks of the running step that have left
#define MCB_STATE_GATE0 4         // [MCB_MAX_GROUPS] pushes drained per pipeline group (zero between steps)
#define MCB_MAX_GROUPS 8

// One whole decode step of the dense dispatcher in ONE persistent kernel: count exchange, then
// num_layers x (all-gather-V push -> one cross-GPU barrier -> reduce-scatter-V), or, for small
// steps, num_layers x (packet all-gather, packet reduce-scatter) with no barrier at all.
typedef struct {
  const void* src[MCB_MAX_TENSORS];          // local inputs [cap, row]
  uint64_t dst_off[MCB_MAX_TENSORS];         // heap: [2][cap * world][row] gathered rows, by layer parity
  uint64_t dst_par_stride[MCB_MAX_TENSORS];  // bytes between the two parities
  uint32_t row_bytes[MCB_MAX_TENSORS];
  int32_t num_tensors;
  int32_t cap;                  // per-rank row capacity
  int32_t num_layers;
  int32_t rsv_dtype;            // 0 = bf16 operands with fp32 accumulation, 1 = fp32
  void* out;                    // local [cap, rsv_row_bytes]
  uint64_t rsv_off;             // heap: [cap * world][rsv_row_bytes] partial sums of every rank
  uint32_t rsv_row_bytes;
  int32_t ll_rows;              // packet mode when the step holds at most this many rows (0 = never)
  uint64_t agv_ll_off;          // heap: [2][ll_rows][sum(row_bytes) / 8] packets of 16 bytes
  uint64_t rsv_ll_off;          // heap: [2][world][ll_src_rows][rsv_row_bytes / 8] packets of 16 bytes
  int32_t ll_src_rows;          // min(cap, ll_rows)
  int32_t groups;               // pipeline groups of the barrier mode (1 = none)
  uint64_t group_min_bytes;     // a group must move at least this many bytes per rank and layer
  const int32_t* n_local;       // device scalar: this rank's row count
  int32_t* step_meta;           // local int32[8]: valid, offset, max, (kept), step number, parity of the
                                //   last layer's gathered buffers, mode (0 barrier, 1 packets), groups used
  uint64_t counts_off;          // heap: int32 counts[2][MCB_MAX_RANKS] of this kernel (by step parity)
  uint64_t credit_off;          // heap: uint32 credit[grid][MCB_MAX_RANKS] of the packet mode (zero at start)
  uint32_t* state;              // local uint32[MCB_STEP_STATE_WORDS]
  // Self-checking build (race tests only): non-zero `check` selects it; the payload is then a hash of
  // (layer, position) that every receiver verifies, mismatches are counted in *check_errors, and
  // the rank sleeps delay_ns (at most 1 ms) before every delay_every-th layer.
  uint32_t* check_errors;
  int32_t check;
  int32_t delay_every;
  uint32_t delay_ns;
  // Non-zero: tensor 0's source is bf16 [cap, fp8_hidden] and is dispatched as 1 x 128 block-scaled e4m3
  // (row_bytes[0] = fp8_hidden bytes), with the fp32 scales as gathered tensor 3 (src[3] unused).
  uint32_t fp8_hidden;
} McbDenseStepArgs;

// All-to-all-V dispatch (one copy of a token per distinct destination rank).
typedef struct {
  const void* x;               // [n, hidden] bf16
  const int64_t* topk_idx;     // [n, topk]
  const float* topk_w;         // [n, topk] (may be NULL)
  uint64_t recv_x_off;         // heap: [world][cap][hidden] bf16, or e4m3 when fp8 != 0
  uint64_t recv_scale_off;     // heap: [world][cap][hidden/128] fp32 (fp8 only)
  uint64_t recv_idx_off;       // heap: [world][cap][topk] int64
  uint64_t recv_w_off;         // heap: [world][cap][topk] fp32
  uint64_t recv_src_off;       // heap: [world][cap] int32 source token index
  uint64_t recv_count_off;     // heap: [MCB_MAX_RANKS] int32 rows received from each source
  int32_t* slot_map;           // local [cap][world] int32: slot on each destination, -1 = not sent
  int32_t* send_count;         // local [MCB_MAX_RANKS + 1] int32 scratch (last word = blocks done)
  const int32_t* n_local;
  int32_t hidden;
  int32_t topk;
  int32_t num_experts;
  int32_t cap;
  int32_t fp8;
  int32_t reserved0;
} McbA2ADispatchArgs;

// One whole decode step of the all-to-all dispatcher in ONE persistent kernel: count exchange, then
// num_layers x (push every token's row and routing to each distinct destination rank -> one
// block-matched cross-GPU barrier -> pull the expert outputs back and sum them).  A token keeps its
// own index as its slot on every destination (receive layout [parity][source][cap]), so no slot
// counters exist; a row is valid on the destination when the stamp in its metadata row equals the
// layer's sequence number (McbA2AStepArgs::step_meta[4] after the step).
typedef struct {
  const void* x;               // [cap, hidden] bf16
  const int64_t* topk_idx;     // [cap, topk]
  const float* topk_w;         // [cap, topk] (may be NULL: weights of 1)
  void* out;                   // [cap, hidden] bf16
  const int32_t* n_local;
  uint64_t recv_x_off;         // heap: [2][world][cap][hidden] bf16, or e4m3 bytes when fp8 != 0
  uint64_t recv_scale_off;     // heap: [2][world][cap][hidden/128] fp32 (fp8 only)
  uint64_t recv_meta_off;      // heap: [2][world][cap][meta_row_bytes]: {stamp, source token, (expert id i32, weight f32) x topk}
  uint64_t y_off;              // heap: [2][world][cap][hidden] bf16 expert outputs (== recv_x_off for the identity expert in bf16)
  uint64_t x_par_stride;       // bytes between the two parities of each buffer
  uint64_t scale_par_stride;
  uint64_t meta_par_stride;
  uint64_t y_par_stride;
  uint32_t meta_row_bytes;     // 8 + 8 * topk rounded up to 16
  int32_t hidden;
  int32_t topk;
  int32_t num_experts;
  int32_t cap;
  int32_t fp8;
  int32_t num_layers;
  int32_t ll_rows;             // packet mode when the step holds at most this many tokens over all ranks (0 = never)
  int32_t* step_meta;          // local int32[8]: valid, offset, max, -, step number, parity of the last layer, mode, stamp of the last layer
  uint64_t counts_off;         // heap: int32 counts[2][MCB_MAX_RANKS] of this kernel
  uint32_t* state;             // local uint32[MCB_STEP_STATE_WORDS] (step_seq, layer_base, -, finished)
  // Packet mode: rows travel as 16-byte {data, flag, data, flag} packets.  Dispatch staging on the
  // destination: [2][world][ll_src_rows][1 + row words + scale words + metadata words] packets (word 0 is
  // a header {routed here?, token} that EVERY rank receives for every token, so a destination knows what
  // to wait for); combine staging on the source: [2][world][ll_src_rows][hidden / 4] packets.
  uint64_t ll_x_off;
  uint64_t ll_y_off;
  uint64_t credit_off;         // heap: uint32 credit[grid][MCB_MAX_RANKS] (zero at start)
  int32_t ll_src_rows;         // min(cap, ll_rows)
  int32_t reserved1;
} McbA2AStepArgs;

// All-to-all-V combine: out[t,:] = sum over destination ranks d of y_d[rank][slot_map[t][d],:].
typedef struct {
  void* out;                   // [n, hidden] bf16
  uint64_t y_off;              // heap: [world][cap][hidden] bf16 expert outputs in receive layout
  const int32_t* slot_map;
  const int32_t* n_local;
  int32_t hidden;
  int32_t cap;
} McbA2ACombineArgs;

// Reduce-scatter + residual add + RMSNorm + all-gather, in place in a heap buffer.
typedef struct {
  uint64_t buf_off;            // heap: [tokens][hidden] bf16 partial sums in, normalised rows out
  void* residual;              // local [tokens/world][hidden] bf16, updated in place
  const void* weight;          // [hidden] bf16
  float eps;
  int32_t hidden;
  int32_t tokens;              // total rows (multiple of world)
  int32_t reserved0;
} McbNormArgs;

#ifdef __cplusplus
}
#endif
