// Grouped expert GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), sm_100a.
//
// The reference has no GEMM at all (its expert is the identity, bench_nvls.py:109-112); this
// is the "real expert" half of the fused dispatcher.  One persistent kernel computes, for a
// table of row tiles (expert, first pair row, row count), either
//   MODE_FC1: act[row, i]  = silu(x[tok(row)] . Wg[e][i]) * (x[tok(row)] . Wu[e][i])
//   MODE_FC2: y[row, h]    = prob[row] * (act[row] . Wd[e][h])
// as D[128 rows, 256 cols] += A[128, K] * B[256, K]^T with one tcgen05.mma per 16 of K:
//   * B (weights, K-major) is streamed by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle,
//     no multicast) as two 128-row boxes per stage: gate rows + matching up rows for FC1, so
//     that the SwiGLU needs no second pass; two consecutive row blocks for FC2;
//   * A (token rows) is gathered by four producer warps straight from the gathered-token
//     buffer through the pair -> token index list (this is the routing permute, fused into the
//     operand load): each thread owns one row and issues asynchronous 16-byte copies
//     (cp.async) into the same 128-byte-swizzled K-major layout, completion arriving on the
//     stage's mbarrier, so the gather runs as many stages ahead as the weight stream does;
//   * accumulators live in TMEM, double buffered (2 x 256 columns), so the epilogue of one
//     tile overlaps the MMAs of the next; the epilogue reads them with tcgen05.ld;
//   * one elected thread issues the MMAs; mbarriers (full/empty per stage, full/empty per
//     accumulator) connect the roles; every wait is bounded and reports through a status word.
// Rows of a tile beyond its row count are padding: their A rows are never written and their
// accumulator rows never read (each output row depends on its own A row only).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mcb_combine.cuh"
#include "mcb_dense.cuh"
#include "mcb_gemm.h"
#include "mcb_launch.h"
#include "mcb_route.cuh"
#include "mcb_tc.cuh"

namespace mcb {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;          // 128 bytes of bf16: one swizzle atom row
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kABytes = kBlockM * kBlockK * 2;   // 16 KiB
constexpr int kBBytes = kBlockN * kBlockK * 2;   // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;
constexpr int kNumThreads = 320;                 // 10 warps
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;

// Instruction descriptor: D=f32, A=B=bf16, both K-major, N=256, M=128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBlockN >> 3) << 17) |
                                ((uint32_t)(kBlockM >> 4) << 24);

template <int MODE>
__device__ __forceinline__ void gemm_device(const CUtensorMap& w_map, const McbGemmArgs& a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full = bars;                       // [kStages]
  uint64_t* empty = bars + kStages;            // [kStages]
  uint64_t* tfull = bars + 2 * kStages;        // [2]
  uint64_t* tempty = bars + 2 * kStages + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1 + 128); mbar_init(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const Abort ab{abort_flag, a.status, a.timeout_ns};

  const int n_tiles = a.n_total / (MODE == MCB_GEMM_FC1 ? 2 * 128 : kBlockN);  // FC1: n_total = 2I, 128 gate + 128 up per tile
  const int num_m_tiles = *a.num_m_tiles;
  const int total = num_m_tiles * n_tiles;
  const int k_blocks = a.k_total / kBlockK;

  if (warp == 0) {
    // ---------------- TMA producer: weights ----------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
        const int e = a.tile_expert[mt];
        int r0, r1;
        if (MODE == MCB_GEMM_FC1) {
          r0 = e * a.n_total + nt * 128;               // gate rows
          r1 = r0 + a.n_total / 2;                     // matching up rows
        } else {
          r0 = e * a.n_total + nt * kBlockN;
          r1 = r0 + 128;
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&empty[s], ph ^ 1u, ab, 1))) break;
          uint8_t* sb = smem + s * kStageBytes + kABytes;
          mbar_arrive_expect_tx(&full[s], kBBytes);
          tma_load_2d(sb, &w_map, &full[s], kb * kBlockK, r0);
          tma_load_2d(sb + 128 * 128, &w_map, &full[s], kb * kBlockK, r1);
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      int acc = 0; uint32_t acc_ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        if (!(ok = mbar_wait(&tempty[acc], acc_ph ^ 1u, ab, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kBlockN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&full[s], ph, ab, 3))) break;
          fence_proxy_async_smem();           // the A rows were written by cp.async, not by TMA
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint64_t da = make_sw128_desc(sa), db = make_sw128_desc(sa + kABytes);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            // 16 bf16 of K = 32 bytes further inside the swizzled row: +2 in 16-byte units
            umma_bf16(d_tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), kInstrDesc, (kb | kk) != 0);
          }
          umma_commit(&empty[s]);             // stage may be refilled once these MMAs have read it
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);             // accumulator complete
        if (++acc == 2) { acc = 0; acc_ph ^= 1u; }
      }
    }
  } else if (warp < 6) {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int q = warp & 3;                  // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    int acc = 0; uint32_t acc_ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
      const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
      const int row0 = a.tile_row0[mt], rows = a.tile_rows[mt];
      if (!(ok = mbar_wait(&tfull[acc], acc_ph, ab, 4))) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kBlockN);
      const bool live = row_in_tile < rows;
      const long long prow = (long long)row0 + row_in_tile;
      if (MODE == MCB_GEMM_FC1) {
        uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) + prow * a.out_row_bytes + (long long)nt * 128 * 2;
#pragma unroll 1
        for (int j = 0; j < 8; ++j) {
          uint32_t g[16], u[16];
          tmem_ld16(t_row + j * 16, g);
          tmem_ld16(t_row + 128 + j * 16, u);
          tmem_ld_wait();
          if (live) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float a0 = silu(__uint_as_float(g[2 * i])) * __uint_as_float(u[2 * i]);
              const float a1 = silu(__uint_as_float(g[2 * i + 1])) * __uint_as_float(u[2 * i + 1]);
              o[i] = pack2(a0, a1);
            }
            uint4* dst = reinterpret_cast<uint4*>(orow + j * 32);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      } else {
        const float p = live ? (a.row_scale ? a.row_scale[prow] : 1.0f) : 0.f;
        uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) + prow * a.out_row_bytes + (long long)nt * kBlockN * 2;
#pragma unroll 1
        for (int j = 0; j < 16; ++j) {
          uint32_t v[16];
          tmem_ld16(t_row + j * 16, v);
          tmem_ld_wait();
          if (live) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = pack2(__uint_as_float(v[2 * i]) * p, __uint_as_float(v[2 * i + 1]) * p);
            uint4* dst = reinterpret_cast<uint4*>(orow + j * 32);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) { acc = 0; acc_ph ^= 1u; }
    }
  } else {
    // ---------------- A producers: gather token rows into swizzled shared memory ----------------
    const int r = threadIdx.x - 6 * 32;      // row of the tile handled by this thread (0..127)
    int s = 0; uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
      const int mt = tile / n_tiles;
      const int row0 = a.tile_row0[mt], rows = a.tile_rows[mt];
      const bool live = r < rows;
      long long src_row = 0;
      if (live) src_row = a.row_index ? (long long)a.row_index[row0 + r] : (long long)(row0 + r);
      const uint8_t* src = reinterpret_cast<const uint8_t*>(a.a_base) + src_row * a.a_row_bytes;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!(ok = mbar_wait(&empty[s], ph ^ 1u, ab, 5))) break;
        if (live) {
          uint8_t* sa = smem + s * kStageBytes + r * 128;
          const uint8_t* g = src + (long long)kb * (kBlockK * 2);
#pragma unroll
          for (int c = 0; c < 8; ++c) cp_async_16(sa + ((c ^ (r & 7)) << 4), g + c * 16);
        }
        cp_async_arrive_noinc(&full[s]);     // arrives when this thread's copies have landed
        if (++s == kStages) { s = 0; ph ^= 1u; }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) __nanosleep(50000);        // let any copy still in flight land before the CTA goes away
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int MODE>
__global__ void __launch_bounds__(kNumThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ McbGemmArgs a) {
  gemm_device<MODE>(w_map, a);
}

// Dispatch, routing and FC1 in ONE kernel: every CTA first pushes its share of this rank's
// tokens to all ranks (multimem.st or flagged packets) and meets the other ranks; after a
// grid-wide barrier the gathered routing is turned into pair lists and row tiles; after a second
// one the same CTAs run the grouped FC1 GEMM, gathering token rows straight from the buffer the
// peers just filled.
__global__ void __launch_bounds__(kNumThreads, 1)
dispatch_route_fc1_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ McbGemmArgs a,
                          const __grid_constant__ McbCtx c, const __grid_constant__ McbAgvArgs agv,
                          const __grid_constant__ McbRouteArgs r) {
  uint32_t ll_launch = 0;
  agv_device<MCB_SITE_FC1_FUSED>(c, agv, ll_launch);          // waits for the previous kernel first
  // The arrival counter is back at zero whenever a launch has ended (its last block resets it).
  uint32_t* arrivals = epoch_ptr(c, MCB_SITE_LAYER, 1);
  grid_sync(c, arrivals, gridDim.x);
  route_device(r);
  grid_sync(c, arrivals, 2u * gridDim.x);
  gemm_device<MCB_GEMM_FC1>(w_map, a);
  launch_end(c, MCB_SITE_FC1_FUSED, ll_launch, arrivals);
}

// FC2 GEMM and the cross-rank combine in ONE kernel: the persistent GEMM CTAs finish their
// tiles (y = prob * act Wd^T), free their TMEM, meet in a grid-wide barrier (all CTAs are
// co-resident: the launch is cooperative), and then run the combine: local pre-sum of each
// token's pairs into the symmetric partial-sum buffer, block-matched cross-GPU barrier,
// multimem.ld_reduce (or peer loads) of the rows this rank owns.
__global__ void __launch_bounds__(kNumThreads, 1)
fc2_combine_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ McbGemmArgs a,
                   const __grid_constant__ McbCtx c, const __grid_constant__ McbCombineArgs cmb) {
  gemm_device<MCB_GEMM_FC2>(w_map, a);
  // grid-wide barrier: every CTA's y rows are written before any CTA sums them
  const uint32_t launch = launch_begin(c, MCB_SITE_FUSED_FC1);
  uint32_t* arrivals = epoch_ptr(c, MCB_SITE_LAYER, 0);
  grid_sync(c, arrivals, gridDim.x);
  combine_body(c, cmb);
  launch_end(c, MCB_SITE_FUSED_FC1, launch, arrivals);
}

}  // namespace mcb

using namespace mcb;

extern "C" {

int mcb_sizeof_gemm_args() { return (int)sizeof(McbGemmArgs); }
int mcb_gemm_smem_bytes() { return kSmemBytes; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Fills `out` (128 bytes, 64-byte aligned host memory) with a tensor map over a row-major bf16
// matrix [rows, cols]: boxes of 128 rows x 64 columns, 128-byte swizzle.
int mcb_make_weight_tmap(void* out, const void* base, uint64_t rows, uint64_t cols) {
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (err != cudaSuccess) return (int)err;
    if (qres != cudaDriverEntryPointSuccess || !fn) return (int)cudaErrorNotSupported;
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if (cols % kBlockK || rows % 128 || (reinterpret_cast<uintptr_t>(base) & 15)) return (int)cudaErrorInvalidValue;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                      dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

static bool configure_gemm_kernels() {
  static int state = 0;   // 0 = not tried, 1 = ok, -1 = failed
  if (state == 0) {
    cudaError_t e1 = cudaFuncSetAttribute(grouped_gemm_kernel<MCB_GEMM_FC1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaError_t e2 = cudaFuncSetAttribute(grouped_gemm_kernel<MCB_GEMM_FC2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaError_t e3 = cudaFuncSetAttribute(fc2_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cudaError_t e4 = cudaFuncSetAttribute(dispatch_route_fc1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    state = (e1 == cudaSuccess && e2 == cudaSuccess && e3 == cudaSuccess && e4 == cudaSuccess) ? 1 : -1;
  }
  return state == 1;
}

// FC2 + combine in one cooperative launch (grid <= number of SMs; one CTA per SM).
int mcb_launch_fc2_combine(const void* tmap, const McbGemmArgs* args, const McbCtx* ctx, const McbCombineArgs* cmb,
                           int grid, int pdl, cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS || !tmap || !args || !ctx || !cmb) return cudaErrorInvalidValue;
  if (args->k_total % kBlockK || args->k_total < kBlockK || args->n_total % kBlockN) return cudaErrorInvalidValue;
  if ((args->a_row_bytes & 15) || (args->out_row_bytes & 15) || cmb->hidden % 8) return cudaErrorInvalidValue;
  if (!configure_gemm_kernels()) return cudaErrorUnknown;
  const CUtensorMap& map = *reinterpret_cast<const CUtensorMap*>(tmap);
  return launch_kernel(fc2_combine_kernel, dim3(grid), dim3(kNumThreads), kSmemBytes, stream, pdl, true, map, *args, *ctx, *cmb);
}

// Dispatch + routing + FC1 in one cooperative launch (grid <= number of SMs).
int mcb_launch_dispatch_route_fc1(const void* tmap, const McbGemmArgs* args, const McbCtx* ctx, const McbAgvArgs* agv,
                                  const McbRouteArgs* route, int grid, int pdl, cudaStream_t stream) {
  if (grid < 1 || grid > MCB_MAX_BLOCKS || !tmap || !args || !ctx || !agv || !route) return cudaErrorInvalidValue;
  if (args->k_total % kBlockK || args->k_total < kBlockK || args->n_total % 256) return cudaErrorInvalidValue;
  if ((args->a_row_bytes & 15) || (args->out_row_bytes & 15)) return cudaErrorInvalidValue;
  if (route->num_local_experts < 1 || route->num_local_experts > kMaxLocalExperts) return cudaErrorInvalidValue;
  if (!configure_gemm_kernels()) return cudaErrorUnknown;
  const CUtensorMap& map = *reinterpret_cast<const CUtensorMap*>(tmap);
  return launch_kernel(dispatch_route_fc1_kernel, dim3(grid), dim3(kNumThreads), kSmemBytes, stream, pdl, true, map,
                       *args, *ctx, *agv, *route);
}

int mcb_launch_grouped_gemm(const void* tmap, const McbGemmArgs* args, int mode, int grid, int pdl, cudaStream_t stream) {
  if (grid < 1 || !tmap || !args) return cudaErrorInvalidValue;
  if (args->k_total % kBlockK || args->k_total < kBlockK) return cudaErrorInvalidValue;
  if (mode == MCB_GEMM_FC1 ? (args->n_total % 256) : (args->n_total % kBlockN)) return cudaErrorInvalidValue;
  if ((args->a_row_bytes & 15) || (args->out_row_bytes & 15)) return cudaErrorInvalidValue;
  if (!configure_gemm_kernels()) return cudaErrorUnknown;
  const CUtensorMap& map = *reinterpret_cast<const CUtensorMap*>(tmap);
  if (mode == MCB_GEMM_FC1)
    return launch_kernel(grouped_gemm_kernel<MCB_GEMM_FC1>, dim3(grid), dim3(kNumThreads), kSmemBytes, stream, pdl, false, map, *args);
  return launch_kernel(grouped_gemm_kernel<MCB_GEMM_FC2>, dim3(grid), dim3(kNumThreads), kSmemBytes, stream, pdl, false, map, *args);
}

}  // extern "C"
