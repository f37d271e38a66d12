// Grouped SwiGLU expert FFN for decode-size batches on the 5th-generation tensor cores, with the
// operands swapped: the WEIGHTS are the M = 128 operand and the tokens of one expert are the small N.
//
// The reference has no expert computation at all (identity expert, bench_nvls.py:109-112).  At
// decode sizes an expert sees a handful of tokens (3 at a global batch of 64, 170 at 4096 with 512
// experts / top-22), and a layer is bound by streaming 6 MB of weights per expert.  With tokens as
// the M operand every expert costs a full 128-row MMA and experts with more than 128 tokens read
// their weights once per 128 tokens; here
//   * a work unit is 128 weight rows x the whole reduction length (256 KB of bf16 at K = 1024) of
//     one expert, multiplied with ALL tokens of that expert in one pass: D[128, N] += W[128, K] X[N, K]^T
//     with N = the expert's token count rounded up to 16 (up to 256 per pass, accumulators double
//     buffered in TMEM), so an MMA costs N / 256 of the padded one and every weight byte is read once;
//   * both projections run in ONE persistent kernel: units 0 .. E * 2I/128 are the gate/up blocks,
//     the rest the down blocks, dealt round-robin over the CTAs, so the weight stream does not stop
//     at a kernel boundary.  A down block of expert e waits until all gate/up blocks of e have
//     stored their activations (a counter per expert; every CTA meets all its gate/up blocks before
//     its first down block, so the wait cannot deadlock);
//   * the gate/up matrix is stored interleaved (row 2i = gate row i, row 2i + 1 = up row i), so a
//     128-row block yields 64 finished activations: the two values meet in neighbouring TMEM lanes
//     and are exchanged with one shuffle;
//   * the weights are PRE-PACKED, once, into the image their tiles have in shared memory: tile
//     (128-row block, 64-column block) is 16 KB of contiguous memory holding the 128 x 64 bf16 values
//     in the K-major layout with 128-byte swizzle that the MMA descriptor expects, and the 16 tiles of
//     a work unit follow one another.  A stage is then filled by ONE bulk copy (cp.async.bulk, no
//     tensor map, no multicast) of a contiguous 16 KB range, so DRAM sees long sequential reads
//     instead of 128 strided 128-byte pieces per tile;
//   * token rows arrive by asynchronous 16-byte copies through the pair -> token list (the routing
//     permute fused into the operand load) into the same swizzled K-major layout, eight neighbouring
//     threads reading the 128 bytes of one row; a pipeline stage holds two 64-column blocks (one 32 KB
//     bulk copy: with 16 KB stages the per-stage work of the single MMA-issuing thread - barrier wait,
//     proxy fence, descriptors, commit - limited the weight stream), and the number of stages grows as
//     the token tile shrinks (5 stages of 36 KB at N = 16; tiles of more than 64 tokens go back to one
//     block per stage, 4 stages of 48 KB at N = 256);
//   * nothing at a unit boundary goes to global memory: the experts' pair offsets sit in shared memory, and
//     the gather indices of the next unit's first pass (and, for a down block, its expert's "gate/up blocks
//     done" counter) are requested while the current unit is still being copied; the routing weights of a
//     pass are fetched once per pass and handed to the epilogue's stores by shuffles.  (With these trips to
//     L2 on the critical path the pipeline drained at every unit: 147.7 -> 128.6 us at 4096 gathered tokens.)
//   * the epilogue reads the accumulators with tcgen05.ld (a lane holds ONE output feature of 16 tokens),
//     turns them through a small shared-memory tile and stores 16 bytes per lane, feature-contiguous as
//     the next GEMM and the combine want them (2-byte stores made the epilogue the slowest role from a
//     few thousand tokens on: 128.4 -> 111.7 us at 4096 gathered tokens);
//   * one elected thread issues tcgen05.mma; every mbarrier wait is bounded and reports through the
//     status words.
#pragma once
#include "mcb_tc.cuh"

namespace mcb {

constexpr int kFfnThreads = 320;            // 10 warps: TMA, MMA, 4 epilogue, 4 token-row producers
constexpr int kFfnRowsM = 128;              // weight rows per unit
constexpr int kFfnBlockK = 64;              // 128 bytes of bf16
constexpr int kFfnMaxN = 256;               // tokens per pass
constexpr int kFfnMaxStages = 12;
constexpr int kFfnMaxSub = 2;               // 64-column blocks per pipeline stage at small token tiles (one 32 KB bulk copy)
constexpr int kFfnABytes = kFfnRowsM * kFfnBlockK * 2;           // 16 KiB per 64-column block
constexpr int kFfnPipeBytes = 196 * 1024;
constexpr int kFfnMaxExperts = 1024;        // local experts (their pair offsets are kept in shared memory)
constexpr int kFfnOffBytes = (kFfnMaxExperts + 1) * 4 + 124;     // rounded to 128
constexpr int kFfnEpiBytes = 4 * 1024;      // one 16 column x 32 feature bf16 transposition tile per epilogue warp
constexpr int kFfnSmemBytes = kFfnPipeBytes + 1024 /*align*/ + 512 /*barriers*/ + kFfnOffBytes + kFfnEpiBytes;

__device__ __forceinline__ int ld_acquire_gpu_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_bf16(void* p, float v) {
  *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(v);
}

struct FfnUnit {
  int fc;          // 0 = gate/up block, 1 = down block
  int e;           // local expert
  int j;           // 128-row block inside the expert's matrix
  int row0;        // first pair row of the expert
  int rows;        // pair rows of the expert
};

// `off` = the expert offsets (a.expert_offset) in shared memory: a unit boundary must not cost a trip to L2.
__device__ __forceinline__ FfnUnit ffn_unit(const McbFfnArgs& a, const int* off, int u, int n1, int n2) {
  FfnUnit r;
  const int u1 = a.num_local_experts * n1;
  r.fc = u >= u1;
  const int v = r.fc ? u - u1 : u;
  const int per = r.fc ? n2 : n1;
  r.e = v / per;
  r.j = v - r.e * per;
  r.row0 = off[r.e];
  r.rows = off[r.e + 1] - r.row0;
  return r;
}
// First unit at or after u (stepping by the grid) whose expert has tokens; >= total when there is none.
__device__ __forceinline__ int ffn_next_unit(const McbFfnArgs& a, const int* off, int u, int total, int n1, int n2) {
  while (u < total && ffn_unit(a, off, u, n1, n2).rows <= 0) u += gridDim.x;
  return u;
}

// Call from all kFfnThreads threads of every CTA of the grid; dynamic shared memory of at least
// kFfnSmemBytes.  a.w1 is the packed interleaved gate/up matrix (E * 2I rows, H columns), a.w2 the
// packed down matrix (E * H rows, I columns): tile (row block v, column block kb) of a matrix with
// KB column blocks starts at byte (v * KB + kb) * 16384.
template <int NSUB>
__device__ __forceinline__ void ffn_device_impl(const McbFfnArgs& a, const int n_slot) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kFfnPipeBytes);
  uint64_t* full = bars;                             // [kFfnMaxStages]
  uint64_t* empty = bars + kFfnMaxStages;            // [kFfnMaxStages]
  uint64_t* tfull = bars + 2 * kFfnMaxStages;        // [2]
  uint64_t* tempty = bars + 2 * kFfnMaxStages + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kFfnMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_off = reinterpret_cast<int*>(smem + kFfnPipeBytes + 512);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kFfnMaxStages; ++s) { mbar_init(&full[s], 1 + 128); mbar_init(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int e = threadIdx.x; e <= a.num_local_experts; e += blockDim.x) s_off[e] = a.expert_offset[e];
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const Abort ab{abort_flag, a.status, a.timeout_ns};

  const int H = a.hidden, I = a.intermediate;
  const int n1 = 2 * I / kFfnRowsM, n2 = H / kFfnRowsM;
  const int total_units = a.num_local_experts * (n1 + n2);
  constexpr int nsub = NSUB;                                    // 64-column blocks per pipeline stage
  const int b_sub_bytes = n_slot * 128;                         // token tile of one 64-column block
  const int stage_bytes = nsub * (kFfnABytes + b_sub_bytes);    // [A block 0][A block 1][B block 0][B block 1]
  int stages = kFfnPipeBytes / stage_bytes;
  if (stages > kFfnMaxStages) stages = kFfnMaxStages;

  constexpr uint32_t kStageA = (uint32_t)(nsub * kFfnABytes);     // weight bytes per stage: one bulk copy

  if (warp == 0) {
    // ---------------- TMA producer: 128 weight rows x 64 columns per stage ----------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const FfnUnit un = ffn_unit(a, s_off, u, n1, n2);
        if (un.rows <= 0) continue;
        const int k_blocks = (un.fc ? I : H) / kFfnBlockK;
        const long long v = (long long)un.e * (un.fc ? n2 : n1) + un.j;       // 128-row block of the matrix
        const uint8_t* tiles = reinterpret_cast<const uint8_t*>(un.fc ? a.w2 : a.w1) + v * k_blocks * (long long)kFfnABytes;
        for (int c0 = 0; c0 < un.rows && ok; c0 += kFfnMaxN) {
          for (int kb = 0; kb < k_blocks; kb += nsub) {
            if (!(ok = mbar_wait(&empty[s], ph ^ 1u, ab, 11))) break;
            mbar_arrive_expect_tx(&full[s], kStageA);
            bulk_load(smem + s * stage_bytes, tiles + (long long)kb * kFfnABytes, kStageA, &full[s]);
            if (++s == stages) { s = 0; ph ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      int acc = 0; uint32_t acc_ph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const FfnUnit un = ffn_unit(a, s_off, u, n1, n2);
        if (un.rows <= 0) continue;
        const int k_blocks = (un.fc ? I : H) / kFfnBlockK;
        for (int c0 = 0; c0 < un.rows && ok; c0 += kFfnMaxN) {
          const int n = un.rows - c0 < kFfnMaxN ? un.rows - c0 : kFfnMaxN;
          const uint32_t idesc = umma_idesc_bf16(kFfnRowsM, (uint32_t)((n + 15) & ~15));
          if (!(ok = mbar_wait(&tempty[acc], acc_ph ^ 1u, ab, 12))) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kFfnMaxN);
          for (int kb = 0; kb < k_blocks; kb += nsub) {
            if (!(ok = mbar_wait(&full[s], ph, ab, 13))) break;
            fence_proxy_async_smem();           // the token rows were written by cp.async, not by TMA
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * stage_bytes);
#pragma unroll
            for (int sub = 0; sub < nsub; ++sub) {
              const uint64_t da = make_sw128_desc(sa + sub * kFfnABytes);
              const uint64_t db = make_sw128_desc(sa + nsub * kFfnABytes + sub * b_sub_bytes);
#pragma unroll
              for (int kk = 0; kk < kFfnBlockK / 16; ++kk)
                umma_bf16(d_tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb | sub | kk) != 0);
            }
            umma_commit(&empty[s]);
            if (++s == stages) { s = 0; ph ^= 1u; }
          }
          if (!ok) break;
          umma_commit(&tfull[acc]);
          if (++acc == 2) { acc = 0; acc_ph ^= 1u; }
        }
      }
    }
  } else if (warp < 6) {
    // ---------------- epilogue: TMEM (lane = weight row, column = token) -> global ----------------
    const int q = warp & 3;                  // TMEM lane quarter this warp may read
    // A lane holds ONE feature of 16 tokens, memory wants the features of a token side by side: the values
    // cross a small tile in shared memory ([column][feature], 64 or 32 bytes per row) and leave as 16-byte
    // stores, two (down) or one (gate/up) per 16 columns instead of sixteen or eight 2-byte ones.
    uint8_t* tile = smem + kFfnPipeBytes + 512 + kFfnOffBytes + q * 1024;
    int acc = 0; uint32_t acc_ph = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
      const FfnUnit un = ffn_unit(a, s_off, u, n1, n2);
      if (un.rows <= 0) continue;
      for (int c0 = 0; c0 < un.rows && ok; c0 += kFfnMaxN) {
        const int n = un.rows - c0 < kFfnMaxN ? un.rows - c0 : kFfnMaxN;
        if (!(ok = mbar_wait(&tfull[acc], acc_ph, ab, 14))) break;
        tc_fence_after();
        const long long prow0 = (long long)un.row0 + c0;
        {
          const int j = un.j;
          const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kFfnMaxN);
          if (!un.fc) {
            // rows alternate gate / up: lane pairs (2i, 2i + 1) hold the two halves of activation i
            const int feat = j * (kFfnRowsM / 2) + q * 16 + (lane >> 1);
            const bool odd = lane & 1;
            uint8_t* obase0 = reinterpret_cast<uint8_t*>(a.act) + (long long)(feat - (lane >> 1)) * 2;   // first feature of the warp
#pragma unroll 1
            for (int cc = 0; cc < n; cc += 16) {
              uint32_t v[16];
              tmem_ld16(t_row + cc, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                // the even lane finishes columns cc .. cc+7, the odd lane columns cc+8 .. cc+15
                const uint32_t send = odd ? v[i] : v[8 + i];
                const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
                const float g = __uint_as_float(odd ? recv : v[i]);
                const float up = __uint_as_float(odd ? v[8 + i] : recv);
                st_bf16(tile + ((odd ? 8 : 0) + i) * 32 + (lane >> 1) * 2, silu(g) * up);
              }
              __syncwarp();
              {   // 16 columns x 16 features: lane l stores half (l & 1) of column l >> 1
                const int col = cc + (lane >> 1);
                const uint4 w = *reinterpret_cast<const uint4*>(tile + (lane >> 1) * 32 + (lane & 1) * 16);
                if (col < n) st_v4(obase0 + (prow0 + col) * (long long)I * 2 + (lane & 1) * 16, w);
              }
              __syncwarp();
            }
          } else {
            const int feat = j * kFfnRowsM + q * 32 + lane;
            uint8_t* obase0 = reinterpret_cast<uint8_t*>(a.y) + (long long)(feat - lane) * 2;             // first feature of the warp
            // routing weights of the pass: lane l keeps those of columns l, l + 32, ... (one trip to L2 for the
            // whole pass instead of one per 16 columns), handed out by shuffles below
            float pp[kFfnMaxN / 32];
#pragma unroll
            for (int i = 0; i < kFfnMaxN / 32; ++i) {
              const int col = lane + 32 * i;
              pp[i] = (a.pair_prob && col < n) ? a.pair_prob[prow0 + col] : 1.0f;
            }
#pragma unroll 1
            for (int cc = 0; cc < n; cc += 16) {
              uint32_t v[16];
              tmem_ld16(t_row + cc, v);
              float mine = pp[0];
#pragma unroll
              for (int i = 1; i < kFfnMaxN / 32; ++i)
                if ((cc >> 5) == i) mine = pp[i];
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int col = cc + i;
                const float p = __shfl_sync(0xffffffffu, mine, col & 31);
                st_bf16(tile + i * 64 + lane * 2, __uint_as_float(v[i]) * p);
              }
              __syncwarp();
#pragma unroll
              for (int h = 0; h < 2; ++h) {   // 16 columns x 32 features: lane l stores quarter (l & 3) of column 8h + (l >> 2)
                const int cl = 8 * h + (lane >> 2);
                const uint4 w = *reinterpret_cast<const uint4*>(tile + cl * 64 + (lane & 3) * 16);
                if (cc + cl < n) st_v4(obase0 + (prow0 + cc + cl) * (long long)H * 2 + (lane & 3) * 16, w);
              }
              __syncwarp();
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        if (++acc == 2) { acc = 0; acc_ph ^= 1u; }
      }
      if (!un.fc && ok) {
        // This warp's quarter of the gate/up block is stored: count it for the expert's down blocks
        // (four counts per block; no barrier between the warps, so nothing can wait for a warp that
        // has given up).
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(&a.ffn_done[un.e], 1);
      }
    }
  } else {
    // ---------------- token-row producers: gather rows into the swizzled K-major B tile ----------------
    // Thread t copies 16-byte chunk (t & 7) of rows (t >> 3), (t >> 3) + 16, ...: the eight threads of a
    // row read its 128 bytes as one line, and a warp's 32 chunks fill four whole shared-memory rows.
    const int t = threadIdx.x - 6 * 32;      // 0..127
    const int chunk = t & 7, rbase = t >> 3;
    int s = 0; uint32_t ph = 0;
    bool ok = true;
    // Everything a unit needs from global memory before its first copy can be issued (the gather indices of
    // its first pass, the "gate/up blocks done" counter of a down block) is requested while the previous
    // unit is still being copied: a unit boundary must not drain the pipeline.
    int srow_n[kFfnMaxN / 16];
    int done_n = 0;
    auto prefetch = [&](const FfnUnit& un) {
      const int n = un.rows < kFfnMaxN ? un.rows : kFfnMaxN;
#pragma unroll
      for (int i = 0; i < kFfnMaxN / 16; ++i) {
        const int r = rbase + 16 * i;
        srow_n[i] = 0;
        if (r < n) srow_n[i] = un.fc ? un.row0 + r : a.pair_token[un.row0 + r];
      }
      if (un.fc && lane == 0) done_n = ld_acquire_gpu_i32(&a.ffn_done[un.e]);
    };
    int u = ffn_next_unit(a, s_off, blockIdx.x, total_units, n1, n2);
    if (u < total_units) prefetch(ffn_unit(a, s_off, u, n1, n2));
    while (u < total_units && ok) {
      const FfnUnit un = ffn_unit(a, s_off, u, n1, n2);
      const int u_next = ffn_next_unit(a, s_off, u + (int)gridDim.x, total_units, n1, n2);
      const int k_blocks = (un.fc ? I : H) / kFfnBlockK;
      if (un.fc) {
        // the activations of this expert are complete once all its gate/up blocks have been counted
        // (four epilogue warps each); one lane per producer warp polls, bounded
        if (lane == 0 && done_n < 4 * n1) {
          const uint64_t t0 = now_ns();
          while (ld_acquire_gpu_i32(&a.ffn_done[un.e]) < 4 * n1) {
            if (*ab.flag) break;
            if (ab.status && *reinterpret_cast<volatile uint32_t*>(ab.status) != 0u) { *ab.flag = 1; break; }
            if (now_ns() - t0 > ab.timeout_ns) {
              *ab.flag = 1;
              if (ab.status && atomicCAS(ab.status, 0u, (uint32_t)MCB_GEMM_ERR_TIMEOUT) == 0u) {
                ab.status[1] = 15; ab.status[2] = blockIdx.x; ab.status[3] = (uint32_t)un.e;
              }
              break;
            }
          }
        }
        __syncwarp();
      }
      const uint64_t src_row_bytes = un.fc ? (uint64_t)I * 2 : a.x_row_bytes;
      const uint8_t* src_base = reinterpret_cast<const uint8_t*>(un.fc ? a.act : a.x) + chunk * 16;
      bool prefetched = false;
      for (int c0 = 0; c0 < un.rows && ok; c0 += kFfnMaxN) {
        const int n = un.rows - c0 < kFfnMaxN ? un.rows - c0 : kFfnMaxN;
        // source rows of this thread's rows of the tile (up to 16 of them)
        int srow[kFfnMaxN / 16];
#pragma unroll
        for (int i = 0; i < kFfnMaxN / 16; ++i) {
          const int r = rbase + 16 * i;
          srow[i] = srow_n[i];
          if (c0 > 0) srow[i] = r < n ? (un.fc ? un.row0 + c0 + r : a.pair_token[un.row0 + c0 + r]) : 0;
        }
        for (int kb = 0; kb < k_blocks; kb += nsub) {
          if (!(ok = mbar_wait(&empty[s], ph ^ 1u, ab, 16))) break;
          uint8_t* sb = smem + s * stage_bytes + nsub * kFfnABytes;
          const uint8_t* g = src_base + (long long)kb * (kFfnBlockK * 2);
#pragma unroll
          for (int i = 0; i < kFfnMaxN / 16; ++i) {
            const int r = rbase + 16 * i;
            if (r < n) {
              const uint8_t* gr = g + (long long)srow[i] * (long long)src_row_bytes;
              uint8_t* dst = sb + r * 128 + ((chunk ^ (r & 7)) << 4);
#pragma unroll
              for (int sub = 0; sub < nsub; ++sub) cp_async_16(dst + sub * b_sub_bytes, gr + sub * (kFfnBlockK * 2));
            }
          }
          cp_async_arrive_noinc(&full[s]);     // arrives when this thread's copies have landed
          if (++s == stages) { s = 0; ph ^= 1u; }
          if (!prefetched && c0 + kFfnMaxN >= un.rows) {       // last pass under way: srow_n is free again
            prefetched = true;
            if (u_next < total_units) prefetch(ffn_unit(a, s_off, u_next, n1, n2));
          }
        }
      }
      u = u_next;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) __nanosleep(50000);        // let any copy still in flight land before the CTA goes away
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Token tile of this launch: the largest expert, rounded up to 16, at most kFfnMaxN per pass.  Two
// 64-column blocks per pipeline stage while the tile is small (the weight stream is then the limit and
// the per-stage work of the MMA-issuing thread must be amortised), one when it is large.
__device__ __forceinline__ void ffn_device(const McbFfnArgs& a) {
  int max_rows = *a.max_rows;
  if (max_rows < 1) max_rows = 1;
  const int n_slot = max_rows >= kFfnMaxN ? kFfnMaxN : ((max_rows + 15) & ~15);
  if (n_slot <= 128) ffn_device_impl<kFfnMaxSub>(a, n_slot);
  else ffn_device_impl<1>(a, n_slot);
}

}  // namespace mcb
