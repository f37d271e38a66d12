// 1 x 128 block-scaled e4m3 quantisation of bf16 rows (scale = amax / 448 per 128 values, 1 for
// an all-zero block; saturating round-to-nearest-even convert), shared by the all-to-all dispatch
// and the dense dispatch.
#pragma once
#include <cuda_fp8.h>

#include "mcb_ptx.cuh"

namespace mcb {

// Quantise 8 bf16 values (one 16-byte pack) to 8 e4m3 bytes: saturating RNE of v / scale.
__device__ __forceinline__ uint2 quant_pack_e4m3(uint4 v, float scale) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint16_t q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // true division (not a reciprocal multiply) so results match an fp32 reference bit for bit
    const float2 f = make_float2(__fdiv_rn(bf16_lo(w[i]), scale), __fdiv_rn(bf16_hi(w[i]), scale));
    q[i] = (uint16_t)__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
  }
  return make_uint2((uint32_t)q[0] | ((uint32_t)q[1] << 16), (uint32_t)q[2] | ((uint32_t)q[3] << 16));
}

__device__ __forceinline__ float pack_absmax(uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) m = fmaxf(m, fmaxf(fabsf(bf16_lo(w[i])), fabsf(bf16_hi(w[i]))));
  return m;
}

// Scale of a 128-value block from its largest magnitude.
__device__ __forceinline__ float e4m3_scale(float amax) { return amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f; }

// Largest magnitude of the 128-value block that starts at `block` (16 packs of 16 bytes), read by
// ONE thread (for the packet mode, where the threads that share a block are not neighbours).
__device__ __forceinline__ float block_absmax_serial(const uint8_t* block) {
  float m = 0.f;
#pragma unroll 4
  for (int p = 0; p < 16; ++p) m = fmaxf(m, pack_absmax(ld_v4(block + p * 16)));
  return m;
}

}  // namespace mcb
