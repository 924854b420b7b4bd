// Helpers shared by the decode-step glue kernels (fl_step.cu) and the fused all-reduce + norm
// kernel (fl_comm.cu): eight bfloat16 values per 16-byte vector, a CTA-wide sum, bfloat16 rounding.
#pragma once

#include "fl_common.cuh"

namespace fl {
namespace {

constexpr int kStepThreads = 256;
constexpr int kMaxChunks = 4;  // 8 elements per thread per chunk: rows up to 8192 wide

__device__ __forceinline__ float bf16_round_f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void unpack8(const uint4& x, float (&f)[8]) {
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    f[2 * k] = bf16_lo(w[k]);
    f[2 * k + 1] = bf16_hi(w[k]);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
    w[k] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Sum over the CTA; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* s_part) {
  v = warp_sum(v);
  __syncthreads();  // s_part may still be read from a previous call
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kStepThreads / 32; ++w) total += s_part[w];
  return total;
}

}  // namespace
}  // namespace fl
