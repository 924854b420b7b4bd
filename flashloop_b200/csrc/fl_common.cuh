// Shared host/device helpers of the flashloop_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/flashloop_b200.h"

namespace fl {

constexpr int kHeadDim = FL_HEAD_DIM;
constexpr int kGroup = FL_GROUP;
constexpr int kWarp = 32;

// ---------------------------------------------------------------------------- host side

void set_error(const char* fmt, ...);

#define FL_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      ::fl::set_error(__VA_ARGS__);      \
      return FL_ERR_ARGUMENT;            \
    }                                    \
  } while (0)

#define FL_CHECK_LAUNCH(what)                                                  \
  do {                                                                         \
    cudaError_t fl_err_ = cudaGetLastError();                                  \
    if (fl_err_ != cudaSuccess) {                                              \
      ::fl::set_error("%s: %s", what, cudaGetErrorString(fl_err_));            \
      return FL_ERR_CUDA;                                                      \
    }                                                                          \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The device-side view of fl_layer (same fields, typed).
struct LayerView {
  int batch, heads, bits, tail_capacity;
  const uint8_t* k_codes[4];
  const __half* k_min[4];
  const __half* k_scale[4];
  const uint8_t* v_rows[4];  // records of FL_V_RECORD_BYTES(bits): codes, min0 min1 scale0 scale1, padding
  const int64_t* row_base[4];
  const int64_t* group_base[4];
  const int32_t* rank[2];
  const int64_t* rank_base;
  const __nv_bfloat16* tail_k[4];
  const __nv_bfloat16* tail_v[4];
  const uint8_t* tail_active[2];
  const int32_t* seq_state;
};

inline LayerView make_view(const fl_layer& l) {
  LayerView v;
  v.batch = l.batch;
  v.heads = l.heads;
  v.bits = l.bits;
  v.tail_capacity = l.tail_capacity;
  for (int s = 0; s < 4; ++s) {
    v.k_codes[s] = static_cast<const uint8_t*>(l.k_codes[s]);
    v.k_min[s] = static_cast<const __half*>(l.k_min[s]);
    v.k_scale[s] = static_cast<const __half*>(l.k_scale[s]);
    v.v_rows[s] = static_cast<const uint8_t*>(l.v_rows[s]);
    v.row_base[s] = l.row_base[s];
    v.group_base[s] = l.group_base[s];
    v.tail_k[s] = static_cast<const __nv_bfloat16*>(l.tail_k[s]);
    v.tail_v[s] = static_cast<const __nv_bfloat16*>(l.tail_v[s]);
  }
  v.rank[0] = l.rank[0];
  v.rank[1] = l.rank[1];
  v.rank_base = l.rank_base;
  v.tail_active[0] = l.tail_active[0];
  v.tail_active[1] = l.tail_active[1];
  v.seq_state = l.seq_state;
  return v;
}

int validate_layer(const fl_layer* layer, int loop, const char* who);

// ---------------------------------------------------------------------------- device side

#ifdef __CUDACC__

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ int warp_min_int(int v) { return __reduce_min_sync(0xffffffffu, v); }
__device__ __forceinline__ int warp_max_int(int v) { return __reduce_max_sync(0xffffffffu, v); }

// (a & mask) | orv in one LOP3.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
  return r;
}

__device__ __forceinline__ __half2 as_half2(uint32_t bits) {
  return *reinterpret_cast<__half2*>(&bits);
}
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// Eight 4-bit codes of one 32-bit word -> four half2 of exact integers, pair k holding the
// codes at nibble positions k and k+4.  0x6400 is 1024.0 in float16: or-ing a 4-bit code into
// its low mantissa bits gives 1024 + code (or 1024 + 16*code for a code at bits 4..7).
__device__ __forceinline__ void unpack4(uint32_t w, __half2 (&h)[4]) {
  const uint32_t kMagic = 0x64006400u;
  const __half2 k1024 = __floats2half2_rn(1024.f, 1024.f);
  const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 k64n = __floats2half2_rn(-64.f, -64.f);
  const uint32_t w8 = w >> 8;
  h[0] = __hsub2(as_half2(and_or(w, 0x000F000Fu, kMagic)), k1024);
  h[1] = __hfma2(as_half2(and_or(w, 0x00F000F0u, kMagic)), k16th, k64n);
  h[2] = __hsub2(as_half2(and_or(w8, 0x000F000Fu, kMagic)), k1024);
  h[3] = __hfma2(as_half2(and_or(w8, 0x00F000F0u, kMagic)), k16th, k64n);
}

// Sixteen 2-bit codes of one 32-bit word -> eight half2, pair k holding positions k and k+8.
__device__ __forceinline__ void unpack2(uint32_t w, __half2 (&h)[8]) {
  const uint32_t kMagic = 0x64006400u;
  const __half2 k1024 = __floats2half2_rn(1024.f, 1024.f);
  const __half2 k4th = __floats2half2_rn(0.25f, 0.25f);
  const __half2 k256n = __floats2half2_rn(-256.f, -256.f);
  const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 k64n = __floats2half2_rn(-64.f, -64.f);
  const __half2 k64th = __floats2half2_rn(0.015625f, 0.015625f);
  const __half2 k16n = __floats2half2_rn(-16.f, -16.f);
  const uint32_t w8 = w >> 8;
  h[0] = __hsub2(as_half2(and_or(w, 0x00030003u, kMagic)), k1024);
  h[1] = __hfma2(as_half2(and_or(w, 0x000C000Cu, kMagic)), k4th, k256n);
  h[2] = __hfma2(as_half2(and_or(w, 0x00300030u, kMagic)), k16th, k64n);
  h[3] = __hfma2(as_half2(and_or(w, 0x00C000C0u, kMagic)), k64th, k16n);
  h[4] = __hsub2(as_half2(and_or(w8, 0x00030003u, kMagic)), k1024);
  h[5] = __hfma2(as_half2(and_or(w8, 0x000C000Cu, kMagic)), k4th, k256n);
  h[6] = __hfma2(as_half2(and_or(w8, 0x00300030u, kMagic)), k16th, k64n);
  h[7] = __hfma2(as_half2(and_or(w8, 0x00C000C0u, kMagic)), k64th, k16n);
}

__device__ __forceinline__ uint4 ldg128(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ uint2 ldg64(const void* p) {
  return __ldg(reinterpret_cast<const uint2*>(p));
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p) {
  return __half2float(*p);
}
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) {
  return *p;
}

// The reference quantiser (flashloop/packing.py:35-46) in float32 with IEEE operations that
// the compiler may not contract or approximate.
__device__ __forceinline__ float quant_scale(float minimum, float maximum, float levels) {
  const float span = __fsub_rn(maximum, minimum);
  return span > 0.f ? __fdiv_rn(span, levels) : 1.f;
}
// The reciprocal the quantiser multiplies by on its fast path; 0 where the reciprocal would
// lose bits (scale far outside the range K/V values live in), which sends every element through
// the division.
__device__ __forceinline__ float quant_inverse(float scale) {
  return (scale > 1e-30f && scale < 1e30f) ? __frcp_rn(scale) : 0.f;
}
// The reference divides: q = (x - min) / scale, IEEE, then rounds half to even.  (x - min) * (1 /
// scale) is within 3e-6 of that quotient for codes up to 15, so unless it sits within 1e-4 of a
// rounding boundary both give the same code; at a boundary the division decides.  Same bits as
// the reference at a fraction of the arithmetic.
__device__ __forceinline__ uint32_t quant_code(float x, float minimum, float scale, float inverse, float levels) {
  const float d = __fsub_rn(x, minimum);
  const float q = __fmul_rn(d, inverse);
  float r = rintf(q);
  if (!(fabsf(fabsf(q - r) - 0.5f) > 1e-4f) || inverse == 0.f) r = rintf(__fdiv_rn(d, scale));
  r = fminf(fmaxf(r, 0.f), levels);
  return static_cast<uint32_t>(r);
}
// Eight codes at once, code k in bits [BITS*k, BITS*k + BITS): the fast path of quant_code for all
// eight and one test whether any of them sits at a rounding boundary, in which case (about once in
// a thousand groups) all eight go through the division.  Same codes as eight quant_code calls.
template <int BITS>
__device__ __forceinline__ uint32_t quant_codes8(const float (&x)[8], float minimum, float scale, float inverse,
                                                 float levels) {
  float r[8];
  bool exact = inverse == 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float q = __fmul_rn(__fsub_rn(x[k], minimum), inverse);
    r[k] = rintf(q);
    exact |= !(fabsf(fabsf(q - r[k]) - 0.5f) > 1e-4f);
  }
  if (exact) {
#pragma unroll
    for (int k = 0; k < 8; ++k) r[k] = rintf(__fdiv_rn(__fsub_rn(x[k], minimum), scale));
  }
  uint32_t packed = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) packed |= static_cast<uint32_t>(fminf(fmaxf(r[k], 0.f), levels)) << (BITS * k);
  return packed;
}
// code * scale + minimum in float32 (two roundings, as torch computes it), then bf16 RNE.
__device__ __forceinline__ float dequant_f32(uint32_t code, __half scale, __half minimum) {
  return __fadd_rn(__fmul_rn(static_cast<float>(code), __half2float(scale)),
                   __half2float(minimum));
}

#endif  // __CUDACC__

}  // namespace fl
