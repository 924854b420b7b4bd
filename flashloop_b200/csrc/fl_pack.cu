// Quantise + pack kernels (row layout and KIVI word layout), decode and layout conversion.
//
// Arithmetic follows the reference's CPU quantiser exactly (flashloop/packing.py:35-46 ==
// flashloop/kivi_backend.py:272-283): float32 min/max, span/levels by IEEE division,
// (x - min)/scale by IEEE subtraction and division, round-half-to-even, clamp; float16
// metadata is the RNE rounding of the float32 values the codes were computed with.
#include "fl_common.cuh"

namespace fl {
namespace {

// ------------------------------------------------------------------------------- K: per channel
// One CTA of 128 threads per (64-token group, bh); thread c owns channel c.
template <typename T, int BITS, bool KIVI>
__global__ void __launch_bounds__(128)
pack_k_kernel(const T* __restrict__ values, int64_t tokens, void* __restrict__ out_codes,
              __half* __restrict__ minimum, __half* __restrict__ scale) {
  constexpr float kLevels = float((1 << BITS) - 1);
  constexpr int kRowBytes = 16 * BITS;
  const int c = threadIdx.x;
  const int64_t g = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int64_t t0 = g * kGroup;
  const int cnt = (tokens - t0) < kGroup ? static_cast<int>(tokens - t0) : kGroup;
  const int64_t groups = (tokens + kGroup - 1) / kGroup;
  // The group's rows are staged in shared memory with 16-byte loads (one read of the input),
  // then every thread walks its own channel.
  __shared__ __align__(16) T tile_in[kGroup][kHeadDim];
  {
    const T* block = values + (bh * tokens + t0) * kHeadDim;
    constexpr int kPer16 = 16 / sizeof(T);               // elements per 16-byte piece
    constexpr int kRowPieces = kHeadDim / kPer16;
    if ((reinterpret_cast<uintptr_t>(block) & 15u) == 0) {
      for (int idx = c; idx < cnt * kRowPieces; idx += 128) {
        const uint4 v = ldg128(block + static_cast<int64_t>(idx) * kPer16);
        *reinterpret_cast<uint4*>(&tile_in[0][0] + static_cast<int64_t>(idx) * kPer16) = v;
      }
    } else {
      for (int i = 0; i < cnt; ++i) tile_in[i][c] = block[static_cast<int64_t>(i) * kHeadDim + c];
    }
  }
  __syncthreads();
  const T* src = &tile_in[0][c];

  float mn = INFINITY, mx = -INFINITY;
  for (int i = 0; i < cnt; ++i) {
    const float x = load_as_float(src + static_cast<int64_t>(i) * kHeadDim);
    mn = fminf(mn, x);
    mx = fmaxf(mx, x);
  }
  const float sc = quant_scale(mn, mx, kLevels);
  const float inv = quant_inverse(sc);
  minimum[(bh * groups + g) * kHeadDim + c] = __float2half_rn(mn);
  scale[(bh * groups + g) * kHeadDim + c] = __float2half_rn(sc);

  if constexpr (KIVI) {
    static_assert(BITS == 4, "the KIVI word layout is 4-bit");
    int32_t* payload = static_cast<int32_t*>(out_codes);
    const int64_t word_rows = (tokens + 7) / 8;
    for (int w = 0; w * 8 < cnt; ++w) {
      uint32_t word = 0;
      if (w * 8 + 8 <= cnt) {
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = load_as_float(src + static_cast<int64_t>(w * 8 + j) * kHeadDim);
        word = quant_codes8<4>(x, mn, sc, inv, kLevels);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = w * 8 + j;
          if (i < cnt) {
            const float x = load_as_float(src + static_cast<int64_t>(i) * kHeadDim);
            word |= quant_code(x, mn, sc, inv, kLevels) << (4 * j);
          }
        }
      }
      payload[(bh * word_rows + t0 / 8 + w) * kHeadDim + c] = static_cast<int32_t>(word);
    }
  } else {
    __shared__ uint8_t tile[kGroup][kHeadDim + 4];
    for (int i = 0; i < cnt; ++i) {
      const float x = load_as_float(src + static_cast<int64_t>(i) * kHeadDim);
      tile[i][c] = static_cast<uint8_t>(quant_code(x, mn, sc, inv, kLevels));
    }
    __syncthreads();    constexpr int kRowWords = kRowBytes / 4;
    constexpr int kPerWord = 32 / BITS;
    uint32_t* dst =
        reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(out_codes) + (bh * tokens + t0) * kRowBytes);
    for (int idx = c; idx < cnt * kRowWords; idx += 128) {
      const int row = idx / kRowWords;
      const int wr = idx % kRowWords;
      uint32_t word = 0;
#pragma unroll
      for (int k = 0; k < kPerWord; ++k) word |= uint32_t(tile[row][wr * kPerWord + k]) << (BITS * k);
      dst[idx] = word;
    }
  }
}

// ------------------------------------------------------------------------------- V: per token
// Half a warp per token: lane l of the half owns channels 8l .. 8l+7 (one 16-byte load of
// bfloat16), so a 64-channel group is eight lanes (three shuffle steps for its minimum and maximum,
// one division for its scale) and a lane's eight codes are one 32-bit word of the row.  A warp takes
// eight tokens, two at a time, their loads issued together.  The KIVI word layout is token-minor
// ([bh][16 words][tokens]): there the CTA's 32 consecutive tokens meet in shared memory and leave
// as 128-byte runs of one word row, instead of one 4-byte store per word.
constexpr int kVWarps = 4;
constexpr int kVPairs = 4;                       // pairs of tokens per warp
constexpr int kVPerCta = kVWarps * kVPairs * 2;  // 32 tokens

template <typename T>
__device__ __forceinline__ void load_eight(const T* src, bool vector_ok, float (&x)[8]) {
  if (!vector_ok) {
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = load_as_float(src + k);
  } else if constexpr (sizeof(T) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = load_as_float(h + k);
  } else {
    const float4 lo = *reinterpret_cast<const float4*>(src);
    const float4 hi = *reinterpret_cast<const float4*>(src + 4);
    x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
    x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
  }
}

template <typename T, int BITS, bool KIVI>
__global__ void __launch_bounds__(kVWarps * 32)
pack_v_kernel(const T* __restrict__ values, int64_t tokens, int64_t total_tokens,
              void* __restrict__ out_codes, __half* __restrict__ minimum,
              __half* __restrict__ scale, int64_t meta_stride) {
  constexpr float kLevels = float((1 << BITS) - 1);
  constexpr int kRowBytes = 16 * BITS;
  __shared__ uint32_t s_words[KIVI ? 16 : 1][KIVI ? kVPerCta + 1 : 1];
  __shared__ __half s_meta[KIVI ? 4 : 1][KIVI ? kVPerCta : 1];  // min of group 0, 1, scale of group 0, 1
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, sub = lane & 15, g = sub >> 3;
  const int64_t cta_first = static_cast<int64_t>(blockIdx.x) * kVPerCta;
  const bool vector_ok = (reinterpret_cast<uintptr_t>(values) & 15u) == 0;
  float xs[kVPairs][8];
#pragma unroll
  for (int j = 0; j < kVPairs; ++j) {
    const int64_t want = cta_first + (warp * kVPairs + j) * 2 + half;
    const int64_t wg = want < total_tokens ? want : total_tokens - 1;
    load_eight(values + wg * kHeadDim + 8 * sub, vector_ok, xs[j]);
  }
#pragma unroll
  for (int j = 0; j < kVPairs; ++j) {
    const int slot = (warp * kVPairs + j) * 2 + half;
    const int64_t wg = cta_first + slot;
    const bool on = wg < total_tokens;  // the shuffles below are for the whole warp
    const float (&x)[8] = xs[j];
    float mn = fminf(fminf(fminf(x[0], x[1]), fminf(x[2], x[3])), fminf(fminf(x[4], x[5]), fminf(x[6], x[7])));
    float mx = fmaxf(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])), fmaxf(fmaxf(x[4], x[5]), fmaxf(x[6], x[7])));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    const float sc = quant_scale(mn, mx, kLevels);
    const float inv = quant_inverse(sc);
    const uint32_t packed = quant_codes8<BITS>(x, mn, sc, inv, kLevels);
    if (!on) continue;
    if constexpr (KIVI) {
      static_assert(BITS == 4, "the KIVI word layout is 4-bit");
      s_words[sub][slot] = packed;
      if ((sub & 7) == 0) {
        s_meta[g][slot] = __float2half_rn(mn);
        s_meta[2 + g][slot] = __float2half_rn(sc);
      }
    } else {
      uint8_t* row = static_cast<uint8_t*>(out_codes) + wg * kRowBytes;
      if constexpr (BITS == 4) {
        reinterpret_cast<uint32_t*>(row)[sub] = packed;
      } else {
        reinterpret_cast<uint16_t*>(row)[sub] = static_cast<uint16_t>(packed);
      }
      if ((sub & 7) == 0) {
        minimum[wg * meta_stride + g] = __float2half_rn(mn);
        scale[wg * meta_stride + g] = __float2half_rn(sc);
      }
    }
  }
  if constexpr (KIVI) {
    __syncthreads();
    // word row r of the CTA's tokens: consecutive tokens of one (b,h) are consecutive words
    for (int idx = threadIdx.x; idx < 16 * kVPerCta; idx += kVWarps * 32) {
      const int r = idx / kVPerCta, slot = idx % kVPerCta;
      const int64_t wg = cta_first + slot;
      if (wg < total_tokens) {
        const int64_t bh = wg / tokens, t = wg % tokens;
        static_cast<int32_t*>(out_codes)[(bh * 16 + r) * tokens + t] = static_cast<int32_t>(s_words[r][slot]);
      }
    }
    for (int idx = threadIdx.x; idx < 4 * kVPerCta; idx += kVWarps * 32) {
      const int which = idx / kVPerCta, slot = idx % kVPerCta;
      const int64_t wg = cta_first + slot;
      if (wg < total_tokens) {
        const int64_t bh = wg / tokens, t = wg % tokens;
        (which < 2 ? minimum : scale)[(bh * 2 + (which & 1)) * tokens + t] = s_meta[which][slot];
      }
    }
  }
}

// ------------------------------------------------------------------------------- decode
template <int BITS>
__global__ void decode_rows_kernel(const uint32_t* __restrict__ codes,
                                   const __half* __restrict__ minimum,
                                   const __half* __restrict__ scale, int per_channel,
                                   int64_t meta_stride, int64_t tokens, int64_t total_words,
                                   __nv_bfloat16* __restrict__ out) {
  constexpr int kRowWords = 16 * BITS / 4;
  constexpr int kPerWord = 32 / BITS;
  const int64_t groups = (tokens + kGroup - 1) / kGroup;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total_words;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = idx / kRowWords;
    const int wr = static_cast<int>(idx % kRowWords);
    const int64_t bh = row / tokens;
    const int64_t t = row % tokens;
    const uint32_t word = codes[idx];
#pragma unroll
    for (int k = 0; k < kPerWord; ++k) {
      const int c = wr * kPerWord + k;
      const uint32_t code = (word >> (BITS * k)) & ((1u << BITS) - 1u);
      const int64_t m = per_channel ? (bh * groups + t / kGroup) * kHeadDim + c
                                    : row * meta_stride + c / kGroup;
      out[row * kHeadDim + c] = __float2bfloat16_rn(dequant_f32(code, scale[m], minimum[m]));
    }
  }
}

// ------------------------------------------------------------------------------- KIVI -> rows
__global__ void kivi_to_rows_k_kernel(const uint32_t* __restrict__ payload, int64_t tokens,
                                      int64_t total_words, uint32_t* __restrict__ codes) {
  const int64_t word_rows = (tokens + 7) / 8;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total_words;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = idx / 16;
    const int wr = static_cast<int>(idx % 16);
    const int64_t bh = row / tokens;
    const int64_t t = row % tokens;
    const uint32_t* src = payload + (bh * word_rows + t / 8) * kHeadDim + wr * 8;
    const int shift = 4 * static_cast<int>(t % 8);
    uint32_t word = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) word |= ((src[k] >> shift) & 0xFu) << (4 * k);
    codes[idx] = word;
  }
}

__global__ void kivi_to_rows_v_kernel(const uint32_t* __restrict__ payload,
                                      const __half* __restrict__ minimum,
                                      const __half* __restrict__ scale, int64_t tokens,
                                      int64_t total_words, uint32_t* __restrict__ codes,
                                      __half* __restrict__ out_min, __half* __restrict__ out_scale,
                                      int64_t meta_stride) {
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total_words;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = idx / 16;
    const int wr = static_cast<int>(idx % 16);
    const int64_t bh = row / tokens;
    const int64_t t = row % tokens;
    codes[idx] = payload[(bh * 16 + wr) * tokens + t];
    if (wr < 2) {
      out_min[row * meta_stride + wr] = minimum[(bh * 2 + wr) * tokens + t];
      out_scale[row * meta_stride + wr] = scale[(bh * 2 + wr) * tokens + t];
    }
  }
}

template <int BITS, bool KIVI>
int launch_pack_k(const void* values, int32_t dtype, int64_t bh, int64_t tokens, void* codes,
                  void* minimum, void* scale, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>((tokens + kGroup - 1) / kGroup), static_cast<unsigned>(bh));
  __half* mn = static_cast<__half*>(minimum);
  __half* sc = static_cast<__half*>(scale);
  switch (dtype) {
    case FL_DTYPE_BF16:
      pack_k_kernel<__nv_bfloat16, BITS, KIVI><<<grid, 128, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(values), tokens, codes, mn, sc);
      break;
    case FL_DTYPE_F16:
      pack_k_kernel<__half, BITS, KIVI><<<grid, 128, 0, stream>>>(
          static_cast<const __half*>(values), tokens, codes, mn, sc);
      break;
    case FL_DTYPE_F32:
      pack_k_kernel<float, BITS, KIVI><<<grid, 128, 0, stream>>>(
          static_cast<const float*>(values), tokens, codes, mn, sc);
      break;
    default:
      set_error("pack K: unknown dtype %d", dtype);
      return FL_ERR_ARGUMENT;
  }
  FL_CHECK_LAUNCH("pack K");
  return FL_OK;
}

template <int BITS, bool KIVI>
int launch_pack_v(const void* values, int32_t dtype, int64_t bh, int64_t tokens, void* codes,
                  void* minimum, void* scale, int64_t meta_stride, cudaStream_t stream) {
  const int64_t total = bh * tokens;
  const int64_t per_cta = kVPerCta;
  const unsigned grid = static_cast<unsigned>((total + per_cta - 1) / per_cta);
  __half* mn = static_cast<__half*>(minimum);
  __half* sc = static_cast<__half*>(scale);
  switch (dtype) {
    case FL_DTYPE_BF16:
      pack_v_kernel<__nv_bfloat16, BITS, KIVI><<<grid, 128, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(values), tokens, total, codes, mn, sc, meta_stride);
      break;
    case FL_DTYPE_F16:
      pack_v_kernel<__half, BITS, KIVI><<<grid, 128, 0, stream>>>(
          static_cast<const __half*>(values), tokens, total, codes, mn, sc, meta_stride);
      break;
    case FL_DTYPE_F32:
      pack_v_kernel<float, BITS, KIVI><<<grid, 128, 0, stream>>>(
          static_cast<const float*>(values), tokens, total, codes, mn, sc, meta_stride);
      break;
    default:
      set_error("pack V: unknown dtype %d", dtype);
      return FL_ERR_ARGUMENT;
  }
  FL_CHECK_LAUNCH("pack V");
  return FL_OK;
}

int check_pack_args(const char* who, const void* values, int64_t bh, int64_t tokens,
                    const void* codes, const void* minimum, const void* scale) {
  FL_REQUIRE(values && codes && minimum && scale, "%s: null pointer", who);
  FL_REQUIRE(bh > 0 && tokens > 0, "%s: batch_heads and tokens must be positive", who);
  FL_REQUIRE(bh <= 65535 * 1024LL && (tokens + kGroup - 1) / kGroup < (1LL << 31),
             "%s: problem too large for one launch", who);
  return FL_OK;
}

unsigned flat_grid(int64_t items) {
  const int64_t blocks = (items + 255) / 256;
  return static_cast<unsigned>(blocks < 148LL * 32 ? blocks : 148LL * 32);
}

}  // namespace
}  // namespace fl

using namespace fl;

extern "C" int fl_pack_k_rows(const void* values, int32_t dtype, int64_t batch_heads,
                              int64_t tokens, int32_t bits, void* codes, void* minimum,
                              void* scale, fl_cuda_stream stream) {
  if (int rc = check_pack_args("fl_pack_k_rows", values, batch_heads, tokens, codes, minimum, scale)) return rc;
  FL_REQUIRE(batch_heads <= 65535, "fl_pack_k_rows: batch_heads above 65535");
  FL_REQUIRE(aligned16(codes), "fl_pack_k_rows: codes must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bits == 4) return launch_pack_k<4, false>(values, dtype, batch_heads, tokens, codes, minimum, scale, s);
  if (bits == 2) return launch_pack_k<2, false>(values, dtype, batch_heads, tokens, codes, minimum, scale, s);
  set_error("fl_pack_k_rows: bits must be 4 or 2, got %d", bits);
  return FL_ERR_ARGUMENT;
}

extern "C" int fl_pack_v_rows(const void* values, int32_t dtype, int64_t batch_heads,
                              int64_t tokens, int32_t bits, void* codes, void* minimum,
                              void* scale, int64_t meta_stride, fl_cuda_stream stream) {
  if (int rc = check_pack_args("fl_pack_v_rows", values, batch_heads, tokens, codes, minimum, scale)) return rc;
  FL_REQUIRE(meta_stride >= 2, "fl_pack_v_rows: meta_stride must be >= 2");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bits == 4) return launch_pack_v<4, false>(values, dtype, batch_heads, tokens, codes, minimum, scale, meta_stride, s);
  if (bits == 2) return launch_pack_v<2, false>(values, dtype, batch_heads, tokens, codes, minimum, scale, meta_stride, s);
  set_error("fl_pack_v_rows: bits must be 4 or 2, got %d", bits);
  return FL_ERR_ARGUMENT;
}

extern "C" int fl_pack_kivi_k(const void* values, int32_t dtype, int64_t batch_heads,
                              int64_t tokens, void* payload, void* minimum, void* scale,
                              fl_cuda_stream stream) {
  if (int rc = check_pack_args("fl_pack_kivi_k", values, batch_heads, tokens, payload, minimum, scale)) return rc;
  FL_REQUIRE(batch_heads <= 65535, "fl_pack_kivi_k: batch_heads above 65535");
  return launch_pack_k<4, true>(values, dtype, batch_heads, tokens, payload, minimum, scale,
                                static_cast<cudaStream_t>(stream));
}

extern "C" int fl_pack_kivi_v(const void* values, int32_t dtype, int64_t batch_heads,
                              int64_t tokens, void* payload, void* minimum, void* scale,
                              fl_cuda_stream stream) {
  if (int rc = check_pack_args("fl_pack_kivi_v", values, batch_heads, tokens, payload, minimum, scale)) return rc;
  return launch_pack_v<4, true>(values, dtype, batch_heads, tokens, payload, minimum, scale, 0,
                                static_cast<cudaStream_t>(stream));
}

extern "C" int fl_decode_rows(const void* codes, const void* minimum, const void* scale,
                              int32_t per_channel, int64_t meta_stride, int64_t batch_heads,
                              int64_t tokens, int32_t bits, void* out, fl_cuda_stream stream) {
  if (int rc = check_pack_args("fl_decode_rows", codes, batch_heads, tokens, out, minimum, scale)) return rc;
  FL_REQUIRE(bits == 4 || bits == 2, "fl_decode_rows: bits must be 4 or 2");
  FL_REQUIRE(per_channel || meta_stride >= 2, "fl_decode_rows: meta_stride must be >= 2 for V");
  const int64_t words = batch_heads * tokens * (16 * bits / 4);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bits == 4) {
    decode_rows_kernel<4><<<flat_grid(words), 256, 0, s>>>(
        static_cast<const uint32_t*>(codes), static_cast<const __half*>(minimum),
        static_cast<const __half*>(scale), per_channel, meta_stride, tokens, words,
        static_cast<__nv_bfloat16*>(out));
  } else {
    decode_rows_kernel<2><<<flat_grid(words), 256, 0, s>>>(
        static_cast<const uint32_t*>(codes), static_cast<const __half*>(minimum),
        static_cast<const __half*>(scale), per_channel, meta_stride, tokens, words,
        static_cast<__nv_bfloat16*>(out));
  }
  FL_CHECK_LAUNCH("fl_decode_rows");
  return FL_OK;
}

extern "C" int fl_kivi_to_rows_k(const void* payload, int64_t batch_heads, int64_t tokens,
                                 void* codes, fl_cuda_stream stream) {
  FL_REQUIRE(payload && codes && batch_heads > 0 && tokens > 0, "fl_kivi_to_rows_k: bad argument");
  const int64_t words = batch_heads * tokens * 16;
  kivi_to_rows_k_kernel<<<flat_grid(words), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(payload), tokens, words, static_cast<uint32_t*>(codes));
  FL_CHECK_LAUNCH("fl_kivi_to_rows_k");
  return FL_OK;
}

extern "C" int fl_kivi_to_rows_v(const void* payload, const void* minimum, const void* scale,
                                 int64_t batch_heads, int64_t tokens, void* codes,
                                 void* out_minimum, void* out_scale, int64_t meta_stride,
                                 fl_cuda_stream stream) {
  FL_REQUIRE(payload && minimum && scale && codes && out_minimum && out_scale && batch_heads > 0 &&
                 tokens > 0 && meta_stride >= 2,
             "fl_kivi_to_rows_v: bad argument");
  const int64_t words = batch_heads * tokens * 16;
  kivi_to_rows_v_kernel<<<flat_grid(words), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(payload), static_cast<const __half*>(minimum),
      static_cast<const __half*>(scale), tokens, words, static_cast<uint32_t*>(codes),
      static_cast<__half*>(out_minimum), static_cast<__half*>(out_scale), meta_stride);
  FL_CHECK_LAUNCH("fl_kivi_to_rows_v");
  return FL_OK;
}
