// Decode append and the 64-token rollover, entirely on the device.
//
// Replaces CrossLoopKVLayer.append_decode_token / _roll_one_group and the block re-encode it
// triggers (flashloop/cache.py:1758-1838 -> from_prefill -> _encode_initial_prefix,
// cache.py:1008-1074): about sixty small Torch launches, eight Triton packs and a
// re-concatenation of every stream per rollover in the reference; three launches per decoded
// token here, two of which return at once unless a sequence's tail has reached 128 tokens.
//
//   append_tail_kernel   writes the token's 4 K + 4 V rows into the BF16 tail rings
//   rollover_kernel      for sequences whose tail is full: the residual chain of the oldest
//                        64 tail tokens (anchor, delta-2, and delta-3/4 of the retained rows,
//                        every subtraction/addition a bfloat16 operation as in the reference)
//                        quantised and written as one new 64-row block of every stream
//   advance_state_kernel per-sequence bookkeeping (seq_state, rank maps, tail_active)
//
// Sequence state is read from device memory, so the three launches are the same for every
// decoded token and can be captured in a CUDA graph.
#include "fl_common.cuh"

namespace fl {
namespace {

struct AppendParams {
  LayerView L;
  uint8_t* k_codes[4];
  __half* k_min[4];
  __half* k_scale[4];
  uint8_t* v_rows[4];
  int32_t* rank[2];
  __nv_bfloat16* tail_k[4];
  __nv_bfloat16* tail_v[4];
  uint8_t* tail_active[2];
  int32_t* seq_state;
  const __nv_bfloat16* keys[4];
  const __nv_bfloat16* values[4];
};

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ------------------------------------------------------------------------------ append
__global__ void __launch_bounds__(128) append_tail_kernel(const AppendParams p) {
  const int64_t bh = blockIdx.x;
  const int b = static_cast<int>(bh / p.L.heads);
  const int32_t* st = p.seq_state + b * FL_STATE_WORDS;
  const int cap = p.L.tail_capacity;
  const int slot = (st[FL_STATE_TAIL_START] + st[FL_STATE_TAIL_LEN]) % cap;
  const int c = threadIdx.x;
  const int64_t dst = (bh * cap + slot) * kHeadDim + c;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    p.tail_k[r][dst] = p.keys[r][bh * kHeadDim + c];
    p.tail_v[r][dst] = p.values[r][bh * kHeadDim + c];
  }
  if (c < 2 && bh % p.L.heads == 0) p.tail_active[c][static_cast<int64_t>(b) * cap + slot] = 1;
}

// ------------------------------------------------------------------------------ rollover
// grid (batch*heads, 2): y == 0 encodes K (thread = channel), y == 1 encodes V (warp = token).
template <int BITS>
__global__ void __launch_bounds__(128) rollover_kernel(const AppendParams p) {
  constexpr float kLevels = float((1 << BITS) - 1);
  constexpr int kRowBytes = 16 * BITS;
  constexpr int kRowWords = kRowBytes / 4;
  constexpr int kPerWord = 32 / BITS;
  const int64_t bh = blockIdx.x;
  const int b = static_cast<int>(bh / p.L.heads);
  const int32_t* st = p.seq_state + b * FL_STATE_WORDS;
  const int cap = p.L.tail_capacity;
  if (st[FL_STATE_TAIL_LEN] + 1 < 2 * kGroup) return;  // the tail (with this step's token) is not full
  const int quant = st[FL_STATE_QUANT_TOKENS];
  const int start = st[FL_STATE_TAIL_START];
  const int row0[4] = {quant, quant, st[FL_STATE_ROWS2], st[FL_STATE_ROWS3]};

  __shared__ uint8_t s_active[2][kGroup];
  __shared__ int s_rank[2][kGroup];   // compact index of token i in streams 2 / 3, -1 if absent
  __shared__ int s_count[2];
  const int tid = threadIdx.x;
  if (tid < kGroup) {
    const int slot = (start + tid) % cap;
    s_active[0][tid] = p.tail_active[0][static_cast<int64_t>(b) * cap + slot];
    s_active[1][tid] = p.tail_active[1][static_cast<int64_t>(b) * cap + slot];
  }
  __syncthreads();
  if (tid < 2) {
    int n = 0;
    for (int i = 0; i < kGroup; ++i) {
      s_rank[tid][i] = s_active[tid][i] ? n : -1;
      n += s_active[tid][i] ? 1 : 0;
    }
    s_count[tid] = n;
  }
  __syncthreads();

  if (blockIdx.y == 0) {
    // ---------------- K: per channel over the block's tokens; thread c owns channel c
    __shared__ __nv_bfloat16 s_recon[kGroup][kHeadDim];
    __shared__ uint8_t s_tile[kGroup][kHeadDim + 4];
    const int c = tid;
#pragma unroll 1
    for (int s = 0; s < 4; ++s) {
      const int rows = s < 2 ? kGroup : s_count[s - 2];
      if (rows == 0) continue;  // uniform over the CTA
      const __nv_bfloat16* src = p.tail_k[s] + bh * cap * kHeadDim + c;
      float mn = INFINITY, mx = -INFINITY;
      for (int i = 0; i < kGroup; ++i) {
        if (s >= 2 && !s_active[s - 2][i]) continue;
        float x = __bfloat162float(src[((start + i) % cap) * kHeadDim]);
        if (s > 0) x = bf16_round(x - __bfloat162float(s_recon[i][c]));
        mn = fminf(mn, x);
        mx = fmaxf(mx, x);
      }
      const float sc = quant_scale(mn, mx, kLevels);
      const float inv = quant_inverse(sc);
      const __half mn16 = __float2half_rn(mn), sc16 = __float2half_rn(sc);
      const int64_t group = p.L.group_base[s][bh] + row0[s] / kGroup;
      p.k_min[s][group * kHeadDim + c] = mn16;
      p.k_scale[s][group * kHeadDim + c] = sc16;
      for (int i = 0; i < kGroup; ++i) {
        if (s >= 2 && !s_active[s - 2][i]) continue;
        float x = __bfloat162float(src[((start + i) % cap) * kHeadDim]);
        const float base = s > 0 ? __bfloat162float(s_recon[i][c]) : 0.f;
        if (s > 0) x = bf16_round(x - base);
        const uint32_t code = quant_code(x, mn, sc, inv, kLevels);
        const int j = s < 2 ? i : s_rank[s - 2][i];
        s_tile[j][c] = static_cast<uint8_t>(code);
        const float dec = bf16_round(dequant_f32(code, sc16, mn16));
        s_recon[i][c] = __float2bfloat16_rn(s > 0 ? base + dec : dec);
      }
      __syncthreads();
      uint32_t* dst = reinterpret_cast<uint32_t*>(p.k_codes[s] + (p.L.row_base[s][bh] + row0[s]) * kRowBytes);
      for (int idx = tid; idx < rows * kRowWords; idx += 128) {
        const int row = idx / kRowWords, wr = idx % kRowWords;
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < kPerWord; ++k) word |= uint32_t(s_tile[row][wr * kPerWord + k]) << (BITS * k);
        dst[idx] = word;
      }
      __syncthreads();
    }
  } else {
    // ---------------- V: per token over 64-channel groups; a warp per token, 4 channels per lane
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 4;
    for (int i = warp; i < kGroup; i += 4) {
      const int slot = (start + i) % cap;
      float recon[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int s = 0; s < 4; ++s) {
        if (s >= 2 && !s_active[s - 2][i]) continue;  // uniform over the warp
        const __nv_bfloat16* src = p.tail_v[s] + (bh * cap + slot) * kHeadDim + 4 * lane;
        float x[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          x[k] = __bfloat162float(src[k]);
          if (s > 0) x[k] = bf16_round(x[k] - recon[k]);
        }
        float mn = fminf(fminf(x[0], x[1]), fminf(x[2], x[3]));
        float mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
          mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const float sc = quant_scale(mn, mx, kLevels);
        const float inv = quant_inverse(sc);
        const __half mn16 = __float2half_rn(mn), sc16 = __float2half_rn(sc);
        uint32_t packed = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t code = quant_code(x[k], mn, sc, inv, kLevels);
          packed |= code << (BITS * k);
          const float dec = bf16_round(dequant_f32(code, sc16, mn16));
          recon[k] = s > 0 ? bf16_round(recon[k] + dec) : dec;
        }
        const int j = s < 2 ? i : s_rank[s - 2][i];
        const int64_t row = p.L.row_base[s][bh] + row0[s] + j;
        uint8_t* dst = p.v_rows[s] + row * (kRowBytes + 16);
        if constexpr (BITS == 4) {
          reinterpret_cast<uint16_t*>(dst)[lane] = static_cast<uint16_t>(packed);
        } else {
          dst[lane] = static_cast<uint8_t>(packed);
        }
        if ((lane & 15) == 0) {
          __half* meta = reinterpret_cast<__half*>(dst + kRowBytes);
          meta[g] = mn16;
          meta[2 + g] = sc16;
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------ bookkeeping
__global__ void advance_state_kernel(const AppendParams p) {
  const int b = blockIdx.x;
  int32_t* st = p.seq_state + b * FL_STATE_WORDS;
  const int cap = p.L.tail_capacity;
  __shared__ int s_rank[2][kGroup];
  const int tid = threadIdx.x;  // 64 threads
  const int tail_len = st[FL_STATE_TAIL_LEN] + 1;
  const bool roll = tail_len >= 2 * kGroup;
  const int quant = st[FL_STATE_QUANT_TOKENS];
  const int start = st[FL_STATE_TAIL_START];
  const int rows2 = st[FL_STATE_ROWS2], rows3 = st[FL_STATE_ROWS3];
  if (roll) {
    if (tid < 2) {
      int n = 0;
      for (int i = 0; i < kGroup; ++i) {
        const bool on = p.tail_active[tid][static_cast<int64_t>(b) * cap + (start + i) % cap] != 0;
        s_rank[tid][i] = on ? (tid == 0 ? rows2 : rows3) + n : -1;
        n += on ? 1 : 0;
      }
    }
    __syncthreads();
    const int64_t base = p.L.rank_base[b] + quant + tid;
    p.rank[0][base] = s_rank[0][tid];
    p.rank[1][base] = s_rank[1][tid];
    const int64_t slot = static_cast<int64_t>(b) * cap + (start + tid) % cap;
    p.tail_active[0][slot] = 0;
    p.tail_active[1][slot] = 0;
  }
  __syncthreads();
  if (tid == 0) {
    if (roll) {
      st[FL_STATE_QUANT_TOKENS] = quant + kGroup;
      st[FL_STATE_ROWS2] = rows2 + kGroup;
      st[FL_STATE_ROWS3] = rows3 + kGroup;
      st[FL_STATE_TAIL_LEN] = tail_len - kGroup;
      st[FL_STATE_TAIL_START] = (start + kGroup) % cap;
    } else {
      st[FL_STATE_TAIL_LEN] = tail_len;
    }
  }
}

}  // namespace
}  // namespace fl

using namespace fl;

extern "C" int fl_append_decode_token(const fl_layer* layer, const void* const* keys,
                                      const void* const* values, fl_cuda_stream stream) {
  const char* who = "fl_append_decode_token";
  if (int rc = validate_layer(layer, 3, who)) return rc;
  FL_REQUIRE(keys && values, "%s: null key/value pointer table", who);
  FL_REQUIRE(layer->tail_capacity >= 2 * kGroup, "%s: tail_capacity must be at least 128", who);
  FL_REQUIRE(layer->tail_active[0] && layer->tail_active[1] && layer->rank[0] && layer->rank[1],
             "%s: tail_active and rank maps are required", who);
  AppendParams p;
  p.L = make_view(*layer);
  for (int s = 0; s < 4; ++s) {
    FL_REQUIRE(keys[s] && values[s], "%s: loop %d K/V pointer is null", who, s);
    FL_REQUIRE(layer->tail_k[s] && layer->tail_v[s], "%s: tail of loop %d is null", who, s);
    p.k_codes[s] = static_cast<uint8_t*>(layer->k_codes[s]);
    p.k_min[s] = static_cast<__half*>(layer->k_min[s]);
    p.k_scale[s] = static_cast<__half*>(layer->k_scale[s]);
    p.v_rows[s] = static_cast<uint8_t*>(layer->v_rows[s]);
    p.tail_k[s] = static_cast<__nv_bfloat16*>(layer->tail_k[s]);
    p.tail_v[s] = static_cast<__nv_bfloat16*>(layer->tail_v[s]);
    p.keys[s] = static_cast<const __nv_bfloat16*>(keys[s]);
    p.values[s] = static_cast<const __nv_bfloat16*>(values[s]);
  }
  p.rank[0] = layer->rank[0];
  p.rank[1] = layer->rank[1];
  p.tail_active[0] = layer->tail_active[0];
  p.tail_active[1] = layer->tail_active[1];
  p.seq_state = layer->seq_state;
  const unsigned bh = static_cast<unsigned>(layer->batch) * layer->heads;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  append_tail_kernel<<<bh, 128, 0, s>>>(p);
  FL_CHECK_LAUNCH("fl_append_decode_token (append)");
  if (layer->bits == 4) {
    rollover_kernel<4><<<dim3(bh, 2), 128, 0, s>>>(p);
  } else {
    rollover_kernel<2><<<dim3(bh, 2), 128, 0, s>>>(p);
  }
  FL_CHECK_LAUNCH("fl_append_decode_token (rollover)");
  advance_state_kernel<<<layer->batch, kGroup, 0, s>>>(p);
  FL_CHECK_LAUNCH("fl_append_decode_token (state)");
  return FL_OK;
}
