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
// grid (batch*heads, 4), 256 threads: y == 0, 1 encode the two channel halves of K, y == 2, 3 the
// even and the odd tokens of V.
//
// K: a stream's 64 x 128 tile of tail rows is copied to shared memory with 16-byte asynchronous
// copies, the tile of the next stream while the codes of this one are packed and stored; thread
// (c, part) owns channel c and sixteen of the tokens (minimum and maximum of a channel are joined
// over the four parts).
// V: a warp per token, four channels per lane, the rows of all four streams fetched together.
constexpr int kRollThreads = 256;

__device__ __forceinline__ void copy16_async(void* dst_shared, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   static_cast<uint32_t>(__cvta_generic_to_shared(dst_shared))),
               "l"(src)
               : "memory");
}

template <int BITS>
__global__ void __launch_bounds__(kRollThreads) rollover_kernel(const AppendParams p) {
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

  if (blockIdx.y < 2) {
    // ---------------- K: per channel over the block's tokens; this CTA owns 64 of the 128 channels
    constexpr int kChan = kHeadDim / 2, kParts = kRollThreads / kChan, kSpan = kGroup / kParts;
    __shared__ __align__(16) __nv_bfloat16 s_x[kGroup][kChan];
    __shared__ __nv_bfloat16 s_recon[kGroup][kChan];
    __shared__ uint8_t s_tile[kGroup][kChan + 4];
    __shared__ float s_lo[kParts][kChan], s_hi[kParts][kChan];
    const int c0 = blockIdx.y * kChan;
    const int c = tid & (kChan - 1), part = tid / kChan;
    const auto fetch = [&](int s) {
      const __nv_bfloat16* src = p.tail_k[s] + bh * cap * kHeadDim + c0;
      for (int idx = tid; idx < kGroup * (kChan / 8); idx += kRollThreads) {
        const int i = idx / (kChan / 8), v = idx % (kChan / 8);
        copy16_async(&s_x[i][8 * v], src + ((start + i) % cap) * kHeadDim + 8 * v);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0);
#pragma unroll 1
    for (int s = 0; s < 4; ++s) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();  // the tile of stream s is in shared memory
      const int rows = s < 2 ? kGroup : s_count[s - 2];
      if (rows == 0) {  // uniform over the CTA
        __syncthreads();
        if (s + 1 < 4) fetch(s + 1);
        continue;
      }
      float mn = INFINITY, mx = -INFINITY;
      for (int i = kSpan * part; i < kSpan * part + kSpan; ++i) {
        if (s >= 2 && !s_active[s - 2][i]) continue;
        float x = __bfloat162float(s_x[i][c]);
        if (s > 0) x = bf16_round(x - __bfloat162float(s_recon[i][c]));
        mn = fminf(mn, x);
        mx = fmaxf(mx, x);
      }
      s_lo[part][c] = mn;
      s_hi[part][c] = mx;
      __syncthreads();
#pragma unroll
      for (int k = 0; k < kParts; ++k) {
        mn = fminf(mn, s_lo[k][c]);
        mx = fmaxf(mx, s_hi[k][c]);
      }
      const float sc = quant_scale(mn, mx, kLevels);
      const float inv = quant_inverse(sc);
      const __half mn16 = __float2half_rn(mn), sc16 = __float2half_rn(sc);
      if (part == 0) {
        const int64_t group = p.L.group_base[s][bh] + row0[s] / kGroup;
        p.k_min[s][group * kHeadDim + c0 + c] = mn16;
        p.k_scale[s][group * kHeadDim + c0 + c] = sc16;
      }
      for (int i = kSpan * part; i < kSpan * part + kSpan; ++i) {
        if (s >= 2 && !s_active[s - 2][i]) continue;
        float x = __bfloat162float(s_x[i][c]);
        const float base = s > 0 ? __bfloat162float(s_recon[i][c]) : 0.f;
        if (s > 0) x = bf16_round(x - base);
        const uint32_t code = quant_code(x, mn, sc, inv, kLevels);
        const int j = s < 2 ? i : s_rank[s - 2][i];
        s_tile[j][c] = static_cast<uint8_t>(code);
        const float dec = bf16_round(dequant_f32(code, sc16, mn16));
        s_recon[i][c] = __float2bfloat16_rn(s > 0 ? base + dec : dec);
      }
      __syncthreads();
      if (s + 1 < 4) fetch(s + 1);  // the tile is no longer read: the next one lands while this one is packed
      // this CTA's half of every code row
      constexpr int kHalfWords = kRowWords / 2;
      uint32_t* dst = reinterpret_cast<uint32_t*>(p.k_codes[s] + (p.L.row_base[s][bh] + row0[s]) * kRowBytes) +
                      blockIdx.y * kHalfWords;
      for (int idx = tid; idx < rows * kHalfWords; idx += kRollThreads) {
        const int row = idx / kHalfWords, wr = idx % kHalfWords;
        uint32_t word = 0;
#pragma unroll
        for (int k = 0; k < kPerWord; ++k) word |= uint32_t(s_tile[row][wr * kPerWord + k]) << (BITS * k);
        dst[row * kRowWords + wr] = word;
      }
      __syncthreads();  // s_tile and s_lo / s_hi are free again
    }
  } else {
    // ---------------- V: per token over 64-channel groups; a warp per token, 4 channels per lane
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 4;
    // two CTAs share a head's 64 tokens: y == 2 takes the even ones, y == 3 the odd ones
    for (int i = 2 * warp + (blockIdx.y - 2); i < kGroup; i += 2 * (kRollThreads / 32)) {
      const int slot = (start + i) % cap;
      uint2 raw[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        raw[s] = ldg64(p.tail_v[s] + (bh * cap + slot) * kHeadDim + 4 * lane);
      }
      float recon[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        if (s >= 2 && !s_active[s - 2][i]) continue;  // uniform over the warp
        float x[4] = {bf16_lo(raw[s].x), bf16_hi(raw[s].x), bf16_lo(raw[s].y), bf16_hi(raw[s].y)};
        if (s > 0) {
#pragma unroll
          for (int k = 0; k < 4; ++k) x[k] = bf16_round(x[k] - recon[k]);
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
  const int tid = threadIdx.x;  // 64 threads
  const int tail_len = st[FL_STATE_TAIL_LEN] + 1;
  const bool roll = tail_len >= 2 * kGroup;
  const int quant = st[FL_STATE_QUANT_TOKENS];
  const int start = st[FL_STATE_TAIL_START];
  const int rows2 = st[FL_STATE_ROWS2], rows3 = st[FL_STATE_ROWS3];
  if (roll) {
    // thread i owns tail token i: its compact rank in streams 2 / 3 is the number of retained tokens
    // before it (a ballot per warp, the first warp's count added in the second)
    __shared__ int s_first[2];
    const int64_t slot = static_cast<int64_t>(b) * cap + (start + tid) % cap;
    const bool on0 = p.tail_active[0][slot] != 0, on1 = p.tail_active[1][slot] != 0;
    const uint32_t m0 = __ballot_sync(0xffffffffu, on0), m1 = __ballot_sync(0xffffffffu, on1);
    const int lane = tid & 31;
    if (tid == 0) {
      s_first[0] = __popc(m0);
      s_first[1] = __popc(m1);
    }
    __syncthreads();
    const uint32_t below = (1u << lane) - 1u;
    const int r0 = __popc(m0 & below) + (tid >= 32 ? s_first[0] : 0);
    const int r1 = __popc(m1 & below) + (tid >= 32 ? s_first[1] : 0);
    const int64_t base = p.L.rank_base[b] + quant + tid;
    p.rank[0][base] = on0 ? rows2 + r0 : -1;
    p.rank[1][base] = on1 ? rows3 + r1 : -1;
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
    rollover_kernel<4><<<dim3(bh, 4), kRollThreads, 0, s>>>(p);
  } else {
    rollover_kernel<2><<<dim3(bh, 4), kRollThreads, 0, s>>>(p);
  }
  FL_CHECK_LAUNCH("fl_append_decode_token (rollover)");
  advance_state_kernel<<<layer->batch, kGroup, 0, s>>>(p);
  FL_CHECK_LAUNCH("fl_append_decode_token (state)");
  return FL_OK;
}
