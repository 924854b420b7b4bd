// Prefill-time residual encoder: the four loops' K/V of a batch of prompts go straight into the
// packed streams of the cache.
//
// Replaces CrossLoopKVLayerBuilder.from_loop1 / add_loop2 / _install_sparse_streams / finalize
// and _encode_initial_prefix (flashloop/cache.py:343-397, 415-439, 469-508, 510-625, 1008-1074):
// per stream a decode of the base, a bfloat16 subtraction, a quantise + pack and a bfloat16
// add-back, each a full-tensor launch (and several full-size temporaries) in the reference.
// Here: one launch for the anchor and delta-2 streams of every 64-token block, one for the
// delta-3 rows and one for the delta-4 rows.  Every subtraction and addition is rounded to
// bfloat16 exactly where the reference's tensor ops round, so codes and metadata are the same
// bits.
//
//   encode_dense_kernel    grid (heads x 64-token blocks, K|V): streams 0 and 1 of one block,
//                          and the block's bfloat16 reconstruction (anchor + delta-2) for later
//   encode_compact_kernel  grid (heads x 64-row groups, K|V): stream 2 or 3 over the retained
//                          rows, 64 compact rows per K metadata group as the reference packs
//                          the compacted tensor; stream 2 adds its decode to the reconstruction
#include "fl_common.cuh"

namespace fl {
namespace {

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

struct EncodeParams {
  LayerView L;
  uint8_t* k_codes[4];
  __half* k_min[4];
  __half* k_scale[4];
  uint8_t* v_rows[4];
  const __nv_bfloat16* keys[4];    // [sequences][heads][tokens][128]
  const __nv_bfloat16* values[4];
  __nv_bfloat16* recon_k;          // [sequences][heads][tokens][128]: anchor + delta-2 (+ delta-3)
  __nv_bfloat16* recon_v;
  const int32_t* positions[2];     // [sequences][positions_stride]: retained positions, ascending, then -1
  int64_t positions_stride;
  int sequence_begin;              // first sequence of the layer these inputs belong to
  int tokens;                      // tokens per input sequence
  int blocks;                      // grid: 64-token blocks (dense) or 64-row groups (compact) per head
  int stream;                      // compact kernel: 2 or 3
  int first_stream, last_stream;   // dense kernel: the streams of this launch (0..1, 0..0 or 1..1)
  int compact_input;               // compact kernel: input row i of a sequence is its i-th retained row
                                   // (otherwise the row of its logical position)
};

// The bfloat16 value a packed K row holds in channel c: code * scale + minimum in float32, rounded
// (flashloop/packing.py:108-132), read back from stream s of the layer under construction.
template <int BITS>
__device__ __forceinline__ float decode_k(const EncodeParams& p, int s, int64_t bh, int row, int c) {
  constexpr int kRowBytes = 16 * BITS;
  constexpr int kPerByte = 8 / BITS;
  const uint8_t byte = p.k_codes[s][(p.L.row_base[s][bh] + row) * kRowBytes + c / kPerByte];
  const uint32_t code = (byte >> (BITS * (c % kPerByte))) & ((1u << BITS) - 1u);
  const int64_t group = p.L.group_base[s][bh] + (row >> 6);
  return bf16_round(dequant_f32(code, p.k_scale[s][group * kHeadDim + c], p.k_min[s][group * kHeadDim + c]));
}
// The same for the lane's four V channels 4*lane .. 4*lane+3 of a record.
template <int BITS>
__device__ __forceinline__ void decode_v4(const EncodeParams& p, int s, int64_t bh, int row, int lane, float (&dec)[4]) {
  constexpr int kRowBytes = 16 * BITS;
  const uint8_t* record = p.v_rows[s] + (p.L.row_base[s][bh] + row) * (kRowBytes + 16);
  uint32_t packed;
  if constexpr (BITS == 4) {
    packed = reinterpret_cast<const uint16_t*>(record)[lane];
  } else {
    packed = record[lane];
  }
  const __half* meta = reinterpret_cast<const __half*>(record + kRowBytes);
  const __half mn16 = meta[lane >> 4], sc16 = meta[2 + (lane >> 4)];
#pragma unroll
  for (int k = 0; k < 4; ++k) dec[k] = bf16_round(dequant_f32((packed >> (BITS * k)) & ((1u << BITS) - 1u), sc16, mn16));
}
// The base a compact stream's residual is taken against at logical position `pos`: decode(anchor)
// + decode(delta-2), and for stream 3 + decode(delta-3) of the position's loop-3 row, each sum
// rounded to bfloat16 (flashloop/cache.py:488-504).
template <int BITS>
__device__ __forceinline__ float base_k(const EncodeParams& p, int s, int b, int64_t bh, int pos, int c) {
  float base = bf16_round(decode_k<BITS>(p, 0, bh, pos, c) + decode_k<BITS>(p, 1, bh, pos, c));
  if (s == 3) {
    const int r3 = p.L.rank[0][p.L.rank_base[b] + pos];
    if (r3 >= 0) base = bf16_round(base + decode_k<BITS>(p, 2, bh, r3, c));
  }
  return base;
}
template <int BITS>
__device__ __forceinline__ void base_v4(const EncodeParams& p, int s, int b, int64_t bh, int pos, int lane,
                                        float (&base)[4]) {
  float d0[4], d1[4];
  decode_v4<BITS>(p, 0, bh, pos, lane, d0);
  decode_v4<BITS>(p, 1, bh, pos, lane, d1);
#pragma unroll
  for (int k = 0; k < 4; ++k) base[k] = bf16_round(d0[k] + d1[k]);
  if (s == 3) {
    const int r3 = p.L.rank[0][p.L.rank_base[b] + pos];
    if (r3 >= 0) {
      decode_v4<BITS>(p, 2, bh, r3, lane, d0);
#pragma unroll
      for (int k = 0; k < 4; ++k) base[k] = bf16_round(base[k] + d0[k]);
    }
  }
}


// Pack one byte-per-code tile of `rows` rows into code rows.
template <int BITS>
__device__ __forceinline__ void store_code_rows(const uint8_t (*tile)[kHeadDim + 4], int rows, uint8_t* dst_rows) {
  constexpr int kRowWords = 16 * BITS / 4;
  constexpr int kPerWord = 32 / BITS;
  uint32_t* dst = reinterpret_cast<uint32_t*>(dst_rows);
  for (int idx = threadIdx.x; idx < rows * kRowWords; idx += 128) {
    const int row = idx / kRowWords, wr = idx % kRowWords;
    uint32_t word = 0;
#pragma unroll
    for (int k = 0; k < kPerWord; ++k) word |= uint32_t(tile[row][wr * kPerWord + k]) << (BITS * k);
    dst[idx] = word;
  }
}

// One V row (a warp, 4 channels per lane): quantise x against its 64-channel group, write the
// record, return the bfloat16 decode in `dec`.
template <int BITS>
__device__ __forceinline__ void encode_v_row(const float (&x)[4], uint8_t* record, int lane, float (&dec)[4]) {
  constexpr float kLevels = float((1 << BITS) - 1);
  constexpr int kRowBytes = 16 * BITS;
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
    dec[k] = bf16_round(dequant_f32(code, sc16, mn16));
  }
  if constexpr (BITS == 4) {
    reinterpret_cast<uint16_t*>(record)[lane] = static_cast<uint16_t>(packed);
  } else {
    record[lane] = static_cast<uint8_t>(packed);
  }
  if ((lane & 15) == 0) {
    __half* meta = reinterpret_cast<__half*>(record + kRowBytes);
    meta[lane >> 4] = mn16;
    meta[2 + (lane >> 4)] = sc16;
  }
}

__device__ __forceinline__ void load4(const __nv_bfloat16* src, float (&x)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  x[0] = bf16_lo(raw.x); x[1] = bf16_hi(raw.x); x[2] = bf16_lo(raw.y); x[3] = bf16_hi(raw.y);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, const float (&x)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
  *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// Rows of 128 bfloat16 between global and shared memory, 16 bytes per thread and step.
// `row_of(i)` gives the global row index of tile row i.
template <typename RowOf>
__device__ __forceinline__ void load_rows(__nv_bfloat16 (*tile)[kHeadDim], const __nv_bfloat16* base, int rows,
                                          RowOf row_of) {
  for (int idx = threadIdx.x; idx < rows * 16; idx += 128) {
    const int i = idx >> 4, piece = idx & 15;
    *reinterpret_cast<uint4*>(&tile[i][piece * 8]) =
        ldg128(base + static_cast<int64_t>(row_of(i)) * kHeadDim + piece * 8);
  }
}
template <typename RowOf>
__device__ __forceinline__ void store_rows(const __nv_bfloat16 (*tile)[kHeadDim], __nv_bfloat16* base, int rows,
                                           RowOf row_of) {
  for (int idx = threadIdx.x; idx < rows * 16; idx += 128) {
    const int i = idx >> 4, piece = idx & 15;
    *reinterpret_cast<uint4*>(base + static_cast<int64_t>(row_of(i)) * kHeadDim + piece * 8) =
        *reinterpret_cast<const uint4*>(&tile[i][piece * 8]);
  }
}

// ------------------------------------------------------------------------------ streams 0 and 1
template <int BITS>
__global__ void __launch_bounds__(128) encode_dense_kernel(const EncodeParams p) {
  constexpr float kLevels = float((1 << BITS) - 1);
  constexpr int kRowBytes = 16 * BITS;
  const int head_in = blockIdx.x / p.blocks;  // (sequence, head) of the inputs
  const int blk = blockIdx.x % p.blocks;
  const int heads = p.L.heads;
  const int b = p.sequence_begin + head_in / heads;
  const int64_t bh = static_cast<int64_t>(b) * heads + head_in % heads;
  const int quant = p.L.seq_state[b * FL_STATE_WORDS + FL_STATE_QUANT_TOKENS];
  const int t0 = blk * kGroup;
  if (t0 >= quant) return;  // the tail stays bfloat16
  const int64_t in_row0 = (static_cast<int64_t>(head_in) * p.tokens + t0) * kHeadDim;
  const int tid = threadIdx.x;
  auto consecutive = [](int i) { return i; };

  if (blockIdx.y == 0) {
    // ---------------- K: per channel over the block's 64 tokens; thread c owns channel c
    __shared__ __align__(16) __nv_bfloat16 s_in[kGroup][kHeadDim];
    __shared__ __align__(16) __nv_bfloat16 s_recon[kGroup][kHeadDim];
    __shared__ uint8_t s_tile[kGroup][kHeadDim + 4];
    const int c = tid;
    if (p.first_stream == 1) {  // delta-2 alone: its base is the anchor as it was packed
      for (int i = 0; i < kGroup; ++i) s_recon[i][c] = __float2bfloat16_rn(decode_k<BITS>(p, 0, bh, t0 + i, c));
    }
#pragma unroll 1
    for (int s = p.first_stream; s <= p.last_stream; ++s) {
      load_rows(s_in, p.keys[s] + in_row0, kGroup, consecutive);
      __syncthreads();
      float mn = INFINITY, mx = -INFINITY;
      for (int i = 0; i < kGroup; ++i) {
        float x = __bfloat162float(s_in[i][c]);
        if (s > 0) x = bf16_round(x - __bfloat162float(s_recon[i][c]));
        mn = fminf(mn, x);
        mx = fmaxf(mx, x);
      }
      const float sc = quant_scale(mn, mx, kLevels);
      const float inv = quant_inverse(sc);
      const __half mn16 = __float2half_rn(mn), sc16 = __float2half_rn(sc);
      const int64_t group = p.L.group_base[s][bh] + blk;
      p.k_min[s][group * kHeadDim + c] = mn16;
      p.k_scale[s][group * kHeadDim + c] = sc16;
      for (int i = 0; i < kGroup; ++i) {
        float x = __bfloat162float(s_in[i][c]);
        const float base = s > 0 ? __bfloat162float(s_recon[i][c]) : 0.f;
        if (s > 0) x = bf16_round(x - base);
        const uint32_t code = quant_code(x, mn, sc, inv, kLevels);
        s_tile[i][c] = static_cast<uint8_t>(code);
        const float dec = bf16_round(dequant_f32(code, sc16, mn16));
        s_recon[i][c] = __float2bfloat16_rn(s > 0 ? base + dec : dec);
      }
      __syncthreads();
      store_code_rows<BITS>(s_tile, kGroup, p.k_codes[s] + (p.L.row_base[s][bh] + t0) * kRowBytes);
      __syncthreads();
    }
    if (p.recon_k) store_rows(s_recon, p.recon_k + in_row0, kGroup, consecutive);
  } else {
    // ---------------- V: per token over 64-channel groups; a warp per token, 4 channels per lane,
    // four tokens at a time so that their loads are in flight together
    const int lane = tid & 31, warp = tid >> 5;
    for (int i0 = warp * 4; i0 < kGroup; i0 += 16) {
      float x0[4][4], x1[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t in = in_row0 + static_cast<int64_t>(i0 + j) * kHeadDim + 4 * lane;
        if (p.first_stream == 0) load4(p.values[0] + in, x0[j]);
        if (p.last_stream == 1) load4(p.values[1] + in, x1[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + j;
        float recon[4], dec[4];
        if (p.first_stream == 0) {
          encode_v_row<BITS>(x0[j], p.v_rows[0] + (p.L.row_base[0][bh] + t0 + i) * (kRowBytes + 16), lane, recon);
        } else {
          decode_v4<BITS>(p, 0, bh, t0 + i, lane, recon);
        }
        if (p.last_stream == 0) continue;
#pragma unroll
        for (int k = 0; k < 4; ++k) x1[j][k] = bf16_round(x1[j][k] - recon[k]);
        encode_v_row<BITS>(x1[j], p.v_rows[1] + (p.L.row_base[1][bh] + t0 + i) * (kRowBytes + 16), lane, dec);
        if (p.recon_v) {
#pragma unroll
          for (int k = 0; k < 4; ++k) recon[k] = bf16_round(recon[k] + dec[k]);
          store4(p.recon_v + in_row0 + static_cast<int64_t>(i) * kHeadDim + 4 * lane, recon);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------ streams 2 and 3
template <int BITS>
__global__ void __launch_bounds__(128) encode_compact_kernel(const EncodeParams p) {
  constexpr float kLevels = float((1 << BITS) - 1);
  constexpr int kRowBytes = 16 * BITS;
  const int s = p.stream;
  const int head_in = blockIdx.x / p.blocks;
  const int grp = blockIdx.x % p.blocks;
  const int heads = p.L.heads;
  const int seq_in = head_in / heads;
  const int b = p.sequence_begin + seq_in;
  const int64_t bh = static_cast<int64_t>(b) * heads + head_in % heads;
  const int quant = p.L.seq_state[b * FL_STATE_WORDS + FL_STATE_QUANT_TOKENS];
  const int j0 = grp * kGroup;
  const int tid = threadIdx.x;

  // the group's compact rows: retained positions inside the packed prefix (an ascending prefix)
  __shared__ int s_pos[kGroup];
  __shared__ int s_rows;
  if (tid < kGroup) {
    const int64_t at = static_cast<int64_t>(seq_in) * p.positions_stride + j0 + tid;
    const int pos = j0 + tid < p.positions_stride ? p.positions[s - 2][at] : -1;
    s_pos[tid] = (pos >= 0 && pos < quant) ? pos : -1;
  }
  __syncthreads();
  if (tid == 0) {
    int n = 0;
    while (n < kGroup && s_pos[n] >= 0) ++n;
    s_rows = n;
  }
  __syncthreads();
  const int rows = s_rows;
  if (rows == 0) return;
  const int64_t in_head = static_cast<int64_t>(head_in) * p.tokens * kHeadDim;
  auto retained = [&](int i) { return s_pos[i]; };
  // where the group's rows sit in the input: at their logical positions, or packed in retained order
  auto input_row = [&](int i) { return p.compact_input ? j0 + i : s_pos[i]; };

  if (blockIdx.y == 0) {
    __shared__ __align__(16) __nv_bfloat16 s_in[kGroup][kHeadDim];
    __shared__ __align__(16) __nv_bfloat16 s_recon[kGroup][kHeadDim];
    __shared__ uint8_t s_tile[kGroup][kHeadDim + 4];
    const int c = tid;
    load_rows(s_in, p.keys[s] + in_head, rows, input_row);
    if (p.recon_k) {
      load_rows(s_recon, p.recon_k + in_head, rows, retained);
    } else {
      for (int i = 0; i < rows; ++i) s_recon[i][c] = __float2bfloat16_rn(base_k<BITS>(p, s, b, bh, s_pos[i], c));
    }
    __syncthreads();
    float mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < rows; ++i) {
      const float x = bf16_round(__bfloat162float(s_in[i][c]) - __bfloat162float(s_recon[i][c]));
      mn = fminf(mn, x);
      mx = fmaxf(mx, x);
    }
    const float sc = quant_scale(mn, mx, kLevels);
    const float inv = quant_inverse(sc);
    const __half mn16 = __float2half_rn(mn), sc16 = __float2half_rn(sc);
    const int64_t group = p.L.group_base[s][bh] + grp;
    p.k_min[s][group * kHeadDim + c] = mn16;
    p.k_scale[s][group * kHeadDim + c] = sc16;
    for (int i = 0; i < rows; ++i) {
      const float base = __bfloat162float(s_recon[i][c]);
      const float x = bf16_round(__bfloat162float(s_in[i][c]) - base);
      const uint32_t code = quant_code(x, mn, sc, inv, kLevels);
      s_tile[i][c] = static_cast<uint8_t>(code);
      if (s == 2) s_recon[i][c] = __float2bfloat16_rn(base + bf16_round(dequant_f32(code, sc16, mn16)));
    }
    __syncthreads();
    store_code_rows<BITS>(s_tile, rows, p.k_codes[s] + (p.L.row_base[s][bh] + j0) * kRowBytes);
    if (s == 2 && p.recon_k) store_rows(s_recon, p.recon_k + in_head, rows, retained);
  } else {
    const int lane = tid & 31, warp = tid >> 5;
    for (int i0 = warp * 4; i0 < rows; i0 += 16) {
      float x[4][4], recon[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = min(i0 + j, rows - 1);
        load4(p.values[s] + in_head + static_cast<int64_t>(input_row(i)) * kHeadDim + 4 * lane, x[j]);
        if (p.recon_v) {
          load4(p.recon_v + in_head + static_cast<int64_t>(s_pos[i]) * kHeadDim + 4 * lane, recon[j]);
        } else {
          base_v4<BITS>(p, s, b, bh, s_pos[i], lane, recon[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + j;
        if (i >= rows) break;
        float dec[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) x[j][k] = bf16_round(x[j][k] - recon[j][k]);
        encode_v_row<BITS>(x[j], p.v_rows[s] + (p.L.row_base[s][bh] + j0 + i) * (kRowBytes + 16), lane, dec);
        if (s == 2 && p.recon_v) {
#pragma unroll
          for (int k = 0; k < 4; ++k) recon[j][k] = bf16_round(recon[j][k] + dec[k]);
          store4(p.recon_v + in_head + static_cast<int64_t>(s_pos[i]) * kHeadDim + 4 * lane, recon[j]);
        }
      }
    }
  }
}

}  // namespace
}  // namespace fl

using namespace fl;

extern "C" int fl_encode_prefill(const fl_layer* layer, int32_t sequence_begin, int32_t sequence_count,
                                 int64_t tokens, const void* const* keys, const void* const* values,
                                 const int32_t* positions3, const int32_t* positions4, int64_t positions_stride,
                                 void* recon_k, void* recon_v, fl_cuda_stream stream) {
  const char* who = "fl_encode_prefill";
  if (int rc = validate_layer(layer, 3, who)) return rc;
  FL_REQUIRE(keys && values && recon_k && recon_v, "%s: null argument", who);
  FL_REQUIRE(sequence_begin >= 0 && sequence_count > 0 && sequence_begin + sequence_count <= layer->batch,
             "%s: sequences [%d, %d) outside the layer's batch of %d", who, sequence_begin,
             sequence_begin + sequence_count, layer->batch);
  FL_REQUIRE(tokens > 0 && tokens < (int64_t(1) << 30), "%s: bad token count", who);
  FL_REQUIRE((positions3 && positions4 && positions_stride > 0) || (!positions3 && !positions4),
             "%s: both position lists or neither", who);
  EncodeParams p;
  p.L = make_view(*layer);
  for (int s = 0; s < 4; ++s) {
    FL_REQUIRE(keys[s] && values[s], "%s: loop %d K/V pointer is null", who, s);
    FL_REQUIRE(aligned16(keys[s]) && aligned16(values[s]), "%s: K/V must be 16-byte aligned", who);
    p.k_codes[s] = static_cast<uint8_t*>(layer->k_codes[s]);
    p.k_min[s] = static_cast<__half*>(layer->k_min[s]);
    p.k_scale[s] = static_cast<__half*>(layer->k_scale[s]);
    p.v_rows[s] = static_cast<uint8_t*>(layer->v_rows[s]);
    p.keys[s] = static_cast<const __nv_bfloat16*>(keys[s]);
    p.values[s] = static_cast<const __nv_bfloat16*>(values[s]);
  }
  FL_REQUIRE(aligned16(recon_k) && aligned16(recon_v), "%s: scratch must be 16-byte aligned", who);
  p.recon_k = static_cast<__nv_bfloat16*>(recon_k);
  p.recon_v = static_cast<__nv_bfloat16*>(recon_v);
  p.positions[0] = positions3;
  p.positions[1] = positions4;
  p.positions_stride = positions_stride;
  p.sequence_begin = sequence_begin;
  p.tokens = static_cast<int>(tokens);
  p.blocks = static_cast<int>(tokens / kGroup);
  p.stream = 0;
  p.first_stream = 0;
  p.last_stream = 1;
  p.compact_input = 0;
  const int64_t heads_in = static_cast<int64_t>(sequence_count) * layer->heads;
  FL_REQUIRE(heads_in * (p.blocks + 1) < (int64_t(1) << 31), "%s: grid too large", who);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p.blocks > 0) {
    const dim3 grid(static_cast<unsigned>(heads_in * p.blocks), 2);
    if (layer->bits == 4) encode_dense_kernel<4><<<grid, 128, 0, st>>>(p); else encode_dense_kernel<2><<<grid, 128, 0, st>>>(p);
    FL_CHECK_LAUNCH("fl_encode_prefill (anchor, delta-2)");
    if (positions3) {
      for (int s = 2; s < 4; ++s) {
        p.stream = s;
        if (layer->bits == 4) encode_compact_kernel<4><<<grid, 128, 0, st>>>(p); else encode_compact_kernel<2><<<grid, 128, 0, st>>>(p);
        FL_CHECK_LAUNCH("fl_encode_prefill (compact stream)");
      }
    }
  }
  return FL_OK;
}

extern "C" int fl_encode_prefill_stage(const fl_layer* layer, int32_t sequence_begin, int32_t sequence_count,
                                       int64_t rows, int32_t stage, const void* keys, const void* values,
                                       const int32_t* positions, int64_t positions_stride, int32_t compact_input,
                                       fl_cuda_stream stream) {
  const char* who = "fl_encode_prefill_stage";
  FL_REQUIRE(stage >= 0 && stage < 4, "%s: stage must be in [0, 3], got %d", who, stage);
  if (int rc = validate_layer(layer, stage, who)) return rc;
  FL_REQUIRE(keys && values, "%s: null K/V", who);
  FL_REQUIRE(aligned16(keys) && aligned16(values), "%s: K/V must be 16-byte aligned", who);
  FL_REQUIRE(sequence_begin >= 0 && sequence_count > 0 && sequence_begin + sequence_count <= layer->batch,
             "%s: sequences [%d, %d) outside the layer's batch of %d", who, sequence_begin,
             sequence_begin + sequence_count, layer->batch);
  FL_REQUIRE(rows > 0 && rows < (int64_t(1) << 30), "%s: bad row count", who);
  FL_REQUIRE(stage < 2 || (positions && positions_stride > 0), "%s: stages 2 and 3 need the retained positions", who);
  EncodeParams p{};
  p.L = make_view(*layer);
  for (int s = 0; s < 4; ++s) {
    p.k_codes[s] = static_cast<uint8_t*>(layer->k_codes[s]);
    p.k_min[s] = static_cast<__half*>(layer->k_min[s]);
    p.k_scale[s] = static_cast<__half*>(layer->k_scale[s]);
    p.v_rows[s] = static_cast<uint8_t*>(layer->v_rows[s]);
  }
  p.keys[stage] = static_cast<const __nv_bfloat16*>(keys);
  p.values[stage] = static_cast<const __nv_bfloat16*>(values);
  p.recon_k = nullptr;
  p.recon_v = nullptr;
  p.sequence_begin = sequence_begin;
  p.tokens = static_cast<int>(rows);
  p.stream = stage;
  p.first_stream = p.last_stream = stage;
  p.compact_input = compact_input ? 1 : 0;
  const int64_t heads_in = static_cast<int64_t>(sequence_count) * layer->heads;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (stage < 2) {
    p.blocks = static_cast<int>(rows / kGroup);
    if (p.blocks == 0) return FL_OK;
    FL_REQUIRE(heads_in * p.blocks < (int64_t(1) << 31), "%s: grid too large", who);
    const dim3 grid(static_cast<unsigned>(heads_in * p.blocks), 2);
    if (layer->bits == 4) encode_dense_kernel<4><<<grid, 128, 0, st>>>(p); else encode_dense_kernel<2><<<grid, 128, 0, st>>>(p);
  } else {
    p.positions[stage - 2] = positions;
    p.positions_stride = positions_stride;
    p.blocks = static_cast<int>((positions_stride + kGroup - 1) / kGroup);
    FL_REQUIRE(heads_in * p.blocks < (int64_t(1) << 31), "%s: grid too large", who);
    const dim3 grid(static_cast<unsigned>(heads_in * p.blocks), 2);
    if (layer->bits == 4) encode_compact_kernel<4><<<grid, 128, 0, st>>>(p); else encode_compact_kernel<2><<<grid, 128, 0, st>>>(p);
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}
