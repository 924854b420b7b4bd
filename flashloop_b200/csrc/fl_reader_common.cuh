// Device helpers shared by the dense reader (fl_reader.cu) and the selected readers
// (fl_selected.cu): code unpacking, float16-pair dot products and accumulation, the online
// softmax state, BF16 row helpers, and the layout of the readers' scratch workspace.
#pragma once

#include <climits>
#include <cstdlib>

#include "fl_common.cuh"

namespace fl {
namespace {

constexpr int kPartialStride = 132;  // acc[128], running max (log2 domain), denominator, pad
constexpr int kMaxSplits = 64;

struct ReaderParams {
  LayerView L;
  int loop;
  const __nv_bfloat16* q;
  const __nv_bfloat16* kcur;
  const __nv_bfloat16* vcur;
  float scaling;
  float scaling_log2;
  float* out;
  float* logits;
  int64_t logits_stride;
  float* partial;
  int* tickets;
  int* status;
  int max_chunks;
  int tail_units;  // dense reader: units a head's tail counts as in the static partition
  // selected readers
  const int32_t* indices;
  const uint8_t* valid;
  int capacity;
  int slots_per_cta;
  const float* weights;
  const float* source_out;
  const float* mass;
  float* cur_logits;
};

// ------------------------------------------------------------------------------ code handling

template <int BITS>
struct Codes;
template <>
struct Codes<4> {
  uint32_t w[4];
};
template <>
struct Codes<2> {
  uint32_t w[2];
};

template <int BITS>
__device__ __forceinline__ Codes<BITS> load_codes_shared(const uint8_t* piece) {
  Codes<BITS> c;
  if constexpr (BITS == 4) {
    const uint4 v = *reinterpret_cast<const uint4*>(piece);
    c.w[0] = v.x; c.w[1] = v.y; c.w[2] = v.z; c.w[3] = v.w;
  } else {
    const uint2 v = *reinterpret_cast<const uint2*>(piece);
    c.w[0] = v.x; c.w[1] = v.y;
  }
  return c;
}

template <int BITS>
constexpr int kCentre = 1 << (BITS - 1);

// Channel (0..31 within the lane) held by half `hi` of pair `p` after unpack_centred.
template <int BITS>
__host__ __device__ constexpr int pair_channel(int p, int hi) {
  return BITS == 4 ? (p / 4) * 8 + (p % 4) + 4 * hi : (p / 8) * 16 + (p % 8) + 8 * hi;
}
// Inverse: accumulator slot 2*p + hi of the lane's channel cc.
template <int BITS>
__host__ __device__ constexpr int channel_slot(int cc) {
  return BITS == 4 ? 2 * ((cc / 8) * 4 + (cc % 8) % 4) + (cc % 8) / 4
                   : 2 * ((cc / 16) * 8 + (cc % 16) % 8) + (cc % 16) / 8;
}

// The lane's 32 codes as 16 half2 of exact integers (code - centre), in pair order.
template <int BITS>
__device__ __forceinline__ void unpack_centred(const Codes<BITS>& c, __half2 (&h)[16]) {
  const uint32_t kMagic = 0x64006400u;
  if constexpr (BITS == 4) {
    const __half2 kOff = __floats2half2_rn(1032.f, 1032.f);
    const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
    const __half2 kOff16 = __floats2half2_rn(-72.f, -72.f);
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
      const uint32_t w = c.w[wd];
      const uint32_t w8 = w >> 8;
      h[4 * wd + 0] = __hsub2(as_half2(and_or(w, 0x000F000Fu, kMagic)), kOff);
      h[4 * wd + 1] = __hfma2(as_half2(and_or(w, 0x00F000F0u, kMagic)), k16th, kOff16);
      h[4 * wd + 2] = __hsub2(as_half2(and_or(w8, 0x000F000Fu, kMagic)), kOff);
      h[4 * wd + 3] = __hfma2(as_half2(and_or(w8, 0x00F000F0u, kMagic)), k16th, kOff16);
    }
  } else {
    const __half2 kOff = __floats2half2_rn(1026.f, 1026.f);
    const __half2 k4th = __floats2half2_rn(0.25f, 0.25f);
    const __half2 kOff4 = __floats2half2_rn(-258.f, -258.f);
    const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
    const __half2 kOff16 = __floats2half2_rn(-66.f, -66.f);
    const __half2 k64th = __floats2half2_rn(0.015625f, 0.015625f);
    const __half2 kOff64 = __floats2half2_rn(-18.f, -18.f);
#pragma unroll
    for (int wd = 0; wd < 2; ++wd) {
      const uint32_t w = c.w[wd];
      const uint32_t w8 = w >> 8;
      h[8 * wd + 0] = __hsub2(as_half2(and_or(w, 0x00030003u, kMagic)), kOff);
      h[8 * wd + 1] = __hfma2(as_half2(and_or(w, 0x000C000Cu, kMagic)), k4th, kOff4);
      h[8 * wd + 2] = __hfma2(as_half2(and_or(w, 0x00300030u, kMagic)), k16th, kOff16);
      h[8 * wd + 3] = __hfma2(as_half2(and_or(w, 0x00C000C0u, kMagic)), k64th, kOff64);
      h[8 * wd + 4] = __hsub2(as_half2(and_or(w8, 0x00030003u, kMagic)), kOff);
      h[8 * wd + 5] = __hfma2(as_half2(and_or(w8, 0x000C000Cu, kMagic)), k4th, kOff4);
      h[8 * wd + 6] = __hfma2(as_half2(and_or(w8, 0x00300030u, kMagic)), k16th, kOff16);
      h[8 * wd + 7] = __hfma2(as_half2(and_or(w8, 0x00C000C0u, kMagic)), k64th, kOff64);
    }
  }
}

// K, fast path: sum over the lane's 32 channels of w_c * (code_c - centre).
template <int BITS>
__device__ __forceinline__ float k_dot_fast(const Codes<BITS>& c, const __half2 (&mult)[16]) {
  __half2 h[16];
  unpack_centred<BITS>(c, h);
  __half2 a0 = __hmul2(h[0], mult[0]);
  __half2 a1 = __hmul2(h[1], mult[1]);
#pragma unroll
  for (int p = 2; p < 16; p += 2) {
    a0 = __hfma2(h[p], mult[p], a0);
    a1 = __hfma2(h[p + 1], mult[p + 1], a1);
  }
  const float2 f0 = __half22float2(a0);
  const float2 f1 = __half22float2(a1);
  return (f0.x + f0.y) + (f1.x + f1.y);
}

template <int BITS>
__device__ __forceinline__ void v_accumulate(const Codes<BITS>& c, __half2 w, __half2 (&hacc)[16]) {
  __half2 h[16];
  unpack_centred<BITS>(c, h);
#pragma unroll
  for (int p = 0; p < 16; ++p) hacc[p] = __hfma2(h[p], w, hacc[p]);
}

__device__ __forceinline__ void flush_pairs(__half2 (&hacc)[16], float (&acc)[32]) {
#pragma unroll
  for (int p = 0; p < 16; ++p) {
    const float2 f = __half22float2(hacc[p]);
    acc[2 * p] += f.x;
    acc[2 * p + 1] += f.y;
    hacc[p] = __floats2half2_rn(0.f, 0.f);
  }
}

// ------------------------------------------------------------------------------ tensor-pipe dot products
//
// The dense reader's contractions (q . K rows, p . V rows) have one query per head, so they are
// GEMVs and HBM-bound; done on the ALU pipes they are issue-bound instead (unpack + centre +
// multiply-add is about twenty issue slots per eight codes).  Handing the multiply-adds and the
// sums over the lane quad to mma.sync.m16n8k16 (float16 operands, float32 accumulators) leaves
// one shift and four logic ops per eight codes on the ALU pipes.  Codes go in uncentred and
// unscaled, exactly as the magic-number unpack leaves them, 1024 + t * code with t = 1 or 16 (4 bits)
// or 1, 4, 16, 64 (2 bits) by position: the other operand carries 1/t, and what the 1024s add up to
// is taken out again as a bias (K: 1024 * sum of the table; V: one more mma with a constant-1024
// operand), computed from the same rounded operands so that it cancels exactly.

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The 1/t of the code at position `cc` (channel within the lane's run of channels).
template <int BITS>
__device__ __forceinline__ float position_factor(int cc) {
  if constexpr (BITS == 4) return (cc & 1) ? 0.0625f : 1.f;
  const int t = cc & 3;
  return t == 0 ? 1.f : (t == 1 ? 0.25f : (t == 2 ? 0.0625f : 0.015625f));
}

// One 32-bit word of codes -> float16 pairs 1024 + t * code, in the pair order of unpack_centred
// (4 bits: four pairs; 2 bits: eight pairs).
template <int BITS>
__device__ __forceinline__ void unpack_raw_word(uint32_t w, uint32_t* h) {
  const uint32_t kMagic = 0x64006400u;
  const uint32_t w8 = w >> 8;
  if constexpr (BITS == 4) {
    h[0] = and_or(w, 0x000F000Fu, kMagic);
    h[1] = and_or(w, 0x00F000F0u, kMagic);
    h[2] = and_or(w8, 0x000F000Fu, kMagic);
    h[3] = and_or(w8, 0x00F000F0u, kMagic);
  } else {
    h[0] = and_or(w, 0x00030003u, kMagic);
    h[1] = and_or(w, 0x000C000Cu, kMagic);
    h[2] = and_or(w, 0x00300030u, kMagic);
    h[3] = and_or(w, 0x00C000C0u, kMagic);
    h[4] = and_or(w8, 0x00030003u, kMagic);
    h[5] = and_or(w8, 0x000C000Cu, kMagic);
    h[6] = and_or(w8, 0x00300030u, kMagic);
    h[7] = and_or(w8, 0x00C000C0u, kMagic);
  }
}

__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}
__device__ __forceinline__ float across_quads_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
  return v;
}
__device__ __forceinline__ float across_quads_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}

// The lane's 32 bf16 channels of a BF16 row (tail or current token): dot with q / weighted add.
__device__ __forceinline__ void load_bf16_row(const __nv_bfloat16* row, int sub, uint32_t (&w)[16]) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint4 x = ldg128(row + sub * 32 + v * 8);
    w[4 * v + 0] = x.x; w[4 * v + 1] = x.y; w[4 * v + 2] = x.z; w[4 * v + 3] = x.w;
  }
}

struct OnlineState {
  float m;        // running maximum of the scaled logits, log2 domain
  float l;        // sum of probabilities of this lane's tokens (equal in the 4 lanes of a quad)
  float vbias;    // sum of p * (v_min + centre * v_scale) of the lane's channel group
  float acc[32];  // sum of p * v_scale * (code - centre), pair order
};

__device__ __forceinline__ void state_init(OnlineState& s) {
  s.m = -INFINITY;
  s.l = 0.f;
  s.vbias = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) s.acc[i] = 0.f;
}

// Raise the running maximum to at least `mx` (warp-uniform) and rescale the sums.
__device__ __forceinline__ void state_raise(OnlineState& s, float mx) {
  if (mx > s.m) {
    const float r = exp2f(s.m - mx);  // exp2f(-inf) == 0 on the first raise
    s.l *= r;
    s.vbias *= r;
#pragma unroll
    for (int i = 0; i < 32; ++i) s.acc[i] *= r;
    s.m = mx;
  }
}

// Reduce the warp's state over its eight quads and park it in shared memory as
// acc[128] (natural channel order), m, l.
template <int BITS>
__device__ __forceinline__ void state_store(OnlineState& s, int lane, float* dst) {
  const int sub = lane & 3;
#pragma unroll
  for (int i = 0; i < 32; ++i) s.acc[i] = across_quads_sum(s.acc[i]);
  const float vb = across_quads_sum(s.vbias);
  const float l = across_quads_sum(s.l);
  if (lane < 4) {
#pragma unroll
    for (int cc = 0; cc < 32; ++cc) dst[sub * 32 + cc] = s.acc[channel_slot<BITS>(cc)] + vb;
    if (lane == 0) {
      dst[128] = s.m;
      dst[129] = l;
    }
  }
}

// One BF16 row (tail or current token) for every quad of the warp: logits, online softmax, PV.
__device__ __forceinline__ float bf16_words_dot(const uint32_t (&w)[16], int sub, const float* s_qf) {
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    dot = fmaf(bf16_lo(w[i]), s_qf[sub * 32 + 2 * i], dot);
    dot = fmaf(bf16_hi(w[i]), s_qf[sub * 32 + 2 * i + 1], dot);
  }
  return dot;
}
template <int BITS>
__device__ __forceinline__ void bf16_words_accumulate(const uint32_t (&w)[16], float pr, float (&acc)[32]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    acc[channel_slot<BITS>(2 * i)] = fmaf(pr, bf16_lo(w[i]), acc[channel_slot<BITS>(2 * i)]);
    acc[channel_slot<BITS>(2 * i + 1)] = fmaf(pr, bf16_hi(w[i]), acc[channel_slot<BITS>(2 * i + 1)]);
  }
}
template <int BITS>
__device__ __forceinline__ float bf16_row_dot(const __nv_bfloat16* row, int sub, const float* s_qf) {
  uint32_t w[16];
  load_bf16_row(row, sub, w);
  return bf16_words_dot(w, sub, s_qf);
}
template <int BITS>
__device__ __forceinline__ void bf16_row_accumulate(const __nv_bfloat16* row, int sub, float pr,
                                                    float (&acc)[32]) {
  uint32_t w[16];
  load_bf16_row(row, sub, w);
  bf16_words_accumulate<BITS>(w, pr, acc);
}

__device__ __forceinline__ uint32_t smem_u32(const void* ptr) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}

template <int BYTES>
__device__ __forceinline__ void cp_async(uint32_t dst_shared, const void* src_global) {
  if constexpr (BYTES == 16) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_shared), "l"(src_global) : "memory");
  } else {
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst_shared), "l"(src_global), "n"(BYTES)
                 : "memory");
  }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The K table of one metadata group, this lane's four channels 4*lane .. 4*lane+3: w_c = q_c *
// scale_c as float16 in the pair order of unpack_centred (the products are exact in float32, so
// rounding them once in float16 arithmetic gives the same table), stored with one 8-byte write
// per lane after the lanes that hold the two halves of a pair have swapped one register.
template <int BITS>
__device__ __forceinline__ void table_store(__half* table, int lane, __half2 q01, __half2 q23, uint2 scale) {
  constexpr int kPartner = BITS == 4 ? 1 : 2;  // pairs are (c, c + 4) or (c, c + 8)
  const __half2 a = __hmul2(q01, as_half2(scale.x));
  const __half2 b = __hmul2(q23, as_half2(scale.y));
  const bool first = (lane & kPartner) == 0;
  const uint32_t mine_a = as_u32(a), mine_b = as_u32(b);
  const uint32_t got = __shfl_xor_sync(0xffffffffu, first ? mine_b : mine_a, kPartner);
  const uint32_t lo = first ? mine_a : got, hi = first ? got : mine_b;
  uint2 out;
  out.x = __byte_perm(lo, hi, 0x5410);  // (lo.low, hi.low)
  out.y = __byte_perm(lo, hi, 0x7632);  // (lo.high, hi.high)
  int at;  // in halves
  if constexpr (BITS == 4) {
    at = 4 * lane;
  } else {
    // lanes 4a .. 4a+3 hold channels 16a .. 16a+15; lanes 4a and 4a+1 store the pairs of the group's
    // channels 0-3 and 4-7 (pairs 0-3, 4-7), lanes 4a+2 and 4a+3 those of their partners' channels
    // 2-3 and 6-7 joined with their own
    at = 16 * (lane >> 2) + 8 * (lane & 1) + 4 * ((lane >> 1) & 1);
  }
  *reinterpret_cast<uint2*>(table + at) = out;
}


// ------------------------------------------------------------------------------ scratch layout
//
// [0, 256): header, word 0 is the status word (raised when a bounded wait ran out);
// then the per-(b,h) tickets padded to 256 bytes; then kMaxSplits partial slots per (b,h).
// The status word sits at a fixed offset so that it means the same to launches of any batch.

constexpr size_t kWorkspaceHeader = 256;

// Multiprocessors of the current device (looked up once per device).
inline int device_sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

inline size_t tickets_bytes(int64_t batch_heads) { return ((batch_heads * sizeof(int) + 255) / 256) * 256; }

inline size_t workspace_bytes(int64_t batch_heads) {
  return kWorkspaceHeader + tickets_bytes(batch_heads) +
         static_cast<size_t>(batch_heads) * kMaxSplits * kPartialStride * sizeof(float);
}

inline int bind_workspace(ReaderParams& p, const fl_layer* layer, int loop, void* workspace, size_t bytes,
                          const char* who) {
  const int64_t bh = static_cast<int64_t>(layer->batch) * layer->heads;
  const size_t need = workspace_bytes(bh);
  if (workspace == nullptr || bytes < need || !aligned16(workspace)) {
    set_error("%s: workspace of %zu bytes (16-byte aligned) required, got %zu", who, need, bytes);
    return FL_ERR_WORKSPACE;
  }
  p.L = make_view(*layer);
  p.loop = loop;
  p.status = static_cast<int*>(workspace);
  p.tickets = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + kWorkspaceHeader);
  p.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kWorkspaceHeader + tickets_bytes(bh));
  p.max_chunks = kMaxSplits;
  return FL_OK;
}

}  // namespace
}  // namespace fl
