// Decode-attention readers over the packed anchor + delta streams (row layout).
//
//   dense_reader_kernel     one launch: QK^T over streams 0..loop + BF16 tail + current token,
//                           online softmax, PV; persistent CTAs that each own a contiguous,
//                           equally large range of 64-token blocks over all (b,h); partials of a
//                           (b,h) merged by its last-arriving CTA (an atomic ticket, no waiting).
//   selected_reader_kernel  the same over a gathered list of selected logical indices, stream by
//                           stream: cached-mass sparse delta, weighted PV, or plain QK.
//
// Work decomposition: a warp handles eight tokens per step, one per lane quad; lane `sub` of a
// quad owns channels 32*sub .. 32*sub+31 of the token's K row and V row, i.e. one 16-byte
// (4-bit) or 8-byte (2-bit) piece of each packed row.  A 64-byte row is one coalesced 128-bit
// load per lane of the quad, eight rows per warp-wide load instruction.
//
// Dequantisation never leaves registers.  Codes are turned into exact float16 integers with
// the 0x6400 magic-number trick and centred (code - 2^(bits-1)); the per-channel K scale is
// folded into the query once per 64-token group (w_c = q_c * s_c, bias = sum_c q_c * (m_c +
// centre * s_c)), the per-token V scale into the probability (W = p * s).  Products accumulate
// in float16 pairs over at most eight terms (K) or one group (V) and are then widened to
// float32.
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

// CTA-level merge of the warps' states, publication of the partial and, in the last CTA of
// this (b,h), the merge over all partials.  Returns true in the CTA that holds the final
// result: `total` (this thread's channel, un-normalised) and `denom`.
template <int NWARPS>
__device__ __forceinline__ bool merge_and_publish(const ReaderParams& p, float (*s_merge)[kPartialStride],
                                                  int* s_last, int64_t bh, int slot, int nslots,
                                                  float& total, float& denom) {
  const int c = threadIdx.x & (kHeadDim - 1);
  const bool worker = threadIdx.x < kHeadDim;
  __syncthreads();
  float mmax = -INFINITY;
#pragma unroll
  for (int w = 0; w < NWARPS; ++w) mmax = fmaxf(mmax, s_merge[w][128]);
  float a = 0.f, l = 0.f;
#pragma unroll
  for (int w = 0; w < NWARPS; ++w) {
    const float mw = s_merge[w][128];
    const float r = (mw == -INFINITY) ? 0.f : exp2f(mw - mmax);
    a += s_merge[w][c] * r;
    l += s_merge[w][129] * r;
  }
  if (nslots == 1) {
    total = a;
    denom = l;
    return true;
  }
  float* mine = p.partial + (bh * p.max_chunks + slot) * kPartialStride;
  if (worker) mine[c] = a;
  if (threadIdx.x == 0) {
    mine[128] = mmax;
    mine[129] = l;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(p.tickets + bh, 1);
    *s_last = (t == nslots - 1);
    if (t == nslots - 1) p.tickets[bh] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!*s_last) return false;
  __threadfence();
  const float* base = p.partial + bh * p.max_chunks * kPartialStride;
  float gm = -INFINITY;
  for (int j = 0; j < nslots; ++j) gm = fmaxf(gm, __ldcg(base + j * kPartialStride + 128));
  a = 0.f;
  l = 0.f;
  for (int j = 0; j < nslots; ++j) {
    const float mj = __ldcg(base + j * kPartialStride + 128);
    const float r = (mj == -INFINITY) ? 0.f : exp2f(mj - gm);
    a += __ldcg(base + j * kPartialStride + c) * r;
    l += __ldcg(base + j * kPartialStride + 129) * r;
  }
  total = a;
  denom = l;
  return true;
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

// ------------------------------------------------------------------------------ dense reader
//
// Eight warps per CTA; each warp owns whole 64-token blocks of the CTA's work items and runs its
// own two-stage shared-memory ring.  A "unit" is one (block, stream, K|V) piece: for K the 64 packed
// rows (4 KiB at 4 bits) plus the scale/min rows of the one or two 64-row groups they live in,
// for V the 64 records (codes and metadata together, one copy).  Lane 0 of the warp arms the stage's
// mbarrier with the byte count and issues the TMA bulk copies (cp.async.bulk, global ->
// shared); the warp then waits on the barrier's phase, computes from shared memory, and
// re-issues the unit two places ahead into the stage it has just drained.  No CTA-wide
// synchronisation happens until the merge that closes a work item, and waits are bounded: a wait that runs out
// raises the status word in the workspace and the kernel runs to its end.

constexpr int kDenseWarps = 8;
constexpr int kDenseThreads = kDenseWarps * kWarp;
constexpr int kStages = 2;
constexpr int kWaitLimit = 1 << 12;
constexpr uint32_t kSuspendNs = 100000;

template <int BITS>
struct Stage {
  static constexpr int kRowBytes = 16 * BITS;
  static constexpr int kRecord = kRowBytes + 16;     // V record: codes, 8 bytes of metadata, padding
  static constexpr int kCodes = kGroup * kRowBytes;  // K unit: 64 code rows, then ...
  static constexpr int kMeta = 1024;                 // ... the scale/min rows of up to two groups
  static constexpr int kBytes = kCodes + kMeta;      // a V unit is 64 records: the same size
  static_assert(kGroup * kRecord <= kBytes, "a V unit must fit the stage");
};

__device__ __forceinline__ uint32_t smem_u32(const void* ptr) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out.  Each try
// lets the hardware suspend the thread for up to kSuspendNs, so a waiting warp issues almost
// nothing; kWaitLimit tries bound the total wait to a fraction of a second.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < kWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendNs)
        : "memory");
    if (done) return true;
  }
  return false;
}

// Rows [r0, r0 + m) of stream s (relative to the (b,h) row base) that hold the tokens of the
// 64-token block starting at t0.  The rows of one block are consecutive.
struct Span {
  int r0;
  int m;
};
__device__ __forceinline__ Span block_span(const LayerView& L, int s, int b, int t0, int lane) {
  if (s < 2) return Span{t0, kGroup};
  const int32_t* rank = L.rank[s - 2] + L.rank_base[b] + t0;
  const int ra = rank[lane], rb = rank[lane + 32];
  const uint32_t ma = __ballot_sync(0xffffffffu, ra >= 0);
  const uint32_t mb = __ballot_sync(0xffffffffu, rb >= 0);
  const int first_a = __shfl_sync(0xffffffffu, ra, ma ? __ffs(ma) - 1 : 0);
  const int first_b = __shfl_sync(0xffffffffu, rb, mb ? __ffs(mb) - 1 : 0);
  Span sp;
  sp.m = __popc(ma) + __popc(mb);
  sp.r0 = ma ? first_a : (mb ? first_b : 0);
  return sp;
}

// Work is counted in units: a head has one unit per 64-token block of its packed prefix plus
// kTailUnits for its BF16 tail and the current token (about what the tail costs a CTA).  The units
// of all heads form one sequence, head after head, and CTA c owns the contiguous range
// [c*U/G, (c+1)*U/G) of it, so every CTA gets the same amount of work whatever the context
// lengths are.  A work item is the part of one head inside that range: some blocks, the tail, or
// both.  A CTA therefore meets a head once, keeps its online-softmax state in registers across all
// of the head's blocks it owns, and merges and publishes once per item: one to three times in all.
constexpr int kTailUnits = 8;

struct ItemDesc {
  int id;  // -1: past the end of this CTA's range
  int bh, b, quant, tail_len, tail_start;
  int blk_begin, blk_end;  // blocks of the head in this item (may be empty)
  int has_tail;            // the item includes the head's tail and current token
  int part, nparts;        // position of this CTA among the CTAs that share the head, and their number
  int first_cta;           // the first of those CTAs
  int rot;                 // block i of the item goes to warp (i + rot) % 8: the round robin over the
                           // warps runs on across the CTA's items
  int64_t row_base[4];     // first row / first K metadata group of this (b,h) in every stream
  int64_t group_base[4];
};

constexpr int kEachCached = 256;  // sequences whose unit counts the CTA keeps in shared memory

__device__ __forceinline__ int units_per_head(const LayerView& L, int b) {
  return L.seq_state[b * FL_STATE_WORDS + FL_STATE_QUANT_TOKENS] / kGroup + kTailUnits;
}
// `each`: the CTA's shared copy of units_per_head for the first kEachCached sequences
__device__ __forceinline__ int units_per_head(const LayerView& L, const int* each, int b) {
  return b < kEachCached ? each[b] : units_per_head(L, b);
}
__device__ __forceinline__ int64_t total_units(const LayerView& L, const int* each) {
  int64_t total = 0;
  for (int b = 0; b < L.batch; ++b) total += static_cast<int64_t>(L.heads) * units_per_head(L, each, b);
  return total;
}

// Walks the items of one CTA in order.  Held by the one thread that describes them.
struct ItemCursor {
  int64_t at, end;     // next unit, end of the CTA's range
  int64_t head_first;  // first unit of the head that contains `at`
  int b, h, each;      // that head, and the units per head of its sequence
  int count;           // items described so far
  int blocks_done;     // blocks in those items
};

__device__ __forceinline__ void cursor_start(const LayerView& L, const int* each, int64_t lo, int64_t hi,
                                             ItemCursor* c) {
  c->at = lo;
  c->end = hi;
  c->count = 0;
  c->blocks_done = 0;
  c->b = 0;
  c->each = units_per_head(L, each, 0);
  int64_t first = 0;
  while (c->b + 1 < L.batch && lo >= first + static_cast<int64_t>(L.heads) * c->each) {
    first += static_cast<int64_t>(L.heads) * c->each;
    ++c->b;
    c->each = units_per_head(L, each, c->b);
  }
  c->h = static_cast<int>((lo - first) / c->each);
  if (c->h >= L.heads) c->h = L.heads - 1;  // only when the range is empty
  c->head_first = first + static_cast<int64_t>(c->h) * c->each;
}

__device__ __forceinline__ void describe_next(const ReaderParams& p, const int* each, int64_t all_units,
                                              ItemCursor* c, ItemDesc* d) {
  const LayerView& L = p.L;
  if (c->at >= c->end) {
    d->id = -1;
    return;
  }
  const int64_t head_end = c->head_first + c->each;
  const int64_t seg_end = head_end < c->end ? head_end : c->end;
  const int blocks = c->each - kTailUnits;
  const int u0 = static_cast<int>(c->at - c->head_first), u1 = static_cast<int>(seg_end - c->head_first);
  const int bh = c->b * L.heads + c->h;
  const int32_t* st = L.seq_state + c->b * FL_STATE_WORDS;
  d->bh = bh;
  d->b = c->b;
  d->quant = st[FL_STATE_QUANT_TOKENS];
  d->tail_len = st[FL_STATE_TAIL_LEN];
  d->tail_start = st[FL_STATE_TAIL_START];
  d->blk_begin = u0 < blocks ? u0 : blocks;
  d->blk_end = u1 < blocks ? u1 : blocks;
  d->has_tail = u0 <= blocks && blocks < u1;
  // CTA that owns unit u: the largest c with c*U/G <= u
  const int64_t grid = gridDim.x;
  const int64_t first_owner = ((c->head_first + 1) * grid - 1) / all_units;
  const int64_t last_owner = (head_end * grid - 1) / all_units;
  d->part = static_cast<int>(static_cast<int64_t>(blockIdx.x) - first_owner);
  d->nparts = static_cast<int>(last_owner - first_owner + 1);
  d->first_cta = static_cast<int>(first_owner);
  d->rot = c->blocks_done % kDenseWarps;
  c->blocks_done += d->blk_end - d->blk_begin;
  // all loads first, then the stores: one memory latency instead of one per stream
  int64_t rows_at[4], groups_at[4];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const bool on = s <= p.loop;
    rows_at[s] = on ? L.row_base[s][bh] : 0;
    groups_at[s] = on ? L.group_base[s][bh] : 0;
  }
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    d->row_base[s] = rows_at[s];
    d->group_base[s] = groups_at[s];
  }
  d->id = c->count++;
  c->at = seg_end;
  if (seg_end == head_end) {  // on to the next head
    c->head_first = head_end;
    if (++c->h == L.heads) {
      c->h = 0;
      if (c->b + 1 < L.batch) {
        ++c->b;
        c->each = units_per_head(L, each, c->b);
      }
    }
  }
}

// Blocks of an item that belong to the warp in position `warp` of the item's round robin
// (blocks warp, warp + 8, ... of the item).
__device__ __forceinline__ int blocks_of_warp(int blk_begin, int blk_end, int warp) {
  const int n = blk_end - blk_begin - warp;
  return n > 0 ? (n + kDenseWarps - 1) / kDenseWarps : 0;
}

template <int BITS, int LOOP>
__global__ void __launch_bounds__(kDenseThreads, 2)
dense_reader_kernel(const __grid_constant__ ReaderParams p) {
  using St = Stage<BITS>;
  constexpr int kRowBytes = St::kRowBytes;
  constexpr int kLaneBytes = kRowBytes / 4;
  extern __shared__ __align__(128) uint8_t s_ring[];  // [warp][stage][St::kBytes]
  __shared__ __align__(16) float s_qf[2][kHeadDim];
  __shared__ __align__(16) __half s_wtab[kDenseWarps][2][kHeadDim];
  __shared__ __align__(16) float s_merge[2][kDenseWarps][kPartialStride];
  __shared__ __align__(8) uint64_t s_bar[kDenseWarps][kStages];
  __shared__ ItemDesc s_item[4];  // current, next, the one being described, and the one still being merged
  __shared__ ItemCursor s_cursor;
  __shared__ int s_each[kEachCached];
  __shared__ int64_t s_all_units;
  __shared__ int s_last[2];

  const LayerView& L = p.L;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int quad = lane >> 2;
  const int sub = lane & 3;
  // the loop is a template parameter: loops 1 and 2 read streams 0 and 1 only, where every token
  // holds a row, so the paths for compact streams drop out of their kernels
  constexpr int streams = LOOP + 1;
  constexpr int units_per_block = 2 * streams;
  constexpr bool kAllRows = LOOP <= 1;
  uint8_t* ring = s_ring + static_cast<size_t>(warp) * kStages * St::kBytes;

  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < kStages; ++k) mbar_init(smem_u32(&s_bar[warp][k]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // this CTA's contiguous range of units; the one thread that describes the items walks it with a
  // cursor kept in shared memory (registers are allocated for every thread)
  for (int bb = tid; bb < L.batch && bb < kEachCached; bb += kDenseThreads) s_each[bb] = units_per_head(L, bb);
  __syncthreads();
  {
    // Every thread finds the CTA's range and the head it starts in (shared-memory reads only), so
    // that the first query is fetched while one thread describes the first two items.
    const int64_t all_units = total_units(L, s_each);
    ItemCursor cursor;
    cursor_start(L, s_each, all_units * blockIdx.x / gridDim.x, all_units * (blockIdx.x + 1) / gridDim.x, &cursor);
    if (tid == kHeadDim) {
      s_all_units = all_units;
      s_cursor = cursor;
      describe_next(p, s_each, all_units, &s_cursor, &s_item[0]);
      describe_next(p, s_each, all_units, &s_cursor, &s_item[1]);
    } else if (tid < kHeadDim && cursor.at < cursor.end) {
      const int64_t first_bh = static_cast<int64_t>(cursor.b) * L.heads + cursor.h;
      s_qf[0][tid] = __bfloat162float(p.q[first_bh * kHeadDim + tid]);
    }
  }
  __syncthreads();

  // Per-warp pipeline counters: units issued / consumed since the kernel started.  Unit g lives
  // in stage g % kStages and completes that stage's phase (g / kStages) & 1.
  uint32_t issued = 0, consumed = 0;
  // Issue cursor: item sequence number, block index within my blocks of that item, unit in block.
  int iss_item = 0, iss_blk = 0, iss_j = 0;
  bool timed_out = false;

  OnlineState S;
  state_init(S);

  for (int k = 0;; ++k) {
    const ItemDesc* curp = &s_item[k % 4];
    if (curp->id < 0) break;
    struct {
      int bh, b, blk_begin, blk_end, has_tail, rot;
    } cur = {curp->bh, curp->b, curp->blk_begin, curp->blk_end, curp->has_tail, curp->rot};
    // (the fields that only the tail and the merge need are read from curp there: its slot is not
    // rewritten before the merge of the item after this one has begun)
    // Look ahead: one thread of the upper half of the CTA (the warps that sit out the merge)
    // describes item k+2, the upper half fetches the query of item k+1.  Both become visible to the
    // other warps at this item's closing barrier.
    if (tid == kHeadDim) describe_next(p, s_each, s_all_units, &s_cursor, &s_item[(k + 2) % 4]);
    if (tid >= kHeadDim) {
      const int next_id = s_item[(k + 1) % 4].id;
      if (next_id >= 0) {
        s_qf[(k + 1) & 1][tid - kHeadDim] = __bfloat162float(
            p.q[static_cast<int64_t>(s_item[(k + 1) % 4].bh) * kHeadDim + tid - kHeadDim]);
      }
    }
    const int64_t bh = cur.bh;
    const int b = cur.b;
    const float* qf = s_qf[k & 1];
    float* logits_row = p.logits ? p.logits + bh * p.logits_stride : nullptr;

    if (cur.blk_end > cur.blk_begin) {
      const int my_first = cur.blk_begin + ((warp - cur.rot) & (kDenseWarps - 1));
      const int my_blocks = blocks_of_warp(cur.blk_begin, cur.blk_end, my_first - cur.blk_begin);
      float lg[8];
      __half2 hacc[16];
      __half2 hbias = __floats2half2_rn(0.f, 0.f);  // sum of p * (v_min + centre * v_scale) of one block
      for (int cb = 0; cb < my_blocks; ++cb) {
        const int blk = my_first + cb * kDenseWarps;
        const int t0 = blk * kGroup;
        for (int j = 0; j < units_per_block; ++j) {
          // ---- keep the ring full: issue units of this item, then of the next one
          while (issued - consumed < static_cast<uint32_t>(kStages)) {
            if (iss_item > k + 1) break;
            const ItemDesc* it = &s_item[iss_item % 4];
            if (it->id < 0) break;
            const int it_pos = (warp - it->rot) & (kDenseWarps - 1);
            const int it_blocks = blocks_of_warp(it->blk_begin, it->blk_end, it_pos);
            if (iss_blk >= it_blocks) {
              ++iss_item;
              iss_blk = 0;
              iss_j = 0;
              continue;
            }
            const int iblk = it->blk_begin + it_pos + iss_blk * kDenseWarps;
            const bool iv = iss_j >= streams;
            const int is = iv ? iss_j - streams : iss_j;
            const Span sp = kAllRows ? Span{iblk * kGroup, kGroup} : block_span(L, is, it->b, iblk * kGroup, lane);
            if (lane == 0) {
              const uint32_t stage_index = issued % kStages;
              const uint32_t bar = smem_u32(&s_bar[warp][stage_index]);
              const uint32_t dst = smem_u32(ring + stage_index * St::kBytes);
              if (sp.m == 0) {
                mbar_arrive(bar);
              } else {
                const int64_t row = it->row_base[is] + sp.r0;
                const uint32_t code_bytes = static_cast<uint32_t>(sp.m) * kRowBytes;
                if (!iv) {
                  const int g0 = sp.r0 >> 6, g1 = (sp.r0 + sp.m - 1) >> 6;
                  const int64_t grp = it->group_base[is] + g0;
                  const uint32_t ng = g1 - g0 + 1;
                  mbar_arrive_expect_tx(bar, code_bytes + ng * 512u);
                  bulk_copy_g2s(dst, L.k_codes[is] + row * kRowBytes, code_bytes, bar);
                  for (uint32_t gi = 0; gi < ng; ++gi) {
                    bulk_copy_g2s(dst + St::kCodes + gi * 512u, L.k_scale[is] + (grp + gi) * kHeadDim, 256u, bar);
                    bulk_copy_g2s(dst + St::kCodes + gi * 512u + 256u, L.k_min[is] + (grp + gi) * kHeadDim, 256u,
                                  bar);
                  }
                } else {
                  const uint32_t record_bytes = static_cast<uint32_t>(sp.m) * St::kRecord;
                  mbar_arrive_expect_tx(bar, record_bytes);
                  bulk_copy_g2s(dst, L.v_rows[is] + row * St::kRecord, record_bytes, bar);
                }
              }
            }
            ++issued;
            if (++iss_j == units_per_block) {
              iss_j = 0;
              ++iss_blk;
            }
          }

          // ---- consume unit (blk, j)
          const bool is_v = j >= streams;
          const int s = is_v ? j - streams : j;
          const uint32_t stage_index = consumed % kStages;
          const uint8_t* stage = ring + stage_index * St::kBytes;
          if (!mbar_wait(smem_u32(&s_bar[warp][stage_index]), (consumed / kStages) & 1u)) timed_out = true;
          const Span sp = kAllRows ? Span{t0, kGroup} : block_span(L, s, b, t0, lane);
          const int32_t* rank = s >= 2 ? L.rank[s - 2] + L.rank_base[b] + t0 : nullptr;
        const int g0 = sp.r0 >> 6;
        const int ng = kAllRows ? 1 : (sp.m > 0 ? ((sp.r0 + sp.m - 1) >> 6) - g0 + 1 : 0);
        // A block whose 64 tokens are all present in one metadata group (always true for streams
        // 0 and 1) takes the branch-free path: row i of the stage is token i.
        const bool full = kAllRows || (sp.m == kGroup && ng == 1);
        if (!is_v) {
          if (s == 0) {
  #pragma unroll
            for (int it = 0; it < 8; ++it) lg[it] = 0.f;
          }
          // w_c = q_c * scale_c and bias = sum_c q_c * (min_c + centre * scale_c) per group
          float kbias0 = 0.f, kbias1 = 0.f;
          for (int gi = 0; gi < ng; ++gi) {
            const uint2 sc = *reinterpret_cast<const uint2*>(stage + St::kCodes + gi * 512 + lane * 8);
            const uint2 mn = *reinterpret_cast<const uint2*>(stage + St::kCodes + gi * 512 + 256 + lane * 8);
            const float2 sc01 = __half22float2(as_half2(sc.x)), sc23 = __half22float2(as_half2(sc.y));
            const float2 mn01 = __half22float2(as_half2(mn.x)), mn23 = __half22float2(as_half2(mn.y));
            const float4 q4 = *reinterpret_cast<const float4*>(&qf[4 * lane]);
            const float kc = float(kCentre<BITS>);
            float bias = q4.x * fmaf(kc, sc01.x, mn01.x);
            bias = fmaf(q4.y, fmaf(kc, sc01.y, mn01.y), bias);
            bias = fmaf(q4.z, fmaf(kc, sc23.x, mn23.x), bias);
            bias = fmaf(q4.w, fmaf(kc, sc23.y, mn23.y), bias);
            __half* tab = &s_wtab[warp][gi][(4 * lane) & ~31];
            const int cc = (4 * lane) & 31;
            tab[channel_slot<BITS>(cc + 0)] = __float2half_rn(q4.x * sc01.x);
            tab[channel_slot<BITS>(cc + 1)] = __float2half_rn(q4.y * sc01.y);
            tab[channel_slot<BITS>(cc + 2)] = __float2half_rn(q4.z * sc23.x);
            tab[channel_slot<BITS>(cc + 3)] = __float2half_rn(q4.w * sc23.y);
            bias = 0.25f * warp_sum(bias);
            if (gi == 0) kbias0 = bias; else kbias1 = bias;
          }
          __syncwarp();
          if (full) {
            __half2 mult[16];
            const uint4* src = reinterpret_cast<const uint4*>(&s_wtab[warp][0][sub * 32]);
  #pragma unroll
            for (int v = 0; v < 4; ++v) {
              const uint4 x = src[v];
              mult[4 * v + 0] = as_half2(x.x); mult[4 * v + 1] = as_half2(x.y);
              mult[4 * v + 2] = as_half2(x.z); mult[4 * v + 3] = as_half2(x.w);
            }
            const uint8_t* piece = stage + quad * kRowBytes + sub * kLaneBytes;
            Codes<BITS> c[8];
  #pragma unroll
            for (int it = 0; it < 8; ++it) c[it] = load_codes_shared<BITS>(piece + it * 8 * kRowBytes);
  #pragma unroll
            for (int it = 0; it < 8; ++it) lg[it] += k_dot_fast<BITS>(c[it], mult) + kbias0;
          } else if (sp.m > 0) {
  #pragma unroll 1
            for (int it = 0; it < 8; ++it) {
              const int r = rank[it * 8 + quad];
              const float add = 0.f;
              if (r >= 0) {
                const int gi = (r >> 6) - g0;
                __half2 mult[16];
                const uint4* src = reinterpret_cast<const uint4*>(&s_wtab[warp][gi][sub * 32]);
  #pragma unroll
                for (int v = 0; v < 4; ++v) {
                  const uint4 x = src[v];
                  mult[4 * v + 0] = as_half2(x.x); mult[4 * v + 1] = as_half2(x.y);
                  mult[4 * v + 2] = as_half2(x.z); mult[4 * v + 3] = as_half2(x.w);
                }
                const Codes<BITS> c =
                    load_codes_shared<BITS>(stage + (r - sp.r0) * kRowBytes + sub * kLaneBytes);
                const float dot = k_dot_fast<BITS>(c, mult) + (gi == 0 ? kbias0 : kbias1);
  #pragma unroll
                for (int k = 0; k < 8; ++k) lg[k] += (k == it) ? dot : add;
              }
            }
          }
          if (s == LOOP) {
            // all streams summed: logits -> probabilities of my eight tokens
            float mx = -INFINITY;
  #pragma unroll
            for (int it = 0; it < 8; ++it) {
              const float raw = quad_sum(lg[it]);
              if (logits_row && sub == 0) logits_row[t0 + it * 8 + quad] = raw * p.scaling;
              lg[it] = raw * p.scaling_log2;
              mx = fmaxf(mx, lg[it]);
            }
            state_raise(S, across_quads_max(mx));
  #pragma unroll
            for (int it = 0; it < 8; ++it) {
              lg[it] = exp2f(lg[it] - S.m);
              S.l += lg[it];
            }
  #pragma unroll
            for (int i = 0; i < 16; ++i) hacc[i] = __floats2half2_rn(0.f, 0.f);
          }
        } else {
          const uint8_t* meta = stage + kRowBytes;  // of record 0
          // my channel group's minimum / scale, duplicated into both halves
          const uint32_t pick = (sub < 2) ? 0x1010u : 0x3232u;
          const __half2 centre2 = __floats2half2_rn(float(kCentre<BITS>), float(kCentre<BITS>));
          if (full) {
            const uint8_t* piece = stage + quad * St::kRecord + sub * kLaneBytes;
  #pragma unroll
            for (int half_block = 0; half_block < 2; ++half_block) {
              Codes<BITS> c[4];
              uint2 mt[4];
  #pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int it = half_block * 4 + k;
                c[k] = load_codes_shared<BITS>(piece + it * 8 * St::kRecord);
                mt[k] = *reinterpret_cast<const uint2*>(meta + (it * 8 + quad) * St::kRecord);
              }
  #pragma unroll
              for (int k = 0; k < 4; ++k) {
                const __half2 vm2 = as_half2(__byte_perm(mt[k].x, 0u, pick));
                const __half2 vs2 = as_half2(__byte_perm(mt[k].y, 0u, pick));
                const __half2 p2 = __float2half2_rn(lg[half_block * 4 + k]);
                hbias = __hfma2(p2, __hfma2(centre2, vs2, vm2), hbias);
                v_accumulate<BITS>(c[k], __hmul2(p2, vs2), hacc);
              }
            }
          } else if (sp.m > 0) {
  #pragma unroll 1
            for (int it = 0; it < 8; ++it) {
              const int r = rank[it * 8 + quad];
              if (r >= 0) {
                const int ri = r - sp.r0;
                float pr = 0.f;
  #pragma unroll
                for (int k = 0; k < 8; ++k) pr = (k == it) ? lg[k] : pr;
                const Codes<BITS> c = load_codes_shared<BITS>(stage + ri * St::kRecord + sub * kLaneBytes);
                const uint2 mt = *reinterpret_cast<const uint2*>(meta + ri * St::kRecord);
                const __half2 vm2 = as_half2(__byte_perm(mt.x, 0u, pick));
                const __half2 vs2 = as_half2(__byte_perm(mt.y, 0u, pick));
                const __half2 p2 = __float2half2_rn(pr);
                hbias = __hfma2(p2, __hfma2(centre2, vs2, vm2), hbias);
                v_accumulate<BITS>(c, __hmul2(p2, vs2), hacc);
              }
            }
          }
          if (s == LOOP) {
            flush_pairs(hacc, S.acc);
            S.vbias += __low2float(hbias);
            hbias = __floats2half2_rn(0.f, 0.f);
          }
        }
          __syncwarp();
          ++consumed;
        }
      }
    }
    // Every unit of this item has been issued: park the issue cursor on the next item, so that
    // it never looks at the descriptor slot thread 0 is about to overwrite.
    if (iss_item <= k) {
      iss_item = k + 1;
      iss_blk = 0;
      iss_j = 0;
    }
    if (cur.has_tail) {
      // ---- the BF16 tail and the current token: entries 0..tail_len (the last is the current),
      // one per lane quad; the V row is fetched together with the K row
      const int entries = curp->tail_len + 1;
      const __nv_bfloat16* tk = L.tail_k[LOOP] + bh * L.tail_capacity * kHeadDim;
      const __nv_bfloat16* tv = L.tail_v[LOOP] + bh * L.tail_capacity * kHeadDim;
      for (int e0 = warp * 8; e0 < entries; e0 += kDenseWarps * 8) {
        const int e = e0 + quad;
        const bool ok = e < entries;
        const int slot = (curp->tail_start + e) % L.tail_capacity;
        const __nv_bfloat16* krow = (e == curp->tail_len) ? p.kcur + bh * kHeadDim : tk + slot * kHeadDim;
        const __nv_bfloat16* vrow = (e == curp->tail_len) ? p.vcur + bh * kHeadDim : tv + slot * kHeadDim;
        uint32_t kw[16], vw[16];
        if (ok) {
          load_bf16_row(krow, sub, kw);
          load_bf16_row(vrow, sub, vw);
        }
        float dot = 0.f;
        if (ok) dot = bf16_words_dot(kw, sub, qf);
        dot = quad_sum(dot);
        if (ok && logits_row && sub == 0) logits_row[curp->quant + e] = dot * p.scaling;
        const float x = ok ? dot * p.scaling_log2 : -INFINITY;
        state_raise(S, across_quads_max(x));
        const float pr = ok ? exp2f(x - S.m) : 0.f;
        S.l += pr;
        if (ok) bf16_words_accumulate<BITS>(vw, pr, S.acc);
      }
    }

    // ---- merge the eight warps' states, publish this CTA's partial of the head, finish the head
    // if every CTA that shares it has published
    const int buf = k & 1;
    state_store<BITS>(S, lane, s_merge[buf][warp]);
    state_init(S);
    __syncthreads();
    if (warp < 4) {
      const int c = tid;
      float mmax = -INFINITY;
#pragma unroll
      for (int w = 0; w < kDenseWarps; ++w) mmax = fmaxf(mmax, s_merge[buf][w][128]);
      float a = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < kDenseWarps; ++w) {
        const float mw = s_merge[buf][w][128];
        const float r = (mw == -INFINITY) ? 0.f : exp2f(mw - mmax);
        a += s_merge[buf][w][c] * r;
        l += s_merge[buf][w][129] * r;
      }
      const int nparts = curp->nparts;
      if (nparts == 1) {
        p.out[bh * kHeadDim + c] = a / l;
      } else {
        // Two partial slots per CTA: only a CTA's first item can continue a head from the CTA
        // before (slot 0) and only its last item can leave a head to the CTA after (slot 1).
        float* mine = p.partial + (2 * blockIdx.x + (curp->part > 0 ? 0 : 1)) * kPartialStride;
        mine[c] = a;
        if (c == 0) {
          mine[128] = mmax;
          mine[129] = l;
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (c == 0) {
          const int t = atomicAdd(p.tickets + bh, 1);
          s_last[buf] = (t == nparts - 1);
          if (t == nparts - 1) p.tickets[bh] = 0;  // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_last[buf]) {
          __threadfence();
          const float* base = p.partial + (2 * curp->first_cta + 1) * kPartialStride;
          const auto part_of = [&](int jj) { return base + (jj > 0 ? (2 * jj - 1) * kPartialStride : 0); };
          float gm = -INFINITY;
          for (int jj = 0; jj < nparts; ++jj) gm = fmaxf(gm, __ldcg(part_of(jj) + 128));
          a = 0.f;
          l = 0.f;
          for (int jj = 0; jj < nparts; ++jj) {
            const float* pj = part_of(jj);
            const float mj = __ldcg(pj + 128);
            const float r = (mj == -INFINITY) ? 0.f : exp2f(mj - gm);
            a += __ldcg(pj + c) * r;
            l += __ldcg(pj + 129) * r;
          }
          p.out[bh * kHeadDim + c] = a / l;
        }
      }
    }
  }

  if (timed_out && lane == 0) atomicExch(p.status, 1);
}

// ------------------------------------------------------------------------------ selected readers
//
// Stream-major gather.  A selected token owns a row in streams 0 and 1 and, where the token was
// retained, in the compact streams 2 and 3, so a token-major walk would run every stream for all
// eight tokens of a pass whenever one of them holds a compact row.  Here every stream is packed
// by itself instead.  A CTA stages a batch of slots (one per thread), builds per stream the list
// of the slots that hold a row there, and cuts the work into passes of at most eight rows of ONE
// stream:
//
//   K pass: up to eight rows of one stream that share a K metadata group (for the compact
//           streams that is a group of 64 compact rows, about 256 tokens wide, so their passes
//           are as full as those of streams 0 and 1).  The warp builds the group's query-folded
//           table (w_c = q_c * scale_c in float16, bias in float32) as the dense reader does and
//           writes one partial logit per row to shared memory.
//   softmax: after a CTA barrier every thread sums the partial logits of its slot over the
//           streams in a fixed order; the batch maximum raises the CTA's running maximum (online
//           softmax at batch granularity) and the probability goes to shared memory.
//   V pass: any eight records of one stream: p * v_scale * (code - centre) into the warp's
//           float16-pair accumulators, widened every sixteen passes.
//
// The passes of a warp are independent of each other, so each warp runs them through a private
// ring of kDepth shared-memory stages filled by 16-byte cp.async copies that every lane issues
// for the pieces it will read itself; the V passes of a batch are already on their way while the
// CTA is still in the softmax barrier.  Tail tokens and the current token (BF16 rows) are passes
// of their own that read global memory directly.
//
// Indices need not be sorted for correctness (an unsorted list only makes more, shorter K passes).

enum { kModeDelta = 0, kModePV = 1, kModeQK = 2 };
constexpr int kGatherWarps = 8;
constexpr int kGatherThreads = kGatherWarps * kWarp;
constexpr int kSlotBatch = kGatherThreads;  // slots staged per round: one per thread
constexpr int kDepth = 4;                   // passes in flight per warp
constexpr int kPassBytes = 1024;            // K: 8 rows (<= 512 B) + one metadata group (512 B); V: 8 records (<= 640 B)
constexpr int kTailClass = 4;               // list of the slots that are tail tokens or the current token
constexpr int kGatherCtasPerSm = 2;
static_assert(kGatherWarps * kDepth * kPassBytes >= kGatherWarps * kPartialStride * 4,
              "the merge buffer reuses the rings");

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
    at = 16 * (lane >> 2) + 8 * ((lane >> 1) & 1) + 4 * (lane & 1);
  }
  *reinterpret_cast<uint2*>(table + at) = out;
}

// The rows to read form one list per batch: the entries of stream 0 in slot order, then those of
// stream 1, 2 and 3.  An entry is (stream << 30) | row, so a stream holds fewer than 2^30 rows
// over all (b,h) pairs.  A V pass is any eight consecutive entries; a K pass is described by 16
// bits: first entry in bits 0..9, rows - 1 in bits 10..12.
constexpr int kMaxEntries = 4 * kSlotBatch;

// STREAMS = loop + 1 is a template parameter, so that the staging of a batch touches only the
// streams the loop reads.
template <int BITS, int MODE, int STREAMS>
__global__ void __launch_bounds__(kGatherThreads, kGatherCtasPerSm)
selected_reader_kernel(const __grid_constant__ ReaderParams p) {
  constexpr int kRowBytes = 16 * BITS;
  constexpr int kRecord = kRowBytes + 16;
  constexpr int kLaneBytes = kRowBytes / 4;
  constexpr uint32_t kFull = 0xffffffffu;
  extern __shared__ __align__(128) uint8_t s_ring[];  // [warp][stage][kPassBytes]
  __shared__ __align__(16) float s_qf[kHeadDim];
  __shared__ __align__(16) __half s_wtab[kGatherWarps][kHeadDim];  // the current K pass's table
  __shared__ uint32_t s_entry[kMaxEntries];
  __shared__ float s_eval[kMaxEntries];     // per entry: its partial logit, then its probability (or weight)
  __shared__ uint16_t s_kdesc[kMaxEntries];
  __shared__ int s_kgroup[kMaxEntries];     // per K pass: its metadata group, counted over all (b,h)
  __shared__ int s_tail[kSlotBatch];        // tail class: ring slot of the entry, -1 = the current token
  __shared__ float s_tval[kSlotBatch];      // ... and its logit, then probability
  __shared__ int s_wcount[5][kGatherWarps], s_woff[5][kGatherWarps];
  __shared__ int s_whead[4][kGatherWarps], s_wfirst[4][kGatherWarps];
  __shared__ int s_count[5], s_ebase[5];    // entries per class; first entry of every stream, then the total
  __shared__ int s_nk_packed;
  __shared__ int s_rbase[4], s_gbase[4];    // first row / first K metadata group of this (b,h) in every stream
  __shared__ const uint8_t* s_kptr[4];
  __shared__ const uint8_t* s_vptr[4];
  __shared__ float s_red[kGatherWarps];
  __shared__ int s_last;

  const LayerView& L = p.L;
  const int64_t bh = blockIdx.y;
  const int b = static_cast<int>(bh / L.heads);
  const int32_t* st = L.seq_state + b * FL_STATE_WORDS;
  const int quant = st[FL_STATE_QUANT_TOKENS];
  const int tail_len = st[FL_STATE_TAIL_LEN];
  const int tail_start = st[FL_STATE_TAIL_START];
  const int cur_pos = quant + tail_len;
  const int nsplits = (p.capacity + p.slots_per_cta - 1) / p.slots_per_cta;
  const int split = blockIdx.x;
  const int slot_begin = split * p.slots_per_cta;
  const int slot_end = min(p.capacity, slot_begin + p.slots_per_cta);
  constexpr int streams = STREAMS;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int quad = lane >> 2;
  const int sub = lane & 3;
  const uint32_t lanes_below = (1u << lane) - 1u;
  uint8_t* const my_ring = s_ring + warp * kDepth * kPassBytes;
  const uint32_t my_ring_u32 = smem_u32(my_ring);
  const int codes_at = quad * kRowBytes + sub * kLaneBytes;  // this lane's codes within a stage
  float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);                // query channels 4*lane .. 4*lane+3
  __half2 q01 = __floats2half2_rn(0.f, 0.f), q23 = q01;
  if constexpr (MODE != kModePV) {
    if (tid < kHeadDim) s_qf[tid] = __bfloat162float(p.q[bh * kHeadDim + tid]);
    const uint2 raw = ldg64(p.q + bh * kHeadDim + 4 * lane);
    q4 = make_float4(bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y));
    q01 = __floats2half2_rn(q4.x, q4.y);
    q23 = __floats2half2_rn(q4.z, q4.w);
  }
  if (tid < 4) {
    const bool have = tid < streams;
    s_rbase[tid] = have ? static_cast<int>(L.row_base[tid][bh]) : 0;
    s_gbase[tid] = have ? static_cast<int>(L.group_base[tid][bh]) : 0;
    s_kptr[tid] = have ? L.k_codes[tid] : nullptr;
    s_vptr[tid] = have ? L.v_rows[tid] : nullptr;
  }

  OnlineState S;
  state_init(S);
  float m_run = MODE == kModePV ? 0.f : -INFINITY;  // the CTA's running maximum (uniform)
  float l_mine = 0.f;                                // sum of the probabilities of this thread's slots
  const int32_t* idx_row = p.indices + bh * p.capacity;
  const uint8_t* valid_row = p.valid ? p.valid + bh * p.capacity : nullptr;
  const __nv_bfloat16* tk = L.tail_k[p.loop] + bh * L.tail_capacity * kHeadDim;
  const __nv_bfloat16* tv = L.tail_v[p.loop] + bh * L.tail_capacity * kHeadDim;
  __half2 hacc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) hacc[i] = __floats2half2_rn(0.f, 0.f);
  int v_passes = 0;

  // equal batches: 410 slots are staged as 205 + 205, not 256 + 154
  const int n_batches = (slot_end - slot_begin + kSlotBatch - 1) / kSlotBatch;
  const int batch_size = n_batches > 0 ? (slot_end - slot_begin + n_batches - 1) / n_batches : kSlotBatch;
  for (int batch_begin = slot_begin; batch_begin < slot_end; batch_begin += batch_size) {
    const int batch_n = min(batch_size, slot_end - batch_begin);
    __syncthreads();  // the previous round's lists and rings are no longer read (and the bases are written)
    // ---- stage this round's slots: index, the row in every stream, class
    int idx = -1;
    bool live = false;    // the slot has something to read
    uint32_t member = 0;  // bit c: the slot is on list c
    int rows[5] = {-1, -1, -1, -1, -1};
    float weight = 0.f;
    if (tid < batch_n) {
      const int j = batch_begin + tid;
      if constexpr (MODE == kModePV) weight = p.weights[bh * p.capacity + j];
      if (!valid_row || valid_row[j]) idx = idx_row[j];
      if (idx >= 0 && idx < quant) {
        live = true;
        rows[0] = idx;
        if (streams >= 2) rows[1] = idx;
        if (streams >= 3) rows[2] = L.rank[0][L.rank_base[b] + idx];
        if (streams >= 4) rows[3] = L.rank[1][L.rank_base[b] + idx];
      } else if (idx >= quant) {
        const bool has_current = (MODE == kModePV) ? p.vcur != nullptr : p.kcur != nullptr;
        if (idx - quant < tail_len) {
          live = true;
          member = 1u << kTailClass;
          rows[4] = (tail_start + idx - quant) % L.tail_capacity;
        } else if (idx == cur_pos && has_current) {
          live = true;
          member = 1u << kTailClass;
        }
      }
      if constexpr (MODE == kModeQK) {
        if (!live) p.logits[bh * p.capacity + j] = 0.f;
      }
    }
#pragma unroll
    for (int s = 0; s < STREAMS; ++s) member |= rows[s] >= 0 ? 1u << s : 0u;
    // ---- the entry lists: every class in slot order, streams 0..3 back to back
    int at[5];  // my entry in every class I am a member of
#pragma unroll
    for (int c = 0; c < 5; ++c) {
      if (c >= STREAMS && c != kTailClass) continue;
      const uint32_t mask = __ballot_sync(kFull, (member >> c) & 1u);
      at[c] = __popc(mask & lanes_below);
      if (lane == 0) s_wcount[c][warp] = __popc(mask);
    }
    __syncthreads();
    if (warp == 0) {  // running entry counts over (stream, warp)
      const int mine = (lane >> 3) < STREAMS ? s_wcount[lane >> 3][lane & 7] : 0;
      int incl = mine;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(kFull, incl, d);
        if (lane >= d) incl += up;
      }
      const int stream_first = __shfl_sync(kFull, incl - mine, lane & ~7);
      s_woff[lane >> 3][lane & 7] = incl - mine;
      if ((lane & 7) == 0) s_ebase[lane >> 3] = stream_first;
      if ((lane & 7) == 7) s_count[lane >> 3] = incl - stream_first;
      if (lane == 31) s_ebase[4] = incl;
    } else if (warp == 1 && lane < kGatherWarps) {
      int off = 0;
      for (int k = 0; k < lane; ++k) off += s_wcount[kTailClass][k];
      s_woff[kTailClass][lane] = off;
      if (lane == kGatherWarps - 1) s_count[kTailClass] = off + s_wcount[kTailClass][lane];
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 5; ++c) {
      if (c >= STREAMS && c != kTailClass) continue;
      at[c] += s_woff[c][warp];
      if ((member >> c) & 1u) {
        if (c < 4) {
          s_entry[at[c]] = (static_cast<uint32_t>(c) << 30) | static_cast<uint32_t>(s_rbase[c] + rows[c]);
          s_eval[at[c]] = weight;  // the weighted-PV reader's probabilities are the caller's
        } else {
          s_tail[at[c]] = rows[4];
          s_tval[at[c]] = weight;
        }
      }
    }
    __syncthreads();
    const int n_entries = s_ebase[4];
    const int n_tail = s_count[kTailClass];
    // ---- K passes: entry i of a stream opens a pass where the metadata group changes and every
    // eight entries after that
    if constexpr (MODE != kModePV) {
      uint32_t run_heads[4];
      bool entry_on[4], run_head[4];
      int group_of[4];
#pragma unroll
      for (int s = 0; s < STREAMS; ++s) {
        entry_on[s] = tid < s_count[s];
        const int first = s_ebase[s];
        const int base = s_rbase[s];
        group_of[s] = entry_on[s] ? (static_cast<int>(s_entry[first + tid] & 0x3fffffffu) - base) >> 6 : -1;
        const int before =
            entry_on[s] && tid > 0 ? (static_cast<int>(s_entry[first + tid - 1] & 0x3fffffffu) - base) >> 6 : -1;
        run_head[s] = entry_on[s] && (tid == 0 || group_of[s] != before);
        run_heads[s] = __ballot_sync(kFull, run_head[s]);
        if (lane == 0) s_whead[s][warp] = run_heads[s] ? warp * 32 + 31 - __clz(run_heads[s]) : -1;
      }
      __syncthreads();
      bool pass_head[4];
      uint32_t pass_heads[4];
      int rank[4];
#pragma unroll
      for (int s = 0; s < STREAMS; ++s) {
        int run_start = 0;
        const uint32_t upto = run_heads[s] & (lanes_below | (1u << lane));
        if (upto) {
          run_start = warp * 32 + 31 - __clz(upto);
        } else {
          for (int w = warp - 1; w >= 0; --w) {
            const int h = s_whead[s][w];
            if (h >= 0) {
              run_start = h;
              break;
            }
          }
        }
        pass_head[s] = entry_on[s] && (run_head[s] || ((tid - run_start) & 7) == 0);
        pass_heads[s] = __ballot_sync(kFull, pass_head[s]);
        rank[s] = __popc(pass_heads[s] & lanes_below);
        if (lane == 0) {
          s_wcount[s][warp] = __popc(pass_heads[s]);
          s_wfirst[s][warp] = pass_heads[s] ? warp * 32 + __ffs(pass_heads[s]) - 1 : -1;
        }
      }
      __syncthreads();
      if (warp == 0) {  // running pass counts over (stream, warp)
        const int mine = (lane >> 3) < STREAMS ? s_wcount[lane >> 3][lane & 7] : 0;
        int incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int up = __shfl_up_sync(kFull, incl, d);
          if (lane >= d) incl += up;
        }
        s_woff[lane >> 3][lane & 7] = incl - mine;
        if (lane == 31) s_nk_packed = incl;
      }
      __syncthreads();
#pragma unroll
      for (int s = 0; s < STREAMS; ++s) {
        if (pass_head[s]) {
          int next = s_count[s];
          const uint32_t above = pass_heads[s] & ~(lanes_below | (1u << lane));
          if (above) {
            next = warp * 32 + __ffs(above) - 1;
          } else {
            for (int w = warp + 1; w < kGatherWarps; ++w) {
              const int h = s_wfirst[s][w];
              if (h >= 0) {
                next = h;
                break;
              }
            }
          }
          const int k = s_woff[s][warp] + rank[s];
          s_kdesc[k] = static_cast<uint16_t>((s_ebase[s] + tid) | ((next - tid - 1) << 10));
          s_kgroup[k] = s_gbase[s] + group_of[s];
        }
      }
      __syncthreads();
    }

    // ---- this warp's passes: K passes warp, warp + 8, ..., then V passes warp, warp + 8, ...
    const int nk_all = MODE == kModePV ? 0 : s_nk_packed;
    const int nv_all = MODE == kModeQK ? 0 : (n_entries + 7) >> 3;
    const int nk_mine = nk_all > warp ? (nk_all - warp + kGatherWarps - 1) / kGatherWarps : 0;
    const int nv_mine = nv_all > warp ? (nv_all - warp + kGatherWarps - 1) / kGatherWarps : 0;
    const int n_mine = nk_mine + nv_mine;
    // Copies of pass q into its stage (one commit group, empty past the end): codes of row i at
    // i * kRowBytes; behind them the K metadata group (scale[128], min[128]) or the V records' 16
    // metadata bytes (record i at 512 + 16 i).
    auto issue = [&](int q) {
      const uint32_t stage = my_ring_u32 + (q & (kDepth - 1)) * kPassBytes;
      if (q < nk_mine) {
        if constexpr (MODE != kModePV) {
          const int k = warp + kGatherWarps * q;
          const uint32_t d = s_kdesc[k];
          const int s = s_entry[d & 1023u] >> 30;
          if (quad <= static_cast<int>(d >> 10)) {
            const uint32_t row = s_entry[(d & 1023u) + quad] & 0x3fffffffu;
            cp_async<kLaneBytes>(stage + codes_at, s_kptr[s] + static_cast<uint64_t>(row) * kRowBytes + sub * kLaneBytes);
          }
          const __half* meta = (lane < 16 ? L.k_scale[s] : L.k_min[s]) +
                               static_cast<int64_t>(s_kgroup[k]) * kHeadDim + (lane & 15) * 8;
          cp_async<16>(stage + 512 + lane * 16, meta);
        }
      } else if (q < n_mine) {
        if constexpr (MODE != kModeQK) {
          const int i = 8 * (warp + kGatherWarps * (q - nk_mine)) + quad;
          if (i < n_entries) {
            const uint32_t e = s_entry[i];
            const uint8_t* record = s_vptr[e >> 30] + static_cast<uint64_t>(e & 0x3fffffffu) * kRecord;
            cp_async<kLaneBytes>(stage + codes_at, record + sub * kLaneBytes);
            if (sub == 0) cp_async<16>(stage + 512 + quad * 16, record + kRowBytes);
          }
        }
      }
      cp_async_commit();
    };
    auto advance = [&](int q) {
      cp_async_wait<kDepth - 2>();  // pass q has landed
      __syncwarp();                 // ... for every lane, and every lane is done with pass q - 1
      issue(q + kDepth - 1);        // into the stage of pass q - 1
    };

#pragma unroll
    for (int q = 0; q < kDepth - 1; ++q) issue(q);

    if constexpr (MODE != kModePV) {
      for (int q = 0; q < nk_mine; ++q) {
        advance(q);
        const uint8_t* stage = my_ring + (q & (kDepth - 1)) * kPassBytes;
        const uint32_t d = s_kdesc[warp + kGatherWarps * q];
        // the group's table and bias = sum_c q_c * (min_c + centre * scale_c)
        const uint2 sc = *reinterpret_cast<const uint2*>(stage + 512 + lane * 8);
        const uint2 mn = *reinterpret_cast<const uint2*>(stage + 512 + 256 + lane * 8);
        table_store<BITS>(s_wtab[warp], lane, q01, q23, sc);
        const float2 sc01 = __half22float2(as_half2(sc.x)), sc23 = __half22float2(as_half2(sc.y));
        const float2 mn01 = __half22float2(as_half2(mn.x)), mn23 = __half22float2(as_half2(mn.y));
        const float kcn = float(kCentre<BITS>);
        float bias = q4.x * fmaf(kcn, sc01.x, mn01.x);
        bias = fmaf(q4.y, fmaf(kcn, sc01.y, mn01.y), bias);
        bias = fmaf(q4.z, fmaf(kcn, sc23.x, mn23.x), bias);
        bias = fmaf(q4.w, fmaf(kcn, sc23.y, mn23.y), bias);
        const Codes<BITS> kc = load_codes_shared<BITS>(stage + codes_at);
        bias = warp_sum(bias);
        __syncwarp();
        __half2 mult[16];
        const uint4* tab4 = reinterpret_cast<const uint4*>(&s_wtab[warp][sub * 32]);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 x = tab4[v];
          mult[4 * v + 0] = as_half2(x.x); mult[4 * v + 1] = as_half2(x.y);
          mult[4 * v + 2] = as_half2(x.z); mult[4 * v + 3] = as_half2(x.w);
        }
        const float dot = quad_sum(k_dot_fast<BITS>(kc, mult)) + bias;
        if (quad <= static_cast<int>(d >> 10) && sub == 0) s_eval[(d & 1023u) + quad] = dot;
      }
      // tail tokens and the current token: BF16 rows, read directly
      for (int i0 = 8 * warp; i0 < n_tail; i0 += 8 * kGatherWarps) {
        const int i = i0 + quad;
        const bool on = i < n_tail;
        const int ring_slot = on ? s_tail[i] : 0;
        const __nv_bfloat16* krow = ring_slot < 0 ? p.kcur + bh * kHeadDim : tk + ring_slot * kHeadDim;
        const float dot = quad_sum(on ? bf16_row_dot<BITS>(krow, sub, s_qf) : 0.f);
        if (on && sub == 0) s_tval[i] = dot;
      }

      __syncthreads();  // every K pass of the batch has written its partial logits
      float logit = 0.f;
#pragma unroll
      for (int s = 0; s < STREAMS; ++s) logit += (member >> s) & 1u ? s_eval[at[s]] : 0.f;
      if ((member >> kTailClass) & 1u) logit = s_tval[at[kTailClass]];
      if constexpr (MODE == kModeQK) {
        if (live) p.logits[bh * p.capacity + batch_begin + tid] = logit;
      } else {
        if (live && idx == cur_pos && p.cur_logits) p.cur_logits[bh] = logit * p.scaling;
        const float x = live ? logit * p.scaling_log2 : -INFINITY;
        const float wmax = warp_max(x);
        if (lane == 0) s_red[warp] = wmax;
        __syncthreads();
        float bmax = s_red[0];
#pragma unroll
        for (int w = 1; w < kGatherWarps; ++w) bmax = fmaxf(bmax, s_red[w]);
        if (bmax > m_run) {
          const float r = exp2f(m_run - bmax);  // exp2f(-inf) == 0 on the first raise
          flush_pairs(hacc, S.acc);             // the float16 partial sums belong to the old maximum
          v_passes = 0;
          l_mine *= r;
          S.vbias *= r;
#pragma unroll
          for (int i = 0; i < 32; ++i) S.acc[i] *= r;
          m_run = bmax;
        }
        const float pr = live ? exp2f(x - m_run) : 0.f;
        l_mine += pr;
#pragma unroll
        for (int s = 0; s < STREAMS; ++s) {
          if ((member >> s) & 1u) s_eval[at[s]] = pr;
        }
        if ((member >> kTailClass) & 1u) s_tval[at[kTailClass]] = pr;
        __syncthreads();
      }
    }

    if constexpr (MODE != kModeQK) {
      const uint32_t pick = (sub < 2) ? 0x1010u : 0x3232u;
      const __half2 centre2 = __floats2half2_rn(float(kCentre<BITS>), float(kCentre<BITS>));
      for (int q = nk_mine; q < n_mine; ++q) {
        advance(q);
        const uint8_t* stage = my_ring + (q & (kDepth - 1)) * kPassBytes;
        const int i = 8 * (warp + kGatherWarps * (q - nk_mine)) + quad;
        const bool on = i < n_entries;
        const float pr = on ? s_eval[i] : 0.f;
        const __half2 p2 = __float2half2_rn(pr);
        const Codes<BITS> vc = load_codes_shared<BITS>(stage + codes_at);
        const uint2 vmeta = *reinterpret_cast<const uint2*>(stage + 512 + quad * 16);
        const __half2 vm2 = as_half2(on ? __byte_perm(vmeta.x, 0u, pick) : 0u);
        const __half2 vs2 = as_half2(on ? __byte_perm(vmeta.y, 0u, pick) : 0u);
        const __half2 hb = __hfma2(centre2, vs2, vm2);
        v_accumulate<BITS>(vc, __hmul2(p2, vs2), hacc);
        S.vbias = fmaf(pr, __low2float(hb), S.vbias);
        // at most 16 float16 terms per accumulator before widening
        if ((++v_passes & 15) == 0) flush_pairs(hacc, S.acc);
      }
      for (int i0 = 8 * warp; i0 < n_tail; i0 += 8 * kGatherWarps) {
        const int i = i0 + quad;
        if (i < n_tail) {
          const int ring_slot = s_tail[i];
          const __nv_bfloat16* vrow = ring_slot < 0 ? p.vcur + bh * kHeadDim : tv + ring_slot * kHeadDim;
          bf16_row_accumulate<BITS>(vrow, sub, s_tval[i], S.acc);
        }
      }
    }
    cp_async_wait<0>();
  }
  if constexpr (MODE == kModeQK) return;
  flush_pairs(hacc, S.acc);
  S.m = m_run;

  __syncthreads();  // every warp has left its ring: the rings become the merge buffer
  float (*s_merge)[kPartialStride] = reinterpret_cast<float (*)[kPartialStride]>(s_ring);
  state_store<BITS>(S, lane, s_merge[warp]);
  const float l_warp = warp_sum(l_mine);
  if (lane == 0) s_merge[warp][129] = l_warp;
  float total, denom;
  if (merge_and_publish<kGatherWarps>(p, s_merge, &s_last, bh, split, nsplits, total, denom)) {
    const int c = threadIdx.x;
    if (c < kHeadDim) {
      if constexpr (MODE == kModeDelta) {
        const float target = denom > 0.f ? total / denom : 0.f;
        p.out[bh * kHeadDim + c] = p.mass[bh] * (target - p.source_out[bh * kHeadDim + c]);
      } else {
        p.out[bh * kHeadDim + c] = total;
      }
    }
  }
}

// ------------------------------------------------------------------------------ host side

// Grid of the persistent dense reader: two CTAs per SM, but never more CTAs than there are tail
// units, so that every CTA's share of the units is non-empty whatever the context lengths are.
unsigned dense_grid(int64_t batch_heads) {
  static const int sm_count = [] {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
  }();
  const int64_t ctas = 2 * static_cast<int64_t>(sm_count < 148 ? sm_count : 148);
  const int64_t cap = batch_heads * kTailUnits;
  return static_cast<unsigned>(cap < ctas ? cap : ctas);
}

int choose_slots_per_cta(int64_t batch_heads, int64_t capacity) {
  // One wave: the grid is kept within the CTAs of the gather kernel that are resident at once
  // where the capacity allows it (a second, partial wave would cost a whole round).
  const int64_t budget = 148 * kGatherCtasPerSm;
  int64_t slots = 32;
  while ((batch_heads * ((capacity + slots - 1) / slots) > budget || (capacity + slots - 1) / slots > kMaxSplits) &&
         slots < capacity)
    slots += 32;
  return static_cast<int>(slots);
}

// tickets[batch_heads] and one status word, padded to 256 bytes
size_t tickets_bytes(int64_t batch_heads) { return (((batch_heads + 3) * sizeof(int) + 255) / 256) * 256; }

// Partial slots per (b,h).  The selected readers split a head over at most kMaxSplits CTAs; the
// dense reader needs two slots per CTA, at most 2 * 8 * batch_heads in all.
int max_partials() {
  static_assert(kMaxSplits >= 2 * kTailUnits, "the dense reader's partials must fit the workspace");
  return kMaxSplits;
}

}  // namespace

int validate_layer(const fl_layer* layer, int loop, const char* who) {
  FL_REQUIRE(layer != nullptr, "%s: null layer", who);
  FL_REQUIRE(layer->batch > 0 && layer->heads > 0, "%s: batch and heads must be positive", who);
  FL_REQUIRE(static_cast<int64_t>(layer->batch) * layer->heads <= 65535, "%s: batch*heads above 65535", who);
  FL_REQUIRE(layer->bits == 4 || layer->bits == 2, "%s: bits must be 4 or 2, got %d", who, layer->bits);
  FL_REQUIRE(loop >= 0 && loop < 4, "%s: loop must be in [0, 3], got %d", who, loop);
  FL_REQUIRE(layer->tail_capacity >= 1, "%s: tail_capacity must be positive", who);
  FL_REQUIRE(layer->seq_state != nullptr, "%s: seq_state is null", who);
  for (int s = 0; s <= loop; ++s) {
    FL_REQUIRE(layer->k_codes[s] && layer->k_min[s] && layer->k_scale[s] && layer->v_rows[s] &&
                   layer->row_base[s] && layer->group_base[s],
               "%s: stream %d has a null pointer", who, s);
    FL_REQUIRE(aligned16(layer->k_codes[s]) && aligned16(layer->v_rows[s]) && aligned16(layer->k_min[s]) &&
                   aligned16(layer->k_scale[s]),
               "%s: stream %d is not 16-byte aligned", who, s);
  }
  if (loop >= 2) {
    FL_REQUIRE(layer->rank[0] && layer->rank_base, "%s: loop %d needs the loop-3 rank map", who, loop);
    if (loop >= 3) FL_REQUIRE(layer->rank[1] != nullptr, "%s: loop 3 needs the loop-4 rank map", who);
  }
  FL_REQUIRE(layer->tail_k[loop] && layer->tail_v[loop], "%s: tail of loop %d is null", who, loop);
  FL_REQUIRE(aligned16(layer->tail_k[loop]) && aligned16(layer->tail_v[loop]),
             "%s: tails must be 16-byte aligned", who);
  return FL_OK;
}

}  // namespace fl

using namespace fl;

extern "C" size_t fl_reader_workspace_bytes(int64_t batch_heads, int64_t max_context_tokens) {
  if (batch_heads <= 0 || max_context_tokens < 0) return 0;
  return tickets_bytes(batch_heads) +
         static_cast<size_t>(batch_heads) * max_partials() * kPartialStride *
             sizeof(float);
}

extern "C" int fl_workspace_status(const void* workspace, int64_t batch_heads, int32_t* status,
                                   fl_cuda_stream stream) {
  FL_REQUIRE(workspace != nullptr && status != nullptr && batch_heads > 0, "fl_workspace_status: bad argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemcpyAsync(status, static_cast<const int*>(workspace) + batch_heads, sizeof(int32_t),
                                    cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    set_error("fl_workspace_status: %s", cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  return FL_OK;
}

extern "C" int fl_workspace_init(void* workspace, size_t bytes, fl_cuda_stream stream) {
  FL_REQUIRE(workspace != nullptr && bytes > 0, "fl_workspace_init: empty workspace");
  const cudaError_t err = cudaMemsetAsync(workspace, 0, bytes, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    set_error("fl_workspace_init: %s", cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  return FL_OK;
}

namespace {

int fill_common(ReaderParams& p, const fl_layer* layer, int loop, void* workspace, size_t workspace_bytes,
                int64_t max_context_tokens, const char* who) {
  const int64_t bh = static_cast<int64_t>(layer->batch) * layer->heads;
  const size_t need = fl_reader_workspace_bytes(bh, max_context_tokens);
  if (workspace == nullptr || workspace_bytes < need || !aligned16(workspace)) {
    set_error("%s: workspace of %zu bytes (16-byte aligned) required, got %zu", who, need, workspace_bytes);
    return FL_ERR_WORKSPACE;
  }
  p.L = make_view(*layer);
  p.loop = loop;
  p.tickets = static_cast<int*>(workspace);
  p.status = p.tickets + bh;
  p.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + tickets_bytes(bh));
  p.max_chunks = max_partials();
  return FL_OK;
}

}  // namespace

namespace fl {
namespace {

template <int BITS, int LOOP>
cudaError_t launch_dense_as(unsigned grid, cudaStream_t s, const ReaderParams& p) {
  constexpr int kSmem = kDenseWarps * kStages * Stage<BITS>::kBytes;
  static const cudaError_t attr = cudaFuncSetAttribute(dense_reader_kernel<BITS, LOOP>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (attr != cudaSuccess) return attr;
  dense_reader_kernel<BITS, LOOP><<<grid, kDenseThreads, kSmem, s>>>(p);
  return cudaSuccess;
}

template <int BITS>
cudaError_t launch_dense_bits(int loop, unsigned grid, cudaStream_t s, const ReaderParams& p) {
  switch (loop) {
    case 0: return launch_dense_as<BITS, 0>(grid, s, p);
    case 1: return launch_dense_as<BITS, 1>(grid, s, p);
    case 2: return launch_dense_as<BITS, 2>(grid, s, p);
    default: return launch_dense_as<BITS, 3>(grid, s, p);
  }
}

cudaError_t launch_dense(int bits, int loop, unsigned grid, cudaStream_t s, const ReaderParams& p) {
  return bits == 4 ? launch_dense_bits<4>(loop, grid, s, p) : launch_dense_bits<2>(loop, grid, s, p);
}

}  // namespace
}  // namespace fl

extern "C" int fl_dense_source_attention(const fl_layer* layer, int32_t loop, const void* query,
                                         const void* current_key, const void* current_value,
                                         float scaling, float* output, float* logits,
                                         int64_t logits_stride, int64_t max_context_tokens,
                                         void* workspace, size_t workspace_bytes,
                                         fl_cuda_stream stream) {
  if (int rc = validate_layer(layer, loop, "fl_dense_source_attention")) return rc;
  FL_REQUIRE(query && current_key && current_value && output, "fl_dense_source_attention: null vector");
  FL_REQUIRE(aligned16(query) && aligned16(current_key) && aligned16(current_value),
             "fl_dense_source_attention: vectors must be 16-byte aligned");
  FL_REQUIRE(max_context_tokens >= 0, "fl_dense_source_attention: negative max_context_tokens");
  FL_REQUIRE(!logits || logits_stride > max_context_tokens,
             "fl_dense_source_attention: logits_stride must exceed max_context_tokens");
  ReaderParams p{};
  if (int rc = fill_common(p, layer, loop, workspace, workspace_bytes, max_context_tokens,
                           "fl_dense_source_attention"))
    return rc;
  const int64_t bh = static_cast<int64_t>(layer->batch) * layer->heads;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kcur = static_cast<const __nv_bfloat16*>(current_key);
  p.vcur = static_cast<const __nv_bfloat16*>(current_value);
  p.scaling = scaling;
  p.scaling_log2 = scaling * 1.4426950408889634f;
  p.out = output;
  p.logits = logits;
  p.logits_stride = logits_stride;
  const unsigned grid = dense_grid(bh);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaError_t err = launch_dense(layer->bits, loop, grid, s, p); err != cudaSuccess) {
    set_error("fl_dense_source_attention: %s", cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  FL_CHECK_LAUNCH("fl_dense_source_attention");
  return FL_OK;
}

namespace {

template <int BITS, int MODE, int STREAMS>
void launch_selected_as(const dim3 grid, const ReaderParams& p, cudaStream_t s) {
  constexpr int kSmem = kGatherWarps * kDepth * kPassBytes;
  static const cudaError_t attr = cudaFuncSetAttribute(
      selected_reader_kernel<BITS, MODE, STREAMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  (void)attr;
  selected_reader_kernel<BITS, MODE, STREAMS><<<grid, kGatherThreads, kSmem, s>>>(p);
}

template <int BITS, int MODE>
void launch_selected_bits(const dim3 grid, const ReaderParams& p, cudaStream_t s) {
  switch (p.loop) {
    case 0: launch_selected_as<BITS, MODE, 1>(grid, p, s); break;
    case 1: launch_selected_as<BITS, MODE, 2>(grid, p, s); break;
    case 2: launch_selected_as<BITS, MODE, 3>(grid, p, s); break;
    default: launch_selected_as<BITS, MODE, 4>(grid, p, s); break;
  }
}

template <int MODE>
int launch_selected(const fl_layer* layer, ReaderParams& p, cudaStream_t s, const char* who) {
  const int64_t bh = static_cast<int64_t>(layer->batch) * layer->heads;
  p.slots_per_cta = choose_slots_per_cta(bh, p.capacity);
  const int splits = (p.capacity + p.slots_per_cta - 1) / p.slots_per_cta;
  const dim3 grid(splits, static_cast<unsigned>(bh));
  if (layer->bits == 4) {
    launch_selected_bits<4, MODE>(grid, p, s);
  } else {
    launch_selected_bits<2, MODE>(grid, p, s);
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}

}  // namespace

extern "C" int fl_sparse_attention_delta(const fl_layer* layer, int32_t loop, const void* query,
                                         const void* current_key, const void* current_value,
                                         const int32_t* indices, const uint8_t* valid,
                                         int64_t capacity, const float* source_output,
                                         const float* global_mass, float scaling, float* output,
                                         float* current_logits, void* workspace,
                                         size_t workspace_bytes, fl_cuda_stream stream) {
  const char* who = "fl_sparse_attention_delta";
  if (int rc = validate_layer(layer, loop, who)) return rc;
  FL_REQUIRE(query && current_key && current_value && indices && valid && source_output && global_mass && output,
             "%s: null argument", who);
  FL_REQUIRE(aligned16(query) && aligned16(current_key) && aligned16(current_value),
             "%s: vectors must be 16-byte aligned", who);
  FL_REQUIRE(capacity > 0 && capacity < (1 << 24), "%s: capacity out of range", who);
  ReaderParams p{};
  if (int rc = fill_common(p, layer, loop, workspace, workspace_bytes, 0, who)) return rc;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kcur = static_cast<const __nv_bfloat16*>(current_key);
  p.vcur = static_cast<const __nv_bfloat16*>(current_value);
  p.scaling = scaling;
  p.scaling_log2 = scaling * 1.4426950408889634f;
  p.out = output;
  p.indices = indices;
  p.valid = valid;
  p.capacity = static_cast<int>(capacity);
  p.source_out = source_output;
  p.mass = global_mass;
  p.cur_logits = current_logits;
  return launch_selected<kModeDelta>(layer, p, static_cast<cudaStream_t>(stream), who);
}

extern "C" int fl_selected_pv(const fl_layer* layer, int32_t loop, const float* weights,
                              const int32_t* indices, const uint8_t* valid, int64_t capacity,
                              const void* current_value, float* output, void* workspace,
                              size_t workspace_bytes, fl_cuda_stream stream) {
  const char* who = "fl_selected_pv";
  if (int rc = validate_layer(layer, loop, who)) return rc;
  FL_REQUIRE(weights && indices && output, "%s: null argument", who);
  FL_REQUIRE(!current_value || aligned16(current_value), "%s: current_value must be 16-byte aligned", who);
  FL_REQUIRE(capacity > 0 && capacity < (1 << 24), "%s: capacity out of range", who);
  ReaderParams p{};
  if (int rc = fill_common(p, layer, loop, workspace, workspace_bytes, 0, who)) return rc;
  p.vcur = static_cast<const __nv_bfloat16*>(current_value);
  p.out = output;
  p.indices = indices;
  p.valid = valid;
  p.capacity = static_cast<int>(capacity);
  p.weights = weights;
  return launch_selected<kModePV>(layer, p, static_cast<cudaStream_t>(stream), who);
}

extern "C" int fl_selected_qk(const fl_layer* layer, int32_t loop, const void* query,
                              const int32_t* indices, const uint8_t* valid, int64_t capacity,
                              const void* current_key, float* logits, fl_cuda_stream stream) {
  const char* who = "fl_selected_qk";
  if (int rc = validate_layer(layer, loop, who)) return rc;
  FL_REQUIRE(query && indices && logits, "%s: null argument", who);
  FL_REQUIRE(aligned16(query) && (!current_key || aligned16(current_key)),
             "%s: vectors must be 16-byte aligned", who);
  FL_REQUIRE(capacity > 0 && capacity < (1 << 24), "%s: capacity out of range", who);
  ReaderParams p{};
  p.L = make_view(*layer);
  p.loop = loop;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kcur = static_cast<const __nv_bfloat16*>(current_key);
  p.scaling = 1.f;
  p.scaling_log2 = 1.f;
  p.logits = logits;
  p.indices = indices;
  p.valid = valid;
  p.capacity = static_cast<int>(capacity);
  p.max_chunks = kMaxSplits;
  return launch_selected<kModeQK>(layer, p, static_cast<cudaStream_t>(stream), who);
}

// ------------------------------------------------------------------------------ scratch-free variant
//
// fl_dense_source_attention_static: the dense reader for callers that cannot hand over a
// scratch buffer because they cannot allocate device memory at the point of the call -- code
// running inside a stream capture, a plugin loaded into a server whose memory is owned by a
// fixed pool it has no handle to, a host language binding without a device allocator.  The
// scratch (tickets, status word, split partials) lives in the file-scope device
// array below, which every GPU that loads this library holds until the process exits.

namespace fl {
namespace {

constexpr int64_t kStaticMaxBatchHeads = 128;
constexpr int64_t kStaticMaxContext = 16384;
// partial slots: two per CTA of the largest grid
constexpr int kStaticSlots = 2 * 2 * 148;
constexpr size_t kStaticHeaderBytes = ((kStaticMaxBatchHeads + 3) * sizeof(int) + 255) / 256 * 256;
constexpr size_t kStaticBytes =
    kStaticHeaderBytes + static_cast<size_t>(kStaticSlots) * kPartialStride * sizeof(float);

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
void* g_static_address[kMaxDevices] = {};

// The array's name is only a host-side handle: the device address has to be asked for, once
// per device, with that device current.  The header words are cleared here so that a first
// call starts from zero whatever a previous, failed launch may have left behind.
int static_scratch_address(void** address, cudaStream_t stream) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= kMaxDevices) {
    set_error("fl_dense_source_attention_static: cannot identify the current device");
    return FL_ERR_CUDA;
  }
  if (g_static_address[device] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      set_error("fl_dense_source_attention_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
      return FL_ERR_CUDA;
    }
    err = cudaMemsetAsync(ptr, 0, kStaticHeaderBytes, stream);
    if (err != cudaSuccess) {
      set_error("fl_dense_source_attention_static: clearing the scratch header failed: %s",
                cudaGetErrorString(err));
      return FL_ERR_CUDA;
    }
    g_static_address[device] = ptr;
  }
  *address = g_static_address[device];
  return FL_OK;
}

}  // namespace
}  // namespace fl

extern "C" int fl_dense_source_attention_static(const fl_layer* layer, int32_t loop, const void* query,
                                                const void* current_key, const void* current_value,
                                                float scaling, float* output, float* logits,
                                                int64_t logits_stride, int64_t max_context_tokens,
                                                fl_cuda_stream stream) {
  const char* who = "fl_dense_source_attention_static";
  if (int rc = validate_layer(layer, loop, who)) return rc;
  FL_REQUIRE(query && current_key && current_value && output, "%s: null vector", who);
  FL_REQUIRE(aligned16(query) && aligned16(current_key) && aligned16(current_value),
             "%s: vectors must be 16-byte aligned", who);
  FL_REQUIRE(!logits || logits_stride > max_context_tokens, "%s: logits_stride must exceed max_context_tokens", who);
  const int64_t bh = static_cast<int64_t>(layer->batch) * layer->heads;
  if (bh > kStaticMaxBatchHeads || max_context_tokens < 0 || max_context_tokens > kStaticMaxContext) {
    set_error("%s: batch*heads %lld (limit %lld) or max_context_tokens %lld (limit %lld) exceeds the built-in "
              "scratch; use fl_dense_source_attention with a caller-provided workspace",
              who, static_cast<long long>(bh), static_cast<long long>(kStaticMaxBatchHeads),
              static_cast<long long>(max_context_tokens), static_cast<long long>(kStaticMaxContext));
    return FL_ERR_UNSUPPORTED;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch, s)) return rc;

  ReaderParams p{};
  p.L = make_view(*layer);
  p.loop = loop;
  p.tickets = static_cast<int*>(scratch);
  p.status = p.tickets + kStaticMaxBatchHeads;
  p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + kStaticHeaderBytes);
  p.max_chunks = kStaticSlots;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kcur = static_cast<const __nv_bfloat16*>(current_key);
  p.vcur = static_cast<const __nv_bfloat16*>(current_value);
  p.scaling = scaling;
  p.scaling_log2 = scaling * 1.4426950408889634f;
  p.out = output;
  p.logits = logits;
  p.logits_stride = logits_stride;
  const unsigned grid = dense_grid(bh);
  if (cudaError_t err = launch_dense(layer->bits, loop, grid, s, p); err != cudaSuccess) {
    set_error("%s: %s", who, cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}
