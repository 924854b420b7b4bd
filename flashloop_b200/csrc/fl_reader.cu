// Dense decode-attention reader over the packed anchor + delta streams (row layout).
//
//   dense_reader_kernel     one launch: QK^T over streams 0..loop + BF16 tail + current token,
//                           online softmax, PV; persistent CTAs that each own a contiguous,
//                           equally large range of 64-token blocks over all (b,h); partials of a
//                           (b,h) merged by its last-arriving CTA (an atomic ticket, no waiting).
//
// The gathered readers (cached-mass sparse delta, weighted PV, selected QK) live in fl_selected.cu.
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
#include "fl_reader_common.cuh"

namespace fl {
namespace {

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
constexpr int kDenseCtasPerSm = 2;
constexpr int kWaitLimit = 1 << 12;
constexpr uint32_t kSuspendNs = 100000;  // (1 us and 100 ns with more tries measured the same)

template <int BITS>
struct Stage {
  static constexpr int kRowBytes = 16 * BITS;
  static constexpr int kRecord = kRowBytes + 16;     // V record: codes, 8 bytes of metadata, padding
  static constexpr int kCodes = kGroup * kRowBytes;  // K unit: 64 code rows, then ...
  static constexpr int kMeta = 1024;                 // ... the scale/min rows of up to two groups
  static constexpr int kBytes = kCodes + kMeta;      // a V unit is 64 records: the same size
  static_assert(kGroup * kRecord <= kBytes, "a V unit must fit the stage");
};

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
// tail_units_of_loop for its BF16 tail and the current token (about what the tail, the merge of the
// head and the switch to the next head cost a CTA, counted in blocks of that loop).  The units
// of all heads form one sequence, head after head, and CTA c owns the contiguous range
// [c*U/G, (c+1)*U/G) of it, so every CTA gets the same amount of work whatever the context
// lengths are.  A work item is the part of one head inside that range: some blocks, the tail, or
// both.  A CTA therefore meets a head once, keeps its online-softmax state in registers across all
// of the head's blocks it owns, and merges and publishes once per item: one to three times in all.
// Units a head's tail, its merge and the switch to the next head are counted as (loop: 0-based).
// Their cost is a time, so it is more blocks of a loop that reads fewer streams per block, and it
// weighs more where heads are short: measured, 24 / 16 units for loops 1 / 2 are 5 % faster than 8 at
// batch 16 x 2048 tokens and 2 % slower at batch 8 x 8192, so the longer count is used up to 4096
// tokens of context (the caller's bound).
inline int tail_units_of_loop(int loop, int64_t max_context_tokens) {
  return max_context_tokens <= 4096 ? 8 + 16 / (loop + 1) : 8;
}

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

__device__ __forceinline__ int units_per_head(const LayerView& L, int tail_units, int b) {
  return L.seq_state[b * FL_STATE_WORDS + FL_STATE_QUANT_TOKENS] / kGroup + tail_units;
}
// `each`: the CTA's shared copy of units_per_head for the first kEachCached sequences
__device__ __forceinline__ int units_per_head(const LayerView& L, int tail_units, const int* each, int b) {
  return b < kEachCached ? each[b] : units_per_head(L, tail_units, b);
}
__device__ __forceinline__ int64_t total_units(const LayerView& L, int tail_units, const int* each) {
  int64_t total = 0;
  for (int b = 0; b < L.batch; ++b) total += static_cast<int64_t>(L.heads) * units_per_head(L, tail_units, each, b);
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

__device__ __forceinline__ void cursor_start(const LayerView& L, int tail_units, const int* each, int64_t lo, int64_t hi,
                                             ItemCursor* c) {
  c->at = lo;
  c->end = hi;
  c->count = 0;
  c->blocks_done = 0;
  c->b = 0;
  c->each = units_per_head(L, tail_units, each, 0);
  int64_t first = 0;
  while (c->b + 1 < L.batch && lo >= first + static_cast<int64_t>(L.heads) * c->each) {
    first += static_cast<int64_t>(L.heads) * c->each;
    ++c->b;
    c->each = units_per_head(L, tail_units, each, c->b);
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
  const int blocks = c->each - p.tail_units;
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
  const int64_t grid = all_units < static_cast<int64_t>(gridDim.x) ? all_units : static_cast<int64_t>(gridDim.x);
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
        c->each = units_per_head(L, p.tail_units, each, c->b);
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

// Online-softmax state of a warp on the tensor-pipe path (loops 1 and 2, where every token holds a
// row in every stream it reads).  Lane (g = lane / 4, j = lane % 4) owns channels 16g .. 16g+15:
// accumulator i holds two of them (rows g and g + 8 of the mma) in columns of both V scale groups,
// acc[i][0] / acc[i][1] = first channel with the scale of channel group 0 / 1, acc[i][2] / acc[i][3]
// the second; the lane's channels live in group g / 4, the other column is dropped at the end.
template <int BITS>
struct MmaState {
  static constexpr int kTypes = BITS == 4 ? 2 : 4;  // positions of a code inside its byte
  float m, l;
  float bm;               // sum of p * v_min of channel group g % 2 over this lane's tokens
  float acc[8][4];        // sum of W * (1024 + t * code), W = p * v_scale / t
  float off[kTypes][4];   // sum of W * 1024 per position type
};

template <int BITS>
__device__ __forceinline__ void mma_state_init(MmaState<BITS>& s) {
  s.m = -INFINITY;
  s.l = 0.f;
  s.bm = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) s.acc[i][k] = 0.f;
#pragma unroll
  for (int i = 0; i < MmaState<BITS>::kTypes; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) s.off[i][k] = 0.f;
}

template <int BITS>
__device__ __forceinline__ void mma_state_raise(MmaState<BITS>& s, float mx) {
  if (mx > s.m) {
    const float r = exp2f(s.m - mx);
    s.l *= r;
    s.bm *= r;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int k = 0; k < 4; ++k) s.acc[i][k] *= r;
#pragma unroll
    for (int i = 0; i < MmaState<BITS>::kTypes; ++i)
#pragma unroll
      for (int k = 0; k < 4; ++k) s.off[i][k] *= r;
    s.m = mx;
  }
}

// Accumulator i of a lane: its two channels (within the lane's sixteen) and its position type.
template <int BITS>
__host__ __device__ constexpr int mma_channel(int i, int second) {
  return BITS == 4 ? 8 * (i / 4) + ((i % 4) / 2) * 4 + (i % 2) + 2 * second : 8 * (i / 4) + (i % 4) + 4 * second;
}
template <int BITS>
__host__ __device__ constexpr int mma_type(int i) {
  return BITS == 4 ? i % 2 : i % 4;
}

// Park the warp's state in shared memory as acc[128] (natural channel order), m, l.
template <int BITS>
__device__ __forceinline__ void mma_state_store(MmaState<BITS>& s, int lane, float* dst) {
  const int g = lane >> 2, grp = g >> 2;
  const float l = across_quads_sum(s.l);
  float bm = s.bm;
  bm += __shfl_xor_sync(0xffffffffu, bm, 1);
  bm += __shfl_xor_sync(0xffffffffu, bm, 2);
  const float bm_mine = __shfl_sync(0xffffffffu, bm, 4 * grp);  // lanes 0-3 hold group 0, lanes 4-7 group 1
  if ((lane & 3) == 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = mma_type<BITS>(i);
      const float o = grp ? s.off[t][1] : s.off[t][0];
      dst[16 * g + mma_channel<BITS>(i, 0)] = (grp ? s.acc[i][1] : s.acc[i][0]) - o + bm_mine;
      dst[16 * g + mma_channel<BITS>(i, 1)] = (grp ? s.acc[i][3] : s.acc[i][2]) - o + bm_mine;
    }
    if (lane == 0) {
      dst[128] = s.m;
      dst[129] = l;
    }
  }
}

// K unit of a full block on the tensor pipe: kc[q] += (rows 16q+g, 16q+g+8) . table, all four
// lanes of a quad (and all eight columns) ending up with the same sums.
template <int BITS>
__device__ __forceinline__ void k_block_mma(const uint8_t* stage, int lane, const uint32_t (&mult)[16],
                                            float (&kc)[4][4]) {
  constexpr int kRowBytes = 16 * BITS, kLaneBytes = kRowBytes / 4;
  constexpr int kWords = BITS, kPairs = 16 / kWords;  // words per lane piece, pairs per word
  const int g = lane >> 2, j = lane & 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint8_t* ra = stage + (16 * q + g) * kRowBytes + j * kLaneBytes;
    const Codes<BITS> ca = load_codes_shared<BITS>(ra);
    const Codes<BITS> cb = load_codes_shared<BITS>(ra + 8 * kRowBytes);
#pragma unroll
    for (int wd = 0; wd < kWords; ++wd) {
      uint32_t ha[kPairs], hb[kPairs];
      unpack_raw_word<BITS>(ca.w[wd], ha);
      unpack_raw_word<BITS>(cb.w[wd], hb);
#pragma unroll
      for (int i = 0; i < kPairs / 2; ++i) {
        mma16816(kc[q], ha[2 * i], hb[2 * i], ha[2 * i + 1], hb[2 * i + 1], mult[wd * kPairs + 2 * i],
                 mult[wd * kPairs + 2 * i + 1]);
      }
    }
  }
}

// V unit of a full block on the tensor pipe.  probs: the warp's 64 probabilities as float16.
// Lane (g, j) reads channels 16g .. 16g+15 of tokens 2j, 2j+1, 2j+8, 2j+9 of every 16-token set and
// supplies the probabilities of those tokens times the V scale of channel group g % 2 (even
// columns of the mma carry group 0, odd columns group 1).
template <int BITS>
__device__ __forceinline__ void v_block_mma(const uint8_t* stage, int lane, const __half* probs,
                                            MmaState<BITS>& st, __half2& hbias) {
  constexpr int kRowBytes = 16 * BITS, kRecord = kRowBytes + 16;
  constexpr int kTypes = MmaState<BITS>::kTypes;
  const int g = lane >> 2, j = lane & 3;
  const uint32_t sel = (g & 1) ? 0x7632u : 0x5410u;
  const uint32_t k1024 = 0x64006400u;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint8_t* rec = stage + (16 * q + 2 * j) * kRecord;  // tokens 2j, 2j+1; +8 records: 2j+8, 2j+9
    uint32_t x[4][BITS / 2];
    uint2 mt[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint8_t* r = rec + ((k & 1) + (k >> 1) * 8) * kRecord;
      if constexpr (BITS == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(r + 8 * g);
        x[k][0] = v.x;
        x[k][1] = v.y;
      } else {
        x[k][0] = *reinterpret_cast<const uint32_t*>(r + 4 * g);
      }
      mt[k] = *reinterpret_cast<const uint2*>(r + kRowBytes);
    }
    const __half2 p01 = *reinterpret_cast<const __half2*>(probs + 16 * q + 2 * j);
    const __half2 p23 = *reinterpret_cast<const __half2*>(probs + 16 * q + 2 * j + 8);
    hbias = __hfma2(p01, as_half2(__byte_perm(mt[0].x, mt[1].x, sel)), hbias);
    hbias = __hfma2(p23, as_half2(__byte_perm(mt[2].x, mt[3].x, sel)), hbias);
    uint32_t w01[kTypes], w23[kTypes];
    w01[0] = as_u32(__hmul2(p01, as_half2(__byte_perm(mt[0].y, mt[1].y, sel))));
    w23[0] = as_u32(__hmul2(p23, as_half2(__byte_perm(mt[2].y, mt[3].y, sel))));
#pragma unroll
    for (int t = 1; t < kTypes; ++t) {
      const float f = BITS == 4 ? 0.0625f : (t == 1 ? 0.25f : (t == 2 ? 0.0625f : 0.015625f));
      const __half2 f2 = __floats2half2_rn(f, f);
      w01[t] = as_u32(__hmul2(as_half2(w01[0]), f2));
      w23[t] = as_u32(__hmul2(as_half2(w23[0]), f2));
    }
#pragma unroll
    for (int t = 0; t < kTypes; ++t) mma16816(st.off[t], k1024, k1024, k1024, k1024, w01[t], w23[t]);
#pragma unroll
    for (int wd = 0; wd < BITS / 2; ++wd) {
      // 16-bit halves of the two tokens of a pair side by side: codes 0-3 (4 bits) or 0-7 (2 bits)
      // of the word in u, the rest in v
      const uint32_t u01 = __byte_perm(x[0][wd], x[1][wd], 0x5410), v01 = __byte_perm(x[0][wd], x[1][wd], 0x7632);
      const uint32_t u23 = __byte_perm(x[2][wd], x[3][wd], 0x5410), v23 = __byte_perm(x[2][wd], x[3][wd], 0x7632);
      if constexpr (BITS == 4) {
        uint32_t e[4], f[4];
        unpack_raw_word<4>(u01, e);
        unpack_raw_word<4>(u23, f);
        // pairs of unpack_raw_word<4> on u: (code 0), (code 1, x16), (code 2), (code 3, x16)
        mma16816(st.acc[4 * wd + 0], e[0], e[2], f[0], f[2], w01[0], w23[0]);
        mma16816(st.acc[4 * wd + 1], e[1], e[3], f[1], f[3], w01[1], w23[1]);
        unpack_raw_word<4>(v01, e);
        unpack_raw_word<4>(v23, f);
        mma16816(st.acc[4 * wd + 2], e[0], e[2], f[0], f[2], w01[0], w23[0]);
        mma16816(st.acc[4 * wd + 3], e[1], e[3], f[1], f[3], w01[1], w23[1]);
      } else {
        uint32_t e[8], f[8];
        unpack_raw_word<2>(u01, e);
        unpack_raw_word<2>(u23, f);
#pragma unroll
        for (int t = 0; t < 4; ++t) mma16816(st.acc[t], e[t], e[t + 4], f[t], f[t + 4], w01[t], w23[t]);
        unpack_raw_word<2>(v01, e);
        unpack_raw_word<2>(v23, f);
#pragma unroll
        for (int t = 0; t < 4; ++t) mma16816(st.acc[4 + t], e[t], e[t + 4], f[t], f[t + 4], w01[t], w23[t]);
      }
    }
  }
}

template <int BITS, int LOOP>
__global__ void __launch_bounds__(kDenseThreads, kDenseCtasPerSm)
dense_reader_kernel(const __grid_constant__ ReaderParams p) {
  using St = Stage<BITS>;
  constexpr int kRowBytes = St::kRowBytes;
  constexpr int kLaneBytes = kRowBytes / 4;
  extern __shared__ __align__(128) uint8_t s_ring[];  // [warp][stage][St::kBytes]
  __shared__ __align__(16) float s_qf[2][kHeadDim];
  __shared__ __align__(16) __half s_wtab[kDenseWarps][2][kHeadDim];
  __shared__ __align__(16) float s_merge[2][(LOOP <= 1 ? 2 : 1) * kDenseWarps][kPartialStride];
  __shared__ __align__(4) __half s_prob[LOOP <= 1 ? kDenseWarps : 1][kGroup];
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
  for (int bb = tid; bb < L.batch && bb < kEachCached; bb += kDenseThreads) s_each[bb] = units_per_head(L, p.tail_units, bb);
  __syncthreads();
  {
    // Every thread finds the CTA's range and the head it starts in (shared-memory reads only), so
    // that the first query is fetched while one thread describes the first two items.
    const int64_t all_units = total_units(L, p.tail_units, s_each);
    ItemCursor cursor;
    // the partition is over min(grid, units) CTAs, so that every CTA that takes part owns at least
    // one unit (a head counts the CTAs that share it as a contiguous range); the others leave at once
    const int64_t ctas = all_units < static_cast<int64_t>(gridDim.x) ? all_units : static_cast<int64_t>(gridDim.x);
    const int64_t me = static_cast<int64_t>(blockIdx.x) < ctas ? static_cast<int64_t>(blockIdx.x) : ctas;
    cursor_start(L, p.tail_units, s_each, all_units * me / ctas, me < ctas ? all_units * (me + 1) / ctas : all_units, &cursor);
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
  MmaState<BITS> M;
  if constexpr (kAllRows) {
    mma_state_init(M);
  } else {
    state_init(S);
  }

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
      float kc[4][4], kb = 0.f;
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
        if constexpr (kAllRows) {
          if (!is_v) {
            if (s == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int c = 0; c < 4; ++c) kc[q][c] = 0.f;
              kb = 0.f;
            }
            // table: w_c = q_c * scale_c / t_c as float16; what the uncentred codes add to every
            // logit, 1024 * sum of the table, goes into the bias with the minima
            {
              const uint2 sc = *reinterpret_cast<const uint2*>(stage + St::kCodes + lane * 8);
              const uint2 mn = *reinterpret_cast<const uint2*>(stage + St::kCodes + 256 + lane * 8);
              const float2 sc01 = __half22float2(as_half2(sc.x)), sc23 = __half22float2(as_half2(sc.y));
              const float2 mn01 = __half22float2(as_half2(mn.x)), mn23 = __half22float2(as_half2(mn.y));
              const float4 q4 = *reinterpret_cast<const float4*>(&qf[4 * lane]);
              const int cc = (4 * lane) & 31;
              const __half w0 = __float2half_rn(q4.x * sc01.x * position_factor<BITS>(0));
              const __half w1 = __float2half_rn(q4.y * sc01.y * position_factor<BITS>(1));
              const __half w2 = __float2half_rn(q4.z * sc23.x * position_factor<BITS>(2));
              const __half w3 = __float2half_rn(q4.w * sc23.y * position_factor<BITS>(3));
              __half* tab = &s_wtab[warp][0][(4 * lane) & ~31];
              tab[channel_slot<BITS>(cc + 0)] = w0;
              tab[channel_slot<BITS>(cc + 1)] = w1;
              tab[channel_slot<BITS>(cc + 2)] = w2;
              tab[channel_slot<BITS>(cc + 3)] = w3;
              float bias = fmaf(q4.x, mn01.x, fmaf(q4.y, mn01.y, fmaf(q4.z, mn23.x, q4.w * mn23.y)));
              bias -= 1024.f * ((__half2float(w0) + __half2float(w1)) + (__half2float(w2) + __half2float(w3)));
              kb += warp_sum(bias);
            }
            __syncwarp();
            uint32_t mult[16];
            {
              const uint4* src = reinterpret_cast<const uint4*>(&s_wtab[warp][0][sub * 32]);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const uint4 x = src[v];
                mult[4 * v + 0] = x.x; mult[4 * v + 1] = x.y; mult[4 * v + 2] = x.z; mult[4 * v + 3] = x.w;
              }
            }
            k_block_mma<BITS>(stage, lane, mult, kc);
            if (s == LOOP) {
              // all streams summed: this lane holds the logits of tokens 16q + quad and 16q + quad + 8
              float mx = -INFINITY;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float raw0 = kc[q][0] + kb, raw1 = kc[q][2] + kb;
                if (logits_row && sub == 0) {
                  logits_row[t0 + 16 * q + quad] = raw0 * p.scaling;
                  logits_row[t0 + 16 * q + quad + 8] = raw1 * p.scaling;
                }
                lg[2 * q] = raw0 * p.scaling_log2;
                lg[2 * q + 1] = raw1 * p.scaling_log2;
                mx = fmaxf(mx, fmaxf(lg[2 * q], lg[2 * q + 1]));
              }
              mma_state_raise(M, across_quads_max(mx));
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float p0 = exp2f(lg[2 * q] - M.m), p1 = exp2f(lg[2 * q + 1] - M.m);
                M.l += p0 + p1;
                if (sub == 0) {
                  s_prob[warp][16 * q + quad] = __float2half_rn(p0);
                  s_prob[warp][16 * q + quad + 8] = __float2half_rn(p1);
                }
              }
            }
          } else {
            v_block_mma<BITS>(stage, lane, s_prob[warp], M, hbias);
            if (s == LOOP) {
              M.bm += __low2float(hbias) + __high2float(hbias);
              hbias = __floats2half2_rn(0.f, 0.f);
            }
          }
        } else if (!is_v) {
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
    if constexpr (kAllRows) {
      mma_state_store<BITS>(M, lane, s_merge[k & 1][warp]);
      mma_state_init(M);
      if (cur.has_tail) state_init(S);
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
    if constexpr (kAllRows) {
      if (cur.has_tail) state_store<BITS>(S, lane, s_merge[buf][kDenseWarps + warp]);
    } else {
      state_store<BITS>(S, lane, s_merge[buf][warp]);
      state_init(S);
    }
    __syncthreads();
    if (warp < 4) {
      const int c = tid;
      const int entries = (kAllRows && cur.has_tail) ? 2 * kDenseWarps : kDenseWarps;
      float mmax = -INFINITY;
#pragma unroll 8
      for (int w = 0; w < entries; ++w) mmax = fmaxf(mmax, s_merge[buf][w][128]);
      float a = 0.f, l = 0.f;
#pragma unroll 8
      for (int w = 0; w < entries; ++w) {
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

// ------------------------------------------------------------------------------ host side

// Grid of the persistent dense reader: two CTAs per SM at most, lined up with the heads where that
// helps, and never more CTAs than there are tail units, so that every CTA's share of the units is
// non-empty whatever the context lengths are.
unsigned dense_grid(int64_t batch_heads, int64_t max_context_tokens, int tail_units) {
  const int sm_count = device_sm_count();
  const int64_t ctas = kDenseCtasPerSm * static_cast<int64_t>(sm_count < 148 ? sm_count : 148);
  // A grid that is a whole multiple of the heads lines the CTAs' shares up with the heads when the
  // contexts are equal.  With one CTA per head nothing is merged across CTAs (256 heads x 2048
  // tokens: 28.6 / 44.0 us against 32.9 / 48.7 for loops 1 / 2 with 296 CTAs); a whole number of
  // CTAs per head saves the second merge of a CTA that straddles two heads, which pays as long as
  // it costs few CTAs (48 heads x 8192 as 6 CTAs per head: 23.5 / 35.6 against 27.9 / 37.9 us; 128
  // heads as two per head, 256 CTAs, is slower: 81 against 75 us for loop 2).  More heads than
  // CTAs keep the full grid: with ragged contexts fewer CTAs only cost bandwidth.
  //
  // Few heads: a head gets at most one CTA per eight units of the longest context it may hold, at
  // least eight, and never more than 32 (two partial slots per CTA, kMaxSplits per head): 16 heads x
  // 8192 tokens 16.3 / 19.3 us against 17.0 / 24.3 with eight CTAs per head, 32 heads 19.4 / 26.9
  // against 20.8 / 30.7; one CTA per four units was slower at 2048 tokens (13.8 against 12.5 us).
  // Should the contexts be so short that there are fewer units than CTAs, the kernel partitions
  // over as many CTAs as there are units and the rest leave at once.
  const int64_t units_at_most = max_context_tokens / kGroup + tail_units;
  int64_t per_head = units_at_most / 8;
  per_head = per_head < 8 ? 8 : (per_head > kMaxSplits / 2 ? kMaxSplits / 2 : per_head);
  if (batch_heads * per_head < ctas) return static_cast<unsigned>(batch_heads * per_head);
  if (batch_heads <= ctas) {
    const int64_t aligned = batch_heads * (ctas / batch_heads);
    // one CTA per head if that fills three quarters of the CTAs (160 heads x 8192 tokens on 160 CTAs
    // are 45-60 % slower than on 296), or a split of the heads that gives up at most 5 % of them
    if (aligned == batch_heads ? aligned * 4 >= ctas * 3 : aligned * 20 >= ctas * 19) return static_cast<unsigned>(aligned);
  }
  return static_cast<unsigned>(ctas);
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
  return workspace_bytes(batch_heads);
}

extern "C" int fl_workspace_status(const void* workspace, int64_t batch_heads, int32_t* status,
                                   fl_cuda_stream stream) {
  FL_REQUIRE(workspace != nullptr && status != nullptr && batch_heads > 0, "fl_workspace_status: bad argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the status word is the first word of the workspace, whatever batch_heads is
  cudaError_t err = cudaMemcpyAsync(status, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
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
  if (int rc = bind_workspace(p, layer, loop, workspace, workspace_bytes, "fl_dense_source_attention")) return rc;
  const int64_t bh = static_cast<int64_t>(layer->batch) * layer->heads;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kcur = static_cast<const __nv_bfloat16*>(current_key);
  p.vcur = static_cast<const __nv_bfloat16*>(current_value);
  p.scaling = scaling;
  p.scaling_log2 = scaling * 1.4426950408889634f;
  p.tail_units = tail_units_of_loop(loop, max_context_tokens);
  p.out = output;
  p.logits = logits;
  p.logits_stride = logits_stride;
  const unsigned grid = dense_grid(bh, max_context_tokens, p.tail_units);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaError_t err = launch_dense(layer->bits, loop, grid, s, p); err != cudaSuccess) {
    set_error("fl_dense_source_attention: %s", cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  FL_CHECK_LAUNCH("fl_dense_source_attention");
  return FL_OK;
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
// the same layout as a caller-provided workspace: status word first, then the tickets
constexpr size_t kStaticHeaderBytes = kWorkspaceHeader + (kStaticMaxBatchHeads * sizeof(int) + 255) / 256 * 256;
constexpr size_t kStaticBytes =
    kStaticHeaderBytes + static_cast<size_t>(kStaticSlots) * kPartialStride * sizeof(float);

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
void* g_static_address[kMaxDevices] = {};

// The array's name is only a host-side handle: the device address has to be asked for, once
// per device, with that device current.  The header words are cleared here so that a first
// call starts from zero whatever a previous, failed launch may have left behind.  The table of
// addresses is filled without a lock: two host threads making the FIRST call on one device at
// the same time may both run this set-up (harmless, both find the same address, but the second
// memset can land after the first thread's launch), so the first call per device belongs to one
// thread.
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
  p.status = static_cast<int*>(scratch);
  p.tickets = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + kWorkspaceHeader);
  p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + kStaticHeaderBytes);
  p.max_chunks = kStaticSlots;
  p.q = static_cast<const __nv_bfloat16*>(query);
  p.kcur = static_cast<const __nv_bfloat16*>(current_key);
  p.vcur = static_cast<const __nv_bfloat16*>(current_value);
  p.scaling = scaling;
  p.scaling_log2 = scaling * 1.4426950408889634f;
  p.tail_units = tail_units_of_loop(loop, max_context_tokens);
  p.out = output;
  p.logits = logits;
  p.logits_stride = logits_stride;
  const unsigned grid = dense_grid(bh, max_context_tokens, p.tail_units);
  if (cudaError_t err = launch_dense(layer->bits, loop, grid, s, p); err != cudaSuccess) {
    set_error("%s: %s", who, cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}

extern "C" int fl_static_status(int32_t* status, fl_cuda_stream stream) {
  FL_REQUIRE(status != nullptr, "fl_static_status: null status");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch, s)) return rc;
  cudaError_t err = cudaMemcpyAsync(status, scratch, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    set_error("fl_static_status: %s", cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  return FL_OK;
}
