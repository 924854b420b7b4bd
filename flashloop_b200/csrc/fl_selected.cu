// Gathered decode-attention readers over a list of selected logical indices: the cached-mass
// sparse delta of loops 3 and 4, the probability-weighted V sum, and the plain selected QK.
//
// Decomposition.  A pass is eight slots of one (b,h), one slot per lane quad; lane `sub` of the
// quad owns channels 32*sub .. 32*sub+31 of every row of its slot.  The passes of all (b,h) pairs
// form one sequence and every warp of the grid owns a contiguous, equally long range of it, so
// the machine is filled evenly whatever batch*heads is.  Warps are autonomous: no CTA barrier
// anywhere.  A warp meets a head in at most two pieces (the end of one head, the start of the
// next); each piece keeps its online-softmax state in registers and is published as a float32
// partial that the last-arriving warp of the head merges (an atomic ticket, nobody waits).
//
// Per piece the warp stages 64 slots at a time: index, validity, the rank-map lookups of the
// compact streams, and a class (rows in streams 0..3 / 0..2 / 0..1, BF16 tail row, nothing).  The
// slots are reordered by class inside the stage, so that the eight slots of a pass hold rows in the
// same streams and a pass runs exactly the streams it needs.  For a pass every lane then issues
// all its loads at once, straight into registers: per stream 16 bytes of K codes, 16 bytes of V
// codes and the V record's 8 metadata bytes.  While they are in flight the warp makes sure the K
// tables of the metadata groups the pass touches are in its table ring: a table is one group's
// scale and minimum rows (512 bytes, fetched with cp.async) folded with the query in place,
// w_c = q_c * scale_c in float16 in the pair order of the unpacked codes plus the float32 bias
// sum_c q_c * (min_c + centre * scale_c).  A ring of four tables per stream covers the groups
// of consecutive passes of an ascending index list; any other order only costs rebuilds.  Then
// K: unpack, float16-pair dot with the quad's table, widen; softmax update per pass; V: p * scale
// folded, float16-pair accumulate, widened every sixteen terms.
#include "fl_reader_common.cuh"

namespace fl {
namespace {

enum { kModeDelta = 0, kModePV = 1, kModeQK = 2 };
constexpr int kSelWarps = 8;
constexpr int kSelThreads = kSelWarps * kWarp;
constexpr int kStageSlots = 64;  // slots a warp stages at a time: two per lane
constexpr int kRing = 4;         // K tables a warp keeps per stream
constexpr int kTableBytes = 512;
constexpr uint32_t kFull = 0xffffffffu;

// Per-warp shared memory.
template <int STREAMS, bool TABLES>
struct alignas(16) WarpScratch {
  int rows[STREAMS][kStageSlots];  // row of the slot in stream s, relative to the (b,h) row base; -1 = none
  int tail[kStageSlots];           // tail-class entries: ring slot of the BF16 row, -1 = the current token
  float val[kStageSlots];          // weighted PV: the slot's weight; QK: the slot's position (as int bits)
  float tval[kStageSlots];         // the same for the tail-class entries
  float qf[kHeadDim];              // the query in float32
  float merge[kPartialStride];     // the piece's state: acc[128], running max, denominator
  const uint8_t* kbase[STREAMS];   // first K row / V record of this (b,h) in every stream
  const uint8_t* vbase[STREAMS];
  const __half* scale_base[STREAMS];  // first K metadata group of this (b,h)
  const __half* min_base[STREAMS];
  alignas(16) uint8_t table[TABLES ? STREAMS : 1][kRing][kTableBytes];
  alignas(16) uint8_t vstage[STREAMS][8][96];  // the V records of the current pass: codes, then 16 metadata bytes
};


template <int BITS>
__device__ __forceinline__ Codes<BITS> zero_codes() {
  Codes<BITS> c;
#pragma unroll
  for (int i = 0; i < BITS; ++i) c.w[i] = 0u;
  return c;
}
template <int BITS>
__device__ __forceinline__ Codes<BITS> load_codes_global(const uint8_t* piece) {
  Codes<BITS> c;
  if constexpr (BITS == 4) {
    const uint4 v = ldg128(piece);
    c.w[0] = v.x; c.w[1] = v.y; c.w[2] = v.z; c.w[3] = v.w;
  } else {
    const uint2 v = ldg64(piece);
    c.w[0] = v.x; c.w[1] = v.y;
  }
  return c;
}

template <int BITS, int MODE, int STREAMS>
__global__ void __launch_bounds__(kSelThreads, 2)
selected_reader_kernel(const __grid_constant__ ReaderParams p) {
  constexpr int kRowBytes = 16 * BITS;
  constexpr int kRecord = kRowBytes + 16;
  constexpr int kLaneBytes = kRowBytes / 4;
  constexpr bool kTables = MODE != kModePV;
  using Scratch = WarpScratch<STREAMS, kTables>;
  extern __shared__ __align__(128) uint8_t s_raw[];

  const LayerView& L = p.L;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int quad = lane >> 2;
  const int sub = lane & 3;
  const uint32_t lanes_below = (1u << lane) - 1u;
  Scratch& sc = reinterpret_cast<Scratch*>(s_raw)[warp];

  const int64_t gw = static_cast<int64_t>(blockIdx.x) * kSelWarps + warp;
  const int64_t n_warps = p.sel_warps;
  if (gw >= n_warps) return;
  const int64_t PH = p.passes_per_head;
  const int64_t all_passes = static_cast<int64_t>(L.batch) * L.heads * PH;
  int64_t at = all_passes * gw / n_warps;
  const int64_t range_end = all_passes * (gw + 1) / n_warps;

  while (at < range_end) {
    // ---- the piece: passes [p0, p1) of head bh
    const int64_t bh = at / PH;
    const int p0 = static_cast<int>(at - bh * PH);
    const int p1 = static_cast<int>(range_end - bh * PH < PH ? range_end - bh * PH : PH);
    const int64_t head_first = bh * PH, head_end = head_first + PH;
    const int first_owner = static_cast<int>(((head_first + 1) * n_warps - 1) / all_passes);
    const int last_owner = static_cast<int>((head_end * n_warps - 1) / all_passes);
    const int nparts = last_owner - first_owner + 1;
    const int part = static_cast<int>(gw) - first_owner;
    at += p1 - p0;

    const int b = static_cast<int>(bh / L.heads);
    const int32_t* st = L.seq_state + b * FL_STATE_WORDS;
    const int quant = st[FL_STATE_QUANT_TOKENS];
    const int tail_len = st[FL_STATE_TAIL_LEN];
    const int tail_start = st[FL_STATE_TAIL_START];
    const int cur_pos = quant + tail_len;
    const int slot_end = min(p.capacity, 8 * p1);
    const int32_t* idx_row = p.indices + bh * p.capacity;
    const uint8_t* valid_row = p.valid ? p.valid + bh * p.capacity : nullptr;
    const __nv_bfloat16* tk = L.tail_k[p.loop] + bh * L.tail_capacity * kHeadDim;
    const __nv_bfloat16* tv = L.tail_v[p.loop] + bh * L.tail_capacity * kHeadDim;

    __syncwarp();  // the previous piece's scratch is no longer read
    if (lane < STREAMS) {
      const int64_t rb = L.row_base[lane][bh], gb = L.group_base[lane][bh];
      sc.kbase[lane] = L.k_codes[lane] + rb * kRowBytes;
      sc.vbase[lane] = L.v_rows[lane] + rb * kRecord;
      sc.scale_base[lane] = L.k_scale[lane] + gb * kHeadDim;
      sc.min_base[lane] = L.k_min[lane] + gb * kHeadDim;
    }
    __half2 q01 = __floats2half2_rn(0.f, 0.f), q23 = q01;  // query channels 4*lane .. 4*lane+3
    float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if constexpr (MODE != kModePV) {
      const uint2 raw = ldg64(p.q + bh * kHeadDim + 4 * lane);
      q4 = make_float4(bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y));
      *reinterpret_cast<float4*>(&sc.qf[4 * lane]) = q4;
      q01 = __floats2half2_rn(q4.x, q4.y);
      q23 = __floats2half2_rn(q4.z, q4.w);
    }
    // the tags of the table ring: lane s * kRing + r holds the group whose table sits in ring
    // place r of stream s (-1: none)
    int tag = -1;

    OnlineState S;
    state_init(S);
    if constexpr (MODE == kModePV) S.m = 0.f;
    __half2 hacc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) hacc[i] = __floats2half2_rn(0.f, 0.f);
    int terms = 0;  // float16 terms in hacc since the last widening

    for (int stage_begin = 8 * p0; stage_begin < slot_end; stage_begin += kStageSlots) {
      const int stage_n = min(kStageSlots, slot_end - stage_begin);
      __syncwarp();  // the previous stage's lists are no longer read
      // ---- stage: two slots per lane; class 0: rows in streams 0..3, 1: 0..2, 2: 0..1, 3: BF16
      // tail row or the current token, 4: nothing to read
      int cls[2], rows[2][4], tslot[2], where[2];
      float value[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int local = lane + 32 * k;
        const int j = stage_begin + local;
        cls[k] = 4;
        tslot[k] = -1;
        value[k] = 0.f;
#pragma unroll
        for (int s = 0; s < 4; ++s) rows[k][s] = -1;
        if (local < stage_n) {
          int idx = -1;
          if (!valid_row || valid_row[j]) idx = idx_row[j];
          if constexpr (MODE == kModePV) value[k] = p.weights[bh * p.capacity + j];
          if constexpr (MODE == kModeQK) value[k] = __int_as_float(j);
          if (idx >= 0 && idx < quant) {
            rows[k][0] = idx;
            if (STREAMS >= 2) rows[k][1] = idx;
            if (STREAMS >= 3) rows[k][2] = L.rank[0][L.rank_base[b] + idx];
            if (STREAMS >= 4) rows[k][3] = L.rank[1][L.rank_base[b] + idx];
            cls[k] = (STREAMS >= 4 && rows[k][3] >= 0) ? 0 : (STREAMS >= 3 && rows[k][2] >= 0) ? 1 : 2;
          } else if (idx >= quant) {
            const bool has_current = (MODE == kModePV) ? p.vcur != nullptr : p.kcur != nullptr;
            if (idx - quant < tail_len) {
              cls[k] = 3;
              tslot[k] = (tail_start + idx - quant) % L.tail_capacity;
            } else if (idx == cur_pos && has_current) {
              cls[k] = 3;
            }
          }
          if constexpr (MODE == kModeQK) {
            if (cls[k] == 4) p.logits[bh * p.capacity + j] = 0.f;
          }
        }
      }
      // ---- positions in class order
      int base = 0, n_packed = 0;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (c == 0 && STREAMS < 4) continue;
        if (c == 1 && STREAMS < 3) continue;
        const uint32_t m0 = __ballot_sync(kFull, cls[0] == c);
        const uint32_t m1 = __ballot_sync(kFull, cls[1] == c);
        if (cls[0] == c) where[0] = base + __popc(m0 & lanes_below);
        if (cls[1] == c) where[1] = base + __popc(m0) + __popc(m1 & lanes_below);
        base += __popc(m0) + __popc(m1);
        if (c == 2) n_packed = base;
      }
      const int n_tail = base - n_packed;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        if (cls[k] < 3) {
#pragma unroll
          for (int s = 0; s < STREAMS; ++s) sc.rows[s][where[k]] = rows[k][s];
          sc.val[where[k]] = value[k];
        } else if (cls[k] == 3) {
          sc.tail[where[k] - n_packed] = tslot[k];
          sc.tval[where[k] - n_packed] = value[k];
        }
      }
      __syncwarp();

      // ---- packed passes
      for (int pass = 0; pass < n_packed; pass += 8) {
        const int e = pass + quad;
        const bool live = e < n_packed;
        int r[STREAMS];
#pragma unroll
        for (int s = 0; s < STREAMS; ++s) r[s] = live ? sc.rows[s][e] : -1;
        uint32_t on[STREAMS];  // quads of the pass that hold a row in stream s (as lane masks)
#pragma unroll
        for (int s = 0; s < STREAMS; ++s) on[s] = __ballot_sync(kFull, r[s] >= 0);

        // K tables the pass needs and the ring does not hold: fetch their raw metadata
        uint32_t fresh = 0;  // bit s * kRing + place: a table to fold once the copies have landed
        if constexpr (kTables) {
#pragma unroll
          for (int s = 0; s < STREAMS; ++s) {
            if (on[s] == 0) continue;
            const int g = r[s] >= 0 ? r[s] >> 6 : -1;
#pragma unroll
            for (int place = 0; place < kRing; ++place) {
              const uint32_t m = __ballot_sync(kFull, g >= 0 && (g & (kRing - 1)) == place);
              if (m == 0) continue;
              const int want = __shfl_sync(kFull, g, __ffs(m) - 1);
              const int have = __shfl_sync(kFull, tag, s * kRing + place);
              if (have == want) continue;
              const __half* src = (lane < 16 ? sc.scale_base[s] : sc.min_base[s]) +
                                  static_cast<int64_t>(want) * kHeadDim + (lane & 15) * 8;
              cp_async<16>(smem_u32(sc.table[s][place]) + lane * 16, src);
              if (lane == s * kRing + place) tag = want;
              fresh |= 1u << (s * kRing + place);
            }
          }
        }
        // every load of the pass at once: the V records through cp.async into the warp's stage,
        // the K codes straight into registers
        if constexpr (MODE != kModeQK) {
#pragma unroll
          for (int s = 0; s < STREAMS; ++s) {
            if (r[s] >= 0) {
              const uint8_t* record = sc.vbase[s] + static_cast<int64_t>(r[s]) * kRecord;
              const uint32_t dst = smem_u32(sc.vstage[s][quad]);
              cp_async<kLaneBytes>(dst + sub * kLaneBytes, record + sub * kLaneBytes);
              if (sub == 0) cp_async<16>(dst + kRowBytes, record + kRowBytes);
            }
          }
        }
        cp_async_commit();
        Codes<BITS> kc[STREAMS];
        if constexpr (MODE != kModePV) {
#pragma unroll
          for (int s = 0; s < STREAMS; ++s) {
            kc[s] = zero_codes<BITS>();
            if (r[s] >= 0)
              kc[s] = load_codes_global<BITS>(sc.kbase[s] + static_cast<int64_t>(r[s]) * kRowBytes + sub * kLaneBytes);
          }
        }

        float logit = 0.f;
        cp_async_wait<0>();
        __syncwarp();
        if constexpr (kTables) {
          // fold the fresh tables in place
          while (fresh) {
            const int which = __ffs(fresh) - 1;
            fresh &= fresh - 1;
            uint8_t* raw = sc.table[which / kRing][which % kRing];
            const uint2 scl = *reinterpret_cast<const uint2*>(raw + lane * 8);
            const uint2 mn = *reinterpret_cast<const uint2*>(raw + 256 + lane * 8);
            const float2 sc01 = __half22float2(as_half2(scl.x)), sc23 = __half22float2(as_half2(scl.y));
            const float2 mn01 = __half22float2(as_half2(mn.x)), mn23 = __half22float2(as_half2(mn.y));
            const float kcn = float(kCentre<BITS>);
            float bias = q4.x * fmaf(kcn, sc01.x, mn01.x);
            bias = fmaf(q4.y, fmaf(kcn, sc01.y, mn01.y), bias);
            bias = fmaf(q4.z, fmaf(kcn, sc23.x, mn23.x), bias);
            bias = fmaf(q4.w, fmaf(kcn, sc23.y, mn23.y), bias);
            bias = warp_sum(bias);
            __syncwarp();  // every lane has read the raw rows
            table_store<BITS>(reinterpret_cast<__half*>(raw), lane, q01, q23, scl);
            if (lane == 0) *reinterpret_cast<float*>(raw + 256) = bias;
          }
          __syncwarp();
          // K: every quad against the table of its row's group
#pragma unroll
          for (int s = 0; s < STREAMS; ++s) {
            if (on[s] == 0) continue;
            const int g = r[s] >= 0 ? r[s] >> 6 : -1;
            const int place = g & (kRing - 1);
            // (the shuffle runs in every lane: behind a short-circuit it would be skipped by the quads
            // without a row while the others wait for them)
            const int held = __shfl_sync(kFull, tag, s * kRing + place);
            bool ready = g >= 0 && held == g;
            if (__any_sync(kFull, ready)) {
              const uint8_t* tab = sc.table[s][ready ? place : 0];
              __half2 mult[16];
              const uint4* tab4 = reinterpret_cast<const uint4*>(tab + sub * 64);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const uint4 x = tab4[v];
                mult[4 * v + 0] = as_half2(x.x); mult[4 * v + 1] = as_half2(x.y);
                mult[4 * v + 2] = as_half2(x.z); mult[4 * v + 3] = as_half2(x.w);
              }
              const float dot = quad_sum(k_dot_fast<BITS>(kc[s], mult)) + *reinterpret_cast<const float*>(tab + 256);
              if (ready) logit += dot;
            }
            // quads whose table lost its ring place to another group of this pass (only when one
            // pass spans more than kRing groups): one group at a time through the same place
            uint32_t pending = __ballot_sync(kFull, g >= 0 && !ready);
            while (pending) {
              const int want = __shfl_sync(kFull, g, __ffs(pending) - 1);
              const int wplace = want & (kRing - 1);
              uint8_t* raw = sc.table[s][wplace];
              const __half* src = (lane < 16 ? sc.scale_base[s] : sc.min_base[s]) +
                                  static_cast<int64_t>(want) * kHeadDim + (lane & 15) * 8;
              __syncwarp();
              cp_async<16>(smem_u32(raw) + lane * 16, src);
              cp_async_commit();
              cp_async_wait<0>();
              __syncwarp();
              const uint2 scl = *reinterpret_cast<const uint2*>(raw + lane * 8);
              const uint2 mn = *reinterpret_cast<const uint2*>(raw + 256 + lane * 8);
              const float2 sc01 = __half22float2(as_half2(scl.x)), sc23 = __half22float2(as_half2(scl.y));
              const float2 mn01 = __half22float2(as_half2(mn.x)), mn23 = __half22float2(as_half2(mn.y));
              const float kcn = float(kCentre<BITS>);
              float bias = q4.x * fmaf(kcn, sc01.x, mn01.x);
              bias = fmaf(q4.y, fmaf(kcn, sc01.y, mn01.y), bias);
              bias = fmaf(q4.z, fmaf(kcn, sc23.x, mn23.x), bias);
              bias = fmaf(q4.w, fmaf(kcn, sc23.y, mn23.y), bias);
              bias = warp_sum(bias);
              __syncwarp();
              table_store<BITS>(reinterpret_cast<__half*>(raw), lane, q01, q23, scl);
              if (lane == 0) *reinterpret_cast<float*>(raw + 256) = bias;  // later passes find the table in the ring
              if (lane == s * kRing + wplace) tag = want;
              __syncwarp();
              __half2 mult[16];
              const uint4* tab4 = reinterpret_cast<const uint4*>(raw + sub * 64);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const uint4 x = tab4[v];
                mult[4 * v + 0] = as_half2(x.x); mult[4 * v + 1] = as_half2(x.y);
                mult[4 * v + 2] = as_half2(x.z); mult[4 * v + 3] = as_half2(x.w);
              }
              const float dot = quad_sum(k_dot_fast<BITS>(kc[s], mult)) + bias;
              const bool mine = g == want && !ready;
              if (mine) {
                logit += dot;
                ready = true;
              }
              pending &= ~__ballot_sync(kFull, mine);
            }
          }
        }

        if constexpr (MODE == kModeQK) {
          if (live && sub == 0) p.logits[bh * p.capacity + __float_as_int(sc.val[e])] = logit;
          continue;
        }
        float pr;
        if constexpr (MODE == kModePV) {
          pr = live ? sc.val[e] : 0.f;
        } else {
          const float x = live ? logit * p.scaling_log2 : -INFINITY;
          const float pmax = across_quads_max(x);
          if (pmax > S.m) {
            flush_pairs(hacc, S.acc);  // the float16 partial sums belong to the old maximum
            terms = 0;
            state_raise(S, pmax);
          }
          pr = live ? exp2f(x - S.m) : 0.f;
          S.l += pr;
        }
        // V
        if (terms + STREAMS > 16) {
          flush_pairs(hacc, S.acc);
          terms = 0;
        }
        const uint32_t pick = (sub < 2) ? 0x1010u : 0x3232u;
        const __half2 centre2 = __floats2half2_rn(float(kCentre<BITS>), float(kCentre<BITS>));
        const __half2 p2 = __float2half2_rn(pr);
#pragma unroll
        for (int s = 0; s < STREAMS; ++s) {
          if (on[s] == 0) continue;
          // quads without a row in this stream read what an earlier pass left in the stage: their
          // metadata is forced to zero, so the (finite) codes contribute nothing
          const uint8_t* record = sc.vstage[s][quad];
          const Codes<BITS> vc = load_codes_shared<BITS>(record + sub * kLaneBytes);
          const uint2 vmeta = *reinterpret_cast<const uint2*>(record + kRowBytes);
          const bool has = r[s] >= 0;
          const __half2 vm2 = as_half2(has ? __byte_perm(vmeta.x, 0u, pick) : 0u);
          const __half2 vs2 = as_half2(has ? __byte_perm(vmeta.y, 0u, pick) : 0u);
          const __half2 hb = __hfma2(centre2, vs2, vm2);
          v_accumulate<BITS>(vc, __hmul2(p2, vs2), hacc);
          S.vbias = fmaf(pr, __low2float(hb), S.vbias);
          ++terms;
        }
      }

      // ---- BF16 rows: tail tokens and the current token, read directly
      for (int t0 = 0; t0 < n_tail; t0 += 8) {
        const int e = t0 + quad;
        const bool live = e < n_tail;
        const int ring_slot = live ? sc.tail[e] : 0;
        float logit = 0.f;
        if constexpr (MODE != kModePV) {
          const __nv_bfloat16* krow = ring_slot < 0 ? p.kcur + bh * kHeadDim : tk + ring_slot * kHeadDim;
          logit = quad_sum(live ? bf16_row_dot<BITS>(krow, sub, sc.qf) : 0.f);
        }
        if constexpr (MODE == kModeQK) {
          if (live && sub == 0) p.logits[bh * p.capacity + __float_as_int(sc.tval[e])] = logit;
          continue;
        }
        float pr;
        if constexpr (MODE == kModePV) {
          pr = live ? sc.tval[e] : 0.f;
        } else {
          if (live && ring_slot < 0 && sub == 0 && p.cur_logits) p.cur_logits[bh] = logit * p.scaling;
          const float x = live ? logit * p.scaling_log2 : -INFINITY;
          const float pmax = across_quads_max(x);
          if (pmax > S.m) {
            flush_pairs(hacc, S.acc);
            terms = 0;
            state_raise(S, pmax);
          }
          pr = live ? exp2f(x - S.m) : 0.f;
          S.l += pr;
        }
        if (live) {
          const __nv_bfloat16* vrow = ring_slot < 0 ? p.vcur + bh * kHeadDim : tv + ring_slot * kHeadDim;
          bf16_row_accumulate<BITS>(vrow, sub, pr, S.acc);
        }
      }
    }
    if constexpr (MODE == kModeQK) continue;

    // ---- close the piece: reduce the warp's state, publish it, merge the head when it is complete
    flush_pairs(hacc, S.acc);
    __syncwarp();
    state_store<BITS>(S, lane, sc.merge);
    __syncwarp();
    float4 a = *reinterpret_cast<const float4*>(&sc.merge[4 * lane]);
    float denom = sc.merge[129];
    bool final_here = nparts == 1;
    if (!final_here) {
      // two partial slots per warp: only a warp's first piece can continue a head from the warp
      // before (slot 0) and only its last piece can leave a head to the warp after (slot 1)
      float* mine = p.partial + (2 * gw + (part > 0 ? 0 : 1)) * kPartialStride;
      *reinterpret_cast<float4*>(&mine[4 * lane]) = a;
      if (lane == 0) {
        mine[128] = sc.merge[128];
        mine[129] = denom;
      }
      __threadfence();
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        const int t = atomicAdd(p.tickets + bh, 1);
        last = t == nparts - 1;
        if (last) p.tickets[bh] = 0;  // ready for the next launch
      }
      last = __shfl_sync(kFull, last, 0);
      if (last) {
        __threadfence();
        const float* first = p.partial + (2 * static_cast<int64_t>(first_owner) + 1) * kPartialStride;
        const auto part_of = [&](int jj) { return jj > 0 ? first + (2 * jj - 1) * kPartialStride : first; };
        float gm = -INFINITY;
        for (int jj = 0; jj < nparts; ++jj) gm = fmaxf(gm, __ldcg(part_of(jj) + 128));
        a = make_float4(0.f, 0.f, 0.f, 0.f);
        denom = 0.f;
        for (int jj = 0; jj < nparts; ++jj) {
          const float* pj = part_of(jj);
          const float mj = __ldcg(pj + 128);
          const float rr = (mj == -INFINITY) ? 0.f : exp2f(mj - gm);
          const float4 x = __ldcg(reinterpret_cast<const float4*>(pj + 4 * lane));
          a.x = fmaf(x.x, rr, a.x); a.y = fmaf(x.y, rr, a.y); a.z = fmaf(x.z, rr, a.z); a.w = fmaf(x.w, rr, a.w);
          denom = fmaf(__ldcg(pj + 129), rr, denom);
        }
        final_here = true;
      }
    }
    if (final_here) {
      float4 o;
      if constexpr (MODE == kModeDelta) {
        const float inv = denom > 0.f ? 1.f / denom : 0.f;
        const float mass = p.mass[bh];
        const float4 src = *reinterpret_cast<const float4*>(p.source_out + bh * kHeadDim + 4 * lane);
        o = make_float4(mass * (a.x * inv - src.x), mass * (a.y * inv - src.y), mass * (a.z * inv - src.z),
                        mass * (a.w * inv - src.w));
      } else {
        o = a;
      }
      *reinterpret_cast<float4*>(p.out + bh * kHeadDim + 4 * lane) = o;
    }
  }
}

// ------------------------------------------------------------------------------ host side

template <int BITS, int MODE, int STREAMS>
cudaError_t launch_selected_as(unsigned grid, const ReaderParams& p, cudaStream_t s) {
  constexpr size_t kSmem = kSelWarps * sizeof(WarpScratch<STREAMS, MODE != kModePV>);
  static const cudaError_t attr = cudaFuncSetAttribute(
      selected_reader_kernel<BITS, MODE, STREAMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (attr != cudaSuccess) return attr;
  selected_reader_kernel<BITS, MODE, STREAMS><<<grid, kSelThreads, kSmem, s>>>(p);
  return cudaSuccess;
}

template <int BITS, int MODE>
cudaError_t launch_selected_bits(unsigned grid, const ReaderParams& p, cudaStream_t s) {
  switch (p.loop) {
    case 0: return launch_selected_as<BITS, MODE, 1>(grid, p, s);
    case 1: return launch_selected_as<BITS, MODE, 2>(grid, p, s);
    case 2: return launch_selected_as<BITS, MODE, 3>(grid, p, s);
    default: return launch_selected_as<BITS, MODE, 4>(grid, p, s);
  }
}

// The passes of all (b,h) pairs are dealt to the warps of the grid in equal contiguous ranges.
// Warps: at most two CTAs per multiprocessor, at most 32 per (b,h) (two partial slots each in a
// workspace of kMaxSplits slots per (b,h)), at least three passes each where there are that many.
template <int MODE>
int launch_selected(const fl_layer* layer, ReaderParams& p, cudaStream_t s, const char* who) {
  const int64_t bh = static_cast<int64_t>(layer->batch) * layer->heads;
  p.passes_per_head = (p.capacity + 7) / 8;
  const int64_t passes = bh * p.passes_per_head;
  int64_t warps = static_cast<int64_t>(2) * device_sm_count() * kSelWarps;
  warps = warps < (kMaxSplits / 2) * bh ? warps : (kMaxSplits / 2) * bh;
  const int64_t by_work = passes / 3 > kSelWarps ? passes / 3 : kSelWarps;
  warps = warps < by_work ? warps : by_work;
  warps = warps < passes ? warps : passes;
  p.sel_warps = static_cast<int>(warps);
  const unsigned grid = static_cast<unsigned>((warps + kSelWarps - 1) / kSelWarps);
  const cudaError_t err = layer->bits == 4 ? launch_selected_bits<4, MODE>(grid, p, s)
                                           : launch_selected_bits<2, MODE>(grid, p, s);
  if (err != cudaSuccess) {
    set_error("%s: %s", who, cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}

}  // namespace
}  // namespace fl

using namespace fl;

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
  FL_REQUIRE(aligned16(source_output) && aligned16(output), "%s: source_output and output must be 16-byte aligned", who);
  FL_REQUIRE(capacity > 0 && capacity < (1 << 24), "%s: capacity out of range", who);
  ReaderParams p{};
  if (int rc = bind_workspace(p, layer, loop, workspace, workspace_bytes, who)) return rc;
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
  FL_REQUIRE(aligned16(output), "%s: output must be 16-byte aligned", who);
  FL_REQUIRE(capacity > 0 && capacity < (1 << 24), "%s: capacity out of range", who);
  ReaderParams p{};
  if (int rc = bind_workspace(p, layer, loop, workspace, workspace_bytes, who)) return rc;
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

