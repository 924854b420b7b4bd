// Gathered decode-attention readers over a list of selected logical indices: the cached-mass
// sparse delta of loops 3 and 4, the probability-weighted V sum, and the plain selected QK.
//
//   selected_reader_kernel  one launch over a gathered list of selected logical indices, stream by
//                           stream; the CTAs that share a (b,h) publish float32 partials that the
//                           last-arriving one merges (an atomic ticket, nobody waits).
#include "fl_reader_common.cuh"

namespace fl {
namespace {

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
constexpr int kDepth = 4;                   // passes in flight per warp (8 measured the same, 16 costs a CTA per SM)
constexpr int kPassBytes = 1024;            // K: 8 rows (<= 512 B) + one metadata group (512 B); V: 8 records (<= 640 B)
constexpr int kTailClass = 4;               // list of the slots that are tail tokens or the current token
constexpr int kGatherCtasPerSm = 2;  // 3 and 4 (fewer slots per CTA) measured 18-22 % slower
static_assert(kGatherWarps * kDepth * kPassBytes >= kGatherWarps * kPartialStride * 4,
              "the merge buffer reuses the rings");


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

}  // namespace
}  // namespace fl

using namespace fl;

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
