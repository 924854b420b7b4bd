// Token retention for the sparse late loops: hidden-delta score, global top-budget selection
// with prefix-scan compaction (positions + rank map), and row gather / scatter.
//
// Replaces _hidden_delta_score (flashloop/engine.py:78-81), select_prefill_tokens
// (flashloop/selection.py:26-69), the nonzero / rank-map construction around it
// (engine.py:276-277, flashloop/cache.py:281-289) and the index_select / index_copy_ row
// movement of the sparse prefill loops (flashloop/prefill.py:144, 154-158, 193-194, 237,
// 252-254).
#include "fl_common.cuh"

namespace fl {
namespace {

// ------------------------------------------------------------------------------ score
// One warp per token row: ||cur - prev|| / max(||cur||, 1e-12) in float32.
__global__ void __launch_bounds__(128)
delta_score_kernel(const __nv_bfloat16* __restrict__ cur, const __nv_bfloat16* __restrict__ prev,
                   int64_t rows, int hidden, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* a = cur + row * hidden;
  const __nv_bfloat16* b = prev + row * hidden;
  float num = 0.f, den = 0.f;
  for (int c = lane * 8; c < hidden; c += 256) {  // hidden is a multiple of 8
    const uint4 x = ldg128(a + c), y = ldg128(b + c);
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float x0 = bf16_lo(xs[k]), x1 = bf16_hi(xs[k]);
      const float d0 = x0 - bf16_lo(ys[k]), d1 = x1 - bf16_hi(ys[k]);
      num = fmaf(d0, d0, fmaf(d1, d1, num));
      den = fmaf(x0, x0, fmaf(x1, x1, den));
    }
  }
  num = warp_sum(num);
  den = warp_sum(den);
  if (lane == 0) out[row] = sqrtf(num) / fmaxf(sqrtf(den), 1e-12f);
}

// ------------------------------------------------------------------------------ retention
constexpr int kRetThreads = 1024;
constexpr int kRetWarps = kRetThreads / 32;

__device__ __forceinline__ uint32_t sortable_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct RetainParams {
  const float* scores;      // [batch][tokens]
  const uint8_t* eligible;  // [batch][tokens] or null (all eligible)
  int tokens;
  double fraction;
  int force_last;
  uint8_t* mask;       // [batch][tokens]
  int32_t* positions;  // [batch][tokens]: the retained positions, ascending, then -1
  int32_t* rank;       // [batch][tokens]: index into positions, or -1
  int32_t* count;      // [batch]
};

// One CTA per sequence.  Candidates are the eligible tokens other than a forced last token;
// `remaining` of them are chosen by radix select (larger score first, lower index on ties),
// then one ordered compaction writes the mask, the ascending positions and the rank map.
__global__ void __launch_bounds__(kRetThreads) retain_kernel(const RetainParams p) {
  extern __shared__ uint32_t s_keys[];  // sortable score, 0 for non-candidates
  __shared__ int s_hist[256];
  __shared__ int s_warp[kRetWarps];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need, s_total;
  const int b = blockIdx.x;
  const int n = p.tokens;
  const float* v = p.scores + static_cast<int64_t>(b) * n;
  const uint8_t* el = p.eligible ? p.eligible + static_cast<int64_t>(b) * n : nullptr;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int last = n - 1;

  // stage keys: candidates get the order-preserving image of their score, which is never 0
  // for a finite float (0 would be the image of an all-ones NaN); everything else gets 0
  int mine = 0;
  for (int i = tid; i < n; i += kRetThreads) {
    const bool cand = (!el || el[i]) && !(p.force_last && i == last);
    s_keys[i] = cand ? sortable_key(v[i]) : 0u;
    mine += cand;
  }
  mine = static_cast<int>(warp_sum(static_cast<float>(mine)));
  if (lane == 0) s_warp[warp] = mine;
  __syncthreads();
  if (tid == 0) {
    int candidates = 0;
    for (int w = 0; w < kRetWarps; ++w) candidates += s_warp[w];
    const int forced = p.force_last ? 1 : 0;
    int budget = static_cast<int>(ceil(static_cast<double>(n) * p.fraction));
    budget = max(1, budget);
    const int count = min(budget, candidates + forced);
    s_total = count;
    s_need = count - forced;  // how many candidates to take
    s_prefix = 0u;
  }
  __syncthreads();
  const int remaining = s_need;
  uint32_t threshold = 0xFFFFFFFFu;
  int need_eq = 0;
  if (remaining > 0) {
    for (int pass = 3; pass >= 0; --pass) {
      for (int i = tid; i < 256; i += kRetThreads) s_hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t himask = pass == 3 ? 0u : (0xFFFFFFFFu << (8 * (pass + 1)));
      for (int i0 = 0; i0 < n; i0 += kRetThreads) {
        const int i = i0 + tid;
        int digit = -1;
        if (i < n) {
          const uint32_t key = s_keys[i];
          if (key != 0u && (key & himask) == prefix) digit = (key >> (8 * pass)) & 0xFF;
        }
        const uint32_t cand = __ballot_sync(0xffffffffu, digit >= 0);
        if (cand == 0u) continue;
        const int lead = __shfl_sync(0xffffffffu, digit, __ffs(cand) - 1);
        const uint32_t same = __ballot_sync(0xffffffffu, digit == lead);
        if (digit == lead) {
          if (lane == __ffs(same) - 1) atomicAdd(&s_hist[lead], __popc(same));
        } else if (digit >= 0) {
          atomicAdd(&s_hist[digit], 1);
        }
      }
      __syncthreads();
      if (tid == 0) {
        int need = s_need, bin = 255;
        for (; bin > 0; --bin) {
          const int cnt = s_hist[bin];
          if (cnt >= need) break;
          need -= cnt;
        }
        s_need = need;
        s_prefix = prefix | (static_cast<uint32_t>(bin) << (8 * pass));
      }
      __syncthreads();
    }
    threshold = s_prefix;
    need_eq = s_need;
  }

  // ordered compaction over contiguous per-thread chunks
  const int per = (n + kRetThreads - 1) / kRetThreads;
  const int begin = min(n, tid * per), end = min(n, begin + per);
  auto classify = [&](int i, bool& gt, bool& eq) {
    const uint32_t key = s_keys[i];
    gt = (p.force_last && i == last) || (remaining > 0 && key != 0u && key > threshold);
    eq = remaining > 0 && key != 0u && key == threshold;
  };
  int my_gt = 0, my_eq = 0;
  for (int i = begin; i < end; ++i) {
    bool gt, eq;
    classify(i, gt, eq);
    my_gt += gt;
    my_eq += eq;
  }
  int inc_gt = my_gt, inc_eq = my_eq;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int ug = __shfl_up_sync(0xffffffffu, inc_gt, o);
    const int ue = __shfl_up_sync(0xffffffffu, inc_eq, o);
    if (lane >= o) {
      inc_gt += ug;
      inc_eq += ue;
    }
  }
  __shared__ int s_wgt[kRetWarps], s_weq[kRetWarps];
  if (lane == 31) {
    s_wgt[warp] = inc_gt;
    s_weq[warp] = inc_eq;
  }
  __syncthreads();
  if (warp == 0) {
    int wg = s_wgt[lane], we = s_weq[lane];
    const int tg = wg, te = we;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int ug = __shfl_up_sync(0xffffffffu, wg, o);
      const int ue = __shfl_up_sync(0xffffffffu, we, o);
      if (lane >= o) {
        wg += ug;
        we += ue;
      }
    }
    s_wgt[lane] = wg - tg;
    s_weq[lane] = we - te;
  }
  __syncthreads();
  int gt_before = s_wgt[warp] + inc_gt - my_gt;
  int eq_before = s_weq[warp] + inc_eq - my_eq;
  uint8_t* mask = p.mask + static_cast<int64_t>(b) * n;
  int32_t* positions = p.positions + static_cast<int64_t>(b) * n;
  int32_t* rank = p.rank + static_cast<int64_t>(b) * n;
  for (int i = begin; i < end; ++i) {
    bool gt, eq;
    classify(i, gt, eq);
    const bool take = gt || (eq && eq_before < need_eq);
    const int pos = gt_before + min(eq_before, need_eq);
    mask[i] = take ? 1 : 0;
    rank[i] = take ? pos : -1;
    if (take) positions[pos] = i;
    gt_before += gt;
    eq_before += eq;
  }
  const int total = s_total;
  for (int i = total + tid; i < n; i += kRetThreads) positions[i] = -1;
  if (tid == 0) p.count[b] = total;
}

// ------------------------------------------------------------------------------ row movement
// rows of `row_bytes` (multiple of 16) between a full array [outer][full_rows][row] and a
// compact array [outer][compact_rows][row]; positions/count are per sequence, `outer` entries
// share the sequence outer / per_sequence.  GATHER: compact <- full; else full <- compact.
template <bool GATHER>
__global__ void __launch_bounds__(256)
move_rows_kernel(uint8_t* __restrict__ full, uint8_t* __restrict__ compact,
                 const int32_t* __restrict__ positions, const int32_t* __restrict__ count,
                 int64_t positions_stride, int per_sequence, int64_t full_rows, int64_t compact_rows,
                 int row_bytes) {
  const int64_t outer = blockIdx.y;
  const int seq = static_cast<int>(outer / per_sequence);
  const int n = count[seq];
  const int vecs = row_bytes / 16;
  const int64_t total = static_cast<int64_t>(n) * vecs;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / vecs;
    const int v = static_cast<int>(idx % vecs);
    const int64_t t = positions[seq * positions_stride + r];
    uint4* f = reinterpret_cast<uint4*>(full + (outer * full_rows + t) * row_bytes) + v;
    uint4* c = reinterpret_cast<uint4*>(compact + (outer * compact_rows + r) * row_bytes) + v;
    if (GATHER) *c = *f; else *f = *c;
  }
}

}  // namespace
}  // namespace fl

using namespace fl;

extern "C" int fl_hidden_delta_score(const void* current, const void* previous, int64_t rows,
                                     int32_t hidden, float* scores, fl_cuda_stream stream) {
  FL_REQUIRE(current && previous && scores, "fl_hidden_delta_score: null argument");
  FL_REQUIRE(rows > 0 && hidden > 0 && hidden % 8 == 0, "fl_hidden_delta_score: hidden must be a multiple of 8");
  FL_REQUIRE(aligned16(current) && aligned16(previous), "fl_hidden_delta_score: inputs must be 16-byte aligned");
  delta_score_kernel<<<static_cast<unsigned>((rows + 3) / 4), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(current), static_cast<const __nv_bfloat16*>(previous), rows, hidden, scores);
  FL_CHECK_LAUNCH("fl_hidden_delta_score");
  return FL_OK;
}

extern "C" int fl_select_prefill_tokens(const float* scores, const uint8_t* eligible, int32_t batch,
                                        int32_t tokens, double fraction, int32_t force_last_token,
                                        uint8_t* mask, int32_t* positions, int32_t* rank,
                                        int32_t* count, fl_cuda_stream stream) {
  const char* who = "fl_select_prefill_tokens";
  FL_REQUIRE(scores && mask && positions && rank && count, "%s: null argument", who);
  FL_REQUIRE(batch > 0 && tokens > 0, "%s: batch and tokens must be positive", who);
  FL_REQUIRE(fraction > 0.0 && fraction <= 1.0, "%s: fraction must be in (0, 1]", who);
  const size_t smem = static_cast<size_t>(tokens) * sizeof(uint32_t);
  FL_REQUIRE(smem <= 200 * 1024, "%s: at most 51200 tokens per sequence", who);
  static const cudaError_t attr =
      cudaFuncSetAttribute(retain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  (void)attr;
  RetainParams p;
  p.scores = scores;
  p.eligible = eligible;
  p.tokens = tokens;
  p.fraction = fraction;
  p.force_last = force_last_token ? 1 : 0;
  p.mask = mask;
  p.positions = positions;
  p.rank = rank;
  p.count = count;
  retain_kernel<<<batch, kRetThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}

namespace {
int move_rows(bool gather, void* full, void* compact, const int32_t* positions, const int32_t* count,
              int64_t positions_stride, int64_t outer, int32_t per_sequence, int64_t full_rows,
              int64_t compact_rows, int32_t row_bytes, cudaStream_t stream, const char* who) {
  FL_REQUIRE(full && compact && positions && count, "%s: null argument", who);
  FL_REQUIRE(outer > 0 && outer <= 65535 && per_sequence > 0 && outer % per_sequence == 0,
             "%s: outer must be a positive multiple of per_sequence (at most 65535)", who);
  FL_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "%s: row_bytes must be a multiple of 16", who);
  FL_REQUIRE(aligned16(full) && aligned16(compact), "%s: arrays must be 16-byte aligned", who);
  FL_REQUIRE(full_rows > 0 && compact_rows > 0, "%s: row counts must be positive", who);
  const int64_t work = compact_rows * (row_bytes / 16);
  const unsigned gx = static_cast<unsigned>(work / 256 + 1 < 1024 ? work / 256 + 1 : 1024);
  const dim3 grid(gx, static_cast<unsigned>(outer));
  if (gather) {
    move_rows_kernel<true><<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(full), static_cast<uint8_t*>(compact),
                                                    positions, count, positions_stride, per_sequence, full_rows,
                                                    compact_rows, row_bytes);
  } else {
    move_rows_kernel<false><<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(full), static_cast<uint8_t*>(compact),
                                                     positions, count, positions_stride, per_sequence, full_rows,
                                                     compact_rows, row_bytes);
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}
}  // namespace

extern "C" int fl_gather_rows(const void* full, void* compact, const int32_t* positions,
                              const int32_t* count, int64_t positions_stride, int64_t outer,
                              int32_t per_sequence, int64_t full_rows, int64_t compact_rows,
                              int32_t row_bytes, fl_cuda_stream stream) {
  return move_rows(true, const_cast<void*>(full), compact, positions, count, positions_stride, outer,
                   per_sequence, full_rows, compact_rows, row_bytes, static_cast<cudaStream_t>(stream),
                   "fl_gather_rows");
}

extern "C" int fl_scatter_rows(void* full, const void* compact, const int32_t* positions,
                               const int32_t* count, int64_t positions_stride, int64_t outer,
                               int32_t per_sequence, int64_t full_rows, int64_t compact_rows,
                               int32_t row_bytes, fl_cuda_stream stream) {
  return move_rows(false, full, const_cast<void*>(compact), positions, count, positions_stride, outer,
                   per_sequence, full_rows, compact_rows, row_bytes, static_cast<cudaStream_t>(stream),
                   "fl_scatter_rows");
}
