// Decode key selection: per (b,h) the `budget` largest of N float32 values by radix select,
// emitted in ascending index order with their softmax mass.
//
// Replaces softmax -> topk -> sort -> gather -> pad -> sum -> divide of
// flashloop/engine.py:440-481 (and select_decode_keys, flashloop/selection.py:72-88).
// Ties are broken towards the lower index.  One CTA per (b,h): four 8-bit radix passes over
// the order-preserving integer image of the floats find the value of rank `budget`; one
// ordered compaction pass (ballot prefix sums) writes the selected indices already sorted.
#include "fl_common.cuh"

namespace fl {
namespace {

constexpr int kSelThreadsMax = 1024;  // 1024 threads per head for long rows, 512 up to 4096 keys (the time of a
                                      // short row is barriers, and those are cheaper among fewer warps)
constexpr int kSelMaxSharedKeys = 50 * 1024;  // keys held in shared memory (200 KiB)

__device__ __forceinline__ uint32_t sortable(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float unsortable(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

template <int WARPS>
__device__ __forceinline__ float block_reduce(float v, float* s_red, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for (int w = 0; w < WARPS; ++w) r = is_max ? fmaxf(r, s_red[w]) : r + s_red[w];
  return r;
}

struct SelectParams {
  const float* values;
  int64_t stride;
  int heads;
  int n_keys;
  const int32_t* seq_state;
  double fraction;
  int is_logits;
  int32_t* indices;
  uint8_t* valid;
  int64_t capacity;
  int32_t* counts;
  float* mass;
  float* weights;
};

// SHARED: the keys of this (b,h) are staged once in shared memory (n <= kSelMaxSharedKeys);
// otherwise every pass re-reads the values from global memory (L2).
template <bool SHARED, int THREADS>
__global__ void __launch_bounds__(THREADS) select_kernel(const SelectParams p) {
  constexpr int kSelThreads = THREADS, kSelWarps = THREADS / 32;
  extern __shared__ uint32_t s_keys[];
  __shared__ int s_hist[256];
  __shared__ float s_red[kSelWarps];
  __shared__ int s_wgt[kSelWarps], s_weq[kSelWarps];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;

  const int64_t bh = blockIdx.x;
  const int b = static_cast<int>(bh / p.heads);
  int n = p.n_keys;
  if (p.seq_state) {
    const int32_t* st = p.seq_state + b * FL_STATE_WORDS;
    n = st[FL_STATE_QUANT_TOKENS] + st[FL_STATE_TAIL_LEN] + 1;
  }
  const float* v = p.values + bh * p.stride;
  int32_t* out_idx = p.indices + bh * p.capacity;
  uint8_t* out_valid = p.valid ? p.valid + bh * p.capacity : nullptr;
  float* out_w = p.weights ? p.weights + bh * p.capacity : nullptr;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  auto key_at = [&](int i) -> uint32_t { return SHARED ? s_keys[i] : sortable(v[i]); };

  // budget = min(n, max(1, ceil(n * fraction))) in double, as Python computes it
  int budget = static_cast<int>(ceil(static_cast<double>(n) * p.fraction));
  budget = min(n, max(1, budget));
  if (budget > p.capacity) budget = static_cast<int>(p.capacity);  // guarded on the host

  // stage the keys; softmax statistics when the inputs are logits
  float vmax = 0.f, inv_z = 1.f;
  {
    float m = -INFINITY;
    for (int i = tid; i < n; i += kSelThreads) {
      const float x = v[i];
      if (SHARED) s_keys[i] = sortable(x);
      m = fmaxf(m, x);
    }
    if (p.is_logits) {
      vmax = block_reduce<kSelWarps>(m, s_red, true);
      float z = 0.f;
      for (int i = tid; i < n; i += kSelThreads) z += expf(unsortable(key_at(i)) - vmax);
      inv_z = 1.f / block_reduce<kSelWarps>(z, s_red, false);
    }
  }
  if (tid == 0) {
    s_prefix = 0u;
    s_need = budget;
  }

  // radix select: the sortable key of rank `budget` (descending), 8 bits per pass.  Float keys
  // share their high bits, so the lanes that hold lane 0's digit are counted with one ballot and
  // one atomic; only the others fall back to their own atomics.
  for (int pass = 3; pass >= 0; --pass) {
    for (int i = tid; i < 256; i += kSelThreads) s_hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t himask = pass == 3 ? 0u : (0xFFFFFFFFu << (8 * (pass + 1)));
    for (int i0 = 0; i0 < n; i0 += kSelThreads) {
      const int i = i0 + tid;
      int digit = -1;  // not a candidate
      if (i < n) {
        const uint32_t key = key_at(i);
        if ((key & himask) == prefix) digit = (key >> (8 * pass)) & 0xFF;
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
    if (warp == 0) {
      // suffix sums over the 256 bins, 8 bins per lane: find the bin holding rank `need`
      int local[8], sum = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        local[k] = s_hist[255 - (lane * 8 + k)];  // lane 0 holds the highest bins
        sum += local[k];
      }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int need = s_need;
      int before = incl - sum;  // keys in higher bins than mine
      int found_bin = -1, found_need = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (found_bin < 0 && before < need && before + local[k] >= need) {
          found_bin = 255 - (lane * 8 + k);
          found_need = need - before;
        }
        before += local[k];
      }
      const uint32_t who = __ballot_sync(0xffffffffu, found_bin >= 0);
      if (who != 0u && lane == __ffs(who) - 1) {
        s_need = found_need;
        s_prefix = prefix | (static_cast<uint32_t>(found_bin) << (8 * pass));
      }
    }
    __syncthreads();
  }
  const uint32_t threshold = s_prefix;  // key of the budget-th largest value
  const int need_eq = s_need;           // how many equal to it are taken, lowest index first

  // ordered compaction: thread t owns the contiguous keys [t*per, (t+1)*per); one block-wide
  // exclusive scan of the (greater, equal) counts gives every thread its output position
  const int per = (n + kSelThreads - 1) / kSelThreads;
  const int begin = min(n, tid * per), end = min(n, begin + per);
  int my_gt = 0, my_eq = 0;
  for (int i = begin; i < end; ++i) {
    const uint32_t key = key_at(i);
    my_gt += key > threshold;
    my_eq += key == threshold;
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
  if (lane == 31) {
    s_wgt[warp] = inc_gt;
    s_weq[warp] = inc_eq;
  }
  __syncthreads();
  if (warp == 0) {
    int wg = lane < kSelWarps ? s_wgt[lane] : 0, we = lane < kSelWarps ? s_weq[lane] : 0;
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
    if (lane < kSelWarps) {
      s_wgt[lane] = wg - tg;  // exclusive
      s_weq[lane] = we - te;
    }
  }
  __syncthreads();
  int gt_before = s_wgt[warp] + inc_gt - my_gt;
  int eq_before = s_weq[warp] + inc_eq - my_eq;
  float mass_part = 0.f;
  for (int i = begin; i < end; ++i) {
    const uint32_t key = key_at(i);
    const bool gt = key > threshold, eq = key == threshold;
    if (gt || (eq && eq_before < need_eq)) {
      const int pos = gt_before + min(eq_before, need_eq);
      const float val = unsortable(key);
      const float w = p.is_logits ? expf(val - vmax) * inv_z : val;
      out_idx[pos] = i;
      if (out_valid) out_valid[pos] = 1;
      if (out_w) out_w[pos] = w;
      mass_part += w;
    }
    gt_before += gt;
    eq_before += eq;
  }
  const float mass = block_reduce<kSelWarps>(mass_part, s_red, false);
  if (tid == 0) {
    p.mass[bh] = mass;
    if (p.counts) p.counts[bh] = budget;
  }
  const float inv_mass = 1.f / mass;
  __syncthreads();
  for (int j = tid; j < p.capacity; j += kSelThreads) {
    if (j < budget) {
      if (out_w) out_w[j] *= inv_mass;
    } else {
      out_idx[j] = 0;
      if (out_valid) out_valid[j] = 0;
      if (out_w) out_w[j] = 0.f;
    }
  }
}

}  // namespace
}  // namespace fl

using namespace fl;

extern "C" int fl_select_decode_keys(const float* values, int64_t values_stride, int32_t batch,
                                     int32_t heads, int32_t n_keys, const int32_t* seq_state,
                                     double fraction, int32_t values_are_logits, int32_t* indices,
                                     uint8_t* valid, int64_t capacity, int32_t* counts,
                                     float* global_mass, float* selected_weights,
                                     fl_cuda_stream stream) {
  const char* who = "fl_select_decode_keys";
  FL_REQUIRE(values && indices && global_mass, "%s: null argument", who);
  FL_REQUIRE(batch > 0 && heads > 0, "%s: batch and heads must be positive", who);
  FL_REQUIRE(fraction > 0.0 && fraction <= 1.0, "%s: fraction must be in (0, 1]", who);
  FL_REQUIRE(seq_state != nullptr || n_keys > 0, "%s: n_keys must be positive", who);
  FL_REQUIRE(capacity > 0, "%s: capacity must be positive", who);
  if (!seq_state) {
    FL_REQUIRE(values_stride >= n_keys, "%s: values_stride below n_keys", who);
    int64_t budget = static_cast<int64_t>(ceil(static_cast<double>(n_keys) * fraction));
    budget = budget < 1 ? 1 : budget;
    budget = budget > n_keys ? n_keys : budget;
    FL_REQUIRE(capacity >= budget, "%s: capacity %lld below the budget %lld", who,
               static_cast<long long>(capacity), static_cast<long long>(budget));
  }
  SelectParams p;
  p.values = values;
  p.stride = values_stride;
  p.heads = heads;
  p.n_keys = n_keys;
  p.seq_state = seq_state;
  p.fraction = fraction;
  p.is_logits = values_are_logits;
  p.indices = indices;
  p.valid = valid;
  p.capacity = capacity;
  p.counts = counts;
  p.mass = global_mass;
  p.weights = selected_weights;
  // keys per head are bounded by the stride of the values (or by n_keys when it is given)
  const int64_t bound = seq_state ? values_stride : n_keys;
  const unsigned grid = static_cast<unsigned>(batch) * heads;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bound <= 4096) {
    select_kernel<true, 512><<<grid, 512, static_cast<size_t>(bound) * sizeof(uint32_t), s>>>(p);
  } else if (bound <= kSelMaxSharedKeys) {
    const size_t smem = static_cast<size_t>(bound) * sizeof(uint32_t);
    static const cudaError_t attr =
        cudaFuncSetAttribute(select_kernel<true, kSelThreadsMax>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSelMaxSharedKeys * sizeof(uint32_t));
    (void)attr;
    select_kernel<true, kSelThreadsMax><<<grid, kSelThreadsMax, smem, s>>>(p);
  } else {
    select_kernel<false, kSelThreadsMax><<<grid, kSelThreadsMax, 0, s>>>(p);
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}
