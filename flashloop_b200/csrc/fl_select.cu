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

constexpr int kSelThreads = 512;
constexpr int kSelWarps = kSelThreads / 32;

__device__ __forceinline__ uint32_t sortable(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float block_reduce(float v, float* s_red, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = is_max ? -INFINITY : 0.f;
  for (int w = 0; w < kSelWarps; ++w) r = is_max ? fmaxf(r, s_red[w]) : r + s_red[w];
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

__global__ void __launch_bounds__(kSelThreads) select_kernel(const SelectParams p) {
  __shared__ int s_hist[256];
  __shared__ float s_red[kSelWarps];
  __shared__ int s_wgt[kSelWarps], s_weq[kSelWarps];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  __shared__ int s_base_gt, s_base_eq;

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

  // budget = min(n, max(1, ceil(n * fraction))) in double, as Python computes it
  int budget = static_cast<int>(ceil(static_cast<double>(n) * p.fraction));
  budget = min(n, max(1, budget));
  if (budget > p.capacity) budget = static_cast<int>(p.capacity);  // guarded on the host

  // softmax statistics when the inputs are logits
  float vmax = 0.f, inv_z = 1.f;
  if (p.is_logits) {
    float m = -INFINITY;
    for (int i = tid; i < n; i += kSelThreads) m = fmaxf(m, v[i]);
    vmax = block_reduce(m, s_red, true);
    float z = 0.f;
    for (int i = tid; i < n; i += kSelThreads) z += expf(v[i] - vmax);
    inv_z = 1.f / block_reduce(z, s_red, false);
  }

  // radix select: the sortable key of rank `budget` (descending)
  if (tid == 0) {
    s_prefix = 0u;
    s_need = budget;
  }
  for (int pass = 3; pass >= 0; --pass) {
    for (int i = tid; i < 256; i += kSelThreads) s_hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t himask = pass == 3 ? 0u : (0xFFFFFFFFu << (8 * (pass + 1)));
    for (int i = tid; i < n; i += kSelThreads) {
      const uint32_t key = sortable(v[i]);
      if ((key & himask) == prefix) atomicAdd(&s_hist[(key >> (8 * pass)) & 0xFF], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int need = s_need;
      int bin = 255;
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
  const uint32_t threshold = s_prefix;  // key of the budget-th largest value
  const int need_eq = s_need;           // how many equal to it are taken, lowest index first
  if (tid == 0) {
    s_base_gt = 0;
    s_base_eq = 0;
  }
  __syncthreads();

  // ordered compaction
  const int lane = tid & 31, warp = tid >> 5;
  float mass_part = 0.f;
  for (int i0 = 0; i0 < n; i0 += kSelThreads) {
    const int i = i0 + tid;
    float val = 0.f;
    bool gt = false, eq = false;
    if (i < n) {
      val = v[i];
      const uint32_t key = sortable(val);
      gt = key > threshold;
      eq = key == threshold;
    }
    const uint32_t bgt = __ballot_sync(0xffffffffu, gt);
    const uint32_t beq = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) {
      s_wgt[warp] = __popc(bgt);
      s_weq[warp] = __popc(beq);
    }
    __syncthreads();
    int gt_before = s_base_gt, eq_before = s_base_eq;
    for (int w = 0; w < warp; ++w) {
      gt_before += s_wgt[w];
      eq_before += s_weq[w];
    }
    const uint32_t lt = (1u << lane) - 1u;
    gt_before += __popc(bgt & lt);
    eq_before += __popc(beq & lt);
    const bool take = gt || (eq && eq_before < need_eq);
    if (take) {
      const int pos = gt_before + min(eq_before, need_eq);
      const float w = p.is_logits ? expf(val - vmax) * inv_z : val;
      out_idx[pos] = i;
      if (out_valid) out_valid[pos] = 1;
      if (out_w) out_w[pos] = w;
      mass_part += w;
    }
    __syncthreads();
    if (tid == 0) {
      int tg = 0, te = 0;
      for (int w = 0; w < kSelWarps; ++w) {
        tg += s_wgt[w];
        te += s_weq[w];
      }
      s_base_gt += tg;
      s_base_eq += te;
    }
    __syncthreads();
  }
  const float mass = block_reduce(mass_part, s_red, false);
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
  select_kernel<<<static_cast<unsigned>(batch) * heads, kSelThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}
