// Elementwise glue of one decode step around the KV readers, one launch each instead of the
// five to eight tensor ops a framework issues: RMSNorm, residual add + RMSNorm (+ the next
// RMSNorm), the Q/K/V split with rotate-half RoPE, and SwiGLU.
//
// These restate the module arithmetic the reference's decode loop calls on an Ouro-style model
// (flashloop/engine.py:396-437 input_layernorm / project_qkv / _apply_rope, :533-537 the
// sandwich norms and fused_mlp; flashloop/weights.py:108-117) with the roundings of bfloat16
// tensor ops: every elementwise result is rounded to bfloat16 where the tensor op would have
// produced a bfloat16 tensor, reductions run in float32.
#include "fl_step_common.cuh"

namespace fl {
namespace {

constexpr int kMaxSplits = 4;  // slices of K a projection may leave to the norm that follows it

struct NormParams {
  const __nv_bfloat16* x;         // [rows][width]: the tensor to normalise, or null with `partial`
  const float* partial;           // [splits][rows][width] or null: x = bf16(sum over the slices, in order)
  int splits;
  int64_t split_stride;           // rows * width
  __nv_bfloat16* sum_out;         // [rows][width] or null: x as rebuilt from `partial`
  const __nv_bfloat16* addend;    // [rows][width] or null: bf16(addend + x) is normalised instead
  const __nv_bfloat16* residual;  // [rows][width] or null
  const __nv_bfloat16* weight;    // [width]
  const __nv_bfloat16* weight2;   // [width] or null: a second norm applied to the sum
  float eps, eps2;
  int width;
  __nv_bfloat16* out;   // [rows][width]: norm(x) (+ residual)
  __nv_bfloat16* out2;  // [rows][width] or null: norm2(out)
};

// out = [residual +] w * bf16(s * rsqrt(mean(s^2) + eps)), s = x or bf16(addend + x);
// out2 = w2 * bf16(out * rsqrt(mean(out^2) + eps2)).
// Everything the row needs (x, addend, residual, both weights) is requested before the first
// reduction, so the kernel pays one round trip to memory instead of three.
__global__ void __launch_bounds__(kStepThreads) norm_kernel(const NormParams p) {
  __shared__ float s_part[kStepThreads / 32];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* x = p.x + row * p.width;
  uint4 raw_x[kMaxChunks], raw_a[kMaxChunks], raw_r[kMaxChunks], raw_w[kMaxChunks], raw_w2[kMaxChunks];
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int e = (c * kStepThreads + threadIdx.x) * 8;
    if (e < p.width) {
      if (p.partial) {
        // the projection's float32 slices, added in order and rounded once: what a projection
        // that sums all of K itself would have stored
        float4 lo[kMaxSplits], hi[kMaxSplits];
#pragma unroll
        for (int s = 0; s < kMaxSplits; ++s) {
          if (s < p.splits) {
            const float* src = p.partial + s * p.split_stride + row * p.width + e;
            lo[s] = __ldg(reinterpret_cast<const float4*>(src));
            hi[s] = __ldg(reinterpret_cast<const float4*>(src + 4));
          }
        }
        float sum[8] = {lo[0].x, lo[0].y, lo[0].z, lo[0].w, hi[0].x, hi[0].y, hi[0].z, hi[0].w};
#pragma unroll
        for (int s = 1; s < kMaxSplits; ++s) {
          if (s < p.splits) {
            sum[0] += lo[s].x; sum[1] += lo[s].y; sum[2] += lo[s].z; sum[3] += lo[s].w;
            sum[4] += hi[s].x; sum[5] += hi[s].y; sum[6] += hi[s].z; sum[7] += hi[s].w;
          }
        }
        raw_x[c] = pack8(sum);
        if (p.sum_out) *reinterpret_cast<uint4*>(p.sum_out + row * p.width + e) = raw_x[c];
      } else {
        raw_x[c] = ldg128(x + e);
      }
      if (p.addend) raw_a[c] = ldg128(p.addend + row * p.width + e);
      if (p.residual) raw_r[c] = ldg128(p.residual + row * p.width + e);
      raw_w[c] = ldg128(p.weight + e);
      if (p.out2) raw_w2[c] = ldg128(p.weight2 + e);
    }
  }
  float v[kMaxChunks][8];
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int e = (c * kStepThreads + threadIdx.x) * 8;
    if (e < p.width) {
      unpack8(raw_x[c], v[c]);
      if (p.addend) {
        float a[8];
        unpack8(raw_a[c], a);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[c][k] = bf16_round_f(a[k] + v[c][k]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) sq = fmaf(v[c][k], v[c][k], sq);
    }
  }
  float inv = rsqrtf(block_sum(sq, s_part) / float(p.width) + p.eps);
  sq = 0.f;
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int e = (c * kStepThreads + threadIdx.x) * 8;
    if (e < p.width) {
      float w[8], r[8];
      unpack8(raw_w[c], w);
      if (p.residual) unpack8(raw_r[c], r);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float y = bf16_round_f(w[k] * bf16_round_f(v[c][k] * inv));
        if (p.residual) y = bf16_round_f(r[k] + y);
        v[c][k] = y;
        sq = fmaf(y, y, sq);
      }
      *reinterpret_cast<uint4*>(p.out + row * p.width + e) = pack8(v[c]);
    }
  }
  if (p.out2 == nullptr) return;
  inv = rsqrtf(block_sum(sq, s_part) / float(p.width) + p.eps2);
#pragma unroll
  for (int c = 0; c < kMaxChunks; ++c) {
    const int e = (c * kStepThreads + threadIdx.x) * 8;
    if (e < p.width) {
      float w[8];
      unpack8(raw_w2[c], w);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[c][k] = w[k] * bf16_round_f(v[c][k] * inv);
      *reinterpret_cast<uint4*>(p.out2 + row * p.width + e) = pack8(v[c]);
    }
  }
}

// One token per row: q/k get rotate-half RoPE, v is copied; outputs are [rows][heads*128].
__global__ void __launch_bounds__(kStepThreads)
rope_split_kernel(const __nv_bfloat16* __restrict__ q_in, const __nv_bfloat16* __restrict__ k_in,
                  const __nv_bfloat16* __restrict__ v_in, int64_t in_stride,
                  const __nv_bfloat16* __restrict__ cosv, const __nv_bfloat16* __restrict__ sinv, int heads,
                  __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                  __nv_bfloat16* __restrict__ v_out) {
  const int64_t row = blockIdx.x;
  const int width = heads * kHeadDim;
  const __nv_bfloat16* cs = cosv + row * kHeadDim;
  const __nv_bfloat16* sn = sinv + row * kHeadDim;
  // a thread handles 8 channels of the first half of a head and their partners in the second
  for (int t = threadIdx.x; t < heads * 8; t += kStepThreads) {
    const int head = t >> 3, c = (t & 7) * 8;
    float c1[8], c2[8], s1[8], s2[8];
    unpack8(ldg128(cs + c), c1);
    unpack8(ldg128(cs + 64 + c), c2);
    unpack8(ldg128(sn + c), s1);
    unpack8(ldg128(sn + 64 + c), s2);
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const __nv_bfloat16* src = (which ? k_in : q_in) + row * in_stride + head * kHeadDim;
      __nv_bfloat16* dst = (which ? k_out : q_out) + row * width + head * kHeadDim;
      float a[8], b[8], lo[8], hi[8];
      unpack8(ldg128(src + c), a);
      unpack8(ldg128(src + 64 + c), b);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        // x * cos + rotate_half(x) * sin with rotate_half = (-second half, first half)
        lo[k] = bf16_round_f(a[k] * c1[k]) + bf16_round_f(-b[k] * s1[k]);
        hi[k] = bf16_round_f(b[k] * c2[k]) + bf16_round_f(a[k] * s2[k]);
      }
      *reinterpret_cast<uint4*>(dst + c) = pack8(lo);
      *reinterpret_cast<uint4*>(dst + 64 + c) = pack8(hi);
    }
  }
  for (int e = threadIdx.x * 8; e < width; e += kStepThreads * 8) {
    *reinterpret_cast<uint4*>(v_out + row * width + e) = ldg128(v_in + row * in_stride + e);
  }
}

// out = bf16(silu(gate)) * up, gate_up = [rows][2 * width]
__global__ void __launch_bounds__(kStepThreads)
swiglu_kernel(const __nv_bfloat16* __restrict__ gate_up, int width, __nv_bfloat16* __restrict__ out) {
  const int64_t row = blockIdx.x;
  const int e = (blockIdx.y * kStepThreads + threadIdx.x) * 8;
  if (e >= width) return;
  float g[8], u[8];
  unpack8(ldg128(gate_up + row * 2 * width + e), g);
  unpack8(ldg128(gate_up + row * 2 * width + width + e), u);
#pragma unroll
  for (int k = 0; k < 8; ++k) g[k] = bf16_round_f(g[k] / (1.f + expf(-g[k]))) * u[k];
  *reinterpret_cast<uint4*>(out + row * width + e) = pack8(g);
}

}  // namespace
}  // namespace fl

using namespace fl;

extern "C" int fl_rmsnorm(const void* x, const void* addend, const void* residual, const void* weight, float eps,
                          const void* weight2, float eps2, int64_t rows, int32_t width, void* out, void* out2,
                          fl_cuda_stream stream) {
  FL_REQUIRE(x && weight && out, "fl_rmsnorm: null argument");
  FL_REQUIRE(rows >= 0 && width > 0 && width % 8 == 0 && width <= kMaxChunks * kStepThreads * 8,
             "fl_rmsnorm: width must be a multiple of 8 up to %d, got %d", kMaxChunks * kStepThreads * 8, width);
  FL_REQUIRE((weight2 == nullptr) == (out2 == nullptr), "fl_rmsnorm: weight2 and out2 go together");
  FL_REQUIRE(aligned16(x) && aligned16(addend) && aligned16(weight) && aligned16(out) && aligned16(residual) &&
                 aligned16(weight2) && aligned16(out2),
             "fl_rmsnorm: pointers must be 16-byte aligned");
  if (rows == 0) return FL_OK;
  NormParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.addend = static_cast<const __nv_bfloat16*>(addend);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.weight = static_cast<const __nv_bfloat16*>(weight);
  p.weight2 = static_cast<const __nv_bfloat16*>(weight2);
  p.eps = eps;
  p.eps2 = eps2;
  p.width = width;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out2 = static_cast<__nv_bfloat16*>(out2);
  norm_kernel<<<static_cast<unsigned>(rows), kStepThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  FL_CHECK_LAUNCH("fl_rmsnorm");
  return FL_OK;
}

extern "C" int fl_rmsnorm_partial(const float* partial, int32_t splits, const void* addend, const void* residual,
                                  const void* weight, float eps, const void* weight2, float eps2, int64_t rows,
                                  int32_t width, void* sum_out, void* out, void* out2, fl_cuda_stream stream) {
  const char* who = "fl_rmsnorm_partial";
  FL_REQUIRE(partial && weight && out, "%s: null argument", who);
  FL_REQUIRE(splits >= 1 && splits <= kMaxSplits, "%s: 1 to %d slices", who, kMaxSplits);
  FL_REQUIRE(rows >= 0 && width > 0 && width % 8 == 0 && width <= kMaxChunks * kStepThreads * 8,
             "%s: width must be a multiple of 8 up to %d, got %d", who, kMaxChunks * kStepThreads * 8, width);
  FL_REQUIRE((weight2 == nullptr) == (out2 == nullptr), "%s: weight2 and out2 go together", who);
  FL_REQUIRE(aligned16(partial) && aligned16(addend) && aligned16(weight) && aligned16(out) && aligned16(residual) &&
                 aligned16(weight2) && aligned16(out2) && aligned16(sum_out),
             "%s: pointers must be 16-byte aligned", who);
  if (rows == 0) return FL_OK;
  NormParams p{};
  p.partial = partial;
  p.splits = splits;
  p.split_stride = rows * width;
  p.sum_out = static_cast<__nv_bfloat16*>(sum_out);
  p.addend = static_cast<const __nv_bfloat16*>(addend);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.weight = static_cast<const __nv_bfloat16*>(weight);
  p.weight2 = static_cast<const __nv_bfloat16*>(weight2);
  p.eps = eps;
  p.eps2 = eps2;
  p.width = width;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out2 = static_cast<__nv_bfloat16*>(out2);
  norm_kernel<<<static_cast<unsigned>(rows), kStepThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}

extern "C" int fl_rope_split(const void* q_in, const void* k_in, const void* v_in, int64_t in_stride,
                             const void* cosv, const void* sinv, int64_t rows, int32_t heads, void* q_out,
                             void* k_out, void* v_out, fl_cuda_stream stream) {
  FL_REQUIRE(q_in && k_in && v_in && cosv && sinv && q_out && k_out && v_out, "fl_rope_split: null argument");
  FL_REQUIRE(rows >= 0 && heads > 0 && in_stride >= heads * kHeadDim && in_stride % 8 == 0,
             "fl_rope_split: bad sizes");
  FL_REQUIRE(aligned16(q_in) && aligned16(k_in) && aligned16(v_in) && aligned16(cosv) && aligned16(sinv) &&
                 aligned16(q_out) && aligned16(k_out) && aligned16(v_out),
             "fl_rope_split: pointers must be 16-byte aligned");
  if (rows == 0) return FL_OK;
  rope_split_kernel<<<static_cast<unsigned>(rows), kStepThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q_in), static_cast<const __nv_bfloat16*>(k_in),
      static_cast<const __nv_bfloat16*>(v_in), in_stride, static_cast<const __nv_bfloat16*>(cosv),
      static_cast<const __nv_bfloat16*>(sinv), heads, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_out), static_cast<__nv_bfloat16*>(v_out));
  FL_CHECK_LAUNCH("fl_rope_split");
  return FL_OK;
}

extern "C" int fl_swiglu(const void* gate_up, int64_t rows, int32_t width, void* out, fl_cuda_stream stream) {
  FL_REQUIRE(gate_up && out, "fl_swiglu: null argument");
  FL_REQUIRE(rows >= 0 && rows < (int64_t(1) << 31) && width > 0 && width % 8 == 0 &&
                 width <= 65535 * kStepThreads * 8,
             "fl_swiglu: bad sizes");
  FL_REQUIRE(aligned16(gate_up) && aligned16(out), "fl_swiglu: pointers must be 16-byte aligned");
  if (rows == 0) return FL_OK;
  const dim3 grid(static_cast<unsigned>(rows), (width / 8 + kStepThreads - 1) / kStepThreads);
  swiglu_kernel<<<grid, kStepThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), width, static_cast<__nv_bfloat16*>(out));
  FL_CHECK_LAUNCH("fl_swiglu");
  return FL_OK;
}
