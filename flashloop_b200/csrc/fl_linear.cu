// The projections of a decode step: out[m][n] = sum_k x[m][k] * W[n][k] for at most sixteen rows
// (one token per sequence), bfloat16 in and out, float32 accumulation.
//
// With sixteen rows the product is a stream over the weights: every weight byte is read once and
// used sixteen times, 16 flop per byte, far below what the tensor pipe needs to be busy, so the
// bound is HBM.  A library GEMM at this shape spends its time in tiles built for hundreds of rows;
// here a CTA owns eight (or sixteen) weight rows at a time, its eight warps split K, and every lane
// keeps 16-byte weight loads in flight.  The multiply-adds go to mma.sync.m16n8k16 (the sixteen
// rows of x are exactly the tile's M): a lane's 16 bytes of a weight row are eight consecutive k,
// fed to two mmas, and since a dot product does not care about the order of its terms the mma's k
// index is simply mapped to "lane j holds k0 + 8j .. 8j+7", for x and W alike, so both operands
// are plain 16-byte loads.  x (32 KB .. 176 KB) stays in L1/L2.
//
//   linear_rows_kernel  one tile of eight weight rows (or a pair of tiles) per CTA, the weights
//                       through registers (two sets, the next batch in flight while this one is
//                       multiplied).  Used where few output rows leave few tiles (o_proj,
//                       down_proj): it uses almost no shared memory, so L1 keeps the whole of x
//                       (128 KB of float32 rows, 176 KB).
//   linear_ring_kernel  pairs of tiles, persistent CTAs (three per SM), the weights through a
//                       per-lane ring of 16-byte asynchronous copies in shared memory that runs on
//                       across the pairs of a CTA.  Used for the wide projections (Q/K/V, gate/up,
//                       more than 4096 output rows) when they have at least two pairs per SM
//                       (a tensor-parallel rank's slice falls back to the register version with a
//                       CTA per pair; from four pairs per SM on, one CTA of sixteen warps per SM
//                       that keeps its x fragments in registers): 7.5 / 11.0 / 36 us against 8.6 / 12.8 / 43 for
//                       the register version at 25 / 46 / 201 MB of weights.  Measured on the way: a
//                       deeper ring is slower (8 stages 14.3 us, 16 stages 17.1 us for gate/up; the
//                       shared memory comes out of L1, where x lives), and a read of the same bytes
//                       in the same pattern without the arithmetic takes 8.5 us.
//   linear_splitk_kernel  float32 partial sums over slices of K for o_proj / down_proj on one GPU;
//                       described where it is defined.
//
// Mode 1 computes SwiGLU on the way out: a CTA takes eight rows of the gate half and the same
// eight of the up half of a fused [2F][K] weight and writes bf16(silu(bf16 gate)) * bf16 up, the
// roundings of the separate launches it replaces.  Mode 2 is the fused Q/K/V projection of one
// token per row with rotate-half RoPE on the way out: a CTA takes eight features of the first half of
// a head and their partners 64 further on, and writes q and k rotated and v as it is, each in
// [rows][heads * 128] (the layout the readers take).  x may be float32 (the readers' output): it is
// rounded to bfloat16 as it is loaded, which is what a separate conversion would have stored.
#include "fl_step_common.cuh"

namespace fl {
namespace {

constexpr int kLinearWarps = 8;
constexpr int kLinearThreads = kLinearWarps * 32;
constexpr int kChunk = 32;  // k per warp-wide 16-byte load of one weight row (4 lanes x 8)
constexpr int kRing = 4;    // stages of a warp's weight ring: three chunks in flight
constexpr int kRingCtasPerSm = 3;
// the ring kernel with the rows of x in registers: one CTA of sixteen warps per SM
constexpr int kWideWarps = 16, kWideRing = 8;
constexpr int kWideChunks = 4;  // chunks of K per warp whose x fragments a lane keeps (K <= 2048)

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

struct LinearParams {
  const void* x;           // [rows][k], bfloat16 or float32
  const __nv_bfloat16* w;  // [n][k]
  __nv_bfloat16* out;      // [rows][out_width]
  int rows, k, out_width;
  int splits;      // split-K kernel: slices of K, one per CTA of a column
  float* partial;  // split-K kernel: [splits][rows][out_width] float32
  int groups;      // ring kernel: tile pairs in all; a CTA takes pairs blockIdx.x, blockIdx.x + gridDim.x, ...
  int up_offset;  // mode 1: the up rows start this many weight rows after the gate rows
  // mode 2
  int heads;
  const __nv_bfloat16* cosv;  // [rows][128]
  const __nv_bfloat16* sinv;
  __nv_bfloat16* k_out;
  __nv_bfloat16* v_out;
};

// Eight consecutive values of a row of x as four bfloat16 pairs.
template <bool F32>
__device__ __forceinline__ uint4 load_x8(const void* x, int64_t element) {
  if constexpr (F32) {
    const float* src = static_cast<const float*>(x) + element;
    const float4 a = __ldg(reinterpret_cast<const float4*>(src));
    const float4 b = __ldg(reinterpret_cast<const float4*>(src + 4));
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
    const __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
    return make_uint4(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1),
                      *reinterpret_cast<const uint32_t*>(&p2), *reinterpret_cast<const uint32_t*>(&p3));
  } else {
    return ldg128(static_cast<const __nv_bfloat16*>(x) + element);
  }
}

// The outputs (m, n0 + n [+ 8 t]) of a tile group from their float32 sums.
template <int TILES, int MODE>
__device__ __forceinline__ void store_outputs(const LinearParams& p, int n0, int m, int n, const float (&sum)[TILES]) {
  if constexpr (MODE == 2) {
    const int width = p.heads * 128;
    const int section = n0 / width;  // 0: q, 1: k, 2: v
    const int c = (n0 & 127) + n;    // feature within the head, first half
    const float a = bf16_round_f(sum[0]), b = bf16_round_f(sum[1]);
    __nv_bfloat16* dst = (section == 0 ? p.out : (section == 1 ? p.k_out : p.v_out)) +
                         static_cast<int64_t>(m) * width + (n0 - section * width) + n;
    if (section < 2) {
      // x * cos + rotate_half(x) * sin with rotate_half = (-second half, first half)
      const float c1 = __bfloat162float(p.cosv[m * 128 + c]), s1 = __bfloat162float(p.sinv[m * 128 + c]);
      const float c2 = __bfloat162float(p.cosv[m * 128 + c + 64]), s2 = __bfloat162float(p.sinv[m * 128 + c + 64]);
      dst[0] = __float2bfloat16_rn(bf16_round_f(a * c1) + bf16_round_f(-b * s1));
      dst[64] = __float2bfloat16_rn(bf16_round_f(b * c2) + bf16_round_f(a * s2));
    } else {
      dst[0] = __float2bfloat16_rn(a);
      dst[64] = __float2bfloat16_rn(b);
    }
  } else {
    __nv_bfloat16* dst = p.out + static_cast<int64_t>(m) * p.out_width + n0 + n;
    if constexpr (MODE == 1) {
      const float gate = bf16_round_f(sum[0]), up = bf16_round_f(sum[1]);
      *dst = __float2bfloat16_rn(bf16_round_f(gate / (1.f + expf(-gate))) * up);
    } else {
#pragma unroll
      for (int t = 0; t < TILES; ++t) dst[8 * t] = __float2bfloat16_rn(sum[t]);
    }
  }
}

// TILES weight-row tiles of eight per CTA.  MODE 0: adjacent tiles, TILES * 8 outputs per row.
// MODE 1 (TILES == 2): tile 0 = gate rows, tile 1 = up rows, eight outputs per row.
// MODE 2 (TILES == 2): tile 0 = features c0 .. c0+7 of a head of q, k or v, tile 1 = c0+64 .. c0+71.
template <int TILES, int MODE, bool F32>
__global__ void __launch_bounds__(kLinearThreads, TILES == 1 ? 3 : 2) linear_rows_kernel(const LinearParams p) {
  __shared__ float s_red[kLinearWarps][TILES][16][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, j = lane & 3;
  // first weight row of tile 0
  const int n0 = MODE == 2 ? (blockIdx.x >> 3) * 128 + (blockIdx.x & 7) * 8 : blockIdx.x * (MODE == 1 ? 8 : 8 * TILES);
  const int K = p.k;
  const __nv_bfloat16* wrow[TILES];
#pragma unroll
  for (int t = 0; t < TILES; ++t) {
    const int n = MODE == 1 ? n0 + t * p.up_offset : (MODE == 2 ? n0 + 64 * t : n0 + 8 * t);
    wrow[t] = p.w + static_cast<int64_t>(n + g) * K + 8 * j;
  }
  const bool row_a = g < p.rows, row_b = g + 8 < p.rows;
  const int64_t xa = static_cast<int64_t>(g) * K + 8 * j, xb = static_cast<int64_t>(g + 8) * K + 8 * j;
  float acc[TILES][4];
#pragma unroll
  for (int t = 0; t < TILES; ++t)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[t][c] = 0.f;

  // chunk c of a row is k in [32c, 32c + 32); the warps take chunks warp, warp + 8, ...; a batch is
  // kDepth of a warp's chunks, and the loads of the next batch are in flight while this one is
  // multiplied (two register sets, the loop unrolled by hand)
  const int chunks = K / kChunk;
  constexpr int kDepth = 2, kStride = kLinearWarps * kDepth;
  const auto load_batch = [&](int c0, uint4 (&wv)[kDepth][TILES], uint4 (&va)[kDepth], uint4 (&vb)[kDepth]) {
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      const int c = c0 + d * kLinearWarps;
      if (c < chunks) {
#pragma unroll
        for (int t = 0; t < TILES; ++t) wv[d][t] = load_stream(wrow[t] + c * kChunk);
      }
    }
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      const int c = c0 + d * kLinearWarps;
      va[d] = make_uint4(0u, 0u, 0u, 0u);
      vb[d] = make_uint4(0u, 0u, 0u, 0u);
      if (c < chunks) {
        if (row_a) va[d] = load_x8<F32>(p.x, xa + c * kChunk);
        if (row_b) vb[d] = load_x8<F32>(p.x, xb + c * kChunk);
      }
    }
  };
  const auto multiply = [&](int c0, const uint4 (&wv)[kDepth][TILES], const uint4 (&va)[kDepth],
                            const uint4 (&vb)[kDepth]) {
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
      if (c0 + d * kLinearWarps < chunks) {
#pragma unroll
        for (int t = 0; t < TILES; ++t) {
          mma_bf16_16816(acc[t], va[d].x, vb[d].x, va[d].y, vb[d].y, wv[d][t].x, wv[d][t].y);
          mma_bf16_16816(acc[t], va[d].z, vb[d].z, va[d].w, vb[d].w, wv[d][t].z, wv[d][t].w);
        }
      }
    }
  };
  uint4 w0[kDepth][TILES], a0[kDepth], b0[kDepth], w1[kDepth][TILES], a1[kDepth], b1[kDepth];
  int c = warp;
  if (c < chunks) {
    load_batch(c, w0, a0, b0);
    while (true) {
      const int cn = c + kStride;
      if (cn < chunks) load_batch(cn, w1, a1, b1);
      multiply(c, w0, a0, b0);
      if (cn >= chunks) break;
      c = cn + kStride;
      if (c < chunks) load_batch(c, w0, a0, b0);
      multiply(cn, w1, a1, b1);
      if (c >= chunks) break;
    }
  }
#pragma unroll
  for (int t = 0; t < TILES; ++t) {
    s_red[warp][t][g][2 * j] = acc[t][0];
    s_red[warp][t][g][2 * j + 1] = acc[t][1];
    s_red[warp][t][g + 8][2 * j] = acc[t][2];
    s_red[warp][t][g + 8][2 * j + 1] = acc[t][3];
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int m = threadIdx.x >> 3, n = threadIdx.x & 7;
    float sum[TILES];
#pragma unroll
    for (int t = 0; t < TILES; ++t) {
      sum[t] = 0.f;
#pragma unroll
      for (int w = 0; w < kLinearWarps; ++w) sum[t] += s_red[w][t][m][n];
    }
    if (m < p.rows) store_outputs<TILES, MODE>(p, n0, m, n, sum);
  }
}

// The ring version.  A tile group is TILES weight-row tiles of eight, laid out as in linear_rows_kernel.
template <int TILES, int MODE>
__device__ __forceinline__ int group_first_row(int group) {
  if constexpr (MODE == 2) return (group >> 3) * 128 + (group & 7) * 8;
  return group * (MODE == 1 ? 8 : 8 * TILES);
}

// WIDE: sixteen warps, one CTA per SM, a ring of eight stages, and the x fragments of the warp's
// chunks loaded once into registers (K <= 2048) instead of through L1 at every pair: the rows of x
// then cross from L2 once per SM and not once per pair.
template <int TILES, int MODE, bool F32, bool WIDE>
__global__ void __launch_bounds__(WIDE ? kWideWarps * 32 : kLinearThreads, WIDE ? 1 : kRingCtasPerSm)
linear_ring_kernel(const LinearParams p) {
  constexpr int kLinearWarps = WIDE ? kWideWarps : fl::kLinearWarps;
  constexpr int kRing = WIDE ? kWideRing : fl::kRing;
  extern __shared__ __align__(16) uint8_t s_ring[];  // [warp][kRing][TILES][32] x 16 bytes
  __shared__ float s_red[2][kLinearWarps][TILES][16][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, j = lane & 3;
  const int K = p.k;
  const bool row_a = g < p.rows, row_b = g + 8 < p.rows;
  const int64_t xa = static_cast<int64_t>(g) * K + 8 * j, xb = static_cast<int64_t>(g + 8) * K + 8 * j;

  // chunk c of a row is k in [32c, 32c + 32); the warps take chunks warp, warp + 8, ... of every
  // group of the CTA.  A lane's 16 bytes of a weight row go through a ring of kRing stages in
  // shared memory that only this lane reads back, filled by 16-byte asynchronous copies which
  // run on across the groups: while a group's sums are joined, the next one's weights are under way.
  const int chunks = K / kChunk;
  const int n_mine = chunks > warp ? (chunks - warp + kLinearWarps - 1) / kLinearWarps : 0;
  uint8_t* const mine = s_ring + (warp * kRing * TILES * 32 + lane) * 16;
  const uint32_t mine_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(mine));
  const auto weight_at = [&](int group, int t) {
    const int n0 = group_first_row<TILES, MODE>(group);
    const int n = MODE == 1 ? n0 + t * p.up_offset : (MODE == 2 ? n0 + 64 * t : n0 + 8 * t);
    return p.w + static_cast<int64_t>(n + g) * K + 8 * j;
  };
  int issue_group = blockIdx.x, issue_chunk = 0, issue_stage = 0;
  const __nv_bfloat16* issue_w[TILES];
#pragma unroll
  for (int t = 0; t < TILES; ++t) issue_w[t] = weight_at(min(issue_group, p.groups - 1), t);
  const auto issue = [&]() {
    if (issue_group < p.groups && n_mine > 0) {
      const int c = warp + kLinearWarps * issue_chunk;
#pragma unroll
      for (int t = 0; t < TILES; ++t) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(mine_u32 + (issue_stage * TILES + t) * 512),
                     "l"(issue_w[t] + c * kChunk)
                     : "memory");
      }
      if (++issue_chunk == n_mine) {
        issue_chunk = 0;
        issue_group += gridDim.x;
        if (issue_group < p.groups) {
#pragma unroll
          for (int t = 0; t < TILES; ++t) issue_w[t] = weight_at(issue_group, t);
        }
      }
    }
    issue_stage = (issue_stage + 1) & (kRing - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const auto load_x = [&](int i, uint4& va, uint4& vb) {
    va = make_uint4(0u, 0u, 0u, 0u);
    vb = make_uint4(0u, 0u, 0u, 0u);
    if (i < n_mine) {
      const int c = warp + kLinearWarps * i;
      if (row_a) va = load_x8<F32>(p.x, xa + c * kChunk);
      if (row_b) vb = load_x8<F32>(p.x, xb + c * kChunk);
    }
  };
#pragma unroll
  for (int i = 0; i < kRing - 1; ++i) issue();
  uint4 xra[WIDE ? kWideChunks : 1], xrb[WIDE ? kWideChunks : 1];
  if constexpr (WIDE) {
#pragma unroll
    for (int i = 0; i < kWideChunks; ++i) load_x(i, xra[i], xrb[i]);
  }

  int stage = 0, round = 0;
  for (int group = blockIdx.x; group < p.groups; group += gridDim.x, round ^= 1) {
    float acc[TILES][4];
#pragma unroll
    for (int t = 0; t < TILES; ++t)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[t][c] = 0.f;
    if constexpr (WIDE) {
#pragma unroll
      for (int i = 0; i < kWideChunks; ++i) {
        if (i < n_mine) {
          issue();  // into the stage this lane read one step ago
          asm volatile("cp.async.wait_group %0;" ::"n"(kRing - 1) : "memory");
#pragma unroll
          for (int t = 0; t < TILES; ++t) {
            const uint4 wv = *reinterpret_cast<const uint4*>(mine + (stage * TILES + t) * 512);
            mma_bf16_16816(acc[t], xra[i].x, xrb[i].x, xra[i].y, xrb[i].y, wv.x, wv.y);
            mma_bf16_16816(acc[t], xra[i].z, xrb[i].z, xra[i].w, xrb[i].w, wv.z, wv.w);
          }
          stage = (stage + 1) & (kRing - 1);
        }
      }
    } else {
      uint4 va[2], vb[2];
      load_x(0, va[0], vb[0]);
      for (int i = 0; i < n_mine; i += 2) {
  #pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (i + h < n_mine) {
            issue();  // into the stage this lane read one step ago
            load_x(i + h + 1, va[h ^ 1], vb[h ^ 1]);
            asm volatile("cp.async.wait_group %0;" ::"n"(kRing - 1) : "memory");
  #pragma unroll
            for (int t = 0; t < TILES; ++t) {
              const uint4 wv = *reinterpret_cast<const uint4*>(mine + (stage * TILES + t) * 512);
              mma_bf16_16816(acc[t], va[h].x, vb[h].x, va[h].y, vb[h].y, wv.x, wv.y);
              mma_bf16_16816(acc[t], va[h].z, vb[h].z, va[h].w, vb[h].w, wv.z, wv.w);
            }
            stage = (stage + 1) & (kRing - 1);
          }
        }
      }
    }
    float(*red)[TILES][16][8] = s_red[round];
#pragma unroll
    for (int t = 0; t < TILES; ++t) {
      red[warp][t][g][2 * j] = acc[t][0];
      red[warp][t][g][2 * j + 1] = acc[t][1];
      red[warp][t][g + 8][2 * j] = acc[t][2];
      red[warp][t][g + 8][2 * j + 1] = acc[t][3];
    }
    __syncthreads();  // the other buffer is written next: nobody returns here before its readers are past
    if (threadIdx.x < 128) {
      const int n0 = group_first_row<TILES, MODE>(group);
      const int m = threadIdx.x >> 3, n = threadIdx.x & 7;
      float sum[TILES];
#pragma unroll
      for (int t = 0; t < TILES; ++t) {
        sum[t] = 0.f;
#pragma unroll
        for (int w = 0; w < kLinearWarps; ++w) sum[t] += red[w][t][m][n];
      }
      if (m < p.rows) store_outputs<TILES, MODE>(p, n0, m, n, sum);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}


// Split-K version for the projections with few output rows (o_proj, down_proj).  There every CTA of
// the kernels above reads the whole of x (128 - 176 KB), and with one set of CTAs per SM that is more
// bytes from L2 than the weights themselves (19 MB against 8 for o_proj, 26 against 23 for
// down_proj).  Here a CTA owns one of `splits` slices of K for good: the x fragments of the slice
// live in registers, and the CTA walks the 8-row tiles of its column (blockIdx.x / splits) with the
// weight ring running on across them.  It writes float32 partial sums [splits][rows][out]; whoever
// reads them adds the slices in order and rounds once (fl_rmsnorm_partial).  Measured at 16 rows:
// o_proj (float32 x) 5.0 us against 6.2, down_proj 8.3 us against 9.2, with four slices.
constexpr int kSplitWarps = 16, kSplitRing = 4, kSplitXChunks = 3;

template <bool F32>
__global__ void __launch_bounds__(kSplitWarps * 32, 1) linear_splitk_kernel(const LinearParams p) {
  extern __shared__ __align__(16) uint8_t s_ring[];  // [warp][kSplitRing][32] x 16 bytes
  __shared__ float s_red[2][kSplitWarps][16][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, j = lane & 3;
  const int K = p.k;
  const int slice = blockIdx.x % p.splits, column = blockIdx.x / p.splits, columns = gridDim.x / p.splits;
  const int slice_chunks = K / kChunk / p.splits;
  const int first_chunk = slice * slice_chunks + warp;
  const int n_mine = slice_chunks > warp ? (slice_chunks - warp + kSplitWarps - 1) / kSplitWarps : 0;
  const int tiles = p.out_width / 8;
  const bool row_a = g < p.rows, row_b = g + 8 < p.rows;
  const int64_t xa = static_cast<int64_t>(g) * K + 8 * j, xb = static_cast<int64_t>(g + 8) * K + 8 * j;
  uint8_t* const mine = s_ring + (warp * kSplitRing * 32 + lane) * 16;
  const uint32_t mine_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(mine));

  int issue_tile = column, issue_chunk = 0, issue_stage = 0;
  const auto issue = [&]() {
    if (issue_tile < tiles && n_mine > 0) {
      const __nv_bfloat16* w = p.w + static_cast<int64_t>(issue_tile * 8 + g) * K + 8 * j +
                               (first_chunk + kSplitWarps * issue_chunk) * kChunk;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(mine_u32 + issue_stage * 512), "l"(w) : "memory");
      if (++issue_chunk == n_mine) {
        issue_chunk = 0;
        issue_tile += columns;
      }
    }
    issue_stage = issue_stage + 1 == kSplitRing ? 0 : issue_stage + 1;
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int i = 0; i < kSplitRing - 1; ++i) issue();
  uint4 xra[kSplitXChunks], xrb[kSplitXChunks];
#pragma unroll
  for (int i = 0; i < kSplitXChunks; ++i) {
    xra[i] = make_uint4(0u, 0u, 0u, 0u);
    xrb[i] = make_uint4(0u, 0u, 0u, 0u);
    if (i < n_mine) {
      const int c = first_chunk + kSplitWarps * i;
      if (row_a) xra[i] = load_x8<F32>(p.x, xa + c * kChunk);
      if (row_b) xrb[i] = load_x8<F32>(p.x, xb + c * kChunk);
    }
  }
  int stage = 0, round = 0;
  for (int tile = column; tile < tiles; tile += columns, round ^= 1) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kSplitXChunks; ++i) {
      if (i < n_mine) {
        issue();  // into the stage this lane read one step ago
        asm volatile("cp.async.wait_group %0;" ::"n"(kSplitRing - 1) : "memory");
        const uint4 wv = *reinterpret_cast<const uint4*>(mine + stage * 512);
        mma_bf16_16816(acc, xra[i].x, xrb[i].x, xra[i].y, xrb[i].y, wv.x, wv.y);
        mma_bf16_16816(acc, xra[i].z, xrb[i].z, xra[i].w, xrb[i].w, wv.z, wv.w);
        stage = stage + 1 == kSplitRing ? 0 : stage + 1;
      }
    }
    float(*red)[16][8] = s_red[round];
    red[warp][g][2 * j] = acc[0];
    red[warp][g][2 * j + 1] = acc[1];
    red[warp][g + 8][2 * j] = acc[2];
    red[warp][g + 8][2 * j + 1] = acc[3];
    __syncthreads();  // the other buffer is written next: nobody returns here before its readers are past
    if (threadIdx.x < 128) {
      const int m = threadIdx.x >> 3, n = threadIdx.x & 7;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kSplitWarps; ++w) sum += red[w][m][n];
      if (m < p.rows) p.partial[(static_cast<int64_t>(slice) * p.rows + m) * p.out_width + tile * 8 + n] = sum;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

}  // namespace
}  // namespace fl

using namespace fl;

namespace fl {
namespace {
template <int TILES, int MODE>
void launch_linear(bool f32, unsigned grid, cudaStream_t s, const LinearParams& p) {
  if (f32) {
    linear_rows_kernel<TILES, MODE, true><<<grid, kLinearThreads, 0, s>>>(p);
  } else {
    linear_rows_kernel<TILES, MODE, false><<<grid, kLinearThreads, 0, s>>>(p);
  }
}
// Pairs of tiles: the ring kernel where there are at least two pairs per SM, else (a tensor-parallel
// rank's slice of a projection) a CTA per pair with the weights through registers.
constexpr int kRingMinGroups = 2 * 148;

template <int MODE, bool F32, bool WIDE>
void launch_ring_as(int groups, cudaStream_t s, const LinearParams& p) {
  constexpr int kWarps = WIDE ? kWideWarps : kLinearWarps;
  constexpr int kSmem = kWarps * (WIDE ? kWideRing : kRing) * 2 * 512;
  static const cudaError_t attr = cudaFuncSetAttribute(linear_ring_kernel<2, MODE, F32, WIDE>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  (void)attr;
  const int slots = 148 * (WIDE ? 1 : kRingCtasPerSm);
  linear_ring_kernel<2, MODE, F32, WIDE><<<static_cast<unsigned>(groups < slots ? groups : slots), kWarps * 32, kSmem, s>>>(p);
}

template <int MODE>
void launch_ring(bool f32, int groups, cudaStream_t s, LinearParams& p) {
  if (groups < kRingMinGroups) {
    launch_linear<2, MODE>(f32, static_cast<unsigned>(groups), s, p);
    return;
  }
  p.groups = groups;
  // four pairs per SM or more: one wide CTA per SM (11.0 against 12.1 us for gate/up, 35.9 against
  // 38.1 us for a 49152-row head); Q/K/V with its 2.6 pairs per SM is better off with one pair
  // per CTA of the three-per-SM version (7.6 against 8.0 us)
  const bool wide = groups >= 4 * 148 && p.k / kChunk <= kWideChunks * kWideWarps;
  if (f32) {
    if (wide) launch_ring_as<MODE, true, true>(groups, s, p); else launch_ring_as<MODE, true, false>(groups, s, p);
  } else {
    if (wide) launch_ring_as<MODE, false, true>(groups, s, p); else launch_ring_as<MODE, false, false>(groups, s, p);
  }
}
}  // namespace
}  // namespace fl

extern "C" int fl_linear_rows(const void* x, int32_t x_dtype, const void* weight, int64_t rows, int32_t out_features,
                              int32_t in_features, int32_t swiglu, void* out, fl_cuda_stream stream) {
  const char* who = "fl_linear_rows";
  FL_REQUIRE(x && weight && out, "%s: null argument", who);
  FL_REQUIRE(x_dtype == FL_DTYPE_BF16 || x_dtype == FL_DTYPE_F32, "%s: x is bfloat16 or float32", who);
  FL_REQUIRE(rows >= 0 && rows <= 16, "%s: at most 16 rows, got %lld", who, static_cast<long long>(rows));
  FL_REQUIRE(in_features > 0 && in_features % kChunk == 0, "%s: in_features must be a multiple of %d", who, kChunk);
  FL_REQUIRE(out_features > 0 && out_features % 16 == 0, "%s: out_features must be a multiple of 16", who);
  FL_REQUIRE(!swiglu || out_features % 32 == 0, "%s: a fused gate/up weight has an even number of 16-row tiles", who);
  FL_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(out), "%s: pointers must be 16-byte aligned", who);
  if (rows == 0) return FL_OK;
  LinearParams p{};
  p.x = x;
  p.w = static_cast<const __nv_bfloat16*>(weight);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.rows = static_cast<int>(rows);
  p.k = in_features;
  p.out_width = out_features;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool f32 = x_dtype == FL_DTYPE_F32;
  if (swiglu) {
    p.out_width = out_features / 2;
    p.up_offset = out_features / 2;
    launch_ring<1>(f32, out_features / 16, s, p);
  } else if (out_features <= 4096) {  // few tiles: eight rows per CTA keep every SM busy
    launch_linear<1, 0>(f32, out_features / 8, s, p);
  } else {
    launch_ring<0>(f32, out_features / 16, s, p);
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}

extern "C" int fl_qkv_rope_rows(const void* x, const void* weight, int64_t rows, int32_t heads, int32_t in_features,
                                const void* cosv, const void* sinv, void* q_out, void* k_out, void* v_out,
                                fl_cuda_stream stream) {
  const char* who = "fl_qkv_rope_rows";
  FL_REQUIRE(x && weight && cosv && sinv && q_out && k_out && v_out, "%s: null argument", who);
  FL_REQUIRE(rows >= 0 && rows <= 16, "%s: at most 16 rows, got %lld", who, static_cast<long long>(rows));
  FL_REQUIRE(heads > 0 && heads <= 4096, "%s: bad head count", who);
  FL_REQUIRE(in_features > 0 && in_features % kChunk == 0, "%s: in_features must be a multiple of %d", who, kChunk);
  FL_REQUIRE(aligned16(x) && aligned16(weight), "%s: pointers must be 16-byte aligned", who);
  if (rows == 0) return FL_OK;
  LinearParams p{};
  p.x = x;
  p.w = static_cast<const __nv_bfloat16*>(weight);
  p.out = static_cast<__nv_bfloat16*>(q_out);
  p.k_out = static_cast<__nv_bfloat16*>(k_out);
  p.v_out = static_cast<__nv_bfloat16*>(v_out);
  p.rows = static_cast<int>(rows);
  p.k = in_features;
  p.heads = heads;
  p.cosv = static_cast<const __nv_bfloat16*>(cosv);
  p.sinv = static_cast<const __nv_bfloat16*>(sinv);
  launch_ring<2>(false, 3 * heads * 8, static_cast<cudaStream_t>(stream), p);
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}

extern "C" int fl_linear_rows_partial(const void* x, int32_t x_dtype, const void* weight, int64_t rows,
                                      int32_t out_features, int32_t in_features, int32_t splits, float* partial,
                                      fl_cuda_stream stream) {
  const char* who = "fl_linear_rows_partial";
  FL_REQUIRE(x && weight && partial, "%s: null argument", who);
  FL_REQUIRE(x_dtype == FL_DTYPE_BF16 || x_dtype == FL_DTYPE_F32, "%s: x is bfloat16 or float32", who);
  FL_REQUIRE(rows >= 0 && rows <= 16, "%s: at most 16 rows, got %lld", who, static_cast<long long>(rows));
  FL_REQUIRE(splits >= 1 && splits <= 8, "%s: 1 to 8 slices of K", who);
  FL_REQUIRE(in_features > 0 && in_features % (kChunk * splits) == 0,
             "%s: in_features must be a multiple of %d x splits", who, kChunk);
  FL_REQUIRE(in_features / kChunk / splits <= kSplitXChunks * kSplitWarps,
             "%s: a slice of K holds at most %d values", who, kSplitXChunks * kSplitWarps * kChunk);
  FL_REQUIRE(out_features > 0 && out_features % 8 == 0, "%s: out_features must be a multiple of 8", who);
  FL_REQUIRE(aligned16(x) && aligned16(weight), "%s: pointers must be 16-byte aligned", who);
  if (rows == 0) return FL_OK;
  LinearParams p{};
  p.x = x;
  p.w = static_cast<const __nv_bfloat16*>(weight);
  p.rows = static_cast<int>(rows);
  p.k = in_features;
  p.out_width = out_features;
  p.splits = splits;
  p.partial = partial;
  constexpr int kSmem = kSplitWarps * kSplitRing * 512;
  static const cudaError_t attr_a = cudaFuncSetAttribute(linear_splitk_kernel<true>,
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  static const cudaError_t attr_b = cudaFuncSetAttribute(linear_splitk_kernel<false>,
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  (void)attr_a;
  (void)attr_b;
  const unsigned grid = static_cast<unsigned>((148 / splits) * splits);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x_dtype == FL_DTYPE_F32) {
    linear_splitk_kernel<true><<<grid, kSplitWarps * 32, kSmem, s>>>(p);
  } else {
    linear_splitk_kernel<false><<<grid, kSplitWarps * 32, kSmem, s>>>(p);
  }
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}
