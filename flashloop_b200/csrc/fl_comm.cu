// Tensor-parallel decode: the sum of the ranks' row-parallel partial outputs (o_proj, down_proj)
// fused with the residual add and the RMSNorms that consume it, as ONE launch per rank over peer
// memory.
//
// The decode step exchanges 2 x layers x 4 loops small tensors ([batch][hidden] bfloat16, 64 KB at
// batch 16): latency, not bandwidth.  Every GPU reaches every peer at full NVLink bandwidth through
// NVSwitch, so the latency-optimal shape is one shot: every rank stores its partial into a slot of
// every peer's receive buffer with plain peer stores, publishes a sequence number behind a
// system-scope fence, waits (bounded) for the sequence numbers of the others to appear in its own
// flags and reduces the slots locally in rank order (float32), then goes straight on to
// `[addend +] sum`, `residual + RMSNorm(.)` and the next RMSNorm exactly as fl_rmsnorm does.
// No collective library on the path, no NVLS objects, no TMA: plain loads and stores on
// cudaIpc-mapped memory, which a CUDA graph can replay.
//
// One CTA per row.  Slots alternate between two halves by the parity of the sequence number: a
// rank can only be one all-reduce ahead of the slowest rank (it needs everybody's partial of call
// k+1 to finish call k+1, and a rank stores that only after it has read call k), so two halves
// are enough.  The sequence number lives in device memory and advances once per launch (the last
// CTA to finish advances it), so replays of a recorded step stay in lockstep across the ranks.
//
// A wait that runs out (a peer that never stored) raises the communicator's status word and the
// kernel runs on with what it has: nothing here can hang a GPU.
#include "fl_step_common.cuh"

namespace fl {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kControlWords = 64;  // [0] sequence number, [1] arrivals of the current launch, [2] status

struct CommView {
  __nv_bfloat16* recv[kMaxRanks];  // recv[r]: rank r's receive buffer [2][world][rows_max][width]
  int* flags[kMaxRanks];           // flags[r]: rank r's flags [2][world][rows_max]
  int* control;                    // this rank's control words
  int rank, world, rows_max, width;
};

struct Comm {
  CommView view;
  void* local;  // this rank's allocation: receive buffer, flags, control words
  void* peers[kMaxRanks];
  size_t bytes;
  int device;
};

inline size_t recv_bytes(int world, int rows_max, int width) {
  return ((static_cast<size_t>(2) * world * rows_max * width * sizeof(__nv_bfloat16) + 255) / 256) * 256;
}
inline size_t flag_bytes(int world, int rows_max) {
  return ((static_cast<size_t>(2) * world * rows_max * sizeof(int) + 255) / 256) * 256;
}

__device__ __forceinline__ int load_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct ReduceNormParams {
  CommView c;
  const __nv_bfloat16* x;         // [rows][width]: this rank's partial sum
  const __nv_bfloat16* addend;    // [rows][width] or null: added to the reduced sum
  const __nv_bfloat16* residual;  // [rows][width] or null
  const __nv_bfloat16* weight;    // [width] or null: null = no norm, `out` receives [addend +] sum
  const __nv_bfloat16* weight2;   // [width] or null
  float eps, eps2;
  __nv_bfloat16* sum_out;  // [rows][width] or null: [addend +] sum before the norm
  __nv_bfloat16* out;
  __nv_bfloat16* out2;
  int skip_store;  // a test's way of making the peers' waits run out: this rank publishes nothing
  int wait_limit;
};

__global__ void __launch_bounds__(kStepThreads) reduce_norm_kernel(const __grid_constant__ ReduceNormParams p) {
  __shared__ float s_part[kStepThreads / 32];
  __shared__ int s_seq;
  const CommView& c = p.c;
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int width = c.width;
  if (tid == 0) s_seq = *reinterpret_cast<volatile int*>(c.control) + 1;
  __syncthreads();
  const int seq = s_seq;
  const int half = seq & 1;
  const int64_t my_slot = (static_cast<int64_t>(half) * c.world + c.rank) * c.rows_max + row;

  // ---- what the row needs besides the sum is requested now: it arrives while the peers are waited for
  uint4 raw_a[kMaxChunks], raw_r[kMaxChunks], raw_w[kMaxChunks], raw_w2[kMaxChunks];
#pragma unroll
  for (int ch = 0; ch < kMaxChunks; ++ch) {
    const int e = (ch * kStepThreads + tid) * 8;
    if (e < width) {
      if (p.addend) raw_a[ch] = ldg128(p.addend + static_cast<int64_t>(row) * width + e);
      if (p.residual) raw_r[ch] = ldg128(p.residual + static_cast<int64_t>(row) * width + e);
      if (p.weight) raw_w[ch] = ldg128(p.weight + e);
      if (p.weight2) raw_w2[ch] = ldg128(p.weight2 + e);
    }
  }

  // ---- this rank's row into every rank's receive buffer (its own included)
  const __nv_bfloat16* x = p.x + static_cast<int64_t>(row) * width;
  if (!p.skip_store) {
#pragma unroll
    for (int ch = 0; ch < kMaxChunks; ++ch) {
      const int e = (ch * kStepThreads + tid) * 8;
      if (e < width) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + e);
        for (int r = 0; r < c.world; ++r) *reinterpret_cast<uint4*>(c.recv[r] + my_slot * width + e) = v;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < c.world && !p.skip_store) store_release_sys(c.flags[tid] + my_slot, seq);

  // ---- wait for everybody's row of this call
  if (tid < c.world) {
    const int* flag = c.flags[c.rank] + (static_cast<int64_t>(half) * c.world + tid) * c.rows_max + row;
    int tries = 0;
    while (load_acquire_sys(flag) != seq) {
      if (++tries >= p.wait_limit) {
        atomicExch(c.control + 2, 1);
        break;
      }
      __nanosleep(40);
    }
  }
  __syncthreads();

  // ---- reduce in rank order, then the norms of fl_rmsnorm on `[addend +] sum`
  float v[kMaxChunks][8];
  float sq = 0.f;
#pragma unroll
  for (int ch = 0; ch < kMaxChunks; ++ch) {
    const int e = (ch * kStepThreads + tid) * 8;
    if (e < width) {
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < c.world; ++r) {
        const int64_t slot = (static_cast<int64_t>(half) * c.world + r) * c.rows_max + row;
        float part[8];
        unpack8(__ldcg(reinterpret_cast<const uint4*>(c.recv[c.rank] + slot * width + e)), part);
#pragma unroll
        for (int k = 0; k < 8; ++k) sum[k] += part[k];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) sum[k] = bf16_round_f(sum[k]);
      if (p.addend) {
        float a[8];
        unpack8(raw_a[ch], a);
#pragma unroll
        for (int k = 0; k < 8; ++k) sum[k] = bf16_round_f(a[k] + sum[k]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[ch][k] = sum[k];
        sq = fmaf(sum[k], sum[k], sq);
      }
      if (p.sum_out) *reinterpret_cast<uint4*>(p.sum_out + static_cast<int64_t>(row) * width + e) = pack8(v[ch]);
      if (!p.weight) *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(row) * width + e) = pack8(v[ch]);
    }
  }
  if (p.weight) {
    float inv = rsqrtf(block_sum(sq, s_part) / float(width) + p.eps);
    sq = 0.f;
#pragma unroll
    for (int ch = 0; ch < kMaxChunks; ++ch) {
      const int e = (ch * kStepThreads + tid) * 8;
      if (e < width) {
        float w[8], r[8];
        unpack8(raw_w[ch], w);
        if (p.residual) unpack8(raw_r[ch], r);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float y = bf16_round_f(w[k] * bf16_round_f(v[ch][k] * inv));
          if (p.residual) y = bf16_round_f(r[k] + y);
          v[ch][k] = y;
          sq = fmaf(y, y, sq);
        }
        *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(row) * width + e) = pack8(v[ch]);
      }
    }
    if (p.out2 != nullptr) {
      inv = rsqrtf(block_sum(sq, s_part) / float(width) + p.eps2);
#pragma unroll
      for (int ch = 0; ch < kMaxChunks; ++ch) {
        const int e = (ch * kStepThreads + tid) * 8;
        if (e < width) {
          float w[8];
          unpack8(raw_w2[ch], w);
#pragma unroll
          for (int k = 0; k < 8; ++k) v[ch][k] = w[k] * bf16_round_f(v[ch][k] * inv);
          *reinterpret_cast<uint4*>(p.out2 + static_cast<int64_t>(row) * width + e) = pack8(v[ch]);
        }
      }
    }
  }

  // ---- the last CTA of the launch advances the sequence number
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int arrived = atomicAdd(c.control + 1, 1);
    if (arrived == static_cast<int>(gridDim.x) - 1) {
      c.control[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(c.control) = seq;
    }
  }
}

}  // namespace
}  // namespace fl

using namespace fl;

extern "C" size_t fl_comm_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" int fl_comm_create(int32_t rank, int32_t world, int32_t rows_max, int32_t width, void** comm_out,
                              void* handle_out) {
  const char* who = "fl_comm_create";
  FL_REQUIRE(comm_out && handle_out, "%s: null output", who);
  FL_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, "%s: rank %d of %d (at most %d ranks)",
             who, rank, world, kMaxRanks);
  FL_REQUIRE(rows_max > 0 && rows_max <= 65535, "%s: rows_max out of range", who);
  FL_REQUIRE(width > 0 && width % 8 == 0 && width <= kStepThreads * kMaxChunks * 8,
             "%s: width must be a multiple of 8, at most %d", who, kStepThreads * kMaxChunks * 8);
  Comm* comm = new Comm();
  comm->bytes = recv_bytes(world, rows_max, width) + flag_bytes(world, rows_max) + kControlWords * sizeof(int);
  cudaError_t err = cudaGetDevice(&comm->device);
  if (err == cudaSuccess) err = cudaMalloc(&comm->local, comm->bytes);
  if (err == cudaSuccess) err = cudaMemset(comm->local, 0, comm->bytes);
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out), comm->local);
  if (err != cudaSuccess) {
    set_error("%s: %s", who, cudaGetErrorString(err));
    delete comm;
    return FL_ERR_CUDA;
  }
  comm->view.rank = rank;
  comm->view.world = world;
  comm->view.rows_max = rows_max;
  comm->view.width = width;
  for (int r = 0; r < kMaxRanks; ++r) comm->peers[r] = nullptr;
  *comm_out = comm;
  return FL_OK;
}

extern "C" int fl_comm_connect(void* comm_ptr, const void* handles) {
  const char* who = "fl_comm_connect";
  FL_REQUIRE(comm_ptr && handles, "%s: null argument", who);
  Comm* comm = static_cast<Comm*>(comm_ptr);
  const CommView& v = comm->view;
  const auto* all = static_cast<const cudaIpcMemHandle_t*>(handles);
  for (int r = 0; r < v.world; ++r) {
    void* base = comm->local;
    if (r != v.rank) {
      const cudaError_t err = cudaIpcOpenMemHandle(&base, all[r], cudaIpcMemLazyEnablePeerAccess);
      if (err != cudaSuccess) {
        set_error("%s: opening rank %d's buffer: %s", who, r, cudaGetErrorString(err));
        return FL_ERR_CUDA;
      }
      comm->peers[r] = base;
    }
    comm->view.recv[r] = static_cast<__nv_bfloat16*>(base);
    comm->view.flags[r] = reinterpret_cast<int*>(static_cast<uint8_t*>(base) + recv_bytes(v.world, v.rows_max, v.width));
  }
  comm->view.control = reinterpret_cast<int*>(static_cast<uint8_t*>(comm->local) +
                                              recv_bytes(v.world, v.rows_max, v.width) +
                                              flag_bytes(v.world, v.rows_max));
  return FL_OK;
}

extern "C" int fl_comm_destroy(void* comm_ptr) {
  if (!comm_ptr) return FL_OK;
  Comm* comm = static_cast<Comm*>(comm_ptr);
  for (int r = 0; r < kMaxRanks; ++r) {
    if (comm->peers[r]) cudaIpcCloseMemHandle(comm->peers[r]);
  }
  cudaFree(comm->local);
  delete comm;
  return FL_OK;
}

extern "C" int fl_comm_status(void* comm_ptr, int32_t* status, int32_t reset, fl_cuda_stream stream) {
  FL_REQUIRE(comm_ptr && status, "fl_comm_status: null argument");
  Comm* comm = static_cast<Comm*>(comm_ptr);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemcpyAsync(status, comm->view.control + 2, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess && reset) err = cudaMemsetAsync(comm->view.control + 2, 0, sizeof(int32_t), s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    set_error("fl_comm_status: %s", cudaGetErrorString(err));
    return FL_ERR_CUDA;
  }
  return FL_OK;
}

extern "C" int fl_allreduce_rmsnorm(void* comm_ptr, const void* x, const void* addend, const void* residual,
                                    const void* weight, float eps, const void* weight2, float eps2, int64_t rows,
                                    void* sum_out, void* out, void* out2, int32_t skip_store, int32_t wait_limit,
                                    fl_cuda_stream stream) {
  const char* who = "fl_allreduce_rmsnorm";
  FL_REQUIRE(comm_ptr && x && out, "%s: null argument", who);
  Comm* comm = static_cast<Comm*>(comm_ptr);
  FL_REQUIRE(comm->view.control != nullptr, "%s: the communicator is not connected", who);
  FL_REQUIRE(rows > 0 && rows <= comm->view.rows_max, "%s: %lld rows (the communicator holds %d)", who,
             static_cast<long long>(rows), comm->view.rows_max);
  FL_REQUIRE(!weight2 || (weight && out2), "%s: the second norm needs the first and an output", who);
  FL_REQUIRE(aligned16(x) && aligned16(out) && (!addend || aligned16(addend)) && (!residual || aligned16(residual)) &&
                 (!weight || aligned16(weight)) && (!weight2 || aligned16(weight2)) && (!sum_out || aligned16(sum_out)) &&
                 (!out2 || aligned16(out2)),
             "%s: tensors must be 16-byte aligned", who);
  ReduceNormParams p{};
  p.c = comm->view;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.addend = static_cast<const __nv_bfloat16*>(addend);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.weight = static_cast<const __nv_bfloat16*>(weight);
  p.weight2 = static_cast<const __nv_bfloat16*>(weight2);
  p.eps = eps;
  p.eps2 = eps2;
  p.sum_out = static_cast<__nv_bfloat16*>(sum_out);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out2 = static_cast<__nv_bfloat16*>(out2);
  p.skip_store = skip_store;
  p.wait_limit = wait_limit > 0 ? wait_limit : (1 << 22);
  reduce_norm_kernel<<<static_cast<unsigned>(rows), kStepThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  FL_CHECK_LAUNCH(who);
  return FL_OK;
}
