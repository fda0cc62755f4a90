// common.cuh -- context, error handling and launch bookkeeping shared by all kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/goneuron_cuda.h"

namespace gn {

// Per-thread message of the most recent failure (gn_last_error()).
inline std::string& last_error() { thread_local std::string e; return e; }
inline int fail(int code, const char* fmt, ...) {
  char buf[1024]; va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
  last_error() = buf; return code;
}

#define GN_CUDA(call)                                                                        \
  do { cudaError_t e_ = (call); if (e_ != cudaSuccess)                                       \
      return gn::fail(e_ == cudaErrorMemoryAllocation ? GN_ERR_OOM : GN_ERR_CUDA, "%s failed at %s:%d: %s", #call, __FILE__, __LINE__, cudaGetErrorString(e_)); } while (0)
#define GN_TRY(call) do { int rc_ = (call); if (rc_ != GN_OK) return rc_; } while (0)

struct NcclApi;   // resolved at run time from libnccl.so.2 (nccl_dl.cuh)

struct Ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t comm_stream = nullptr;   // gradient all-reduces run here, overlapped with the rest of the backward pass
  int rank = 0, world = 1;
  void* comm = nullptr;            // ncclComm_t
  NcclApi* nccl = nullptr;
  int sm_count = 148;
  int sm_reserve = 0;              // SMs the persistent kernels leave free (for the collectives' CTAs when several ranks run); see persist_sms()
  int64_t launches = 0;            // kernels launched by this library on this context
  // contraction profiling (gn_model_set_profiling)
  int profile = 0;
  double gemm_flops = 0; float gemm_ms = 0; int64_t gemm_launches = 0;
  double gemm_bytes = 0, split_bytes = 0;   // algorithmic bytes of the step's contraction launches (operand planes + output + residual) / of its operand split passes
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> ev_pool; size_t ev_used = 0;
  int* d_status = nullptr;         // device word set by kernels whose bounded waits gave up
  bool tc_ok = false;              // tcgen05 engine usable (driver entry point for tensor maps found)
  void* encode_tiled = nullptr;    // cuTensorMapEncodeTiled
  unsigned spin_limit = 1u << 24;  // polls per bounded device-side wait (gn_ctx_set_spin_limit)
  bool tc_tile_queue = false;      // persistent contraction draws its tiles from a queue instead of a fixed share per CTA (GONEURON_CUDA_TC_TILE_QUEUE)
  int* tc_queue_pool = nullptr; int tc_queue_used = 0;      // zeroed counters for those queues
  bool tc_tail_split = true;       // left-over tiles of a short last round run as half tiles (GONEURON_CUDA_TC_TAIL_SPLIT=0 switches it off)
  int tc_force_bn = 0, tc_kslice = 0;   // experiment switches of the contraction engine (GONEURON_CUDA_TC_BN / _KSLICE); 0 = automatic
  void* tc_scratch = nullptr;      // operand planes of the contraction engine (TcScratch, owned)
  void* attn_scratch = nullptr;    // operand planes of the tcgen05 attention kernels (AttnTcScratch, owned)
  const void* weight_planes = nullptr;   // the running model's table of prepared weight planes (WeightPlaneTable), or null
  std::mutex run_mu;               // serialises every entry point that launches work on this context (they share the scratch above)
  cudaEvent_t t0 = nullptr, t1 = nullptr;   // gn_timer_start / gn_timer_stop
  // Scratch objects created on demand for this context (operand planes of the contraction and attention engines),
  // all released by gn_shutdown.
  std::vector<std::pair<void*, void (*)(void*)>> owned; std::mutex owned_mu;
  template <class T> T* own(T* p) { std::lock_guard<std::mutex> lk(owned_mu); owned.push_back({p, [](void* q) { delete static_cast<T*>(q); }}); return p; }
  void release_owned() { std::lock_guard<std::mutex> lk(owned_mu); for (auto& e : owned) e.second(e.first); owned.clear(); }
};

inline unsigned cdiv(long a, long b) { return (unsigned)((a + b - 1) / b); }

// Every kernel launch of the library goes through this macro so that the launch count is exact.
#define GN_LAUNCH(ctx, kernel, grid, block, smem, ...)                         \
  do { kernel<<<(grid), (block), (smem), (ctx)->stream>>>(__VA_ARGS__); (ctx)->launches++; } while (0)

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GN_ERR_CUDA, "kernel launch failed (%s): %s", what, cudaGetErrorString(e));
  return GN_OK;
}

// Host <-> device copies always go through the context's own stream and wait for it.  (The synchronous cudaMemcpy /
// cudaMemset run on the legacy default stream, which a non-blocking stream does not wait for, and may return before
// the transfer has landed: work issued that way can overtake, or be overtaken by, kernels of the context's stream.)
inline cudaError_t copy_h2d(Ctx* c, void* dst, const void* src, size_t bytes) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream); return e != cudaSuccess ? e : cudaStreamSynchronize(c->stream);
}
inline cudaError_t copy_d2h(Ctx* c, void* dst, const void* src, size_t bytes) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream); return e != cudaSuccess ? e : cudaStreamSynchronize(c->stream);
}

// Contraction profiling (gn_model_set_profiling): one CUDA-event pair around each contraction KERNEL launch (the operand
// split passes are separate, memory-bound kernels and are not inside the bracket).
struct ProfScope {
  Ctx* c; cudaEvent_t e1 = nullptr;
  explicit ProfScope(Ctx* ctx) : c(ctx) {
    if (!c->profile) return;
    if (c->ev_used == c->ev_pool.size()) { cudaEvent_t a, b; if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return; c->ev_pool.push_back({a, b}); }
    cudaEventRecord(c->ev_pool[c->ev_used].first, c->stream); e1 = c->ev_pool[c->ev_used].second; c->ev_used++;
  }
  ~ProfScope() { if (e1) cudaEventRecord(e1, c->stream); }
};

// Owning device buffer.
struct DevBuf {
  float* p = nullptr; size_t n = 0;
  DevBuf() {}
  DevBuf(const DevBuf&) = delete; DevBuf& operator=(const DevBuf&) = delete;
  DevBuf(DevBuf&& o) noexcept : p(o.p), n(o.n) { o.p = nullptr; o.n = 0; }
  DevBuf& operator=(DevBuf&& o) noexcept { release(); p = o.p; n = o.n; o.p = nullptr; o.n = 0; return *this; }
  ~DevBuf() { release(); }
  void release() { if (p) cudaFree(p); p = nullptr; n = 0; }
  int alloc(size_t count) {
    release(); if (count == 0) return GN_OK;
    cudaError_t e = cudaMalloc(&p, count * sizeof(float));
    if (e != cudaSuccess) { p = nullptr; return fail(GN_ERR_OOM, "cudaMalloc of %zu bytes failed: %s", count * sizeof(float), cudaGetErrorString(e)); }
    n = count; return GN_OK;
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum / max; every thread receives the result.  `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) { float t = lane < nw ? red[lane] : 0.f; t = warp_sum(t); if (lane == 0) red[32] = t; }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) { float t = lane < nw ? red[lane] : -INFINITY; t = warp_max(t); if (lane == 0) red[32] = t; }
  __syncthreads();
  return red[32];
}

}  // namespace gn
