// gemm_static.cuh -- gn_op_gemm_nt_static: the tensor-core product C = A B^T + bias for callers that
// must not allocate device memory.
//
// Who that is: a host that has already handed every byte of HBM to its own pool (a later cudaMalloc can
// only fail or fragment it), and a host with a latency budget per step, because cudaMalloc / cudaFree take
// the driver's allocator lock and cudaFree waits for the device.  The regular path (gemm_tc) keeps its
// operand planes in buffers that grow on demand with cudaMalloc; this variant keeps them in one
// fixed array that is part of the library image instead.
//
// Cost and limit: GN_STATIC_SCRATCH_BYTES (16 MiB) of device memory are held on every GPU that loads the
// library, from load until the process exits, whether or not this entry point is ever called.  A problem
// needs 2 * (M + N) * roundup8(K) floats of it; larger problems are rejected with GN_ERR_INVALID_ARG.
//
// Sharing: there is ONE array per GPU.  Every call on that GPU uses it and leaves its operand planes behind;
// each call rewrites all of the part it reads (padding columns included), so nothing needs clearing
// between calls, but two calls whose kernels overlap on the same GPU (two contexts, two host threads) race
// on it.  Run them one after the other.
//
// Set-up: a __device__ array's name is only a host-side handle in host code, not an address a kernel can use,
// so the first call on each device looks the real address up with cudaGetSymbolAddress (with that device
// current) and caches it.  Make that first call before any stream capture begins.
#pragma once
#include "common.cuh"
#include "gemm_tc.cuh"

namespace gn {

constexpr long GN_STATIC_SCRATCH_FLOATS = 4L << 20;                     // 16 MiB
constexpr long GN_STATIC_SCRATCH_BYTES = GN_STATIC_SCRATCH_FLOATS * 4;
static __device__ __align__(256) float gn_static_scratch[GN_STATIC_SCRATCH_FLOATS];

constexpr int GN_STATIC_MAX_DEVICES = 64;
// Device address of gn_static_scratch on `device` (which must be current); resolved once per device.
inline int static_scratch_ptr(int device, float** out) {
  static std::mutex mu; static float* table[GN_STATIC_MAX_DEVICES] = {nullptr};
  if (device < 0 || device >= GN_STATIC_MAX_DEVICES) return fail(GN_ERR_INVALID_ARG, "device index %d out of range", device);
  std::lock_guard<std::mutex> lk(mu);
  if (!table[device]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, gn_static_scratch);
    if (e != cudaSuccess || !p) return fail(GN_ERR_CUDA, "cudaGetSymbolAddress(gn_static_scratch) on device %d: %s", device, cudaGetErrorString(e));
    table[device] = p;
  }
  *out = table[device]; return GN_OK;
}

}  // namespace gn

extern "C" int gn_op_gemm_nt_static(gn_ctx* ctx, int M, int N, int K, const float* A_dev, const float* B_dev, const float* bias_dev, float* C_dev) {
  using namespace gn;
  if (!ctx || !ctx->alive || !A_dev || !B_dev || !C_dev || M <= 0 || N <= 0 || K <= 0) return fail(GN_ERR_INVALID_ARG, "op_gemm_nt_static: bad argument");
  Ctx* c = &ctx->c;
  if (!c->tc_ok) return fail(GN_ERR_UNSUPPORTED, "the tensor-core engine is not available on this context");
  const long ldp = tc_ldp(K);
  const long need = 2 * ((long)M + N) * ldp;
  if (need > GN_STATIC_SCRATCH_FLOATS)
    return fail(GN_ERR_INVALID_ARG, "op_gemm_nt_static: M=%d N=%d K=%d needs %ld scratch floats, the fixed array holds %ld (2*(M+N)*roundup8(K) must not exceed it)",
                M, N, K, need, GN_STATIC_SCRATCH_FLOATS);
  GN_CUDA(cudaSetDevice(c->device));
  float* base = nullptr; GN_TRY(static_scratch_ptr(c->device, &base));
  float *a_hi = base, *a_lo = a_hi + (long)M * ldp, *b_hi = a_lo + (long)M * ldp, *b_lo = b_hi + (long)N * ldp;
  TcPlanes PA{a_hi, a_lo, M, K, (int)ldp, 1}, PB{b_hi, b_lo, N, K, (int)ldp, 1};
  GN_TRY(tc_split(c, TcSrc{A_dev, (long)K, 1, 0, 0, 1}, PA));
  GN_TRY(tc_split(c, TcSrc{B_dev, (long)K, 1, 0, 0, 1}, PB));
  TcParams ep{C_dev, (long)N, 0, 0, bias_dev, nullptr, 0, 0, 0, GN_ACT_LINEAR, M, N, K, 1, 0, c->d_status, nullptr, 0, 1};
  GN_TRY(tc_launch(c, PA, PB, ep));
  GN_CUDA(cudaStreamSynchronize(c->stream));
  int st = 0; GN_CUDA(copy_d2h(c, &st, c->d_status, sizeof(int)));
  if (st != 0) { cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream); cudaStreamSynchronize(c->stream); return fail(GN_ERR_TIMEOUT, "a device-side bounded wait gave up (status word %d)", st); }
  return GN_OK;
}
