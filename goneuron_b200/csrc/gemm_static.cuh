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
// needs (M + N) * (roundup8(K) + 1) floats of it (two fp16 planes per operand element and one scale per operand row);
// larger problems are
// rejected with GN_ERR_INVALID_ARG.  Long contractions are cut into accumulator runs exactly as in the regular
// path (more launches, no allocation).
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
  const long need = ((long)M + N) * (ldp + 1);
  if (need > GN_STATIC_SCRATCH_FLOATS)
    return fail(GN_ERR_INVALID_ARG, "op_gemm_nt_static: M=%d N=%d K=%d needs %ld scratch floats, the fixed array holds %ld ((M+N)*(roundup8(K)+1) must not exceed it)",
                M, N, K, need, GN_STATIC_SCRATCH_FLOATS);
  std::lock_guard<std::mutex> lk(c->run_mu);
  GN_CUDA(cudaSetDevice(c->device));
  float* base = nullptr; GN_TRY(static_scratch_ptr(c->device, &base));
  float* scales = base + ((long)M + N) * ldp;          // [M] for A, then [N] for B; (M + N) * ldp is a multiple of 8 floats, so B's start is 16-byte aligned when M % 4 == 0
  float* sb = scales + (((long)M + 3) & ~3L);
  if (sb + N > base + GN_STATIC_SCRATCH_FLOATS) return fail(GN_ERR_INVALID_ARG, "op_gemm_nt_static: M=%d N=%d K=%d does not fit the fixed array", M, N, K);
  BfPlanes PA{reinterpret_cast<__half*>(base), scales, M, K, (int)ldp, 1}, PB{reinterpret_cast<__half*>(base + (long)M * ldp), sb, N, K, (int)ldp, 1};
  GN_TRY(tc_split(c, TcSrc{A_dev, (long)K, 1, 0, 0, 1}, PA, nullptr));
  GN_TRY(tc_split(c, TcSrc{B_dev, (long)K, 1, 0, 0, 1}, PB, nullptr));
  TcParams ep{C_dev, (long)N, 0, 0, bias_dev, nullptr, 0, 0, 0, GN_ACT_LINEAR, M, N, K, 1, 0, c->d_status, nullptr, 0, 1};
  GN_TRY(tc_run(c, PA, PB, ep));
  GN_CUDA(cudaStreamSynchronize(c->stream));
  return check_status_word(c);
}
