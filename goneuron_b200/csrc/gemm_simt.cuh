// gemm_simt.cuh -- strided, batched fp32 contraction on the CUDA cores.
//
// C[b](m,n) = act( alpha * sum_k A[b](m,k) * B[b](k,n) + bias[n] + R[b](m,n) )
// with arbitrary element strides for A and B, so every transpose variant of the
// training step (X*W^T, dZ*W, dZ^T*X, Q*K^T, P*V, dS^T*Q ...) and every sub-view
// (one head of a [tokens, d] tensor, the last token of every sequence) is the same
// kernel.  It is the exact-fp32 engine: small and oddly shaped contractions use it,
// and the tensor-core engine is checked against it.
#pragma once
#include "common.cuh"

namespace gn {

enum { GEMM_KBEG_AT_M0 = 1, GEMM_KEND_AT_M0 = 2, GEMM_SKIP_UPPER = 4 };

struct GemmDesc {
  int M = 0, N = 0, K = 0;
  const float* A = nullptr; long sa_m = 0, sa_k = 0;
  const float* B = nullptr; long sb_k = 0, sb_n = 0;   // B(k,n)
  float* C = nullptr; long ldc = 0;
  const float* bias = nullptr;                          // [N]
  const float* R = nullptr; long ldr = 0;               // residual added to the result (may alias C)
  int act = GN_ACT_LINEAR;                              // LINEAR or RELU
  // optional gate: result(m,n) is zeroed unless mask[(m / mask_group) * mask_ld + n] > 0 (the ReLU pattern of the
  // last token of row m's sequence, see relu_mask semantics in model.cu)
  const float* mask = nullptr; long mask_ld = 0; int mask_group = 1;
  float alpha = 1.f;
  bool reuse_a_planes = false;                          // A is the same tensor as in the previous tensor-core call of this context
  const void* b_planes = nullptr;                       // tensor-core engine: prepared operand planes of B (a BfPlanes), e.g. of a weight matrix
  const void* a_planes = nullptr;                       // ... and of A (written by the epilogue of the contraction that produced A)
  const void* plane_out = nullptr;                      // tensor-core engine: a TcPlaneOut; the result is written as operand planes instead of fp32
  float* a_rownorm = nullptr;                           // tensor-core engine: receives the L2 norm of every row of A (from the split pass)
  int batch1 = 1, batch2 = 1;                           // batch index b -> (b / batch2, b % batch2)
  long a_b1 = 0, a_b2 = 0, b_b1 = 0, b_b2 = 0, c_b1 = 0, c_b2 = 0, r_b1 = 0, r_b2 = 0;
  // Causal structure of attention: tiles that are entirely masked are never touched.
  //   GEMM_SKIP_UPPER : do not compute output tiles with n0 > m0 + BM - 1 (S = Q K^T)
  //   GEMM_KEND_AT_M0 : contraction index stops at m0 + BM            (P V, dS K)
  //   GEMM_KBEG_AT_M0 : contraction index starts at m0                (dS^T Q, P^T dA)
  int flags = 0;
};

constexpr int SG_BM = 128, SG_BN = 128, SG_BK = 16, SG_PAD = 4, SG_THREADS = 256;

template <bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(SG_THREADS) gemm_simt_kernel(GemmDesc g) {
  __shared__ __align__(16) float As[SG_BK][SG_BM + SG_PAD];
  __shared__ __align__(16) float Bs[SG_BK][SG_BN + SG_PAD];
  const int b = blockIdx.z, b1 = b / g.batch2, b2 = b % g.batch2;
  const float* A = g.A + b1 * g.a_b1 + b2 * g.a_b2;
  const float* B = g.B + b1 * g.b_b1 + b2 * g.b_b2;
  float* C = g.C + b1 * g.c_b1 + b2 * g.c_b2;
  const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
  if ((g.flags & GEMM_SKIP_UPPER) && n0 > m0 + SG_BM - 1) return;
  int kbeg = 0, kend = g.K;
  if (g.flags & GEMM_KBEG_AT_M0) kbeg = (m0 / SG_BK) * SG_BK;
  if (g.flags & GEMM_KEND_AT_M0) kend = min(g.K, m0 + SG_BM);
  const int t = threadIdx.x, ty = t / 16, tx = t % 16;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

  for (int k0 = kbeg; k0 < kend; k0 += SG_BK) {
#pragma unroll
    for (int e = 0; e < 8; e++) {
      int idx = t + SG_THREADS * e;
      int m, k;
      if (A_KFAST) { k = idx % SG_BK; m = idx / SG_BK; } else { m = idx % SG_BM; k = idx / SG_BM; }
      int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < g.M && gk < kend) ? A[gm * g.sa_m + gk * g.sa_k] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 8; e++) {
      int idx = t + SG_THREADS * e;
      int n, k;
      if (B_NFAST) { n = idx % SG_BN; k = idx / SG_BN; } else { k = idx % SG_BK; n = idx / SG_BK; }
      int gn_ = n0 + n, gk = k0 + k;
      Bs[k][n] = (gn_ < g.N && gk < kend) ? B[gk * g.sb_k + gn_ * g.sb_n] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SG_BK; k++) {
      float4 a0 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      float4 a1 = *reinterpret_cast<const float4*>(&As[k][64 + ty * 4]);
      float4 c0 = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      float4 c1 = *reinterpret_cast<const float4*>(&Bs[k][64 + tx * 4]);
      float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      float bv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  const float* R = g.R ? g.R + b1 * g.r_b1 + b2 * g.r_b2 : nullptr;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (n >= g.N) continue;
      float v = g.alpha * acc[i][j];
      if (g.bias) v += g.bias[n];
      if (R) v += R[m * g.ldr + n];
      if (g.act == GN_ACT_RELU) v = v > 0.f ? v : 0.f;
      if (g.mask && !(g.mask[(long)(m / g.mask_group) * g.mask_ld + n] > 0.f)) v = 0.f;
      C[m * g.ldc + n] = v;
    }
  }
}

// Skinny outputs (N <= 16, both operands K-major, one problem): the tiled kernel would run a handful of CTAs over a
// long K loop.  Here one block owns one output row: its threads stride over K with all N sums in registers, then
// combine through shared memory.  C(m,n) = act(sum_k A(m,k) B(n,k) + bias[n] + R(m,n)).
constexpr int SKINNY_N = 16;
__global__ void __launch_bounds__(256) gemm_skinny_kernel(GemmDesc g) {
  __shared__ float red[8][SKINNY_N];
  const int m = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const float* a = g.A + (long)m * g.sa_m;
  float acc[SKINNY_N];
#pragma unroll
  for (int n = 0; n < SKINNY_N; n++) acc[n] = 0.f;
  for (int k = threadIdx.x; k < g.K; k += 256) {
    const float av = a[k];
#pragma unroll
    for (int n = 0; n < SKINNY_N; n++) if (n < g.N) acc[n] = fmaf(av, g.B[(long)n * g.sb_n + k], acc[n]);
  }
#pragma unroll
  for (int n = 0; n < SKINNY_N; n++) { const float v = warp_sum(acc[n]); if (lane == 0) red[w][n] = v; }
  __syncthreads();
  if (threadIdx.x < g.N) {
    const int n = threadIdx.x;
    float v = 0.f;
    for (int q = 0; q < 8; q++) v += red[q][n];
    if (g.bias) v += g.bias[n];
    if (g.R) v += g.R[(long)m * g.ldr + n];
    if (g.act == GN_ACT_RELU) v = v > 0.f ? v : 0.f;
    g.C[(long)m * g.ldc + n] = v;
  }
}
inline bool gemm_skinny_ok(const GemmDesc& g) {
  return g.batch1 * g.batch2 == 1 && g.N <= SKINNY_N && g.K >= 256 && g.sa_k == 1 && g.sb_k == 1 && !g.mask && g.alpha == 1.f && g.flags == 0 &&
         (g.act == GN_ACT_LINEAR || g.act == GN_ACT_RELU);
}

// Sum of at most 64 outer products: C[M,N] = sum_k A(m,k) B(k,n) with both operands stored contraction-major (A(m,k) at
// A[k * sa_k + m], B(k,n) at B[k * sb_k + n]) -- the weight gradient of an inner Dense layer, which only sees one input
// row per sample (layer.go:591-625), when the batch (or a rank's shard of it) is small.  Every block stages both operand
// panels of its 64 x 64 output tile in shared memory once; each thread owns a 4 x 4 patch.  The general kernel runs such a
// product on 64 blocks of 128 x 128 with a contraction of two 16-steps; this one fills the SMs and is bound by writing C.
constexpr int OS_KMAX = 64;
__global__ void __launch_bounds__(256) outer_sum_kernel(const float* __restrict__ A, long sa_k, const float* __restrict__ B, long sb_k, float* __restrict__ C, long ldc,
                                                        int M, int N, int K, float alpha) {
  __shared__ __align__(16) float As[OS_KMAX][64];
  __shared__ __align__(16) float Bs[OS_KMAX][64];
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int i = tid; i < K * 64; i += 256) {
    const int k = i >> 6, c = i & 63;
    As[k][c] = m0 + c < M ? A[(long)k * sa_k + m0 + c] : 0.f;
    Bs[k][c] = n0 + c < N ? B[(long)k * sb_k + n0 + c] : 0.f;
  }
  __syncthreads();
  float acc[4][4] = {};
  for (int k = 0; k < K; k++) {
    const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]), b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
    const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
  const bool vec = (ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 && n0 + tx * 4 + 3 < N;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i; if (m >= M) break;
    float* crow = C + (long)m * ldc + n0 + tx * 4;
    if (vec) *reinterpret_cast<float4*>(crow) = make_float4(alpha * acc[i][0], alpha * acc[i][1], alpha * acc[i][2], alpha * acc[i][3]);
    else
      for (int j = 0; j < 4; j++) if (n0 + tx * 4 + j < N) crow[j] = alpha * acc[i][j];
  }
}
inline bool gemm_outer_small_ok(const GemmDesc& g) {
  return g.sa_m == 1 && g.sb_n == 1 && g.K >= 1 && g.K <= OS_KMAX && g.batch1 * g.batch2 == 1 && !g.bias && !g.R && !g.mask && g.act == GN_ACT_LINEAR && g.flags == 0 &&
         !g.a_planes && !g.b_planes && !g.plane_out && !g.a_rownorm && (long)g.M * g.N >= 64 * 64;
}

inline int gemm_simt(Ctx* ctx, const GemmDesc& g) {
  if (g.M <= 0 || g.N <= 0) return GN_OK;
  if (gemm_outer_small_ok(g)) {
    GN_LAUNCH(ctx, outer_sum_kernel, dim3(cdiv(g.N, 64), cdiv(g.M, 64)), 256, 0, g.A, g.sa_k, g.B, g.sb_k, g.C, g.ldc, g.M, g.N, g.K, g.alpha);
    return check_launch("outer_sum");
  }
  if (gemm_skinny_ok(g)) { GN_LAUNCH(ctx, gemm_skinny_kernel, g.M, 256, 0, g); return check_launch("gemm_skinny"); }
  dim3 grid(cdiv(g.N, SG_BN), cdiv(g.M, SG_BM), g.batch1 * g.batch2);
  bool ak = (g.sa_k == 1), bn = (g.sb_n == 1);
  if (ak && bn) GN_LAUNCH(ctx, (gemm_simt_kernel<true, true>), grid, SG_THREADS, 0, g);
  else if (ak && !bn) GN_LAUNCH(ctx, (gemm_simt_kernel<true, false>), grid, SG_THREADS, 0, g);
  else if (!ak && bn) GN_LAUNCH(ctx, (gemm_simt_kernel<false, true>), grid, SG_THREADS, 0, g);
  else GN_LAUNCH(ctx, (gemm_simt_kernel<false, false>), grid, SG_THREADS, 0, g);
  return check_launch("gemm_simt");
}

}  // namespace gn
