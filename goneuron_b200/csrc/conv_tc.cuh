// conv_tc.cuh -- Conv2D as implicit GEMM on the tcgen05 contraction engine (gemm_tc.cuh), all three directions.
//
//   forward   z[(b,oh,ow), oc]  = sum_{(ic,kh,kw)} patch[(b,oh,ow), (ic,kh,kw)] * W[oc, (ic,kh,kw)] + bias[oc]
//             (conv2d.go:716-959)                  M = B*oH*oW rows, N = outC, K = inC*k*k
//   dgrad     dx[(b,ih,iw), ic] = sum_{(oc,kh,kw)} gpatch[(b,ih,iw), (oc,kh,kw)] * Wd[ic, (oc,kh,kw)]       (stride 1)
//             (conv2d.go:1151-1162)                M = B*H*W, N = inC, K = outC*k*k, gpatch taps mirrored
//   wgrad     per sample b:  dW_b[oc, (ic,kh,kw)] = sum_{(oh,ow)} g[b,oc,(oh,ow)] * patchT_b[(ic,kh,kw), (oh,ow)]
//             (conv2d.go:1113-1150)                M = outC, N = inC*k*k + 1, K = oH*oW, one problem per sample; the extra
//             output column contracts g with a row of ones and is the sample's bias gradient; the samples' results are
//             then added in batch order, which is also the order in which the reference accumulates them.
//
// "Implicit" here means that the patch matrix never exists in fp32: the engine's operand planes (two fp16 planes and
// a power-of-two scale per row, see gemm_tc.cuh) are written straight from the NCHW tensor by the gather kernels
// below, with the im2col addressing (zero padding = out-of-range taps contribute 0) done on the fly.  The output tile
// is stored by the contraction kernel's epilogue directly in NCHW (one output row = one pixel per thread, so a warp
// writes 32 neighbouring pixels of a channel at a time), bias and ReLU included.
#pragma once
#include "common.cuh"
#include "gemm_tc.cuh"
#include "conv_lstm.cuh"

namespace gn {

// Source geometry of a patch gather: element (row = (b, oy, ox), kidx = (ch, kh, kw)) = src[b, ch, oy*s + dir*kh + off, ox*s + dir*kw + off]
// or 0 outside the source.  forward: dir = +1, off = -pad; input gradient (stride 1): dir = -1, off = +pad.
struct PatchGeom { int C, k, s, dir, off, sH, sW, oH, oW; };

__device__ __forceinline__ float patch_elem(const float* __restrict__ sb, const PatchGeom& g, int oy, int ox, int kidx) {
  const int kw = kidx % g.k; const int r = kidx / g.k; const int kh = r % g.k, ch = r / g.k;
  const int iy = oy * g.s + g.dir * kh + g.off, ix = ox * g.s + g.dir * kw + g.off;
  if (iy < 0 || iy >= g.sH || ix < 0 || ix >= g.sW) return 0.f;
  return sb[((long)ch * g.sH + iy) * g.sW + ix];
}
// One warp per plane row (one output position), lanes over the contraction index.  rows = B*oH*oW, K = C*k*k.
__global__ void __launch_bounds__(256) conv_patch_rows_split_kernel(const float* __restrict__ src, PatchGeom g, long rows, int K, __half* __restrict__ p0, __half* __restrict__ p1,
                                                                    float* __restrict__ inv_scale, int ldp) {
  const int lane = threadIdx.x & 31;
  const long r = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int P = g.oH * g.oW; const long b = r / P; const int pix = (int)(r - b * P), oy = pix / g.oW, ox = pix - oy * g.oW;
  const float* sb = src + b * (long)g.C * g.sH * g.sW;
  float mx = 0.f;
  for (int kidx = lane; kidx < K; kidx += 32) mx = fmaxf(mx, fabsf(patch_elem(sb, g, oy, ox, kidx)));
  mx = warp_max(mx);
  float inv; const float sc = row_scale(mx, &inv);
  if (lane == 0) inv_scale[r] = inv;
  __half* q0 = p0 + r * ldp; __half* q1 = p1 + r * ldp;
  for (int kidx = lane; kidx < ldp; kidx += 32) {
    const float v = kidx < K ? patch_elem(sb, g, oy, ox, kidx) * sc : 0.f;
    const __half h = __float2half_rn(v);
    q0[kidx] = h; q1[kidx] = __float2half_rn(v - __half2float(h));
  }
}
// Transposed patches of one sample for the weight gradient: plane row = (b, kidx), kidx in [0, K] with row K = ones;
// contraction index = output position.  One warp per plane row, lanes over the positions.
__global__ void __launch_bounds__(256) conv_patch_cols_split_kernel(const float* __restrict__ src, PatchGeom g, int B, int K, __half* __restrict__ p0, __half* __restrict__ p1,
                                                                    float* __restrict__ inv_scale, int ldp) {
  const int lane = threadIdx.x & 31, P = g.oH * g.oW, rows = K + 1;
  const long r = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= (long)B * rows) return;
  const long b = r / rows; const int kidx = (int)(r - b * rows);
  const float* sb = src + b * (long)g.C * g.sH * g.sW;
  auto elem = [&](int pix) -> float { if (kidx == K) return 1.f; const int oy = pix / g.oW; return patch_elem(sb, g, oy, pix - oy * g.oW, kidx); };
  float mx = 0.f;
  for (int pix = lane; pix < P; pix += 32) mx = fmaxf(mx, fabsf(elem(pix)));
  mx = warp_max(mx);
  float inv; const float sc = row_scale(mx, &inv);
  if (lane == 0) inv_scale[r] = inv;
  __half* q0 = p0 + r * ldp; __half* q1 = p1 + r * ldp;
  for (int pix = lane; pix < ldp; pix += 32) {
    const float v = pix < P ? elem(pix) * sc : 0.f;
    const __half h = __float2half_rn(v);
    q0[pix] = h; q1[pix] = __float2half_rn(v - __half2float(h));
  }
}
// Wd[ic, (oc,kh,kw)] = W[oc, ic, kh, kw]: the weight matrix of the input-gradient product
__global__ void conv_w_dgrad_layout_kernel(const float* __restrict__ W, float* __restrict__ Wd, int outC, int inC, int kk) {
  const int n = outC * inC * kk;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int t = i % kk; const int r = i / kk; const int ic = r % inC, oc = r / inC;
    Wd[((long)ic * outC + oc) * kk + t] = W[i];
  }
}
// dW[oc, kidx] += sum_b part[b][oc][kidx] (kidx < K), db[oc] += sum_b part[b][oc][K]; samples added in batch order
__global__ void conv_wgrad_reduce_kernel(const float* __restrict__ part, int B, int outC, int K, float* __restrict__ dW, float* __restrict__ db) {
  const int n = outC * (K + 1), i = blockIdx.x * blockDim.x + threadIdx.x; if (i >= n) return;
  float s = 0.f;
  for (int b = 0; b < B; b++) s += part[(long)b * n + i];
  const int oc = i / (K + 1), kidx = i - oc * (K + 1);
  if (kidx < K) dW[(long)oc * K + kidx] += s; else db[oc] += s;
}

inline bool conv_tc_supported(Ctx* ctx, const ConvShape& c) {
  static const bool off = [] { const char* e = getenv("GONEURON_CUDA_CONV"); return e && !strcmp(e, "direct"); }();
  if (off || !ctx->tc_ok) return false;
  const long K = (long)c.inC * c.k * c.k, Kd = (long)c.outC * c.k * c.k, P = (long)c.oH * c.oW;
  return c.oH > 0 && c.oW > 0 && K <= 8192 && Kd <= 8192 && P <= 65536 && (long)c.B * P <= 0x3fffffffL && (long)c.B * c.H * c.W <= 0x3fffffffL && c.B <= 65535;
}
static inline void conv_tc_count(Ctx* ctx, double M, double N, double K) { ctx->gemm_flops += 2.0 * M * N * K; ctx->gemm_launches++; }

// out (and z, when the activation needs the pre-activation kept) in NCHW.  Activations other than LINEAR / RELU are applied by the caller on z.
inline int conv_tc_forward(Ctx* ctx, const ConvShape& c, const float* x, const float* W, const float* bias, float* dst, int epilogue_act) {
  const int K = c.inC * c.k * c.k, P = c.oH * c.oW; const long M = (long)c.B * P;
  BfPlanes A, Bp; GN_TRY(tc_planes(ctx, 0, 1, M, K, &A)); GN_TRY(tc_planes(ctx, 1, 1, c.outC, K, &Bp));
  PatchGeom g{c.inC, c.k, c.s, 1, -c.p, c.H, c.W, c.oH, c.oW};
  GN_LAUNCH(ctx, conv_patch_rows_split_kernel, cdiv(M, 8), 256, 0, x, g, M, K, A.p0(), A.p1(), A.inv_scale, A.ldp);
  ctx->split_bytes += 8.0 * (double)M * K;
  GN_TRY(tc_split(ctx, TcSrc{W, (long)K, 1, 0, 0, 1}, Bp, nullptr));
  TcParams ep{dst, (long)c.outC, 0, 0, bias, nullptr, 0, 0, 0, epilogue_act, (int)M, c.outC, K, 1, 0, ctx->d_status, nullptr, 0, 1};
  ep.nchw_P = P;
  conv_tc_count(ctx, (double)M, c.outC, K);
  return tc_run(ctx, A, Bp, ep);
}
// dx in NCHW from dz (gradient with respect to the pre-activation, NCHW); stride 1 only.  `wtmp`: outC*inC*k*k floats.
inline int conv_tc_dgrad(Ctx* ctx, const ConvShape& c, const float* dz, const float* W, float* wtmp, float* dx) {
  const int kk = c.k * c.k, Kd = c.outC * kk, P = c.H * c.W; const long M = (long)c.B * P;
  BfPlanes A, Bp; GN_TRY(tc_planes(ctx, 0, 1, M, Kd, &A)); GN_TRY(tc_planes(ctx, 1, 1, c.inC, Kd, &Bp));
  PatchGeom g{c.outC, c.k, 1, -1, c.p, c.oH, c.oW, c.H, c.W};
  GN_LAUNCH(ctx, conv_patch_rows_split_kernel, cdiv(M, 8), 256, 0, dz, g, M, Kd, A.p0(), A.p1(), A.inv_scale, A.ldp);
  ctx->split_bytes += 8.0 * (double)M * Kd;
  GN_LAUNCH(ctx, conv_w_dgrad_layout_kernel, cdiv((long)Kd * c.inC, 256), 256, 0, W, wtmp, c.outC, c.inC, kk);
  GN_TRY(tc_split(ctx, TcSrc{wtmp, (long)Kd, 1, 0, 0, 1}, Bp, nullptr));
  TcParams ep{dx, (long)c.inC, 0, 0, nullptr, nullptr, 0, 0, 0, GN_ACT_LINEAR, (int)M, c.inC, Kd, 1, 0, ctx->d_status, nullptr, 0, 1};
  ep.nchw_P = P;
  conv_tc_count(ctx, (double)M, c.inC, Kd);
  return tc_run(ctx, A, Bp, ep);
}
// gW[outC, inC*k*k] += ..., gb[outC] += ...; `part`: B * outC * (inC*k*k + 1) floats.
inline int conv_tc_wgrad(Ctx* ctx, const ConvShape& c, const float* dz, const float* x, float* part, float* gW, float* gb) {
  const int K = c.inC * c.k * c.k, P = c.oH * c.oW, N = K + 1;
  BfPlanes A, Bp; GN_TRY(tc_planes(ctx, 0, c.B, c.outC, P, &A)); GN_TRY(tc_planes(ctx, 1, c.B, N, P, &Bp));
  GN_TRY(tc_split(ctx, TcSrc{dz, (long)P, 1, (long)c.outC * P, 0, 1}, A, nullptr));          // g[b] is [outC][P] as stored
  PatchGeom g{c.inC, c.k, c.s, 1, -c.p, c.H, c.W, c.oH, c.oW};
  GN_LAUNCH(ctx, conv_patch_cols_split_kernel, cdiv((long)c.B * N, 8), 256, 0, x, g, c.B, K, Bp.p0(), Bp.p1(), Bp.inv_scale, Bp.ldp);
  ctx->split_bytes += 8.0 * (double)c.B * N * P;
  TcParams ep{part, (long)N, (long)c.outC * N, 0, nullptr, nullptr, 0, 0, 0, GN_ACT_LINEAR, c.outC, N, P, 1, 0, ctx->d_status, nullptr, 0, 1};
  conv_tc_count(ctx, (double)c.B * c.outC, N, P);
  GN_TRY(tc_run(ctx, A, Bp, ep));
  GN_LAUNCH(ctx, conv_wgrad_reduce_kernel, cdiv((long)c.outC * N, 128), 128, 0, (const float*)part, c.B, c.outC, K, gW, gb);
  return check_launch("conv_tc_wgrad");
}

}  // namespace gn
