// conv_lstm.cuh -- Conv2D / MaxPool2D kernels (NCHW) and the LSTM recurrence kernels.
#pragma once
#include <cooperative_groups.h>
#include "common.cuh"
#include "rowops.cuh"

namespace gn {
namespace cg = cooperative_groups;

struct ConvShape { int B, inC, outC, k, s, p, H, W, oH, oW; };

// z[b,oc,oh,ow] = bias[oc] + sum_{ic,kh,kw} W[oc,ic,kh,kw] x[b,ic,oh*s+kh-p,ow*s+kw-p]; a = act(z)
// reference: conv2d.go:716-959 (zero padding = out-of-range taps skipped; bias added last)
__global__ void conv2d_fwd_kernel(const float* __restrict__ x, const float* __restrict__ Wt, const float* __restrict__ bias,
                                  float* __restrict__ z, float* __restrict__ a, ConvShape c, int act, float alpha) {
  long total = (long)c.B * c.outC * c.oH * c.oW;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int ow = (int)(i % c.oW); long r = i / c.oW; int oh = (int)(r % c.oH); r /= c.oH; int oc = (int)(r % c.outC); int b = (int)(r / c.outC);
    const float* xb = x + (long)b * c.inC * c.H * c.W;
    const float* w = Wt + (long)oc * c.inC * c.k * c.k;
    float acc = 0.f;
    for (int ic = 0; ic < c.inC; ic++)
      for (int kh = 0; kh < c.k; kh++) {
        int ih = oh * c.s + kh - c.p; if (ih < 0 || ih >= c.H) continue;
        for (int kw = 0; kw < c.k; kw++) {
          int iw = ow * c.s + kw - c.p; if (iw < 0 || iw >= c.W) continue;
          acc = fmaf(__ldg(w + (ic * c.k + kh) * c.k + kw), xb[((long)ic * c.H + ih) * c.W + iw], acc);
        }
      }
    acc += bias[oc];
    z[i] = acc; a[i] = act_fwd(act, acc, alpha);
  }
}
// dx[b,ic,ih,iw] = sum_{oc,kh,kw} g[b,oc,oh,ow] W[oc,ic,kh,kw] with oh*s+kh-p = ih   (conv2d.go:1151-1162)
__global__ void conv2d_dgrad_kernel(const float* __restrict__ g, const float* __restrict__ Wt, float* __restrict__ dx, ConvShape c) {
  long total = (long)c.B * c.inC * c.H * c.W;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int iw = (int)(i % c.W); long r = i / c.W; int ih = (int)(r % c.H); r /= c.H; int ic = (int)(r % c.inC); int b = (int)(r / c.inC);
    const float* gb = g + (long)b * c.outC * c.oH * c.oW;
    float acc = 0.f;
    for (int oc = 0; oc < c.outC; oc++)
      for (int kh = 0; kh < c.k; kh++) {
        int th = ih + c.p - kh; if (th < 0 || th % c.s) continue; int oh = th / c.s; if (oh >= c.oH) continue;
        for (int kw = 0; kw < c.k; kw++) {
          int tw = iw + c.p - kw; if (tw < 0 || tw % c.s) continue; int ow = tw / c.s; if (ow >= c.oW) continue;
          acc = fmaf(gb[((long)oc * c.oH + oh) * c.oW + ow], __ldg(Wt + (((long)oc * c.inC + ic) * c.k + kh) * c.k + kw), acc);
        }
      }
    dx[i] = acc;
  }
}
// One block per weight: dW[oc,ic,kh,kw] += sum_{b,oh,ow} g * x ; blocks >= nW reduce one bias each.
__global__ void conv2d_wgrad_kernel(const float* __restrict__ g, const float* __restrict__ x, float* __restrict__ dW, float* __restrict__ db, ConvShape c) {
  __shared__ float red[33];
  int nW = c.outC * c.inC * c.k * c.k;
  int wi = blockIdx.x;
  long span = (long)c.B * c.oH * c.oW;
  float s = 0.f;
  if (wi < nW) {
    int kw = wi % c.k; int r = wi / c.k; int kh = r % c.k; r /= c.k; int ic = r % c.inC; int oc = r / c.inC;
    for (long i = threadIdx.x; i < span; i += blockDim.x) {
      int ow = (int)(i % c.oW); long q = i / c.oW; int oh = (int)(q % c.oH); int b = (int)(q / c.oH);
      int ih = oh * c.s + kh - c.p, iw = ow * c.s + kw - c.p;
      if (ih < 0 || ih >= c.H || iw < 0 || iw >= c.W) continue;
      s = fmaf(g[(((long)b * c.outC + oc) * c.oH + oh) * c.oW + ow], x[(((long)b * c.inC + ic) * c.H + ih) * c.W + iw], s);
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) dW[wi] += s;
  } else {
    int oc = wi - nW;
    for (long i = threadIdx.x; i < span; i += blockDim.x) {
      long q = i / ((long)c.oH * c.oW); long rem = i % ((long)c.oH * c.oW);
      s += g[((long)q * c.outC + oc) * c.oH * c.oW + rem];
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) db[oc] += s;
  }
}

// Weight gradient, tiled: one block per (oc, ic) pair and batch slice, so the K*K taps of the pair share every load of
// g and the input plane is read from L1; partial sums go to part[slice][nW + outC] (bias partials from the ic == 0
// blocks) and conv2d_wgrad_final_kernel adds the slices in order.  Same sums as conv2d_wgrad_kernel.
template <int K>
__global__ void __launch_bounds__(256) conv2d_wgrad_tile_kernel(const float* __restrict__ g, const float* __restrict__ x, float* __restrict__ part, ConvShape c, int slices) {
  __shared__ float red[8][K * K + 1];
  const int pair = blockIdx.x, oc = pair / c.inC, ic = pair % c.inC, sl = blockIdx.y;
  const int bper = (c.B + slices - 1) / slices, b0 = sl * bper, b1 = min(c.B, b0 + bper);
  const int npos = c.oH * c.oW, nW = c.outC * c.inC * K * K;
  float acc[K * K], sb = 0.f;
#pragma unroll
  for (int t = 0; t < K * K; t++) acc[t] = 0.f;
  const long span = (long)max(0, b1 - b0) * npos;
  for (long i = threadIdx.x; i < span; i += 256) {
    const int b = b0 + (int)(i / npos), pos = (int)(i % npos), oh = pos / c.oW, ow = pos - oh * c.oW;
    const float gv = g[(((long)b * c.outC + oc) * c.oH + oh) * c.oW + ow];
    sb += gv;
    const float* xb = x + ((long)b * c.inC + ic) * c.H * c.W;
#pragma unroll
    for (int kh = 0; kh < K; kh++) {
      const int ih = oh * c.s + kh - c.p; if (ih < 0 || ih >= c.H) continue;
#pragma unroll
      for (int kw = 0; kw < K; kw++) {
        const int iw = ow * c.s + kw - c.p; if (iw < 0 || iw >= c.W) continue;
        acc[kh * K + kw] = fmaf(gv, xb[ih * c.W + iw], acc[kh * K + kw]);
      }
    }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int t = 0; t < K * K; t++) { const float v = warp_sum(acc[t]); if (lane == 0) red[w][t] = v; }
  sb = warp_sum(sb); if (lane == 0) red[w][K * K] = sb;
  __syncthreads();
  if (threadIdx.x <= K * K) {
    float v = 0.f;
    for (int q = 0; q < 8; q++) v += red[q][threadIdx.x];
    float* prow = part + (long)sl * (nW + c.outC);
    if (threadIdx.x < K * K) prow[(long)pair * K * K + threadIdx.x] = v;
    else if (ic == 0) prow[nW + oc] = v;
  }
}
__global__ void conv2d_wgrad_final_kernel(const float* __restrict__ part, int slices, int n, float* __restrict__ dW) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i >= n) return;
  float s = 0.f;
  for (int k = 0; k < slices; k++) s += part[(long)k * n + i];
  dW[i] += s;                                             // weights, then biases: the gradient slice is laid out W | b
}
// Input gradient for stride 1 (no division in the tap loops); same sum as conv2d_dgrad_kernel.
template <int K>
__global__ void __launch_bounds__(256) conv2d_dgrad_s1_kernel(const float* __restrict__ g, const float* __restrict__ Wt, float* __restrict__ dx, ConvShape c) {
  const long total = (long)c.B * c.inC * c.H * c.W;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int iw = (int)(i % c.W); long r = i / c.W; const int ih = (int)(r % c.H); r /= c.H; const int ic = (int)(r % c.inC), b = (int)(r / c.inC);
    const float* gb = g + (long)b * c.outC * c.oH * c.oW;
    float acc = 0.f;
    for (int oc = 0; oc < c.outC; oc++) {
      const float* gp = gb + (long)oc * c.oH * c.oW; const float* wp = Wt + ((long)oc * c.inC + ic) * K * K;
#pragma unroll
      for (int kh = 0; kh < K; kh++) {
        const int oh = ih + c.p - kh; if (oh < 0 || oh >= c.oH) continue;
#pragma unroll
        for (int kw = 0; kw < K; kw++) {
          const int ow = iw + c.p - kw; if (ow < 0 || ow >= c.oW) continue;
          acc = fmaf(gp[oh * c.oW + ow], __ldg(wp + kh * K + kw), acc);
        }
      }
    }
    dx[i] = acc;
  }
}

// ---------------------------------------------------------------- Conv1D
// Input [B, inC, L], output [B, outC, oL], weights [outC, inC, k].  reference: conv1d.go:178-216 (the sum starts from the
// bias), :254-288 (the backward pass uses the incoming gradient as it is: no activation derivative).
struct Conv1Shape { int B, inC, outC, k, s, p, L, oL; };
__global__ void conv1d_fwd_kernel(const float* __restrict__ x, const float* __restrict__ Wt, const float* __restrict__ bias, float* __restrict__ y,
                                  Conv1Shape c, int act, float alpha) {
  long total = (long)c.B * c.outC * c.oL;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int ol = (int)(i % c.oL); long r = i / c.oL; int oc = (int)(r % c.outC); int b = (int)(r / c.outC);
    const float* xb = x + (long)b * c.inC * c.L; const float* w = Wt + (long)oc * c.inC * c.k;
    float sum = bias[oc];
    for (int ic = 0; ic < c.inC; ic++) for (int k = 0; k < c.k; k++) {
      int pos = ol * c.s + k - c.p;
      if (pos >= 0 && pos < c.L) sum = fmaf(xb[(long)ic * c.L + pos], __ldg(w + ic * c.k + k), sum);
    }
    y[i] = act_fwd(act, sum, alpha);
  }
}
__global__ void conv1d_dgrad_kernel(const float* __restrict__ g, const float* __restrict__ Wt, float* __restrict__ dx, Conv1Shape c) {
  long total = (long)c.B * c.inC * c.L;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int pos = (int)(i % c.L); long r = i / c.L; int ic = (int)(r % c.inC); int b = (int)(r / c.inC);
    const float* gb = g + (long)b * c.outC * c.oL;
    float acc = 0.f;
    for (int oc = 0; oc < c.outC; oc++) for (int k = 0; k < c.k; k++) {
      int t = pos + c.p - k; if (t < 0 || t % c.s) continue; int ol = t / c.s; if (ol >= c.oL) continue;
      acc = fmaf(gb[(long)oc * c.oL + ol], __ldg(Wt + ((long)oc * c.inC + ic) * c.k + k), acc);
    }
    dx[i] = acc;
  }
}
// One block per weight: dW[oc,ic,k] += sum_{b,ol} g x ; blocks >= nW reduce one bias each.
__global__ void conv1d_wgrad_kernel(const float* __restrict__ g, const float* __restrict__ x, float* __restrict__ dW, float* __restrict__ db, Conv1Shape c) {
  __shared__ float red[33];
  const int nW = c.outC * c.inC * c.k, wi = blockIdx.x; const long span = (long)c.B * c.oL;
  float s = 0.f;
  if (wi < nW) {
    const int k = wi % c.k; int r = wi / c.k; const int ic = r % c.inC, oc = r / c.inC;
    for (long i = threadIdx.x; i < span; i += blockDim.x) {
      const int ol = (int)(i % c.oL), b = (int)(i / c.oL), pos = ol * c.s + k - c.p;
      if (pos < 0 || pos >= c.L) continue;
      s = fmaf(g[((long)b * c.outC + oc) * c.oL + ol], x[((long)b * c.inC + ic) * c.L + pos], s);
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) dW[wi] += s;
  } else {
    const int oc = wi - nW;
    for (long i = threadIdx.x; i < span; i += blockDim.x) s += g[((long)(i / c.oL) * c.outC + oc) * c.oL + i % c.oL];
    s = block_sum(s, red);
    if (threadIdx.x == 0) db[oc] += s;
  }
}

struct PoolShape { int B, C, k, s, p, H, W, oH, oW; };
// reference: maxpool2d.go:192-221 (init -inf, strict '>', first maximum wins, argmax = flat CHW index)
__global__ void maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int* __restrict__ arg, PoolShape c) {
  long total = (long)c.B * c.C * c.oH * c.oW;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int ow = (int)(i % c.oW); long r = i / c.oW; int oh = (int)(r % c.oH); r /= c.oH; int ch = (int)(r % c.C); int b = (int)(r / c.C);
    const float* xb = x + (long)b * c.C * c.H * c.W;
    float mv = -INFINITY; int mi = -1;
    for (int kh = 0; kh < c.k; kh++) for (int kw = 0; kw < c.k; kw++) {
      int ih = oh * c.s + kh - c.p, iw = ow * c.s + kw - c.p;
      if (ih >= 0 && ih < c.H && iw >= 0 && iw < c.W) { int idx = (ch * c.H + ih) * c.W + iw; float v = xb[idx]; if (v > mv) { mv = v; mi = idx; } }
    }
    y[i] = mv; arg[i] = mi;
  }
}
// dx zero-filled beforehand; windows may overlap when stride < kernel, hence the atomic add (maxpool2d.go:395-406)
__global__ void maxpool_bwd_kernel(const float* __restrict__ g, const int* __restrict__ arg, float* __restrict__ dx, PoolShape c) {
  long total = (long)c.B * c.C * c.oH * c.oW; long per_out = (long)c.C * c.oH * c.oW, per_in = (long)c.C * c.H * c.W;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int a = arg[i]; if (a >= 0) atomicAdd(dx + (i / per_out) * per_in + a, g[i]);
  }
}

// Average pooling: mean over the taps inside the input (padded taps are not counted; a window with no valid tap
// gives 0).  reference: avgpool2d.go:172-228
__global__ void avgpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, PoolShape c) {
  long total = (long)c.B * c.C * c.oH * c.oW;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int ow = (int)(i % c.oW); long r = i / c.oW; int oh = (int)(r % c.oH); r /= c.oH;      // r = b * C + ch
    const float* xp = x + r * c.H * c.W;
    float sum = 0.f; int cnt = 0;
    for (int kh = 0; kh < c.k; kh++) for (int kw = 0; kw < c.k; kw++) {
      int ih = oh * c.s + kh - c.p, iw = ow * c.s + kw - c.p;
      if (ih >= 0 && ih < c.H && iw >= 0 && iw < c.W) { sum += xp[ih * c.W + iw]; cnt++; }
    }
    y[i] = cnt > 0 ? sum * (1.f / (float)cnt) : 0.f;
  }
}
// Backward in gather form (one thread per input element, no atomics): dx = sum over the windows that contain the element
// of g / count(window), windows visited in the reference's (oh, ow) order.  reference: avgpool2d.go:441-468
__global__ void avgpool_bwd_kernel(const float* __restrict__ g, float* __restrict__ dx, PoolShape c) {
  long total = (long)c.B * c.C * c.H * c.W;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int iw = (int)(i % c.W); long r = i / c.W; int ih = (int)(r % c.H); r /= c.H;          // r = b * C + ch
    const float* gp = g + r * c.oH * c.oW;
    float acc = 0.f;
    for (int oh = 0; oh < c.oH; oh++) {
      int kh = ih - oh * c.s + c.p; if (kh < 0 || kh >= c.k) continue;
      for (int ow = 0; ow < c.oW; ow++) {
        int kw = iw - ow * c.s + c.p; if (kw < 0 || kw >= c.k) continue;
        int cnt = 0;
        for (int a = 0; a < c.k; a++) for (int b = 0; b < c.k; b++) {
          int h2 = oh * c.s + a - c.p, w2 = ow * c.s + b - c.p;
          if (h2 >= 0 && h2 < c.H && w2 >= 0 && w2 < c.W) cnt++;
        }
        acc += gp[oh * c.oW + ow] * (1.f / (float)cnt);
      }
    }
    dx[i] = acc;
  }
}

// ---------------------------------------------------------------- LSTM
// Forward recurrence of one sample per block, thread i = hidden unit i.
// reference: lstm.go:276-407.  The reference's gate helpers (lstm.go:1065-1101) run over the first H of the
// 4H pre-activation rows, so only the input gate receives Wx*x + Wh*h; forget, cell and output gates see
// their biases alone and are constant over time.
// Saves per (sample, t): input-gate pre-activation, cell state, hidden state.
// `xproj` != 0: pre_i already holds the input projection Wx[0:H] x_t of every (sample, t) (one tensor-core contraction
// over all B*T rows, issued before this kernel); the kernel then only runs the recurrent part.
__global__ void lstm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ Wx, const float* __restrict__ Wh, const float* __restrict__ bias,
                                float* __restrict__ pre_i, float* __restrict__ c_all, float* __restrict__ h_all, float* __restrict__ out,
                                int T, int in, int H, int return_seq, int xproj) {
  extern __shared__ float sm[];
  float* WhT = sm;                 // [H][H]  WhT[j*H+i] = Wh[i,j], rows 0..H-1 of the 4H
  float* WxT = WhT + (long)H * H;  // [in][H]
  float* hbuf = WxT + (long)in * H;  // [2][H]
  float* xbuf = hbuf + 2 * H;        // [in]
  const int s = blockIdx.x, i = threadIdx.x;
  for (int e = threadIdx.x; e < H * H; e += blockDim.x) { int r = e / H, j = e % H; WhT[j * H + r] = Wh[e]; }
  if (!xproj) for (int e = threadIdx.x; e < H * in; e += blockDim.x) { int r = e / in, j = e % in; WxT[j * H + r] = Wx[e]; }
  if (i < H) { hbuf[i] = 0.f; hbuf[H + i] = 0.f; }
  float bi = 0.f, fg = 0.f, cg = 0.f, og = 0.f, c = 0.f;
  if (i < H) { bi = bias[i]; fg = act_fwd(GN_ACT_SIGMOID, bias[H + i]); cg = act_fwd(GN_ACT_TANH, bias[2 * H + i]); og = act_fwd(GN_ACT_SIGMOID, bias[3 * H + i]); }
  __syncthreads();
  const float* xs = x + (long)s * T * in;
  for (int t = 0; t < T; t++) {
    if (!xproj) { for (int e = threadIdx.x; e < in; e += blockDim.x) xbuf[e] = xs[(long)t * in + e]; }
    __syncthreads();
    const float* hp = hbuf + (t & 1) * H; float* hn = hbuf + ((t + 1) & 1) * H;
    if (i < H) {
      float sx = 0.f;
      if (xproj) sx = pre_i[((long)s * T + t) * H + i];
      else for (int j = 0; j < in; j++) sx = fmaf(WxT[j * H + i], xbuf[j], sx);
      float pre = bi + sx;
      for (int j = 0; j < H; j++) pre = fmaf(WhT[j * H + i], hp[j], pre);
      float ig = act_fwd(GN_ACT_SIGMOID, pre);
      c = fg * c + ig * cg;
      float h = og * act_fwd(GN_ACT_TANH, c);
      long o = ((long)s * T + t) * H + i;
      pre_i[o] = pre; c_all[o] = c; h_all[o] = h; hn[i] = h;
      if (return_seq) out[o] = h; else if (t == T - 1) out[(long)s * H + i] = h;
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------- GRU
// Forward recurrence of one sample per block, thread i = hidden unit i.  reference: gru.go:192-288.
// `pre` [B, T, 3H] holds b + Wx x_t of every step on entry (one contraction over all B*T rows, issued before) and the
// complete pre-activations (update | reset | candidate) on exit.  The layer has 2H recurrent rows: the candidate's
// recurrent product uses the reset gate's rows on r (.) h_prev (gru.go:247-258).
__global__ void gru_fwd_kernel(const float* __restrict__ Wh, float* __restrict__ pre, float* __restrict__ h_all, float* __restrict__ out, int T, int H, int return_seq) {
  extern __shared__ float sm[];
  float* WzT = sm;                   // [H][H]  WzT[j*H+i] = Wh[i, j]        (update rows)
  float* WrT = WzT + (long)H * H;    // [H][H]  WrT[j*H+i] = Wh[H + i, j]    (reset rows)
  float* hbuf = WrT + (long)H * H;   // [2][H]
  float* rh = hbuf + 2 * H;          // [H]  r (.) h_prev
  const int s = blockIdx.x, i = threadIdx.x;
  for (int e = threadIdx.x; e < H * H; e += blockDim.x) { const int r = e / H, j = e % H; WzT[j * H + r] = Wh[e]; WrT[j * H + r] = Wh[(long)H * H + e]; }
  if (i < H) { hbuf[i] = 0.f; hbuf[H + i] = 0.f; }
  __syncthreads();
  for (int t = 0; t < T; t++) {
    const float* hp = hbuf + (t & 1) * H; float* hn = hbuf + ((t + 1) & 1) * H;
    float* pr = pre + ((long)s * T + t) * 3 * H;
    float pz = 0.f, prr = 0.f, z = 0.f, hprev = 0.f;
    if (i < H) {
      pz = pr[i]; prr = pr[H + i]; hprev = hp[i];
      for (int j = 0; j < H; j++) { const float hj = hp[j]; pz = fmaf(WzT[j * H + i], hj, pz); prr = fmaf(WrT[j * H + i], hj, prr); }
      z = act_fwd(GN_ACT_SIGMOID, pz);
      rh[i] = act_fwd(GN_ACT_SIGMOID, prr) * hprev;
    }
    __syncthreads();
    if (i < H) {
      float pc = pr[2 * H + i];
      for (int j = 0; j < H; j++) pc = fmaf(WrT[j * H + i], rh[j], pc);
      const float c = act_fwd(GN_ACT_TANH, pc);
      const float h = hprev + z * (c - hprev);
      pr[i] = pz; pr[H + i] = prr; pr[2 * H + i] = pc;
      const long o = ((long)s * T + t) * H + i;
      h_all[o] = h; hn[i] = h;
      if (return_seq) out[o] = h; else if (t == T - 1) out[(long)s * H + i] = h;
    }
    __syncthreads();
  }
}
// Back-propagation through time of one sample per block.  reference: gru.go:360-534 with unroller.go:190-209, literal:
// the reset gate's delta is never formed (stays zero), the candidate's gradient is scaled by (1 - z) and the
// hidden-state pass-through by z, the candidate's contribution to dh_prev is indexed by the output unit's reset gate,
// and dh_prev is ADDED to the incoming gradient before it is handed to the previous step.
// Writes the gate deltas D [B,T,3H] (update | zero | candidate), h_{t-1} [B,T,H] and r (.) h_{t-1} [B,T,H] for the
// weight-gradient contractions.
__global__ void gru_bwd_kernel(const float* __restrict__ gout, const float* __restrict__ Wh, const float* __restrict__ pre, const float* __restrict__ h_all,
                               float* __restrict__ D, float* __restrict__ hprev_all, float* __restrict__ rh_all, int T, int H, int return_seq) {
  extern __shared__ float sm[];
  float* dU = sm; float* dCr = sm + H;
  const int s = blockIdx.x, i = threadIdx.x;
  float cur = 0.f;
  for (int t = T - 1; t >= 0; t--) {
    float z = 0.f;
    if (i < H) {
      if (return_seq) cur += gout[((long)s * T + t) * H + i]; else if (t == T - 1) cur += gout[(long)s * H + i];
      const float* pr = pre + ((long)s * T + t) * 3 * H;
      z = act_fwd(GN_ACT_SIGMOID, pr[i]);
      const float r = act_fwd(GN_ACT_SIGMOID, pr[H + i]), c = act_fwd(GN_ACT_TANH, pr[2 * H + i]);
      const long o = ((long)s * T + t) * H + i;
      const float hprev = t > 0 ? h_all[o - H] : 0.f;
      const float du = cur * (c - hprev) * z * (1.f - z);
      const float dc = cur * (1.f - z) * (1.f - c * c);
      float* Dr = D + ((long)s * T + t) * 3 * H;
      Dr[i] = du; Dr[H + i] = 0.f; Dr[2 * H + i] = dc;
      hprev_all[o] = hprev; rh_all[o] = r * hprev;
      dU[i] = du; dCr[i] = dc * r;
    }
    __syncthreads();
    if (i < H) {
      float sum = 0.f;
      for (int j = 0; j < H; j++) sum = fmaf(Wh[(long)j * H + i], dU[j], sum);
      for (int j = 0; j < H; j++) sum = fmaf(Wh[((long)H + j) * H + i], dCr[j], sum);
      cur = cur + (sum + cur * z);
    }
    __syncthreads();
  }
}
// Back-propagation through time of one sample per block; writes the gate deltas D[s,t,4H].
// reference: lstm.go:476-698 + unroller.go:190-209: the hidden-state gradient handed to step t-1 is the
// gradient of step t PLUS Wh^T d (a running sum), because LSTM.Backward adds dhPrev into its argument.
__global__ void lstm_bwd_kernel(const float* __restrict__ gout, const float* __restrict__ Wh, const float* __restrict__ bias,
                                const float* __restrict__ pre_i, const float* __restrict__ c_all, float* __restrict__ D,
                                int T, int H, int return_seq) {
  extern __shared__ float sm[];
  float* d = sm;   // [4H]
  const int s = blockIdx.x, i = threadIdx.x;
  float cur = 0.f, dcNext = 0.f, bf = 0.f, bg = 0.f, bo = 0.f;
  if (i < H) { bf = bias[H + i]; bg = bias[2 * H + i]; bo = bias[3 * H + i]; }
  for (int t = T - 1; t >= 0; t--) {
    if (i < H) {
      if (return_seq) cur += gout[((long)s * T + t) * H + i]; else if (t == T - 1) cur += gout[(long)s * H + i];
      long o = ((long)s * T + t) * H + i;
      float pre = pre_i[o], c = c_all[o], cprev = t > 0 ? c_all[o - H] : 0.f;
      float ig = act_fwd(GN_ACT_SIGMOID, pre), fg = act_fwd(GN_ACT_SIGMOID, bf), cgt = act_fwd(GN_ACT_TANH, bg), og = act_fwd(GN_ACT_SIGMOID, bo);
      float tanhC = act_fwd(GN_ACT_TANH, c);
      float dc = cur * og * (1.f - tanhC * tanhC) + dcNext;
      float di = dc * cgt * act_der(GN_ACT_SIGMOID, pre);
      float df = dc * cprev * act_der(GN_ACT_SIGMOID, bf);
      float dg = dc * ig * act_der(GN_ACT_TANH, bg);
      float dout = cur * tanhC * act_der(GN_ACT_SIGMOID, bo);
      dcNext = dc * fg;
      d[i] = di; d[H + i] = df; d[2 * H + i] = dg; d[3 * H + i] = dout;
      float* Dr = D + ((long)s * T + t) * 4 * H;
      Dr[i] = di; Dr[H + i] = df; Dr[2 * H + i] = dg; Dr[3 * H + i] = dout;
    }
    __syncthreads();
    if (i < H) {
      float sum = 0.f;
      for (int r = 0; r < 4 * H; r++) sum = fmaf(Wh[(long)r * H + i], d[r], sum);
      cur += sum;
    }
    __syncthreads();
  }
}

// The reference clips the WHOLE accumulated LSTM gradient to L2 norm <= 1 after every time-step of every
// sample (lstm.go:694, :725-751), so the gradient of a worker chunk is a sequential recurrence over its
// (sample, t) updates  g <- clip(g + d_k (x) [x_last ; h_{t-1} ; 1]).  One thread-block cluster runs one
// chunk: the 4H gradient rows are split over the cluster's CTAs, each keeps its rows in shared memory,
// and the squared norm is exchanged through distributed shared memory once per update.
// Row r of the running gradient is [gWx[r,:] | gWh[r,:] | gb[r]].
constexpr int SCAN_CLUSTER = 8, SCAN_THREADS = 256;
__global__ void __launch_bounds__(SCAN_THREADS) lstm_grad_scan_kernel(
    const float* __restrict__ D, const float* __restrict__ x, const float* __restrict__ h_all, float* __restrict__ out,
    int T, int in, int H, int n_samples_total, int chunk, int first_sample_offset) {
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = cluster.block_rank();
  const int cl = blockIdx.x / SCAN_CLUSTER;                    // which worker chunk
  const int R4 = 4 * H, ZW = in + H + 1;
  const int rpc = (R4 + SCAN_CLUSTER - 1) / SCAN_CLUSTER, row0 = rank * rpc, nrows = max(0, min(rpc, R4 - row0));
  extern __shared__ float sm[];
  float* acc = sm;                         // [rpc][ZW]
  float* dsh = acc + (long)rpc * ZW;       // [rpc]
  float* zsh = dsh + rpc;                  // [ZW]
  float* red = zsh + ZW;                   // [33]
  __shared__ float part[2][SCAN_CLUSTER];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = SCAN_THREADS >> 5;
  for (int e = tid; e < rpc * ZW; e += SCAN_THREADS) acc[e] = 0.f;
  cluster.sync();
  // samples of this chunk, relative to the tensors passed in
  int s_begin = cl * chunk - first_sample_offset, s_end = min(n_samples_total, s_begin + chunk);
  s_begin = max(s_begin, 0);
  long step = 0;
  for (int s = s_begin; s < s_end; s++) {
    for (int t = T - 1; t >= 0; t--, step++) {
      const int buf = (int)(step & 1);
      const float* Dr = D + ((long)s * T + t) * R4 + row0;
      for (int e = tid; e < nrows; e += SCAN_THREADS) dsh[e] = Dr[e];
      for (int e = tid; e < ZW; e += SCAN_THREADS) {
        float v;
        if (e < in) v = x[(long)s * T * in + (long)(T - 1) * in + e];           // lstm.go:592-621: input of the LAST forward call
        else if (e < in + H) v = t > 0 ? h_all[((long)s * T + (t - 1)) * H + (e - in)] : 0.f;
        else v = 1.f;
        zsh[e] = v;
      }
      __syncthreads();
      float sq = 0.f;
      for (int r = warp; r < nrows; r += nwarps) {
        float dr = dsh[r]; float* a = acc + (long)r * ZW;
        for (int c = lane; c < ZW; c += 32) { float v = fmaf(dr, zsh[c], a[c]); a[c] = v; sq = fmaf(v, v, sq); }
      }
      sq = block_sum(sq, red);
      if (tid < SCAN_CLUSTER) { float* remote = cluster.map_shared_rank(&part[buf][rank], tid); *remote = sq; }
      cluster.sync();
      float total = 0.f;
#pragma unroll
      for (int q = 0; q < SCAN_CLUSTER; q++) total += part[buf][q];
      float norm = sqrtf(total);
      if (norm > 1.f) {
        float sc = 1.f / norm;
        for (int r = warp; r < nrows; r += nwarps) { float* a = acc + (long)r * ZW; for (int c = lane; c < ZW; c += 32) a[c] *= sc; }
      }
    }
  }
  __syncthreads();
  // write out in the flat layout: gWx[4H,in] | gWh[4H,H] | gb[4H]
  float* o = out + (long)cl * ((long)R4 * ZW);
  for (int e = tid; e < nrows * ZW; e += SCAN_THREADS) {
    int r = e / ZW, c = e % ZW, gr = row0 + r; float v = acc[(long)r * ZW + c];
    if (c < in) o[(long)gr * in + c] = v;
    else if (c < in + H) o[(long)R4 * in + (long)gr * H + (c - in)] = v;
    else o[(long)R4 * in + (long)R4 * H + gr] = v;
  }
  cluster.sync();
}


// ---------------------------------------------------------------- the same recurrence through Gram matrices
// Every update is rank one, u_k = d_k (x) z_k, so the gradient after any number of clipped updates is a weighted sum
// g = sum_j w_j u_j, and the only thing the clipping needs is the norm:
//     |g + u_k|^2 = |g|^2 + 2 <g, u_k> + |u_k|^2,   <u_j, u_k> = <d_j, d_k> <z_j, z_k> =: G[j,k].
// With f_k the clip factor of update k and S_k = f_0 ... f_k, the coefficient of u_j after update k is S_k / S_{j-1},
// hence <g_{k-1}, u_k> = S_{k-1} sum_{j<k} G[j,k] / S_{j-1}.  The two Gram products and the final g = (diag(w) D)^T Z
// are contractions (tensor cores); what stays sequential is one dot product of length k per update.
//
// Rows of Dm [n, 4H] and Zm [n, in+H+1] in update order: chunk by chunk, samples ascending, time descending.
__global__ void lstm_gather_updates_kernel(const float* __restrict__ D, const float* __restrict__ x, const float* __restrict__ h_all,
                                           float* __restrict__ Dm, float* __restrict__ Zm, int T, int in, int H, long n_updates) {
  const int R4 = 4 * H, ZW = in + H + 1;
  const long k = blockIdx.x; if (k >= n_updates) return;
  const int s = (int)(k / T), t = T - 1 - (int)(k % T);
  for (int e = threadIdx.x; e < R4 + ZW; e += blockDim.x) {
    if (e < R4) Dm[k * R4 + e] = D[((long)s * T + t) * R4 + e];
    else {
      const int c = e - R4; float v;
      if (c < in) v = x[(long)s * T * in + (long)(T - 1) * in + c];                 // input of the LAST forward call (lstm.go:592-621)
      else if (c < in + H) v = t > 0 ? h_all[((long)s * T + (t - 1)) * H + (c - in)] : 0.f;
      else v = 1.f;
      Zm[k * ZW + c] = v;
    }
  }
}
// G <- G (.) G2 on the lower triangles (row k, columns j <= k) of `nb` matrices of size Kc x Kc
__global__ void lstm_gram_mul_kernel(float* __restrict__ G, const float* __restrict__ G2, int Kc, long total) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int j = (int)(i % Kc), k = (int)((i / Kc) % Kc);
    if (j <= k) G[i] *= G2[i];
  }
}
// The updates of a worker chunk are walked in groups of GRAM_BS.  cw[j] holds the CURRENT coefficient of update j (the
// product of all clip factors applied since it was added: at most 1, and free to underflow to 0, which is then also
// what the literal recurrence has made of that update).  For the group starting at k0,
//     v[r] = sum_{j<k0} cw[j] G[k0+r, j] = <g_{k0-1}, u_{k0+r}>
// is a matrix-vector product over all SMs (lstm_gram_prefix_kernel, one block per row and chunk); inside the group the
// earlier updates only get scaled by s = product of the group's clip factors so far, and the group's own GRAM_BS
// coefficients live in shared memory and are walked sequentially by one warp (lstm_gram_group_kernel), which finally
// scales cw[0..k0) by s and appends its own.  The two kernels are launched once per group; the stream orders them.
// The norm recurrence and the coefficients are kept in double.  n2[chunk] = |g|^2.
constexpr int GRAM_BS = 128, GRAM_MAX_K = 1 << 20;
constexpr size_t GRAM_GROUP_SMEM = (size_t)GRAM_BS * (GRAM_BS + 1) * sizeof(float);
__global__ void lstm_gram_prefix_kernel(const float* __restrict__ G, const double* __restrict__ cw, double* __restrict__ v, int Kc, long n_total, int k0) {
  __shared__ double red[8];
  const int chunk = blockIdx.y, r = blockIdx.x, tid = threadIdx.x;
  const long first = (long)chunk * Kc; const int n = (int)max(0L, min((long)Kc, n_total - first));
  if (k0 + r >= n) return;
  const float* row = G + (long)chunk * Kc * Kc + (long)(k0 + r) * Kc; const double* c = cw + first;
  double acc = 0.0;
  int j = tid;
  for (; j + 3 * 256 < k0; j += 4 * 256)
    acc += (c[j] * (double)row[j] + c[j + 256] * (double)row[j + 256]) + (c[j + 512] * (double)row[j + 512] + c[j + 768] * (double)row[j + 768]);
  for (; j < k0; j += 256) acc += c[j] * (double)row[j];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((tid & 31) == 0) red[tid >> 5] = acc;
  __syncthreads();
  if (tid == 0) { double a = 0.0; for (int q = 0; q < 8; q++) a += red[q]; v[(long)chunk * GRAM_BS + r] = a; }
}
// One warp walks the group.  Lane l owns rows l, l+32, ... of the diagonal block and keeps for each of them
//     q[r'] = <g, u_{k0+r'}>  under the gradient g as it stands after the steps done so far,
// which starts at v[r'] and follows q <- f (q + G[r'][r]) when step r adds u_r and scales by the clip factor f.  Step r
// therefore needs one broadcast of q[r] and no reduction.  The factors are kept, and the group's coefficients are
// their suffix products.
__global__ void __launch_bounds__(256) lstm_gram_group_kernel(const float* __restrict__ G, double* __restrict__ cw, const double* __restrict__ v,
                                                              double* __restrict__ n2buf, int Kc, long n_total, int k0) {
  constexpr int QN = GRAM_BS / 32;
  extern __shared__ __align__(16) float gram_smem[];
  float (*Gd)[GRAM_BS + 1] = reinterpret_cast<float (*)[GRAM_BS + 1]>(gram_smem);
  __shared__ double fr[GRAM_BS], om[GRAM_BS];
  const int chunk = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long first = (long)chunk * Kc; const int n = (int)max(0L, min((long)Kc, n_total - first));
  if (k0 >= n) return;
  const int nb = min(GRAM_BS, n - k0);
  const float* Gc = G + (long)chunk * Kc * Kc; double* c = cw + first;
  for (int e = tid; e < GRAM_BS * GRAM_BS; e += 256) {
    const int r = e / GRAM_BS, q = e % GRAM_BS;
    Gd[r][q] = (r < nb && q < nb) ? Gc[(long)(k0 + r) * Kc + k0 + q] : 0.f;
  }
  __syncthreads();
  if (warp == 0) {
    double n2 = k0 == 0 ? 0.0 : n2buf[chunk];
    double q[QN];
#pragma unroll
    for (int i = 0; i < QN; i++) { const int r = lane + 32 * i; q[i] = (k0 > 0 && r < nb) ? v[(long)chunk * GRAM_BS + r] : 0.0; }
    // the block's column r and its diagonal entry are fetched one step ahead, so that the step itself is only the
    // broadcast, the norm update and the clip factor (single-precision reciprocal square root + one Newton step)
    float gcol[QN], gdiag = Gd[0][0];
#pragma unroll
    for (int i2 = 0; i2 < QN; i2++) gcol[i2] = Gd[lane + 32 * i2][0];
#pragma unroll
    for (int i = 0; i < QN; i++) {
      for (int rl = 0; rl < 32; rl++) {
        const int r = 32 * i + rl;
        if (r >= nb) break;
        const double qr = __shfl_sync(0xffffffffu, q[i], rl);
        float ncol[QN]; const int rn = min(r + 1, GRAM_BS - 1);
#pragma unroll
        for (int i2 = 0; i2 < QN; i2++) ncol[i2] = Gd[lane + 32 * i2][rn];
        const float ndiag = Gd[rn][rn];
        double qg[QN];
#pragma unroll
        for (int i2 = 0; i2 < QN; i2++) qg[i2] = q[i2] + (double)gcol[i2];
        const double np = n2 + 2.0 * qr + (double)gdiag;
        double f0 = (double)rsqrtf((float)np);
        f0 = f0 * (1.5 - 0.5 * np * f0 * f0);
        const bool clip = np > 1.0;                                               // clip to norm 1 (lstm.go:738-750)
        const double f = clip ? f0 : 1.0;
        n2 = clip ? 1.0 : np;
#pragma unroll
        for (int i2 = 0; i2 < QN; i2++) { q[i2] = f * qg[i2]; gcol[i2] = ncol[i2]; }
        gdiag = ndiag;
        if (lane == 0) fr[r] = f;
      }
    }
    __syncwarp();
    if (lane == 0) {
      double a = 1.0;
      for (int r = nb - 1; r >= 0; r--) { a *= fr[r]; om[r] = a; }
      n2buf[chunk] = n2;
    }
  }
  __syncthreads();
  const double sg = om[0];
  for (int j = tid; j < k0; j += 256) c[j] *= sg;
  if (tid < nb) c[k0 + tid] = om[tid];
}
// w[j] = (float) cw[j], zero beyond the chunk's last update
__global__ void lstm_gram_weights_kernel(const double* __restrict__ cw, float* __restrict__ w, int Kc, long n_total, long total) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long chunk = i / Kc; const long n = max(0L, min((long)Kc, n_total - chunk * Kc));
    w[i] = (i - chunk * Kc) < n ? (float)cw[i] : 0.f;
  }
}
__global__ void lstm_scale_rows_kernel(float* __restrict__ Dm, const float* __restrict__ w, int R4, long total) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) Dm[i] *= w[i / R4];
}
// chunk results [nchunks][4H][in+H+1] -> flat layout gWx[4H,in] | gWh[4H,H] | gb[4H], chunks added in worker order
__global__ void lstm_scatter_grad_kernel(const float* __restrict__ Gc, int nchunks, int in, int H, float* __restrict__ out) {
  const int R4 = 4 * H, ZW = in + H + 1; const long total = (long)R4 * ZW;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / ZW), c = (int)(i % ZW);
    float v = 0.f; for (int q = 0; q < nchunks; q++) v += Gc[(long)q * total + i];
    if (c < in) out[(long)r * in + c] = v; else if (c < in + H) out[(long)R4 * in + (long)r * H + (c - in)] = v; else out[(long)R4 * in + (long)R4 * H + r] = v;
  }
}

}  // namespace gn
