// rowops.cuh -- the memory-bound kernels of the training step: activations and their
// derivatives, (log-)softmax heads with the reference's loss gradients, LayerNorm,
// embedding / positional table / CLS pooling, the attention row kernels, reductions over
// samples and tokens, and the fused Adam update.  All are coalesced, 128-bit where the
// shape allows, and reduce with warp shuffles.
#pragma once
#include <cuda_fp16.h>
#include "common.cuh"

namespace gn {

// ---------------------------------------------------------------- activations
// reference: internal/activations/activations.go:25-58, :135-143 (float64 libm then rounded), :62-82 (LeakyReLU),
// :241-275 (GELU, tanh form: Activate in float32 around a float64 tanh, Derivative in float64), :277-309 (SiLU), :311-340 (ELU)
__host__ __device__ inline float act_alpha_of(int act, int bits) {
  float a = 0.f; memcpy(&a, &bits, 4);
  if (bits == 0) a = act == GN_ACT_LEAKY_RELU ? 0.01f : (act == GN_ACT_ELU ? 1.0f : 0.f);
  return a;
}
__device__ __forceinline__ float act_fwd(int act, float x, float alpha = 0.f) {
  switch (act) {
    case GN_ACT_RELU: return x > 0.f ? x : 0.f;
    case GN_ACT_SIGMOID: return 1.f / (1.f + (float)exp((double)-x));
    case GN_ACT_TANH: return (float)tanh((double)x);
    case GN_ACT_LEAKY_RELU: return x > 0.f ? x : alpha * x;
    case GN_ACT_ELU: return x > 0.f ? x : alpha * ((float)exp((double)x) - 1.f);
    case GN_ACT_GELU: { float x3 = x * x * x; float arg = 0.7978845608028654f * (x + 0.044715f * x3); return 0.5f * x * (1.f + (float)tanh((double)arg)); }
    case GN_ACT_SILU: { if (x >= 0.f) return x * (1.f / (1.f + (float)exp((double)-x))); float e = (float)exp((double)x); return x * e / (1.f + e); }
    default: return x;
  }
}
__device__ __forceinline__ float act_der(int act, float x, float alpha = 0.f) {
  switch (act) {
    case GN_ACT_RELU: return x > 0.f ? 1.f : 0.f;
    case GN_ACT_SIGMOID: { float s = 1.f / (1.f + (float)exp((double)-x)); return s * (1.f - s); }
    case GN_ACT_TANH: { float t = (float)tanh((double)x); return 1.f - t * t; }
    case GN_ACT_LEAKY_RELU: return x > 0.f ? 1.f : alpha;
    case GN_ACT_ELU: return x > 0.f ? 1.f : alpha * (float)exp((double)x);
    case GN_ACT_GELU: {
      const double c = 0.044715, k = 0.7978845608028654, xd = (double)x, x2 = xd * xd, t = tanh(k * (xd + c * xd * x2));
      return (float)(0.5 * (1.0 + t) + 0.5 * xd * (1.0 - t * t) * k * (1.0 + 3.0 * c * x2));
    }
    case GN_ACT_SILU: { float sg; if (x >= 0.f) sg = 1.f / (1.f + (float)exp((double)-x)); else { float e = (float)exp((double)x); sg = e / (1.f + e); } return sg + x * sg * (1.f - sg); }
    default: return 1.f;
  }
}
__global__ void act_forward_kernel(const float* __restrict__ z, float* __restrict__ a, long n, int act, float alpha = 0.f) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) a[i] = act_fwd(act, z[i], alpha);
}
// dz = dA * act'(z)   (Dense.Backward default branch, layer.go:563-567; Conv2D.Backward conv2d.go:1133)
__global__ void act_backward_kernel(const float* __restrict__ dA, const float* __restrict__ z, float* __restrict__ dz, long n, int act, float alpha = 0.f) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) dz[i] = dA[i] * act_der(act, z[i], alpha);
}

// ---------------------------------------------------------------- softmax heads
// One block per row.  reference: activations.go:160-183 / :204-236
__global__ void softmax_rows_kernel(const float* __restrict__ z, float* __restrict__ out, int n, int log_mode) {
  __shared__ float red[33];
  const float* zr = z + (long)blockIdx.x * n; float* o = out + (long)blockIdx.x * n;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, zr[i]);
  mx = block_max(mx, red);
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += expf(zr[i] - mx);
  s = block_sum(s, red);
  if (log_mode) { float ls = logf(s); for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = zr[i] - mx - ls; }
  else for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = expf(zr[i] - mx) / s;
}

// Per-sample loss value and dL/dy.  reference: loss.go:53-68,91-105 (MSE), :120-140,165-178 (CrossEntropy:
// value = -sum y*log(max(p,1e-10)); gradient returned as p - y).
__global__ void loss_rows_kernel(const float* __restrict__ p, const float* __restrict__ y, float* __restrict__ grad,
                                 float* __restrict__ loss, int n, int kind) {
  __shared__ float red[33];
  const long off = (long)blockIdx.x * n;
  float s = 0.f;
  if (kind == GN_LOSS_MSE) {
    float f = 2.f / (float)n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { float d = p[off + i] - y[off + i]; s += d * d; grad[off + i] = f * d; }
    s = block_sum(s, red);
    if (threadIdx.x == 0) loss[blockIdx.x] = s / (float)n;
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float pr = p[off + i], yy = y[off + i];
      grad[off + i] = pr - yy;
      if (yy != 0.f) s -= yy * logf(fmaxf(pr, 1e-10f));
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) loss[blockIdx.x] = s;
  }
}

// Dense.Backward for a Softmax head (layer.go:516-528):  dz_k = sum_i g_i p_i (delta_ik - p_k) = p_k (g_k - sum_i g_i p_i)
// and for a LogSoftmax head (layer.go:547-559):          dz_k = sum_i g_i (delta_ik - e^{l_k})  = g_k - e^{l_k} sum_i g_i
__global__ void head_jacobian_kernel(const float* __restrict__ g, const float* __restrict__ out, float* __restrict__ dz, int n, int log_mode) {
  __shared__ float red[33];
  const long off = (long)blockIdx.x * n;
  float s = 0.f;
  if (log_mode) for (int i = threadIdx.x; i < n; i += blockDim.x) s += g[off + i];
  else for (int i = threadIdx.x; i < n; i += blockDim.x) s += g[off + i] * out[off + i];
  s = block_sum(s, red);
  if (log_mode) for (int i = threadIdx.x; i < n; i += blockDim.x) dz[off + i] = g[off + i] - expf(out[off + i]) * s;
  else for (int i = threadIdx.x; i < n; i += blockDim.x) dz[off + i] = out[off + i] * (g[off + i] - s);
}

// mean loss = sum_s loss_s / global_batch; sequential like net.go:711-716 (one thread: B is small)
__global__ void loss_total_kernel(const float* __restrict__ loss, int n, float* __restrict__ out_sum) {
  if (threadIdx.x == 0 && blockIdx.x == 0) { float s = 0.f; for (int i = 0; i < n; i++) s += loss[i]; out_sum[0] = s; }
}

// ---------------------------------------------------------------- reductions
// out[c] (=|+=) sum_r in[r*ld + c], rows in `chunks` slabs, partials reduced in slab order.
__global__ void colsum_partial_kernel(const float* __restrict__ in, long ld, int R, int C, float* __restrict__ part) {
  int c = blockIdx.x * blockDim.x + threadIdx.x; if (c >= C) return;
  int chunks = gridDim.y, per = (R + chunks - 1) / chunks, r0 = blockIdx.y * per, r1 = min(R, r0 + per);
  float s = 0.f;
  for (int r = r0; r < r1; r++) s += in[(long)r * ld + c];
  part[(long)blockIdx.y * C + c] = s;
}
__global__ void colsum_final_kernel(const float* __restrict__ part, int chunks, int C, float* __restrict__ out, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x; if (c >= C) return;
  float s = 0.f;
  for (int k = 0; k < chunks; k++) s += part[(long)k * C + c];
  out[c] = accumulate ? out[c] + s : s;
}
// delta[s, c] = sum_t in[s, t, c]   ([B,T,C] -> [B,C]); the reference adds per-token terms one token after another.
__global__ void token_sum_kernel(const float* __restrict__ in, int T, int C, float* __restrict__ out) {
  // block = 128 columns x 4 groups of tokens; each group adds every 4th token, four loads in flight per thread
  __shared__ float part[4][128];
  const int c = blockIdx.x * 128 + threadIdx.x, grp = threadIdx.y;
  float s = 0.f;
  if (c < C) {
    const float* p = in + (long)blockIdx.y * T * C + c;
    int t = grp;
    for (; t + 12 < T; t += 16) {
      float a0 = p[(long)t * C], a1 = p[(long)(t + 4) * C], a2 = p[(long)(t + 8) * C], a3 = p[(long)(t + 12) * C];
      s += (a0 + a1) + (a2 + a3);
    }
    for (; t < T; t += 4) s += p[(long)t * C];
  }
  part[grp][threadIdx.x] = s;
  __syncthreads();
  if (grp == 0 && c < C) out[(long)blockIdx.y * C + c] = (part[0][threadIdx.x] + part[1][threadIdx.x]) + (part[2][threadIdx.x] + part[3][threadIdx.x]);
}

// The same sum with 16-byte loads: block = 32 column groups of 4 x 8 groups of tokens (C a multiple of 4, aligned rows).
__global__ void __launch_bounds__(256) token_sum_vec_kernel(const float* __restrict__ in, int T, int C, float* __restrict__ out) {
  __shared__ float4 part[8][32];
  const int c = (blockIdx.x * 32 + threadIdx.x) * 4, grp = threadIdx.y;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c < C) {
    const float* p = in + (long)blockIdx.y * T * C + c;
    int t = grp;
    for (; t + 24 < T; t += 32) {
      const float4 a0 = *reinterpret_cast<const float4*>(p + (long)t * C), a1 = *reinterpret_cast<const float4*>(p + (long)(t + 8) * C);
      const float4 a2 = *reinterpret_cast<const float4*>(p + (long)(t + 16) * C), a3 = *reinterpret_cast<const float4*>(p + (long)(t + 24) * C);
      s.x += (a0.x + a1.x) + (a2.x + a3.x); s.y += (a0.y + a1.y) + (a2.y + a3.y); s.z += (a0.z + a1.z) + (a2.z + a3.z); s.w += (a0.w + a1.w) + (a2.w + a3.w);
    }
    for (; t < T; t += 8) { const float4 a = *reinterpret_cast<const float4*>(p + (long)t * C); s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w; }
  }
  part[grp][threadIdx.x] = s;
  __syncthreads();
  if (grp == 0 && c < C) {
    float4 r = part[0][threadIdx.x];
#pragma unroll
    for (int g = 1; g < 8; g++) { const float4 q = part[g][threadIdx.x]; r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w; }
    *reinterpret_cast<float4*>(out + (long)blockIdx.y * C + c) = r;
  }
}

// Token sums from the 32-row partial sums a plane-writing contraction leaves behind (TcParams::rowsum32): T / 32 rows per
// sequence, added in order.
__global__ void __launch_bounds__(128) token_sum_part32_kernel(const float* __restrict__ part, int groups, int C, float* __restrict__ out) {
  const int c = (blockIdx.x * 128 + threadIdx.x) * 4; if (c >= C) return;
  const float* p = part + (long)blockIdx.y * groups * C + c;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int g = 0; g < groups; g++) { const float4 q = *reinterpret_cast<const float4*>(p + (long)g * C); s.x += q.x; s.y += q.y; s.z += q.z; s.w += q.w; }
  *reinterpret_cast<float4*>(out + (long)blockIdx.y * C + c) = s;
}
// The same sum over a tensor that exists only as operand planes (two fp16 planes and an inverse scale per row, written by a
// contraction's epilogue): element = (p0 + p1) * inv_scale[row].  Same block shape as above: 4 columns per thread.
__global__ void __launch_bounds__(256) token_sum_planes_kernel(const __half* __restrict__ p0, const __half* __restrict__ p1, const float* __restrict__ inv, long ldp,
                                                               int T, int C, float* __restrict__ out) {
  __shared__ float4 part[8][32];
  const int c = (blockIdx.x * 32 + threadIdx.x) * 4, grp = threadIdx.y;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c < C) {
    const long row0 = (long)blockIdx.y * T;
    for (int t = grp; t < T; t += 8) {
      const long o = (row0 + t) * ldp + c; const float is = inv[row0 + t];
      const uint2 a = *reinterpret_cast<const uint2*>(p0 + o), b = *reinterpret_cast<const uint2*>(p1 + o);
      const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&a.x)), a1 = __half22float2(*reinterpret_cast<const __half2*>(&a.y));
      const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&b.x)), b1 = __half22float2(*reinterpret_cast<const __half2*>(&b.y));
      s.x += (a0.x + b0.x) * is; s.y += (a0.y + b0.y) * is; s.z += (a1.x + b1.x) * is; s.w += (a1.y + b1.y) * is;
    }
  }
  part[grp][threadIdx.x] = s;
  __syncthreads();
  if (grp == 0 && c < C) {
    float4 r = part[0][threadIdx.x];
#pragma unroll
    for (int g = 1; g < 8; g++) { const float4 q = part[g][threadIdx.x]; r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w; }
    *reinterpret_cast<float4*>(out + (long)blockIdx.y * C + c) = r;
  }
}

// ---------------------------------------------------------------- LayerNorm
// One warp per row.  reference: layernorm.go:268-301
__global__ void layernorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                     float* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ std_out, long rows, int n, float eps) {
  long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); if (row >= rows) return;
  int lane = threadIdx.x & 31;
  const float* xr = x + row * n; float* yr = y + row * n;
  float s = 0.f;
  for (int i = lane; i < n; i += 32) s += xr[i];
  float mean = warp_sum(s) / (float)n;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) { float d = xr[i] - mean; ss += d * d; }
  float var = warp_sum(ss) / (float)n;
  float sd = sqrtf(var + eps);
  for (int i = lane; i < n; i += 32) yr[i] = gamma[i] * ((xr[i] - mean) / sd) + beta[i];
  if (lane == 0) { mean_out[row] = mean; std_out[row] = sd; }
}
// reference: layernorm.go:389-417 -- the second term is divided by N*std*std (not std^3).
// dx may alias g.
__global__ void layernorm_bwd_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ mean_in, const float* __restrict__ std_in, float* dx, long rows, int n) {
  long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); if (row >= rows) return;
  int lane = threadIdx.x & 31;
  const float* xr = x + row * n; const float* gr = g + row * n; float* dr = dx + row * n;
  float mean = mean_in[row], sd = std_in[row];
  float sg = 0.f, sgx = 0.f;
  for (int i = lane; i < n; i += 32) { float q = gr[i] * gamma[i]; sg += q; sgx += q * (xr[i] - mean); }
  sg = warp_sum(sg); sgx = warp_sum(sgx);
  float fn = (float)n;
  for (int i = lane; i < n; i += 32) {
    float q = gr[i] * gamma[i], d = xr[i] - mean;
    float v = (q - sg / fn) / sd;
    v -= (d * sgx) / (fn * sd * sd);
    dr[i] = v;
  }
}
// gGamma[c] += sum_r g*(x-mean)/std ; gBeta[c] += sum_r g     (layernorm.go:421-433)
__global__ void layernorm_pgrad_partial_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ mean_in,
                                               const float* __restrict__ std_in, long rows, int n, float* __restrict__ part) {
  int c = blockIdx.x * blockDim.x + threadIdx.x; if (c >= n) return;
  long chunks = gridDim.y, per = (rows + chunks - 1) / chunks, r0 = blockIdx.y * per, r1 = min(rows, r0 + per);
  float sgam = 0.f, sbet = 0.f;
  for (long r = r0; r < r1; r++) { float gg = g[r * n + c]; sgam += gg * ((x[r * n + c] - mean_in[r]) / std_in[r]); sbet += gg; }
  part[((long)blockIdx.y * 2) * n + c] = sgam; part[((long)blockIdx.y * 2 + 1) * n + c] = sbet;
}
// block = 32 columns x 32 groups of chunks (1024 threads); the groups are combined through shared memory in a fixed order
__global__ void __launch_bounds__(1024) layernorm_pgrad_final_kernel(const float* __restrict__ part, int chunks, int n, float* __restrict__ gGamma, float* __restrict__ gBeta) {
  __shared__ float sa[32][33], sb[32][33];
  const int tx = threadIdx.x & 31, grp = threadIdx.x >> 5, c = blockIdx.x * 32 + tx;
  float a = 0.f, b = 0.f;
  if (c < n) for (int k = grp; k < chunks; k += 32) { a += part[((long)k * 2) * n + c]; b += part[((long)k * 2 + 1) * n + c]; }
  sa[grp][tx] = a; sb[grp][tx] = b;
  __syncthreads();
  if (grp == 0 && c < n) {
    float ta = 0.f, tb = 0.f;
    for (int k = 0; k < 32; k++) { ta += sa[k][tx]; tb += sb[k][tx]; }
    gGamma[c] += ta; gBeta[c] += tb;
  }
}

// Row-in-registers variants for n = 128 * NV (NV <= 16): one warp per row, the row is read once with 16-byte loads
// and kept in registers between the reduction and the output pass.  Same arithmetic as the kernels above.
// Optional second output of the row-in-registers kernels: the row as operand planes of the contraction engine (two fp16
// planes with row stride n, the row's inverse scale, its 2-norm) -- the kernel holds the whole row, so the row maximum
// and norm cost two warp reductions, and the separate split pass (a second read of the tensor) is not needed for the contraction that
// consumes this output.
struct RowPlaneOut { __half* p0 = nullptr; __half* p1 = nullptr; float* inv = nullptr; float* rownorm = nullptr; };
template <int NV>
__device__ __forceinline__ void row_planes_emit(const float4 (&o)[NV], long row, int lane, const RowPlaneOut& po) {
  constexpr int n = 128 * NV;
  float mx = 0.f, sq = 0.f;
#pragma unroll
  for (int k = 0; k < NV; k++) {
    mx = fmaxf(mx, fmaxf(fmaxf(fabsf(o[k].x), fabsf(o[k].y)), fmaxf(fabsf(o[k].z), fabsf(o[k].w))));
    sq += (o[k].x * o[k].x + o[k].y * o[k].y) + (o[k].z * o[k].z + o[k].w * o[k].w);
  }
  mx = warp_max(mx); sq = warp_sum(sq);
  float inv; const float sc = row_scale(mx, &inv);
  if (lane == 0) { po.inv[row] = inv; if (po.rownorm) po.rownorm[row] = sqrtf(sq) * 1.0001f; }
  uint2* h = reinterpret_cast<uint2*>(po.p0 + row * n) + lane; uint2* l = reinterpret_cast<uint2*>(po.p1 + row * n) + lane;
#pragma unroll
  for (int k = 0; k < NV; k++) {
    uint2 a, b; split2_pair(o[k].x, o[k].y, sc, a.x, b.x); split2_pair(o[k].z, o[k].w, sc, a.y, b.y);
    h[32 * k] = a; l[32 * k] = b;
  }
}
template <int NV>
__global__ void __launch_bounds__(256) layernorm_fwd_vec_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                float* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ std_out, long rows, float eps,
                                                                const RowPlaneOut po) {
  constexpr int n = 128 * NV;
  const long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5); if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float4* xr = reinterpret_cast<const float4*>(x + row * n) + lane;
  float4 v[NV];
#pragma unroll
  for (int k = 0; k < NV; k++) v[k] = xr[32 * k];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < NV; k++) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
  const float mean = warp_sum(s) / (float)n;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; k++) { float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean; ss += (a * a + b * b) + (c * c + d * d); }
  const float sd = sqrtf(warp_sum(ss) / (float)n + eps), isd = 1.f / sd;     // one reciprocal per row instead of a division per element
  float4* yr = reinterpret_cast<float4*>(y + row * n) + lane;
#pragma unroll
  for (int k = 0; k < NV; k++) {
    const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma) + lane + 32 * k), be = __ldg(reinterpret_cast<const float4*>(beta) + lane + 32 * k);
    v[k] = make_float4(ga.x * ((v[k].x - mean) * isd) + be.x, ga.y * ((v[k].y - mean) * isd) + be.y, ga.z * ((v[k].z - mean) * isd) + be.z, ga.w * ((v[k].w - mean) * isd) + be.w);
    yr[32 * k] = v[k];
  }
  if (lane == 0) { mean_out[row] = mean; std_out[row] = sd; }
  if (po.p0) row_planes_emit<NV>(v, row, lane, po);
}
template <int NV>
__global__ void __launch_bounds__(256) layernorm_bwd_vec_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ gamma,
                                                                const float* __restrict__ mean_in, const float* __restrict__ std_in, float* dx, long rows,
                                                                const RowPlaneOut po) {
  constexpr int n = 128 * NV;
  const long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5); if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float4* xr = reinterpret_cast<const float4*>(x + row * n) + lane;
  const float4* gr = reinterpret_cast<const float4*>(g + row * n) + lane;
  float4 q[NV], d[NV];
#pragma unroll
  for (int k = 0; k < NV; k++) { q[k] = gr[32 * k]; d[k] = xr[32 * k]; }
  const float mean = mean_in[row], sd = std_in[row];
  float sg = 0.f, sgx = 0.f;
#pragma unroll
  for (int k = 0; k < NV; k++) {
    const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma) + lane + 32 * k);
    q[k].x *= ga.x; q[k].y *= ga.y; q[k].z *= ga.z; q[k].w *= ga.w;
    d[k].x -= mean; d[k].y -= mean; d[k].z -= mean; d[k].w -= mean;
    sg += (q[k].x + q[k].y) + (q[k].z + q[k].w);
    sgx += (q[k].x * d[k].x + q[k].y * d[k].y) + (q[k].z * d[k].z + q[k].w * d[k].w);
  }
  sg = warp_sum(sg); sgx = warp_sum(sgx);
  const float fn = (float)n, sgn = sg / fn, isd = 1.f / sd, w = sgx / (fn * sd * sd);     // reciprocals per row, not per element
  float4* dr = reinterpret_cast<float4*>(dx + row * n) + lane;
#pragma unroll
  for (int k = 0; k < NV; k++) {
    q[k] = make_float4((q[k].x - sgn) * isd - d[k].x * w, (q[k].y - sgn) * isd - d[k].y * w,
                       (q[k].z - sgn) * isd - d[k].z * w, (q[k].w - sgn) * isd - d[k].w * w);
    dr[32 * k] = q[k];
  }
  if (po.p0) row_planes_emit<NV>(q, row, lane, po);
}
// Partial column sums for gGamma / gBeta with 16-byte loads: block = 256 threads = up to 1024 columns, grid.x covers the
// columns, grid.y the row chunks; part layout as in layernorm_pgrad_partial_kernel.
__global__ void __launch_bounds__(256) layernorm_pgrad_partial_vec_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ mean_in,
                                                                          const float* __restrict__ std_in, long rows, int n, float* __restrict__ part) {
  const int c = (blockIdx.x * 256 + threadIdx.x) * 4; if (c >= n) return;
  const long chunks = gridDim.y, per = (rows + chunks - 1) / chunks, r0 = blockIdx.y * per, r1 = min(rows, r0 + per);
  float4 sgam = make_float4(0.f, 0.f, 0.f, 0.f), sbet = sgam;
#pragma unroll 4
  for (long r = r0; r < r1; r++) {
    const float4 gg = *reinterpret_cast<const float4*>(g + r * n + c), xx = *reinterpret_cast<const float4*>(x + r * n + c);
    const float mean = mean_in[r], isd = 1.f / std_in[r];
    sgam.x += gg.x * ((xx.x - mean) * isd); sgam.y += gg.y * ((xx.y - mean) * isd); sgam.z += gg.z * ((xx.z - mean) * isd); sgam.w += gg.w * ((xx.w - mean) * isd);
    sbet.x += gg.x; sbet.y += gg.y; sbet.z += gg.z; sbet.w += gg.w;
  }
  *reinterpret_cast<float4*>(part + ((long)blockIdx.y * 2) * n + c) = sgam;
  *reinterpret_cast<float4*>(part + ((long)blockIdx.y * 2 + 1) * n + c) = sbet;
}

// ---------------------------------------------------------------- RMSNorm
// One warp per row.  reference: rmsnorm.go:222-240 (forward), :301-330 (backward); the row's rms is kept for the backward.
__global__ void rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, float* __restrict__ y, float* __restrict__ rms_out, long rows, int n, float eps) {
  long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); if (row >= rows) return;
  int lane = threadIdx.x & 31;
  const float* xr = x + row * n; float* yr = y + row * n;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) ss += xr[i] * xr[i];
  const float r = (float)sqrt((double)(warp_sum(ss) / (float)n + eps));
  for (int i = lane; i < n; i += 32) yr[i] = (xr[i] / r) * gamma[i];
  if (lane == 0) rms_out[row] = r;
}
// dx may alias g.
__global__ void rmsnorm_bwd_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ rms_in,
                                   float* dx, long rows, int n) {
  long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); if (row >= rows) return;
  int lane = threadIdx.x & 31;
  const float* xr = x + row * n; const float* gr = g + row * n; float* dr = dx + row * n;
  const float r = rms_in[row], inv = 1.f / r;
  float s = 0.f;
  for (int i = lane; i < n; i += 32) s += gr[i] * gamma[i] * xr[i];
  const float factor = warp_sum(s) / ((float)n * r * r);
  for (int i = lane; i < n; i += 32) dr[i] = (gamma[i] * inv) * (gr[i] - xr[i] * factor);
}
// gGamma[c] partial sums over a chunk of rows: sum_r g * (x / rms)    (rmsnorm.go:322-330); part[chunk][n]
__global__ void rmsnorm_pgrad_partial_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ rms_in, long rows, int n, float* __restrict__ part) {
  int c = blockIdx.x * blockDim.x + threadIdx.x; if (c >= n) return;
  long chunks = gridDim.y, per = (rows + chunks - 1) / chunks, r0 = blockIdx.y * per, r1 = min(rows, r0 + per);
  float s = 0.f;
  for (long r = r0; r < r1; r++) s += g[r * n + c] * (x[r * n + c] * (1.f / rms_in[r]));
  part[(long)blockIdx.y * n + c] = s;
}
__global__ void rmsnorm_pgrad_final_kernel(const float* __restrict__ part, int chunks, int n, float* __restrict__ gGamma) {
  int c = blockIdx.x * blockDim.x + threadIdx.x; if (c >= n) return;
  float a = 0.f;
  for (int k = 0; k < chunks; k++) a += part[(long)k * n + c];
  gGamma[c] += a;
}

// ---------------------------------------------------------------- Dropout
// The reference's generator (layer.go:61-75): s <- s * 6364136223846793005 + 1, value = float32(s >> 33) / 2^31, one
// stream per layer seeded with 42 and consumed element by element, sample by sample (dropout.go:139-152).  Draw k of the
// stream is reached by composing the affine map k times (square and multiply), so every thread can enter the stream at
// its own elements: element i of global sample g of a batch that starts after `count` draws uses draw count + g n + i + 1.
// `cnt` = the two state floats (count mod 2^20, count >> 20).
__device__ __forceinline__ unsigned long long lcg_jump(unsigned long long s0, unsigned long long k) {
  unsigned long long A = 1, C = 0, a = 6364136223846793005ull, c = 1;
  while (k) { if (k & 1) { A = A * a; C = C * a + c; } c = c * (a + 1); a = a * a; k >>= 1; }
  return A * s0 + C;
}
constexpr int DROP_RUN = 8;      // consecutive elements per thread (one jump, then the recurrence)
__global__ void dropout_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, float* __restrict__ mask, const float* __restrict__ cnt,
                                   long total, int n, float p, long first_elem) {
  const unsigned long long count = (unsigned long long)cnt[0] + ((unsigned long long)cnt[1] << 20);
  const float scale = 1.0f / (1.0f - p);
  for (long e0 = (blockIdx.x * (long)blockDim.x + threadIdx.x) * DROP_RUN; e0 < total; e0 += (long)gridDim.x * blockDim.x * DROP_RUN) {
    unsigned long long s = lcg_jump(42ull, count + (unsigned long long)(first_elem + e0));
#pragma unroll
    for (int j = 0; j < DROP_RUN; j++) {
      const long e = e0 + j; if (e >= total) break;
      s = s * 6364136223846793005ull + 1ull;
      const float r = (float)(s >> 33) / 2147483648.0f;
      const bool keep = !(r < p);
      mask[e] = keep ? 1.f : 0.f; y[e] = keep ? x[e] * scale : 0.f;
    }
  }
}
__global__ void dropout_bwd_kernel(const float* __restrict__ g, const float* __restrict__ mask, float* __restrict__ dx, long total, float p) {
  const float scale = 1.0f / (1.0f - p);
  for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) dx[e] = mask[e] > 0.f ? g[e] * scale : 0.f;
}
// after a training batch: the stream has moved on by `add` draws (global batch x elements per sample)
__global__ void dropout_advance_kernel(float* __restrict__ cnt, unsigned long long add) {
  const unsigned long long c = (unsigned long long)cnt[0] + ((unsigned long long)cnt[1] << 20) + add;
  cnt[0] = (float)(c & 0xfffffull); cnt[1] = (float)(c >> 20);
}

// ---------------------------------------------------------------- embedding / positional / CLS
// out[s,t,:] = E[floor(id)] (+ P[t,:])   reference: embedding.go:120-136, transformer.go:80-82
// A token id outside [0, V) is an error in the reference (embedding.go:124-129): the kernel records it in the status
// word (GN_STATUS_BAD_TOKEN; the host turns it into GN_ERR_INVALID_ARG and the step changes nothing) and carries on
// with a clamped id, so that nothing is read out of bounds.
constexpr int GN_STATUS_BAD_TOKEN = 100;
__global__ void embedding_fwd_kernel(const float* __restrict__ ids, const float* __restrict__ E, const float* __restrict__ P,
                                     float* __restrict__ out, long tokens, int T, int d, int V, int* __restrict__ idx_out, int* __restrict__ status) {
  long tok = blockIdx.x; if (tok >= tokens) return;
  int id = (int)floorf(ids[tok]);
  if (id < 0 || id >= V || !(ids[tok] == ids[tok])) { if (threadIdx.x == 0) atomicCAS(status, 0, GN_STATUS_BAD_TOKEN); id = id < 0 ? 0 : V - 1; }
  if (threadIdx.x == 0 && idx_out) idx_out[tok] = id;
  const float* e = E + (long)id * d; float* o = out + tok * d;
  if (P) { const float* p = P + (long)(tok % T) * d; for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = e[i] + p[i]; }
  else for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = e[i];
}
__global__ void posenc_fwd_kernel(const float* __restrict__ x, const float* __restrict__ P, float* __restrict__ out, long total, long per_sample) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) out[i] = x[i] + P[i % per_sample];
}
// Embedding.Backward zeroes its whole gradient at every call (embedding.go:151-154), so only the last
// sample of each worker chunk reaches the table.  Gradient of ONE such sample, added to the table: block t handles
// position t, and only if t is the first position of its token id; it then adds the rows of all positions with that
// id in ascending order, exactly the sum the reference's loop forms for that table row (embedding.go:156-180), and adds
// the result to the row.  No two blocks touch the same row, so there are no atomics and the result does not depend on
// scheduling; the samples of a batch are processed by consecutive launches in sample order (the order in which the
// reference adds its workers' gradients, net.go:694-700).
__global__ void embedding_bwd_sample_kernel(const float* __restrict__ g, const int* __restrict__ ids, float* __restrict__ gE, int T, int d) {
  extern __shared__ int same[];                 // positions after t that hold the same id
  __shared__ int n_same, first;
  const int t = blockIdx.x, id = ids[t];
  if (threadIdx.x == 0) {
    first = 1; n_same = 0;
    for (int u = 0; u < t; u++) if (ids[u] == id) { first = 0; break; }
    if (first) for (int u = t + 1; u < T; u++) if (ids[u] == id) same[n_same++] = u;
  }
  __syncthreads();
  if (!first) return;
  float* dst = gE + (long)id * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float s = g[(long)t * d + i];
    for (int k = 0; k < n_same; k++) s += g[(long)same[k] * d + i];
    dst[i] += s;
  }
}
// Multi-GPU exchange of the few samples that reach the table: slot q of the buffers belongs to the q-th qualifying
// sample of the global batch; the rank that owns it copies its gradient rows [T, d] and token ids (as floats) there,
// every other rank leaves zeros, and a sum all-reduce of the small buffers gives every rank all of them.
__global__ void embedding_pack_kernel(const float* __restrict__ g, const int* __restrict__ idx, float* __restrict__ rows, float* __restrict__ ids, int T, int d) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < d; i += blockDim.x) rows[(long)t * d + i] = g[(long)t * d + i];
  if (threadIdx.x == 0) ids[t] = (float)idx[t];
}
__global__ void ids_to_int_kernel(const float* __restrict__ f, int* __restrict__ out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) out[i] = (int)f[i];
}
// CLSPooling: y[s,:] = x[s,0,:]; backward: zeros except token 0   transformer.go:1684, :1715-1724
__global__ void cls_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int T, int d) {
  const float* src = x + (long)blockIdx.x * T * d; float* dst = y + (long)blockIdx.x * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
}
__global__ void cls_bwd_kernel(const float* __restrict__ g, float* __restrict__ dx, int T, int d, long total) {
  long per = (long)T * d;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    long s = i / per, r = i % per;
    dx[i] = r < d ? g[s * d + r] : 0.f;
  }
}

// ---------------------------------------------------------------- attention row kernels
// P[i, :] = softmax over j <= i of S[i,j] * inv_scale, zeros for j > i.  reference: transformer.go:470-491
// (masked scores are -1e9 before the softmax, whose exponentials are exactly 0 in fp32).
// One warp per row; rows are [batch*heads*T].
__global__ void attn_softmax_kernel(float* __restrict__ S, int T, float inv_scale, int causal, long rows) {
  long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); if (row >= rows) return;
  int lane = threadIdx.x & 31; int i = (int)(row % T); int lim = causal ? i + 1 : T;
  float* r = S + row * T;
  float mx = -INFINITY;
  for (int j = lane; j < lim; j += 32) mx = fmaxf(mx, r[j] * inv_scale);
  mx = warp_max(mx);
  float s = 0.f;
  for (int j = lane; j < lim; j += 32) s += expf(r[j] * inv_scale - mx);
  s = warp_sum(s);
  for (int j = lane; j < T; j += 32) r[j] = j < lim ? expf(r[j] * inv_scale - mx) / s : 0.f;
}
// dS[i,j] = P[i,j] * (dP[i,j] - sum_k dP[i,k] P[i,k]) * inv_scale for j <= i, else 0.  transformer.go:625-648
__global__ void attn_ds_kernel(const float* __restrict__ P, float* __restrict__ dP, int T, float inv_scale, int causal, long rows) {
  long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); if (row >= rows) return;
  int lane = threadIdx.x & 31; int i = (int)(row % T); int lim = causal ? i + 1 : T;
  const float* p = P + row * T; float* d = dP + row * T;
  float s = 0.f;
  for (int j = lane; j < lim; j += 32) s += d[j] * p[j];
  s = warp_sum(s);
  for (int j = lane; j < T; j += 32) d[j] = j < lim ? p[j] * (d[j] - s) * inv_scale : 0.f;
}
// dZ1[s,t,c] = dM[s,t,c] * 1[M[s,T-1,c] > 0]: inside a TransformerBlock every token's ff1.Backward uses
// the pre-activation of the LAST token (layer.go:563-567 via transformer.go:1238-1250).
__global__ void relu_mask_last_token_kernel(float* __restrict__ dM, const float* __restrict__ M, int T, int C, long total) {
  long per = (long)T * C;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    long s = i / per; int c = (int)(i % C);
    if (!(M[s * per + (long)(T - 1) * C + c] > 0.f)) dM[i] = 0.f;
  }
}

// ---------------------------------------------------------------- misc elementwise
// ---------------------------------------------------------------- TransformerBlock variants
// Rotary embeddings on a [tokens, D] tensor in place (transformer.go:212-236): within every head, element i of the first
// half and element i + hd/2 are rotated by the angle of (position, i); `tab` holds cos | sin per (position, i), computed on
// the host with the reference's float32 / float64 conversions.  sign = -1 applies the conjugate (backward pass).
__global__ void rope_kernel(float* __restrict__ x, const float* __restrict__ tab, long tokens, int T, int D, int hd, float sign) {
  const int half = hd >> 1; const long per = (long)(D >> 1), total = tokens * per;
  for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    const long tok = e / per; const int r = (int)(e - tok * per), h = r / half, i = r - h * half, t = (int)(tok % T);
    const float c = tab[((long)t * half + i) * 2], s = sign * tab[((long)t * half + i) * 2 + 1];
    float* p = x + tok * D + (long)h * hd + i;
    const float v1 = p[0], v2 = p[half];
    p[0] = v1 * c - v2 * s; p[half] = v1 * s + v2 * c;
  }
}
// rows [B, C] <- the last token's row of every sequence of in [B, T, C]
__global__ void last_token_rows_kernel(const float* __restrict__ in, float* __restrict__ out, int T, int C, long total) {
  for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) { const long s = e / C; out[e] = in[(s * T + (T - 1)) * C + (e - s * C)]; }
}
// dz[s,t,:] *= act'(z_last[s,:]): a Dense layer called token by token differentiates at its LAST call's pre-activation (layer.go:563-567)
__global__ void scale_by_last_deriv_kernel(float* __restrict__ dz, const float* __restrict__ z_last, int T, int C, long total, int act) {
  for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) { const long row = e / C; dz[e] *= act_der(act, z_last[(row / T) * C + (e - row * C)]); }
}
// SwiGLU (swiglu.go:163-170): out = swish(gate) * up
__global__ void swiglu_fwd_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ out, long n) {
  for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x) { const float g = gate[e]; out[e] = (g * act_fwd(GN_ACT_SIGMOID, g)) * up[e]; }
}
// SwiGLU backward inside a TransformerBlock (swiglu.go:203-216 with the pairing of transformer.go:1238-1250): the gradient of
// token t meets the saved state of token T-1-t.  Results are written at the PARTNER's row, where the weight-gradient
// contraction with the layer's inputs needs them.
__global__ void swiglu_bwd_paired_kernel(const float* __restrict__ dOut, const float* __restrict__ gate, const float* __restrict__ up,
                                         float* __restrict__ dGateP, float* __restrict__ dUpP, int T, int C, long total) {
  for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    const long row = e / C; const int c = (int)(e - row * C); const long s = row / T; const int t = (int)(row - s * T);
    const long pe = (s * T + (T - 1 - t)) * C + c;            // partner element
    const float g = gate[pe], u = up[pe], sig = act_fwd(GN_ACT_SIGMOID, g), sw = g * sig, go = dOut[e];
    dUpP[pe] = go * sw; dGateP[pe] = go * (sw + sig * (1.f - sw)) * u;
  }
}
// out[s,t,:] = a[s,t,:] + b[s,T-1-t,:]
__global__ void add_token_reversed_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int T, int C, long total) {
  for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    const long row = e / C; const int c = (int)(e - row * C); const long s = row / T; const int t = (int)(row - s * T);
    out[e] = a[e] + b[(s * T + (T - 1 - t)) * C + c];
  }
}

__global__ void add3_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ c, float* __restrict__ out, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) out[i] = a[i] + b[i] + (c ? c[i] : 0.f);
}
__global__ void scale_kernel(float* __restrict__ x, long n, float s) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) x[i] *= s;
}

// ---------------------------------------------------------------- Adam
// reference: opt.go:237-251.  Every operation is rounded separately (no fused multiply-add), as the Go
// code does, so that the update is bit-identical to the CPU path for identical gradients.
//   g' = g * grad_scale (the 1/batch averaging of net.go:702-706, folded into this pass)
//   m = b1*m + (1-b1)*g' ; v = b2*v + (1-b2)*g'*g' ; p -= effLR * m / (sqrt(v) + eps)
// `status` (may be null): the context's status word; when a bounded wait of an earlier kernel of this step gave up, the
// gradients are not trustworthy and the pass leaves the parameters and moments untouched.
__global__ void adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, long n,
                            float effLR, float b1, float b2, float omb1, float omb2, float eps, float grad_scale, const int* __restrict__ status) {
  if (status && *status != 0) return;
  // The four arrays are slices of the flat buffers at the same offset, so they share their position relative to a
  // 16-byte boundary: `head` leading elements are handled one by one, then float4s, then the tail.
  const long head = min(n, (long)((4 - ((reinterpret_cast<uintptr_t>(p) >> 2) & 3)) & 3));
  const long n4 = (n - head) >> 2;
  float4* p4 = reinterpret_cast<float4*>(p + head); const float4* g4 = reinterpret_cast<const float4*>(g + head);
  float4* m4 = reinterpret_cast<float4*>(m + head); float4* v4 = reinterpret_cast<float4*>(v + head);
  auto upd = [&](float& pp, float gg, float& mm, float& vv) {
    float gs = __fmul_rn(gg, grad_scale);
    mm = __fadd_rn(__fmul_rn(b1, mm), __fmul_rn(omb1, gs));
    vv = __fadd_rn(__fmul_rn(b2, vv), __fmul_rn(__fmul_rn(omb2, gs), gs));
    pp = __fsub_rn(pp, __fdiv_rn(__fmul_rn(effLR, mm), __fadd_rn(__fsqrt_rn(vv), eps)));
  };
  const long tid = blockIdx.x * (long)blockDim.x + threadIdx.x, nthreads = (long)gridDim.x * blockDim.x;
  for (long i = tid; i < n4; i += nthreads) {
    float4 P = p4[i], G = g4[i], M = m4[i], V = v4[i];
    upd(P.x, G.x, M.x, V.x); upd(P.y, G.y, M.y, V.y); upd(P.z, G.z, M.z, V.z); upd(P.w, G.w, M.w, V.w);
    p4[i] = P; m4[i] = M; v4[i] = V;
  }
  if (tid < head) upd(p[tid], g[tid], m[tid], v[tid]);
  for (long i = head + (n4 << 2) + tid; i < n; i += nthreads) upd(p[i], g[i], m[i], v[i]);
}


// ---------------------------------------------------------------- BatchNorm2D (NCHW)
// The reference normalises ONE sample at a time, so the statistics of a (sample, channel) pair are taken over that
// sample's S = H*W positions (batchnorm2d.go:336-377).  One block per (sample, channel).
// stat layout: [B*C] mean | [B*C] std | [B*C] variance.
__global__ void bn_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta, float* __restrict__ y,
                              float* __restrict__ stat, int C, int S, long BC, float eps) {
  __shared__ float red[33];
  const long bc = blockIdx.x; const int c = (int)(bc % C);
  const float* xp = x + bc * S; float* yp = y + bc * S;
  float s = 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) s += xp[i];
  const float mean = block_sum(s, red) * (1.f / (float)S);
  float ss = 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) { float d = xp[i] - mean; ss += d * d; }
  const float var = block_sum(ss, red) * (1.f / (float)S);
  const float sd = sqrtf(var + eps), istd = 1.f / sd, g = gamma[c], b = beta[c];
  for (int i = threadIdx.x; i < S; i += blockDim.x) yp[i] = g * ((xp[i] - mean) * istd) + b;
  if (threadIdx.x == 0) { stat[bc] = mean; stat[BC + bc] = sd; stat[2 * BC + bc] = var; }
}
// running = (1 - momentum) * running + momentum * statistic, once per sample in batch order (batchnorm2d.go:352, :376)
__global__ void bn_running_kernel(const float* __restrict__ stat, float* __restrict__ run, int B, int C, long BC, float mom) {
  int c = blockIdx.x * blockDim.x + threadIdx.x; if (c >= C) return;
  float rm = run[c], rv = run[C + c];
  for (int b = 0; b < B; b++) { rm = (1.f - mom) * rm + mom * stat[(long)b * C + c]; rv = (1.f - mom) * rv + mom * stat[2 * BC + (long)b * C + c]; }
  run[c] = rm; run[C + c] = rv;
}
// The same walk over per-sample statistics gathered from every rank (mean and variance as separate [B, C] arrays in
// global sample order), so that every replica applies the updates of the whole global batch in the reference's order.
__global__ void bn_running_gathered_kernel(const float* __restrict__ mean, const float* __restrict__ var, float* __restrict__ run, int B, int C, float mom) {
  int c = blockIdx.x * blockDim.x + threadIdx.x; if (c >= C) return;
  float rm = run[c], rv = run[C + c];
  for (int b = 0; b < B; b++) { rm = (1.f - mom) * rm + mom * mean[(long)b * C + c]; rv = (1.f - mom) * rv + mom * var[(long)b * C + c]; }
  run[c] = rm; run[C + c] = rv;
}
// inference mode: running statistics (batchnorm2d.go:492-509)
__global__ void bn_eval_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ run,
                               float* __restrict__ y, int C, int S, long total, float eps) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int c = (int)((i / S) % C);
    y[i] = gamma[c] * ((x[i] - run[c]) / sqrtf(run[C + c] + eps)) + beta[c];
  }
}
// reference: batchnorm2d.go:626-660, m = S.  pg: per (sample, channel) contributions [B, 2C] = gGamma | gBeta, summed over samples afterwards.
__global__ void bn_bwd_kernel(const float* __restrict__ g, const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ stat,
                              float* __restrict__ dx, float* __restrict__ pg, int C, int S, long BC) {
  __shared__ float red[33];
  const long bc = blockIdx.x; const int c = (int)(bc % C); const long b = bc / C;
  const float* xp = x + bc * S; const float* gp = g + bc * S; float* dp = dx + bc * S;
  const float mean = stat[bc], sd = stat[BC + bc], gm = gamma[c], m = (float)S;
  float sg = 0.f, sgx = 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) { float gg = gp[i]; sg += gg; sgx += gg * (xp[i] - mean); }
  sg = block_sum(sg, red); sgx = block_sum(sgx, red);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    float d = xp[i] - mean, gi = gp[i] * gm;
    dp[i] = gi / sd - (sg * gm) / m / sd - d * (sgx * gm) / m / (sd * sd * sd);
  }
  if (threadIdx.x == 0) { pg[b * 2 * C + c] = sgx / sd; pg[b * 2 * C + C + c] = sg; }     // sum g*(x-mean)/std ; sum g
}

}  // namespace gn
