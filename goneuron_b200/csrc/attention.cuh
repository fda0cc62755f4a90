// attention.cuh -- fused causal multi-head attention, forward and backward, without materialising the
// [T, T] score matrices in HBM.
//
// reference: internal/layer/transformer.go:470-503 (forward: scores = q.k / sqrt(hd), masked entries -1e9,
// row softmax, weighted sum of v) and :589-657 (backward: probabilities recomputed from q and k, explicit
// softmax Jacobian, dQ / dK / dV).  The Jacobian row term sum_k dP_k P_k equals dO . O (O = P V), which is
// what the backward kernels use; the row maximum and the row sum of the forward softmax are kept per row.
//
// Arithmetic: every product runs as 3xTF32 (hi*hi + hi*lo + lo*hi with fp32 accumulation) on warp-level
// tensor-core MMAs, the operands being split in registers, so accuracy is fp32-level.  One CTA = 64 query
// (or key) rows of one head, 4 warps x 16 rows, key (query) blocks of 64 streamed through shared memory;
// causal blocks above the diagonal are never visited.
//
// Q, K, V, O, dO and the outputs are [batch*T, D] row-major with head h in columns [h*HD, (h+1)*HD).
#pragma once
#include "common.cuh"

namespace gn {

constexpr int AT_BLK = 64, AT_THREADS = 128;

struct FragA { uint32_t hi[4], lo[4]; };
struct FragB { uint32_t hi[2], lo[2]; };

// hi = x with the 13 low mantissa bits cleared (exactly a TF32 value; a logic op, full rate -- the cvt.rna
// conversion runs on a slow pipe), lo = x - hi (exact; the MMA reads its leading 10 mantissa bits).
__device__ __forceinline__ void split32(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma8(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma3(float (&d)[4], const FragA& a, const FragB& b) { mma8(d, a.lo, b.hi); mma8(d, a.hi, b.lo); mma8(d, a.hi, b.hi); }

// A(r, k) = s[(row0 + r) * LD + k0 + k], 16 x 8.  Fragment order: (g,t) (g+8,t) (g,t+4) (g+8,t+4).
__device__ __forceinline__ void load_a(FragA& f, const float* s, int LD, int row0, int k0, int g, int t) {
  const float* p = s + (row0 + g) * LD + k0 + t;
  split32(p[0], f.hi[0], f.lo[0]); split32(p[8 * LD], f.hi[1], f.lo[1]); split32(p[4], f.hi[2], f.lo[2]); split32(p[8 * LD + 4], f.hi[3], f.lo[3]);
}
// B(k, n) = s[(n0 + n) * LD + k0 + k], 8 x 8: the contraction runs along the shared-memory row.
__device__ __forceinline__ void load_b_nk(FragB& f, const float* s, int LD, int n0, int k0, int g, int t) {
  const float* p = s + (n0 + g) * LD + k0 + t;
  split32(p[0], f.hi[0], f.lo[0]); split32(p[4], f.hi[1], f.lo[1]);
}
// B(k, n) = s[(k0 + k') * LD + n0 + n] with the contraction index permuted: MMA k-index t <-> row k0 + 2t,
// t + 4 <-> row k0 + 2t + 1.  This is the order in which an accumulator fragment holds its 8 columns
// (thread t owns columns 2t and 2t+1), so an accumulator can be fed back as the A operand without shuffles.
__device__ __forceinline__ void load_b_kn2(FragB& f, const float* s, int LD, int k0, int n0, int g, int t) {
  const float* p = s + (k0 + 2 * t) * LD + n0 + g;
  split32(p[0], f.hi[0], f.lo[0]); split32(p[LD], f.hi[1], f.lo[1]);
}
// accumulator fragment (rows g, g+8; columns 2t, 2t+1) as A operand in the permuted order above
__device__ __forceinline__ void acc_to_a(FragA& f, const float (&c)[4]) {
  split32(c[0], f.hi[0], f.lo[0]); split32(c[2], f.hi[1], f.lo[1]); split32(c[1], f.hi[2], f.lo[2]); split32(c[3], f.hi[3], f.lo[3]);
}
// 64 x HD tile of a [*, D] tensor into shared memory (row stride LD), rows >= T zero-filled
template <int HD>
__device__ __forceinline__ void load_tile(float* s, const float* src, long base, int row0, int T, int D) {
  constexpr int LD = HD + 4, V4 = HD / 4;
  for (int e = threadIdx.x; e < AT_BLK * V4; e += AT_THREADS) {
    int r = e / V4, c4 = e - r * V4, row = row0 + r;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < T) v = *reinterpret_cast<const float4*>(src + base + (long)row * D + c4 * 4);
    *reinterpret_cast<float4*>(s + r * LD + c4 * 4) = v;
  }
}
__device__ __forceinline__ float quad_max(float v) { v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1)); return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2)); }
__device__ __forceinline__ float quad_sum(float v) { v += __shfl_xor_sync(0xffffffffu, v, 1); return v + __shfl_xor_sync(0xffffffffu, v, 2); }

// ---------------------------------------------------------------- forward
template <int HD>
__global__ void __launch_bounds__(AT_THREADS) attn_fwd_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                                                               float* __restrict__ O, float* __restrict__ Mst, float* __restrict__ Lst,
                                                               int T, int D, int H, int causal, float inv_scale) {
  constexpr int LD = HD + 4, NT = HD / 8;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm; float* Ks = Qs + AT_BLK * LD; float* Vs = Ks + AT_BLK * LD;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z, q0 = qb * AT_BLK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const long base = (long)b * T * D + (long)h * HD;
  load_tile<HD>(Qs, Q, base, q0, T, D);
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  const int nkb = causal ? qb + 1 : (T + AT_BLK - 1) / AT_BLK;
  const int r0 = warp * 16, i0 = q0 + r0 + g, i1 = i0 + 8;
  for (int kb = 0; kb < nkb; kb++) {
    __syncthreads();
    load_tile<HD>(Ks, K, base, kb * AT_BLK, T, D);
    load_tile<HD>(Vs, V, base, kb * AT_BLK, T, D);
    __syncthreads();
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < NT; ks++) {
      FragA a; load_a(a, Qs, LD, r0, ks * 8, g, t);
#pragma unroll
      for (int n = 0; n < 8; n++) { FragB bf; load_b_nk(bf, Ks, LD, n * 8, ks * 8, g, t); mma3(s[n], a, bf); }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 8; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        int j = kb * AT_BLK + n * 8 + 2 * t + (e & 1), i = (e < 2) ? i0 : i1;
        float v = s[n][e] * inv_scale;
        if (j >= T || (causal && j > i)) v = -INFINITY;
        s[n][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    mx0 = quad_max(mx0); mx1 = quad_max(mx1);
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float c0 = __expf(m[0] - mn0), c1 = __expf(m[1] - mn1);
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int n = 0; n < 8; n++) {
      s[n][0] = __expf(s[n][0] - mn0); s[n][1] = __expf(s[n][1] - mn0); s[n][2] = __expf(s[n][2] - mn1); s[n][3] = __expf(s[n][3] - mn1);
      rs0 += s[n][0] + s[n][1]; rs1 += s[n][2] + s[n][3];
    }
    rs0 = quad_sum(rs0); rs1 = quad_sum(rs1);
    l[0] = l[0] * c0 + rs0; l[1] = l[1] * c1 + rs1; m[0] = mn0; m[1] = mn1;
#pragma unroll
    for (int d = 0; d < NT; d++) { o[d][0] *= c0; o[d][1] *= c0; o[d][2] *= c1; o[d][3] *= c1; }
#pragma unroll
    for (int kt = 0; kt < 8; kt++) {
      FragA a; acc_to_a(a, s[kt]);
#pragma unroll
      for (int d = 0; d < NT; d++) { FragB bf; load_b_kn2(bf, Vs, LD, kt * 8, d * 8, g, t); mma3(o[d], a, bf); }
    }
  }
  const float il0 = 1.f / l[0], il1 = 1.f / l[1];
#pragma unroll
  for (int d = 0; d < NT; d++) {
    if (i0 < T) *reinterpret_cast<float2*>(O + base + (long)i0 * D + d * 8 + 2 * t) = make_float2(o[d][0] * il0, o[d][1] * il0);
    if (i1 < T) *reinterpret_cast<float2*>(O + base + (long)i1 * D + d * 8 + 2 * t) = make_float2(o[d][2] * il1, o[d][3] * il1);
  }
  if (t == 0) {
    const long sb = ((long)b * H + h) * T;
    if (i0 < T) { Mst[sb + i0] = m[0]; Lst[sb + i0] = l[0]; }
    if (i1 < T) { Mst[sb + i1] = m[1]; Lst[sb + i1] = l[1]; }
  }
}

// Dv[b,h,i] = sum_d dO[b,i,h*HD+d] * O[b,i,h*HD+d]   (= sum_k dP_ik P_ik, the softmax-Jacobian row term)
__global__ void attn_rowdot_kernel(const float* __restrict__ dO, const float* __restrict__ O, float* __restrict__ Dv, int T, int D, int H, int HD, long rows) {
  long w = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); if (w >= rows) return;     // w = (b*T + i)*H + h
  int lane = threadIdx.x & 31; int h = (int)(w % H); long tok = w / H; int i = (int)(tok % T); long b = tok / T;
  const float* p = dO + tok * D + (long)h * HD; const float* q = O + tok * D + (long)h * HD;
  float s = 0.f;
  for (int d = lane; d < HD; d += 32) s = fmaf(p[d], q[d], s);
  s = warp_sum(s);
  if (lane == 0) Dv[(b * H + h) * T + i] = s;
}

// The same for head size 64 and D = 64 H (rows of all heads are then consecutive 64-float segments): 16 threads per row,
// 16-byte loads, two rows in flight per thread.
__global__ void __launch_bounds__(256) attn_rowdot64_kernel(const float* __restrict__ dO, const float* __restrict__ O, float* __restrict__ Dv, int T, int H, long rows) {
  const long gid = (long)blockIdx.x * 256 + threadIdx.x, half = (long)gridDim.x * 16;      // rows per pass of the grid
  const int l16 = threadIdx.x & 15;
  for (long w = gid >> 4; w < rows; w += 2 * half) {
    const long w2 = w + half;
    const float4 a = *reinterpret_cast<const float4*>(dO + w * 64 + l16 * 4), b = *reinterpret_cast<const float4*>(O + w * 64 + l16 * 4);
    float4 c = make_float4(0.f, 0.f, 0.f, 0.f), d = c;
    if (w2 < rows) { c = *reinterpret_cast<const float4*>(dO + w2 * 64 + l16 * 4); d = *reinterpret_cast<const float4*>(O + w2 * 64 + l16 * 4); }
    float s = (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w), s2 = (c.x * d.x + c.y * d.y) + (c.z * d.z + c.w * d.w);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) { s += __shfl_xor_sync(0xffffffffu, s, o); s2 += __shfl_xor_sync(0xffffffffu, s2, o); }
    if (l16 == 0) {
      { const int h = (int)(w % H); const long tok = w / H; Dv[((tok / T) * H + h) * T + tok % T] = s; }
      if (w2 < rows) { const int h = (int)(w2 % H); const long tok = w2 / H; Dv[((tok / T) * H + h) * T + tok % T] = s2; }
    }
  }
}


// ---------------------------------------------------------------- backward: dQ
// One CTA = 64 query rows; for every key block at or below the diagonal: S = Q K^T, P = exp(S/sqrt(hd) - m) / l,
// dP = dO V^T, dS = P (dP - Dv) / sqrt(hd), dQ += dS K.
template <int HD>
__global__ void __launch_bounds__(AT_THREADS) attn_bwd_dq_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                                                                  const float* __restrict__ dO, const float* __restrict__ Mst, const float* __restrict__ Lst,
                                                                  const float* __restrict__ Dv, float* __restrict__ dQ, int T, int D, int H, int causal, float inv_scale) {
  constexpr int LD = HD + 4, NT = HD / 8;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm; float* Gs = Qs + AT_BLK * LD; float* Ks = Gs + AT_BLK * LD; float* Vs = Ks + AT_BLK * LD;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z, q0 = qb * AT_BLK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const long base = (long)b * T * D + (long)h * HD, sb = ((long)b * H + h) * T;
  load_tile<HD>(Qs, Q, base, q0, T, D);
  load_tile<HD>(Gs, dO, base, q0, T, D);
  const int r0 = warp * 16, i0 = q0 + r0 + g, i1 = i0 + 8;
  const float m0 = i0 < T ? Mst[sb + i0] : 0.f, m1 = i1 < T ? Mst[sb + i1] : 0.f;
  const float il0 = i0 < T ? 1.f / Lst[sb + i0] : 0.f, il1 = i1 < T ? 1.f / Lst[sb + i1] : 0.f;
  const float d0 = i0 < T ? Dv[sb + i0] : 0.f, d1 = i1 < T ? Dv[sb + i1] : 0.f;
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
  const int nkb = causal ? qb + 1 : (T + AT_BLK - 1) / AT_BLK;
  for (int kb = 0; kb < nkb; kb++) {
    __syncthreads();
    load_tile<HD>(Ks, K, base, kb * AT_BLK, T, D);
    load_tile<HD>(Vs, V, base, kb * AT_BLK, T, D);
    __syncthreads();
    float s[8][4], dp[8][4];
#pragma unroll
    for (int n = 0; n < 8; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < NT; ks++) {
      FragA a, ga; load_a(a, Qs, LD, r0, ks * 8, g, t); load_a(ga, Gs, LD, r0, ks * 8, g, t);
#pragma unroll
      for (int n = 0; n < 8; n++) {
        FragB bf; load_b_nk(bf, Ks, LD, n * 8, ks * 8, g, t); mma3(s[n], a, bf);
        load_b_nk(bf, Vs, LD, n * 8, ks * 8, g, t); mma3(dp[n], ga, bf);
      }
    }
#pragma unroll
    for (int n = 0; n < 8; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int j = kb * AT_BLK + n * 8 + 2 * t + (e & 1), i = (e < 2) ? i0 : i1;
        const bool masked = j >= T || i >= T || (causal && j > i);
        const float p = masked ? 0.f : __expf(s[n][e] * inv_scale - (e < 2 ? m0 : m1)) * (e < 2 ? il0 : il1);
        s[n][e] = p * (dp[n][e] - (e < 2 ? d0 : d1)) * inv_scale;        // dS
      }
#pragma unroll
    for (int kt = 0; kt < 8; kt++) {
      FragA a; acc_to_a(a, s[kt]);
#pragma unroll
      for (int d = 0; d < NT; d++) { FragB bf; load_b_kn2(bf, Ks, LD, kt * 8, d * 8, g, t); mma3(acc[d], a, bf); }
    }
  }
#pragma unroll
  for (int d = 0; d < NT; d++) {
    if (i0 < T) *reinterpret_cast<float2*>(dQ + base + (long)i0 * D + d * 8 + 2 * t) = make_float2(acc[d][0], acc[d][1]);
    if (i1 < T) *reinterpret_cast<float2*>(dQ + base + (long)i1 * D + d * 8 + 2 * t) = make_float2(acc[d][2], acc[d][3]);
  }
}

// ---------------------------------------------------------------- backward: dK, dV
// One CTA = 64 key rows; for every query block at or above the diagonal the TRANSPOSED tiles are formed directly:
// S^T = K Q^T, P^T, dP^T = V dO^T, dS^T = P^T (dP^T - Dv[query]) / sqrt(hd); dK += dS^T Q, dV += P^T dO.
template <int HD>
__global__ void __launch_bounds__(AT_THREADS) attn_bwd_dkv_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                                                                   const float* __restrict__ dO, const float* __restrict__ Mst, const float* __restrict__ Lst,
                                                                   const float* __restrict__ Dv, float* __restrict__ dK, float* __restrict__ dV,
                                                                   int T, int D, int H, int causal, float inv_scale) {
  constexpr int LD = HD + 4, NT = HD / 8;
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm; float* Vs = Ks + AT_BLK * LD; float* Qs = Vs + AT_BLK * LD; float* Gs = Qs + AT_BLK * LD;
  float* st_m = Gs + AT_BLK * LD; float* st_il = st_m + AT_BLK; float* st_d = st_il + AT_BLK;
  const int kbk = blockIdx.x, h = blockIdx.y, b = blockIdx.z, k0 = kbk * AT_BLK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const long base = (long)b * T * D + (long)h * HD, sb = ((long)b * H + h) * T;
  load_tile<HD>(Ks, K, base, k0, T, D);
  load_tile<HD>(Vs, V, base, k0, T, D);
  const int r0 = warp * 16, j0 = k0 + r0 + g, j1 = j0 + 8;
  float ak[NT][4], av[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++) { ak[i][0] = ak[i][1] = ak[i][2] = ak[i][3] = 0.f; av[i][0] = av[i][1] = av[i][2] = av[i][3] = 0.f; }
  const int nqb = (T + AT_BLK - 1) / AT_BLK;
  for (int qb = causal ? kbk : 0; qb < nqb; qb++) {
    __syncthreads();
    load_tile<HD>(Qs, Q, base, qb * AT_BLK, T, D);
    load_tile<HD>(Gs, dO, base, qb * AT_BLK, T, D);
    if (threadIdx.x < AT_BLK) {
      const int i = qb * AT_BLK + threadIdx.x;
      st_m[threadIdx.x] = i < T ? Mst[sb + i] : 0.f; st_il[threadIdx.x] = i < T ? 1.f / Lst[sb + i] : 0.f; st_d[threadIdx.x] = i < T ? Dv[sb + i] : 0.f;
    }
    __syncthreads();
    float s[8][4], dp[8][4];
#pragma unroll
    for (int n = 0; n < 8; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < NT; ks++) {
      FragA a, va; load_a(a, Ks, LD, r0, ks * 8, g, t); load_a(va, Vs, LD, r0, ks * 8, g, t);
#pragma unroll
      for (int n = 0; n < 8; n++) {
        FragB bf; load_b_nk(bf, Qs, LD, n * 8, ks * 8, g, t); mma3(s[n], a, bf);
        load_b_nk(bf, Gs, LD, n * 8, ks * 8, g, t); mma3(dp[n], va, bf);
      }
    }
    // rows = keys j (g, g+8), columns = queries i (2t, 2t+1 of n-tile n)
#pragma unroll
    for (int n = 0; n < 8; n++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int ci = n * 8 + 2 * t + (e & 1), i = qb * AT_BLK + ci, j = (e < 2) ? j0 : j1;
        const bool masked = j >= T || i >= T || (causal && j > i);
        const float p = masked ? 0.f : __expf(s[n][e] * inv_scale - st_m[ci]) * st_il[ci];
        dp[n][e] = p * (dp[n][e] - st_d[ci]) * inv_scale;                 // dS^T
        s[n][e] = p;                                                     // P^T
      }
#pragma unroll
    for (int kt = 0; kt < 8; kt++) {
      FragA ap, ads; acc_to_a(ap, s[kt]); acc_to_a(ads, dp[kt]);
#pragma unroll
      for (int d = 0; d < NT; d++) {
        FragB bf; load_b_kn2(bf, Qs, LD, kt * 8, d * 8, g, t); mma3(ak[d], ads, bf);
        load_b_kn2(bf, Gs, LD, kt * 8, d * 8, g, t); mma3(av[d], ap, bf);
      }
    }
  }
#pragma unroll
  for (int d = 0; d < NT; d++) {
    if (j0 < T) { *reinterpret_cast<float2*>(dK + base + (long)j0 * D + d * 8 + 2 * t) = make_float2(ak[d][0], ak[d][1]);
                  *reinterpret_cast<float2*>(dV + base + (long)j0 * D + d * 8 + 2 * t) = make_float2(av[d][0], av[d][1]); }
    if (j1 < T) { *reinterpret_cast<float2*>(dK + base + (long)j1 * D + d * 8 + 2 * t) = make_float2(ak[d][2], ak[d][3]);
                  *reinterpret_cast<float2*>(dV + base + (long)j1 * D + d * 8 + 2 * t) = make_float2(av[d][2], av[d][3]); }
  }
}

// ---------------------------------------------------------------- launchers
inline bool attn_fused_supported(int hd, int D) { return (hd == 16 || hd == 32 || hd == 64) && D % 4 == 0; }

template <int HD>
inline int attn_fwd_launch(Ctx* ctx, const float* Q, const float* K, const float* V, float* O, float* M, float* L, int B, int T, int D, int H, int causal) {
  size_t smem = (size_t)3 * AT_BLK * (HD + 4) * sizeof(float);
  GN_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  GN_LAUNCH(ctx, attn_fwd_kernel<HD>, dim3(cdiv(T, AT_BLK), H, B), AT_THREADS, smem, Q, K, V, O, M, L, T, D, H, causal, 1.f / sqrtf((float)HD));
  return check_launch("attn_fwd");
}
template <int HD>
inline int attn_bwd_launch(Ctx* ctx, const float* Q, const float* K, const float* V, const float* O, const float* dO, const float* M, const float* L, float* Dv,
                           float* dQ, float* dK, float* dV, int B, int T, int D, int H, int causal) {
  const float inv_scale = 1.f / sqrtf((float)HD);
  long rows = (long)B * T * H;
  GN_LAUNCH(ctx, attn_rowdot_kernel, cdiv(rows, 8), 256, 0, dO, O, Dv, T, D, H, HD, rows);
  size_t smem_q = (size_t)4 * AT_BLK * (HD + 4) * sizeof(float), smem_kv = smem_q + 3 * AT_BLK * sizeof(float);
  GN_CUDA(cudaFuncSetAttribute(attn_bwd_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q));
  GN_CUDA(cudaFuncSetAttribute(attn_bwd_dkv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
  dim3 grid(cdiv(T, AT_BLK), H, B);
  GN_LAUNCH(ctx, attn_bwd_dq_kernel<HD>, grid, AT_THREADS, smem_q, Q, K, V, dO, M, L, Dv, dQ, T, D, H, causal, inv_scale);
  GN_LAUNCH(ctx, attn_bwd_dkv_kernel<HD>, grid, AT_THREADS, smem_kv, Q, K, V, dO, M, L, Dv, dK, dV, T, D, H, causal, inv_scale);
  return check_launch("attn_bwd");
}
inline int attn_fwd(Ctx* ctx, int hd, const float* Q, const float* K, const float* V, float* O, float* M, float* L, int B, int T, int D, int H, int causal) {
  if (hd == 64) return attn_fwd_launch<64>(ctx, Q, K, V, O, M, L, B, T, D, H, causal);
  if (hd == 32) return attn_fwd_launch<32>(ctx, Q, K, V, O, M, L, B, T, D, H, causal);
  return attn_fwd_launch<16>(ctx, Q, K, V, O, M, L, B, T, D, H, causal);
}
inline int attn_bwd(Ctx* ctx, int hd, const float* Q, const float* K, const float* V, const float* O, const float* dO, const float* M, const float* L, float* Dv,
                    float* dQ, float* dK, float* dV, int B, int T, int D, int H, int causal) {
  if (hd == 64) return attn_bwd_launch<64>(ctx, Q, K, V, O, dO, M, L, Dv, dQ, dK, dV, B, T, D, H, causal);
  if (hd == 32) return attn_bwd_launch<32>(ctx, Q, K, V, O, dO, M, L, Dv, dQ, dK, dV, B, T, D, H, causal);
  return attn_bwd_launch<16>(ctx, Q, K, V, O, dO, M, L, Dv, dQ, dK, dV, B, T, D, H, causal);
}

}  // namespace gn
