// gemm_tc.cuh -- fp32-accurate contraction on the 5th-generation tensor cores (sm_100a).
//
//   C[M,N] = act( A[M,K] * B[N,K]^T + bias[N] + R[M,N] )
//
// Split-operand scheme.  Every fp32 operand x is written as hi = tf32(x) and lo = x - hi (exact in fp32), and
//     a*b  =  hi_a*hi_b  +  lo_a*b  +  a*lo_b      (the dropped lo*lo term is ~2^-22 relative).
// The large term runs as one TF32 MMA (both factors are exact TF32 values, fp32 accumulation).  The two cross
// terms are about 2^-11 of the product, so their factors only need a few bits: they run as BF16 MMAs on
// lo (rounded to bf16) and on a bf16 copy of the other operand, which contributes a relative error of about
// 2^-8 * 2^-11 = 2^-19 per product -- the size of the fp32 rounding noise of a long sum -- at half the tensor
// time of a TF32 MMA.  Per 32 contraction indices that is 4 TF32 + 4 BF16 instructions of the same size
// instead of the 12 TF32 instructions of the plain 3xTF32 scheme (which this file used first; measured
// 228-238 TFLOP/s fp32-equivalent, i.e. at the ceiling of one sixth of the bf16 rate).
// The operand planes (hi as fp32, the bf16 copy, lo as bf16: 8 bytes per element) are written by a
// memory-bound pass (split_rows_kernel / split_cols_kernel), K-major, so the contraction kernel itself is a
// pure TMA -> shared memory -> tcgen05.mma pipeline:
//
//   warp 0   TMA producer: 6 tiled bulk copies per stage (hi: 128-byte swizzle; bf16 planes: 64-byte
//            swizzle; 3-D maps, third coordinate = problem index of a batch)
//   warp 1   allocates TMEM, issues tcgen05.mma.kind::tf32 / kind::f16 (one elected lane), commits to mbarriers
//   warps 2-5  epilogue: tcgen05.ld of the accumulators, bias / residual / ReLU / gate, one output row
//              per thread with 16-byte stores
//
// Persistent: one CTA per SM walks 128 x BN output tiles (BN = 128, or 64 for narrow outputs), 3 stages of
// 64 KB, and TMEM holds two accumulator slots so the epilogue of tile i runs under the mainloop of tile i+1.
// Each slot has two accumulators: the hi*hi products go to one, the small cross terms to the other, and the
// epilogue adds them.  The tensor core truncates when it aligns a product sum to the running accumulator, an
// error proportional to the accumulator's magnitude per MMA; keeping the cross terms out of the large
// accumulator keeps the number of such truncations on it at one per 8 contraction indices.
// Every mbarrier wait is bounded; a wait that gives up sets the context's status word and the kernel
// still runs to its end (TMEM is always released).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdlib>
#include "common.cuh"
#include "gemm_simt.cuh"

namespace gn {

constexpr int TC_BM = 128, TC_THREADS = 192;
constexpr unsigned TC_SPIN_LIMIT = 1u << 24;
constexpr int TC_KSLICE = 4096;     // longest accumulator run, see gemm_tc()
constexpr int TC_FLAG_VEC = 4096;   // epilogue may use 16-byte accesses (set by the host when every pointer and stride allows it)
// One stage = 32 contraction indices of both operands: hi plane (fp32, 128-byte rows) + bf16 copy + bf16 lo (64-byte rows).
constexpr int TC_BK = 32;
template <int BN> struct TcCfg {
  static constexpr int A_HI = TC_BM * TC_BK * 4, A_BF = TC_BM * TC_BK * 2;       // 16 KB, 8 KB
  static constexpr int B_HI = BN * TC_BK * 4, B_BF = BN * TC_BK * 2;
  static constexpr int A_BYTES = A_HI + 2 * A_BF, B_BYTES = B_HI + 2 * B_BF;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (200 * 1024) / STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
  static_assert(2 * STAGES + 5 <= 32, "barrier area");
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: returns false when it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned it = 0; it < TC_SPIN_LIMIT; it++) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are 128 bytes apart, groups of 8
// rows 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100), layout type 2 = SWIZZLE_128B.
// With 64-byte rows (make_desc<16>: 16 fp32 or 32 bf16 per row): groups of 8 rows are 512 bytes apart and the layout
// type is 4 = SWIZZLE_64B.
template <int BK>
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  constexpr uint64_t sbo = (8 * BK * 4) >> 4, layout = BK == 32 ? 2 : 4;
  return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | (sbo << 32) | (1ull << 46) | (layout << 61);
}
// Instruction descriptor: D = f32 (bits 4-5 = 1), A = B = tf32 (bits 7-9, 10-12 = 2), both K-major,
// N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// The same for kind::f16 with A = B = bf16 (format code 1), D = f32.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ float tf32_round(float x) { uint32_t u; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x)); return __uint_as_float(u); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

// Output side of one launch.  Batched problems: problem z = blockIdx.z -> (z / batch2, z % batch2) selects the
// output (and residual) sub-matrix; the operand planes of problem z are slice z of the 3-D tensor maps.
struct TcParams {
  float* C; long ldc, c_b1, c_b2; const float* bias; const float* R; long ldr, r_b1, r_b2;
  int act, M, N, K, batch2, flags; int* status;
  const float* mask; long mask_ld; int mask_group;    // optional gate, see GemmDesc::mask
};

// Epilogue of one output tile, executed by one warp for its TMEM lane quadrant: one output row per thread
// (TMEM lane = row), 32 consecutive columns per tcgen05.ld, written as 8 float4.  Bias, residual and gate values
// of a chunk are fetched before the TMEM wait so that their latency overlaps.  `acc_main` / `acc_cross` are the
// TMEM column offsets of the two accumulators of this tile.
template <int BN>
__device__ __forceinline__ void tc_epilogue_tile(const TcParams& ep, uint32_t tmem_base, uint32_t acc_main, uint32_t acc_cross,
                                                 int m0, int n0, int z, int quad, int lane, int nkb) {
    const int z1 = z / ep.batch2, z2 = z % ep.batch2;
    float* C = ep.C + z1 * ep.c_b1 + z2 * ep.c_b2;
    const float* R = ep.R ? ep.R + z1 * ep.r_b1 + z2 * ep.r_b2 : nullptr;
    const int row = m0 + quad * 32 + lane;
    const bool row_ok = row < ep.M;
    const float* Rrow = (R && row_ok) ? R + (long)row * ep.ldr : nullptr;
    const float* Mrow = (ep.mask && row_ok) ? ep.mask + (long)(row / ep.mask_group) * ep.mask_ld : nullptr;
    float* Crow = C + (long)row * ep.ldc;
    const bool vec = (ep.flags & TC_FLAG_VEC) != 0;
    for (int c = 0; c < BN / 32; c++) {
      const int col0 = n0 + c * 32;
      if (col0 >= ep.N) break;
      uint32_t r[32], q[32];
      if (nkb > 0) {
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32);
        tmem_ld32(taddr + acc_main, r);
        tmem_ld32(taddr + acc_cross, q);
      }
      if (vec) {
        float4 rv[8], mv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const bool in = col0 + 4 * j < ep.N;
          rv[j] = (Rrow && in) ? *reinterpret_cast<const float4*>(Rrow + col0 + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
          mv[j] = (Mrow && in) ? *reinterpret_cast<const float4*>(Mrow + col0 + 4 * j) : make_float4(1.f, 1.f, 1.f, 1.f);
        }
        if (nkb > 0) asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 8; j++) {
          if (!row_ok || col0 + 4 * j >= ep.N) continue;
          float4 bv = ep.bias ? __ldg(reinterpret_cast<const float4*>(ep.bias + col0 + 4 * j)) : make_float4(0.f, 0.f, 0.f, 0.f);
          float4 v;
          v.x = (nkb > 0 ? __uint_as_float(r[4 * j]) + __uint_as_float(q[4 * j]) : 0.f) + bv.x + rv[j].x;
          v.y = (nkb > 0 ? __uint_as_float(r[4 * j + 1]) + __uint_as_float(q[4 * j + 1]) : 0.f) + bv.y + rv[j].y;
          v.z = (nkb > 0 ? __uint_as_float(r[4 * j + 2]) + __uint_as_float(q[4 * j + 2]) : 0.f) + bv.z + rv[j].z;
          v.w = (nkb > 0 ? __uint_as_float(r[4 * j + 3]) + __uint_as_float(q[4 * j + 3]) : 0.f) + bv.w + rv[j].w;
          if (ep.act == GN_ACT_RELU) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
          if (!(mv[j].x > 0.f)) v.x = 0.f; if (!(mv[j].y > 0.f)) v.y = 0.f; if (!(mv[j].z > 0.f)) v.z = 0.f; if (!(mv[j].w > 0.f)) v.w = 0.f;
          *reinterpret_cast<float4*>(Crow + col0 + 4 * j) = v;
        }
      } else {
        if (nkb > 0) asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; j++) {
          const int col = col0 + j;
          if (!row_ok || col >= ep.N) continue;
          float v = nkb > 0 ? __uint_as_float(r[j]) + __uint_as_float(q[j]) : 0.f;
          if (ep.bias) v += ep.bias[col];
          if (Rrow) v += Rrow[col];
          if (ep.act == GN_ACT_RELU) v = fmaxf(v, 0.f);
          if (Mrow && !(Mrow[col] > 0.f)) v = 0.f;
          Crow[col] = v;
        }
      }
    }
  }

__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

template <int BN, int NSLOTS>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persist_kernel(const __grid_constant__ CUtensorMap mapAhi, const __grid_constant__ CUtensorMap mapAxb, const __grid_constant__ CUtensorMap mapAlo,
                       const __grid_constant__ CUtensorMap mapBhi, const __grid_constant__ CUtensorMap mapBxb, const __grid_constant__ CUtensorMap mapBlo,
                       TcParams ep, int tiles_m, int tiles_n, int total_tiles) {
  using Cfg = TcCfg<BN>;
  static_assert(NSLOTS * 2 * BN <= 512 && (NSLOTS == 1 || NSLOTS == 2), "accumulator slots must fit the 512 TMEM columns");
  constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES, BK = TC_BK;
  constexpr uint32_t TMEM_COLS = NSLOTS * 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);       // full[S], empty[S], tfull[2], tempty[2]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // stage layout: A_hi | A_xb | A_lo | B_hi | B_xb | B_lo
  constexpr uint32_t OFF_AXB = Cfg::A_HI, OFF_ALO = Cfg::A_HI + Cfg::A_BF, OFF_BHI = Cfg::A_BYTES, OFF_BXB = OFF_BHI + Cfg::B_HI, OFF_BLO = OFF_BXB + Cfg::B_BF;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> coordinates and contraction range (identical in every role)
  auto decode = [&](int tile, int& m0, int& n0, int& z, int& kb0, int& nkb) -> bool {
    const int nt = tile % tiles_n, q = tile / tiles_n, mt = q % tiles_m; z = q / tiles_m;
    m0 = mt * TC_BM; n0 = nt * BN;
    if ((ep.flags & GEMM_SKIP_UPPER) && n0 > m0 + TC_BM - 1) return false;
    int kbeg = 0, kend = ep.K;
    if (ep.flags & GEMM_KBEG_AT_M0) kbeg = (m0 / BK) * BK;
    if (ep.flags & GEMM_KEND_AT_M0) kend = min(ep.K, m0 + TC_BM);
    kb0 = kbeg / BK; nkb = (kend - kbeg + BK - 1) / BK;
    return true;
  };

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true; uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int m0, n0, z, kb0, nkb; if (!decode(tile, m0, n0, z, kb0, nkb)) continue;
        for (int i = 0; i < nkb; i++, it++) {
          const uint32_t s = it % STAGES, use = it / STAGES; const int kc = (kb0 + i) * BK;
          if (use > 0) ok &= mbar_wait(empty0 + 8 * s, (use - 1) & 1);
          const uint32_t base = smem_u32(smem + s * STAGE_BYTES), bar = full0 + 8 * s;
          mbar_expect_tx(bar, STAGE_BYTES);
          tma_load_3d(base, &mapAhi, kc, m0, z, bar);
          tma_load_3d(base + OFF_AXB, &mapAxb, kc, m0, z, bar);
          tma_load_3d(base + OFF_ALO, &mapAlo, kc, m0, z, bar);
          tma_load_3d(base + OFF_BHI, &mapBhi, kc, n0, z, bar);
          tma_load_3d(base + OFF_BXB, &mapBxb, kc, n0, z, bar);
          tma_load_3d(base + OFF_BLO, &mapBlo, kc, n0, z, bar);
        }
      }
      if (!ok) atomicExch(ep.status, 1);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true; uint32_t it = 0, lt = 0;
      constexpr uint32_t idesc = make_idesc(TC_BM, BN), idesc_bf = make_idesc_bf16(TC_BM, BN);
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int m0, n0, z, kb0, nkb; if (!decode(tile, m0, n0, z, kb0, nkb)) continue;
        const uint32_t slot = NSLOTS == 2 ? (lt & 1) : 0, u = NSLOTS == 2 ? (lt >> 1) : lt; lt++;
        ok &= mbar_wait(tempty0 + 8 * slot, (u & 1) ^ 1);          // slot drained by the epilogue (passes at once the first time)
        tc_fence_after();
        const uint32_t acc_main = tmem_base + slot * 2 * BN, acc_cross = acc_main + BN;
        for (int i = 0; i < nkb; i++, it++) {
          const uint32_t s = it % STAGES, use = it / STAGES;
          ok &= mbar_wait(full0 + 8 * s, use & 1);
          tc_fence_after();
          const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t ahi = make_desc<32>(base), axb = make_desc<16>(base + OFF_AXB), alo = make_desc<16>(base + OFF_ALO);
          const uint64_t bhi = make_desc<32>(base + OFF_BHI), bxb = make_desc<16>(base + OFF_BXB), blo = make_desc<16>(base + OFF_BLO);
#pragma unroll
          for (int k = 0; k < 2; k++) {                      // bf16: 16 contraction indices = 32 bytes per instruction
            const uint64_t adv = (uint64_t)(2 * k);
            tc_mma_bf16(acc_cross, alo + adv, bxb + adv, idesc_bf, (i > 0 || k > 0) ? 1u : 0u);
            tc_mma_bf16(acc_cross, axb + adv, blo + adv, idesc_bf, 1u);
          }
#pragma unroll
          for (int k = 0; k < 4; k++) {                      // tf32: 8 contraction indices = 32 bytes per instruction
            const uint64_t adv = (uint64_t)(2 * k);
            tc_mma_tf32(acc_main, ahi + adv, bhi + adv, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(empty0 + 8 * s);
        }
        tc_commit(tfull0 + 8 * slot);
      }
      if (!ok) atomicExch(ep.status, 2);
    }
  } else {
    const int quad = warp & 3; uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      int m0, n0, z, kb0, nkb; if (!decode(tile, m0, n0, z, kb0, nkb)) continue;
      const uint32_t slot = NSLOTS == 2 ? (lt & 1) : 0, u = NSLOTS == 2 ? (lt >> 1) : lt; lt++;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(tfull0 + 8 * slot, u & 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok && lane == 0) atomicExch(ep.status, 3);
      tc_fence_after();
      tc_epilogue_tile<BN>(ep, tmem_base, slot * 2 * BN, slot * 2 * BN + BN, m0, n0, z, quad, lane, nkb);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * slot);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

// ------------------------------------------------------------------ operand split (memory-bound)
// Batched, strided split: planes[z][r][c] (row stride ldp, c < ldp, zero beyond cols) of the source element
// (z, r, c) at p + (z / batch2) * b1 + (z % batch2) * b2 + r * s_r + c * s_c.  One of s_r, s_c is 1:
// s_c == 1 reads rows directly; s_r == 1 (the operand is the transpose of what is stored) goes through a shared tile.
// Three planes per operand: hi = tf32(x) as fp32, xb = bf16(x), lo = bf16(x - hi).
struct TcSrc { const float* p; long s_r, s_c, b1, b2; int batch2; };
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&v);
}
__global__ void __launch_bounds__(256) split_rows_kernel(TcSrc s, int rows, int cols, float* __restrict__ hi, __nv_bfloat16* __restrict__ xb,
                                                         __nv_bfloat16* __restrict__ lo, int ldp) {
  // four float4 per thread, all loads issued before the first store; blockIdx.y = problem index
  const int z = blockIdx.y, ldp4 = ldp >> 2, total = rows * ldp4;
  const float* base = s.p + (z / s.batch2) * s.b1 + (z % s.batch2) * s.b2;
  const int idx0 = blockIdx.x * 1024 + threadIdx.x;
  float4 x[4]; long o[4];
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int idx = idx0 + 256 * k;
    o[k] = -1;
    if (idx >= total) continue;
    const int r = idx / ldp4, c = (idx - r * ldp4) << 2;
    const float* src = base + (long)r * s.s_r + c;
    if (c + 3 < cols && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) x[k] = *reinterpret_cast<const float4*>(src);
    else { x[k].x = c < cols ? src[0] : 0.f; x[k].y = c + 1 < cols ? src[1] : 0.f; x[k].z = c + 2 < cols ? src[2] : 0.f; x[k].w = c + 3 < cols ? src[3] : 0.f; }
    o[k] = ((long)z * rows + r) * ldp + c;
  }
#pragma unroll
  for (int k = 0; k < 4; k++) {
    if (o[k] < 0) continue;
    const float4 h = make_float4(tf32_round(x[k].x), tf32_round(x[k].y), tf32_round(x[k].z), tf32_round(x[k].w));
    *reinterpret_cast<float4*>(hi + o[k]) = h;
    *reinterpret_cast<uint2*>(xb + o[k]) = make_uint2(pack_bf16(x[k].x, x[k].y), pack_bf16(x[k].z, x[k].w));
    *reinterpret_cast<uint2*>(lo + o[k]) = make_uint2(pack_bf16(x[k].x - h.x, x[k].y - h.y), pack_bf16(x[k].z - h.z, x[k].w - h.w));
  }
}
__global__ void split_cols_kernel(TcSrc s, int rows, int cols, float* __restrict__ hi, __nv_bfloat16* __restrict__ xb, __nv_bfloat16* __restrict__ lo, int ldp) {
  __shared__ float t[32][33];
  const int z = blockIdx.z, c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const float* src = s.p + (z / s.batch2) * s.b1 + (z % s.batch2) * s.b2;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) { int c = c0 + j, r = r0 + threadIdx.x; t[j][threadIdx.x] = (r < rows && c < cols) ? src[r + c * s.s_c] : 0.f; }
  __syncthreads();
  const long zo = (long)z * rows * ldp;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < ldp) {
      const float x = t[threadIdx.x][j], h = tf32_round(x); const long o = zo + (long)r * ldp + c;
      hi[o] = h; xb[o] = __float2bfloat16_rn(x); lo[o] = __float2bfloat16_rn(x - h);
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Operand planes, [nbatch][rows][ldp] each, K valid columns starting at column koff (a slice of a longer contraction):
// `hi` fp32; `lo` is a buffer of the same size holding the two bf16 planes one after the other (bf16 copy, then lo).
// The attention kernels use the same struct for their own fp32 hi / fp32 lo planes (tc_make_map on either pointer).
struct TcPlanes {
  float* hi; float* lo; int rows, K, ldp, nbatch; int koff = 0;
  __nv_bfloat16* xb() const { return reinterpret_cast<__nv_bfloat16*>(lo); }
  __nv_bfloat16* lob() const { return xb() + (size_t)nbatch * rows * ldp; }
};
inline int tc_ldp(int K) { return ((K + 7) / 8) * 8; }              // plane row stride: a multiple of 16 bytes for TMA in bf16 too

struct TcScratch { DevBuf a_hi, a_lo, b_hi, b_lo; const float* last_a = nullptr; int last_m = 0, last_k = 0; long last_ld = 0; };
inline TcScratch& tc_scratch(Ctx* ctx) { static thread_local std::vector<std::pair<Ctx*, TcScratch*>> tab; for (auto& e : tab) if (e.first == ctx) return *e.second; tab.push_back({ctx, ctx->own(new TcScratch())}); return *tab.back().second; }

inline void tc_init(Ctx* ctx) {
  ctx->tc_ok = false;
  void* fn = nullptr; cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess) { cudaGetLastError(); return; }
  bool ok = true;
  ok &= cudaFuncSetAttribute(gemm_tc_persist_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<128>::SMEM_BYTES) == cudaSuccess;
  ok &= cudaFuncSetAttribute(gemm_tc_persist_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<64>::SMEM_BYTES) == cudaSuccess;
  if (!ok) { cudaGetLastError(); return; }
  ctx->encode_tiled = fn; ctx->tc_ok = true;
}

// fp32 plane, 32 columns (128 bytes, 128-byte swizzle) x box_rows per copy
inline int tc_make_map(Ctx* ctx, CUtensorMap* map, const TcPlanes& p, const float* base, int box_rows, int bk = 32) {
  cuuint64_t dims[3] = {(cuuint64_t)p.K, (cuuint64_t)p.rows, (cuuint64_t)p.nbatch};
  cuuint64_t strides[2] = {(cuuint64_t)p.ldp * 4, (cuuint64_t)p.rows * p.ldp * 4};
  cuuint32_t box[3] = {(cuuint32_t)bk, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = ((PFN_encodeTiled)ctx->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)(base + p.koff), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                    bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GN_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (rows %d K %d ld %d batch %d)", (int)r, p.rows, p.K, p.ldp, p.nbatch);
  return GN_OK;
}
// bf16 plane, box_cols columns x box_rows per copy: 32 columns = 64 bytes with the 64-byte swizzle (contraction engine),
// 64 columns = 128 bytes with the 128-byte swizzle (attention tiles)
inline int tc_make_map_bf16(Ctx* ctx, CUtensorMap* map, const TcPlanes& p, const __nv_bfloat16* base, int box_rows, int box_cols = TC_BK) {
  cuuint64_t dims[3] = {(cuuint64_t)p.K, (cuuint64_t)p.rows, (cuuint64_t)p.nbatch};
  cuuint64_t strides[2] = {(cuuint64_t)p.ldp * 2, (cuuint64_t)p.rows * p.ldp * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = ((PFN_encodeTiled)ctx->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)(base + p.koff), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                    box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GN_ERR_CUDA, "cuTensorMapEncodeTiled (bf16) failed with %d (rows %d K %d ld %d batch %d)", (int)r, p.rows, p.K, p.ldp, p.nbatch);
  return GN_OK;
}

// Writes the planes of an operand.
inline int tc_split(Ctx* ctx, const TcSrc& src, const TcPlanes& p) {
  if (src.s_c == 1) {
    if (p.nbatch > 65535) return fail(GN_ERR_UNSUPPORTED, "tc_split: more than 65535 problems in a batch");
    GN_LAUNCH(ctx, split_rows_kernel, dim3(cdiv((long)p.rows * (p.ldp >> 2), 1024), p.nbatch), 256, 0, src, p.rows, p.K, p.hi, p.xb(), p.lob(), p.ldp);
  } else if (src.s_r == 1) {
    GN_LAUNCH(ctx, split_cols_kernel, dim3(cdiv(p.ldp, 32), cdiv(p.rows, 32), p.nbatch), dim3(32, 8), 0, src, p.rows, p.K, p.hi, p.xb(), p.lob(), p.ldp);
  } else return fail(GN_ERR_UNSUPPORTED, "tc_split: neither stride of the operand is 1");
  return check_launch("tc_split");
}

template <int BN>
inline int tc_launch_persist(Ctx* ctx, const TcPlanes& A, const TcPlanes& B, const TcParams& ep) {
  CUtensorMap mAh, mAx, mAl, mBh, mBx, mBl;
  GN_TRY(tc_make_map(ctx, &mAh, A, A.hi, TC_BM)); GN_TRY(tc_make_map_bf16(ctx, &mAx, A, A.xb(), TC_BM)); GN_TRY(tc_make_map_bf16(ctx, &mAl, A, A.lob(), TC_BM));
  GN_TRY(tc_make_map(ctx, &mBh, B, B.hi, BN)); GN_TRY(tc_make_map_bf16(ctx, &mBx, B, B.xb(), BN)); GN_TRY(tc_make_map_bf16(ctx, &mBl, B, B.lob(), BN));
  const int tiles_m = cdiv(ep.M, TC_BM), tiles_n = cdiv(ep.N, BN); const long total = (long)tiles_m * tiles_n * A.nbatch;
  if (total > 0x7fffffffL) return fail(GN_ERR_UNSUPPORTED, "too many output tiles");
  const unsigned grid = (unsigned)std::min<long>(total, ctx->sm_count);
  ProfScope prof(ctx);
  GN_LAUNCH(ctx, (gemm_tc_persist_kernel<BN, 2>), grid, TC_THREADS, (TcCfg<BN>::SMEM_BYTES), mAh, mAx, mAl, mBh, mBx, mBl, ep, tiles_m, tiles_n, (int)total);
  return check_launch("gemm_tc_persist");
}
// C[z] = A[z] * B[z]^T from prepared planes; the N tile follows the output width.
inline int tc_launch(Ctx* ctx, const TcPlanes& A, const TcPlanes& B, const TcParams& ep_in) {
  if (!ctx->tc_ok) return fail(GN_ERR_UNSUPPORTED, "tcgen05 engine unavailable");
  TcParams ep = ep_in;
  if (A.K != B.K || A.nbatch != B.nbatch || A.rows != ep.M || B.rows != ep.N || A.K != ep.K) return fail(GN_ERR_INVALID_ARG, "tc_launch: operand shapes disagree");
  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  bool vec = ep.N % 4 == 0 && ep.ldc % 4 == 0 && ep.c_b1 % 4 == 0 && ep.c_b2 % 4 == 0 && a16(ep.C) && (!ep.bias || a16(ep.bias));
  if (ep.R) vec = vec && ep.ldr % 4 == 0 && ep.r_b1 % 4 == 0 && ep.r_b2 % 4 == 0 && a16(ep.R);
  if (ep.mask) vec = vec && ep.mask_ld % 4 == 0 && a16(ep.mask);
  if (vec) ep.flags |= TC_FLAG_VEC;
  if (ep.N <= 64) return tc_launch_persist<64>(ctx, A, B, ep);
  return tc_launch_persist<128>(ctx, A, B, ep);
}

// Can the engine run this contraction at all?  One of each operand's strides must be 1; LINEAR/RELU epilogue; alpha 1.
inline bool gemm_tc_supported(Ctx* ctx, const GemmDesc& g) {
  if (!ctx->tc_ok) return false;
  if (g.alpha != 1.f) return false;
  if (!(g.sa_k == 1 || g.sa_m == 1)) return false;
  if (!(g.sb_k == 1 || g.sb_n == 1)) return false;
  if (g.act != GN_ACT_LINEAR && g.act != GN_ACT_RELU) return false;
  return g.M > 0 && g.N > 0 && g.K > 0;
}
// Is it worth it?  Small or skinny problems stay on the SIMT engine.
inline bool gemm_tc_eligible(Ctx* ctx, const GemmDesc& g) {
  if (!gemm_tc_supported(ctx, g)) return false;
  return g.M >= 16 && g.N >= 32 && g.K >= 32 && (double)g.M * g.N * g.K * g.batch1 * g.batch2 >= 1.0e8;
}

// General entry: splits both operands into the context's scratch planes, then runs the contraction.
inline int gemm_tc(Ctx* ctx, const GemmDesc& g) {
  if (!gemm_tc_supported(ctx, g)) return fail(GN_ERR_UNSUPPORTED, "tcgen05 engine cannot run this contraction");
  TcScratch& sc = tc_scratch(ctx);
  const int nb = g.batch1 * g.batch2, ldp = tc_ldp(g.K);
  size_t na = (size_t)nb * g.M * ldp, nbb = (size_t)nb * g.N * ldp;
  if (sc.a_hi.n < na) { GN_CUDA(cudaStreamSynchronize(ctx->stream)); GN_TRY(sc.a_hi.alloc(na)); GN_TRY(sc.a_lo.alloc(na)); sc.last_a = nullptr; }
  if (sc.b_hi.n < nbb) { GN_CUDA(cudaStreamSynchronize(ctx->stream)); GN_TRY(sc.b_hi.alloc(nbb)); GN_TRY(sc.b_lo.alloc(nbb)); }
  TcPlanes A{sc.a_hi.p, sc.a_lo.p, g.M, g.K, ldp, nb}, B{sc.b_hi.p, sc.b_lo.p, g.N, g.K, ldp, nb};
  if (g.reuse_a_planes && nb == 1 && sc.last_a == g.A && sc.last_m == g.M && sc.last_k == g.K && sc.last_ld == g.sa_m && g.sa_k == 1) {
    // same tensor as the previous call (the Q, K and V projections share their input): planes still valid
  } else {
    GN_TRY(tc_split(ctx, TcSrc{g.A, g.sa_m, g.sa_k, g.a_b1, g.a_b2, g.batch2}, A));
    sc.last_a = (nb == 1 && g.sa_k == 1) ? g.A : nullptr; sc.last_m = g.M; sc.last_k = g.K; sc.last_ld = g.sa_m;
  }
  GN_TRY(tc_split(ctx, TcSrc{g.B, g.sb_n, g.sb_k, g.b_b1, g.b_b2, g.batch2}, B));
  TcParams ep{g.C, g.ldc, g.c_b1, g.c_b2, g.bias, g.R, g.ldr, g.r_b1, g.r_b2, g.act, g.M, g.N, g.K, g.batch2, g.flags, ctx->d_status, g.mask, g.mask_ld, g.mask_group};
  // The tensor core truncates when it adds a product group to the accumulator, so the error of one accumulator run grows
  // with its length (measured 3e-6 at K = 1024, 1.2e-5 at K = 4096, normalised).  Long contractions (weight gradients
  // over all tokens of a batch) are therefore cut into slices of TC_KSLICE, each slice adding its result to C through
  // the epilogue's residual path, i.e. in properly rounded fp32.
  if (g.K <= TC_KSLICE || (g.flags & (GEMM_KBEG_AT_M0 | GEMM_KEND_AT_M0))) return tc_launch(ctx, A, B, ep);
  for (int k0 = 0; k0 < g.K; k0 += TC_KSLICE) {
    const int kl = std::min(TC_KSLICE, g.K - k0); const bool first = k0 == 0, last = k0 + kl >= g.K;
    TcPlanes As = A, Bs = B; As.koff = k0; As.K = kl; Bs.koff = k0; Bs.K = kl;
    TcParams es = ep; es.K = kl;
    if (!first) { es.bias = nullptr; es.R = g.C; es.ldr = g.ldc; es.r_b1 = g.c_b1; es.r_b2 = g.c_b2; }
    if (!last) { es.act = GN_ACT_LINEAR; es.mask = nullptr; }
    GN_TRY(tc_launch(ctx, As, Bs, es));
  }
  return GN_OK;
}

}  // namespace gn
