// gemm_tc.cuh -- fp32-accurate contraction on the 5th-generation tensor cores (sm_100a).
//
//   C[M,N] = act( A[M,K] * B[N,K]^T + bias[N] + R[M,N] )
//
// 3xTF32: every fp32 operand x is split into hi = tf32(x) and lo = x - hi (exact in fp32), and the
// product is accumulated as  lo*hi + hi*lo + hi*hi  in one fp32 TMEM accumulator, which restores
// fp32-level accuracy (the dropped lo*lo term is ~2^-22 relative).  The split is materialised by a
// memory-bound pass (split_tf32_kernel / split_tf32_transpose_kernel) into K-major planes, so the
// contraction kernel itself is a pure TMA -> shared memory -> tcgen05.mma pipeline:
//
//   warp 0   TMA producer: 4 tiled bulk copies per stage (A_hi, A_lo, B_hi, B_lo; 128-byte swizzle)
//   warp 1   allocates TMEM, issues tcgen05.mma.kind::tf32 (one elected lane), commits to mbarriers
//   warps 2-5  epilogue: tcgen05.ld of the accumulator, bias / residual / ReLU, transposed through
//              shared memory so that global stores are 128-byte coalesced
//
// Tile 128 x 256 x 32, 2 stages of 96 KB.  Two accumulators of 128 lanes x 256 columns fill the 512 TMEM
// columns: the hi*hi products go to one, the small cross terms (hi*lo, lo*hi) to the other, and the epilogue
// adds them.  The tensor core truncates when it aligns a product sum to the running accumulator, an error
// proportional to the accumulator's magnitude per MMA; keeping the cross terms out of the large accumulator
// cuts the number of such truncations on it by three.
// Every mbarrier wait is bounded; a wait that gives up sets the context's status word and the kernel
// still runs to its end (TMEM is always released).
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "gemm_simt.cuh"

namespace gn {

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 32, TC_STAGES = 2, TC_THREADS = 192;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 4, TC_B_BYTES = TC_BN * TC_BK * 4;
constexpr int TC_STAGE_BYTES = 2 * TC_A_BYTES + 2 * TC_B_BYTES;        // 96 KB
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr unsigned TC_SPIN_LIMIT = 1u << 24;

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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
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
// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are 128 bytes apart, groups of 8
// rows 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100), layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D = f32 (bits 4-5 = 1), A = B = tf32 (bits 7-9, 10-12 = 2), both K-major,
// N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

struct TcEpilogue {
  float* C; long ldc; const float* bias; const float* R; long ldr; int act; int M, N, K; int* status;
};

__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapAhi, const __grid_constant__ CUtensorMap mapAlo,
               const __grid_constant__ CUtensorMap mapBhi, const __grid_constant__ CUtensorMap mapBlo, TcEpilogue ep) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);      // 128B-swizzle tiles need 1024-byte alignment
  uint64_t* bars = (uint64_t*)(smem + TC_STAGES * TC_STAGE_BYTES);                   // full[S], empty[S], accum
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * TC_STAGES + 1);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TC_STAGES), accum = smem_u32(bars + 2 * TC_STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * TC_BN;
  const int nkb = (ep.K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * TC_BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < nkb; kb++) {
        const int s = kb % TC_STAGES, use = kb / TC_STAGES;
        if (use > 0) ok &= mbar_wait(empty0 + 8 * s, (use - 1) & 1);
        const uint32_t base = smem_u32(smem + s * TC_STAGE_BYTES), bar = full0 + 8 * s;
        mbar_expect_tx(bar, TC_STAGE_BYTES);
        tma_load_2d(base, &mapAhi, kb * TC_BK, m0, bar);
        tma_load_2d(base + TC_A_BYTES, &mapAlo, kb * TC_BK, m0, bar);
        tma_load_2d(base + 2 * TC_A_BYTES, &mapBhi, kb * TC_BK, n0, bar);
        tma_load_2d(base + 2 * TC_A_BYTES + TC_B_BYTES, &mapBlo, kb * TC_BK, n0, bar);
      }
      if (!ok) atomicExch(ep.status, 1);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      constexpr uint32_t idesc = make_idesc(TC_BM, TC_BN);
      for (int kb = 0; kb < nkb; kb++) {
        const int s = kb % TC_STAGES, use = kb / TC_STAGES;
        ok &= mbar_wait(full0 + 8 * s, use & 1);
        tc_fence_after();
        const uint32_t base = smem_u32(smem + s * TC_STAGE_BYTES);
        const uint64_t ahi = make_desc(base), alo = make_desc(base + TC_A_BYTES);
        const uint64_t bhi = make_desc(base + 2 * TC_A_BYTES), blo = make_desc(base + 2 * TC_A_BYTES + TC_B_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 8; k++) {
          const uint64_t adv = (uint64_t)((k * 8 * 4) >> 4);          // 8 tf32 = 32 bytes along K inside the swizzle atom
          const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
          tc_mma_tf32(tmem_base + TC_BN, alo + adv, bhi + adv, idesc, acc);     // cross terms -> second accumulator
          tc_mma_tf32(tmem_base + TC_BN, ahi + adv, blo + adv, idesc, 1u);
          tc_mma_tf32(tmem_base, ahi + adv, bhi + adv, idesc, acc);             // main term
        }
        tc_commit(empty0 + 8 * s);           // frees this stage once the MMAs above have read it
      }
      tc_commit(accum);                      // accumulator complete
      if (!ok) atomicExch(ep.status, 2);
    }
  } else {
    // epilogue warps: TMEM lane quadrant = warp % 4
    const int quad = warp & 3;
    bool ok = true;
    if (lane == 0) ok = mbar_wait(accum, 0);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok && lane == 0) atomicExch(ep.status, 3);
    __syncwarp();
    tc_fence_after();
    // the pipeline stages are idle once the accumulator barrier fired: reuse stage memory as a per-warp 32x33 transpose tile
    float* tile = (float*)smem + (warp - 2) * (32 * 33);
    const int row_base = m0 + quad * 32;
    for (int c = 0; c < TC_BN / 32; c++) {
      const int col0 = n0 + c * 32;
      if (col0 >= ep.N) break;
      uint32_t r[32], q[32];
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32);
      tmem_ld32(taddr, r);
      tmem_ld32(taddr + TC_BN, q);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(q[j]));
#pragma unroll
      for (int j = 0; j < 32; j++) tile[lane * 33 + j] = __uint_as_float(r[j]);     // thread = row, conflict-free (stride 33)
      __syncwarp();
      const int col = col0 + lane;
      const float bv = (ep.bias && col < ep.N) ? ep.bias[col] : 0.f;
      if (col < ep.N) {
        for (int rr = 0; rr < 32; rr++) {
          const int row = row_base + rr;
          if (row >= ep.M) break;
          float v = tile[rr * 33 + lane] + bv;
          if (ep.R) v += ep.R[(long)row * ep.ldr + col];
          if (ep.act == GN_ACT_RELU) v = v > 0.f ? v : 0.f;
          ep.C[(long)row * ep.ldc + col] = v;
        }
      }
      __syncwarp();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * TC_BN)) : "memory");
}

// ------------------------------------------------------------------ operand split (memory-bound)
__device__ __forceinline__ float tf32_round(float x) { uint32_t u; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x)); return __uint_as_float(u); }
// hi/lo planes [rows, ldp] of a K-major source [rows, cols] (row stride ld); columns cols..ldp-1 are zero-filled
__global__ void split_tf32_kernel(const float* __restrict__ src, long ld, int rows, int cols, float* __restrict__ hi, float* __restrict__ lo, int ldp) {
  long total = (long)rows * ldp;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    int c = (int)(i % ldp); long r = i / ldp;
    float x = c < cols ? src[r * ld + c] : 0.f;
    float h = tf32_round(x);
    hi[i] = h; lo[i] = x - h;
  }
}
// planes of the TRANSPOSE: source [rows, cols] (row stride ld) -> hi/lo [cols, ldp] (ldp >= rows), through a 32x32 shared tile
__global__ void split_tf32_transpose_kernel(const float* __restrict__ src, long ld, int rows, int cols, float* __restrict__ hi, float* __restrict__ lo, int ldp) {
  __shared__ float t[32][33];
  int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) { int r = r0 + j, c = c0 + threadIdx.x; t[j][threadIdx.x] = (r < rows && c < cols) ? src[(long)r * ld + c] : 0.f; }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int c = c0 + j, r = r0 + threadIdx.x;
    if (c < cols && r < ldp) { float x = t[threadIdx.x][j]; float h = tf32_round(x); hi[(long)c * ldp + r] = h; lo[(long)c * ldp + r] = x - h; }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct TcScratch { DevBuf a_hi, a_lo, b_hi, b_lo; };
inline TcScratch& tc_scratch(Ctx* ctx) { static thread_local std::vector<std::pair<Ctx*, TcScratch*>> tab; for (auto& e : tab) if (e.first == ctx) return *e.second; tab.push_back({ctx, new TcScratch()}); return *tab.back().second; }

inline void tc_init(Ctx* ctx) {
  ctx->tc_ok = false;
  void* fn = nullptr; cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess) { cudaGetLastError(); return; }
  if (cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES) != cudaSuccess) { cudaGetLastError(); return; }
  ctx->encode_tiled = fn; ctx->tc_ok = true;
}

// Can the engine run this contraction at all?  A must be K-major; B either K-major (X W^T) or N-major (dZ W, via the
// transposing split); single problem; no causal tile flags; fp32 alpha of 1.
inline bool gemm_tc_supported(Ctx* ctx, const GemmDesc& g) {
  if (!ctx->tc_ok) return false;
  if (g.batch1 * g.batch2 != 1 || g.flags != 0 || g.alpha != 1.f) return false;
  if (g.sa_k != 1) return false;
  if (!(g.sb_k == 1 || g.sb_n == 1)) return false;
  if (g.act != GN_ACT_LINEAR && g.act != GN_ACT_RELU) return false;
  return g.M > 0 && g.N > 0 && g.K > 0;
}
// Is it worth it?  Small or skinny problems stay on the SIMT engine.
inline bool gemm_tc_eligible(Ctx* ctx, const GemmDesc& g) {
  if (!gemm_tc_supported(ctx, g)) return false;
  return g.M >= 128 && g.N >= 64 && g.K >= 64 && (double)g.M * g.N * g.K >= 1.0e8;
}

inline int tc_make_map(Ctx* ctx, CUtensorMap* map, const float* base, int rows, int cols, int ldp, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ldp * 4};
  cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = ((PFN_encodeTiled)ctx->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GN_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (rows %d cols %d ld %d)", (int)r, rows, cols, ldp);
  return GN_OK;
}

inline int gemm_tc(Ctx* ctx, const GemmDesc& g) {
  if (!gemm_tc_supported(ctx, g)) return fail(GN_ERR_UNSUPPORTED, "tcgen05 engine cannot run this contraction");
  TcScratch& sc = tc_scratch(ctx);
  const int ldp = ((g.K + 3) / 4) * 4;                    // plane row stride: a multiple of 16 bytes for TMA
  size_t na = (size_t)g.M * ldp, nb = (size_t)g.N * ldp;
  if (sc.a_hi.n < na) { GN_CUDA(cudaStreamSynchronize(ctx->stream)); GN_TRY(sc.a_hi.alloc(na)); GN_TRY(sc.a_lo.alloc(na)); }
  if (sc.b_hi.n < nb) { GN_CUDA(cudaStreamSynchronize(ctx->stream)); GN_TRY(sc.b_hi.alloc(nb)); GN_TRY(sc.b_lo.alloc(nb)); }
  long ga = std::min<long>(((long)na + 255) / 256, (long)ctx->sm_count * 32);
  GN_LAUNCH(ctx, split_tf32_kernel, (unsigned)ga, 256, 0, g.A, g.sa_m, g.M, g.K, sc.a_hi.p, sc.a_lo.p, ldp);
  if (g.sb_k == 1) {
    long gb = std::min<long>(((long)nb + 255) / 256, (long)ctx->sm_count * 32);
    GN_LAUNCH(ctx, split_tf32_kernel, (unsigned)gb, 256, 0, g.B, g.sb_n, g.N, g.K, sc.b_hi.p, sc.b_lo.p, ldp);
  } else {
    // B(k,n) = src[k*sb_k + n]: source is [K rows, N cols]; planes hold its transpose [N, K]
    dim3 grid(cdiv(g.N, 32), cdiv(ldp, 32)), block(32, 8);
    GN_LAUNCH(ctx, split_tf32_transpose_kernel, grid, block, 0, g.B, g.sb_k, g.K, g.N, sc.b_hi.p, sc.b_lo.p, ldp);
  }
  CUtensorMap mAh, mAl, mBh, mBl;
  GN_TRY(tc_make_map(ctx, &mAh, sc.a_hi.p, g.M, g.K, ldp, TC_BM)); GN_TRY(tc_make_map(ctx, &mAl, sc.a_lo.p, g.M, g.K, ldp, TC_BM));
  GN_TRY(tc_make_map(ctx, &mBh, sc.b_hi.p, g.N, g.K, ldp, TC_BN)); GN_TRY(tc_make_map(ctx, &mBl, sc.b_lo.p, g.N, g.K, ldp, TC_BN));
  TcEpilogue ep{g.C, g.ldc, g.bias, g.R, g.ldr, g.act, g.M, g.N, g.K, ctx->d_status};
  dim3 grid(cdiv(g.N, TC_BN), cdiv(g.M, TC_BM));
  GN_LAUNCH(ctx, gemm_tc_kernel, grid, TC_THREADS, TC_SMEM_BYTES, mAh, mAl, mBh, mBl, ep);
  return check_launch("gemm_tc");
}

}  // namespace gn
