// gemm_tc.cuh -- fp32-accurate contraction on the 5th-generation tensor cores (sm_100a).
//
//   C[M,N] = act( A[M,K] * B[N,K]^T + bias[N] + R[M,N] )
//
// Split-operand scheme (three half-precision products per fp32 product).  Every operand row (one output row's or
// output column's K-vector) is first multiplied by a power of two s that brings its largest magnitude into
// [2^14, 2^15), and each scaled element is written as
//     x s = x0 + x1 + r,   x0 = fp16(x s),  x1 = fp16(x s - x0),  |r| <= 2^-22 |x s| + 2^-25
// (fp16 carries 11 significant bits, so two planes hold 22 of the 24 bits of an fp32 mantissa; elements far below the
// row's maximum land in fp16's subnormal range, where the absolute error 2^-25 is 2^-39 of the row's maximum).  Then
//     a*b  =  ( a0*b0  +  a0*b1 + a1*b0 ) / (s_a s_b)      (dropped: a1*b1, r_a*b, a*r_b -- each about 2^-22 |a b|).
// All three terms are tcgen05.mma.kind::f16 instructions with fp32 accumulation in tensor memory; a product of two
// fp16 numbers is exact in fp32, and the division by the two powers of two in the epilogue is exact.  Against the
// other ways of reaching fp32 accuracy on these tensor cores -- three TF32 instructions (6 units of tensor time per
// product, 8-byte operand planes), or one TF32 and two BF16 instructions (4 units, 8 bytes; what this file did
// before) -- this costs 3 units and the operand planes are 4 bytes per element, the size of the fp32 source.  That
// halves what the kernel pulls through L2 and shared memory, which matters because the kernel is bound by
// shared-memory bandwidth, not by the tensor pipe: with 128 x 128 tiles every MMA re-reads both operands from shared
// memory (8 KB per 64 tensor cycles = the full 128 B/clk) while TMA writes the next stage into the same memory.  The
// large-problem variant therefore uses 128 x 256 tiles (12 KB per 128 tensor cycles).
//
// The operand planes (K-major fp16, row stride a multiple of 8 elements) and the per-row inverse scales are written
// by a memory-bound pass (split2_rows_kernel / split2_cols_kernel); the contraction kernel itself is a pure
// TMA -> shared memory -> tcgen05.mma pipeline:
//
//   warp 0   TMA producer: 4 tiled bulk copies per stage (64-byte rows, 64-byte swizzle; 3-D maps, third
//            coordinate = problem index of a batch)
//   warp 1   allocates TMEM, issues the MMAs (one elected lane), commits to mbarriers
//   warps 2-5  epilogue: tcgen05.ld of the accumulators, scales / bias / residual / ReLU / gate, one output row
//              per thread with 16-byte stores
//
// Persistent: one CTA per SM walks 128 x BN output tiles.  TMEM holds two accumulator slots, so the epilogue
// of tile i runs under the mainloop of tile i+1.  The tensor core truncates when it adds a group of products
// to the accumulator, an error proportional to the accumulator's magnitude per MMA instruction.  With BN = 64
// or 128 each slot therefore has two accumulators -- the a0*b0 products go to one, the small cross terms to
// the other, and the epilogue adds them -- and with BN = 256 (one accumulator per slot, 512 columns in all) the
// host cuts long contractions into shorter accumulator runs instead.
// Every mbarrier wait is bounded.  A wait that gives up sets the context's status word and a flag in shared
// memory; every role of the CTA then leaves its loops without issuing further copies or MMAs, the producer
// waits (bounded) for its copies in flight, the MMA role for its instructions in flight, and TMEM is released.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdlib>
#include "common.cuh"
#include "gemm_simt.cuh"

namespace gn {

constexpr int TC_BM = 128;
constexpr int TC_EPI_WARPS = 8;                 // two warps per TMEM lane quadrant, each takes half of a tile's columns
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS;   // TMA warp, MMA warp, epilogue warps
constexpr unsigned TC_SPIN_LIMIT = 1u << 24;    // default number of polls of one wait (Ctx::spin_limit overrides it)
constexpr unsigned TC_DRAIN_LIMIT = 1u << 20;   // polls spent waiting for own work in flight after a wait gave up
constexpr int TC_QUEUE_POOL = 2048;   // tile-queue counters per context before the pool is cleared again
constexpr int TC_FLAG_VEC = 4096;   // epilogue may use 16-byte accesses (set by the host when every pointer and stride allows it)
// One stage = 32 contraction indices of both operands: two fp16 planes each, 64-byte rows.
constexpr int TC_BK = 32;
template <int BN> struct TcCfg {
  static constexpr int A_PL = TC_BM * TC_BK * 2, B_PL = BN * TC_BK * 2;           // one plane of a stage: 8 KB, BN * 64 B
  static constexpr int STAGE_BYTES = 2 * A_PL + 2 * B_PL;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES > 8 ? 8 : (192 * 1024) / STAGE_BYTES;
  static constexpr int COLV_FLOATS = TC_EPI_WARPS * BN;                           // per epilogue warp: scale and bias of its BN / 2 columns
  static constexpr int STG_FLOATS = TC_EPI_WARPS * 32 * 20;                       // per epilogue warp: 32 rows x 16 (+4) accumulators in transit
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + (COLV_FLOATS + STG_FLOATS) * 4;
  static constexpr bool MERGED = BN > 128;                                        // one accumulator per slot
  static constexpr int SLOT_COLS = MERGED ? BN : 2 * BN;
  static constexpr int TMEM_COLS = 2 * SLOT_COLS;
  static_assert(2 * STAGES + 6 <= 30, "barrier area");
  static_assert(TMEM_COLS <= 512, "accumulator slots must fit the 512 TMEM columns");
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: returns false when it gave up -- after `limit` polls, or as soon as `*abort_flag` (a word in
// shared memory that a role of this CTA sets when one of its own waits gave up) is non-zero.  A poll is
// mbarrier.try_wait, which may suspend the thread for a while by itself; limits below 4096 poll with the
// non-suspending mbarrier.test_wait instead, so that a small limit really is a short time (the failure-detection
// tests rely on that to make a wait run out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned limit = TC_SPIN_LIMIT, const volatile int* abort_flag = nullptr) {
  if (limit < 4096u) {
    for (unsigned it = 0; it < limit; it++) {
      uint32_t done;
      asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
      if (done) return true;
    }
    return false;
  }
  for (unsigned it = 0; it < limit; it++) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if (abort_flag && (it & 63) == 63 && *abort_flag) return false;
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
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
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
// Instruction descriptor of kind::f16 with A = B = fp16 (format code 0 at bits 7-9 and 10-12), D = f32 (bits 4-5 = 1), both
// operands K-major, N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N) {
  return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}


// ------------------------------------------------------------------ splitting a value into operand planes
// Power of two s that brings a row whose largest magnitude is mx into [2^14, 2^15) (fp16 overflows at 65504), and its
// inverse.  s = 1 for a row of zeros (and for a row that holds an infinity or a NaN, which the products then carry on).
__device__ __forceinline__ float row_scale(float mx, float* inv) {
  if (!(mx > 0.f) || !(mx <= 3.0e38f)) { *inv = 1.f; return 1.f; }
  int se = 14 - (((__float_as_int(mx) >> 23) & 0xff) - 127);
  se = max(-100, min(100, se));
  *inv = __int_as_float((127 - se) << 23); return __int_as_float((127 + se) << 23);
}
// (x s) -> (fp16(x s), fp16(x s - fp16(x s))) for two neighbouring elements, packed
__device__ __forceinline__ void split2_pair(float a, float b, float s, uint32_t& p0, uint32_t& p1) {
  a *= s; b *= s;
  const __half2 h = __floats2half2_rn(a, b);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
  p0 = *reinterpret_cast<const uint32_t*>(&h); p1 = *reinterpret_cast<const uint32_t*>(&l);
}

// Output side of one launch.  Batched problems: problem z -> (z / batch2, z % batch2) selects the
// output (and residual) sub-matrix; the operand planes of problem z are slice z of the 3-D tensor maps.
struct TcParams {
  float* C; long ldc, c_b1, c_b2; const float* bias; const float* R; long ldr, r_b1, r_b2;
  int act, M, N, K, batch2, flags; int* status;
  const float* mask; long mask_ld; int mask_group;    // optional gate, see GemmDesc::mask
  const float* isa = nullptr; const float* isb = nullptr;   // inverse row scales of the operand planes: [nbatch][M], [nbatch][N]
  unsigned spin_limit = TC_SPIN_LIMIT;                // polls per wait before the kernel gives up
  int nchw_P = 0;      // > 0: output row r = (sample r / P, position r % P) is stored as C[sample][col][position] (N channels of P positions)
  // Plane output (out_p0 != null): the result is not stored as fp32 but directly as the operand planes of the next
  // contraction (two fp16 planes [M][out_ldp] and an inverse scale per row), see TcPlaneOut.  C may then be null.
  __half* out_p0 = nullptr; __half* out_p1 = nullptr; float* out_inv = nullptr; long out_ldp = 0;
  const float* a_rownorm = nullptr; const int* b_maxabs = nullptr;     // the bound's factors: |row of A|_2 and max |entry of B (and bias)| as float bits
  float* c_last = nullptr; int last_T = 0;                             // fp32 copy of the rows r with r % last_T == last_T - 1: c_last[(r / last_T) * N + col]
  float* rowsum32 = nullptr;                                           // plane output: sums of the result over every 32 consecutive rows, [ceil(M / 32)][N]
};

// Epilogue of one output tile.  Eight warps share it: a warp may only read the TMEM lanes of its quadrant (warp % 4), so
// two warps serve each quadrant and take half of the tile's columns each (`chalf`); one output row per thread (TMEM lane
// = row), 32 consecutive columns per tcgen05.ld, written as 8 float4.  The per-column factors (inverse scale of B's
// rows, bias) of the warp's columns are staged in shared memory by tc_epilogue_stage BEFORE the warp waits for the
// accumulator, so that their latency is hidden behind the MMAs; residual and gate values of a chunk are fetched before
// the TMEM wait for the same reason.  (With four warps and the factors fetched per chunk the epilogue of a tile took as
// long as its MMAs at K = 1024 and held the tensor pipe back.)  `acc_main` / `acc_cross` are the TMEM column offsets of
// the two accumulators of this tile (MERGED: there is only acc_main); `bw` is the tile's width (BN, or BN / 2 for a half tile).
template <int BN>
__device__ __forceinline__ void tc_epilogue_stage(const TcParams& ep, int n0, int z, int chalf, int lane, int bw, float* colv) {
    if (!(ep.flags & TC_FLAG_VEC)) return;
    const int ncw = bw / 2, cbase = n0 + chalf * ncw;
    const float* isb = ep.isb + (long)z * ep.N;
    __syncwarp();
    for (int i = lane * 4; i < ncw; i += 128) {
      const int col = cbase + i; const bool in = col < ep.N;
      *reinterpret_cast<float4*>(colv + i) = in ? __ldg(reinterpret_cast<const float4*>(isb + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(colv + BN / 2 + i) = (in && ep.bias) ? __ldg(reinterpret_cast<const float4*>(ep.bias + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncwarp();
}
// `stg`: this warp's staging buffer of 32 rows x TC_STG_LD floats.  The TMEM load gives every thread ITS row (lane =
// row), and a store of that shape touches 32 different 128-byte lines per instruction -- measured: 19 000 cycles of
// epilogue per 128 x 256 tile, twice that for the two planes of a plane output, which then set the pace instead of the
// MMAs.  So the accumulators of 16 columns go through shared memory and come back with four neighbouring lanes on one
// row (8 rows per instruction); scale, bias, residual, activation and gate are applied on that side, where the residual
// and gate reads are coalesced too.
constexpr int TC_STG_LD = 20;
template <int BN, bool MERGED>
__device__ __forceinline__ void tc_epilogue_tile(const TcParams& ep, uint32_t tmem_base, uint32_t acc_main, uint32_t acc_cross,
                                                 int m0, int n0, int z, int quad, int chalf, int lane, int nkb, int bw, const float* colv, float* stg) {
    const int z1 = z / ep.batch2, z2 = z % ep.batch2;
    float* C = ep.C + z1 * ep.c_b1 + z2 * ep.c_b2;
    const float* R = ep.R ? ep.R + z1 * ep.r_b1 + z2 * ep.r_b2 : nullptr;
    const bool vec = (ep.flags & TC_FLAG_VEC) != 0;
    const float* isb = ep.isb + (long)z * ep.N;
    const int nch = bw / 64;                                               // chunks of 32 columns per warp
    if (vec) {
      // after the transposition: lane -> row 8 t + lane / 4 of the warp's 32 (t = 0..3), columns 4 (lane % 4) .. + 3 of 16
      const int rl = lane >> 2, c4 = (lane & 3) * 4, rbase = m0 + quad * 32;
      float isa4[4], osc4[4];
#pragma unroll
      for (int t = 0; t < 4; t++) {
        const int row = rbase + 8 * t + rl; const bool row_ok = row < ep.M;
        isa4[t] = row_ok ? ep.isa[(long)z * ep.M + row] : 1.f;              // 1 / (scale of this output row's A vector), a power of two
        osc4[t] = 1.f;                                                       // plane output: this row's scale
        if (ep.out_p0 && row_ok) {
          const float an = ep.a_rownorm[row], bound = sqrtf(fmaf(an, an, 1.f)) * sqrtf((float)ep.K + 1.f) * __int_as_float(*ep.b_maxabs);
          float oinv; osc4[t] = row_scale(bound, &oinv);
          if (n0 == 0 && chalf == 0 && c4 == 0) ep.out_inv[row] = oinv;
        }
      }
      for (int cc = 0; cc < nch; cc++) {
        const int c = chalf * nch + cc, col0 = n0 + c * 32;
        if (col0 >= ep.N) break;
        uint32_t r[32], q[MERGED ? 1 : 32];
        if (nkb > 0) {
          const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32);
          tmem_ld32(taddr + acc_main, r);
          if constexpr (!MERGED) tmem_ld32(taddr + acc_cross, q);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if constexpr (!MERGED) {
#pragma unroll
            for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(q[j]));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j++) r[j] = 0u;
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int col = col0 + 16 * h + c4; const bool col_ok = col < ep.N;
          // residual and gate of this half, fetched before the exchange so that their latency overlaps it
          float4 rv[4], mv[4];
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const int row = rbase + 8 * t + rl; const bool in = col_ok && row < ep.M;
            rv[t] = (R && in) ? *reinterpret_cast<const float4*>(R + (long)row * ep.ldr + col) : make_float4(0.f, 0.f, 0.f, 0.f);
            mv[t] = (ep.mask && in) ? *reinterpret_cast<const float4*>(ep.mask + (long)(row / ep.mask_group) * ep.mask_ld + col) : make_float4(1.f, 1.f, 1.f, 1.f);
          }
          __syncwarp();                                       // the previous half has been read back
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 a = make_float4(__uint_as_float(r[16 * h + j]), __uint_as_float(r[16 * h + j + 1]), __uint_as_float(r[16 * h + j + 2]), __uint_as_float(r[16 * h + j + 3]));
            *reinterpret_cast<float4*>(stg + lane * TC_STG_LD + j) = a;
          }
          __syncwarp();
          const float4 sv = *reinterpret_cast<const float4*>(colv + cc * 32 + 16 * h + c4), bv = *reinterpret_cast<const float4*>(colv + BN / 2 + cc * 32 + 16 * h + c4);
          float4 csum = make_float4(0.f, 0.f, 0.f, 0.f);      // plane output: this lane's part of the warp's 32-row column sums
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const int row = rbase + 8 * t + rl;
            if (!col_ok || row >= ep.M) continue;
            const float4 a = *reinterpret_cast<const float4*>(stg + (8 * t + rl) * TC_STG_LD + c4);
            const float isa = isa4[t];
            float4 v;
            v.x = a.x * isa * sv.x + bv.x + rv[t].x; v.y = a.y * isa * sv.y + bv.y + rv[t].y;
            v.z = a.z * isa * sv.z + bv.z + rv[t].z; v.w = a.w * isa * sv.w + bv.w + rv[t].w;
            if (ep.act == GN_ACT_RELU) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
            if (!(mv[t].x > 0.f)) v.x = 0.f; if (!(mv[t].y > 0.f)) v.y = 0.f; if (!(mv[t].z > 0.f)) v.z = 0.f; if (!(mv[t].w > 0.f)) v.w = 0.f;
            if (ep.out_p0) {
              uint2 p0, p1; split2_pair(v.x, v.y, osc4[t], p0.x, p1.x); split2_pair(v.z, v.w, osc4[t], p0.y, p1.y);
              const long o = (long)row * ep.out_ldp + col;
              *reinterpret_cast<uint2*>(ep.out_p0 + o) = p0; *reinterpret_cast<uint2*>(ep.out_p1 + o) = p1;
              if (ep.c_last && row % ep.last_T == ep.last_T - 1) *reinterpret_cast<float4*>(ep.c_last + (long)(row / ep.last_T) * ep.N + col) = v;
              csum.x += v.x; csum.y += v.y; csum.z += v.z; csum.w += v.w;
            } else *reinterpret_cast<float4*>(C + (long)row * ep.ldc + col) = v;
          }
          if (ep.rowsum32) {
            // the consumer of a plane output's token sums (the weight gradient of the layer below) gets them from here instead
            // of re-reading the planes: rows 8 t + rl of this lane, then the eight lanes that share its columns, in a fixed order
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
              csum.x += __shfl_xor_sync(0xffffffffu, csum.x, o); csum.y += __shfl_xor_sync(0xffffffffu, csum.y, o);
              csum.z += __shfl_xor_sync(0xffffffffu, csum.z, o); csum.w += __shfl_xor_sync(0xffffffffu, csum.w, o);
            }
            if (rl == 0 && col_ok && rbase < ep.M) *reinterpret_cast<float4*>(ep.rowsum32 + (long)(rbase >> 5) * ep.N + col) = csum;
          }
        }
      }
      __syncwarp();
      return;
    }
    // scalar path (unaligned operands, NCHW store): one output row per thread
    const int row = m0 + quad * 32 + lane;
    const bool row_ok = row < ep.M;
    const float* Rrow = (R && row_ok) ? R + (long)row * ep.ldr : nullptr;
    const float* Mrow = (ep.mask && row_ok) ? ep.mask + (long)(row / ep.mask_group) * ep.mask_ld : nullptr;
    float* Crow = C + (long)row * ep.ldc;
    const float isa = row_ok ? ep.isa[(long)z * ep.M + row] : 1.f;
    for (int cc = 0; cc < nch; cc++) {
      const int c = chalf * nch + cc, col0 = n0 + c * 32;
      if (col0 >= ep.N) break;
      uint32_t r[32], q[MERGED ? 1 : 32];
      if (nkb > 0) {
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32);
        tmem_ld32(taddr + acc_main, r);
        if constexpr (!MERGED) tmem_ld32(taddr + acc_cross, q);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
#pragma unroll
      for (int j = 0; j < 32; j++) {
        const int col = col0 + j;
        if (!row_ok || col >= ep.N) continue;
        float a = 0.f;
        if (nkb > 0) { if constexpr (MERGED) a = __uint_as_float(r[j]); else a = __uint_as_float(r[j]) + __uint_as_float(q[j]); }
        float v = a * isa * isb[col];
        if (ep.bias) v += ep.bias[col];
        if (Rrow) v += Rrow[col];
        if (ep.act == GN_ACT_RELU) v = fmaxf(v, 0.f);
        if (Mrow && !(Mrow[col] > 0.f)) v = 0.f;
        if (ep.nchw_P > 0) C[((long)(row / ep.nchw_P) * ep.N + col) * ep.nchw_P + row % ep.nchw_P] = v;
        else Crow[col] = v;
      }
    }
  }

__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persist_kernel(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
                       const __grid_constant__ CUtensorMap mapB0, const __grid_constant__ CUtensorMap mapB1,
                       TcParams ep, int tiles_m, int tiles_n, int total_tiles, int full_end, int n_half, int* tile_queue) {
  using Cfg = TcCfg<BN>;
  constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES, BK = TC_BK;
  constexpr bool MERGED = Cfg::MERGED;
  constexpr uint32_t TMEM_COLS = Cfg::TMEM_COLS, SLOT_COLS = Cfg::SLOT_COLS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);       // full[S], empty[S], tfull[2], tempty[2], drain
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 5);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);       // set by the first role whose wait gave up
  uint64_t* qbars = bars + 2 * STAGES + 6;                         // tile queue: qfull[4], qempty[4], then the four queued items
  volatile int* qitem = (volatile int*)(qbars + 8);
  const uint32_t qfull0 = smem_u32(qbars), qempty0 = smem_u32(qbars + 4);
  float* colv_all = (float*)(smem + STAGES * STAGE_BYTES + 256);   // epilogue warps' column factors
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
  const uint32_t drain = smem_u32(bars + 2 * STAGES + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // stage layout: A plane 0 | A plane 1 | B plane 0 | B plane 1
  constexpr uint32_t OFF_A1 = Cfg::A_PL, OFF_B0 = 2 * Cfg::A_PL, OFF_B1 = OFF_B0 + Cfg::B_PL;
  const unsigned limit = ep.spin_limit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, TC_EPI_WARPS); }
    mbar_init(drain, 1);
    for (int b = 0; b < 4; b++) { mbar_init(qfull0 + 8 * b, 1); mbar_init(qempty0 + 8 * b, 1 + TC_EPI_WARPS); }
    *abort_flag = 0;
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

  // Work list of this CTA (identical in every role): tiles blockIdx.x, + gridDim.x, ... below full_end; then, when the
  // tiles left over would occupy at most half of the CTAs (n_half = twice their number, else 0), one HALF of a left-over
  // tile each (BN / 2 columns), so that the last, short round costs about 0.6 instead of 1 tile time.
  // a wait gave up: record which role, and tell the other roles of this CTA to stop
  auto give_up = [&](int code) { atomicExch(ep.status, code); *abort_flag = 1; __threadfence_block(); };
  auto item = [&](long t, int& tile, int& half) -> bool {
    if (t < full_end) { tile = (int)t; half = -1; return true; }
    const long h = t - full_end;
    if (h >= n_half) return false;
    tile = full_end + (int)(h >> 1); half = (int)(h & 1); return true;
  };
  // With a tile queue (tile_queue != null: a zeroed counter in global memory) the producer thread draws the items with
  // atomicAdd and hands each to the MMA thread and the epilogue warps through a four-entry ring in shared memory, so a
  // CTA that gets its SM late (other kernels -- the collectives of a multi-GPU step -- holding SMs when the launch
  // starts) simply finds less left to do, instead of the whole launch waiting for its fixed share.
  const bool queued = tile_queue != nullptr;
  auto work = [&](int k, int& tile, int& half) -> bool {
    if (!queued) return item((long)blockIdx.x + (long)k * gridDim.x, tile, half);
    const uint32_t qs = (uint32_t)k & 3, qu = (uint32_t)k >> 2; int t = -1;
    if (warp == 0) {                                      // producer thread: draw and publish
      if (qu > 0 && !mbar_wait(qempty0 + 8 * qs, (qu - 1) & 1, limit, abort_flag)) { if (!*abort_flag) give_up(4); return false; }
      t = atomicAdd(tile_queue, 1);
      if ((long)t >= (long)full_end + n_half) t = -1;
      qitem[qs] = t;
      mbar_arrive(qfull0 + 8 * qs);
    } else {                                              // consumers: one thread per warp reads
      if (lane == 0) {
        if (mbar_wait(qfull0 + 8 * qs, qu & 1, limit, abort_flag)) { t = qitem[qs]; mbar_arrive(qempty0 + 8 * qs); }
        else if (!*abort_flag) give_up(5);
      }
      if (warp >= 2) t = __shfl_sync(0xffffffffu, t, 0);
    }
    return t >= 0 && item(t, tile, half);
  };
  // tile -> coordinates and contraction range
  auto decode = [&](int tile, int half, int& m0, int& n0, int& z, int& kb0, int& nkb) -> bool {
    const int nt = tile % tiles_n, q = tile / tiles_n, mt = q % tiles_m; z = q / tiles_m;
    m0 = mt * TC_BM; n0 = nt * BN + (half > 0 ? BN / 2 : 0);
    if ((ep.flags & GEMM_SKIP_UPPER) && n0 > m0 + TC_BM - 1) return false;
    int kbeg = 0, kend = ep.K;
    if (ep.flags & GEMM_KBEG_AT_M0) kbeg = (m0 / BK) * BK;
    if (ep.flags & GEMM_KEND_AT_M0) kend = min(ep.K, m0 + TC_BM);
    kb0 = kbeg / BK; nkb = (kend - kbeg + BK - 1) / BK;
    return true;
  };

  uint32_t issued = 0;          // producer thread: stages whose copies it has started
  if (warp == 0) {
    if (lane == 0) {
      bool ok = true; uint32_t it = 0;
      int tile, half;
      for (int w = 0; ok && work(w, tile, half); w++) {
        int m0, n0, z, kb0, nkb; if (!decode(tile, half, m0, n0, z, kb0, nkb)) continue;
        for (int i = 0; i < nkb; i++, it++) {
          const uint32_t s = it % STAGES, use = it / STAGES; const int kc = (kb0 + i) * BK;
          if (use > 0 && !mbar_wait(empty0 + 8 * s, (use - 1) & 1, limit, abort_flag)) { ok = false; break; }
          const uint32_t base = smem_u32(smem + s * STAGE_BYTES), bar = full0 + 8 * s;
          mbar_expect_tx(bar, half < 0 ? STAGE_BYTES : STAGE_BYTES - Cfg::B_PL);
          tma_load_3d(base, &mapA0, kc, m0, z, bar);
          tma_load_3d(base + OFF_A1, &mapA1, kc, m0, z, bar);
          tma_load_3d(base + OFF_B0, &mapB0, kc, n0, z, bar);          // the B copies are BN / 2 rows each
          tma_load_3d(base + OFF_B1, &mapB1, kc, n0, z, bar);
          if (half < 0) {
            tma_load_3d(base + OFF_B0 + Cfg::B_PL / 2, &mapB0, kc, n0 + BN / 2, z, bar);
            tma_load_3d(base + OFF_B1 + Cfg::B_PL / 2, &mapB1, kc, n0 + BN / 2, z, bar);
          }
        }
      }
      if (!ok && !*abort_flag) give_up(1);
      issued = it;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true; uint32_t it = 0, lt = 0;
      constexpr uint32_t idesc_full = make_idesc_f16(TC_BM, BN), idesc_half = make_idesc_f16(TC_BM, BN / 2);
      int tile, half;
      for (int w = 0; ok && work(w, tile, half); w++) {
        int m0, n0, z, kb0, nkb; if (!decode(tile, half, m0, n0, z, kb0, nkb)) continue;
        const uint32_t idesc = half < 0 ? idesc_full : idesc_half;
        const uint32_t slot = lt & 1, u = lt >> 1; lt++;
        if (!mbar_wait(tempty0 + 8 * slot, (u & 1) ^ 1, limit, abort_flag)) { ok = false; break; }     // slot drained by the epilogue (passes at once the first time)
        tc_fence_after();
        const uint32_t acc_main = tmem_base + slot * SLOT_COLS, acc_cross = MERGED ? acc_main : acc_main + BN;
        for (int i = 0; i < nkb; i++, it++) {
          const uint32_t s = it % STAGES, use = it / STAGES;
          if (!mbar_wait(full0 + 8 * s, use & 1, limit, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t a0 = make_desc<16>(base), a1 = make_desc<16>(base + OFF_A1), b0 = make_desc<16>(base + OFF_B0), b1 = make_desc<16>(base + OFF_B1);
#pragma unroll
          for (int k = 0; k < 2; k++) {                      // 16 contraction indices = 32 bytes per instruction
            const uint64_t adv = (uint64_t)(2 * k);
            if constexpr (MERGED) {
              // small terms first, so that they meet the accumulator before the large term of this group is added
              tc_mma_f16(acc_main, a1 + adv, b0 + adv, idesc, (i > 0 || k > 0) ? 1u : 0u);
              tc_mma_f16(acc_main, a0 + adv, b1 + adv, idesc, 1u);
              tc_mma_f16(acc_main, a0 + adv, b0 + adv, idesc, 1u);
            } else {
              tc_mma_f16(acc_cross, a1 + adv, b0 + adv, idesc, (i > 0 || k > 0) ? 1u : 0u);
              tc_mma_f16(acc_cross, a0 + adv, b1 + adv, idesc, 1u);
              tc_mma_f16(acc_main, a0 + adv, b0 + adv, idesc, (i > 0 || k > 0) ? 1u : 0u);
            }
          }
          tc_commit(empty0 + 8 * s);
        }
        if (ok) tc_commit(tfull0 + 8 * slot);
      }
      if (!ok) {
        if (!*abort_flag) give_up(2);
        tc_commit(drain);                                   // own instructions in flight must finish before TMEM is released
        mbar_wait(drain, 0, TC_DRAIN_LIMIT);
      }
    }
  } else {
    const int quad = warp & 3, chalf = (warp - 2) >> 2; uint32_t lt = 0;
    float* colv = colv_all + (warp - 2) * BN;
    float* stg = colv_all + Cfg::COLV_FLOATS + (warp - 2) * 32 * TC_STG_LD;
    int tile, half;
    for (int w = 0; work(w, tile, half); w++) {
      int m0, n0, z, kb0, nkb; if (!decode(tile, half, m0, n0, z, kb0, nkb)) continue;
      const uint32_t slot = lt & 1, u = lt >> 1; lt++;
      const int bw = half < 0 ? BN : BN / 2;
      tc_epilogue_stage<BN>(ep, n0, z, chalf, lane, bw, colv);
      int ok = 1;
      if (lane == 0) ok = mbar_wait(tfull0 + 8 * slot, u & 1, limit, abort_flag) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { if (lane == 0 && !*abort_flag) give_up(3); break; }
      tc_fence_after();
      tc_epilogue_tile<BN, MERGED>(ep, tmem_base, slot * SLOT_COLS, slot * SLOT_COLS + BN, m0, n0, z, quad, chalf, lane, nkb, bw, colv, stg);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * slot);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0 && *abort_flag) {
    // a wait gave up somewhere in this CTA: the producer's last copies may still be in flight and nobody consumes
    // them any more; the CTA must not exit (and hand its shared memory on) before they have landed
    const uint32_t n_back = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
    for (uint32_t j = issued - n_back; j < issued; j++) mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1, TC_DRAIN_LIMIT);
  }
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
}

// ------------------------------------------------------------------ operand split (memory-bound)
// Batched, strided split: planes[z][r][c] (row stride ldp, c < ldp, zero beyond cols) of the source element
// (z, r, c) at p + (z / batch2) * b1 + (z % batch2) * b2 + r * s_r + c * s_c.  One of s_r, s_c is 1:
// s_c == 1 reads rows directly; s_r == 1 (the operand is the transpose of what is stored) goes through a shared tile.
// Two fp16 planes per operand, p0 = fp16(x s), p1 = fp16(x s - p0), and the inverse 1/s of every plane row's scale.
struct TcSrc { const float* p; long s_r, s_c, b1, b2; int batch2; };
// One warp per plane row: first the row's largest magnitude (the row is read a second time from L1 / L2 afterwards),
// then eight elements per lane and step (two 16-byte loads, one 16-byte store per plane).  blockIdx.y = problem index.
// `rownorm` (may be null): receives the L2 norm of every row (a factor of the bound of a plane-output contraction).
__global__ void __launch_bounds__(256) split2_rows_kernel(TcSrc s, int rows, int cols, __half* __restrict__ p0, __half* __restrict__ p1, float* __restrict__ inv_scale, int ldp,
                                                          float* __restrict__ rownorm) {
  const int z = blockIdx.y, lane = threadIdx.x & 31;
  const long r = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  const float* src = s.p + (z / s.batch2) * s.b1 + (z % s.batch2) * s.b2 + r * s.s_r;
  const bool vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  const int cols8 = vec ? (cols & ~7) : 0;                  // columns handled with 16-byte loads
  float mx = 0.f, sq = 0.f;
  for (int c = lane * 8; c < cols8; c += 256) {
    const float4 a = *reinterpret_cast<const float4*>(src + c), b = *reinterpret_cast<const float4*>(src + c + 4);
    mx = fmaxf(mx, fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))), fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w)))));
    sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
  }
  for (int c = cols8 + lane; c < cols; c += 32) { const float v = src[c]; mx = fmaxf(mx, fabsf(v)); sq += v * v; }
  mx = warp_max(mx);
  if (rownorm) { sq = warp_sum(sq); if (lane == 0) rownorm[(long)z * rows + r] = sqrtf(sq) * 1.0001f; }
  float inv; const float sc = row_scale(mx, &inv);
  if (lane == 0) inv_scale[(long)z * rows + r] = inv;
  const long o = ((long)z * rows + r) * ldp;
  for (int c = lane * 8; c < ldp; c += 256) {
    float t[8];
    if (c + 7 < cols8) {
      const float4 a = *reinterpret_cast<const float4*>(src + c), b = *reinterpret_cast<const float4*>(src + c + 4);
      t[0] = a.x; t[1] = a.y; t[2] = a.z; t[3] = a.w; t[4] = b.x; t[5] = b.y; t[6] = b.z; t[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) t[j] = c + j < cols ? src[c + j] : 0.f;
    }
    uint4 a, b;
    split2_pair(t[0], t[1], sc, a.x, b.x); split2_pair(t[2], t[3], sc, a.y, b.y);
    split2_pair(t[4], t[5], sc, a.z, b.z); split2_pair(t[6], t[7], sc, a.w, b.w);
    *reinterpret_cast<uint4*>(p0 + o + c) = a;
    *reinterpret_cast<uint4*>(p1 + o + c) = b;
  }
}
// Largest magnitude of every plane row of a transposed operand (= of every column of the stored matrix): a block covers
// 64 plane rows x 256 contraction indices, reads run along the stored matrix's fast index, one atomicMax per row and block
// on the bit pattern (non-negative floats order like integers).  `mx` must be zero on entry.
__global__ void __launch_bounds__(256) colmax_kernel(TcSrc s, int rows, int cols, int* __restrict__ mx) {
  __shared__ float red[4][64];
  const int z = blockIdx.z, r = blockIdx.x * 64 + (threadIdx.x & 63), cy = threadIdx.x >> 6;
  const float* src = s.p + (z / s.batch2) * s.b1 + (z % s.batch2) * s.b2;
  float m = 0.f;
  if (r < rows) for (int c = blockIdx.y * 256 + cy; c < min(cols, (int)(blockIdx.y + 1) * 256); c += 4) m = fmaxf(m, fabsf(src[r + (long)c * s.s_c]));
  red[cy][threadIdx.x & 63] = m;
  __syncthreads();
  if (threadIdx.x < 64 && r < rows) {
    m = fmaxf(fmaxf(red[0][threadIdx.x], red[1][threadIdx.x]), fmaxf(red[2][threadIdx.x], red[3][threadIdx.x]));
    if (!(m <= 3.0e38f)) m = 3.4e38f;                       // an infinity or a NaN in the column: row_scale() then uses s = 1
    atomicMax(mx + (long)z * rows + r, __float_as_int(m));
  }
}
// Transposing split: 64 x 64 source tile through shared memory; reads run along the source's fast index (r), each
// thread then writes two neighbouring contraction indices of one plane row as one 4-byte word.  `mx` = colmax_kernel's result.
__global__ void __launch_bounds__(256) split2_cols_kernel(TcSrc s, int rows, int cols, __half* __restrict__ p0, __half* __restrict__ p1, const int* __restrict__ mx,
                                                          float* __restrict__ inv_scale, int ldp) {
  __shared__ float t[64][65];
  const int z = blockIdx.z, c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const float* src = s.p + (z / s.batch2) * s.b1 + (z % s.batch2) * s.b2;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int j = ty; j < 64; j += 4) { const int c = c0 + j, r = r0 + tx; t[j][tx] = (r < rows && c < cols) ? src[r + (long)c * s.s_c] : 0.f; }
  __syncthreads();
  const long zo = (long)z * rows * ldp;
  const int cx = (threadIdx.x & 31) * 2, ry = threadIdx.x >> 5;
  for (int j = ry; j < 64; j += 8) {
    const int r = r0 + j, c = c0 + cx;
    if (r < rows && c < ldp) {
      float inv; const float sc = row_scale(__int_as_float(mx[(long)z * rows + r]), &inv);
      if (c == 0) inv_scale[(long)z * rows + r] = inv;
      uint32_t a, b; split2_pair(t[cx][j], t[cx + 1][j], sc, a, b);
      const long o = zo + (long)r * ldp + c;
      *reinterpret_cast<uint32_t*>(p0 + o) = a; *reinterpret_cast<uint32_t*>(p1 + o) = b;
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Operand planes of the contraction engine: two fp16 planes [nbatch][rows][ldp] in one buffer, plane 1 after plane 0, and
// the inverse scale of every plane row [nbatch][rows].
struct BfPlanes {
  __half* base; float* inv_scale; int rows, K, ldp, nbatch; int koff = 0;
  size_t plane_elems() const { return (size_t)nbatch * rows * ldp; }
  __half* p0() const { return base; }
  __half* p1() const { return base + plane_elems(); }
};
// Where a contraction's result goes when it is only ever used as the A operand of another contraction (the FFN's hidden
// activation and its gradient: half of all operand elements of a TransformerBlock).  A row's scale must be known before
// its first element is written, and a tile sees only 256 of the row's columns, so the scale comes from a bound instead of
// the row's maximum: |sum_k a_k b_k + bias| <= sqrt(|a|^2 + 1) * sqrt(K + 1) * max(|B|, |bias|) (Cauchy-Schwarz).  For
// random-sign data the bound is about 8-16 times the row's actual maximum, i.e. 3-4 of the planes' 22 bits; it can never
// be exceeded, so the fp16 planes cannot overflow.  `last`: fp32 copy of every sequence's last row (the only rows of
// these tensors that are read as numbers: ReLU gate and weight-gradient input of the reference's last-token rule).
struct TcPlaneOut { BfPlanes planes; const int* b_maxabs; float* last; int last_T; float* rowsum32 = nullptr; };
inline int tc_ldp(int K) { return ((K + 7) / 8) * 8; }              // plane row stride: a multiple of 16 bytes for TMA
inline size_t bf_plane_floats(long nbatch, long rows, long ldp) { return (size_t)nbatch * rows * ldp; }   // two fp16 planes = one float per element

// Per-context operand-plane scratch of the contraction engine (calls on a context are serialised by Ctx::run_mu).
struct TcScratch { DevBuf a, b, sa, sb, mx; const float* last_a = nullptr; int last_m = 0, last_k = 0; long last_ld = 0; };
inline TcScratch& tc_scratch(Ctx* ctx) { if (!ctx->tc_scratch) ctx->tc_scratch = ctx->own(new TcScratch()); return *static_cast<TcScratch*>(ctx->tc_scratch); }

// Operand planes for `nbatch` problems of rows x K in the context's scratch (which = 0: A side, 1: B side).
inline int tc_planes(Ctx* ctx, int which, long nbatch, long rows, int K, BfPlanes* out) {
  TcScratch& sc = tc_scratch(ctx);
  const int ldp = tc_ldp(K); const size_t n = bf_plane_floats(nbatch, rows, ldp), ns = (size_t)nbatch * rows;
  if (rows > 0x7fffffffL || nbatch > 65535) return fail(GN_ERR_UNSUPPORTED, "tc_planes: operand too large");
  DevBuf& pl = which == 0 ? sc.a : sc.b; DevBuf& scl = which == 0 ? sc.sa : sc.sb;
  if (pl.n < n) { GN_CUDA(cudaStreamSynchronize(ctx->stream)); GN_TRY(pl.alloc(n)); }
  if (scl.n < ns) { GN_CUDA(cudaStreamSynchronize(ctx->stream)); GN_TRY(scl.alloc(ns + 1024)); }
  if (sc.mx.n < ns) { GN_CUDA(cudaStreamSynchronize(ctx->stream)); GN_TRY(sc.mx.alloc(ns + 1024)); }
  if (which == 0) sc.last_a = nullptr;
  *out = BfPlanes{reinterpret_cast<__half*>(pl.p), scl.p, (int)rows, K, ldp, (int)nbatch}; return GN_OK;
}
inline int* tc_rowmax_buf(Ctx* ctx) { return reinterpret_cast<int*>(tc_scratch(ctx).mx.p); }

template <int BN> inline bool tc_set_smem() { return cudaFuncSetAttribute(gemm_tc_persist_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<BN>::SMEM_BYTES) == cudaSuccess; }
inline void tc_init(Ctx* ctx) {
  ctx->tc_ok = false;
  void* fn = nullptr; cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess) { cudaGetLastError(); return; }
  if (!(tc_set_smem<64>() && tc_set_smem<128>() && tc_set_smem<256>())) { cudaGetLastError(); return; }
  ctx->encode_tiled = fn; ctx->tc_ok = true;
  if (const char* e = getenv("GONEURON_CUDA_TC_BN")) ctx->tc_force_bn = atoi(e);
  if (const char* e = getenv("GONEURON_CUDA_TC_KSLICE")) ctx->tc_kslice = atoi(e);
  if (const char* e = getenv("GONEURON_CUDA_TC_TAIL_SPLIT")) ctx->tc_tail_split = atoi(e) != 0;
  if (const char* e = getenv("GONEURON_CUDA_TC_TILE_QUEUE")) ctx->tc_tile_queue = atoi(e) != 0;
  if (!ctx->tc_queue_pool) {
    // (cleared on the legacy stream, which the context's non-blocking stream does not wait for: hence the device-wide wait)
    if (cudaMalloc(&ctx->tc_queue_pool, TC_QUEUE_POOL * sizeof(int)) != cudaSuccess || cudaMemset(ctx->tc_queue_pool, 0, TC_QUEUE_POOL * sizeof(int)) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess) {
      cudaGetLastError(); ctx->tc_queue_pool = nullptr; ctx->tc_tile_queue = false;
    }
  }
}

// 16-bit plane [nbatch][rows][ldp], K valid columns from column koff, box_cols columns x box_rows per copy: 32 columns = 64
// bytes with the 64-byte swizzle (contraction engine), 64 columns = 128 bytes with the 128-byte swizzle (attention tiles)
inline int tc_make_map_bf16_raw(Ctx* ctx, CUtensorMap* map, const void* base_v, int K, int rows, int ldp, int nbatch, int koff, int box_rows, int box_cols,
                                CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) {
  const uint16_t* base = static_cast<const uint16_t*>(base_v);
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)nbatch};
  cuuint64_t strides[2] = {(cuuint64_t)ldp * 2, (cuuint64_t)rows * ldp * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = ((PFN_encodeTiled)ctx->encode_tiled)(map, dtype, 3, (void*)(base + koff), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                    box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GN_ERR_CUDA, "cuTensorMapEncodeTiled (16-bit) failed with %d (rows %d K %d ld %d batch %d)", (int)r, rows, K, ldp, nbatch);
  return GN_OK;
}

// Writes the planes and inverse row scales of an operand.  `mx` (only used by the transposing variant): nbatch * rows ints.
inline int tc_split(Ctx* ctx, const TcSrc& src, const BfPlanes& p, int* mx, float* rownorm = nullptr) {
  if (rownorm && src.s_c != 1) return fail(GN_ERR_UNSUPPORTED, "tc_split: row norms are only formed by the row-wise split");
  if (src.s_c == 1) {
    if (p.nbatch > 65535) return fail(GN_ERR_UNSUPPORTED, "tc_split: more than 65535 problems in a batch");
    GN_LAUNCH(ctx, split2_rows_kernel, dim3(cdiv(p.rows, 8), p.nbatch), 256, 0, src, p.rows, p.K, p.p0(), p.p1(), p.inv_scale, p.ldp, rownorm);
  } else if (src.s_r == 1) {
    if (p.nbatch > 65535 || cdiv(p.rows, 64) > 65535 || cdiv(p.K, 256) > 65535) return fail(GN_ERR_UNSUPPORTED, "tc_split: operand too large for the transposing split");
    if (!mx) return fail(GN_ERR_INVALID_ARG, "tc_split: the transposing split needs a row-maximum buffer");
    GN_CUDA(cudaMemsetAsync(mx, 0, (size_t)p.nbatch * p.rows * sizeof(int), ctx->stream));
    GN_LAUNCH(ctx, colmax_kernel, dim3(cdiv(p.rows, 64), cdiv(p.K, 256), p.nbatch), 256, 0, src, p.rows, p.K, mx);
    GN_LAUNCH(ctx, split2_cols_kernel, dim3(cdiv(p.ldp, 64), cdiv(p.rows, 64), p.nbatch), 256, 0, src, p.rows, p.K, p.p0(), p.p1(), (const int*)mx, p.inv_scale, p.ldp);
  } else return fail(GN_ERR_UNSUPPORTED, "tc_split: neither stride of the operand is 1");
  ctx->split_bytes += 8.0 * (double)p.nbatch * p.rows * p.K;
  return check_launch("tc_split");
}

// SMs a persistent kernel spreads over.  With several ranks the gradient all-reduces run beside the backward pass; a
// persistent kernel that waits for the SMs their CTAs hold takes as long as the collective, so it leaves them some.
inline int persist_sms(const Ctx* ctx) { return std::max(1, ctx->sm_count - ctx->sm_reserve); }
// Number of left-over tiles of the last round that are run as two half tiles each (0: none): only when they would keep at
// most half of the CTAs busy, and not for the triangular products (their tiles differ in length anyway).
inline long tc_tail_halves(Ctx* ctx, long total_tiles, int bn, int flags) {
  if (!ctx->tc_tail_split || bn < 128 || total_tiles <= persist_sms(ctx) || (flags & (GEMM_SKIP_UPPER | GEMM_KBEG_AT_M0 | GEMM_KEND_AT_M0))) return 0;
  const long left = total_tiles % persist_sms(ctx);
  return 2 * left <= persist_sms(ctx) ? left : 0;
}
// A zeroed counter for one launch's tile queue, from a pool that is cleared when it has been used up (in stream order, so
// every earlier launch has finished with its counter by then).
inline int tc_next_queue(Ctx* ctx, int** out) {
  if (!ctx->tc_queue_pool) return fail(GN_ERR_CUDA, "tile-queue pool missing");
  if (ctx->tc_queue_used >= TC_QUEUE_POOL) { GN_CUDA(cudaMemsetAsync(ctx->tc_queue_pool, 0, TC_QUEUE_POOL * sizeof(int), ctx->stream)); ctx->tc_queue_used = 0; }
  *out = ctx->tc_queue_pool + ctx->tc_queue_used++; return GN_OK;
}
template <int BN>
inline int tc_launch_persist(Ctx* ctx, const BfPlanes& A, const BfPlanes& B, const TcParams& ep) {
  CUtensorMap mA0, mA1, mB0, mB1;
  constexpr CUtensorMapDataType F16 = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  GN_TRY(tc_make_map_bf16_raw(ctx, &mA0, A.p0(), A.K, A.rows, A.ldp, A.nbatch, A.koff, TC_BM, TC_BK, F16)); GN_TRY(tc_make_map_bf16_raw(ctx, &mA1, A.p1(), A.K, A.rows, A.ldp, A.nbatch, A.koff, TC_BM, TC_BK, F16));
  // the B tile of a stage arrives as two copies of BN / 2 rows, so that a half tile (see the kernel's work list) is one of them
  GN_TRY(tc_make_map_bf16_raw(ctx, &mB0, B.p0(), B.K, B.rows, B.ldp, B.nbatch, B.koff, BN / 2, TC_BK, F16)); GN_TRY(tc_make_map_bf16_raw(ctx, &mB1, B.p1(), B.K, B.rows, B.ldp, B.nbatch, B.koff, BN / 2, TC_BK, F16));
  const int tiles_m = cdiv(ep.M, TC_BM), tiles_n = cdiv(ep.N, BN); const long total = (long)tiles_m * tiles_n * A.nbatch;
  if (total > 0x7fffffffL) return fail(GN_ERR_UNSUPPORTED, "too many output tiles");
  const unsigned grid = (unsigned)std::min<long>(total, persist_sms(ctx));
  const long left = tc_tail_halves(ctx, total, BN, ep.flags);
  const int full_end = (int)(total - left), n_half = (int)(2 * left);
  int* queue = nullptr;
  if (ctx->tc_tile_queue && total > grid) GN_TRY(tc_next_queue(ctx, &queue));
  ProfScope prof(ctx);
  GN_LAUNCH(ctx, (gemm_tc_persist_kernel<BN>), grid, TC_THREADS, (TcCfg<BN>::SMEM_BYTES), mA0, mA1, mB0, mB1, ep, tiles_m, tiles_n, (int)total, full_end, n_half, queue);
  return check_launch("gemm_tc_persist");
}
// Output tile width for a problem: 64 for narrow outputs; 256 (three quarters of the shared-memory traffic per MMA
// cycle of the 128-wide tile) when the problem still fills the SMs evenly with tiles of that size.
inline int tc_pick_bn(Ctx* ctx, int M, int N, long nbatch, int flags) {
  if (ctx->tc_force_bn == 64 || ctx->tc_force_bn == 128 || ctx->tc_force_bn == 256) return ctx->tc_force_bn;
  if (N <= 64) return 64;
  if (N <= 128 || (flags & (GEMM_SKIP_UPPER | GEMM_KBEG_AT_M0 | GEMM_KEND_AT_M0))) return 128;
  auto cost = [&](int bn, double rate) {
    const long tiles = (long)cdiv(M, TC_BM) * cdiv(N, bn) * nbatch;
    double waves = std::ceil((double)tiles / persist_sms(ctx));
    if (tc_tail_halves(ctx, tiles, bn, flags) > 0) waves -= 0.38;       // a half tile costs about 0.62 of a whole one
    return waves * bn / rate;
  };
  return cost(256, 1.3) < cost(128, 1.0) ? 256 : 128;
}
// C[z] = A[z] * B[z]^T from prepared planes, one accumulator run over the whole contraction.
inline int tc_launch(Ctx* ctx, const BfPlanes& A, const BfPlanes& B, const TcParams& ep_in, int bn) {
  if (!ctx->tc_ok) return fail(GN_ERR_UNSUPPORTED, "tcgen05 engine unavailable");
  TcParams ep = ep_in; ep.spin_limit = ctx->spin_limit; ep.isa = A.inv_scale; ep.isb = B.inv_scale;
  if (A.K != B.K || A.nbatch != B.nbatch || A.rows != ep.M || B.rows != ep.N || A.K != ep.K) return fail(GN_ERR_INVALID_ARG, "tc_launch: operand shapes disagree");
  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  bool vec = ep.N % 4 == 0 && ep.ldc % 4 == 0 && ep.c_b1 % 4 == 0 && ep.c_b2 % 4 == 0 && a16(ep.C) && (!ep.bias || a16(ep.bias)) && a16(ep.isb);
  if (ep.R) vec = vec && ep.ldr % 4 == 0 && ep.r_b1 % 4 == 0 && ep.r_b2 % 4 == 0 && a16(ep.R);
  if (ep.mask) vec = vec && ep.mask_ld % 4 == 0 && a16(ep.mask);
  if (ep.nchw_P > 0) { if (ep.R || A.nbatch != 1) return fail(GN_ERR_UNSUPPORTED, "tc_launch: NCHW store with a residual or a batch"); vec = false; }
  if (ep.out_p0) {
    if (!(ep.N % 4 == 0 && (!ep.bias || a16(ep.bias)) && a16(ep.isb) && (!ep.mask || (ep.mask_ld % 4 == 0 && a16(ep.mask))) && ep.out_ldp % 4 == 0 && (!ep.c_last || a16(ep.c_last))))
      return fail(GN_ERR_INVALID_ARG, "tc_launch: plane output needs 16-byte aligned operands");
    vec = true;
  }
  if (vec) ep.flags |= TC_FLAG_VEC;
  {
    double by = 4.0 * ((double)ep.M + ep.N) * ep.K + 4.0 * (double)ep.M * ep.N * (ep.R ? 2 : 1);
    if (ep.flags & (GEMM_SKIP_UPPER | GEMM_KBEG_AT_M0 | GEMM_KEND_AT_M0)) by *= 0.5;
    ctx->gemm_bytes += by * A.nbatch;
  }
  if (bn == 64) return tc_launch_persist<64>(ctx, A, B, ep);
  if (bn == 256) return tc_launch_persist<256>(ctx, A, B, ep);
  return tc_launch_persist<128>(ctx, A, B, ep);
}
// The tensor core truncates when it adds a product group to the accumulator, so the error of one accumulator run grows
// with the number of MMA instructions that feed it (one per 16 contraction indices and term).  Long contractions (weight
// gradients over all tokens of a batch) are therefore cut into slices, each slice adding its result to C through the
// epilogue's residual path, i.e. in properly rounded fp32: 4096 indices per run with separate accumulators for the
// large and the small terms, 2048 with the single accumulator of the 256-wide tile.
inline int tc_run_rows(Ctx* ctx, const BfPlanes& A, const BfPlanes& B, const TcParams& ep, int bn) {
  const int kslice = ctx->tc_kslice > 0 ? ctx->tc_kslice : (bn == 256 ? 2048 : 4096);
  if (ep.K <= kslice || (ep.flags & (GEMM_KBEG_AT_M0 | GEMM_KEND_AT_M0))) return tc_launch(ctx, A, B, ep, bn);
  if (ep.out_p0) return fail(GN_ERR_UNSUPPORTED, "a contraction that writes operand planes must fit one accumulator run (K = %d)", ep.K);
  for (int k0 = 0; k0 < ep.K; k0 += kslice) {
    const int kl = std::min(kslice, ep.K - k0); const bool first = k0 == 0, last = k0 + kl >= ep.K;
    BfPlanes As = A, Bs = B; As.koff = A.koff + k0; As.K = kl; Bs.koff = B.koff + k0; Bs.K = kl;
    TcParams es = ep; es.K = kl;
    if (!first) { es.bias = nullptr; es.R = ep.C; es.ldr = ep.ldc; es.r_b1 = ep.c_b1; es.r_b2 = ep.c_b2; }
    if (!last) { es.act = GN_ACT_LINEAR; es.mask = nullptr; }
    GN_TRY(tc_launch(ctx, As, Bs, es, bn));
  }
  return GN_OK;
}
inline int tc_run(Ctx* ctx, const BfPlanes& A, const BfPlanes& B, const TcParams& ep) {
  // (Running the rows of a short last wave as a second launch with 128-wide tiles was measured at 16 384 rows: the second
  // launch's fixed cost ate the 9 % it should have saved, so every product is one tiling.)
  return tc_run_rows(ctx, A, B, ep, tc_pick_bn(ctx, ep.M, ep.N, A.nbatch, ep.flags));
}

// ------------------------------------------------------------------ prepared planes of weight matrices
// A weight matrix W [out, in] is an operand twice per training step: as stored (rows = out, contraction over in) in the
// forward product X W^T, and transposed (rows = in, contraction over out) in the input-gradient product dZ W.  Splitting it
// at each use costs two small launches per orientation and matrix, work that does not shrink when the batch is sharded over
// GPUs.  Instead all registered matrices are split once per parameter update, both orientations from one read, by two
// launches in all: the matrices get ONE power-of-two scale each (their entries are of similar size, unlike activation
// rows), found by wplanes_max_kernel, and wplanes_split_kernel writes every 64 x 64 tile as stored and transposed.
struct WPlaneJob { const float* src; const float* bias; int out, in, ldp_r, ldp_c; __half *r0, *r1, *c0, *c1; float *inv_r, *inv_c; int tile0, tiles_in; };
__device__ __forceinline__ int wplane_find(const WPlaneJob* jobs, int njobs, int tile) {
  int lo = 0, hi = njobs - 1;
  while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (jobs[mid].tile0 <= tile) lo = mid; else hi = mid - 1; }
  return lo;
}
__global__ void __launch_bounds__(256) wplanes_max_kernel(const WPlaneJob* __restrict__ jobs, int njobs, int* __restrict__ mx, int tile_off) {
  __shared__ float red[33];
  const int tile = blockIdx.x + tile_off;
  const int j = wplane_find(jobs, njobs, tile); const WPlaneJob jb = jobs[j];
  const int t = tile - jb.tile0, r0 = (t / jb.tiles_in) * 64, c0 = (t % jb.tiles_in) * 64;
  float m = 0.f;
  for (int e = threadIdx.x; e < 4096; e += 256) { const int r = r0 + (e >> 6), c = c0 + (e & 63); if (r < jb.out && c < jb.in) m = fmaxf(m, fabsf(jb.src[(long)r * jb.in + c])); }
  if (jb.bias && c0 == 0 && threadIdx.x < 64 && r0 + (int)threadIdx.x < jb.out) m = fmaxf(m, fabsf(jb.bias[r0 + threadIdx.x]));      // the layer's biases count towards the maximum (bounds of plane-output contractions)
  m = block_max(m, red);
  if (threadIdx.x == 0) { if (!(m <= 3.0e38f)) m = 3.4e38f; atomicMax(mx + j, __float_as_int(m)); }
}
__global__ void __launch_bounds__(256) wplanes_split_kernel(const WPlaneJob* __restrict__ jobs, int njobs, const int* __restrict__ mx, int tile_off) {
  __shared__ float tl[64][65];
  const int tile = blockIdx.x + tile_off;
  const int j = wplane_find(jobs, njobs, tile); const WPlaneJob jb = jobs[j];
  const int t = tile - jb.tile0, r0 = (t / jb.tiles_in) * 64, c0 = (t % jb.tiles_in) * 64;
  float inv; const float sc = row_scale(__int_as_float(mx[j]), &inv);
  for (int e = threadIdx.x; e < 4096; e += 256) { const int rr = e >> 6, cc = e & 63; const int r = r0 + rr, c = c0 + cc; tl[rr][cc] = (r < jb.out && c < jb.in) ? jb.src[(long)r * jb.in + c] : 0.f; }
  __syncthreads();
  const int x2 = (threadIdx.x & 31) * 2, y = threadIdx.x >> 5;
  for (int rr = y; rr < 64; rr += 8) {                        // as stored: plane row = out index, two neighbouring in indices per thread
    const int r = r0 + rr, c = c0 + x2;
    if (r < jb.out && c < jb.in) {                            // (in is even-padded by ldp_r; an odd last column writes its zero neighbour)
      uint32_t a, b; split2_pair(tl[rr][x2], tl[rr][x2 + 1], sc, a, b);
      const long o = (long)r * jb.ldp_r + c;
      *reinterpret_cast<uint32_t*>(jb.r0 + o) = a; *reinterpret_cast<uint32_t*>(jb.r1 + o) = b;
    }
    if (c0 == 0 && x2 == 0 && r < jb.out) jb.inv_r[r] = inv;
  }
  for (int cc = y; cc < 64; cc += 8) {                        // transposed: plane row = in index, two neighbouring out indices per thread
    const int c = c0 + cc, r = r0 + x2;
    if (c < jb.in && r < jb.out) {
      uint32_t a, b; split2_pair(tl[x2][cc], tl[x2 + 1][cc], sc, a, b);
      const long o = (long)c * jb.ldp_c + r;
      *reinterpret_cast<uint32_t*>(jb.c0 + o) = a; *reinterpret_cast<uint32_t*>(jb.c1 + o) = b;
    }
    if (r0 == 0 && x2 == 0 && c < jb.in) jb.inv_c[c] = inv;
  }
}
// Host side of the table: one entry per registered matrix, looked up by the matrix's device address.
struct WeightPlaneEntry { const float* src; int out, in; BfPlanes rows, cols; const float* bias = nullptr; const int* maxabs = nullptr; int layer = -1; int tile0 = 0, tiles = 0; };
struct WeightPlaneTable {
  std::vector<WeightPlaneEntry> e; DevBuf planes, scales, mx, jobs; int total_tiles = 0; bool dirty = true;
  // entries [j0, j1) that belong to model layer `layer` (they are registered layer by layer, so the range is contiguous)
  void layer_range(int layer, int* j0, int* j1) const {
    *j0 = *j1 = 0; bool in = false;
    for (int j = 0; j < (int)e.size(); j++) if (e[j].layer == layer) { if (!in) { *j0 = j; in = true; } *j1 = j + 1; }
  }
  const WeightPlaneEntry* find(const float* p) const { for (auto& x : e) if (x.src == p) return &x; return nullptr; }
};
// Lays the table out for the matrices (src, out, in) and allocates its buffers (planes zeroed once: the padding columns
// of a plane row are never written afterwards and must read as zero).
inline int wplanes_build(Ctx* ctx, WeightPlaneTable& t, const std::vector<WeightPlaneEntry>& mats) {
  t.e = mats; size_t halves = 0, nscale = 0; int tiles = 0; std::vector<WPlaneJob> jobs;
  for (auto& x : t.e) {
    const int lr = tc_ldp(x.in), lc = tc_ldp(x.out);
    halves += 2 * ((size_t)x.out * lr + (size_t)x.in * lc); nscale += (size_t)x.out + x.in + 8;
  }
  if (t.e.empty()) return GN_OK;
  GN_TRY(t.planes.alloc(halves / 2 + 64)); GN_TRY(t.scales.alloc(nscale)); GN_TRY(t.mx.alloc(t.e.size() + 4));
  GN_CUDA(cudaMemsetAsync(t.planes.p, 0, (halves / 2 + 64) * 4, ctx->stream));
  __half* hp = reinterpret_cast<__half*>(t.planes.p); float* sp = t.scales.p;
  for (auto& x : t.e) {
    const int lr = tc_ldp(x.in), lc = tc_ldp(x.out);
    x.rows = BfPlanes{hp, sp, x.out, x.in, lr, 1}; hp += 2 * (size_t)x.out * lr; sp += (x.out + 3) & ~3;
    x.cols = BfPlanes{hp, sp, x.in, x.out, lc, 1}; hp += 2 * (size_t)x.in * lc; sp += (x.in + 3) & ~3;
    x.maxabs = reinterpret_cast<const int*>(t.mx.p) + jobs.size();
    WPlaneJob jb{x.src, x.bias, x.out, x.in, lr, lc, x.rows.p0(), x.rows.p1(), x.cols.p0(), x.cols.p1(), x.rows.inv_scale, x.cols.inv_scale, tiles, (int)cdiv(x.in, 64)};
    x.tile0 = tiles; x.tiles = (int)cdiv(x.out, 64) * (int)cdiv(x.in, 64);
    tiles += x.tiles; jobs.push_back(jb);
  }
  t.total_tiles = tiles;
  GN_TRY(t.jobs.alloc((jobs.size() * sizeof(WPlaneJob) + 3) / 4));
  GN_CUDA(copy_h2d(ctx, t.jobs.p, jobs.data(), jobs.size() * sizeof(WPlaneJob)));
  t.dirty = true; return GN_OK;
}
// Re-splits every registered matrix if the parameters changed since the last call.
// Entries [j0, j1) only, on `stream`: used right behind a layer's parameter update when the update runs layer by layer.
inline int wplanes_refresh_range(Ctx* ctx, WeightPlaneTable& t, int j0, int j1, cudaStream_t stream) {
  if (j1 <= j0) return GN_OK;
  const int nj = (int)t.e.size(), tile_off = t.e[j0].tile0, ntiles = t.e[j1 - 1].tile0 + t.e[j1 - 1].tiles - tile_off;
  GN_CUDA(cudaMemsetAsync(reinterpret_cast<int*>(t.mx.p) + j0, 0, (size_t)(j1 - j0) * sizeof(int), stream));
  wplanes_max_kernel<<<ntiles, 256, 0, stream>>>(reinterpret_cast<const WPlaneJob*>(t.jobs.p), nj, reinterpret_cast<int*>(t.mx.p), tile_off);
  wplanes_split_kernel<<<ntiles, 256, 0, stream>>>(reinterpret_cast<const WPlaneJob*>(t.jobs.p), nj, reinterpret_cast<const int*>(t.mx.p), tile_off);
  ctx->launches += 2;
  double elems = 0; for (int j = j0; j < j1; j++) elems += (double)t.e[j].out * t.e[j].in;
  ctx->split_bytes += 16.0 * elems;                          // 4 B read twice, 8 B written
  return check_launch("wplanes_refresh");
}
inline int wplanes_refresh(Ctx* ctx, WeightPlaneTable& t) {
  if (t.e.empty() || !t.dirty) return GN_OK;
  GN_TRY(wplanes_refresh_range(ctx, t, 0, (int)t.e.size(), ctx->stream));
  t.dirty = false; return GN_OK;
}
// Prepared planes for B of this contraction, if B is a registered matrix used in one of its two orientations.
inline const BfPlanes* wplanes_lookup(Ctx* ctx, const GemmDesc& g, const WeightPlaneEntry** entry = nullptr) {
  const WeightPlaneTable* t = static_cast<const WeightPlaneTable*>(ctx->weight_planes);
  if (!t || t->dirty || g.batch1 * g.batch2 != 1) return nullptr;
  const WeightPlaneEntry* x = t->find(g.B); if (!x) return nullptr;
  if (entry) *entry = x;
  if (g.sb_k == 1 && g.sb_n == x->in && g.N == x->out && g.K == x->in) return &x->rows;     // B(k, n) = W[n, k]
  if (g.sb_n == 1 && g.sb_k == x->in && g.N == x->in && g.K == x->out) return &x->cols;     // B(k, n) = W[k, n]
  return nullptr;
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
  const int nb = g.batch1 * g.batch2;
  const float* last_a = sc.last_a; const float* pa = sc.a.p; const float* psa = sc.sa.p;   // tc_planes() forgets the A planes' origin when it hands the buffer out
  BfPlanes A, B; GN_TRY(tc_planes(ctx, 0, nb, g.M, g.K, &A)); GN_TRY(tc_planes(ctx, 1, nb, g.N, g.K, &B));
  int* mx = tc_rowmax_buf(ctx);
  sc.last_a = (sc.a.p == pa && sc.sa.p == psa) ? last_a : nullptr;                          // still valid unless a buffer was replaced
  if (g.a_planes) {
    A = *static_cast<const BfPlanes*>(g.a_planes);
    if (A.rows != g.M || A.K != g.K || A.nbatch != nb) return fail(GN_ERR_INVALID_ARG, "gemm_tc: prepared planes of A do not match the contraction");
  } else if (!g.a_rownorm && g.reuse_a_planes && nb == 1 && sc.last_a == g.A && sc.last_m == g.M && sc.last_k == g.K && sc.last_ld == g.sa_m && g.sa_k == 1) {
    // same tensor as the previous call (the Q, K and V projections share their input): planes still valid
  } else {
    GN_TRY(tc_split(ctx, TcSrc{g.A, g.sa_m, g.sa_k, g.a_b1, g.a_b2, g.batch2}, A, mx, g.a_rownorm));
    sc.last_a = (nb == 1 && g.sa_k == 1) ? g.A : nullptr; sc.last_m = g.M; sc.last_k = g.K; sc.last_ld = g.sa_m;
  }
  if (g.b_planes) {
    B = *static_cast<const BfPlanes*>(g.b_planes);
    if (B.rows != g.N || B.K != g.K || B.nbatch != nb) return fail(GN_ERR_INVALID_ARG, "gemm_tc: prepared planes of B do not match the contraction");
  } else GN_TRY(tc_split(ctx, TcSrc{g.B, g.sb_n, g.sb_k, g.b_b1, g.b_b2, g.batch2}, B, mx));
  TcParams ep{g.C, g.ldc, g.c_b1, g.c_b2, g.bias, g.R, g.ldr, g.r_b1, g.r_b2, g.act, g.M, g.N, g.K, g.batch2, g.flags, ctx->d_status, g.mask, g.mask_ld, g.mask_group};
  if (g.plane_out) {
    const TcPlaneOut& po = *static_cast<const TcPlaneOut*>(g.plane_out);
    if (nb != 1 || g.R || !g.a_rownorm || !po.b_maxabs || g.N % 32 || po.planes.rows != g.M || po.planes.K != g.N || (g.flags & (GEMM_SKIP_UPPER | GEMM_KBEG_AT_M0 | GEMM_KEND_AT_M0)))
      return fail(GN_ERR_INVALID_ARG, "gemm_tc: this contraction cannot write its result as operand planes");
    ep.out_p0 = po.planes.p0(); ep.out_p1 = po.planes.p1(); ep.out_inv = po.planes.inv_scale; ep.out_ldp = po.planes.ldp;
    ep.a_rownorm = g.a_rownorm; ep.b_maxabs = po.b_maxabs; ep.c_last = po.last; ep.last_T = po.last_T > 0 ? po.last_T : 1; ep.rowsum32 = po.rowsum32;
  }
  return tc_run(ctx, A, B, ep);
}

}  // namespace gn
