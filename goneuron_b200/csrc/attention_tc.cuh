// attention_tc.cuh -- multi-head attention (head size 64) on the tcgen05 tensor cores with the score tile, the
// probabilities and the output accumulator resident in tensor memory.
//
// reference: internal/layer/transformer.go:470-503 (forward) -- same arithmetic as attention.cuh: scores =
// q.k / sqrt(hd), masked entries removed, row softmax, weighted sum of v; row maximum and row sum kept per row.
//
// Operands: the split planes of gemm_tc.cuh's scheme (hi = tf32(x) as fp32, bf16(x), bf16(x - hi); every product is one
// TF32 MMA on hi x hi plus two BF16 MMAs for the cross terms), one problem per (batch, head):
//   Qp, Kp : [B*H][T][64]   (contraction over the head dimension is along the row)
//   Vt     : [B*H][64][T]   (transposed, so that the contraction over the keys is along the row as well)
// (attn_split_kernel writes both kinds from one read of the tensor)
// and fetched by TMA into 128-byte-swizzled tiles.  One tile = 128 query rows of one head; key blocks of 64.
//   warp 0    : TMA producer (Q once; K and Vt blocks through two stages each)
//   warp 1    : MMA issuer.  S_j = Q K_j^T (both operands in shared memory) into one of two 64-column TMEM buffers;
//               O += P_j V_j with P read from TMEM as the A operand and Vt_j from shared memory.
//   warps 2-9 : two threads per query row (TMEM lane = row, 32 of the 64 columns each): tcgen05.ld of S_j, running
//               maximum (exchanged through shared memory) and sum, p = exp(s - m), hi written over S_j in place and
//               bf16(p), bf16(p - hi) packed two per column into a second buffer (tcgen05.st); when a row maximum
//               moved, the output accumulator is rescaled in TMEM after the previous P V has completed.  One warp per
//               scheduler could not keep up with the tensor pipe (measured: 25 % tensor activity); two do.
// The issue order S_0, S_1, PV_0, S_2, PV_1, ... keeps the tensor pipe busy with S_{j+1} (and PV_{j-1}) while the
// softmax of block j runs.  Every wait is bounded; a wait that gives up sets the status word at once, which makes
// every other wait of the launch give up within a few polls (see WAIT below).
#pragma once
#include "attention.cuh"
#include "gemm_tc.cuh"

namespace gn {

constexpr int ATC_BQ = 128, ATC_BK = 64, ATC_HD = 64, ATC_THREADS = 320;
constexpr int ATC_Q_BYTES = 4 * ATC_BQ * 128;   // hi (two chunks of 32 floats) + bf16 copy + bf16 lo: 64 KB
constexpr int ATC_K_BYTES = 4 * ATC_BK * 128;   // 32 KB
constexpr int ATC_V_BYTES = 4 * ATC_HD * 128;   // 32 KB
constexpr int ATC_FWD_SMEM = ATC_Q_BYTES + 2 * (ATC_K_BYTES + ATC_V_BYTES) + 1024 + 256 + 2 * 256 * 4;
// TMEM columns: S / P_hi buffers [0,128), packed bf16 P | P_lo buffers [128,256), two output accumulators [256,384)
constexpr uint32_t ATC_COL_S = 0, ATC_COL_PLO = 128, ATC_COL_O = 256, ATC_TMEM_COLS = 512;

__device__ __forceinline__ void tc_mma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
                 "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
// 32 fp32 values -> hi (TF32, in place) and the packed bf16 pairs of the value and of value - hi (16 words each)
__device__ __forceinline__ void split_pack32(uint32_t (&v)[32], uint32_t (&xb)[16], uint32_t (&lob)[16]) {
#pragma unroll
  for (int e = 0; e < 16; e++) {
    const float a = __uint_as_float(v[2 * e]), b = __uint_as_float(v[2 * e + 1]);
    const uint32_t ha = v[2 * e] & 0xffffe000u, hb = v[2 * e + 1] & 0xffffe000u;
    xb[e] = pack_bf16(a, b); lob[e] = pack_bf16(a - __uint_as_float(ha), b - __uint_as_float(hb));
    v[2 * e] = ha; v[2 * e + 1] = hb;
  }
}
__device__ __forceinline__ float fast_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// one lane polls, the warp gets the verdict
__device__ __forceinline__ bool warp_mbar_wait(uint32_t bar, uint32_t parity, int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Tensor maps of a launch: three per operand (hi fp32 | bf16 copy | bf16 lo).
template <int N> struct AttnMaps { CUtensorMap m[N]; };

// Persistent: gridDim.x CTAs (one per SM) walk the tiles; tile id = blockIdx.x + i * gridDim.x names (batch*head, query
// block), the query block being rotated by i so that every CTA sees short and long causal tiles alike (gridDim.x is a
// multiple of the number of query blocks).  All counters below run across tiles, so the barriers' phases simply continue:
// the producer prefetches the next tile's Q as soon as the last score product of the current tile has completed, and
// the first score products of the next tile run while the elementwise warps finish the current tile and write it out
// (the output accumulator is double-buffered for that).
__global__ void __launch_bounds__(ATC_THREADS, 1)
attn_tc_fwd_kernel(const __grid_constant__ AttnMaps<9> maps, float* __restrict__ O, float* __restrict__ Mst, float* __restrict__ Lst, int T, int D, int H, int causal, float inv_scale,
                   int ntiles, int* status, unsigned spin_limit) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + ATC_Q_BYTES;                                   // two stages of ATC_K_BYTES
  uint8_t* sV = sK + 2 * ATC_K_BYTES;                                 // two stages of ATC_V_BYTES
  uint64_t* bars = (uint64_t*)(sV + 2 * ATC_V_BYTES);
  uint32_t* tmem_slot = (uint32_t*)(bars + 20);
  float* xch = (float*)(bars + 32);                                   // [2][2][128] row maxima / sums exchanged between the two threads of a row
  // barriers: 0 q_full | 1,2 k_full | 3,4 k_empty | 5,6 v_full | 7,8 v_empty | 9,10 s_full | 11,12 p_full | 13 pv_done
  //           14 q_empty | 15,16 o_free
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Bounded waits that fail fast: the first wait that gives up records its role in the status word at once, and every
  // later wait of every role and CTA (they all poll that word) gives up after at most 64 polls, so a launch whose pipeline
  // is stuck ends in milliseconds instead of polling each wait to its limit.  The copy and MMA threads stop issuing at
  // their first failed wait (arming a barrier whose previous phase has not completed is undefined), then let what
  // they have in flight finish.  The elementwise warps keep their loop structure (they meet at named barriers, so no
  // warp may leave early) and only touch tensor memory, count-256 barriers and in-range global rows; what they compute
  // after that point is discarded by the host (GN_ERR_TIMEOUT).
  const unsigned limit = spin_limit;
  auto WAIT = [&](uint32_t bar, uint32_t parity, int code) -> bool { if (mbar_wait(bar, parity, limit, status)) return true; atomicCAS(status, 0, code); return false; };
  auto WWAIT = [&](uint32_t bar, uint32_t parity, int code) -> bool { int w = 1; if (lane == 0) w = WAIT(bar, parity, code) ? 1 : 0; return __shfl_sync(0xffffffffu, w, 0) != 0; };
  const int ntq = T / ATC_BQ;
  // tile -> problem z, first query row, number of key blocks
  auto decode = [&](int id, int i, int& z, int& q0, int& nblk) {
    z = id / ntq; q0 = ((id % ntq + i) % ntq) * ATC_BQ;
    nblk = causal ? (q0 + ATC_BQ) / ATC_BK : T / ATC_BK;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 18; i++) mbar_init(BAR(i), (i == 11 || i == 12 || i == 15 || i == 16) ? 256 : 1);      // 17: drain
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(ATC_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, q0, nblk; decode(id, tt, z, q0, nblk);
        if (tt > 0 && !WAIT(BAR(14), (tt - 1) & 1, 11)) { ok = false; break; }
        mbar_expect_tx(BAR(0), ATC_Q_BYTES);
        for (int c = 0; c < 2; c++) tma_load_3d(smem_u32(sQ + c * 16384), &maps.m[0], c * 32, q0, z, BAR(0));
        tma_load_3d(smem_u32(sQ + 32768), &maps.m[1], 0, q0, z, BAR(0));
        tma_load_3d(smem_u32(sQ + 49152), &maps.m[2], 0, q0, z, BAR(0));
        for (int j = 0; j < nblk; j++, g++) {
          const uint32_t s = g & 1, u = g >> 1;
          if (u > 0 && !WAIT(BAR(3 + s), (u - 1) & 1, 11)) { ok = false; break; }
          mbar_expect_tx(BAR(1 + s), ATC_K_BYTES);
          for (int c = 0; c < 2; c++) tma_load_3d(smem_u32(sK + s * ATC_K_BYTES + c * 8192), &maps.m[3], c * 32, j * ATC_BK, z, BAR(1 + s));
          tma_load_3d(smem_u32(sK + s * ATC_K_BYTES + 16384), &maps.m[4], 0, j * ATC_BK, z, BAR(1 + s));
          tma_load_3d(smem_u32(sK + s * ATC_K_BYTES + 24576), &maps.m[5], 0, j * ATC_BK, z, BAR(1 + s));
          if (u > 0 && !WAIT(BAR(7 + s), (u - 1) & 1, 11)) { ok = false; break; }
          mbar_expect_tx(BAR(5 + s), ATC_V_BYTES);
          for (int c = 0; c < 2; c++) tma_load_3d(smem_u32(sV + s * ATC_V_BYTES + c * 8192), &maps.m[6], j * ATC_BK + c * 32, 0, z, BAR(5 + s));
          tma_load_3d(smem_u32(sV + s * ATC_V_BYTES + 16384), &maps.m[7], j * ATC_BK, 0, z, BAR(5 + s));
          tma_load_3d(smem_u32(sV + s * ATC_V_BYTES + 24576), &maps.m[8], j * ATC_BK, 0, z, BAR(5 + s));
        }
      }
      if (!ok || *(volatile int*)status) for (int i = 0; i < 200; i++) __nanosleep(1000);                 // own copies in flight land before the CTA exits
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true; uint32_t g0 = 0;
      constexpr uint32_t idesc = make_idesc(ATC_BQ, 64), idesc_bf = make_idesc_bf16(ATC_BQ, 64);
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, q0, nblk; decode(id, tt, z, q0, nblk);
        const uint32_t ob = tt & 1;
        auto issue_s = [&](int j) {
          const uint32_t g = g0 + j, s = g & 1, u = g >> 1;
          if (!ok || !WAIT(BAR(1 + s), u & 1, 12)) { ok = false; return; }
          tc_fence_after();
          const uint32_t acc = tmem_base + ATC_COL_S + s * 64;
          const uint32_t kb = smem_u32(sK + s * ATC_K_BYTES), qa = smem_u32(sQ);
#pragma unroll
          for (int k = 0; k < 4; k++) {                      // cross terms: bf16, 16 head columns per instruction
            const uint64_t adv = (uint64_t)(2 * k);
            tc_mma_bf16(acc, make_desc<32>(qa + 49152) + adv, make_desc<32>(kb + 16384) + adv, idesc_bf, k ? 1u : 0u);
            tc_mma_bf16(acc, make_desc<32>(qa + 32768) + adv, make_desc<32>(kb + 24576) + adv, idesc_bf, 1u);
          }
#pragma unroll
          for (int c = 0; c < 2; c++)
#pragma unroll
            for (int k = 0; k < 4; k++) {                    // main term: tf32, 8 head columns per instruction
              const uint64_t adv = (uint64_t)(2 * k);
              tc_mma_tf32(acc, make_desc<32>(qa + c * 16384) + adv, make_desc<32>(kb + c * 8192) + adv, idesc, 1u);
            }
          tc_commit(BAR(3 + s));
          tc_commit(BAR(9 + s));
          if (j == nblk - 1) tc_commit(BAR(14));             // Q may be replaced
        };
        auto issue_pv = [&](int j) {
          const uint32_t g = g0 + j, s = g & 1, u = g >> 1;
          if (!ok || !WAIT(BAR(11 + s), u & 1, 12) || !WAIT(BAR(5 + s), u & 1, 12)) { ok = false; return; }
          tc_fence_after();
          const uint32_t vb = smem_u32(sV + s * ATC_V_BYTES);
          const uint32_t ph = tmem_base + ATC_COL_S + s * 64, pl = tmem_base + ATC_COL_PLO + s * 64, acc = tmem_base + ATC_COL_O + ob * 64;
#pragma unroll
          for (int k = 0; k < 4; k++) {                      // cross terms: packed bf16 P (16 keys = 8 columns per instruction)
            const uint64_t adv = (uint64_t)(2 * k);
            tc_mma_bf16_ts(acc, pl + 32 + k * 8, make_desc<32>(vb + 16384) + adv, idesc_bf, (j | k) ? 1u : 0u);
            tc_mma_bf16_ts(acc, pl + k * 8, make_desc<32>(vb + 24576) + adv, idesc_bf, 1u);
          }
#pragma unroll
          for (int kk = 0; kk < 8; kk++) {                   // main term: tf32 P_hi (8 keys = 8 columns per instruction)
            const int c = kk >> 2; const uint64_t adv = (uint64_t)(2 * (kk & 3));
            tc_mma_tf32_ts(acc, ph + kk * 8, make_desc<32>(vb + c * 8192) + adv, idesc, 1u);
          }
          tc_commit(BAR(7 + s));
          tc_commit(BAR(13));
        };
        if (!WAIT(BAR(0), tt & 1, 12)) { ok = false; break; }
        if (tt >= 2 && !WAIT(BAR(15 + ob), ((tt >> 1) - 1) & 1, 12)) { ok = false; break; }     // this accumulator has been written out
        issue_s(0);
        if (nblk > 1) issue_s(1);
        for (int j = 0; j < nblk; j++) {
          issue_pv(j);
          if (j + 2 < nblk) issue_s(j + 2);
        }
        g0 += nblk;
      }
      if (!ok || *(volatile int*)status) { tc_commit(BAR(17)); mbar_wait(BAR(17), 0, TC_DRAIN_LIMIT); }     // own instructions in flight finish before TMEM is released
    }
  } else {
    // two threads per query row: `half` selects 32 of the 64 columns of a block (and of the accumulator)
    const int quad = warp & 3, half = (warp - 2) >> 2, row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + 32 * half;
    const uint32_t pk_base = tmem_base + ((uint32_t)(quad * 32) << 16) + 16 * half;     // packed bf16 planes: 16 columns per half
    const float cs = inv_scale * 1.44269504088896341f;      // scores -> log2 units
    bool ok = true; uint32_t g0 = 0, xc = 0;
    for (int id = blockIdx.x, tt = 0; id < ntiles; id += gridDim.x, tt++) {
      int z, q0, nblk; decode(id, tt, z, q0, nblk);
      const int qi = q0 + row; const uint32_t ob = tt & 1;
      float m_run = -INFINITY, l_part = 0.f;                // running maximum (scaled scores), this thread's part of the row sum
      for (int j = 0; j < nblk; j++) {
        const uint32_t g = g0 + j, s = g & 1, u = g >> 1; const int key0 = j * ATC_BK + 32 * half;
        ok &= WWAIT(BAR(9 + s), u & 1, 13);
        tc_fence_after();
        uint32_t a[32];
        tmem_ld32(lane_base + ATC_COL_S + s * 64, a);
        tmem_wait_ld();
        if (causal && j * ATC_BK + ATC_BK - 1 > q0) {       // the block reaches above the diagonal for some row of the tile
#pragma unroll
          for (int e = 0; e < 32; e++) if (key0 + e > qi) a[e] = __float_as_uint(-INFINITY);
        }
        float bm = -INFINITY;
#pragma unroll
        for (int e = 0; e < 32; e++) bm = fmaxf(bm, __uint_as_float(a[e]));
        float* xb = xch + (xc++ & 1) * 256;
        xb[half * 128 + row] = bm;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        bm = fmaxf(bm, xb[(half ^ 1) * 128 + row]);
        const float m_new = fmaxf(m_run, bm * inv_scale);
        const float corr = fast_ex2((m_run - m_new) * 1.44269504088896341f);
        const float mneg = -m_new * 1.44269504088896341f;
        float rs = 0.f;
#pragma unroll
        for (int e = 0; e < 32; e++) { const float p = fast_ex2(fmaf(__uint_as_float(a[e]), cs, mneg)); rs += p; a[e] = __float_as_uint(p); }
        uint32_t pb[16], plb[16];
        split_pack32(a, pb, plb);
        tmem_st32(lane_base + ATC_COL_S + s * 64, a);                                // P_hi over S, 32-bit columns
        tmem_st16(pk_base + ATC_COL_PLO + s * 64, pb);                               // bf16(P), two keys per column
        tmem_st16(pk_base + ATC_COL_PLO + s * 64 + 32, plb);                         // bf16(P - P_hi)
        l_part = l_part * corr + rs; m_run = m_new;
        // The accumulator may only be touched between P V products.  The wait is unconditional: a parity wait is only
        // unambiguous when no completion of this barrier has been skipped (the first block of a tile skips none: the
        // previous tile's write-out has waited for its last product).
        if (j > 0) ok &= WWAIT(BAR(13), (g - 1) & 1, 13);
        if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
          tc_fence_after();
          tmem_ld32(lane_base + ATC_COL_O + ob * 64, a);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; e++) a[e] = __float_as_uint(__uint_as_float(a[e]) * corr);
          tmem_st32(lane_base + ATC_COL_O + ob * 64, a);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(BAR(11 + s));
      }
      ok &= WWAIT(BAR(13), (g0 + nblk - 1) & 1, 13);
      tc_fence_after();
      {
        uint32_t a[32];
        tmem_ld32(lane_base + ATC_COL_O + ob * 64, a);
        float* xb = xch + (xc++ & 1) * 256;
        xb[half * 128 + row] = l_part;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const float l_run = l_part + xb[(half ^ 1) * 128 + row];
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(BAR(15 + ob));                          // the accumulator is in registers: the MMA warp may reuse it
        const float il = 1.f / l_run;
        const int bz = z / H, h = z % H;
        float* orow = O + ((long)bz * T + qi) * D + (long)h * ATC_HD + 32 * half;
#pragma unroll
        for (int e = 0; e < 8; e++)
          *reinterpret_cast<float4*>(orow + 4 * e) = make_float4(__uint_as_float(a[4 * e]) * il, __uint_as_float(a[4 * e + 1]) * il, __uint_as_float(a[4 * e + 2]) * il, __uint_as_float(a[4 * e + 3]) * il);
        if (half == 0) { Mst[(long)z * T + qi] = m_run; Lst[(long)z * T + qi] = l_run; }
      }
      g0 += nblk;
    }
    (void)ok;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ATC_TMEM_COLS) : "memory");
}

// ------------------------------------------------------------------ backward
// reference: internal/layer/transformer.go:589-657.  One kernel template, three uses; each CTA owns a tile of 128
// rows ("row tile", operand planes resident in shared memory) and walks 64-wide blocks of the other index:
//   MODE 0 (dQ): rows = queries.  S = Q K_j^T, dP = dO V_j^T, dS = P (dP - Dv) / sqrt(hd), dQ += dS K_j
//   MODE 1 (dK): rows = keys.     S^T = K Q_i^T, dP^T = V dO_i^T, dS^T likewise,         dK += dS^T Q_i
//   MODE 2 (dV): rows = keys.     S^T = K Q_i^T, P^T,                                     dV += P^T dO_i
// with P = exp(S / sqrt(hd) - m) / l recomputed from the saved row statistics (per row of the tile in MODE 0, per
// column in MODES 1 and 2, staged in shared memory).  R1, R2 = row-tile operands; C1, C2 = block operands of the two
// score-shaped products ([64 rows][64]); C3 = block operand of the accumulating product, taken from TRANSPOSED planes
// ([64 head columns][T]) so that its contraction index runs along the row.  dS (P in MODE 2) goes back to tensor
// memory as hi/lo and is the A operand of the accumulating product.  TMEM: two sets of {S, dP / dS_hi, dS_lo} so that
// the score products of block n+1 run under the elementwise work of block n; two accumulators in the last 128 columns
// (the kernel is persistent: the next tile starts while the previous one is written out).
// Warps: 0 = TMA producer for R1, R2, C1, C2; 1 = MMA issuer; 2-9 = elementwise (two threads per tile row);
// 10 = TMA producer for C3 (its buffer is released much later than C1 / C2, so it gets its own thread).
constexpr int ATB_THREADS = 352;
constexpr int ATB_R_BYTES = 4 * 128 * 128, ATB_C_BYTES = 4 * 64 * 128;      // 64 KB, 32 KB
template <int MODE> struct AtbCfg {
  static constexpr int NR = MODE == 2 ? 1 : 2;                                 // row-tile operands, score-shaped products
  static constexpr int SMEM = NR * ATB_R_BYTES + (NR + 1) * ATB_C_BYTES + 1024 + 256 + 2 * 3 * 64 * 4;
};
constexpr uint32_t ATB_COL_S = 0, ATB_COL_DP = 128, ATB_COL_LO = 256, ATB_COL_ACC = 384;      // two accumulators of 64 columns

template <int MODE>
__global__ void __launch_bounds__(ATB_THREADS, 1)
attn_tc_bwd_kernel(const __grid_constant__ AttnMaps<15> maps, const float* __restrict__ Mst, const float* __restrict__ Lst, const float* __restrict__ Dv,
                   float* __restrict__ Out, int T, int D, int H, int causal, float inv_scale, int ntiles, int* status, unsigned spin_limit) {
  constexpr int NR = AtbCfg<MODE>::NR;
  constexpr bool TRANS = MODE != 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sR = smem;                                    // NR row-tile operands
  uint8_t* sC = sR + NR * ATB_R_BYTES;                   // NR block operands of the score products
  uint8_t* sC3 = sC + NR * ATB_C_BYTES;
  uint64_t* bars = (uint64_t*)(sC3 + ATB_C_BYTES);
  uint32_t* tmem_slot = (uint32_t*)(bars + 16);
  float* st = (float*)(bars + 32);                       // [2][3][64] column statistics (MODES 1, 2)
  // barriers: 0 r_full | 1 c12_full | 2 c12_empty | 3 c3_full | 4 c3_empty | 5,6 sd_full | 7,8 ds_full | 9 tile_done
  //           10 r_empty | 11,12 acc_free
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Bounded waits that fail fast: the first wait that gives up records its role in the status word at once, and every
  // later wait of every role and CTA (they all poll that word) gives up after at most 64 polls, so a launch whose pipeline
  // is stuck ends in milliseconds instead of polling each wait to its limit.  The copy and MMA threads stop issuing at
  // their first failed wait (arming a barrier whose previous phase has not completed is undefined), then let what
  // they have in flight finish.  The elementwise warps keep their loop structure (they meet at named barriers, so no
  // warp may leave early) and only touch tensor memory, count-256 barriers and in-range global rows; what they compute
  // after that point is discarded by the host (GN_ERR_TIMEOUT).
  const unsigned limit = spin_limit;
  auto WAIT = [&](uint32_t bar, uint32_t parity, int code) -> bool { if (mbar_wait(bar, parity, limit, status)) return true; atomicCAS(status, 0, code); return false; };
  auto WWAIT = [&](uint32_t bar, uint32_t parity, int code) -> bool { int w = 1; if (lane == 0) w = WAIT(bar, parity, code) ? 1 : 0; return __shfl_sync(0xffffffffu, w, 0) != 0; };
  const int ntr = T / 128;
  // persistent, as in the forward kernel: tile id -> problem z, first row of the tile, first block and number of blocks
  auto decode = [&](int id, int i, int& z, int& r0, int& b0, int& nb) {
    z = id / ntr; r0 = ((id % ntr + i) % ntr) * 128;
    b0 = (TRANS && causal) ? r0 / 64 : 0;
    nb = TRANS ? T / 64 - b0 : (causal ? (r0 + 128) / 64 : T / 64);
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 14; i++) mbar_init(BAR(i), (i == 7 || i == 8 || i == 11 || i == 12) ? 256 : 1);      // 13: drain
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, r0, b0, nb; decode(id, tt, z, r0, b0, nb);
        if (tt > 0 && !WAIT(BAR(10), (tt - 1) & 1, 21)) { ok = false; break; }
        mbar_expect_tx(BAR(0), NR * ATB_R_BYTES);
        // maps: R1 = 0..2, R2 = 3..5, C1 = 6..8, C2 = 9..11, C3 = 12..14 (hi | bf16 copy | bf16 lo each)
        for (int o = 0; o < NR; o++) {
          const uint32_t base = smem_u32(sR + o * ATB_R_BYTES);
          for (int c = 0; c < 2; c++) tma_load_3d(base + c * 16384, &maps.m[3 * o], c * 32, r0, z, BAR(0));
          tma_load_3d(base + 32768, &maps.m[3 * o + 1], 0, r0, z, BAR(0));
          tma_load_3d(base + 49152, &maps.m[3 * o + 2], 0, r0, z, BAR(0));
        }
        for (int n = 0; n < nb; n++, g++) {
          const int row = (b0 + n) * 64;
          if (g > 0 && !WAIT(BAR(2), (g - 1) & 1, 21)) { ok = false; break; }
          mbar_expect_tx(BAR(1), NR * ATB_C_BYTES);
          for (int o = 0; o < NR; o++) {
            const uint32_t base = smem_u32(sC + o * ATB_C_BYTES);
            for (int c = 0; c < 2; c++) tma_load_3d(base + c * 8192, &maps.m[6 + 3 * o], c * 32, row, z, BAR(1));
            tma_load_3d(base + 16384, &maps.m[7 + 3 * o], 0, row, z, BAR(1));
            tma_load_3d(base + 24576, &maps.m[8 + 3 * o], 0, row, z, BAR(1));
          }
        }
      }
      if (!ok || *(volatile int*)status) for (int i = 0; i < 200; i++) __nanosleep(1000);                 // own copies in flight land before the CTA exits
    }
  } else if (warp == 10) {
    if (lane == 0) {
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, r0, b0, nb; decode(id, tt, z, r0, b0, nb);
        for (int n = 0; n < nb; n++, g++) {
          const int col = (b0 + n) * 64;
          if (g > 0 && !WAIT(BAR(4), (g - 1) & 1, 22)) { ok = false; break; }
          mbar_expect_tx(BAR(3), ATB_C_BYTES);
          for (int c = 0; c < 2; c++) tma_load_3d(smem_u32(sC3 + c * 8192), &maps.m[12], col + c * 32, 0, z, BAR(3));
          tma_load_3d(smem_u32(sC3 + 16384), &maps.m[13], col, 0, z, BAR(3));
          tma_load_3d(smem_u32(sC3 + 24576), &maps.m[14], col, 0, z, BAR(3));
        }
      }
      if (!ok || *(volatile int*)status) for (int i = 0; i < 200; i++) __nanosleep(1000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true; uint32_t g0 = 0;
      constexpr uint32_t idesc = make_idesc(128, 64), idesc_bf = make_idesc_bf16(128, 64);
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, r0, b0, nb; decode(id, tt, z, r0, b0, nb);
        const uint32_t ab = tt & 1;
        auto issue_sd = [&](int n) {
          const uint32_t g = g0 + n, s = g & 1;
          if (!ok || !WAIT(BAR(1), g & 1, 23)) { ok = false; return; }
          tc_fence_after();
#pragma unroll
          for (int prod = 0; prod < NR; prod++) {
            const uint32_t acc = tmem_base + (prod == 0 ? ATB_COL_S : ATB_COL_DP) + s * 64;
            const uint32_t ra = smem_u32(sR + prod * ATB_R_BYTES), cb = smem_u32(sC + prod * ATB_C_BYTES);
#pragma unroll
            for (int k = 0; k < 4; k++) {                    // cross terms: bf16, 16 head columns per instruction
              const uint64_t adv = (uint64_t)(2 * k);
              tc_mma_bf16(acc, make_desc<32>(ra + 49152) + adv, make_desc<32>(cb + 16384) + adv, idesc_bf, k ? 1u : 0u);
              tc_mma_bf16(acc, make_desc<32>(ra + 32768) + adv, make_desc<32>(cb + 24576) + adv, idesc_bf, 1u);
            }
#pragma unroll
            for (int c = 0; c < 2; c++)
#pragma unroll
              for (int k = 0; k < 4; k++) {                  // main term: tf32, 8 head columns per instruction
                const uint64_t adv = (uint64_t)(2 * k);
                tc_mma_tf32(acc, make_desc<32>(ra + c * 16384) + adv, make_desc<32>(cb + c * 8192) + adv, idesc, 1u);
              }
          }
          tc_commit(BAR(2));
          tc_commit(BAR(5 + s));
          if (n == nb - 1) tc_commit(BAR(10));               // the row tile may be replaced
        };
        auto issue_acc = [&](int n) {
          const uint32_t g = g0 + n, s = g & 1, u = g >> 1;
          if (!ok || !WAIT(BAR(7 + s), u & 1, 23) || !WAIT(BAR(3), g & 1, 23)) { ok = false; return; }
          tc_fence_after();
          const uint32_t cb = smem_u32(sC3);
          const uint32_t ph = tmem_base + (MODE == 2 ? ATB_COL_S : ATB_COL_DP) + s * 64, pl = tmem_base + ATB_COL_LO + s * 64,
                         acc = tmem_base + ATB_COL_ACC + ab * 64;
#pragma unroll
          for (int k = 0; k < 4; k++) {                      // cross terms: packed bf16 (16 block columns = 8 TMEM columns per instruction)
            const uint64_t adv = (uint64_t)(2 * k);
            tc_mma_bf16_ts(acc, pl + 32 + k * 8, make_desc<32>(cb + 16384) + adv, idesc_bf, (n | k) ? 1u : 0u);
            tc_mma_bf16_ts(acc, pl + k * 8, make_desc<32>(cb + 24576) + adv, idesc_bf, 1u);
          }
#pragma unroll
          for (int kk = 0; kk < 8; kk++) {                   // main term: tf32 hi (8 columns per instruction)
            const int c = kk >> 2; const uint64_t adv = (uint64_t)(2 * (kk & 3));
            tc_mma_tf32_ts(acc, ph + kk * 8, make_desc<32>(cb + c * 8192) + adv, idesc, 1u);
          }
          tc_commit(BAR(4));
          if (n == nb - 1) tc_commit(BAR(9));
        };
        if (!WAIT(BAR(0), tt & 1, 23)) { ok = false; break; }
        if (tt >= 2 && !WAIT(BAR(11 + ab), ((tt >> 1) - 1) & 1, 23)) { ok = false; break; }     // this accumulator has been written out
        issue_sd(0);
        if (nb > 1) issue_sd(1);
        for (int n = 0; n < nb; n++) {
          issue_acc(n);
          if (n + 2 < nb) issue_sd(n + 2);
        }
        g0 += nb;
      }
      if (!ok || *(volatile int*)status) { tc_commit(BAR(13)); mbar_wait(BAR(13), 0, TC_DRAIN_LIMIT); }     // own instructions in flight finish before TMEM is released
    }
  } else {
    // two threads per tile row: `half` selects 32 of the 64 columns of a block (and of the accumulator)
    const int quad = warp & 3, half = (warp - 2) >> 2, row = quad * 32 + lane, et = (warp - 2) * 32 + lane;   // et: 0..255
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + 32 * half;
    const uint32_t pk_base = tmem_base + ((uint32_t)(quad * 32) << 16) + 16 * half;     // packed bf16 planes: 16 columns per half
    constexpr float LOG2E = 1.44269504088896341f;
    const float cs = inv_scale * LOG2E, oscale = MODE == 2 ? 1.f : inv_scale;
    bool ok = true; uint32_t g0 = 0;
    for (int id = blockIdx.x, tt = 0; id < ntiles; id += gridDim.x, tt++) {
      int z, r0, b0, nb; decode(id, tt, z, r0, b0, nb);
      const int ri = r0 + row; const long sb = (long)z * T; const uint32_t ab = tt & 1;
      float mneg_r = 0.f, il_r = 0.f, d_r = 0.f;        // -m log2(e), scale / l, Dv of this row (MODE 0)
      if (!TRANS) { mneg_r = -Mst[sb + ri] * LOG2E; il_r = oscale / Lst[sb + ri]; d_r = Dv[sb + ri]; }
      for (int n = 0; n < nb; n++) {
        const uint32_t g = g0 + n, s = g & 1, u = g >> 1; const int c0 = (b0 + n) * 64;
        float* stm = st + s * 192; float* stl = stm + 64; float* std_ = stm + 128;
        if (TRANS) {
          if (et < 64) { stm[et] = -Mst[sb + c0 + et] * LOG2E; stl[et] = oscale / Lst[sb + c0 + et]; if (MODE == 1) std_[et] = Dv[sb + c0 + et]; }
          asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        ok &= WWAIT(BAR(5 + s), u & 1, 24);
        tc_fence_after();
        uint32_t a[32], b[32];
        tmem_ld32(lane_base + ATB_COL_S + s * 64, a);
        if (MODE != 2) tmem_ld32(lane_base + ATB_COL_DP + s * 64, b);
        tmem_wait_ld();
        // does the block reach across the diagonal for some row of the tile?
        const bool diag = causal && (TRANS ? r0 + 127 > c0 : c0 + 63 > r0);
#pragma unroll
        for (int e = 0; e < 32; e++) {
          const int col = 32 * half + e;
          float v = fast_ex2(fmaf(__uint_as_float(a[e]), cs, TRANS ? stm[col] : mneg_r)) * (TRANS ? stl[col] : il_r);   // P (times 1/sqrt(hd) for dS)
          if (MODE != 2) v *= __uint_as_float(b[e]) - (TRANS ? std_[col] : d_r);                                        // dS
          if (diag && (TRANS ? ri > c0 + col : c0 + col > ri)) v = 0.f;
          a[e] = __float_as_uint(v);
        }
        uint32_t xb[16], lob[16];
        split_pack32(a, xb, lob);
        tmem_st32(lane_base + (MODE == 2 ? ATB_COL_S : ATB_COL_DP) + s * 64, a);      // hi, 32-bit columns
        tmem_st16(pk_base + ATB_COL_LO + s * 64, xb);                                 // bf16 copy, two block columns per TMEM column
        tmem_st16(pk_base + ATB_COL_LO + s * 64 + 32, lob);                           // bf16 lo
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(BAR(7 + s));
      }
      ok &= WWAIT(BAR(9), tt & 1, 24);
      tc_fence_after();
      {
        uint32_t a[32];
        tmem_ld32(lane_base + ATB_COL_ACC + ab * 64, a);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(BAR(11 + ab));                          // the accumulator is in registers: the MMA warp may reuse it
        const int bz = z / H, h = z % H;
        float* orow = Out + ((long)bz * T + ri) * D + (long)h * ATC_HD + 32 * half;
#pragma unroll
        for (int e = 0; e < 8; e++)
          *reinterpret_cast<float4*>(orow + 4 * e) = make_float4(__uint_as_float(a[4 * e]), __uint_as_float(a[4 * e + 1]), __uint_as_float(a[4 * e + 2]), __uint_as_float(a[4 * e + 3]));
      }
      g0 += nb;
    }
    (void)ok;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}

// ------------------------------------------------------------------ host side
struct AttnTcScratch { DevBuf buf[16]; };
inline AttnTcScratch& attn_tc_scratch(Ctx* ctx) {
  if (!ctx->attn_scratch) ctx->attn_scratch = ctx->own(new AttnTcScratch());
  return *static_cast<AttnTcScratch*>(ctx->attn_scratch);
}
inline int attn_tc_buf(Ctx* ctx, int i, size_t n, float** out) {
  DevBuf& b = attn_tc_scratch(ctx).buf[i];
  if (b.n < n) { GN_CUDA(cudaStreamSynchronize(ctx->stream)); GN_TRY(b.alloc(n)); }
  *out = b.p; return GN_OK;
}
inline bool attn_tc_supported(Ctx* ctx, int hd, int T, int B, int H, int D) {
  static const bool off = [] { const char* e = getenv("GONEURON_CUDA_ATTENTION"); return e && !strcmp(e, "mma"); }();
  return !off && ctx->tc_ok && hd == ATC_HD && T % ATC_BQ == 0 && (long)B * H <= 65535 && D % 4 == 0;
}
// Operand planes of one [B*T, D] tensor for all (batch, head) problems, from ONE read of the tensor:
//   row planes  [Z][T][64]  (ROWS)  and / or  transposed planes [Z][64][T]  (COLS),   z = batch * H + head,
// three planes each: hi = tf32(x) as fp32, bf16(x), bf16(x - hi).
// One CTA = a 64 x 64 tile (64 tokens of one head); the transposition goes through shared memory.
template <bool ROWS, bool COLS>
__global__ void __launch_bounds__(256) attn_split_kernel(const float* __restrict__ X, float* __restrict__ rhi, __nv_bfloat16* __restrict__ rxb,
                                                         __nv_bfloat16* __restrict__ rlo, float* __restrict__ chi, __nv_bfloat16* __restrict__ cxb,
                                                         __nv_bfloat16* __restrict__ clo, int T, int D, int H) {
  __shared__ float tile[64][65];
  const int z = blockIdx.y, b = z / H, h = z % H, t0 = blockIdx.x * 64, i = threadIdx.x;
  const int c4 = i & 15, r0 = i >> 4;
  float4 x[4];
#pragma unroll
  for (int r = 0; r < 4; r++) x[r] = *reinterpret_cast<const float4*>(X + ((long)b * T + t0 + r0 + 16 * r) * D + (long)h * 64 + c4 * 4);
#pragma unroll
  for (int r = 0; r < 4; r++) {
    const int row = r0 + 16 * r;
    if (ROWS) {
      const float4 hv = make_float4(tf32_round(x[r].x), tf32_round(x[r].y), tf32_round(x[r].z), tf32_round(x[r].w));
      const long o = ((long)z * T + t0 + row) * 64 + c4 * 4;
      *reinterpret_cast<float4*>(rhi + o) = hv;
      *reinterpret_cast<uint2*>(rxb + o) = make_uint2(pack_bf16(x[r].x, x[r].y), pack_bf16(x[r].z, x[r].w));
      *reinterpret_cast<uint2*>(rlo + o) = make_uint2(pack_bf16(x[r].x - hv.x, x[r].y - hv.y), pack_bf16(x[r].z - hv.z, x[r].w - hv.w));
    }
    if (COLS) { tile[row][c4 * 4] = x[r].x; tile[row][c4 * 4 + 1] = x[r].y; tile[row][c4 * 4 + 2] = x[r].z; tile[row][c4 * 4 + 3] = x[r].w; }
  }
  if (COLS) {
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; r++) {
      const int d = r0 + 16 * r;                          // head column -> plane row; c4 -> 4 consecutive tokens
      const float4 v = make_float4(tile[c4 * 4][d], tile[c4 * 4 + 1][d], tile[c4 * 4 + 2][d], tile[c4 * 4 + 3][d]);
      const float4 hv = make_float4(tf32_round(v.x), tf32_round(v.y), tf32_round(v.z), tf32_round(v.w));
      const long o = ((long)z * 64 + d) * T + t0 + c4 * 4;
      *reinterpret_cast<float4*>(chi + o) = hv;
      *reinterpret_cast<uint2*>(cxb + o) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
      *reinterpret_cast<uint2*>(clo + o) = make_uint2(pack_bf16(v.x - hv.x, v.y - hv.y), pack_bf16(v.z - hv.z, v.w - hv.w));
    }
  }
}
// slot / slot + 1 receive the row planes (hi | the two bf16 planes), cslot / cslot + 1 the transposed ones (a negative
// slot = not wanted)
inline int attn_tc_planes(Ctx* ctx, const float* X, int slot, int cslot, int B, int T, int D, int H, TcPlanes* rows, TcPlanes* cols) {
  const int Z = B * H; const size_t n = (size_t)Z * T * ATC_HD;
  TcPlanes r{nullptr, nullptr, T, ATC_HD, ATC_HD, Z}, c{nullptr, nullptr, ATC_HD, T, T, Z};
  if (slot >= 0) { GN_TRY(attn_tc_buf(ctx, slot, n, &r.hi)); GN_TRY(attn_tc_buf(ctx, slot + 1, n, &r.lo)); *rows = r; }
  if (cslot >= 0) { GN_TRY(attn_tc_buf(ctx, cslot, n, &c.hi)); GN_TRY(attn_tc_buf(ctx, cslot + 1, n, &c.lo)); *cols = c; }
  const dim3 grid(T / 64, Z);
  __nv_bfloat16* nb = nullptr;
  if (slot >= 0 && cslot >= 0) GN_LAUNCH(ctx, (attn_split_kernel<true, true>), grid, 256, 0, X, r.hi, r.xb(), r.lob(), c.hi, c.xb(), c.lob(), T, D, H);
  else if (slot >= 0) GN_LAUNCH(ctx, (attn_split_kernel<true, false>), grid, 256, 0, X, r.hi, r.xb(), r.lob(), (float*)nullptr, nb, nb, T, D, H);
  else GN_LAUNCH(ctx, (attn_split_kernel<false, true>), grid, 256, 0, X, (float*)nullptr, nb, nb, c.hi, c.xb(), c.lob(), T, D, H);
  return check_launch("attn_split");
}
// the three tensor maps of one operand: hi (fp32, 32 columns per copy), bf16 copy and bf16 lo (64 columns per copy)
inline int attn_tc_maps(Ctx* ctx, CUtensorMap* m, const TcPlanes& p, int box_rows) {
  GN_TRY(tc_make_map(ctx, &m[0], p, p.hi, box_rows));
  GN_TRY(tc_make_map_bf16(ctx, &m[1], p, p.xb(), box_rows, 64));
  return tc_make_map_bf16(ctx, &m[2], p, p.lob(), box_rows, 64);
}
inline int attn_tc_fwd(Ctx* ctx, const float* Q, const float* K, const float* V, float* O, float* M, float* L, int B, int T, int D, int H, int causal) {
  TcPlanes pq, pk, pv;
  GN_TRY(attn_tc_planes(ctx, Q, 0, -1, B, T, D, H, &pq, nullptr));
  GN_TRY(attn_tc_planes(ctx, K, 2, -1, B, T, D, H, &pk, nullptr));
  GN_TRY(attn_tc_planes(ctx, V, -1, 4, B, T, D, H, nullptr, &pv));
  AttnMaps<9> maps;
  GN_TRY(attn_tc_maps(ctx, &maps.m[0], pq, ATC_BQ)); GN_TRY(attn_tc_maps(ctx, &maps.m[3], pk, ATC_BK)); GN_TRY(attn_tc_maps(ctx, &maps.m[6], pv, ATC_HD));
  GN_CUDA(cudaFuncSetAttribute(attn_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_FWD_SMEM));
  const int ntq = T / ATC_BQ, ntiles = ntq * B * H;
  const int grid = std::min(ntiles, std::max(1, ctx->sm_count / ntq) * ntq);      // a multiple of the query blocks per problem
  GN_LAUNCH(ctx, attn_tc_fwd_kernel, grid, ATC_THREADS, ATC_FWD_SMEM, maps, O, M, L, T, D, H, causal, 1.f / sqrtf((float)ATC_HD), ntiles, ctx->d_status, ctx->spin_limit);
  return check_launch("attn_tc_fwd");
}

template <int MODE>
inline int attn_tc_bwd_launch(Ctx* ctx, const TcPlanes& r1, const TcPlanes& r2, const TcPlanes& c1, const TcPlanes& c2, const TcPlanes& c3,
                              const float* M, const float* L, const float* Dv, float* out, int B, int T, int D, int H, int causal) {
  AttnMaps<15> maps;
  GN_TRY(attn_tc_maps(ctx, &maps.m[0], r1, 128)); GN_TRY(attn_tc_maps(ctx, &maps.m[3], r2, 128));
  GN_TRY(attn_tc_maps(ctx, &maps.m[6], c1, 64)); GN_TRY(attn_tc_maps(ctx, &maps.m[9], c2, 64)); GN_TRY(attn_tc_maps(ctx, &maps.m[12], c3, ATC_HD));
  GN_CUDA(cudaFuncSetAttribute(attn_tc_bwd_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, AtbCfg<MODE>::SMEM));
  const int ntr = T / 128, ntiles = ntr * B * H;
  const int grid = std::min(ntiles, std::max(1, ctx->sm_count / ntr) * ntr);      // a multiple of the row tiles per problem
  GN_LAUNCH(ctx, attn_tc_bwd_kernel<MODE>, grid, ATB_THREADS, AtbCfg<MODE>::SMEM, maps, M, L, Dv, out, T, D, H, causal, 1.f / sqrtf((float)ATC_HD), ntiles, ctx->d_status, ctx->spin_limit);
  return check_launch("attn_tc_bwd");
}
// dQ, dK, dV from Q, K, V, O, dO and the forward's row statistics; Dv receives the row products dO . O
inline int attn_tc_bwd(Ctx* ctx, const float* Q, const float* K, const float* V, const float* O, const float* dO, const float* M, const float* L, float* Dv,
                       float* dQ, float* dK, float* dV, int B, int T, int D, int H, int causal) {
  const long rows = (long)B * T * H;
  if (D == H * ATC_HD && ((reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(O)) & 15) == 0)
    GN_LAUNCH(ctx, attn_rowdot64_kernel, (unsigned)std::min<long>(cdiv(rows, 32), (long)ctx->sm_count * 16), 256, 0, dO, O, Dv, T, H, rows);
  else GN_LAUNCH(ctx, attn_rowdot_kernel, cdiv(rows, 8), 256, 0, dO, O, Dv, T, D, H, ATC_HD, rows);
  TcPlanes qp, kp, vp, gp, qt, kt, gt;
  GN_TRY(attn_tc_planes(ctx, Q, 0, 10, B, T, D, H, &qp, &qt));
  GN_TRY(attn_tc_planes(ctx, K, 2, 12, B, T, D, H, &kp, &kt));
  GN_TRY(attn_tc_planes(ctx, V, 6, -1, B, T, D, H, &vp, nullptr));
  GN_TRY(attn_tc_planes(ctx, dO, 8, 14, B, T, D, H, &gp, &gt));
  GN_TRY(attn_tc_bwd_launch<0>(ctx, qp, gp, kp, vp, kt, M, L, Dv, dQ, B, T, D, H, causal));
  GN_TRY(attn_tc_bwd_launch<1>(ctx, kp, vp, qp, gp, qt, M, L, Dv, dK, B, T, D, H, causal));
  GN_TRY(attn_tc_bwd_launch<2>(ctx, kp, kp, qp, qp, gt, M, L, Dv, dV, B, T, D, H, causal));
  return GN_OK;
}

}  // namespace gn
