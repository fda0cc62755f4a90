// attention_tc.cuh -- multi-head attention (head size 64) on the tcgen05 tensor cores with the score tile, the
// probabilities and the output accumulator resident in tensor memory.
//
// reference: internal/layer/transformer.go:470-503 (forward) and :589-657 (backward) -- same arithmetic as
// attention.cuh: scores = q.k / sqrt(hd), masked entries removed, row softmax, weighted sum of v; row maximum and row
// sum kept per row; the backward pass recomputes the probabilities from them.
//
// Operands: the scaled fp16 planes of gemm_tc.cuh's scheme, one problem z per (batch, head).  x s = hi + lo with both
// parts fp16, s a power of two PER PROBLEM AND TENSOR (the largest magnitude of the problem's 64 x T entries lands in
// [2^14, 2^15)); every product is three kind::f16 MMAs (lo x hi, hi x lo, hi x hi, the small terms first).  An fp16 pair
// resolves 22 bits of every entry down to 2^-17 of the largest one, so one scale per problem is enough -- and it has to
// be constant along a contraction, which for the products over the keys means constant over the problem.
//   row planes        [Z][T][64]   (contraction over the head dimension along the row): Q, K, V, dO
//   transposed planes [Z][64][T]   (contraction over the keys / queries along the row):  V (forward), K, Q, dO (backward)
// (attn_prep_* write both kinds from one read of the tensor, after one pass that finds the scales.)  The tiles are
// fetched by TMA into 128-byte-swizzled shared memory: 4 bytes per element instead of the 8 of the TF32 + 2 x BF16 planes
// this engine used before, which is what makes room for multi-stage block operands.
//
// What bounds these kernels is not arithmetic.  A clock trace of the previous version (one MMA-issuing thread,
// single-stage block operands, 48 small MMAs per 64-key block) showed the issuing thread busy 5200 cycles per block for
// 1300 cycles of tensor work, behind it a single-buffered TMA fetch, and the elementwise warps waiting.  Hence here:
//   * one MMA-issuing warp per product of a block, ordered through mbarriers only;
//   * 36 instead of 48 MMAs per block (three fp16 terms instead of two BF16 + a TF32 term at half the depth);
//   * three or four shared-memory stages for the block operands, three or four TMEM stages for the score tiles;
//   * sixteen elementwise warps (four threads per tile row, 16 columns each): their chain is latency-bound;
//   * the write-out of a tile deferred until the next tile's first block has been handed on.
// The same trace now: 2450 cycles per block in the backward kernels, i.e. 68 cycles per 128 x 64 x 16 MMA whichever
// warp issues it, against 32 cycles of arithmetic.  Keeping the row-tile operand in tensor memory (copied there by the
// elementwise warps when a tile starts, so that a score product fetches 2 instead of 6 KB per MMA from shared memory)
// was built and measured: 3 to 14 % slower -- the products with the A operand in tensor memory take as long per MMA,
// and the planes cost a score stage.  The MMA rate at N = 64 is what is left.
// P (forward), dS / P^T (backward) go back to tensor memory as fp16 hi | lo pairs, written over the score columns they
// were computed from -- each thread's 16 columns hold exactly its 8 + 8 packed words, so no thread overwrites what
// another still has to read -- and are the A operand of the accumulating product.
// Every wait is bounded; a wait that gives up sets the status word at once, which makes every other wait of the launch
// give up within a few polls (see WAIT below).
#pragma once
#include "attention.cuh"
#include "gemm_tc.cuh"

namespace gn {

constexpr int ATC_BQ = 128, ATC_BK = 64, ATC_HD = 64;
constexpr int ATC_CW = 16, ATC_NPART = 64 / ATC_CW, ATC_EW_WARPS = 4 * ATC_NPART, ATC_EW_THREADS = 32 * ATC_EW_WARPS;
constexpr int ATC_THREADS = 96 + ATC_EW_THREADS;      // forward: warp 0 TMA, warps 1 and 2 MMA issuers, 16 elementwise warps
constexpr int ATB_THREADS = 128 + ATC_EW_THREADS;     // backward: warp 0 TMA, warps 1-3 MMA issuers, 16 elementwise warps
constexpr int ATC_R_BYTES = 2 * 128 * 128;            // a 128-row tile: hi | lo, 128-byte rows: 32 KB
constexpr int ATC_C_BYTES = 2 * 64 * 128;             // a 64-row block: hi | lo: 16 KB
constexpr float ATC_PSCALE = 16384.f;                 // probabilities (at most 1) as fp16 pairs
// Forward: the running maximum is only moved when it grows by more than 2^ATF_LAZY_LOG2 (then the accumulator is
// rescaled); otherwise the stale maximum stays the reference point -- the row statistics kept for the backward pass are
// the pair that was used, so exp(s - m) / l is the same probability either way.  The unnormalised p can then reach
// 2^ATF_LAZY_LOG2, hence the smaller plane scale.
constexpr float ATF_LAZY_LOG2 = 6.f, ATF_PSCALE = 256.f;

__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                 "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
                 "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ float fast_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 16 fp32 values (one k-step of the accumulating product) times `s` -> 8 packed fp16 hi words, 8 packed lo words, laid
// out hi | lo in the 16 columns the values came from
__device__ __forceinline__ void pack_planes16(const float (&v)[16], float s, uint32_t (&w)[16]) {
#pragma unroll
  for (int e = 0; e < 8; e++) split2_pair(v[2 * e], v[2 * e + 1], s, w[e], w[8 + e]);
}
// The three MMAs of one 16-deep step of an fp32-accurate product, small terms first.  SS: both operands in shared memory.
__device__ __forceinline__ void mma3_ss(uint32_t acc, uint64_t a_hi, uint64_t a_lo, uint64_t b_hi, uint64_t b_lo, uint32_t idesc, bool first) {
  tc_mma_f16(acc, a_lo, b_hi, idesc, first ? 0u : 1u);
  tc_mma_f16(acc, a_hi, b_lo, idesc, 1u);
  tc_mma_f16(acc, a_hi, b_hi, idesc, 1u);
}
// TS: the A operand (hi at tmem_a, lo 8 columns further) in tensor memory.
__device__ __forceinline__ void mma3_ts(uint32_t acc, uint32_t tmem_a, uint64_t b_hi, uint64_t b_lo, uint32_t idesc, bool first) {
  tc_mma_f16_ts(acc, tmem_a + 8, b_hi, idesc, first ? 0u : 1u);
  tc_mma_f16_ts(acc, tmem_a, b_lo, idesc, 1u);
  tc_mma_f16_ts(acc, tmem_a, b_hi, idesc, 1u);
}

// Tensor maps of a launch: two per operand (hi, lo).
template <int N> struct AttnMaps { CUtensorMap m[N]; };

// ------------------------------------------------------------------ forward
// Persistent: gridDim.x CTAs (one per SM) walk the tiles; tile id = blockIdx.x + i * gridDim.x names (batch*head, query
// block), the query block being rotated by i so that every CTA sees short and long causal tiles alike (gridDim.x is a
// multiple of the number of query blocks).  All counters run across tiles, so the barriers' phases simply continue.
//   warp 0 : TMA producer: Q (two buffers, the next tile's Q arrives under the current tile), K and V^T blocks (four stages)
//   warp 1 : issues S_j = Q K_j^T into one of four 64-column TMEM buffers, as soon as P V of block j-4 has left it
//   warp 2 : issues O += P_j V_j (P from TMEM, V^T_j from shared memory) into one of two output accumulators
//   warps 3-18 : softmax.  tcgen05.ld of S_j, running maximum (exchanged through shared memory) and sum, p = exp(s - m)
//            written back as fp16 planes; when a row maximum moved by more than 2^6, the output accumulator is rescaled
//            in TMEM after the previous P V has completed.  The write-out of a finished tile waits until the first
//            block of the next tile has been handed to the P V issuer.
// (A trace of the two-buffer version: S_{j+2} waited for P V_j, the softmax for S_{j+2}, 2700 cycles per block, and
// 6000 cycles at every tile boundary for the write-out and the next tile's scale factors.)
constexpr int ATF_NK = 4, ATF_NSS = 4;
constexpr int ATF_SMEM = 2 * ATC_R_BYTES + 2 * ATF_NK * ATC_C_BYTES + 1024 + 512 + 2 * ATC_NPART * 128 * 4;
constexpr uint32_t ATF_COL_S = 0, ATF_COL_O = 64 * ATF_NSS, ATF_TMEM_COLS = 512;
// barriers: q_full 0,1 | q_empty 2,3 | k_full 4-7 | k_empty 8-11 | v_full 12-15 | v_empty 16-19 | s_full 20-23 | p_full 24-27
//           s_free 28-31 (P V of the buffer has completed) | o_free 32,33 | drains 34,35
__global__ void __launch_bounds__(ATC_THREADS, 1)
attn_tc_fwd_kernel(const __grid_constant__ AttnMaps<6> maps, float* __restrict__ O, float* __restrict__ Mst, float* __restrict__ Lst,
                   const float* __restrict__ isq, const float* __restrict__ isk, const float* __restrict__ isv,
                   int T, int D, int H, int causal, float inv_scale, int ntiles, int* status, unsigned spin_limit) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                                                 // two tiles of ATC_R_BYTES
  uint8_t* sK = sQ + 2 * ATC_R_BYTES;                                 // ATF_NK stages of ATC_C_BYTES
  uint8_t* sV = sK + ATF_NK * ATC_C_BYTES;
  uint64_t* bars = (uint64_t*)(sV + ATF_NK * ATC_C_BYTES);
  uint32_t* tmem_slot = (uint32_t*)(bars + 40);
  float* xch = (float*)(bars + 64);                                   // [2][ATC_NPART][128] row maxima / sums exchanged between the threads of a row
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  constexpr int NSS = ATF_NSS, QF = 0, QE = 2, KF = 4, KE = 8, VF = 12, VE = 16, SF = 20, PF = 24, SFREE = 28, OFREE = 32, DRAIN = 34;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Bounded waits that fail fast: the first wait that gives up records its role in the status word at once, and every
  // later wait of every role and CTA (they all poll that word) gives up after at most 64 polls, so a launch whose pipeline
  // is stuck ends in milliseconds instead of polling each wait to its limit.  The copy and MMA threads stop issuing at
  // their first failed wait (arming a barrier whose previous phase has not completed is undefined), then let what
  // they have in flight finish.  The elementwise warps keep their loop structure (they meet at named barriers, so no
  // warp may leave early) and only touch tensor memory, count-512 barriers and in-range global rows; what they compute
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
    for (int i = 0; i < 36; i++) mbar_init(BAR(i), ((i >= PF && i < PF + NSS) || i == OFREE || i == OFREE + 1) ? ATC_EW_THREADS : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(ATF_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t idesc = make_idesc_f16(ATC_BQ, 64);

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, q0, nblk; decode(id, tt, z, q0, nblk);
        const uint32_t qb = tt & 1;
        if (tt >= 2 && !WAIT(BAR(QE + qb), ((tt >> 1) - 1) & 1, 11)) { ok = false; break; }
        mbar_expect_tx(BAR(QF + qb), ATC_R_BYTES);
        tma_load_3d(smem_u32(sQ + qb * ATC_R_BYTES), &maps.m[0], 0, q0, z, BAR(QF + qb));
        tma_load_3d(smem_u32(sQ + qb * ATC_R_BYTES + ATC_R_BYTES / 2), &maps.m[1], 0, q0, z, BAR(QF + qb));
        for (int j = 0; j < nblk; j++, g++) {
          const uint32_t s = g % ATF_NK, u = g / ATF_NK;
          if (u > 0 && !WAIT(BAR(KE + s), (u - 1) & 1, 11)) { ok = false; break; }
          mbar_expect_tx(BAR(KF + s), ATC_C_BYTES);
          tma_load_3d(smem_u32(sK + s * ATC_C_BYTES), &maps.m[2], 0, j * ATC_BK, z, BAR(KF + s));
          tma_load_3d(smem_u32(sK + s * ATC_C_BYTES + ATC_C_BYTES / 2), &maps.m[3], 0, j * ATC_BK, z, BAR(KF + s));
          if (u > 0 && !WAIT(BAR(VE + s), (u - 1) & 1, 11)) { ok = false; break; }
          mbar_expect_tx(BAR(VF + s), ATC_C_BYTES);
          tma_load_3d(smem_u32(sV + s * ATC_C_BYTES), &maps.m[4], j * ATC_BK, 0, z, BAR(VF + s));
          tma_load_3d(smem_u32(sV + s * ATC_C_BYTES + ATC_C_BYTES / 2), &maps.m[5], j * ATC_BK, 0, z, BAR(VF + s));
        }
      }
      if (!ok || *(volatile int*)status) for (int i = 0; i < 200; i++) __nanosleep(1000);                 // own copies in flight land before the CTA exits
    }
  } else if (warp == 1) {
    if (lane == 0) {                                          // score products
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, q0, nblk; decode(id, tt, z, q0, nblk);
        const uint32_t qb = tt & 1;
        if (!WAIT(BAR(QF + qb), (tt >> 1) & 1, 12)) { ok = false; break; }
        const uint32_t qa = smem_u32(sQ + qb * ATC_R_BYTES);
        const uint64_t q_hi = make_desc<32>(qa), q_lo = make_desc<32>(qa + ATC_R_BYTES / 2);
        for (int j = 0; j < nblk; j++, g++) {
          const uint32_t s = g % ATF_NK, u = g / ATF_NK, sb = g % NSS, su = g / NSS;
          if (!WAIT(BAR(KF + s), u & 1, 12)) { ok = false; break; }
          if (su > 0 && !WAIT(BAR(SFREE + sb), (su - 1) & 1, 12)) { ok = false; break; }      // P V of block g - NSS has read this buffer
          tc_fence_after();
          const uint32_t acc = tmem_base + ATF_COL_S + sb * 64, kb = smem_u32(sK + s * ATC_C_BYTES);
          const uint64_t k_hi = make_desc<32>(kb), k_lo = make_desc<32>(kb + ATC_C_BYTES / 2);
#pragma unroll
          for (int k = 0; k < 4; k++) { const uint64_t adv = (uint64_t)(2 * k); mma3_ss(acc, q_hi + adv, q_lo + adv, k_hi + adv, k_lo + adv, idesc, k == 0); }
          tc_commit(BAR(KE + s));
          tc_commit(BAR(SF + sb));
          if (j == nblk - 1) tc_commit(BAR(QE + qb));          // this Q buffer may be replaced
        }
      }
      if (!ok || *(volatile int*)status) { tc_commit(BAR(DRAIN)); mbar_wait(BAR(DRAIN), 0, TC_DRAIN_LIMIT); }     // own instructions in flight finish before TMEM is released
    }
  } else if (warp == 2) {
    if (lane == 0) {                                          // accumulating products
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, q0, nblk; decode(id, tt, z, q0, nblk);
        const uint32_t ob = tt & 1;
        if (tt >= 2 && !WAIT(BAR(OFREE + ob), ((tt >> 1) - 1) & 1, 14)) { ok = false; break; }     // this accumulator has been written out
        for (int j = 0; j < nblk; j++, g++) {
          const uint32_t s = g % ATF_NK, u = g / ATF_NK, sb = g % NSS, su = g / NSS;
          if (!WAIT(BAR(PF + sb), su & 1, 14) || !WAIT(BAR(VF + s), u & 1, 14)) { ok = false; break; }
          tc_fence_after();
          const uint32_t acc = tmem_base + ATF_COL_O + ob * 64, pa = tmem_base + ATF_COL_S + sb * 64, vb = smem_u32(sV + s * ATC_C_BYTES);
          const uint64_t v_hi = make_desc<32>(vb), v_lo = make_desc<32>(vb + ATC_C_BYTES / 2);
#pragma unroll
          for (int k = 0; k < 4; k++) { const uint64_t adv = (uint64_t)(2 * k); mma3_ts(acc, pa + 16 * k, v_hi + adv, v_lo + adv, idesc, j == 0 && k == 0); }
          tc_commit(BAR(VE + s));
          tc_commit(BAR(SFREE + sb));
        }
      }
      if (!ok || *(volatile int*)status) { tc_commit(BAR(DRAIN + 1)); mbar_wait(BAR(DRAIN + 1), 0, TC_DRAIN_LIMIT); }
    }
  } else {
    // four threads per query row: `part` selects 16 of the 64 columns of a block (and of the accumulator)
    constexpr int CW = ATC_CW;
    const int quad = warp & 3, part = (warp - 3) >> 2, row = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + CW * part;
    bool ok = true; uint32_t g0 = 0, xc = 0;
    constexpr float LOG2E = 1.44269504088896341f;
    // write-out of a finished tile: wait for its last P V, scale, store
    int pend_tt = -1; uint32_t pend_g = 0; float pend_il = 0.f; float* pend_row = nullptr;
    auto write_out = [&]() {
      ok &= WWAIT(BAR(SFREE + pend_g % NSS), (pend_g / NSS) & 1, 13);       // the tile's last P V has completed
      tc_fence_after();
      uint32_t a[CW];
      tmem_ld16(lane_base + ATF_COL_O + (pend_tt & 1) * 64, a);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(BAR(OFREE + (pend_tt & 1)));              // the accumulator is in registers: the MMA warp may reuse it
#pragma unroll
      for (int e = 0; e < CW / 4; e++)
        *reinterpret_cast<float4*>(pend_row + 4 * e) = make_float4(__uint_as_float(a[4 * e]) * pend_il, __uint_as_float(a[4 * e + 1]) * pend_il, __uint_as_float(a[4 * e + 2]) * pend_il, __uint_as_float(a[4 * e + 3]) * pend_il);
      pend_tt = -1;
    };
    // scale factors of the first tile; those of the following tile are fetched while a tile runs
    float nsc = 0.f, nisv = 0.f;
    if (blockIdx.x < ntiles) { const int z0 = blockIdx.x / ntq; nsc = inv_scale * isq[z0] * isk[z0]; nisv = isv[z0]; }
    for (int id = blockIdx.x, tt = 0; id < ntiles; id += gridDim.x, tt++) {
      int z, q0, nblk; decode(id, tt, z, q0, nblk);
      const int qi = q0 + row; const uint32_t ob = tt & 1;
      const float sc = nsc, isv_z = nisv;                   // accumulator -> scaled score; 1 / scale of V
      const float cs = sc * LOG2E;                          // ... in log2 units
      if (id + (int)gridDim.x < ntiles) { const int zn = (id + (int)gridDim.x) / ntq; nsc = inv_scale * isq[zn] * isk[zn]; nisv = isv[zn]; }
      float m_run = -INFINITY, l_part = 0.f;                // reference maximum (scaled scores), this thread's part of the row sum
      for (int j = 0; j < nblk; j++) {
        const uint32_t g = g0 + j, sb = g % NSS, su = g / NSS; const int key0 = j * ATC_BK + CW * part;
        ok &= WWAIT(BAR(SF + sb), su & 1, 13);
        tc_fence_after();
        uint32_t a[CW];
        tmem_ld16(lane_base + ATF_COL_S + sb * 64, a);
        tmem_wait_ld();
        if (causal && j * ATC_BK + ATC_BK - 1 > q0) {       // the block reaches above the diagonal for some row of the tile
#pragma unroll
          for (int e = 0; e < CW; e++) if (key0 + e > qi) a[e] = __float_as_uint(-INFINITY);
        }
        float bm = -INFINITY;
#pragma unroll
        for (int e = 0; e < CW; e++) bm = fmaxf(bm, __uint_as_float(a[e]));
        float* xb = xch + (xc++ & 1) * (ATC_NPART * 128);
        xb[part * 128 + row] = bm;
        asm volatile("bar.sync 1, %0;" ::"n"(ATC_EW_THREADS) : "memory");
#pragma unroll
        for (int o = 1; o < ATC_NPART; o++) bm = fmaxf(bm, xb[((part + o) & (ATC_NPART - 1)) * 128 + row]);
        // the reference point moves only when the maximum grew by more than 2^ATF_LAZY_LOG2 (the four threads of a row
        // hold the same bm and m_run, so they decide alike)
        const float m_blk = bm * sc;
        const bool move = !((m_blk - m_run) * LOG2E <= ATF_LAZY_LOG2);      // also true for the first block (m_run = -inf)
        const float m_new = move ? fmaxf(m_run, m_blk) : m_run;
        const float corr = move ? fast_ex2((m_run - m_new) * LOG2E) : 1.f;
        const float mneg = -m_new * LOG2E;
        float rs = 0.f, p[CW];
#pragma unroll
        for (int e = 0; e < CW; e++) { p[e] = fast_ex2(fmaf(__uint_as_float(a[e]), cs, mneg)); rs += p[e]; }
        pack_planes16(p, ATF_PSCALE, a);
        tmem_st16(lane_base + ATF_COL_S + sb * 64, a);      // fp16 hi | lo of this thread's 16 keys = one 16-deep step of P V
        l_part = l_part * corr + rs; m_run = m_new;
        // The accumulator may only be touched between P V products; the previous one signals s_free of ITS buffer.
        if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
          ok &= WWAIT(BAR(SFREE + (g - 1) % NSS), ((g - 1) / NSS) & 1, 13);
          tc_fence_after();
          tmem_ld16(lane_base + ATF_COL_O + ob * 64, a);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < CW; e++) a[e] = __float_as_uint(__uint_as_float(a[e]) * corr);
          tmem_st16(lane_base + ATF_COL_O + ob * 64, a);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(BAR(PF + sb));
        if (j == 0 && pend_tt >= 0) write_out();            // the previous tile, now that this tile's first block is on its way
      }
      {
        float* xb = xch + (xc++ & 1) * (ATC_NPART * 128);
        xb[part * 128 + row] = l_part;
        asm volatile("bar.sync 1, %0;" ::"n"(ATC_EW_THREADS) : "memory");
        float l_run = 0.f;
#pragma unroll
        for (int o = 0; o < ATC_NPART; o++) l_run += xb[o * 128 + row];              // the same order in every thread of the row
        const int bz = z / H, h = z % H;
        pend_tt = tt; pend_g = g0 + nblk - 1; pend_il = isv_z * (1.f / ATF_PSCALE) / l_run;
        pend_row = O + ((long)bz * T + qi) * D + (long)h * ATC_HD + CW * part;
        if (part == 0) { Mst[(long)z * T + qi] = m_run; Lst[(long)z * T + qi] = l_run; }
      }
      g0 += nblk;
    }
    if (pend_tt >= 0) write_out();
    (void)ok;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ATF_TMEM_COLS) : "memory");
}

// ------------------------------------------------------------------ backward
// One kernel template, three uses; each CTA owns a tile of 128 rows ("row tile", operand planes resident in shared
// memory) and walks 64-wide blocks of the other index:
//   MODE 0 (dQ): rows = queries.  S = Q K_j^T, dP = dO V_j^T, dS = P (dP - Dv) / sqrt(hd), dQ += dS K_j
//   MODE 1 (dK): rows = keys.     S^T = K Q_i^T, dP^T = V dO_i^T, dS^T likewise,         dK += dS^T Q_i
//   MODE 2 (dV): rows = keys.     S^T = K Q_i^T, P^T,                                     dV += P^T dO_i
// with P = exp(S / sqrt(hd) - m) / l recomputed from the saved row statistics (per row of the tile in MODE 0, per
// column in MODES 1 and 2, staged in shared memory).  R1, R2 = row-tile operands; C1, C2 = block operands of the two
// score-shaped products ([64 rows][64]); C3 = block operand of the accumulating product, taken from TRANSPOSED planes
// ([64 head columns][T]) so that its contraction index runs along the row.
// dS is the A operand of the accumulating product and needs a scale that is constant over the whole tile row (all
// blocks add into one accumulator), so it cannot come from the values: it comes from a bound.  |dP_ij| <= |dO_i| |V_j|
// and |D_i| <= max_j |dP_ij|, P <= 1, so |dS_ij| <= (|dO_i| max_j |V_j| + |D_i|) / sqrt(hd) for a query row and
// (max_i |dO_i| |V_j| + max_i |D_i|) / sqrt(hd) for a key row; the norms come from the scale pass over dO and V.  The
// bound is loose by the usual Cauchy-Schwarz factor, which an fp16 pair absorbs (22 bits down to 2^-17 of the scale).
// TMEM: three sets of {S, dP}; the planes of dS (P^T in MODE 2) are written over dP (over S); two accumulators.
// Warps: 0 = TMA producer; 1, 2 = issuers of the two score-shaped products (S, dP); 3 = issuer of the accumulating
// product; 4-19 elementwise.  The write-out of a finished tile is deferred until the elementwise warps have done the
// first block of the next tile, so that the score pipeline does not wait for it.
constexpr int ATB_NS = 3;
template <int MODE> struct AtbCfg {
  static constexpr int NR = MODE == 2 ? 1 : 2;                                 // row-tile operands, score-shaped products
  static constexpr int SMEM = NR * ATC_R_BYTES + ATB_NS * (NR + 1) * ATC_C_BYTES + 1024 + 512 + 2 * 3 * 64 * 4;
};
constexpr int ATB_NT = 3;                                                                       // TMEM stages of {S, dP}
constexpr uint32_t ATB_COL_S = 0, ATB_COL_DP = 64, ATB_COL_ACC = 128 * ATB_NT, ATB_TMEM_COLS = 512;      // stage t at + 128 t; two accumulators of 64 columns
struct AtbScales {
  const float *ir1, *ir2, *ic1, *ic2, *ic3;      // inverse plane scales per problem
  const float* rnorm;                            // MODES 0, 1: 2-norm of every row of the tile's side of the bound (dO rows / V rows), [Z][T]
  const int* zmaxn;                              // MODES 0, 1: per problem, the largest row norm of the other side (V / dO), float bits
  const int* zmaxd;                              // MODE 1: per problem, max |Dv|, float bits
};
// barriers: r_full 0 | r_empty 1 | c_full 2-4 | c_empty 5-7 | c3_full 8-10 | c3_empty 11-13 | sd_full 14-16 | ds_full 17-19
//           sd_free 20-22 (the accumulating product has read the stage) | tile_done 23 | acc_free 24,25 | drains 26-28
template <int MODE>
__global__ void __launch_bounds__(ATB_THREADS, 1)
attn_tc_bwd_kernel(const __grid_constant__ AttnMaps<10> maps, const float* __restrict__ Mst, const float* __restrict__ Lst, const float* __restrict__ Dv,
                   float* __restrict__ Out, const AtbScales sc, int T, int D, int H, int causal, float inv_scale, int ntiles, int* status, unsigned spin_limit) {
  constexpr int NR = AtbCfg<MODE>::NR, NS = ATB_NS;
  constexpr bool TRANS = MODE != 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sR = smem;                                    // NR row-tile operands
  uint8_t* sC = sR + NR * ATC_R_BYTES;                   // NS stages of NR block operands of the score products
  uint8_t* sC3 = sC + NS * NR * ATC_C_BYTES;             // NS stages
  uint64_t* bars = (uint64_t*)(sC3 + NS * ATC_C_BYTES);
  uint32_t* tmem_slot = (uint32_t*)(bars + 32);
  float* st = (float*)(bars + 64);                       // [2][3][64] column statistics (MODES 1, 2)
  constexpr int NT = ATB_NT, RF = 0, RE = 1, CF = 2, CE = 5, C3F = 8, C3E = 11, SDF = 14, DSF = 17, SDFREE = 20, TDONE = 23, ACCFREE = 24, DRAIN = 26;
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // bounded waits that fail fast, as in the forward kernel
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
    for (int i = 0; i < 29; i++)      // r_empty, c_empty and sd_full collect one commit per score-shaped product
      mbar_init(BAR(i), ((i >= DSF && i < DSF + NT) || i == ACCFREE || i == ACCFREE + 1) ? ATC_EW_THREADS : (i == RE || (i >= CE && i < CE + NS) || (i >= SDF && i < SDF + NT)) ? NR : 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(ATB_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t idesc = make_idesc_f16(128, 64);

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, r0, b0, nb; decode(id, tt, z, r0, b0, nb);
        if (tt > 0 && !WAIT(BAR(RE), (tt - 1) & 1, 21)) { ok = false; break; }
        mbar_expect_tx(BAR(RF), NR * ATC_R_BYTES);
        // maps: R1 = 0,1  R2 = 2,3  C1 = 4,5  C2 = 6,7  C3 = 8,9  (hi, lo each)
        for (int o = 0; o < NR; o++) {
          const uint32_t base = smem_u32(sR + o * ATC_R_BYTES);
          tma_load_3d(base, &maps.m[2 * o], 0, r0, z, BAR(RF));
          tma_load_3d(base + ATC_R_BYTES / 2, &maps.m[2 * o + 1], 0, r0, z, BAR(RF));
        }
        for (int n = 0; n < nb; n++, g++) {
          const uint32_t s = g % NS, u = g / NS; const int row = (b0 + n) * 64;
          if (u > 0 && !WAIT(BAR(CE + s), (u - 1) & 1, 21)) { ok = false; break; }
          mbar_expect_tx(BAR(CF + s), NR * ATC_C_BYTES);
          for (int o = 0; o < NR; o++) {
            const uint32_t base = smem_u32(sC + (s * NR + o) * ATC_C_BYTES);
            tma_load_3d(base, &maps.m[4 + 2 * o], 0, row, z, BAR(CF + s));
            tma_load_3d(base + ATC_C_BYTES / 2, &maps.m[5 + 2 * o], 0, row, z, BAR(CF + s));
          }
          if (u > 0 && !WAIT(BAR(C3E + s), (u - 1) & 1, 22)) { ok = false; break; }
          mbar_expect_tx(BAR(C3F + s), ATC_C_BYTES);
          tma_load_3d(smem_u32(sC3 + s * ATC_C_BYTES), &maps.m[8], row, 0, z, BAR(C3F + s));
          tma_load_3d(smem_u32(sC3 + s * ATC_C_BYTES + ATC_C_BYTES / 2), &maps.m[9], row, 0, z, BAR(C3F + s));
        }
      }
      if (!ok || *(volatile int*)status) for (int i = 0; i < 200; i++) __nanosleep(1000);                 // own copies in flight land before the CTA exits
    }
  } else if (warp == 1 || warp == 2) {
    const int prod = warp - 1;                                // warp 1: S, warp 2: dP
    if (lane == 0 && prod < NR) {
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, r0, b0, nb; decode(id, tt, z, r0, b0, nb);
        if (!WAIT(BAR(RF), tt & 1, 23)) { ok = false; break; }
        const uint32_t ra = smem_u32(sR + prod * ATC_R_BYTES);
        const uint64_t r_hi = make_desc<32>(ra), r_lo = make_desc<32>(ra + ATC_R_BYTES / 2);
        for (int n = 0; n < nb; n++, g++) {
          const uint32_t s = g % NS, u = g / NS, sb = g % NT, su = g / NT;
          if (!WAIT(BAR(CF + s), u & 1, 23)) { ok = false; break; }
          if (su > 0 && !WAIT(BAR(SDFREE + sb), (su - 1) & 1, 23)) { ok = false; break; }    // the accumulating product of block g - NT has read this stage
          tc_fence_after();
          const uint32_t acc = tmem_base + 128 * sb + (prod == 0 ? ATB_COL_S : ATB_COL_DP);
          const uint32_t cb = smem_u32(sC + (s * NR + prod) * ATC_C_BYTES);
          const uint64_t c_hi = make_desc<32>(cb), c_lo = make_desc<32>(cb + ATC_C_BYTES / 2);
#pragma unroll
          for (int k = 0; k < 4; k++) { const uint64_t adv = (uint64_t)(2 * k); mma3_ss(acc, r_hi + adv, r_lo + adv, c_hi + adv, c_lo + adv, idesc, k == 0); }
          tc_commit(BAR(CE + s));
          tc_commit(BAR(SDF + sb));
          if (n == nb - 1) tc_commit(BAR(RE));                 // the row tile may be replaced
        }
      }
      if (!ok || *(volatile int*)status) { tc_commit(BAR(DRAIN + prod)); mbar_wait(BAR(DRAIN + prod), 0, TC_DRAIN_LIMIT); }     // own instructions in flight finish before TMEM is released
    }
  } else if (warp == 3) {
    if (lane == 0) {                                          // accumulating products
      bool ok = true; uint32_t g = 0;
      for (int id = blockIdx.x, tt = 0; id < ntiles && ok; id += gridDim.x, tt++) {
        int z, r0, b0, nb; decode(id, tt, z, r0, b0, nb);
        const uint32_t ab = tt & 1;
        if (tt >= 2 && !WAIT(BAR(ACCFREE + ab), ((tt >> 1) - 1) & 1, 25)) { ok = false; break; }     // this accumulator has been written out
        for (int n = 0; n < nb; n++, g++) {
          const uint32_t s = g % NS, u = g / NS, sb = g % NT, su = g / NT;
          if (!WAIT(BAR(DSF + sb), su & 1, 25) || !WAIT(BAR(C3F + s), u & 1, 25)) { ok = false; break; }
          tc_fence_after();
          const uint32_t cb = smem_u32(sC3 + s * ATC_C_BYTES);
          const uint64_t c_hi = make_desc<32>(cb), c_lo = make_desc<32>(cb + ATC_C_BYTES / 2);
          const uint32_t pa = tmem_base + 128 * sb + (MODE == 2 ? ATB_COL_S : ATB_COL_DP), acc = tmem_base + ATB_COL_ACC + ab * 64;
#pragma unroll
          for (int k = 0; k < 4; k++) { const uint64_t adv = (uint64_t)(2 * k); mma3_ts(acc, pa + 16 * k, c_hi + adv, c_lo + adv, idesc, n == 0 && k == 0); }
          tc_commit(BAR(C3E + s));
          tc_commit(BAR(SDFREE + sb));
          if (n == nb - 1) tc_commit(BAR(TDONE));
        }
      }
      if (!ok || *(volatile int*)status) { tc_commit(BAR(DRAIN + 2)); mbar_wait(BAR(DRAIN + 2), 0, TC_DRAIN_LIMIT); }
    }
  } else {
    // four threads per tile row: `part` selects 16 of the 64 columns of a block (and of the accumulator)
    constexpr int CW = ATC_CW;
    const int quad = warp & 3, part = (warp - 4) >> 2, row = quad * 32 + lane, et = (warp - 4) * 32 + lane;   // et: 0..511
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + CW * part;
    constexpr float LOG2E = 1.44269504088896341f;
    const float oscale = MODE == 2 ? 1.f : inv_scale;
    bool ok = true; uint32_t g0 = 0;
    // write-out of a finished tile: wait for its last accumulating product, scale, store
    float pf_m = 0.f, pf_l = 1.f, pf_d = 0.f;              // TRANS: prefetched statistics of column et of the coming block
    if (TRANS && et < 64 && (int)blockIdx.x < ntiles) {
      int z0, r00, b00, nb0; decode(blockIdx.x, 0, z0, r00, b00, nb0);
      const long i0 = (long)z0 * T + b00 * 64 + et;
      pf_m = Mst[i0]; pf_l = Lst[i0]; if (MODE == 1) pf_d = Dv[i0];
    }
    int pend_tt = -1; float pend_os = 0.f; float* pend_row = nullptr;
    auto write_out = [&]() {
      ok &= WWAIT(BAR(TDONE), pend_tt & 1, 24);
      tc_fence_after();
      uint32_t a[CW];
      tmem_ld16(lane_base + ATB_COL_ACC + (pend_tt & 1) * 64, a);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(BAR(ACCFREE + (pend_tt & 1)));            // the accumulator is in registers: the MMA warp may reuse it
#pragma unroll
      for (int e = 0; e < CW / 4; e++)
        *reinterpret_cast<float4*>(pend_row + 4 * e) = make_float4(__uint_as_float(a[4 * e]) * pend_os, __uint_as_float(a[4 * e + 1]) * pend_os, __uint_as_float(a[4 * e + 2]) * pend_os, __uint_as_float(a[4 * e + 3]) * pend_os);
      pend_tt = -1;
    };
    for (int id = blockIdx.x, tt = 0; id < ntiles; id += gridDim.x, tt++) {
      int z, r0, b0, nb; decode(id, tt, z, r0, b0, nb);
      const int ri = r0 + row; const long sb_ = (long)z * T;
      const float cs = inv_scale * LOG2E * sc.ir1[z] * sc.ic1[z];               // score accumulator -> scaled score in log2 units
      const float idp = MODE == 2 ? 0.f : sc.ir2[z] * sc.ic2[z];                // dP accumulator -> dP
      float mneg_r = 0.f, il_r = 0.f, d_r = 0.f;        // -m log2(e), scale / l, Dv of this row (MODE 0)
      if (!TRANS) { mneg_r = -Mst[sb_ + ri] * LOG2E; il_r = oscale / Lst[sb_ + ri]; d_r = Dv[sb_ + ri]; }
      // scale of this row's dS planes (a bound, see above); P^T in MODE 2 is at most 1
      float a_scale = ATC_PSCALE, a_inv = 1.f / ATC_PSCALE;
      if (MODE == 0) a_scale = row_scale(1.001f * inv_scale * (sc.rnorm[sb_ + ri] * __int_as_float(sc.zmaxn[z]) + fabsf(d_r)), &a_inv);
      if (MODE == 1) a_scale = row_scale(1.001f * inv_scale * (sc.rnorm[sb_ + ri] * __int_as_float(sc.zmaxn[z]) + __int_as_float(sc.zmaxd[z])), &a_inv);
      for (int n = 0; n < nb; n++) {
        const uint32_t g = g0 + n, s2 = g % NT, su = g / NT; const int c0 = (b0 + n) * 64;
        float* stm = st + (g & 1) * 192; float* stl = stm + 64; float* std_ = stm + 128;
        if (TRANS) {
          // column statistics of this block, fetched while the previous block was processed; the next block's (the next
          // tile's first block's) are requested here and arrive under this block's work
          if (et < 64) {
            stm[et] = -pf_m * LOG2E; stl[et] = oscale / pf_l; if (MODE == 1) std_[et] = pf_d;
            long nxt = -1;
            if (n + 1 < nb) nxt = sb_ + c0 + 64 + et;
            else if (id + (int)gridDim.x < ntiles) { int zn, rn, bn0, nbn; decode(id + (int)gridDim.x, tt + 1, zn, rn, bn0, nbn); nxt = (long)zn * T + bn0 * 64 + et; }
            if (nxt >= 0) { pf_m = Mst[nxt]; pf_l = Lst[nxt]; if (MODE == 1) pf_d = Dv[nxt]; }
          }
          asm volatile("bar.sync 1, %0;" ::"n"(ATC_EW_THREADS) : "memory");
        }
        ok &= WWAIT(BAR(SDF + s2), su & 1, 24);
        tc_fence_after();
        uint32_t a[CW], b[CW];
        tmem_ld16(lane_base + 128 * s2 + ATB_COL_S, a);
        if (MODE != 2) tmem_ld16(lane_base + 128 * s2 + ATB_COL_DP, b);
        tmem_wait_ld();
        // does the block reach across the diagonal for some row of the tile?
        const bool diag = causal && (TRANS ? r0 + 127 > c0 : c0 + 63 > r0);
        float v[CW];
#pragma unroll
        for (int e = 0; e < CW; e++) {
          const int col = CW * part + e;
          float x = fast_ex2(fmaf(__uint_as_float(a[e]), cs, TRANS ? stm[col] : mneg_r)) * (TRANS ? stl[col] : il_r);   // P (times 1/sqrt(hd) for dS)
          if (MODE != 2) x *= __uint_as_float(b[e]) * idp - (TRANS ? std_[col] : d_r);                                  // dS
          if (diag && (TRANS ? ri > c0 + col : c0 + col > ri)) x = 0.f;
          v[e] = x;
        }
        pack_planes16(v, a_scale, a);
        tmem_st16(lane_base + 128 * s2 + (MODE == 2 ? ATB_COL_S : ATB_COL_DP), a);      // fp16 hi | lo of this thread's 16 block columns
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(BAR(DSF + s2));
        if (n == 0 && pend_tt >= 0) write_out();            // the previous tile, now that this tile's first block is on its way
      }
      {
        const int bz = z / H, h = z % H;
        pend_tt = tt; pend_os = a_inv * sc.ic3[z];
        pend_row = Out + ((long)bz * T + ri) * D + (long)h * ATC_HD + CW * part;
      }
      g0 += nb;
    }
    if (pend_tt >= 0) write_out();
    (void)ok;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ATB_TMEM_COLS) : "memory");
}

// ------------------------------------------------------------------ operand planes
// Up to four tensors [B*T, D] per launch (blockIdx.z).  Pass 1 finds, per problem z = batch * H + head, the largest
// magnitude (-> the plane scale) and, where wanted, the 2-norm of every row and its maximum per problem (the factors of
// the dS bound).  Pass 2 writes the fp16 hi / lo planes, as rows [Z][T][64] and / or transposed [Z][64][T], from one read.
// One CTA = a 64 x 64 tile (64 tokens of one head); the transposition goes through shared memory.
struct AttnPrepJob {
  const float* X; __half *rh, *rl, *ch, *cl;      // row planes, transposed planes (null = not wanted)
  int* amax; float* inv;                          // [Z]: max |x| as float bits (pass 1), inverse scale (pass 2)
  float* rnorm; int* nmax;                        // optional: [Z][T] row norms, [Z] their maximum as float bits
};
struct AttnPrepJobs { AttnPrepJob j[4]; };
__global__ void __launch_bounds__(256) attn_prep_max_kernel(const AttnPrepJobs jobs, int T, int D, int H) {
  __shared__ float red[33];
  const AttnPrepJob& jb = jobs.j[blockIdx.z];
  const int z = blockIdx.y, b = z / H, h = z % H, t0 = blockIdx.x * 64, i = threadIdx.x, c4 = i & 15, r0 = i >> 4;
  float m = 0.f, nm = 0.f;
#pragma unroll
  for (int r = 0; r < 4; r++) {
    const int row = r0 + 16 * r;
    const float4 x = *reinterpret_cast<const float4*>(jb.X + ((long)b * T + t0 + row) * D + (long)h * 64 + c4 * 4);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
    if (jb.rnorm) {                                        // 16 consecutive lanes hold one row
      float sq = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      const float nr = sqrtf(sq) * 1.0001f;
      if (c4 == 0) jb.rnorm[(long)z * T + t0 + row] = nr;
      nm = fmaxf(nm, nr);
    }
  }
  m = block_max(m, red);
  if (i == 0) { if (!(m <= 3.0e38f)) m = 3.4e38f; atomicMax(jb.amax + z, __float_as_int(m)); }
  if (jb.rnorm) {
    __syncthreads();
    nm = block_max(nm, red);
    if (i == 0) { if (!(nm <= 3.0e38f)) nm = 3.4e38f; atomicMax(jb.nmax + z, __float_as_int(nm)); }
  }
}
__global__ void __launch_bounds__(256) attn_prep_split_kernel(const AttnPrepJobs jobs, int T, int D, int H) {
  __shared__ float tile[64][65];
  const AttnPrepJob& jb = jobs.j[blockIdx.z];
  const int z = blockIdx.y, b = z / H, h = z % H, t0 = blockIdx.x * 64, i = threadIdx.x;
  const int c4 = i & 15, r0 = i >> 4;
  float inv; const float s = row_scale(__int_as_float(jb.amax[z]), &inv);
  if (blockIdx.x == 0 && i == 0) jb.inv[z] = inv;
  float4 x[4];
#pragma unroll
  for (int r = 0; r < 4; r++) x[r] = *reinterpret_cast<const float4*>(jb.X + ((long)b * T + t0 + r0 + 16 * r) * D + (long)h * 64 + c4 * 4);
#pragma unroll
  for (int r = 0; r < 4; r++) {
    const int row = r0 + 16 * r;
    if (jb.rh) {
      uint2 hi, lo; split2_pair(x[r].x, x[r].y, s, hi.x, lo.x); split2_pair(x[r].z, x[r].w, s, hi.y, lo.y);
      const long o = ((long)z * T + t0 + row) * 64 + c4 * 4;
      *reinterpret_cast<uint2*>(jb.rh + o) = hi; *reinterpret_cast<uint2*>(jb.rl + o) = lo;
    }
    if (jb.ch) { tile[row][c4 * 4] = x[r].x; tile[row][c4 * 4 + 1] = x[r].y; tile[row][c4 * 4 + 2] = x[r].z; tile[row][c4 * 4 + 3] = x[r].w; }
  }
  if (jb.ch) {
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; r++) {
      const int d = r0 + 16 * r;                          // head column -> plane row; c4 -> 4 consecutive tokens
      uint2 hi, lo; split2_pair(tile[c4 * 4][d], tile[c4 * 4 + 1][d], s, hi.x, lo.x); split2_pair(tile[c4 * 4 + 2][d], tile[c4 * 4 + 3][d], s, hi.y, lo.y);
      const long o = ((long)z * 64 + d) * T + t0 + c4 * 4;
      *reinterpret_cast<uint2*>(jb.ch + o) = hi; *reinterpret_cast<uint2*>(jb.cl + o) = lo;
    }
  }
}
// per problem, max |Dv| (a factor of the key-side dS bound)
__global__ void __launch_bounds__(128) attn_dmax_kernel(const float* __restrict__ Dv, int T, int* __restrict__ out) {
  __shared__ float red[33];
  float m = 0.f;
  for (int t = threadIdx.x; t < T; t += 128) m = fmaxf(m, fabsf(Dv[(long)blockIdx.x * T + t]));
  m = block_max(m, red);
  if (threadIdx.x == 0) { if (!(m <= 3.0e38f)) m = 3.4e38f; out[blockIdx.x] = __float_as_int(m * 1.0001f); }
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
// The planes of one tensor: hi and lo, as rows [Z][T][64] and / or transposed [Z][64][T]; one inverse scale per problem.
struct AttnPlanes { __half *rh = nullptr, *rl = nullptr, *ch = nullptr, *cl = nullptr; float* inv = nullptr; float* rnorm = nullptr; int* nmax = nullptr; };
// Planes of Q, K and V that a training forward pass leaves behind for the backward pass of the same layer (row and
// transposed planes of each, V's row norms): the backward pass then only has to prepare dO.  Costs 24 bytes per element
// of a projection and layer, kept until the layer's backward pass; if the allocation fails the backward pass prepares
// its operands itself as before.  GONEURON_CUDA_ATTENTION_KEEP_PLANES=0 switches it off.
struct AttnSaved { DevBuf store; bool valid = false; AttnPlanes q, k, v; int B = 0; };
inline bool attn_keep_planes() { static const bool on = [] { const char* e = getenv("GONEURON_CUDA_ATTENTION_KEEP_PLANES"); return !(e && !strcmp(e, "0")); }(); return on; }
// Lays out the storage for `n` tensors (rows / cols / norms wanted per tensor) and runs the two passes.  Storage: the
// context's scratch (slots 2 i = row planes of tensor i, 2 i + 1 = its transposed planes, 8 = per-problem words, 9 = row
// norms), or, when `store` is given, that buffer (planes of tensor i at (2 i) ne and (2 i + 1) ne, then words, then norms).
inline size_t attn_store_floats(int n, int Z, int T) { return (size_t)2 * n * Z * T * ATC_HD + (size_t)Z * 16 + (size_t)Z * T * 2; }
inline int attn_tc_prepare(Ctx* ctx, int n, const float* const* X, const bool* want_rows, const bool* want_cols, const bool* want_norm, AttnPlanes* out,
                           int B, int T, int D, int H, int** zwords_extra, float* store = nullptr) {
  const int Z = B * H; const size_t ne = (size_t)Z * T * ATC_HD;      // elements of a tensor; hi + lo planes = ne floats
  float *words, *norms;
  if (store) { words = store + (size_t)2 * n * ne; norms = words + (size_t)Z * 16; }
  else { GN_TRY(attn_tc_buf(ctx, 8, (size_t)Z * 16, &words)); GN_TRY(attn_tc_buf(ctx, 9, (size_t)Z * T * 2, &norms)); }   // per tensor: amax, inv, nmax; one extra row for the caller
  GN_CUDA(cudaMemsetAsync(words, 0, (size_t)Z * 16 * sizeof(float), ctx->stream));
  AttnPrepJobs jobs{}; int nn = 0;
  for (int i = 0; i < n; i++) {
    AttnPrepJob& j = jobs.j[i]; j.X = X[i];
    if (want_rows[i]) { float* p; if (store) p = store + (size_t)(2 * i) * ne; else GN_TRY(attn_tc_buf(ctx, 2 * i, ne, &p)); j.rh = reinterpret_cast<__half*>(p); j.rl = j.rh + ne; }
    if (want_cols[i]) { float* p; if (store) p = store + (size_t)(2 * i + 1) * ne; else GN_TRY(attn_tc_buf(ctx, 2 * i + 1, ne, &p)); j.ch = reinterpret_cast<__half*>(p); j.cl = j.ch + ne; }
    j.amax = reinterpret_cast<int*>(words) + (size_t)(3 * i) * Z; j.inv = words + (size_t)(3 * i + 1) * Z;
    if (want_norm[i]) {
      if (nn >= 2) return fail(GN_ERR_INVALID_ARG, "attn_tc_prepare: at most two tensors with row norms");
      j.rnorm = norms + (size_t)(nn++) * Z * T; j.nmax = reinterpret_cast<int*>(words) + (size_t)(3 * i + 2) * Z;
    }
    out[i] = AttnPlanes{j.rh, j.rl, j.ch, j.cl, j.inv, j.rnorm, j.nmax};
  }
  if (zwords_extra) *zwords_extra = reinterpret_cast<int*>(words) + (size_t)12 * Z;
  const dim3 grid(T / 64, Z, n);
  GN_LAUNCH(ctx, attn_prep_max_kernel, grid, 256, 0, jobs, T, D, H);
  GN_LAUNCH(ctx, attn_prep_split_kernel, grid, 256, 0, jobs, T, D, H);
  return check_launch("attn_prep");
}
// the two tensor maps (hi, lo) of row planes [Z][T][64] with `box_rows` rows per copy, or of transposed planes [Z][64][T]
inline int attn_tc_maps_rows(Ctx* ctx, CUtensorMap* m, const AttnPlanes& p, int T, int Z, int box_rows) {
  GN_TRY(tc_make_map_bf16_raw(ctx, &m[0], p.rh, ATC_HD, T, ATC_HD, Z, 0, box_rows, 64, CU_TENSOR_MAP_DATA_TYPE_FLOAT16));
  return tc_make_map_bf16_raw(ctx, &m[1], p.rl, ATC_HD, T, ATC_HD, Z, 0, box_rows, 64, CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
}
inline int attn_tc_maps_cols(Ctx* ctx, CUtensorMap* m, const AttnPlanes& p, int T, int Z) {
  GN_TRY(tc_make_map_bf16_raw(ctx, &m[0], p.ch, T, ATC_HD, T, Z, 0, ATC_HD, 64, CU_TENSOR_MAP_DATA_TYPE_FLOAT16));
  return tc_make_map_bf16_raw(ctx, &m[1], p.cl, T, ATC_HD, T, Z, 0, ATC_HD, 64, CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
}
inline int attn_tc_fwd(Ctx* ctx, const float* Q, const float* K, const float* V, float* O, float* M, float* L, int B, int T, int D, int H, int causal,
                       AttnSaved* save = nullptr) {
  const int Z = B * H;
  const float* X[3] = {Q, K, V};
  AttnPlanes p[3];
  if (save) save->valid = false;
  if (save && attn_keep_planes()) {
    const size_t need = attn_store_floats(3, Z, T);
    if (save->store.n < need) {
      GN_CUDA(cudaStreamSynchronize(ctx->stream));
      if (save->store.alloc(need) != GN_OK) { cudaGetLastError(); save = nullptr; }      // no room: the backward pass prepares its own operands
    }
  } else save = nullptr;
  if (save) {
    const bool all[3] = {true, true, true}, norm[3] = {false, false, true};
    GN_TRY(attn_tc_prepare(ctx, 3, X, all, all, norm, p, B, T, D, H, nullptr, save->store.p));
    save->q = p[0]; save->k = p[1]; save->v = p[2]; save->B = B; save->valid = true;
  } else {
    const bool rows[3] = {true, true, false}, cols[3] = {false, false, true}, norm[3] = {false, false, false};
    GN_TRY(attn_tc_prepare(ctx, 3, X, rows, cols, norm, p, B, T, D, H, nullptr));
  }
  AttnMaps<6> maps;
  GN_TRY(attn_tc_maps_rows(ctx, &maps.m[0], p[0], T, Z, ATC_BQ)); GN_TRY(attn_tc_maps_rows(ctx, &maps.m[2], p[1], T, Z, ATC_BK)); GN_TRY(attn_tc_maps_cols(ctx, &maps.m[4], p[2], T, Z));
  GN_CUDA(cudaFuncSetAttribute(attn_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATF_SMEM));
  const int ntq = T / ATC_BQ, ntiles = ntq * Z;
  const int grid = std::min(ntiles, std::max(1, persist_sms(ctx) / ntq) * ntq);      // a multiple of the query blocks per problem
  GN_LAUNCH(ctx, attn_tc_fwd_kernel, grid, ATC_THREADS, ATF_SMEM, maps, O, M, L, (const float*)p[0].inv, (const float*)p[1].inv, (const float*)p[2].inv,
            T, D, H, causal, 1.f / sqrtf((float)ATC_HD), ntiles, ctx->d_status, ctx->spin_limit);
  return check_launch("attn_tc_fwd");
}

template <int MODE>
inline int attn_tc_bwd_launch(Ctx* ctx, const AttnPlanes& r1, const AttnPlanes& r2, const AttnPlanes& c1, const AttnPlanes& c2, const AttnPlanes& c3,
                              const float* rnorm, const int* zmaxn, const int* zmaxd,
                              const float* M, const float* L, const float* Dv, float* out, int B, int T, int D, int H, int causal) {
  const int Z = B * H;
  AttnMaps<10> maps;
  GN_TRY(attn_tc_maps_rows(ctx, &maps.m[0], r1, T, Z, 128)); GN_TRY(attn_tc_maps_rows(ctx, &maps.m[2], r2, T, Z, 128));
  GN_TRY(attn_tc_maps_rows(ctx, &maps.m[4], c1, T, Z, 64)); GN_TRY(attn_tc_maps_rows(ctx, &maps.m[6], c2, T, Z, 64)); GN_TRY(attn_tc_maps_cols(ctx, &maps.m[8], c3, T, Z));
  GN_CUDA(cudaFuncSetAttribute(attn_tc_bwd_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, AtbCfg<MODE>::SMEM));
  AtbScales sc{r1.inv, r2.inv, c1.inv, c2.inv, c3.inv, rnorm, zmaxn, zmaxd};
  const int ntr = T / 128, ntiles = ntr * Z;
  const int grid = std::min(ntiles, std::max(1, persist_sms(ctx) / ntr) * ntr);      // a multiple of the row tiles per problem
  GN_LAUNCH(ctx, attn_tc_bwd_kernel<MODE>, grid, ATB_THREADS, AtbCfg<MODE>::SMEM, maps, M, L, Dv, out, sc, T, D, H, causal, 1.f / sqrtf((float)ATC_HD), ntiles, ctx->d_status, ctx->spin_limit);
  return check_launch("attn_tc_bwd");
}
// dQ, dK, dV from Q, K, V, O, dO and the forward's row statistics; Dv receives the row products dO . O
inline int attn_tc_bwd(Ctx* ctx, const float* Q, const float* K, const float* V, const float* O, const float* dO, const float* M, const float* L, float* Dv,
                       float* dQ, float* dK, float* dV, int B, int T, int D, int H, int causal, AttnSaved* saved = nullptr) {
  const long rows = (long)B * T * H; const int Z = B * H;
  if (D == H * ATC_HD && ((reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(O)) & 15) == 0)
    GN_LAUNCH(ctx, attn_rowdot64_kernel, (unsigned)std::min<long>(cdiv(rows, 32), (long)ctx->sm_count * 16), 256, 0, dO, O, Dv, T, H, rows);
  else GN_LAUNCH(ctx, attn_rowdot_kernel, cdiv(rows, 8), 256, 0, dO, O, Dv, T, D, H, ATC_HD, rows);
  AttnPlanes p[4]; int* zmaxd = nullptr;
  if (saved && saved->valid && saved->B == B) {
    // Q, K, V were prepared by this layer's forward pass: only dO is left
    const float* X[1] = {dO}; const bool yes[1] = {true};
    GN_TRY(attn_tc_prepare(ctx, 1, X, yes, yes, yes, &p[3], B, T, D, H, &zmaxd));
    p[0] = saved->q; p[1] = saved->k; p[2] = saved->v; saved->valid = false;
  } else {
    // tensors: 0 = Q, 1 = K, 2 = V, 3 = dO
    const float* X[4] = {Q, K, V, dO}; const bool rw[4] = {true, true, true, true}, cl[4] = {true, true, false, true}, nm[4] = {false, false, true, true};
    GN_TRY(attn_tc_prepare(ctx, 4, X, rw, cl, nm, p, B, T, D, H, &zmaxd));
  }
  GN_LAUNCH(ctx, attn_dmax_kernel, Z, 128, 0, (const float*)Dv, T, zmaxd);
  const AttnPlanes &q = p[0], &k = p[1], &v = p[2], &g = p[3];
  GN_TRY(attn_tc_bwd_launch<0>(ctx, q, g, k, v, k, g.rnorm, v.nmax, nullptr, M, L, Dv, dQ, B, T, D, H, causal));
  GN_TRY(attn_tc_bwd_launch<1>(ctx, k, v, q, g, q, v.rnorm, g.nmax, zmaxd, M, L, Dv, dK, B, T, D, H, causal));
  GN_TRY(attn_tc_bwd_launch<2>(ctx, k, k, q, q, g, nullptr, nullptr, nullptr, M, L, Dv, dV, B, T, D, H, causal));
  return GN_OK;
}

}  // namespace gn
