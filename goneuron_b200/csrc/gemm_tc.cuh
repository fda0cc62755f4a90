// gemm_tc.cuh -- tensor-core contraction engine (placeholder while the tcgen05 kernel is brought up).
#pragma once
#include "common.cuh"
#include "gemm_simt.cuh"
namespace gn {
inline void tc_init(Ctx* ctx) { ctx->tc_ok = false; }
inline bool gemm_tc_supported(Ctx*, const GemmDesc&) { return false; }
inline bool gemm_tc_eligible(Ctx*, const GemmDesc&) { return false; }
inline int gemm_tc(Ctx*, const GemmDesc&) { return fail(GN_ERR_UNSUPPORTED, "tcgen05 engine not built"); }
}
