// ops_tier.cuh -- per-layer entry points: one layer's kernels on host arrays, so that a single kernel can be compared
// with the CPU restatement (and a failing layer isolated) without running a whole training step.  They launch exactly
// the kernels the training step uses.  Test tier: every call allocates, copies in, runs, copies out.
#pragma once

namespace gn {
struct HostIO {      // device copies of host arrays for one call
  Ctx* c; std::vector<std::unique_ptr<DevBuf>> bufs; int rc = GN_OK;
  explicit HostIO(Ctx* ctx) : c(ctx) {}
  float* in(const float* h, size_t n) { float* d = out(n); if (d && h && rc == GN_OK && copy_h2d(c, d, h, n * 4) != cudaSuccess) rc = fail(GN_ERR_CUDA, "host to device copy failed"); return d; }
  float* out(size_t n) { bufs.emplace_back(new DevBuf()); if (rc == GN_OK) rc = bufs.back()->alloc(std::max<size_t>(n, 4)); return bufs.back()->p; }
  float* zeros(size_t n) { float* d = out(n); if (d && rc == GN_OK && (cudaMemsetAsync(d, 0, std::max<size_t>(n, 4) * 4, c->stream) != cudaSuccess)) rc = fail(GN_ERR_CUDA, "memset failed"); return d; }
  int back(float* h, const float* d, size_t n) { if (!h) return GN_OK; return copy_d2h(c, h, d, n * 4) == cudaSuccess ? GN_OK : fail(GN_ERR_CUDA, "device to host copy failed"); }
};
}  // namespace gn

extern "C" {

int gn_op_layernorm(gn_ctx* ctx, int64_t rows, int n, const float* x, const float* gamma, const float* beta, const float* dy,
                    float* y, float* dx, float* dgamma, float* dbeta) {
  using namespace gn;
  if (!ctx || !ctx->alive || !x || !gamma || !beta || !y || rows <= 0 || n <= 0) return fail(GN_ERR_INVALID_ARG, "op_layernorm: bad argument");
  if (dy && (!dx || !dgamma || !dbeta)) return fail(GN_ERR_INVALID_ARG, "op_layernorm: dy given without dx, dgamma, dbeta");
  Ctx* c = &ctx->c; std::lock_guard<std::mutex> run_lk(c->run_mu); GN_CUDA(cudaSetDevice(c->device));
  HostIO io(c); const size_t tot = (size_t)rows * n;
  float *dX = io.in(x, tot), *dG = io.in(gamma, n), *dB = io.in(beta, n), *dY = io.out(tot), *mean = io.out(rows), *sd = io.out(rows);
  GN_TRY(io.rc);
  GN_TRY(layernorm_forward(c, dX, dG, dB, dY, mean, sd, rows, n));
  GN_TRY(io.back(y, dY, tot));
  if (dy) {
    gn_model tmp; tmp.ctx = ctx;
    float *dDy = io.in(dy, tot), *dDx = io.out(tot), *gG = io.zeros(n), *gB = io.zeros(n);
    GN_TRY(io.rc);
    GN_TRY(layernorm_backward(&tmp, dDy, dX, dG, mean, sd, dDx, gG, gB, rows, n));
    GN_TRY(io.back(dx, dDx, tot)); GN_TRY(io.back(dgamma, gG, n)); GN_TRY(io.back(dbeta, gB, n));
    GN_CUDA(cudaStreamSynchronize(c->stream));
  }
  return GN_OK;
}

int gn_op_conv2d(gn_ctx* ctx, int engine, int B, int in_c, int out_c, int kernel, int stride, int pad, int H, int W, int activation,
                 const float* x, const float* w, const float* bias, const float* dy, float* y, float* dx, float* dw, float* db) {
  using namespace gn;
  if (!ctx || !ctx->alive || !x || !w || !bias || !y || B <= 0 || in_c <= 0 || out_c <= 0 || kernel <= 0 || stride <= 0 || pad < 0 || H <= 0 || W <= 0)
    return fail(GN_ERR_INVALID_ARG, "op_conv2d: bad argument");
  if (dy && (!dx || !dw || !db)) return fail(GN_ERR_INVALID_ARG, "op_conv2d: dy given without dx, dw, db");
  if (activation < GN_ACT_LINEAR || activation > GN_ACT_ELU || activation == GN_ACT_SOFTMAX || activation == GN_ACT_LOGSOFTMAX) return fail(GN_ERR_UNSUPPORTED, "op_conv2d: activation %d", activation);
  Ctx* c = &ctx->c; std::lock_guard<std::mutex> run_lk(c->run_mu); GN_CUDA(cudaSetDevice(c->device));
  ConvShape cs{B, in_c, out_c, kernel, stride, pad, H, W, (H + 2 * pad - kernel) / stride + 1, (W + 2 * pad - kernel) / stride + 1};
  if (cs.oH <= 0 || cs.oW <= 0) return fail(GN_ERR_INVALID_ARG, "op_conv2d: empty output");
  if (engine == 1 && !conv_tc_supported(c, cs)) return fail(GN_ERR_UNSUPPORTED, "op_conv2d: the tensor-core engine does not take this shape");
  const size_t nx = (size_t)B * in_c * H * W, ny = (size_t)B * out_c * cs.oH * cs.oW, nW = (size_t)out_c * in_c * kernel * kernel;
  HostIO io(c);
  float* P = io.out(nW + out_c); GN_TRY(io.rc);                               // W | b, as in the flat parameter layout
  GN_CUDA(copy_h2d(c, P, w, nW * 4)); GN_CUDA(copy_h2d(c, P + nW, bias, (size_t)out_c * 4));
  float *dX = io.in(x, nx), *Z = io.out(ny), *A = io.out(ny);
  GN_TRY(io.rc);
  GN_TRY(conv_forward(c, cs, activation, act_alpha_of(activation, 0), dX, P, Z, A, engine == 1));
  GN_TRY(io.back(y, A, ny));
  if (dy) {
    gn_model tmp; tmp.ctx = ctx;
    float *G = io.in(dy, ny), *gP = io.zeros(nW + out_c), *dDx = io.out(nx);
    GN_TRY(io.rc);
    GN_TRY(conv_backward(&tmp, cs, activation, act_alpha_of(activation, 0), G, dX, P, Z, A, gP, gP + nW, dDx, engine == 1));
    GN_TRY(io.back(dx, dDx, nx)); GN_TRY(io.back(dw, gP, nW)); GN_TRY(io.back(db, gP + nW, out_c));
    GN_CUDA(cudaStreamSynchronize(c->stream));
  }
  return check_status_word(c);
}

int gn_op_softmax_ce(gn_ctx* ctx, int B, int V, int log_softmax, const float* z, const float* y, float* out, float* loss, float* dz) {
  using namespace gn;
  if (!ctx || !ctx->alive || !z || !y || !out || B <= 0 || V <= 0) return fail(GN_ERR_INVALID_ARG, "op_softmax_ce: bad argument");
  Ctx* c = &ctx->c; std::lock_guard<std::mutex> run_lk(c->run_mu); GN_CUDA(cudaSetDevice(c->device));
  HostIO io(c); const size_t tot = (size_t)B * V;
  float *Z = io.in(z, tot), *Y = io.in(y, tot), *A = io.out(tot), *G = io.out(tot), *Ls = io.out(B), *DZ = io.out(tot);
  GN_TRY(io.rc);
  GN_LAUNCH(c, softmax_rows_kernel, B, 256, 0, Z, A, V, log_softmax ? 1 : 0);
  GN_LAUNCH(c, loss_rows_kernel, B, 256, 0, (const float*)A, (const float*)Y, G, Ls, V, (int)GN_LOSS_CROSS_ENTROPY);
  GN_LAUNCH(c, head_jacobian_kernel, B, 256, 0, (const float*)G, (const float*)A, DZ, V, log_softmax ? 1 : 0);
  GN_TRY(check_launch("op_softmax_ce"));
  GN_TRY(io.back(out, A, tot)); GN_TRY(io.back(loss, Ls, B)); GN_TRY(io.back(dz, DZ, tot));
  return GN_OK;
}

int gn_op_lstm(gn_ctx* ctx, int engine, int B, int T, int in_size, int H, const float* x, const float* wx, const float* wh, const float* bias,
               const float* dh_last, float* h_all, float* c_all, float* dgate) {
  using namespace gn;
  if (!ctx || !ctx->alive || !x || !wx || !wh || !bias || !h_all || !c_all || B <= 0 || T <= 0 || in_size <= 0 || H <= 0 || H > 1024) return fail(GN_ERR_INVALID_ARG, "op_lstm: bad argument");
  if (dh_last && !dgate) return fail(GN_ERR_INVALID_ARG, "op_lstm: dh_last given without dgate");
  Ctx* c = &ctx->c; std::lock_guard<std::mutex> run_lk(c->run_mu); GN_CUDA(cudaSetDevice(c->device));
  HostIO io(c); const size_t th = (size_t)B * T * H;
  float *X = io.in(x, (size_t)B * T * in_size), *Wx = io.in(wx, (size_t)4 * H * in_size), *Wh = io.in(wh, (size_t)4 * H * H), *Bi = io.in(bias, (size_t)4 * H);
  float *pre = io.out(th), *C_ = io.out(th), *Hh = io.out(th), *out = io.out((size_t)B * H);
  GN_TRY(io.rc);
  const int threads = ((H + 31) / 32) * 32;
  const size_t smem = ((size_t)H * H + (size_t)in_size * H + 2 * H + in_size) * sizeof(float);
  if (smem > 200 * 1024) return fail(GN_ERR_UNSUPPORTED, "op_lstm: hidden size %d needs %zu bytes of shared memory", H, smem);
  GN_CUDA(cudaFuncSetAttribute(lstm_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int xproj = 0;
  if (engine == 1) {
    GemmDesc g; g.M = B * T; g.N = H; g.K = in_size; g.A = X; g.sa_m = in_size; g.sa_k = 1; g.B = Wx; g.sb_k = 1; g.sb_n = in_size; g.C = pre; g.ldc = H;
    if (!gemm_tc_supported(c, g)) return fail(GN_ERR_UNSUPPORTED, "op_lstm: the tensor-core engine is not available");
    GN_TRY(gemm_tc(c, g)); xproj = 1;
  }
  GN_LAUNCH(c, lstm_fwd_kernel, B, threads, smem, (const float*)X, (const float*)Wx, (const float*)Wh, (const float*)Bi, pre, C_, Hh, out, T, in_size, H, 0, xproj);
  GN_TRY(check_launch("op_lstm forward"));
  GN_TRY(io.back(h_all, Hh, th)); GN_TRY(io.back(c_all, C_, th));
  if (dh_last) {
    float *G = io.in(dh_last, (size_t)B * H), *D = io.out(4 * th);
    GN_TRY(io.rc);
    GN_LAUNCH(c, lstm_bwd_kernel, B, threads, (size_t)4 * H * sizeof(float), (const float*)G, (const float*)Wh, (const float*)Bi, (const float*)pre, (const float*)C_, D, T, H, 0);
    GN_TRY(check_launch("op_lstm backward"));
    GN_TRY(io.back(dgate, D, 4 * th));
  }
  return check_status_word(c);
}

}  // extern "C"
