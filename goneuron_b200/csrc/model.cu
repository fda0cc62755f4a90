// model.cu -- the compiled model (execution plan over device-resident tensors) and the C ABI.
//
// One gn_model owns: the flat parameter buffer, the flat gradient buffer and the Adam moments, all in the
// reference's flat layout (Network.initBuffers, internal/net/net.go:91-127); per-layer activation buffers
// sized for the largest batch seen; and shared scratch.  One gn_train_batch call runs the whole
// Network.TrainBatch (net.go:412-436, :721-784) for a batch on the device.
//
// Batch-level restatement of the per-sample reference semantics:
//  * top-level Dense / Conv2D use each sample's own input and pre-activation (layer.go:488-667);
//  * Dense layers inside MultiHeadAttention / TransformerBlock are called once per token and keep only their
//    LAST call's input and pre-activation (layer.go:352, :496-497, :563-567), so per sample
//        gW = (sum_t dz_t) (x) x_{T-1},   FFN ReLU mask of every token = mask of token T-1
//    which at batch level is  gW = Delta^T * X_last  (a contraction over the batch) with Delta[s] = sum_t dz[s,t];
//  * Embedding gradient: only the last sample of each worker chunk (embedding.go:151-154);
//  * LSTM: see conv_lstm.cuh.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>

#include "common.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "rowops.cuh"
#include "conv_lstm.cuh"
#include "attention.cuh"
#include "attention_tc.cuh"
#include "conv_tc.cuh"
#include "nccl_dl.cuh"

namespace gn {

// ------------------------------------------------------------------ contraction dispatch
static bool force_simt_engine() { static const bool f = [] { const char* e = getenv("GONEURON_CUDA_ENGINE"); return e && strcmp(e, "simt") == 0; }(); return f; }
// Chooses the tensor-core engine for large K-major x K-major products and the SIMT engine for the rest.
static int gemm(Ctx* ctx, const GemmDesc& g) {
  int rc;
  if (!force_simt_engine() && gemm_tc_eligible(ctx, g) && !gemm_outer_small_ok(g)) {     // brackets its kernel launches itself
    GemmDesc h = g; if (!h.b_planes) h.b_planes = wplanes_lookup(ctx, g);                 // weight matrices come with prepared planes
    rc = gemm_tc(ctx, h);
  }
  else { ProfScope prof(ctx); rc = gemm_simt(ctx, g); }
  double nb = (double)g.batch1 * g.batch2;
  double flops = 2.0 * g.M * (double)g.N * g.K * nb;
  if (g.flags & (GEMM_SKIP_UPPER | GEMM_KBEG_AT_M0 | GEMM_KEND_AT_M0)) flops *= 0.5;   // causal: about half the tiles exist
  ctx->gemm_flops += flops; ctx->gemm_launches++;
  return rc;
}
// Y[M,N] = X[M,K] * W[N,K]^T + bias (+R) (act)           -- Dense forward at batch level
static int gemm_nt(Ctx* ctx, int M, int N, int K, const float* X, long ldx, const float* W, const float* bias, float* Y, long ldy,
                   int act = GN_ACT_LINEAR, const float* R = nullptr, long ldr = 0) {
  GemmDesc g; g.M = M; g.N = N; g.K = K; g.A = X; g.sa_m = ldx; g.sa_k = 1; g.B = W; g.sb_k = 1; g.sb_n = K;
  g.C = Y; g.ldc = ldy; g.bias = bias; g.act = act; g.R = R; g.ldr = ldr; return gemm(ctx, g);
}
// dX[M,K] = dZ[M,N] * W[N,K] (+R)                          -- gradIn = W^T dz   (layer.go:631-663)
static int gemm_nn(Ctx* ctx, int M, int N, int K, const float* dZ, long ldz, const float* W, float* dX, long ldx, const float* R = nullptr, long ldr = 0) {
  GemmDesc g; g.M = M; g.N = K; g.K = N; g.A = dZ; g.sa_m = ldz; g.sa_k = 1; g.B = W; g.sb_k = K; g.sb_n = 1;
  g.C = dX; g.ldc = ldx; g.R = R; g.ldr = ldr; return gemm(ctx, g);
}
// gW[N,K] = dZ[R,N]^T * X[R,K]                              -- gradW += dz (x) x   (layer.go:591-625)
static int gemm_tn(Ctx* ctx, int R, int N, int K, const float* dZ, long ldz, const float* X, long ldx, float* gW) {
  GemmDesc g; g.M = N; g.N = K; g.K = R; g.A = dZ; g.sa_m = 1; g.sa_k = ldz; g.B = X; g.sb_k = ldx; g.sb_n = 1;
  g.C = gW; g.ldc = K; return gemm(ctx, g);
}

struct LayerRT;
static bool ffn_planes_possible(Ctx* ctx, const LayerRT& l, int N, const float* w1, const float* w2);

// ------------------------------------------------------------------ model
struct LayerRT {
  gn_layer_desc d{};
  int in_size = 0, out_size = 0;
  int64_t p_off = 0, p_cnt = 0;
  // forward state kept for backward
  DevBuf out, z;                       // activation / pre-activation  [cap, out_size]
  DevBuf q, k, v, att, r1, n1, mid, r2, stat;   // TransformerBlock
  DevBuf att_m, att_l, att_d;          // fused attention: per-row softmax maximum, sum, and dO.O  [batch*heads*T]
  AttnSaved attn_saved;                // tcgen05 attention: operand planes of Q, K, V kept from the training forward pass for the backward pass
  DevBuf gate, up, zlast, rope;        // TransformerBlock variants: SwiGLU projections [tokens, ff]; GELU: last token's pre-activation [batch, ff]; cos | sin table
  int ff_act = GN_ACT_RELU; bool rms = false, use_rope = false;
  DevBuf mid_inv, mid_last;            // FFN hidden activation kept as operand planes (in `mid`): row scales [tokens], fp32 last-token rows [batch, ff]
  bool mid_is_planes = false;          // set by the forward pass, read by the backward pass
  DevBuf pre_i, c_all, h_all, dgate;   // LSTM
  DevBuf idx;                          // int32 payload: MaxPool argmax / embedding token ids
  const float* fin = nullptr;          // input of the last forward call (device pointer, not owned)
  int64_t s_off = 0, s_cnt = 0;        // BatchNorm2D: slice of the model's state buffer (running mean | running variance)
  bool grad_replicated = false;        // multi-GPU: every rank already holds the gradient of the whole global batch (no all-reduce)
  float bn_eps = 1e-5f, bn_mom = 0.1f;
};

}  // namespace gn

struct gn_ctx { gn::Ctx c; bool alive = true; };

struct gn_model {
  gn_ctx* ctx = nullptr;
  std::mutex mu;
  std::vector<gn::LayerRT> L;
  int loss_kind = 0, W = 1;
  int64_t P = 0; int in_size = 0, out_size = 0;
  gn::DevBuf params, grads, m1, v2, state; int64_t NS = 0;
  int cur_first_sample = 0;             // global index of the first sample of the batch being processed (Dropout's stream position)
  int cur_global_batch = 0;             // size of the global batch being processed (all ranks)
  bool wplanes_layerwise = false;       // this step renewed the weight planes layer by layer behind the parameter update
  const float* fwd_planes_src = nullptr; gn::BfPlanes fwd_planes{};     // operand planes of the tensor at fwd_planes_src, written by the LayerNorm that produced it
  float lr = 1e-3f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f; int timestep = 0;
  int cap = 0;                          // batch capacity of the activation buffers
  gn::DevBuf xin, yin, lossg, loss_s, loss_sum;
  std::vector<gn::DevBuf> scratch;      // growable shared scratch, by slot
  float last_inv_batch = 1.f;
  float* h_ret = nullptr;               // pinned host block: [0] loss sum, [1] status word (bits), read back once per step
  gn_step_stats stats{};
  cudaEvent_t ev0 = nullptr, ev1 = nullptr, ar0 = nullptr, ar1 = nullptr, comm_done = nullptr, gather_ev = nullptr;
  std::vector<cudaEvent_t> layer_ev;    // gradient of layer i complete (multi-GPU: releases its all-reduce)
  bool alive = true;
  bool has_lstm = false;
  gn::WeightPlaneTable wplanes;         // prepared tensor-core operand planes of the Dense / TransformerBlock weight matrices
};

namespace gn {

enum Slot { S_BNG = 0, S_EMB, S_GRAM0, S_GRAM1, S_DM, S_ZM, S_W, S_TV, S_G0, S_G1, S_ND0, S_ND1, S_ND2, S_ND3, S_ND4, S_NFF, S_NFF2, S_NFF3, S_RN, S_NFFI, S_LNP0, S_LNI0, S_LNP1, S_LNI1, S_RS32, S_ATT0, S_ATT1, S_DELTA, S_PART, S_PART2, S_DZ, S_SCAN, S_COUNT };

static int ensure(gn_model* m, int slot, size_t n, float** out) {
  if ((int)m->scratch.size() < S_COUNT) m->scratch.resize(S_COUNT);
  DevBuf& b = m->scratch[slot];
  if (b.n < n) { GN_CUDA(cudaStreamSynchronize(m->ctx->c.stream)); GN_TRY(b.alloc(n)); }
  *out = b.p; return GN_OK;
}

// All-gather of equal per-rank pieces on the communication stream, ordered after everything queued on the main stream so
// far; the main stream then waits for the result.  `send` may be the rank's own piece inside `recv` (in place).
static int all_gather_on_comm(gn_model* m, const float* send, float* recv, size_t count_per_rank, const char* what) {
  Ctx* ctx = &m->ctx->c;
  GN_CUDA(cudaEventRecord(m->gather_ev, ctx->stream));
  GN_CUDA(cudaStreamWaitEvent(ctx->comm_stream, m->gather_ev, 0));
  int rc = ctx->nccl->AllGather(send, recv, count_per_rank, NCCL_FLOAT32, ctx->comm, ctx->comm_stream);
  if (rc) return fail(GN_ERR_NCCL, "ncclAllGather(%s): %s", what, ctx->nccl->GetErrorString(rc));
  GN_CUDA(cudaEventRecord(m->gather_ev, ctx->comm_stream));
  GN_CUDA(cudaStreamWaitEvent(ctx->stream, m->gather_ev, 0));
  return GN_OK;
}

static int plan_layers(gn_model* m, const gn_layer_desc* layers, int n) {
  int cur = -1; int64_t off = 0;
  for (int i = 0; i < n; i++) {
    LayerRT l; l.d = layers[i]; const gn_layer_desc& d = l.d;
    switch (d.kind) {
      case GN_LAYER_DENSE:
        if (d.in_size <= 0 || d.out_size <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: Dense sizes must be positive", i);
        if (d.activation < GN_ACT_LINEAR || d.activation > GN_ACT_ELU) return fail(GN_ERR_UNSUPPORTED, "layer %d: activation %d", i, d.activation);
        l.in_size = d.in_size; l.out_size = d.out_size; l.p_cnt = (int64_t)d.in_size * d.out_size + d.out_size; break;
      case GN_LAYER_CONV2D: {
        if (d.in_size <= 0 || d.out_size <= 0 || d.kernel <= 0 || d.stride <= 0 || d.in_h <= 0 || d.in_w <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: bad Conv2D descriptor", i);
        if (d.activation == GN_ACT_SOFTMAX || d.activation == GN_ACT_LOGSOFTMAX) return fail(GN_ERR_UNSUPPORTED, "layer %d: Conv2D with a softmax activation", i);
        if (d.activation < GN_ACT_LINEAR || d.activation > GN_ACT_ELU) return fail(GN_ERR_UNSUPPORTED, "layer %d: activation %d", i, d.activation);
        int oh = (d.in_h + 2 * d.padding - d.kernel) / d.stride + 1, ow = (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1;
        l.in_size = d.in_size * d.in_h * d.in_w; l.out_size = d.out_size * oh * ow;
        l.p_cnt = (int64_t)d.out_size * d.in_size * d.kernel * d.kernel + d.out_size; break; }
      case GN_LAYER_CONV1D: {
        if (d.in_size <= 0 || d.out_size <= 0 || d.kernel <= 0 || d.stride <= 0 || d.padding < 0 || d.in_w <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: bad Conv1D descriptor", i);
        if (d.activation < GN_ACT_LINEAR || d.activation > GN_ACT_ELU || d.activation == GN_ACT_SOFTMAX || d.activation == GN_ACT_LOGSOFTMAX)
          return fail(GN_ERR_UNSUPPORTED, "layer %d: Conv1D activation %d", i, d.activation);
        const int ol = (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1;
        if (ol <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: Conv1D output length %d", i, ol);
        l.in_size = d.in_size * d.in_w; l.out_size = d.out_size * ol; l.p_cnt = (int64_t)d.out_size * d.in_size * d.kernel + d.out_size; break; }
      case GN_LAYER_MAXPOOL2D:
      case GN_LAYER_AVGPOOL2D: {
        if (d.in_size <= 0 || d.kernel <= 0 || d.stride <= 0 || d.padding < 0 || d.in_h <= 0 || d.in_w <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: bad pooling descriptor", i);
        int oh = (d.in_h + 2 * d.padding - d.kernel) / d.stride + 1, ow = (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1;
        l.in_size = d.in_size * d.in_h * d.in_w; l.out_size = d.in_size * oh * ow; break; }
      case GN_LAYER_FLATTEN:
        if (cur < 0) return fail(GN_ERR_INVALID_ARG, "Flatten cannot be the first layer");
        l.in_size = l.out_size = cur; break;
      case GN_LAYER_LSTM_UNROLLED:
        if (d.in_size <= 0 || d.out_size <= 0 || d.seq_len <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: bad LSTM descriptor", i);
        if (d.out_size > 1024) return fail(GN_ERR_UNSUPPORTED, "layer %d: LSTM hidden size > 1024", i);
        l.in_size = d.seq_len * d.in_size; l.out_size = d.return_seq ? d.seq_len * d.out_size : d.out_size;
        l.p_cnt = (int64_t)4 * d.out_size * d.in_size + (int64_t)4 * d.out_size * d.out_size + 4 * d.out_size; m->has_lstm = true; break;
      case GN_LAYER_GRU_UNROLLED:
        if (d.in_size <= 0 || d.out_size <= 0 || d.seq_len <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: bad GRU descriptor", i);
        if (((size_t)2 * d.out_size * d.out_size + 3 * (size_t)d.out_size) * sizeof(float) > 200 * 1024) return fail(GN_ERR_UNSUPPORTED, "layer %d: GRU hidden size %d (both recurrent matrices must fit shared memory)", i, d.out_size);
        l.in_size = d.seq_len * d.in_size; l.out_size = d.return_seq ? d.seq_len * d.out_size : d.out_size;
        l.p_cnt = (int64_t)3 * d.out_size * d.in_size + (int64_t)2 * d.out_size * d.out_size + 3 * d.out_size; break;
      case GN_LAYER_EMBEDDING: {
        int T = d.seq_len; for (int j = i + 1; j < n && T <= 0; j++) T = layers[j].seq_len;
        if (T <= 0 || d.in_size <= 0 || d.out_size <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: Embedding needs vocab, dim and a sequence length", i);
        l.d.seq_len = T; l.in_size = T; l.out_size = T * d.out_size; l.p_cnt = (int64_t)d.in_size * d.out_size; break; }
      case GN_LAYER_POSENC:
        if (d.seq_len <= 0 || d.dim <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: bad PositionalEncoding descriptor", i);
        l.in_size = l.out_size = d.seq_len * d.dim; l.p_cnt = (int64_t)d.seq_len * d.dim; break;
      case GN_LAYER_TRANSFORMER_BLOCK:
        if (d.seq_len <= 0 || d.dim <= 0 || d.heads <= 0 || d.ff_dim <= 0 || d.dim % d.heads) return fail(GN_ERR_INVALID_ARG, "layer %d: bad TransformerBlock descriptor (dim must be divisible by heads)", i);
        if (d.activation != 0 && d.activation != GN_ACT_RELU && d.activation != GN_ACT_GELU && d.activation != GN_ACT_SILU) return fail(GN_ERR_UNSUPPORTED, "layer %d: TransformerBlock feed-forward activation %d", i, d.activation);
        l.ff_act = d.activation == 0 ? GN_ACT_RELU : d.activation; l.rms = d.kernel != 0; l.use_rope = d.stride != 0;
        if (l.use_rope && (d.dim / d.heads) % 2) return fail(GN_ERR_INVALID_ARG, "layer %d: rotary embeddings need an even head size", i);
        l.in_size = l.out_size = d.seq_len * d.dim;
        l.p_cnt = 4 * ((int64_t)d.dim * d.dim + d.dim) + (l.rms ? 2 : 4) * (int64_t)d.dim
                + (l.ff_act == GN_ACT_SILU ? 2 * (int64_t)d.dim * d.ff_dim : (int64_t)d.dim * d.ff_dim + d.ff_dim) + ((int64_t)d.ff_dim * d.dim + d.dim); break;
      case GN_LAYER_CLS_POOLING:
        if (d.seq_len <= 0 || d.dim <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: bad CLSPooling descriptor", i);
        l.in_size = d.seq_len * d.dim; l.out_size = d.dim; break;
      case GN_LAYER_DROPOUT: {
        float pr = 0.f; memcpy(&pr, &d.dim, 4);
        if (d.in_size <= 0 || !(pr >= 0.f && pr < 1.f)) return fail(GN_ERR_INVALID_ARG, "layer %d: bad Dropout descriptor", i);
        if (cur >= 0 && cur != d.in_size) return fail(GN_ERR_INVALID_ARG, "layer %d: Dropout size %d does not match its input %lld", i, d.in_size, (long long)cur);
        if (m->W > 1) return fail(GN_ERR_UNSUPPORTED, "layer %d: Dropout with more than one virtual worker (every worker clone restarts the random stream)", i);
        l.in_size = l.out_size = d.in_size; l.s_off = m->NS; l.s_cnt = 2; m->NS += 2; l.bn_mom = pr; break; }
      case GN_LAYER_BATCHNORM2D:
        if (d.in_size <= 0 || d.in_h <= 0 || d.in_w <= 0) return fail(GN_ERR_INVALID_ARG, "layer %d: bad BatchNorm2D descriptor", i);
        l.in_size = l.out_size = d.in_size * d.in_h * d.in_w; l.p_cnt = 2 * (int64_t)d.in_size; l.s_off = m->NS; l.s_cnt = 2 * (int64_t)d.in_size; m->NS += l.s_cnt;
        if (d.reserved) memcpy(&l.bn_eps, &d.reserved, 4); if (d.dim) memcpy(&l.bn_mom, &d.dim, 4); break;
      case GN_LAYER_LAYERNORM:
        if (cur < 0 || d.dim <= 0 || cur % d.dim) return fail(GN_ERR_INVALID_ARG, "layer %d: LayerNorm width must divide the input size", i);
        l.in_size = l.out_size = cur; l.p_cnt = 2 * (int64_t)d.dim; break;
      case GN_LAYER_RMSNORM:
        if (cur < 0 || d.dim <= 0 || cur % d.dim) return fail(GN_ERR_INVALID_ARG, "layer %d: RMSNorm width must divide the input size", i);
        l.in_size = l.out_size = cur; l.p_cnt = d.dim; l.bn_eps = 1e-5f; if (d.reserved) memcpy(&l.bn_eps, &d.reserved, 4); break;
      default: return fail(GN_ERR_UNSUPPORTED, "layer %d: unknown layer kind %d", i, d.kind);
    }
    if (cur >= 0 && l.in_size != cur) return fail(GN_ERR_INVALID_ARG, "layer %d: input size mismatch: expected %d, got %d", i, l.in_size, cur);
    if (i == 0) m->in_size = l.in_size;
    cur = l.out_size; l.p_off = off; off += l.p_cnt;
    m->L.push_back(std::move(l));
  }
  m->out_size = cur; m->P = off; return GN_OK;
}

// (Re)allocates every per-layer activation buffer for `cap` samples.
static int alloc_activations(gn_model* m, int cap) {
  GN_CUDA(cudaStreamSynchronize(m->ctx->c.stream));
  size_t c = (size_t)cap;
  GN_TRY(m->xin.alloc(c * m->in_size)); GN_TRY(m->yin.alloc(c * m->out_size));
  GN_TRY(m->lossg.alloc(c * m->out_size)); GN_TRY(m->loss_s.alloc(c)); GN_TRY(m->loss_sum.alloc(4));
  for (auto& l : m->L) {
    const gn_layer_desc& d = l.d;
    switch (d.kind) {
      case GN_LAYER_DENSE:
        GN_TRY(l.out.alloc(c * l.out_size));
        if (d.activation != GN_ACT_LINEAR && d.activation != GN_ACT_RELU) GN_TRY(l.z.alloc(c * l.out_size));
        break;
      case GN_LAYER_CONV2D: GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.z.alloc(c * l.out_size)); break;
      case GN_LAYER_MAXPOOL2D: GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.idx.alloc(c * l.out_size)); break;
      case GN_LAYER_AVGPOOL2D: GN_TRY(l.out.alloc(c * l.out_size)); break;
      case GN_LAYER_CONV1D: GN_TRY(l.out.alloc(c * l.out_size)); break;
      case GN_LAYER_DROPOUT: GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.z.alloc(c * l.out_size)); break;      // z = the mask
      case GN_LAYER_FLATTEN: break;
      case GN_LAYER_LSTM_UNROLLED: {
        size_t th = c * d.seq_len * d.out_size;
        GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.pre_i.alloc(th)); GN_TRY(l.c_all.alloc(th)); GN_TRY(l.h_all.alloc(th)); GN_TRY(l.dgate.alloc(4 * th)); break; }
      case GN_LAYER_GRU_UNROLLED: {
        size_t th = c * d.seq_len * d.out_size;     // pre_i: pre-activations [.,T,3H]; c_all: h_{t-1}; z: r (.) h_{t-1}; dgate: deltas [.,T,3H]
        GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.pre_i.alloc(3 * th)); GN_TRY(l.c_all.alloc(th)); GN_TRY(l.h_all.alloc(th)); GN_TRY(l.z.alloc(th)); GN_TRY(l.dgate.alloc(3 * th)); break; }
      case GN_LAYER_EMBEDDING: GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.idx.alloc(c * d.seq_len)); break;
      case GN_LAYER_POSENC: GN_TRY(l.out.alloc(c * l.out_size)); break;
      case GN_LAYER_TRANSFORMER_BLOCK: {
        size_t nd = c * d.seq_len * d.dim, nf = c * d.seq_len * d.ff_dim, nt = c * d.seq_len;
        GN_TRY(l.q.alloc(nd)); GN_TRY(l.k.alloc(nd)); GN_TRY(l.v.alloc(nd)); GN_TRY(l.att.alloc(nd)); GN_TRY(l.r1.alloc(nd)); GN_TRY(l.n1.alloc(nd));
        GN_TRY(l.mid.alloc(nf)); GN_TRY(l.r2.alloc(nd)); GN_TRY(l.out.alloc(nd)); GN_TRY(l.stat.alloc(4 * nt));
        GN_TRY(l.att_m.alloc(nt * d.heads)); GN_TRY(l.att_l.alloc(nt * d.heads)); GN_TRY(l.att_d.alloc(nt * d.heads));
        GN_TRY(l.mid_inv.alloc(nt)); GN_TRY(l.mid_last.alloc(c * d.ff_dim));
        if (l.ff_act == GN_ACT_SILU) { GN_TRY(l.gate.alloc(nf)); GN_TRY(l.up.alloc(nf)); }
        if (l.ff_act == GN_ACT_GELU) GN_TRY(l.zlast.alloc(c * d.ff_dim));
        break; }
      case GN_LAYER_CLS_POOLING: GN_TRY(l.out.alloc(c * l.out_size)); break;
      case GN_LAYER_LAYERNORM: GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.stat.alloc(2 * c * (l.in_size / d.dim))); break;
      case GN_LAYER_RMSNORM: GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.stat.alloc(c * (l.in_size / d.dim))); break;
      case GN_LAYER_BATCHNORM2D: GN_TRY(l.out.alloc(c * l.out_size)); GN_TRY(l.stat.alloc(3 * c * d.in_size)); break;
    }
  }
  m->cap = cap; return GN_OK;
}

static inline unsigned ew_grid(Ctx* ctx, long n, int block = 256) { long g = (n + block - 1) / block; long mx = (long)ctx->sm_count * 16; return (unsigned)std::max<long>(1, std::min(g, mx)); }

// out[c] (=|+=) sum over R rows of in[r*ld + c]
static int colsum(gn_model* m, const float* in, long ld, int R, int C, float* out, bool accumulate) {
  Ctx* ctx = &m->ctx->c;
  int chunks = std::max(1, std::min(R / 64, 128));
  float* part; GN_TRY(ensure(m, S_PART, (size_t)chunks * C * 2, &part));
  GN_LAUNCH(ctx, colsum_partial_kernel, dim3(cdiv(C, 128), chunks), 128, 0, in, ld, R, C, part);
  GN_LAUNCH(ctx, colsum_final_kernel, cdiv(C, 128), 128, 0, part, chunks, C, out, accumulate ? 1 : 0);
  return check_launch("colsum");
}

// LayerNorm forward: the row-in-registers kernel when the row length allows it.
// `po` (optional): the output also as operand planes; *emitted tells the caller whether the kernel that ran could do it
// (the row-in-registers kernels for widths 128, 256, 512, 1024).
static bool layernorm_vec_width(int n) { return n == 128 || n == 256 || n == 512 || n == 1024; }
static int layernorm_forward(Ctx* ctx, const float* x, const float* gamma, const float* beta, float* y, float* mean, float* sd, long rows, int n,
                             const RowPlaneOut* po = nullptr, bool* emitted = nullptr) {
  const bool vec = n % 128 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta)) & 15) == 0;
  const RowPlaneOut out = (po && vec && layernorm_vec_width(n)) ? *po : RowPlaneOut{};
  if (emitted) *emitted = out.p0 != nullptr;
  switch (vec ? n / 128 : 0) {
    case 1: GN_LAUNCH(ctx, layernorm_fwd_vec_kernel<1>, cdiv(rows, 8), 256, 0, x, gamma, beta, y, mean, sd, rows, 1e-5f, out); break;
    case 2: GN_LAUNCH(ctx, layernorm_fwd_vec_kernel<2>, cdiv(rows, 8), 256, 0, x, gamma, beta, y, mean, sd, rows, 1e-5f, out); break;
    case 4: GN_LAUNCH(ctx, layernorm_fwd_vec_kernel<4>, cdiv(rows, 8), 256, 0, x, gamma, beta, y, mean, sd, rows, 1e-5f, out); break;
    case 8: GN_LAUNCH(ctx, layernorm_fwd_vec_kernel<8>, cdiv(rows, 8), 256, 0, x, gamma, beta, y, mean, sd, rows, 1e-5f, out); break;
    default: GN_LAUNCH(ctx, layernorm_fwd_kernel, cdiv(rows, 8), 256, 0, x, gamma, beta, y, mean, sd, rows, n, 1e-5f);
  }
  return check_launch("layernorm_forward");
}


// The two norms of a TransformerBlock: LayerNorm (row mean and deviation in stat[0:rows], stat[rows:2 rows]) or RMSNorm
// (row RMS in stat[0:rows]); rmsnorm.go:157-240, :246-336.
static int block_norm_forward(Ctx* ctx, bool rms, const float* x, const float* gamma, const float* beta, float* y, float* stat, long rows, int n,
                              const RowPlaneOut* po = nullptr, bool* emitted = nullptr) {
  if (emitted) *emitted = false;
  if (!rms) return layernorm_forward(ctx, x, gamma, beta, y, stat, stat + rows, rows, n, po, emitted);
  GN_LAUNCH(ctx, rmsnorm_fwd_kernel, cdiv(rows, 8), 256, 0, x, gamma, y, stat, rows, n, 1e-5f);
  return check_launch("rmsnorm_forward");
}
static int layernorm_backward(gn_model* m, const float* g, const float* x, const float* gamma, const float* mean, const float* sd, float* dx,
                              float* gGamma, float* gBeta, long rows, int n, const RowPlaneOut* po = nullptr, bool* emitted = nullptr);
static int block_norm_backward(gn_model* m, bool rms, const float* g, const float* x, const float* gamma, const float* stat, float* dx, float* gGamma, float* gBeta, long rows, int n,
                               const RowPlaneOut* po = nullptr, bool* emitted = nullptr) {
  if (emitted) *emitted = false;
  if (!rms) return layernorm_backward(m, g, x, gamma, stat, stat + rows, dx, gGamma, gBeta, rows, n, po, emitted);
  Ctx* ctx = &m->ctx->c;
  const int chunks = (int)std::max<long>(1, std::min<long>(rows / 64, 128));
  float* part; GN_TRY(ensure(m, S_PART2, (size_t)chunks * n, &part));
  GN_LAUNCH(ctx, rmsnorm_pgrad_partial_kernel, dim3(cdiv(n, 128), chunks), 128, 0, g, x, stat, rows, n, part);
  GN_LAUNCH(ctx, rmsnorm_pgrad_final_kernel, cdiv(n, 128), 128, 0, part, chunks, n, gGamma);
  GN_LAUNCH(ctx, rmsnorm_bwd_kernel, cdiv(rows, 8), 256, 0, g, x, gamma, stat, dx, rows, n);
  return check_launch("rmsnorm_backward");
}
// cos | sin of the rotary embedding per (position, pair index), with the reference's conversions (transformer.go:217-221):
// theta and position * theta are rounded to float32, cos and sin taken in float64 and rounded to float32.
static int rope_table(Ctx* ctx, LayerRT& l) {
  const int T = l.d.seq_len, hd = l.d.dim / l.d.heads, half = hd / 2;
  if (l.rope.n >= (size_t)T * half * 2) return GN_OK;
  std::vector<float> tab((size_t)T * half * 2);
  for (int t = 0; t < T; t++) for (int i = 0; i < half; i++) {
    const float theta = (float)std::pow(10000.0, -(double)(2 * i) / (double)hd);
    const float mt = (float)t * theta;
    tab[((size_t)t * half + i) * 2] = (float)std::cos((double)mt); tab[((size_t)t * half + i) * 2 + 1] = (float)std::sin((double)mt);
  }
  GN_TRY(l.rope.alloc(tab.size()));
  GN_CUDA(copy_h2d(ctx, l.rope.p, tab.data(), tab.size() * 4)); return GN_OK;
}

// A LayerNorm of a block can hand its output to the next contraction as operand planes (RowPlaneOut) when that
// contraction runs on the tensor-core engine; `slotp` / `sloti` receive the planes and the inverse row scales.
static bool norm_planes_wanted(Ctx* ctx, bool rms, int rows, int n, int consumer_n) {
  static const bool off = getenv("GONEURON_CUDA_NO_NORM_PLANES") != nullptr;
  if (off || rms || force_simt_engine() || !layernorm_vec_width(n)) return false;
  GemmDesc g; g.M = rows; g.N = consumer_n; g.K = n; g.sa_m = n; g.sa_k = 1; g.sb_k = 1; g.sb_n = n;
  return gemm_tc_eligible(ctx, g) && !gemm_outer_small_ok(g);
}
static int norm_planes_alloc(gn_model* m, int slotp, int sloti, int rows, int n, RowPlaneOut* po, BfPlanes* planes, float* rownorm) {
  float *pp, *pi; GN_TRY(ensure(m, slotp, (size_t)rows * n, &pp)); GN_TRY(ensure(m, sloti, (size_t)rows, &pi));
  *planes = BfPlanes{reinterpret_cast<__half*>(pp), pi, rows, n, n, 1};
  *po = RowPlaneOut{planes->p0(), planes->p1(), pi, rownorm};
  return GN_OK;
}

// The fused kernels (attention.cuh) are the default; GONEURON_CUDA_ATTENTION=unfused selects the path that
// materialises the score matrices and runs the five products as batched contractions on the tcgen05 engine.
static bool use_fused_attention(const gn_layer_desc& d) {
  static const bool unfused = [] { const char* e = getenv("GONEURON_CUDA_ATTENTION"); return e && strcmp(e, "unfused") == 0; }();
  return !unfused && attn_fused_supported(d.dim / d.heads, d.dim);
}

// ---------------------------------------------------------------- Conv2D (both paths)
// z / out: [B, outC, oH, oW].  Implicit GEMM on the tensor cores when `allow_tc` and the engine takes the shape (bias
// and ReLU in the epilogue, other activations from the kept pre-activation z); else the direct kernel (writes z and out).
static int conv_forward(Ctx* ctx, const ConvShape& c, int act, float alpha, const float* x, const float* p, float* z, float* out, bool allow_tc) {
  const long n = (long)c.B * c.outC * c.oH * c.oW; const float* bias = p + (long)c.outC * c.inC * c.k * c.k;
  if (allow_tc && conv_tc_supported(ctx, c)) {
    const bool in_epilogue = act == GN_ACT_LINEAR || act == GN_ACT_RELU;
    GN_TRY(conv_tc_forward(ctx, c, x, p, bias, in_epilogue ? out : z, in_epilogue ? act : GN_ACT_LINEAR));
    if (!in_epilogue) GN_LAUNCH(ctx, act_forward_kernel, ew_grid(ctx, n), 256, 0, z, out, n, act, alpha);
  } else GN_LAUNCH(ctx, conv2d_fwd_kernel, ew_grid(ctx, n), 256, 0, x, p, bias, z, out, c, act, alpha);
  return check_launch("conv_forward");
}
// g: gradient with respect to the activation; gW / gb are added to; dx (may be null) is written.
static int conv_backward(gn_model* m, const ConvShape& c, int act, float alpha, const float* g, const float* x, const float* p, const float* z, const float* out,
                         float* gW, float* gb, float* dx, bool allow_tc) {
  Ctx* ctx = &m->ctx->c;
  const long n = (long)c.B * c.outC * c.oH * c.oW; float* dzb; GN_TRY(ensure(m, S_DZ, (size_t)n, &dzb));
  // ReLU'(z) = [z > 0] = [a > 0], so ReLU (and the identity) work from the activation; the others need the pre-activation
  const float* zsrc = (act == GN_ACT_RELU || act == GN_ACT_LINEAR) ? out : z;
  GN_LAUNCH(ctx, act_backward_kernel, ew_grid(ctx, n), 256, 0, g, zsrc, dzb, n, act, alpha);
  const int nW = c.outC * c.inC * c.k * c.k;
  const bool conv_tc = allow_tc && conv_tc_supported(ctx, c);
  if (conv_tc) {
    float* part; GN_TRY(ensure(m, S_PART, (size_t)c.B * (nW + c.outC), &part));
    GN_TRY(conv_tc_wgrad(ctx, c, dzb, x, part, gW, gb));
  } else if (c.k == 3 || c.k == 5 || c.k == 1) {
    const int pairs = c.outC * c.inC, slices = std::max(1, std::min(c.B, (4 * ctx->sm_count + pairs - 1) / pairs)), ng = nW + c.outC;
    float* part; GN_TRY(ensure(m, S_PART, (size_t)slices * ng, &part));
    if (c.k == 3) GN_LAUNCH(ctx, conv2d_wgrad_tile_kernel<3>, dim3(pairs, slices), 256, 0, dzb, x, part, c, slices);
    else if (c.k == 5) GN_LAUNCH(ctx, conv2d_wgrad_tile_kernel<5>, dim3(pairs, slices), 256, 0, dzb, x, part, c, slices);
    else GN_LAUNCH(ctx, conv2d_wgrad_tile_kernel<1>, dim3(pairs, slices), 256, 0, dzb, x, part, c, slices);
    GN_LAUNCH(ctx, conv2d_wgrad_final_kernel, cdiv(ng, 256), 256, 0, part, slices, ng, gW);          // weights, then biases: gb follows gW
  } else GN_LAUNCH(ctx, conv2d_wgrad_kernel, nW + c.outC, 256, 0, dzb, x, gW, gb, c);
  if (dx) {
    const long ni = (long)c.B * c.inC * c.H * c.W;
    if (conv_tc && c.s == 1) { float* wtmp; GN_TRY(ensure(m, S_DELTA, (size_t)nW, &wtmp)); GN_TRY(conv_tc_dgrad(ctx, c, dzb, p, wtmp, dx)); }
    else if (c.s == 1 && c.k == 3) GN_LAUNCH(ctx, conv2d_dgrad_s1_kernel<3>, ew_grid(ctx, ni), 256, 0, dzb, p, dx, c);
    else if (c.s == 1 && c.k == 5) GN_LAUNCH(ctx, conv2d_dgrad_s1_kernel<5>, ew_grid(ctx, ni), 256, 0, dzb, p, dx, c);
    else GN_LAUNCH(ctx, conv2d_dgrad_kernel, ew_grid(ctx, ni), 256, 0, dzb, p, dx, c);
  }
  return check_launch("conv_backward");
}

// ---------------------------------------------------------------- forward
static int attention_forward(gn_model* m, LayerRT& l, int B, float* P) {
  Ctx* ctx = &m->ctx->c; const gn_layer_desc& d = l.d;
  const int T = d.seq_len, D = d.dim, Hh = d.heads, hd = D / Hh; const long TD = (long)T * D, TT = (long)T * T;
  GemmDesc g; g.M = T; g.N = T; g.K = hd; g.A = l.q.p; g.sa_m = D; g.sa_k = 1; g.B = l.k.p; g.sb_k = 1; g.sb_n = D;
  g.C = P; g.ldc = T; g.batch1 = B; g.batch2 = Hh; g.a_b1 = TD; g.a_b2 = hd; g.b_b1 = TD; g.b_b2 = hd; g.c_b1 = Hh * TT; g.c_b2 = TT;
  g.flags = d.causal ? GEMM_SKIP_UPPER : 0;
  GN_TRY(gemm(ctx, g));
  long rows = (long)B * Hh * T;
  float inv_scale = 1.f / sqrtf((float)hd);
  GN_LAUNCH(ctx, attn_softmax_kernel, cdiv(rows, 8), 256, 0, P, T, inv_scale, d.causal, rows);
  GemmDesc o; o.M = T; o.N = hd; o.K = T; o.A = P; o.sa_m = T; o.sa_k = 1; o.B = l.v.p; o.sb_k = D; o.sb_n = 1;
  o.C = l.att.p; o.ldc = D; o.batch1 = B; o.batch2 = Hh; o.a_b1 = Hh * TT; o.a_b2 = TT; o.b_b1 = TD; o.b_b2 = hd; o.c_b1 = TD; o.c_b2 = hd;
  o.flags = d.causal ? GEMM_KEND_AT_M0 : 0;
  return gemm(ctx, o);
}

// Views into a TransformerBlock's slice of a flat buffer: MHA (wQ, wK, wV, wOut, each W | b) | norm1 | norm2 | ff1 | ff2
// (transformer.go:1038-1056).  RMSNorm has a gain only (be1 = be2 = null); a SwiGLU first layer is W (gate) | V (up) without
// biases (w1 = W, v1 = V, b1 = null).
struct BlockParams { const float *wq, *bq, *wk, *bk, *wv, *bv, *wo, *bo, *g1, *be1, *g2, *be2, *w1, *b1, *v1, *w2, *b2; };
static BlockParams block_params(const float* p, int D, int F, bool rms = false, int ff_act = GN_ACT_RELU) {
  BlockParams b; long dd = (long)D * D;
  b.wq = p; b.bq = p + dd; p += dd + D; b.wk = p; b.bk = p + dd; p += dd + D; b.wv = p; b.bv = p + dd; p += dd + D; b.wo = p; b.bo = p + dd; p += dd + D;
  if (rms) { b.g1 = p; b.be1 = nullptr; p += D; b.g2 = p; b.be2 = nullptr; p += D; }
  else { b.g1 = p; b.be1 = p + D; p += 2 * D; b.g2 = p; b.be2 = p + D; p += 2 * D; }
  if (ff_act == GN_ACT_SILU) { b.w1 = p; b.v1 = p + (long)D * F; b.b1 = nullptr; p += 2 * (long)D * F; }
  else { b.w1 = p; b.b1 = p + (long)D * F; b.v1 = nullptr; p += (long)D * F + F; }
  b.w2 = p; b.b2 = p + (long)F * D; return b;
}

static int forward(gn_model* m, const float* x, int B, const float** y_out, bool training) {
  Ctx* ctx = &m->ctx->c;
  GN_TRY(wplanes_refresh(ctx, m->wplanes));          // no-op unless the parameters changed since the last pass
  ctx->weight_planes = &m->wplanes;
  m->fwd_planes_src = nullptr;
  const float* cur = x;
  for (size_t li = 0; li < m->L.size(); li++) {
    LayerRT& l = m->L[li]; const gn_layer_desc& d = l.d; const float* p = m->params.p + l.p_off;
    l.fin = cur;
    switch (d.kind) {
      case GN_LAYER_DENSE: {
        const float* W = p; const float* bias = p + (long)d.in_size * d.out_size;
        if (d.activation == GN_ACT_LINEAR || d.activation == GN_ACT_RELU) {
          GN_TRY(gemm_nt(ctx, B, d.out_size, d.in_size, cur, d.in_size, W, bias, l.out.p, d.out_size, d.activation));
        } else {
          GN_TRY(gemm_nt(ctx, B, d.out_size, d.in_size, cur, d.in_size, W, bias, l.z.p, d.out_size));
          if (d.activation == GN_ACT_SOFTMAX || d.activation == GN_ACT_LOGSOFTMAX)
            GN_LAUNCH(ctx, softmax_rows_kernel, B, 256, 0, l.z.p, l.out.p, d.out_size, d.activation == GN_ACT_LOGSOFTMAX ? 1 : 0);
          else { long n = (long)B * d.out_size; GN_LAUNCH(ctx, act_forward_kernel, ew_grid(ctx, n), 256, 0, l.z.p, l.out.p, n, d.activation, act_alpha_of(d.activation, d.reserved)); }
        }
        cur = l.out.p; break; }
      case GN_LAYER_CONV2D: {
        ConvShape c{B, d.in_size, d.out_size, d.kernel, d.stride, d.padding, d.in_h, d.in_w,
                    (d.in_h + 2 * d.padding - d.kernel) / d.stride + 1, (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1};
        GN_TRY(conv_forward(ctx, c, d.activation, act_alpha_of(d.activation, d.reserved), cur, p, l.z.p, l.out.p, !force_simt_engine()));
        cur = l.out.p; break; }
      case GN_LAYER_MAXPOOL2D: {
        PoolShape c{B, d.in_size, d.kernel, d.stride, d.padding, d.in_h, d.in_w,
                    (d.in_h + 2 * d.padding - d.kernel) / d.stride + 1, (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1};
        long n = (long)B * l.out_size;
        GN_LAUNCH(ctx, maxpool_fwd_kernel, ew_grid(ctx, n), 256, 0, cur, l.out.p, (int*)l.idx.p, c);
        cur = l.out.p; break; }
      case GN_LAYER_CONV1D: {
        Conv1Shape c{B, d.in_size, d.out_size, d.kernel, d.stride, d.padding, d.in_w, (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1};
        long n = (long)B * l.out_size;
        GN_LAUNCH(ctx, conv1d_fwd_kernel, ew_grid(ctx, n), 256, 0, cur, p, p + (long)d.out_size * d.in_size * d.kernel, l.out.p, c, d.activation, act_alpha_of(d.activation, d.reserved));
        cur = l.out.p; break; }
      case GN_LAYER_DROPOUT:
        if (training) {
          const long tot = (long)B * l.in_size;
          GN_LAUNCH(ctx, dropout_fwd_kernel, ew_grid(ctx, cdiv(tot, DROP_RUN)), 256, 0, cur, l.out.p, l.z.p, (const float*)(m->state.p + l.s_off), tot, l.in_size, l.bn_mom,
                    (long)m->cur_first_sample * l.in_size);
          cur = l.out.p;
        }
        break;
      case GN_LAYER_AVGPOOL2D: {
        PoolShape c{B, d.in_size, d.kernel, d.stride, d.padding, d.in_h, d.in_w,
                    (d.in_h + 2 * d.padding - d.kernel) / d.stride + 1, (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1};
        long n = (long)B * l.out_size;
        GN_LAUNCH(ctx, avgpool_fwd_kernel, ew_grid(ctx, n), 256, 0, cur, l.out.p, c);
        cur = l.out.p; break; }
      case GN_LAYER_FLATTEN: break;
      case GN_LAYER_LSTM_UNROLLED: {
        int H = d.out_size, in = d.in_size; int threads = ((H + 31) / 32) * 32;
        size_t smem = ((size_t)H * H + (size_t)in * H + 2 * H + in) * sizeof(float);
        if (smem > 200 * 1024) return fail(GN_ERR_UNSUPPORTED, "LSTM of hidden size %d needs %zu bytes of shared memory", H, smem);
        GN_CUDA(cudaFuncSetAttribute(lstm_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        // The input projection has no recurrence in it: Wx[0:H] x_t for all B*T rows is one contraction on the tensor cores
        // (only the first H of the 4H gate rows receive it, lstm.go:319-326, :1065-1101); the kernel then adds the bias and
        // the recurrent product step by step.
        int xproj = 0;
        {
          GemmDesc g; g.M = B * d.seq_len; g.N = H; g.K = in; g.A = cur; g.sa_m = in; g.sa_k = 1; g.B = p; g.sb_k = 1; g.sb_n = in; g.C = l.pre_i.p; g.ldc = H;
          if (!force_simt_engine() && gemm_tc_supported(ctx, g)) { GN_TRY(gemm_tc(ctx, g)); ctx->gemm_flops += 2.0 * g.M * (double)g.N * g.K; ctx->gemm_launches++; xproj = 1; }
        }
        GN_LAUNCH(ctx, lstm_fwd_kernel, B, threads, smem, cur, p, p + (long)4 * H * in, p + (long)4 * H * in + (long)4 * H * H,
                  l.pre_i.p, l.c_all.p, l.h_all.p, l.out.p, d.seq_len, in, H, d.return_seq, xproj);
        cur = l.out.p; break; }
      case GN_LAYER_GRU_UNROLLED: {
        const int H = d.out_size, in = d.in_size, T = d.seq_len, threads = ((H + 31) / 32) * 32;
        const float* Wx = p; const float* Wh = p + (long)3 * H * in; const float* bias = Wh + (long)2 * H * H;
        // input projection of all three gates and all B*T rows as one contraction (bias in its epilogue), then the recurrence
        GN_TRY(gemm_nt(ctx, B * T, 3 * H, in, cur, in, Wx, bias, l.pre_i.p, 3 * H));
        const size_t smem = ((size_t)2 * H * H + 3 * (size_t)H) * sizeof(float);
        GN_CUDA(cudaFuncSetAttribute(gru_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        GN_LAUNCH(ctx, gru_fwd_kernel, B, threads, smem, Wh, l.pre_i.p, l.h_all.p, l.out.p, T, H, d.return_seq);
        cur = l.out.p; break; }
      case GN_LAYER_EMBEDDING: {
        // fused with a directly following PositionalEncoding
        long tokens = (long)B * d.seq_len; const float* P = nullptr;
        bool fuse = li + 1 < m->L.size() && m->L[li + 1].d.kind == GN_LAYER_POSENC && m->L[li + 1].d.dim == d.out_size;
        if (fuse) P = m->params.p + m->L[li + 1].p_off;
        float* dst = fuse ? m->L[li + 1].out.p : l.out.p;
        GN_LAUNCH(ctx, embedding_fwd_kernel, (unsigned)tokens, 128, 0, cur, p, P, dst, tokens, d.seq_len, d.out_size, d.in_size, (int*)l.idx.p, ctx->d_status);
        cur = dst; if (fuse) li++; break; }
      case GN_LAYER_POSENC: {
        long n = (long)B * l.out_size;
        GN_LAUNCH(ctx, posenc_fwd_kernel, ew_grid(ctx, n), 256, 0, cur, p, l.out.p, n, (long)l.out_size);
        cur = l.out.p; break; }
      case GN_LAYER_TRANSFORMER_BLOCK: {
        const int T = d.seq_len, D = d.dim, F = d.ff_dim; const int N = B * T; BlockParams bp = block_params(p, D, F, l.rms, l.ff_act);
        {   // the Q, K and V projections read the same input: its operand planes come from the LayerNorm that produced it
            // (the previous block's), or are still in the engine's scratch after the first of the three
          GemmDesc g; g.M = N; g.N = D; g.K = D; g.A = cur; g.sa_m = D; g.sa_k = 1; g.sb_k = 1; g.sb_n = D; g.ldc = D;
          const bool have = m->fwd_planes_src == cur && m->fwd_planes.rows == N && m->fwd_planes.K == D;
          if (have) g.a_planes = &m->fwd_planes;
          g.B = bp.wq; g.bias = bp.bq; g.C = l.q.p; GN_TRY(gemm(ctx, g));
          g.reuse_a_planes = true;
          g.B = bp.wk; g.bias = bp.bk; g.C = l.k.p; GN_TRY(gemm(ctx, g));
          g.B = bp.wv; g.bias = bp.bv; g.C = l.v.p; GN_TRY(gemm(ctx, g));
          m->fwd_planes_src = nullptr;
        }
        if (l.use_rope) {   // rotary embeddings on q and k, in place: attention and its backward pass see the rotated tensors (transformer.go:457-461)
          GN_TRY(rope_table(ctx, l));
          const long tot = (long)N * (D / 2);
          GN_LAUNCH(ctx, rope_kernel, ew_grid(ctx, tot), 256, 0, l.q.p, (const float*)l.rope.p, (long)N, T, D, D / d.heads, 1.f);
          GN_LAUNCH(ctx, rope_kernel, ew_grid(ctx, tot), 256, 0, l.k.p, (const float*)l.rope.p, (long)N, T, D, D / d.heads, 1.f);
        }
        if (use_fused_attention(d)) {
          if (attn_tc_supported(ctx, D / d.heads, T, B, d.heads, D)) GN_TRY(attn_tc_fwd(ctx, l.q.p, l.k.p, l.v.p, l.att.p, l.att_m.p, l.att_l.p, B, T, D, d.heads, d.causal, training ? &l.attn_saved : nullptr));
          else GN_TRY(attn_fwd(ctx, D / d.heads, l.q.p, l.k.p, l.v.p, l.att.p, l.att_m.p, l.att_l.p, B, T, D, d.heads, d.causal));
        } else {
          float* P; GN_TRY(ensure(m, S_ATT0, (size_t)B * d.heads * T * T, &P));
          GN_TRY(attention_forward(m, l, B, P));
        }
        GN_TRY(gemm_nt(ctx, N, D, D, l.att.p, D, bp.wo, bp.bo, l.r1.p, D, GN_ACT_LINEAR, cur, D));          // res1 = x + att
        float* st = l.stat.p;
        // norm 1 hands its output to ff1 as operand planes (and the row norms ff1's plane-writing epilogue needs)
        RowPlaneOut po1{}; BfPlanes n1p{}; bool n1_planes = false; float* rn1 = nullptr;
        if (norm_planes_wanted(ctx, l.rms, N, D, F)) { GN_TRY(ensure(m, S_RN, (size_t)N, &rn1)); GN_TRY(norm_planes_alloc(m, S_LNP0, S_LNI0, N, D, &po1, &n1p, rn1)); }
        GN_TRY(block_norm_forward(ctx, l.rms, l.r1.p, bp.g1, bp.be1, l.n1.p, st, (long)N, D, po1.p0 ? &po1 : nullptr, &n1_planes));
        {   // feed-forward: ff1 -> ff2, res2 = norm1 + ff
          GemmDesc g1; g1.M = N; g1.N = F; g1.K = D; g1.A = l.n1.p; g1.sa_m = D; g1.sa_k = 1; g1.B = bp.w1; g1.sb_k = 1; g1.sb_n = D; g1.C = l.mid.p; g1.ldc = F; g1.bias = bp.b1;
          if (n1_planes) g1.a_planes = &n1p;
          const long nf = (long)N * F;
          BfPlanes midp{reinterpret_cast<__half*>(l.mid.p), l.mid_inv.p, N, F, F, 1};
          l.mid_is_planes = ffn_planes_possible(ctx, l, N, bp.w1, bp.w2);
          if (l.mid_is_planes) {
            // the hidden activation is only ever the A operand of ff2 (and, for its last-token rows, a gate and a weight-gradient
            // input): the epilogue writes it as operand planes into the same buffer, no fp32 copy and no split pass
            const WeightPlaneEntry* we = nullptr; wplanes_lookup(ctx, g1, &we);
            float* rn; GN_TRY(ensure(m, S_RN, (size_t)N, &rn));
            TcPlaneOut po{midp, we->maxabs, l.mid_last.p, T};
            g1.act = GN_ACT_RELU; g1.C = nullptr; g1.plane_out = &po; g1.a_rownorm = rn; GN_TRY(gemm(ctx, g1));
          } else if (l.ff_act == GN_ACT_RELU) { g1.act = GN_ACT_RELU; GN_TRY(gemm(ctx, g1)); }
          else if (l.ff_act == GN_ACT_GELU) {
            // the pre-activation of every sequence's last token is what the backward pass differentiates at (layer.go:563-567)
            GN_TRY(gemm(ctx, g1));
            GN_LAUNCH(ctx, last_token_rows_kernel, ew_grid(ctx, (long)B * F), 256, 0, (const float*)l.mid.p, l.zlast.p, T, F, (long)B * F);
            GN_LAUNCH(ctx, act_forward_kernel, ew_grid(ctx, nf), 256, 0, (const float*)l.mid.p, l.mid.p, nf, (int)GN_ACT_GELU, 0.f);
          } else {              // SwiGLU: gate and up projections (no biases) share the input's operand planes
            g1.C = l.gate.p; g1.bias = nullptr; GN_TRY(gemm(ctx, g1));
            g1.B = bp.v1; g1.C = l.up.p; g1.reuse_a_planes = true; GN_TRY(gemm(ctx, g1));
            GN_LAUNCH(ctx, swiglu_fwd_kernel, ew_grid(ctx, nf), 256, 0, (const float*)l.gate.p, (const float*)l.up.p, l.mid.p, nf);
          }
          GemmDesc g2; g2.M = N; g2.N = D; g2.K = F; g2.A = l.mid.p; g2.sa_m = F; g2.sa_k = 1; g2.B = bp.w2; g2.sb_k = 1; g2.sb_n = F; g2.C = l.r2.p; g2.ldc = D; g2.bias = bp.b2; g2.R = l.n1.p; g2.ldr = D;
          if (l.mid_is_planes) g2.a_planes = &midp;
          GN_TRY(gemm(ctx, g2));
        }
        {   // norm 2 hands its output to the next block's projections as operand planes
          RowPlaneOut po2{}; BfPlanes outp{}; bool emitted = false;
          const bool next_is_block = li + 1 < m->L.size() && m->L[li + 1].d.kind == GN_LAYER_TRANSFORMER_BLOCK && m->L[li + 1].d.dim == D && m->L[li + 1].d.seq_len == T;
          if (next_is_block && norm_planes_wanted(ctx, l.rms, N, D, D)) GN_TRY(norm_planes_alloc(m, S_LNP1, S_LNI1, N, D, &po2, &outp, nullptr));
          GN_TRY(block_norm_forward(ctx, l.rms, l.r2.p, bp.g2, bp.be2, l.out.p, st + 2 * N, (long)N, D, po2.p0 ? &po2 : nullptr, &emitted));
          if (emitted) { m->fwd_planes = outp; m->fwd_planes_src = l.out.p; }
        }
        cur = l.out.p; break; }
      case GN_LAYER_CLS_POOLING:
        GN_LAUNCH(ctx, cls_fwd_kernel, B, 128, 0, cur, l.out.p, d.seq_len, d.dim); cur = l.out.p; break;
      case GN_LAYER_BATCHNORM2D: {
        const int C = d.in_size, S = d.in_h * d.in_w; const long BC = (long)B * C; float* run = m->state.p + l.s_off;
        if (training) {
          GN_LAUNCH(ctx, bn_fwd_kernel, (unsigned)BC, 256, 0, cur, p, p + C, l.out.p, l.stat.p, C, S, BC, l.bn_eps);
          if (ctx->world > 1) {
            // the running statistics move once per sample in batch order (batchnorm2d.go:352, :376): every rank gathers the
            // per-sample statistics of the whole global batch and walks them in that order, so the replicas stay identical
            const int GB = m->cur_global_batch;
            if (GB != B * ctx->world) return fail(GN_ERR_INVALID_ARG, "BatchNorm2D on %d ranks needs equal shards (global batch %d, this rank %d)", ctx->world, GB, B);
            float* g; GN_TRY(ensure(m, S_BNG, (size_t)2 * GB * C, &g));
            GN_TRY(all_gather_on_comm(m, l.stat.p, g, (size_t)BC, "BatchNorm2D means"));
            GN_TRY(all_gather_on_comm(m, l.stat.p + 2 * BC, g + (size_t)GB * C, (size_t)BC, "BatchNorm2D variances"));
            GN_LAUNCH(ctx, bn_running_gathered_kernel, cdiv(C, 128), 128, 0, (const float*)g, (const float*)(g + (size_t)GB * C), run, GB, C, l.bn_mom);
          } else GN_LAUNCH(ctx, bn_running_kernel, cdiv(C, 128), 128, 0, l.stat.p, run, B, C, BC, l.bn_mom);
        } else {
          long n = BC * S; GN_LAUNCH(ctx, bn_eval_kernel, ew_grid(ctx, n), 256, 0, cur, p, p + C, run, l.out.p, C, S, n, l.bn_eps);
        }
        cur = l.out.p; break; }
      case GN_LAYER_LAYERNORM: {
        long rows = (long)B * (l.in_size / d.dim);
        GN_TRY(layernorm_forward(ctx, cur, p, p + d.dim, l.out.p, l.stat.p, l.stat.p + rows, rows, d.dim));
        cur = l.out.p; break; }
      case GN_LAYER_RMSNORM: {
        long rows = (long)B * (l.in_size / d.dim);
        GN_LAUNCH(ctx, rmsnorm_fwd_kernel, cdiv(rows, 8), 256, 0, cur, p, l.out.p, l.stat.p, rows, d.dim, l.bn_eps);
        cur = l.out.p; break; }
    }
    GN_TRY(check_launch("forward"));
  }
  *y_out = cur; return GN_OK;
}

// LayerNorm backward: dx, and gGamma / gBeta accumulated into the gradient slice.
static int layernorm_backward(gn_model* m, const float* g, const float* x, const float* gamma, const float* mean, const float* sd, float* dx,
                              float* gGamma, float* gBeta, long rows, int n, const RowPlaneOut* po, bool* emitted) {
  Ctx* ctx = &m->ctx->c;
  const bool vec = n % 128 == 0 && ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(gamma)) & 15) == 0;
  const RowPlaneOut out = (po && vec && layernorm_vec_width(n)) ? *po : RowPlaneOut{};
  if (emitted) *emitted = out.p0 != nullptr;
  if (vec) {
    const int chunks = (int)std::max<long>(1, std::min<long>(rows / 32, 4L * ctx->sm_count));
    float* part; GN_TRY(ensure(m, S_PART2, (size_t)chunks * 2 * n, &part));
    GN_LAUNCH(ctx, layernorm_pgrad_partial_vec_kernel, dim3(cdiv(n, 1024), chunks), 256, 0, g, x, mean, sd, rows, n, part);
    GN_LAUNCH(ctx, layernorm_pgrad_final_kernel, cdiv(n, 32), 1024, 0, part, chunks, n, gGamma, gBeta);
  } else {
    const int chunks = (int)std::max<long>(1, std::min<long>(rows / 64, 128));
    float* part; GN_TRY(ensure(m, S_PART2, (size_t)chunks * 2 * n, &part));
    GN_LAUNCH(ctx, layernorm_pgrad_partial_kernel, dim3(cdiv(n, 128), chunks), 128, 0, g, x, mean, sd, rows, n, part);
    GN_LAUNCH(ctx, layernorm_pgrad_final_kernel, cdiv(n, 32), 1024, 0, part, chunks, n, gGamma, gBeta);
  }
  switch (vec ? n / 128 : 0) {
    case 1: GN_LAUNCH(ctx, layernorm_bwd_vec_kernel<1>, cdiv(rows, 8), 256, 0, g, x, gamma, mean, sd, dx, rows, out); break;
    case 2: GN_LAUNCH(ctx, layernorm_bwd_vec_kernel<2>, cdiv(rows, 8), 256, 0, g, x, gamma, mean, sd, dx, rows, out); break;
    case 4: GN_LAUNCH(ctx, layernorm_bwd_vec_kernel<4>, cdiv(rows, 8), 256, 0, g, x, gamma, mean, sd, dx, rows, out); break;
    case 8: GN_LAUNCH(ctx, layernorm_bwd_vec_kernel<8>, cdiv(rows, 8), 256, 0, g, x, gamma, mean, sd, dx, rows, out); break;
    default: GN_LAUNCH(ctx, layernorm_bwd_kernel, cdiv(rows, 8), 256, 0, g, x, gamma, mean, sd, dx, rows, n);
  }
  return check_launch("layernorm_backward");
}

// ---------------------------------------------------------------- backward
// Gradient of one inner Dense of a TransformerBlock at batch level:
//   gb = sum over all tokens of dz ; gW = Delta^T * X_last with Delta[s] = sum_t dz[s,t], X_last[s] = x[s,T-1]
// `x_last` != null: the last-token inputs as a dense [B, in] array instead of a strided view of x; `dz_planes` != null: dz
// exists only as operand planes.
static int inner_dense_param_grads(gn_model* m, const float* dz, int B, int T, int out, const float* x, int in, float* gW, float* gb,
                                   const float* x_last = nullptr, const BfPlanes* dz_planes = nullptr, const float* dz_rowsum32 = nullptr) {
  Ctx* ctx = &m->ctx->c; float* delta; GN_TRY(ensure(m, S_DELTA, (size_t)B * out, &delta));
  if (dz_rowsum32) GN_LAUNCH(ctx, token_sum_part32_kernel, dim3(cdiv(out, 512), B), 128, 0, dz_rowsum32, T / 32, out, delta);
  else if (dz_planes) GN_LAUNCH(ctx, token_sum_planes_kernel, dim3(cdiv(out, 128), B), dim3(32, 8), 0, (const __half*)dz_planes->p0(), (const __half*)dz_planes->p1(), (const float*)dz_planes->inv_scale, (long)dz_planes->ldp, T, out, delta);
  else if (out % 4 == 0 && ((reinterpret_cast<uintptr_t>(dz) | reinterpret_cast<uintptr_t>(delta)) & 15) == 0)
    GN_LAUNCH(ctx, token_sum_vec_kernel, dim3(cdiv(out, 128), B), dim3(32, 8), 0, dz, T, out, delta);
  else GN_LAUNCH(ctx, token_sum_kernel, dim3(cdiv(out, 128), B), dim3(128, 4), 0, dz, T, out, delta);
  GN_TRY(colsum(m, delta, out, B, out, gb, false));
  if (x_last) return gemm_tn(ctx, B, out, in, delta, out, x_last, (long)in, gW);
  return gemm_tn(ctx, B, out, in, delta, out, x + (long)(T - 1) * in, (long)T * in, gW);
}
// Can the FFN's hidden activation (and its gradient) of this block live as operand planes only?  The two contractions on
// either side must both run on the tensor-core engine with prepared weight planes, and the plane-writing epilogue's shape
// rules must hold.
static bool ffn_planes_possible(Ctx* ctx, const LayerRT& l, int N, const float* w1, const float* w2) {
  static const bool off = getenv("GONEURON_CUDA_NO_PLANE_OUTPUT") != nullptr;
  const gn_layer_desc& d = l.d; const int D = d.dim, F = d.ff_dim;
  if (off || force_simt_engine() || l.ff_act != GN_ACT_RELU || F % 32 || D % 32 || D > 2048 || F % 4) return false;
  if ((reinterpret_cast<uintptr_t>(w1 + (long)D * F) & 15) != 0) return false;                                 // ff1's bias is read with 16-byte loads
  GemmDesc a; a.M = N; a.N = F; a.K = D; a.B = w1; a.sb_k = 1; a.sb_n = D; a.sa_k = 1; a.sa_m = D;            // n1 W1^T        -> planes
  GemmDesc b; b.M = N; b.N = F; b.K = D; b.B = w2; b.sb_k = F; b.sb_n = 1; b.sa_k = 1; b.sa_m = D;            // dR2 W2         -> planes
  GemmDesc c; c.M = N; c.N = D; c.K = F; c.B = w2; c.sb_k = 1; c.sb_n = F; c.sa_k = 1; c.sa_m = F;            // planes W2^T    (consumer, forward)
  GemmDesc e; e.M = N; e.N = D; e.K = F; e.B = w1; e.sb_k = D; e.sb_n = 1; e.sa_k = 1; e.sa_m = F;            // planes W1      (consumer, backward)
  return gemm_tc_eligible(ctx, a) && gemm_tc_eligible(ctx, b) && gemm_tc_eligible(ctx, c) && gemm_tc_eligible(ctx, e) && wplanes_lookup(ctx, a) && wplanes_lookup(ctx, b);
}

static int block_backward(gn_model* m, LayerRT& l, int B, const float* xin, const float* gout, float* dx) {
  Ctx* ctx = &m->ctx->c; const gn_layer_desc& d = l.d;
  const int T = d.seq_len, D = d.dim, F = d.ff_dim, Hh = d.heads, hd = D / Hh; const int N = B * T; const long ND = (long)N * D;
  BlockParams bp = block_params(m->params.p + l.p_off, D, F, l.rms, l.ff_act); BlockParams gp = block_params(m->grads.p + l.p_off, D, F, l.rms, l.ff_act);
  float *dR2, *dM, *comb, *dR1, *dA, *P = nullptr, *dP = nullptr; float* st = l.stat.p;
  const bool fused = use_fused_attention(d);
  GN_TRY(ensure(m, S_ND0, ND, &dR2)); GN_TRY(ensure(m, S_NFF, (size_t)N * F, &dM)); GN_TRY(ensure(m, S_ND1, ND, &comb));
  GN_TRY(ensure(m, S_ND2, ND, &dR1)); GN_TRY(ensure(m, S_ND3, ND, &dA));
  if (!fused) { GN_TRY(ensure(m, S_ATT0, (size_t)B * Hh * T * T, &P)); GN_TRY(ensure(m, S_ATT1, (size_t)B * Hh * T * T, &dP)); }
  // norm 2
  // its result goes to the contraction with W2 as operand planes, with the row norms that contraction's plane-writing epilogue needs
  RowPlaneOut pob{}; BfPlanes dR2p{}; bool dR2_planes = false; float* rnb = nullptr;
  if (norm_planes_wanted(ctx, l.rms, N, D, F)) { GN_TRY(ensure(m, S_RN, (size_t)N, &rnb)); GN_TRY(norm_planes_alloc(m, S_LNP0, S_LNI0, N, D, &pob, &dR2p, rnb)); }
  GN_TRY(block_norm_backward(m, l.rms, gout, l.r2.p, bp.g2, st + 2 * N, dR2, (float*)gp.g2, (float*)gp.be2, (long)N, D, pob.p0 ? &pob : nullptr, &dR2_planes));
  // ff2 then ff1, token by token in the reference (transformer.go:1238-1250)
  GN_TRY(inner_dense_param_grads(m, dR2, B, T, D, l.mid.p, F, (float*)gp.w2, (float*)gp.b2, l.mid_is_planes ? l.mid_last.p : nullptr));
  {
    // dM[s,t,:] = W2^T dR2[s,t,:]; with a ReLU first layer gated by the ReLU pattern of the LAST token of sequence s (fused into the epilogue)
    GemmDesc g; g.M = N; g.N = F; g.K = D; g.A = dR2; g.sa_m = D; g.sa_k = 1; g.B = bp.w2; g.sb_k = F; g.sb_n = 1; g.C = dM; g.ldc = F;
    if (dR2_planes) g.a_planes = &dR2p;
    if (l.mid_is_planes) { g.mask = l.mid_last.p; g.mask_ld = F; g.mask_group = T; }
    else if (l.ff_act == GN_ACT_RELU) { g.mask = l.mid.p + (long)(T - 1) * F; g.mask_ld = (long)T * F; g.mask_group = T; }
    const long nf = (long)N * F;
    if (l.mid_is_planes) {
      // the gradient of the hidden activation likewise only feeds a token sum and the next contraction: planes only
      const WeightPlaneEntry* we = nullptr; wplanes_lookup(ctx, g, &we);
      float *rn, *dinv; GN_TRY(ensure(m, S_RN, (size_t)N, &rn)); GN_TRY(ensure(m, S_NFFI, (size_t)N, &dinv));
      BfPlanes dMp{reinterpret_cast<__half*>(dM), dinv, N, F, F, 1};
      TcPlaneOut po{dMp, we->maxabs, nullptr, 1};
      float* rs32 = nullptr;                               // 32-row sums of dM from the epilogue: the token sums of the ff1 weight gradient
      if (T % 32 == 0 && F % 4 == 0) { GN_TRY(ensure(m, S_RS32, (size_t)(N / 32) * F, &rs32)); po.rowsum32 = rs32; }
      g.C = nullptr; g.plane_out = &po; g.a_rownorm = rn; GN_TRY(gemm(ctx, g));
      GemmDesc h; h.M = N; h.N = D; h.K = F; h.A = dM; h.sa_m = F; h.sa_k = 1; h.B = bp.w1; h.sb_k = D; h.sb_n = 1; h.C = comb; h.ldc = D; h.R = dR2; h.ldr = D; h.a_planes = &dMp;
      GN_TRY(inner_dense_param_grads(m, nullptr, B, T, F, l.n1.p, D, (float*)gp.w1, (float*)gp.b1, nullptr, &dMp, rs32));
      GN_TRY(gemm(ctx, h));
    } else if (l.ff_act != GN_ACT_SILU) {
      GN_TRY(gemm(ctx, g));
      if (l.ff_act == GN_ACT_GELU) GN_LAUNCH(ctx, scale_by_last_deriv_kernel, ew_grid(ctx, nf), 256, 0, dM, (const float*)l.zlast.p, T, F, nf, (int)GN_ACT_GELU);
      GemmDesc h; h.M = N; h.N = D; h.K = F; h.A = dM; h.sa_m = F; h.sa_k = 1; h.B = bp.w1; h.sb_k = D; h.sb_n = 1; h.C = comb; h.ldc = D; h.R = dR2; h.ldr = D;   // combined = gradRes2 + W1^T dz1
      GN_TRY(inner_dense_param_grads(m, dM, B, T, F, l.n1.p, D, (float*)gp.w1, (float*)gp.b1));
      GN_TRY(gemm(ctx, h));
    } else {
      GN_TRY(gemm(ctx, g));
      // SwiGLU keeps every call's state and pops it in reverse (swiglu.go:186-201): token t's gradient meets token T-1-t's
      // input and projections.  The deltas are written at the partner's row, so the weight gradients are plain contractions
      // over all tokens with the layer's inputs; the input gradient comes out in partner order and is reversed when it is
      // added to the residual path.
      float *dGP, *dUP, *Y;
      GN_TRY(ensure(m, S_NFF2, (size_t)nf, &dGP)); GN_TRY(ensure(m, S_NFF3, (size_t)nf, &dUP)); GN_TRY(ensure(m, S_ND3, ND, &Y));
      GN_LAUNCH(ctx, swiglu_bwd_paired_kernel, ew_grid(ctx, nf), 256, 0, (const float*)dM, (const float*)l.gate.p, (const float*)l.up.p, dGP, dUP, T, F, nf);
      GN_TRY(gemm_tn(ctx, N, F, D, dGP, F, l.n1.p, D, (float*)gp.w1));
      GN_TRY(gemm_tn(ctx, N, F, D, dUP, F, l.n1.p, D, (float*)gp.v1));
      GN_TRY(gemm_nn(ctx, N, F, D, dGP, F, bp.w1, Y, D));
      GN_TRY(gemm_nn(ctx, N, F, D, dUP, F, bp.v1, Y, D, Y, D));
      GN_LAUNCH(ctx, add_token_reversed_kernel, ew_grid(ctx, ND), 256, 0, (const float*)dR2, (const float*)Y, comb, T, D, ND);
    }
  }
  // norm 1
  RowPlaneOut poa{}; BfPlanes dR1p{}; bool dR1_planes = false;
  if (norm_planes_wanted(ctx, l.rms, N, D, D)) GN_TRY(norm_planes_alloc(m, S_LNP0, S_LNI0, N, D, &poa, &dR1p, nullptr));      // the planes of dR2 are dead by now
  GN_TRY(block_norm_backward(m, l.rms, comb, l.r1.p, bp.g1, st, dR1, (float*)gp.g1, (float*)gp.be1, (long)N, D, poa.p0 ? &poa : nullptr, &dR1_planes));
  // output projection
  GN_TRY(inner_dense_param_grads(m, dR1, B, T, D, l.att.p, D, (float*)gp.wo, (float*)gp.bo));
  {
    GemmDesc g; g.M = N; g.N = D; g.K = D; g.A = dR1; g.sa_m = D; g.sa_k = 1; g.B = bp.wo; g.sb_k = D; g.sb_n = 1; g.C = dA; g.ldc = D;      // dA = dR1 Wo
    if (dR1_planes) g.a_planes = &dR1p;
    GN_TRY(gemm(ctx, g));
  }
  // attention: recompute P (transformer.go:610-622), then dP, dS, dQ, dK, dV
  float *dQ, *dK, *dV;
  GN_TRY(ensure(m, S_ND0, ND, &dQ)); GN_TRY(ensure(m, S_ND1, ND, &dK)); GN_TRY(ensure(m, S_ND4, ND, &dV));   // dR2 / comb are dead by now
  if (fused) {
    static const bool tc_bwd = [] { const char* e = getenv("GONEURON_CUDA_ATTENTION_BWD"); return !(e && !strcmp(e, "mma")); }();
    if (tc_bwd && attn_tc_supported(ctx, hd, T, B, Hh, D)) GN_TRY(attn_tc_bwd(ctx, l.q.p, l.k.p, l.v.p, l.att.p, dA, l.att_m.p, l.att_l.p, l.att_d.p, dQ, dK, dV, B, T, D, Hh, d.causal, &l.attn_saved));
    else GN_TRY(attn_bwd(ctx, hd, l.q.p, l.k.p, l.v.p, l.att.p, dA, l.att_m.p, l.att_l.p, l.att_d.p, dQ, dK, dV, B, T, D, Hh, d.causal));
  } else {
    const long TD = (long)T * D, TT = (long)T * T; const float inv_scale = 1.f / sqrtf((float)hd); const long rows = (long)B * Hh * T;
    GemmDesc g; g.M = T; g.N = T; g.K = hd; g.A = l.q.p; g.sa_m = D; g.sa_k = 1; g.B = l.k.p; g.sb_k = 1; g.sb_n = D;
    g.C = P; g.ldc = T; g.batch1 = B; g.batch2 = Hh; g.a_b1 = TD; g.a_b2 = hd; g.b_b1 = TD; g.b_b2 = hd; g.c_b1 = Hh * TT; g.c_b2 = TT;
    g.flags = d.causal ? GEMM_SKIP_UPPER : 0; GN_TRY(gemm(ctx, g));
    GN_LAUNCH(ctx, attn_softmax_kernel, cdiv(rows, 8), 256, 0, P, T, inv_scale, d.causal, rows);
    g.A = dA; g.B = l.v.p; g.C = dP; GN_TRY(gemm(ctx, g));                               // dP = dA V^T
    GN_LAUNCH(ctx, attn_ds_kernel, cdiv(rows, 8), 256, 0, P, dP, T, inv_scale, d.causal, rows);   // dP <- dS (scaled)
    GemmDesc q; q.M = T; q.N = hd; q.K = T; q.batch1 = B; q.batch2 = Hh; q.a_b1 = Hh * TT; q.a_b2 = TT; q.b_b1 = TD; q.b_b2 = hd; q.c_b1 = TD; q.c_b2 = hd; q.ldc = D;
    q.sb_k = D; q.sb_n = 1;
    q.A = dP; q.sa_m = T; q.sa_k = 1; q.B = l.k.p; q.C = dQ; q.flags = d.causal ? GEMM_KEND_AT_M0 : 0; GN_TRY(gemm(ctx, q));     // dQ = dS K
    q.A = dP; q.sa_m = 1; q.sa_k = T; q.B = l.q.p; q.C = dK; q.flags = d.causal ? GEMM_KBEG_AT_M0 : 0; GN_TRY(gemm(ctx, q));     // dK = dS^T Q
    q.A = P; q.B = dA; q.C = dV; GN_TRY(gemm(ctx, q));                                                                          // dV = P^T dA
  }
  if (l.use_rope) {   // the conjugate rotation on the gradients of q and k (transformer.go:659-663)
    const long tot = (long)N * (D / 2);
    GN_LAUNCH(ctx, rope_kernel, ew_grid(ctx, tot), 256, 0, dQ, (const float*)l.rope.p, (long)N, T, D, hd, -1.f);
    GN_LAUNCH(ctx, rope_kernel, ew_grid(ctx, tot), 256, 0, dK, (const float*)l.rope.p, (long)N, T, D, hd, -1.f);
  }
  // q, k, v projections; gradIn = dq + dk + dv, block input gradient = gradRes1 + gradIn
  GN_TRY(inner_dense_param_grads(m, dQ, B, T, D, xin, D, (float*)gp.wq, (float*)gp.bq));
  GN_TRY(inner_dense_param_grads(m, dK, B, T, D, xin, D, (float*)gp.wk, (float*)gp.bk));
  GN_TRY(inner_dense_param_grads(m, dV, B, T, D, xin, D, (float*)gp.wv, (float*)gp.bv));
  GN_TRY(gemm_nn(ctx, N, D, D, dQ, D, bp.wq, dx, D, dR1, D));
  GN_TRY(gemm_nn(ctx, N, D, D, dK, D, bp.wk, dx, D, dx, D));
  GN_TRY(gemm_nn(ctx, N, D, D, dV, D, bp.wv, dx, D, dx, D));
  return check_launch("block_backward");
}

static int lstm_backward(gn_model* m, LayerRT& l, size_t li, int B, const float* xin, const float* gout, int global_batch, int first_sample, float* dx) {
  Ctx* ctx = &m->ctx->c; const gn_layer_desc& d = l.d; const int H = d.out_size, in = d.in_size, T = d.seq_len;
  const float* p = m->params.p + l.p_off; const float* Wx = p; const float* Wh = p + (long)4 * H * in; const float* bias = Wh + (long)4 * H * H;
  int threads = ((H + 31) / 32) * 32;
  GN_LAUNCH(ctx, lstm_bwd_kernel, B, threads, (size_t)4 * H * sizeof(float), gout, Wh, bias, l.pre_i.p, l.c_all.p, l.dgate.p, T, H, d.return_seq);
  if (li > 0) GN_TRY(gemm_nn(ctx, B * T, 4 * H, in, l.dgate.p, 4 * H, Wx, dx, in));   // dx_t = Wx^T d_t
  // The clipping recurrence (lstm.go:694, :725-751) walks the rank-1 updates d_k z_k^T of a whole worker chunk in sample
  // order, and a chunk may span ranks.  With more than one rank every rank therefore gathers the update factors of the
  // whole global batch (rows in global sample order, all-gather over NVLink) and runs the identical scan over all chunks:
  // each replica ends up with the complete LSTM gradient, and this layer's slice is not all-reduced.
  const int world = ctx->world; const int GB = world > 1 ? global_batch : B; const int row0 = world > 1 ? first_sample : 0;
  if (world > 1 && GB != B * world) return fail(GN_ERR_INVALID_ARG, "LSTM on %d ranks needs equal shards (global batch %d, this rank %d)", world, GB, B);
  l.grad_replicated = world > 1;
  int chunk = (global_batch + m->W - 1) / m->W, nchunks = (GB + chunk - 1) / chunk;
  {
    // Gram-matrix form of the clipping recurrence (conv_lstm.cuh): the default whenever its matrices fit.  The
    // cluster kernel below runs only for chunks too long for it, or when GONEURON_CUDA_LSTM_SCAN=cluster asks for it.
    static const int mode = [] { const char* e = getenv("GONEURON_CUDA_LSTM_SCAN"); return !e ? 0 : (strcmp(e, "cluster") == 0 ? 1 : (strcmp(e, "gram") == 0 ? 2 : 0)); }();
    const long Kc = (long)chunk * T, n_updates = (long)GB * T, n_local = (long)B * T; const int R4g = 4 * H, ZWg = in + H + 1;
    const bool fits = Kc <= GRAM_MAX_K && (double)nchunks * Kc * Kc * 8 <= 8.0e9;
    if (world > 1 && !(mode != 1 && fits)) return fail(GN_ERR_UNSUPPORTED, "LSTM on more than one GPU needs the Gram form of the clipping recurrence (worker chunk of %ld updates)", Kc);
    if (mode != 1 && fits) {
      float *G0, *G1, *Dm, *Zm, *wv, *res;
      GN_TRY(ensure(m, S_GRAM0, (size_t)nchunks * Kc * Kc, &G0)); GN_TRY(ensure(m, S_GRAM1, (size_t)nchunks * Kc * Kc, &G1));
      GN_TRY(ensure(m, S_DM, (size_t)nchunks * Kc * R4g, &Dm)); GN_TRY(ensure(m, S_ZM, (size_t)nchunks * Kc * ZWg, &Zm));
      GN_TRY(ensure(m, S_W, (size_t)nchunks * Kc, &wv)); GN_TRY(ensure(m, S_SCAN, (size_t)nchunks * R4g * ZWg, &res));
      if ((long)nchunks * Kc > n_updates) {     // the last chunk is short: its unused rows must be zero for the final contraction
        GN_CUDA(cudaMemsetAsync(Dm, 0, (size_t)nchunks * Kc * R4g * 4, ctx->stream)); GN_CUDA(cudaMemsetAsync(Zm, 0, (size_t)nchunks * Kc * ZWg * 4, ctx->stream));
        GN_CUDA(cudaMemsetAsync(wv, 0, (size_t)nchunks * Kc * 4, ctx->stream));
      }
      float* Dloc = Dm + (size_t)row0 * T * R4g; float* Zloc = Zm + (size_t)row0 * T * ZWg;      // this rank's rows inside the global arrays
      GN_LAUNCH(ctx, lstm_gather_updates_kernel, (unsigned)n_local, 128, 0, (const float*)l.dgate.p, xin, (const float*)l.h_all.p, Dloc, Zloc, T, in, H, n_local);
      if (world > 1) {
        GN_TRY(all_gather_on_comm(m, Dloc, Dm, (size_t)n_local * R4g, "LSTM update factors D"));
        GN_TRY(all_gather_on_comm(m, Zloc, Zm, (size_t)n_local * ZWg, "LSTM update factors Z"));
      }
      GemmDesc g; g.M = (int)Kc; g.N = (int)Kc; g.batch1 = nchunks; g.c_b1 = Kc * Kc; g.ldc = Kc; g.flags = GEMM_SKIP_UPPER;
      g.K = R4g; g.A = Dm; g.sa_m = R4g; g.sa_k = 1; g.B = Dm; g.sb_k = 1; g.sb_n = R4g; g.a_b1 = g.b_b1 = Kc * R4g; g.C = G0; GN_TRY(gemm(ctx, g));
      g.K = ZWg; g.A = Zm; g.sa_m = ZWg; g.B = Zm; g.sb_n = ZWg; g.a_b1 = g.b_b1 = Kc * ZWg; g.C = G1; GN_TRY(gemm(ctx, g));
      const long tot = (long)nchunks * Kc * Kc;
      GN_LAUNCH(ctx, lstm_gram_mul_kernel, ew_grid(ctx, tot), 256, 0, G0, (const float*)G1, (int)Kc, tot);
      // cw (double) | v (double, one group) | |g|^2 per chunk (double) live in one scratch slot
      float* tv; GN_TRY(ensure(m, S_TV, (size_t)2 * ((size_t)nchunks * Kc + (size_t)nchunks * GRAM_BS + 2 * nchunks + 2), &tv));
      double* tco = reinterpret_cast<double*>(tv); double* vbuf = tco + (size_t)nchunks * Kc; double* state = vbuf + (size_t)nchunks * GRAM_BS;
      GN_CUDA(cudaFuncSetAttribute(lstm_gram_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GRAM_GROUP_SMEM));
      for (int k0 = 0; k0 < Kc; k0 += GRAM_BS) {
        if (k0 > 0) GN_LAUNCH(ctx, lstm_gram_prefix_kernel, dim3(GRAM_BS, nchunks), 256, 0, (const float*)G0, (const double*)tco, vbuf, (int)Kc, n_updates, k0);
        GN_LAUNCH(ctx, lstm_gram_group_kernel, nchunks, 256, GRAM_GROUP_SMEM, (const float*)G0, tco, (const double*)vbuf, state, (int)Kc, n_updates, k0);
      }
      const long wtot = (long)nchunks * Kc;
      GN_LAUNCH(ctx, lstm_gram_weights_kernel, ew_grid(ctx, wtot), 256, 0, (const double*)tco, wv, (int)Kc, n_updates, wtot);
      const long dtot = (long)nchunks * Kc * R4g;
      GN_LAUNCH(ctx, lstm_scale_rows_kernel, ew_grid(ctx, dtot), 256, 0, Dm, (const float*)wv, R4g, dtot);
      GemmDesc f; f.M = R4g; f.N = ZWg; f.K = (int)Kc; f.batch1 = nchunks; f.A = Dm; f.sa_m = 1; f.sa_k = R4g; f.a_b1 = Kc * R4g;
      f.B = Zm; f.sb_k = ZWg; f.sb_n = 1; f.b_b1 = Kc * ZWg; f.C = res; f.ldc = ZWg; f.c_b1 = (long)R4g * ZWg; GN_TRY(gemm(ctx, f));
      GN_LAUNCH(ctx, lstm_scatter_grad_kernel, cdiv((long)R4g * ZWg, 256), 256, 0, (const float*)res, nchunks, in, H, m->grads.p + l.p_off);
      return check_launch("lstm_backward(gram)");
    }
  }
  const int R4 = 4 * H, ZW = in + H + 1, rpc = (R4 + SCAN_CLUSTER - 1) / SCAN_CLUSTER;
  size_t smem = ((size_t)rpc * ZW + rpc + ZW + 33) * sizeof(float);
  if (smem > 220 * 1024) return fail(GN_ERR_UNSUPPORTED, "LSTM gradient of %d x %d per cluster CTA exceeds shared memory", rpc, ZW);
  float* scan; GN_TRY(ensure(m, S_SCAN, (size_t)nchunks * R4 * ZW, &scan));
  GN_CUDA(cudaFuncSetAttribute(lstm_grad_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg{}; cfg.gridDim = dim3(nchunks * SCAN_CLUSTER); cfg.blockDim = dim3(SCAN_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
  cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = SCAN_CLUSTER; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  GN_CUDA(cudaLaunchKernelEx(&cfg, lstm_grad_scan_kernel, (const float*)l.dgate.p, xin, (const float*)l.h_all.p, scan, T, in, H, B, chunk, 0));
  ctx->launches++;
  // worker gradients are summed in worker order (net.go:694-700)
  GN_LAUNCH(ctx, colsum_final_kernel, cdiv((long)R4 * ZW, 128), 128, 0, scan, nchunks, R4 * ZW, m->grads.p + l.p_off, 0);
  return check_launch("lstm_backward");
}

static int adam_launch(Ctx* ctx, float* p, const float* g, float* m1, float* v, int64_t n, float lr, float b1, float b2, float eps, int t, float grad_scale,
                       const int* status, cudaStream_t stream);

static int backward(gn_model* m, const float* /*x*/, int B, const float* gloss, int global_batch, int first_sample) {
  Ctx* ctx = &m->ctx->c;
  const float* g = gloss;
  float* pp[2] = {nullptr, nullptr}; int flip = 0;
  size_t maxio = 0; for (auto& l : m->L) maxio = std::max<size_t>(maxio, std::max(l.in_size, l.out_size));
  GN_TRY(ensure(m, S_G0, (size_t)B * maxio, &pp[0])); GN_TRY(ensure(m, S_G1, (size_t)B * maxio, &pp[1]));
  // This layer's slice of the flat gradient buffer is final: sum it over the ranks while earlier layers still compute
  // (unless every rank already holds the whole sum), and apply this slice's Adam update right behind it on the
  // communication stream -- the layer's parameters are not read again in this step -- so that neither the exchange
  // nor the optimiser pass is left over when the backward pass ends.  GONEURON_CUDA_COMM=end issues the same sequence
  // for all layers after the backward pass instead (no overlap; for measurements).
  static const bool comm_at_end = [] { const char* e = getenv("GONEURON_CUDA_COMM"); return e && !strcmp(e, "end"); }();
  std::vector<int> deferred;
  auto layer_comm = [&](int li) -> int {
    LayerRT& l = m->L[li]; float* gr = m->grads.p + l.p_off;
    GN_CUDA(cudaEventRecord(m->layer_ev[li], ctx->stream));
    GN_CUDA(cudaStreamWaitEvent(ctx->comm_stream, m->layer_ev[li], 0));
    if (!l.grad_replicated) {
      int rc = ctx->nccl->AllReduce(gr, gr, (size_t)l.p_cnt, NCCL_FLOAT32, NCCL_SUM, ctx->comm, ctx->comm_stream);
      if (rc) return fail(GN_ERR_NCCL, "ncclAllReduce(grads of layer %d): %s", li, ctx->nccl->GetErrorString(rc));
    }
    GN_TRY(adam_launch(ctx, m->params.p + l.p_off, gr, m->m1.p + l.p_off, m->v2.p + l.p_off, l.p_cnt, m->lr, m->b1, m->b2, m->eps, m->timestep + 2,
                       (float)(1.0 / (double)global_batch), ctx->d_status, ctx->comm_stream));
    // ... and the layer's prepared operand planes right behind the update, still hidden behind the earlier layers' backward pass
    if (!m->wplanes.e.empty()) {
      int j0, j1; m->wplanes.layer_range(li, &j0, &j1);
      GN_TRY(wplanes_refresh_range(ctx, m->wplanes, j0, j1, ctx->comm_stream));
      m->wplanes_layerwise = true;
    }
    return GN_OK;
  };
  for (int li = (int)m->L.size() - 1; li >= 0; li--) {
    LayerRT& l = m->L[li]; const gn_layer_desc& d = l.d;
    const float* xin = l.fin;
    const float* p = m->params.p + l.p_off; float* gr = m->grads.p + l.p_off;
    float* dx = pp[flip]; bool need_dx = li > 0;
    switch (d.kind) {
      case GN_LAYER_DENSE: {
        const float* W = p; long wn = (long)d.in_size * d.out_size; const float* dz = g;
        if (d.activation != GN_ACT_LINEAR) {
          float* dzb; GN_TRY(ensure(m, S_DZ, (size_t)B * d.out_size, &dzb)); long n = (long)B * d.out_size;
          if (d.activation == GN_ACT_SOFTMAX || d.activation == GN_ACT_LOGSOFTMAX)
            GN_LAUNCH(ctx, head_jacobian_kernel, B, 256, 0, g, l.out.p, dzb, d.out_size, d.activation == GN_ACT_LOGSOFTMAX ? 1 : 0);
          else GN_LAUNCH(ctx, act_backward_kernel, ew_grid(ctx, n), 256, 0, g, d.activation == GN_ACT_RELU ? l.out.p : l.z.p, dzb, n, d.activation, act_alpha_of(d.activation, d.reserved));
          dz = dzb;
        }
        GN_TRY(colsum(m, dz, d.out_size, B, d.out_size, gr + wn, false));
        GN_TRY(gemm_tn(ctx, B, d.out_size, d.in_size, dz, d.out_size, xin, d.in_size, gr));
        if (need_dx) { GN_TRY(gemm_nn(ctx, B, d.out_size, d.in_size, dz, d.out_size, W, dx, d.in_size)); g = dx; flip ^= 1; }
        break; }
      case GN_LAYER_CONV2D: {
        ConvShape c{B, d.in_size, d.out_size, d.kernel, d.stride, d.padding, d.in_h, d.in_w,
                    (d.in_h + 2 * d.padding - d.kernel) / d.stride + 1, (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1};
        const int nW = d.out_size * d.in_size * d.kernel * d.kernel;
        GN_TRY(conv_backward(m, c, d.activation, act_alpha_of(d.activation, d.reserved), g, xin, p, l.z.p, l.out.p, gr, gr + nW, need_dx ? dx : nullptr, !force_simt_engine()));
        if (need_dx) { g = dx; flip ^= 1; }
        break; }
      case GN_LAYER_MAXPOOL2D: {
        PoolShape c{B, d.in_size, d.kernel, d.stride, d.padding, d.in_h, d.in_w,
                    (d.in_h + 2 * d.padding - d.kernel) / d.stride + 1, (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1};
        GN_CUDA(cudaMemsetAsync(dx, 0, (size_t)B * l.in_size * sizeof(float), ctx->stream));
        long n = (long)B * l.out_size;
        GN_LAUNCH(ctx, maxpool_bwd_kernel, ew_grid(ctx, n), 256, 0, g, (const int*)l.idx.p, dx, c);
        g = dx; flip ^= 1; break; }
      case GN_LAYER_CONV1D: {
        Conv1Shape c{B, d.in_size, d.out_size, d.kernel, d.stride, d.padding, d.in_w, (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1};
        const int nW = d.out_size * d.in_size * d.kernel;
        GN_LAUNCH(ctx, conv1d_wgrad_kernel, nW + d.out_size, 256, 0, g, xin, gr, gr + nW, c);
        if (need_dx) { long ni = (long)B * l.in_size; GN_LAUNCH(ctx, conv1d_dgrad_kernel, ew_grid(ctx, ni), 256, 0, g, p, dx, c); g = dx; flip ^= 1; }
        break; }
      case GN_LAYER_DROPOUT:
        if (need_dx) { long n = (long)B * l.in_size; GN_LAUNCH(ctx, dropout_bwd_kernel, ew_grid(ctx, n), 256, 0, g, (const float*)l.z.p, dx, n, l.bn_mom); g = dx; flip ^= 1; }
        break;
      case GN_LAYER_AVGPOOL2D: {
        PoolShape c{B, d.in_size, d.kernel, d.stride, d.padding, d.in_h, d.in_w,
                    (d.in_h + 2 * d.padding - d.kernel) / d.stride + 1, (d.in_w + 2 * d.padding - d.kernel) / d.stride + 1};
        if (need_dx) { long n = (long)B * l.in_size; GN_LAUNCH(ctx, avgpool_bwd_kernel, ew_grid(ctx, n), 256, 0, g, dx, c); g = dx; flip ^= 1; }
        break; }
      case GN_LAYER_FLATTEN: break;
      case GN_LAYER_LSTM_UNROLLED:
        GN_TRY(lstm_backward(m, l, li, B, xin, g, global_batch, first_sample, dx)); if (need_dx) { g = dx; flip ^= 1; } break;
      case GN_LAYER_GRU_UNROLLED: {
        const int H = d.out_size, in = d.in_size, T = d.seq_len, threads = ((H + 31) / 32) * 32;
        const float* Wx = p; const float* Wh = p + (long)3 * H * in;
        float* gWx = gr; float* gWh = gr + (long)3 * H * in; float* gb = gWh + (long)2 * H * H;
        GN_LAUNCH(ctx, gru_bwd_kernel, B, threads, (size_t)2 * H * sizeof(float), g, Wh, (const float*)l.pre_i.p, (const float*)l.h_all.p, l.dgate.p, l.c_all.p, l.z.p, T, H, d.return_seq);
        // input weights and biases: every step's delta meets the input of the LAST forward call (gru.go:429-447), so per sample
        // gWx = (sum_t d_t) (x) x_{T-1}: the same batch-level contraction as the inner Dense layers of a TransformerBlock
        GN_TRY(inner_dense_param_grads(m, l.dgate.p, B, T, 3 * H, xin, in, gWx, gb));
        // recurrent weights: update rows from h_{t-1}, reset rows from the candidate's delta and r (.) h_{t-1} (gru.go:450-476)
        GN_TRY(gemm_tn(ctx, B * T, H, H, l.dgate.p, 3 * H, l.c_all.p, H, gWh));
        GN_TRY(gemm_tn(ctx, B * T, H, H, l.dgate.p + 2 * H, 3 * H, l.z.p, H, gWh + (long)H * H));
        if (need_dx) { GN_TRY(gemm_nn(ctx, B * T, 3 * H, in, l.dgate.p, 3 * H, Wx, dx, in)); g = dx; flip ^= 1; }
        break; }
      case GN_LAYER_EMBEDDING: {
        // Only the last sample of every worker chunk reaches the table (embedding.go:151-154): global samples
        // c*chunk + chunk - 1 and the very last one.
        const int chunk = (global_batch + m->W - 1) / m->W, T = d.seq_len, dim = d.out_size;
        const int nq = (global_batch + chunk - 1) / chunk;                       // qualifying samples of the global batch
        auto q_sample = [&](int q) { return std::min(global_batch - 1, q * chunk + chunk - 1); };
        const size_t smem = (size_t)T * sizeof(int);
        if (smem > 48 * 1024) GN_CUDA(cudaFuncSetAttribute(embedding_bwd_sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const bool sparse = ctx->world > 1 && (double)nq * T * (dim + 1) < 0.5 * (double)l.p_cnt;
        if (sparse) {
          // few samples, large table: exchange those samples' rows (nq * T * (dim + 1) floats) instead of all-reducing the table;
          // every rank then builds the complete table gradient itself
          float* buf; GN_TRY(ensure(m, S_EMB, (size_t)nq * T * (dim + 1) + (size_t)nq * T, &buf));
          float* rows = buf; float* idsf = buf + (size_t)nq * T * dim; int* idsi = reinterpret_cast<int*>(idsf + (size_t)nq * T);
          GN_CUDA(cudaMemsetAsync(buf, 0, (size_t)nq * T * (dim + 1) * sizeof(float), ctx->stream));
          for (int q = 0; q < nq; q++) {
            const int sl = q_sample(q) - first_sample; if (sl < 0 || sl >= B) continue;
            GN_LAUNCH(ctx, embedding_pack_kernel, T, 128, 0, g + (size_t)sl * T * dim, (const int*)l.idx.p + (size_t)sl * T, rows + (size_t)q * T * dim, idsf + (size_t)q * T, T, dim);
          }
          GN_CUDA(cudaEventRecord(m->gather_ev, ctx->stream));
          GN_CUDA(cudaStreamWaitEvent(ctx->comm_stream, m->gather_ev, 0));
          int rc = ctx->nccl->AllReduce(buf, buf, (size_t)nq * T * (dim + 1), NCCL_FLOAT32, NCCL_SUM, ctx->comm, ctx->comm_stream);
          if (rc) return fail(GN_ERR_NCCL, "ncclAllReduce(embedding rows): %s", ctx->nccl->GetErrorString(rc));
          GN_CUDA(cudaEventRecord(m->gather_ev, ctx->comm_stream));
          GN_CUDA(cudaStreamWaitEvent(ctx->stream, m->gather_ev, 0));
          GN_LAUNCH(ctx, ids_to_int_kernel, cdiv((long)nq * T, 256), 256, 0, (const float*)idsf, idsi, nq * T);
          for (int q = 0; q < nq; q++)
            GN_LAUNCH(ctx, embedding_bwd_sample_kernel, T, 128, smem, (const float*)(rows + (size_t)q * T * dim), (const int*)(idsi + (size_t)q * T), gr, T, dim);
          l.grad_replicated = true;
        } else {
          for (int q = 0; q < nq; q++) {
            const int sl = q_sample(q) - first_sample; if (sl < 0 || sl >= B) continue;
            GN_LAUNCH(ctx, embedding_bwd_sample_kernel, T, 128, smem, g + (size_t)sl * T * dim, (const int*)l.idx.p + (size_t)sl * T, gr, T, dim);
          }
          l.grad_replicated = false;
        }
        break; }
      case GN_LAYER_POSENC:
        GN_TRY(colsum(m, g, l.out_size, B, l.out_size, gr, false)); break;     // gP = sum over samples; dx = g
      case GN_LAYER_TRANSFORMER_BLOCK:
        GN_TRY(block_backward(m, l, B, xin, g, dx)); g = dx; flip ^= 1; break;
      case GN_LAYER_CLS_POOLING: {
        long n = (long)B * l.in_size;
        GN_LAUNCH(ctx, cls_bwd_kernel, ew_grid(ctx, n), 256, 0, g, dx, d.seq_len, d.dim, n); g = dx; flip ^= 1; break; }
      case GN_LAYER_BATCHNORM2D: {
        const int C = d.in_size, S = d.in_h * d.in_w; const long BC = (long)B * C;
        float* pg; GN_TRY(ensure(m, S_DELTA, (size_t)B * 2 * C, &pg));
        GN_LAUNCH(ctx, bn_bwd_kernel, (unsigned)BC, 256, 0, g, xin, p, l.stat.p, dx, pg, C, S, BC);
        GN_TRY(colsum(m, pg, 2 * C, B, 2 * C, gr, false));
        g = dx; flip ^= 1; break; }
      case GN_LAYER_LAYERNORM: {
        long rows = (long)B * (l.in_size / d.dim);
        GN_TRY(layernorm_backward(m, g, xin, p, l.stat.p, l.stat.p + rows, dx, gr, gr + d.dim, rows, d.dim));
        g = dx; flip ^= 1; break; }
      case GN_LAYER_RMSNORM: {
        long rows = (long)B * (l.in_size / d.dim);
        const int chunks = (int)std::max<long>(1, std::min<long>(rows / 64, 128));
        float* part; GN_TRY(ensure(m, S_PART2, (size_t)chunks * d.dim, &part));
        GN_LAUNCH(ctx, rmsnorm_pgrad_partial_kernel, dim3(cdiv(d.dim, 128), chunks), 128, 0, g, xin, (const float*)l.stat.p, rows, d.dim, part);
        GN_LAUNCH(ctx, rmsnorm_pgrad_final_kernel, cdiv(d.dim, 128), 128, 0, part, chunks, d.dim, gr);
        if (need_dx) { GN_LAUNCH(ctx, rmsnorm_bwd_kernel, cdiv(rows, 8), 256, 0, g, xin, p, (const float*)l.stat.p, dx, rows, d.dim); g = dx; flip ^= 1; }
        break; }
    }
    GN_TRY(check_launch("backward"));
    if (ctx->world > 1 && l.p_cnt > 0) {
      if (comm_at_end) deferred.push_back(li); else GN_TRY(layer_comm(li));
    }
  }
  for (int li : deferred) GN_TRY(layer_comm(li));
  return GN_OK;
}

// ---------------------------------------------------------------- Adam
static void adam_coeffs(float lr, float b1, float b2, int t, float* effLR) {
  // opt.go:237-242: bias terms through float64 pow, rounded to float32; sqrt through float64
  float bias1 = (float)(1.0 - std::pow((double)b1, (double)t));
  float bias2 = (float)(1.0 - std::pow((double)b2, (double)t));
  *effLR = lr * (float)std::sqrt((double)bias2) / bias1;
}
static int adam_launch(Ctx* ctx, float* p, const float* g, float* m1, float* v, int64_t n, float lr, float b1, float b2, float eps, int t, float grad_scale,
                       const int* status = nullptr, cudaStream_t stream = nullptr) {
  float effLR; adam_coeffs(lr, b1, b2, t, &effLR);
  adam_kernel<<<ew_grid(ctx, (n + 3) / 4), 256, 0, stream ? stream : ctx->stream>>>(p, g, m1, v, (long)n, effLR, b1, b2, 1.f - b1, 1.f - b2, eps, grad_scale, status);
  ctx->launches++;
  return check_launch("adam");
}
// Meaning of a non-zero status word.
static int status_error(int st) {
  if (st == GN_STATUS_BAD_TOKEN) return fail(GN_ERR_INVALID_ARG, "a token id outside [0, vocabulary) was given to an Embedding layer (embedding.go:124-129); parameters and optimiser state are unchanged");
  return fail(GN_ERR_TIMEOUT, "a device-side bounded wait gave up (status word %d); parameters and optimiser state are unchanged", st);
}
// Reads the status word; non-zero clears it and becomes an error (GN_ERR_TIMEOUT: a bounded device-side wait gave up).
static int check_status_word(Ctx* c) {
  int st = 0; GN_CUDA(copy_d2h(c, &st, c->d_status, sizeof(int)));
  if (st != 0) { cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream); cudaStreamSynchronize(c->stream); return status_error(st); }
  return GN_OK;
}

// The step proper.  Anything that fails after work has been queued must not leave that work running behind the caller's
// back: train_step() below drains both streams before it reports the error.
static int train_step_issue(gn_model* m, const float* x_dev, const float* y_dev, int B, int global_batch, int first_sample) {
  Ctx* ctx = &m->ctx->c;
  GN_CUDA(cudaEventRecord(m->ev0, ctx->stream));
  GN_CUDA(cudaMemsetAsync(m->grads.p, 0, (size_t)m->P * sizeof(float), ctx->stream));     // Network.ClearGradients, net.go:813-823
  const float* yp;
  m->cur_first_sample = first_sample; m->cur_global_batch = global_batch;
  GN_TRY(forward(m, x_dev, B, &yp, true));
  for (auto& l : m->L) if (l.d.kind == GN_LAYER_DROPOUT)          // every rank moves the stream on by the whole global batch
    GN_LAUNCH(ctx, dropout_advance_kernel, 1, 1, 0, m->state.p + l.s_off, (unsigned long long)global_batch * (unsigned long long)l.in_size);
  GN_LAUNCH(ctx, loss_rows_kernel, B, 256, 0, yp, y_dev, m->lossg.p, m->loss_s.p, m->out_size, m->loss_kind);
  GN_LAUNCH(ctx, loss_total_kernel, 1, 32, 0, m->loss_s.p, B, m->loss_sum.p);
  GN_TRY(backward(m, x_dev, B, m->lossg.p, global_batch, first_sample));
  if (ctx->world > 1) {
    // loss sum over the ranks, then the main stream waits for the communication stream (per-layer gradient
    // all-reduces were issued during the backward pass); ar0..ar1 brackets the exposed wait
    GN_CUDA(cudaEventRecord(m->layer_ev.back(), ctx->stream));
    GN_CUDA(cudaStreamWaitEvent(ctx->comm_stream, m->layer_ev.back(), 0));
    int rc = ctx->nccl->AllReduce(m->loss_sum.p, m->loss_sum.p, 1, NCCL_FLOAT32, NCCL_SUM, ctx->comm, ctx->comm_stream);
    if (rc) return fail(GN_ERR_NCCL, "ncclAllReduce(loss): %s", ctx->nccl->GetErrorString(rc));
    GN_CUDA(cudaEventRecord(m->comm_done, ctx->comm_stream));
    GN_CUDA(cudaEventRecord(m->ar0, ctx->stream));
    GN_CUDA(cudaStreamWaitEvent(ctx->stream, m->comm_done, 0));
    GN_CUDA(cudaEventRecord(m->ar1, ctx->stream));
  }
  // Network.Step (net.go:260-284): NewStep() then StepInPlace with t = timestep + 1.  The pass reads the status word
  // first: after a bounded wait gave up it changes nothing.
  float inv = (float)(1.0 / (double)global_batch);                                        // net.go:703
  m->last_inv_batch = inv;
  if (ctx->world == 1) GN_TRY(adam_launch(ctx, m->params.p, m->grads.p, m->m1.p, m->v2.p, m->P, m->lr, m->b1, m->b2, m->eps, m->timestep + 2, inv, ctx->d_status));
  // (with more than one rank the update was applied slice by slice behind each layer's all-reduce, see backward())
  GN_CUDA(cudaEventRecord(m->ev1, ctx->stream));
  // one read-back for the caller: the loss sum and the status word land in the same pinned block, one wait
  GN_CUDA(cudaMemcpyAsync(&m->h_ret[0], m->loss_sum.p, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  GN_CUDA(cudaMemcpyAsync(&m->h_ret[1], ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  GN_CUDA(cudaStreamSynchronize(ctx->stream));
  return GN_OK;
}

static int train_step(gn_model* m, const float* x_dev, const float* y_dev, int B, int global_batch, int first_sample, float* mean_loss) {
  Ctx* ctx = &m->ctx->c;
  if (global_batch <= 0) { global_batch = B; first_sample = 0; }
  if (B > m->cap) GN_TRY(alloc_activations(m, B));
  int64_t launches0 = ctx->launches; ctx->gemm_flops = 0; ctx->gemm_launches = 0; ctx->gemm_ms = 0; ctx->ev_used = 0; ctx->gemm_bytes = 0; ctx->split_bytes = 0;
  m->wplanes_layerwise = false;
  int rc = train_step_issue(m, x_dev, y_dev, B, global_batch, first_sample);
  if (rc != GN_OK) {
    // drain what was queued before the failure (both streams) so that nothing of this step runs after the call returned
    const std::string msg = last_error();
    if (ctx->comm_stream) cudaStreamSynchronize(ctx->comm_stream);
    cudaStreamSynchronize(ctx->stream); cudaGetLastError();
    last_error() = msg; return rc;
  }
  int st; memcpy(&st, &m->h_ret[1], sizeof(int));
  if (st != 0) {    // the Adam pass saw the same word and left parameters, moments and the step counter alone
    cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream); cudaStreamSynchronize(ctx->stream);
    return status_error(st);
  }
  m->timestep += 1;
  m->wplanes.dirty = !m->wplanes_layerwise;          // the parameters moved: their operand planes are stale, unless they were renewed layer by layer behind the update
  m->wplanes_layerwise = false;
  if (mean_loss) *mean_loss = m->h_ret[0] / (float)global_batch;
  m->stats.kernel_launches = ctx->launches - launches0;
  cudaEventElapsedTime(&m->stats.step_ms, m->ev0, m->ev1);
  m->stats.allreduce_ms = 0.f; if (ctx->world > 1) cudaEventElapsedTime(&m->stats.allreduce_ms, m->ar0, m->ar1);
  m->stats.gemm_flops = ctx->gemm_flops; m->stats.gemm_launches = ctx->gemm_launches; m->stats.gemm_ms = 0.f;
  m->stats.gemm_bytes = ctx->gemm_bytes; m->stats.split_bytes = ctx->split_bytes;
  if (ctx->profile) { float tot = 0.f; for (size_t i = 0; i < ctx->ev_used; i++) { float ms = 0.f; cudaEventElapsedTime(&ms, ctx->ev_pool[i].first, ctx->ev_pool[i].second); tot += ms; } m->stats.gemm_ms = tot; }
  return GN_OK;
}

static int make_ctx(int device, int rank, int world, const unsigned char* id, gn_ctx** out) {
  if (!out) return fail(GN_ERR_INVALID_ARG, "out is null");
  int n = 0; cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) return fail(GN_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  if (device < 0 || device >= n) return fail(GN_ERR_INVALID_ARG, "device %d out of range [0,%d)", device, n);
  GN_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop; GN_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return fail(GN_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
  // a context that fails half way releases what it already holds
  struct Guard { gn_ctx* c; ~Guard() { if (!c) return;
      if (c->c.comm && c->c.nccl) c->c.nccl->CommDestroy(c->c.comm);
      if (c->c.comm_stream) cudaStreamDestroy(c->c.comm_stream);
      if (c->c.d_status) cudaFree(c->c.d_status);
      if (c->c.tc_queue_pool) cudaFree(c->c.tc_queue_pool);
      if (c->c.stream) cudaStreamDestroy(c->c.stream);
      delete c; } } guard{new gn_ctx()};
  gn_ctx* c = guard.c;
  c->c.device = device; c->c.rank = rank; c->c.world = world; c->c.sm_count = prop.multiProcessorCount;
  if (const char* e = getenv("GONEURON_CUDA_SM_RESERVE")) c->c.sm_reserve = std::max(0, std::min(atoi(e), prop.multiProcessorCount / 2));
  GN_CUDA(cudaStreamCreateWithFlags(&c->c.stream, cudaStreamNonBlocking));
  GN_CUDA(cudaMalloc(&c->c.d_status, sizeof(int)));
  GN_CUDA(cudaMemsetAsync(c->c.d_status, 0, sizeof(int), c->c.stream)); GN_CUDA(cudaStreamSynchronize(c->c.stream));
  tc_init(&c->c);
  if (world > 1) {
    NcclApi* api = nccl_api(); if (!api) return fail(GN_ERR_NCCL, "libnccl.so.2 could not be loaded");
    NcclUniqueId uid; memcpy(uid.internal, id, GN_UNIQUE_ID_BYTES);
    c->c.nccl = api;
    int rc = api->CommInitRank(&c->c.comm, world, uid, rank);
    if (rc) { c->c.comm = nullptr; return fail(GN_ERR_NCCL, "ncclCommInitRank: %s", api->GetErrorString(rc)); }
    GN_CUDA(cudaStreamCreateWithFlags(&c->c.comm_stream, cudaStreamNonBlocking));
  }
  guard.c = nullptr;
  *out = c; return GN_OK;
}

}  // namespace gn

using namespace gn;

#define CHECK_MODEL(m) do { if (!(m) || !(m)->alive) return fail(GN_ERR_INVALID_ARG, "model handle is null or destroyed"); } while (0)
#define USE_DEVICE(m) GN_CUDA(cudaSetDevice((m)->ctx->c.device))

extern "C" {

const char* gn_last_error(void) { return last_error().c_str(); }

int gn_init(int device, gn_ctx** out) { return make_ctx(device, 0, 1, nullptr, out); }

int gn_get_unique_id(unsigned char id[GN_UNIQUE_ID_BYTES]) {
  if (!id) return fail(GN_ERR_INVALID_ARG, "id is null");
  NcclApi* api = nccl_api(); if (!api) return fail(GN_ERR_NCCL, "libnccl.so.2 could not be loaded");
  NcclUniqueId uid; int rc = api->GetUniqueId(&uid); if (rc) return fail(GN_ERR_NCCL, "ncclGetUniqueId: %s", api->GetErrorString(rc));
  memcpy(id, uid.internal, GN_UNIQUE_ID_BYTES); return GN_OK;
}

int gn_init_rank(int device, int rank, int world_size, const unsigned char id[GN_UNIQUE_ID_BYTES], gn_ctx** out) {
  if (world_size < 1 || rank < 0 || rank >= world_size) return fail(GN_ERR_INVALID_ARG, "rank %d / world %d invalid", rank, world_size);
  if (world_size > 1 && !id) return fail(GN_ERR_INVALID_ARG, "id is null");
  return make_ctx(device, rank, world_size, id, out);
}

int gn_shutdown(gn_ctx* ctx) {
  if (!ctx || !ctx->alive) return GN_OK;
  cudaSetDevice(ctx->c.device);
  if (ctx->c.stream) cudaStreamSynchronize(ctx->c.stream);
  if (ctx->c.comm_stream) { cudaStreamSynchronize(ctx->c.comm_stream); }
  if (ctx->c.comm && ctx->c.nccl) ctx->c.nccl->CommDestroy(ctx->c.comm);
  for (auto& e : ctx->c.ev_pool) { cudaEventDestroy(e.first); cudaEventDestroy(e.second); }
  ctx->c.ev_pool.clear();
  ctx->c.release_owned();                               // operand-plane scratch of the contraction and attention engines
  if (ctx->c.d_status) cudaFree(ctx->c.d_status);
  if (ctx->c.tc_queue_pool) { cudaFree(ctx->c.tc_queue_pool); ctx->c.tc_queue_pool = nullptr; }
  if (ctx->c.t0) { cudaEventDestroy(ctx->c.t0); cudaEventDestroy(ctx->c.t1); ctx->c.t0 = ctx->c.t1 = nullptr; }
  if (ctx->c.stream) cudaStreamDestroy(ctx->c.stream);
  if (ctx->c.comm_stream) cudaStreamDestroy(ctx->c.comm_stream);
  ctx->c.comm_stream = nullptr;
  ctx->c.comm = nullptr; ctx->c.d_status = nullptr; ctx->c.stream = nullptr; ctx->alive = false;
  return GN_OK;   // the handle itself stays allocated so that a second call is harmless
}

int gn_ctx_world_size(gn_ctx* ctx, int* world_size, int* rank) {
  if (!ctx || !ctx->alive) return fail(GN_ERR_INVALID_ARG, "context is null or shut down");
  if (world_size) *world_size = ctx->c.world; if (rank) *rank = ctx->c.rank; return GN_OK;
}

int gn_ctx_set_spin_limit(gn_ctx* ctx, unsigned int polls) {
  if (!ctx || !ctx->alive) return fail(GN_ERR_INVALID_ARG, "context is null or shut down");
  ctx->c.spin_limit = polls == 0 ? TC_SPIN_LIMIT : polls; return GN_OK;
}

int gn_synchronize(gn_ctx* ctx) {
  if (!ctx || !ctx->alive) return fail(GN_ERR_INVALID_ARG, "context is null or shut down");
  GN_CUDA(cudaSetDevice(ctx->c.device)); GN_CUDA(cudaStreamSynchronize(ctx->c.stream)); return GN_OK;
}

int gn_timer_start(gn_ctx* ctx) {
  if (!ctx || !ctx->alive) return fail(GN_ERR_INVALID_ARG, "context is null or shut down");
  GN_CUDA(cudaSetDevice(ctx->c.device));
  if (!ctx->c.t0) { GN_CUDA(cudaEventCreate(&ctx->c.t0)); GN_CUDA(cudaEventCreate(&ctx->c.t1)); }
  GN_CUDA(cudaEventRecord(ctx->c.t0, ctx->c.stream)); return GN_OK;
}
int gn_timer_stop(gn_ctx* ctx, float* ms) {
  if (!ctx || !ctx->alive || !ms || !ctx->c.t0) return fail(GN_ERR_INVALID_ARG, "timer not started");
  GN_CUDA(cudaSetDevice(ctx->c.device));
  GN_CUDA(cudaEventRecord(ctx->c.t1, ctx->c.stream)); GN_CUDA(cudaEventSynchronize(ctx->c.t1));
  GN_CUDA(cudaEventElapsedTime(ms, ctx->c.t0, ctx->c.t1)); return GN_OK;
}

int gn_model_create(gn_ctx* ctx, const gn_layer_desc* layers, int n_layers, int loss_kind, int virtual_workers, gn_model** out) {
  if (!ctx || !ctx->alive) return fail(GN_ERR_INVALID_ARG, "context is null or shut down");
  if (!layers || n_layers <= 0 || !out) return fail(GN_ERR_INVALID_ARG, "layers/out is null or n_layers <= 0");
  if (loss_kind != GN_LOSS_MSE && loss_kind != GN_LOSS_CROSS_ENTROPY) return fail(GN_ERR_UNSUPPORTED, "loss kind %d", loss_kind);
  GN_CUDA(cudaSetDevice(ctx->c.device));
  std::unique_ptr<gn_model> m(new gn_model());
  m->ctx = ctx; m->loss_kind = loss_kind; m->W = virtual_workers < 1 ? 1 : virtual_workers;
  GN_TRY(plan_layers(m.get(), layers, n_layers));
  size_t P = (size_t)std::max<int64_t>(m->P, 4);
  GN_TRY(m->params.alloc(P)); GN_TRY(m->grads.alloc(P)); GN_TRY(m->m1.alloc(P)); GN_TRY(m->v2.alloc(P));
  // cudaMemset is asynchronous to the host and runs on the legacy default stream, which the context's non-blocking
  // stream does not wait for: a memset issued that way can land AFTER the first training step has written its
  // gradients (seen as all-zero LSTM gradients after the GPU had been idle).  So: the context's own stream, then wait.
  {
    cudaStream_t st = ctx->c.stream;
    GN_CUDA(cudaMemsetAsync(m->params.p, 0, P * 4, st)); GN_CUDA(cudaMemsetAsync(m->grads.p, 0, P * 4, st));
    GN_CUDA(cudaMemsetAsync(m->m1.p, 0, P * 4, st)); GN_CUDA(cudaMemsetAsync(m->v2.p, 0, P * 4, st));
    GN_CUDA(cudaStreamSynchronize(st));
  }
  if (ctx->c.tc_ok && !force_simt_engine() && !getenv("GONEURON_CUDA_NO_WEIGHT_PLANES")) {
    // weight matrices large enough to run on the tensor-core engine get prepared operand planes (both orientations)
    std::vector<WeightPlaneEntry> mats; int cur_layer = 0;
    auto add = [&](int64_t off, int out, int in, bool has_bias = true) {
      if ((double)out * in < 64.0 * 64.0) return;
      WeightPlaneEntry e{m->params.p + off, out, in, {}, {}}; e.bias = has_bias ? m->params.p + off + (int64_t)out * in : nullptr; e.layer = cur_layer; mats.push_back(e);
    };
    for (auto& l : m->L) {
      const gn_layer_desc& d = l.d; cur_layer = (int)(&l - m->L.data());
      if (d.kind == GN_LAYER_DENSE) add(l.p_off, d.out_size, d.in_size);
      else if (d.kind == GN_LAYER_TRANSFORMER_BLOCK) {
        const int64_t dd = (int64_t)d.dim * d.dim + d.dim; int64_t o = l.p_off;
        for (int k = 0; k < 4; k++) { add(o, d.dim, d.dim); o += dd; }
        o += (l.rms ? 2 : 4) * (int64_t)d.dim;
        if (l.ff_act == GN_ACT_SILU) { add(o, d.ff_dim, d.dim, false); add(o + (int64_t)d.dim * d.ff_dim, d.ff_dim, d.dim, false); o += 2 * (int64_t)d.dim * d.ff_dim; }
        else { add(o, d.ff_dim, d.dim); o += (int64_t)d.dim * d.ff_dim + d.ff_dim; }
        add(o, d.dim, d.ff_dim);
      }
    }
    GN_TRY(wplanes_build(&ctx->c, m->wplanes, mats));
  }
  if (m->NS > 0) {
    GN_TRY(m->state.alloc((size_t)m->NS));
    std::vector<float> init((size_t)m->NS, 0.f);     // running mean 0, running variance 1 (batchnorm2d.go:124-128)
    for (auto& l : m->L) if (l.d.kind == GN_LAYER_BATCHNORM2D) for (int64_t k = l.s_cnt / 2; k < l.s_cnt; k++) init[l.s_off + k] = 1.f;
    GN_CUDA(copy_h2d(&ctx->c, m->state.p, init.data(), (size_t)m->NS * 4));
  }
  GN_CUDA(cudaEventCreate(&m->ev0)); GN_CUDA(cudaEventCreate(&m->ev1)); GN_CUDA(cudaEventCreate(&m->ar0)); GN_CUDA(cudaEventCreate(&m->ar1));
  GN_CUDA(cudaEventCreateWithFlags(&m->comm_done, cudaEventDisableTiming)); GN_CUDA(cudaEventCreateWithFlags(&m->gather_ev, cudaEventDisableTiming));
  m->layer_ev.resize(m->L.size() + 1);
  for (auto& e : m->layer_ev) GN_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  m->scratch.resize(S_COUNT);
  GN_CUDA(cudaHostAlloc((void**)&m->h_ret, 4 * sizeof(float), cudaHostAllocDefault));
  *out = m.release(); return GN_OK;
}

int gn_model_destroy(gn_model* m) {
  if (!m || !m->alive) return GN_OK;
  std::lock_guard<std::mutex> lk(m->mu);
  cudaSetDevice(m->ctx->c.device);
  if (m->ctx->alive && m->ctx->c.stream) cudaStreamSynchronize(m->ctx->c.stream);
  if (m->ctx->c.weight_planes == &m->wplanes) m->ctx->c.weight_planes = nullptr;
  m->wplanes = gn::WeightPlaneTable();
  m->L.clear(); m->scratch.clear(); m->state.release(); m->params.release(); m->grads.release(); m->m1.release(); m->v2.release();
  m->xin.release(); m->yin.release(); m->lossg.release(); m->loss_s.release(); m->loss_sum.release();
  if (m->ev0) cudaEventDestroy(m->ev0); if (m->ev1) cudaEventDestroy(m->ev1); if (m->ar0) cudaEventDestroy(m->ar0); if (m->ar1) cudaEventDestroy(m->ar1);
  if (m->comm_done) cudaEventDestroy(m->comm_done); if (m->gather_ev) cudaEventDestroy(m->gather_ev); m->gather_ev = nullptr; for (auto e : m->layer_ev) cudaEventDestroy(e); m->layer_ev.clear();
  if (m->h_ret) cudaFreeHost(m->h_ret); m->h_ret = nullptr;
  m->ev0 = m->ev1 = m->ar0 = m->ar1 = m->comm_done = nullptr; m->alive = false; return GN_OK;
}

int gn_model_param_count(gn_model* m, int64_t* n) { CHECK_MODEL(m); if (!n) return fail(GN_ERR_INVALID_ARG, "n is null"); *n = m->P; return GN_OK; }
int gn_model_in_size(gn_model* m, int64_t* n) { CHECK_MODEL(m); if (!n) return fail(GN_ERR_INVALID_ARG, "n is null"); *n = m->in_size; return GN_OK; }
int gn_model_out_size(gn_model* m, int64_t* n) { CHECK_MODEL(m); if (!n) return fail(GN_ERR_INVALID_ARG, "n is null"); *n = m->out_size; return GN_OK; }

int gn_model_set_params(gn_model* m, const float* host, int64_t n) {
  CHECK_MODEL(m); if (!host || n != m->P) return fail(GN_ERR_INVALID_ARG, "set_params: expected %lld floats, got %lld", (long long)m->P, (long long)n);
  std::lock_guard<std::mutex> lk(m->mu); USE_DEVICE(m);
  GN_CUDA(cudaMemcpyAsync(m->params.p, host, (size_t)n * 4, cudaMemcpyHostToDevice, m->ctx->c.stream));
  m->wplanes.dirty = true;
  GN_CUDA(cudaStreamSynchronize(m->ctx->c.stream)); return GN_OK;
}
int gn_model_get_params(gn_model* m, float* host, int64_t n) {
  CHECK_MODEL(m); if (!host || n != m->P) return fail(GN_ERR_INVALID_ARG, "get_params: expected %lld floats, got %lld", (long long)m->P, (long long)n);
  std::lock_guard<std::mutex> lk(m->mu); USE_DEVICE(m);
  GN_CUDA(cudaMemcpyAsync(host, m->params.p, (size_t)n * 4, cudaMemcpyDeviceToHost, m->ctx->c.stream));
  GN_CUDA(cudaStreamSynchronize(m->ctx->c.stream)); return GN_OK;
}
int gn_model_get_grads(gn_model* m, float* host, int64_t n) {
  CHECK_MODEL(m); if (!host || n != m->P) return fail(GN_ERR_INVALID_ARG, "get_grads: expected %lld floats, got %lld", (long long)m->P, (long long)n);
  std::lock_guard<std::mutex> lk(m->mu); USE_DEVICE(m);
  GN_CUDA(cudaMemcpyAsync(host, m->grads.p, (size_t)n * 4, cudaMemcpyDeviceToHost, m->ctx->c.stream));
  GN_CUDA(cudaStreamSynchronize(m->ctx->c.stream));
  // the device keeps the batch-summed gradient; the 1/batch factor of net.go:702-706 is applied inside the Adam
  // pass and here, with the same float32 multiplication
  const float inv = m->last_inv_batch;
  for (int64_t i = 0; i < n; i++) host[i] *= inv;
  return GN_OK;
}

int gn_model_state_count(gn_model* m, int64_t* n) { CHECK_MODEL(m); if (!n) return fail(GN_ERR_INVALID_ARG, "n is null"); *n = m->NS; return GN_OK; }
int gn_model_get_state(gn_model* m, float* host, int64_t n) {
  CHECK_MODEL(m); if (n != m->NS || (n > 0 && !host)) return fail(GN_ERR_INVALID_ARG, "get_state: expected %lld floats, got %lld", (long long)m->NS, (long long)n);
  if (n == 0) return GN_OK;
  std::lock_guard<std::mutex> lk(m->mu); USE_DEVICE(m);
  GN_CUDA(cudaStreamSynchronize(m->ctx->c.stream)); GN_CUDA(copy_d2h(&m->ctx->c, host, m->state.p, (size_t)n * 4)); return GN_OK;
}
int gn_model_set_state(gn_model* m, const float* host, int64_t n) {
  CHECK_MODEL(m); if (n != m->NS || (n > 0 && !host)) return fail(GN_ERR_INVALID_ARG, "set_state: expected %lld floats, got %lld", (long long)m->NS, (long long)n);
  if (n == 0) return GN_OK;
  std::lock_guard<std::mutex> lk(m->mu); USE_DEVICE(m);
  GN_CUDA(cudaStreamSynchronize(m->ctx->c.stream)); GN_CUDA(copy_h2d(&m->ctx->c, m->state.p, host, (size_t)n * 4)); return GN_OK;
}

int gn_adam_set(gn_model* m, float lr, float beta1, float beta2, float eps, int timestep) {
  CHECK_MODEL(m); std::lock_guard<std::mutex> lk(m->mu);
  // zero betas / eps select the defaults, as Adam.StepInPlace does (opt.go:211-223)
  m->lr = lr; m->b1 = beta1 == 0.f ? 0.9f : beta1; m->b2 = beta2 == 0.f ? 0.999f : beta2; m->eps = eps == 0.f ? 1e-8f : eps;
  if (timestep >= 0) m->timestep = timestep; return GN_OK;
}
int gn_adam_get_state(gn_model* m, float* m1, float* v, int64_t n, int* timestep) {
  CHECK_MODEL(m); if (n != m->P) return fail(GN_ERR_INVALID_ARG, "adam state: expected %lld floats", (long long)m->P);
  std::lock_guard<std::mutex> lk(m->mu); USE_DEVICE(m);
  if (m1) GN_CUDA(copy_d2h(&m->ctx->c, m1, m->m1.p, (size_t)n * 4));
  if (v) GN_CUDA(copy_d2h(&m->ctx->c, v, m->v2.p, (size_t)n * 4));
  if (timestep) *timestep = m->timestep; return GN_OK;
}
int gn_adam_set_state(gn_model* m, const float* m1, const float* v, int64_t n, int timestep) {
  CHECK_MODEL(m); if (n != m->P || !m1 || !v) return fail(GN_ERR_INVALID_ARG, "adam state: expected %lld floats", (long long)m->P);
  std::lock_guard<std::mutex> lk(m->mu); USE_DEVICE(m);
  GN_CUDA(copy_h2d(&m->ctx->c, m->m1.p, m1, (size_t)n * 4)); GN_CUDA(copy_h2d(&m->ctx->c, m->v2.p, v, (size_t)n * 4));
  if (timestep >= 0) m->timestep = timestep; return GN_OK;
}

int gn_train_batch_device(gn_model* m, const float* x_dev, const float* y_dev, int batch, int global_batch, int first_sample, float* mean_loss) {
  CHECK_MODEL(m); if (!x_dev || !y_dev || batch <= 0) return fail(GN_ERR_INVALID_ARG, "train_batch: null input or batch <= 0");
  std::lock_guard<std::mutex> lk(m->mu); std::lock_guard<std::mutex> run_lk(m->ctx->c.run_mu); USE_DEVICE(m);
  return train_step(m, x_dev, y_dev, batch, global_batch, first_sample, mean_loss);
}

int gn_train_batch(gn_model* m, const float* x, const float* y, int batch, int global_batch, int first_sample, float* mean_loss) {
  CHECK_MODEL(m); if (!x || !y || batch <= 0) return fail(GN_ERR_INVALID_ARG, "train_batch: null input or batch <= 0");
  std::lock_guard<std::mutex> lk(m->mu); std::lock_guard<std::mutex> run_lk(m->ctx->c.run_mu); USE_DEVICE(m);
  if (batch > m->cap) GN_TRY(alloc_activations(m, batch));
  cudaStream_t s = m->ctx->c.stream;
  GN_CUDA(cudaMemcpyAsync(m->xin.p, x, (size_t)batch * m->in_size * 4, cudaMemcpyHostToDevice, s));
  GN_CUDA(cudaMemcpyAsync(m->yin.p, y, (size_t)batch * m->out_size * 4, cudaMemcpyHostToDevice, s));
  return train_step(m, m->xin.p, m->yin.p, batch, global_batch, first_sample, mean_loss);
}

int gn_forward_batch(gn_model* m, const float* x, int batch, float* out) {
  CHECK_MODEL(m); if (!x || !out || batch <= 0) return fail(GN_ERR_INVALID_ARG, "forward_batch: null pointer or batch <= 0");
  std::lock_guard<std::mutex> lk(m->mu); std::lock_guard<std::mutex> run_lk(m->ctx->c.run_mu); USE_DEVICE(m);
  if (batch > m->cap) GN_TRY(alloc_activations(m, batch));
  cudaStream_t s = m->ctx->c.stream;
  GN_CUDA(cudaMemcpyAsync(m->xin.p, x, (size_t)batch * m->in_size * 4, cudaMemcpyHostToDevice, s));
  const float* yp; GN_TRY(forward(m, m->xin.p, batch, &yp, false));
  GN_CUDA(cudaMemcpyAsync(out, yp, (size_t)batch * m->out_size * 4, cudaMemcpyDeviceToHost, s));
  GN_CUDA(cudaStreamSynchronize(s)); return check_status_word(&m->ctx->c);
}

int gn_device_alloc(gn_ctx* ctx, int64_t n, float** dev) {
  if (!ctx || !ctx->alive || !dev || n <= 0) return fail(GN_ERR_INVALID_ARG, "device_alloc: bad argument");
  GN_CUDA(cudaSetDevice(ctx->c.device)); cudaError_t e = cudaMalloc(dev, (size_t)n * 4);
  if (e != cudaSuccess) return fail(GN_ERR_OOM, "cudaMalloc(%lld floats): %s", (long long)n, cudaGetErrorString(e)); return GN_OK;
}
int gn_device_free(gn_ctx* ctx, float* dev) { if (!ctx || !ctx->alive) return GN_OK; cudaSetDevice(ctx->c.device); if (dev) cudaFree(dev); return GN_OK; }
int gn_device_upload(gn_ctx* ctx, float* dev, const float* host, int64_t n) {
  if (!ctx || !ctx->alive || !dev || !host) return fail(GN_ERR_INVALID_ARG, "device_upload: bad argument");
  GN_CUDA(cudaSetDevice(ctx->c.device)); GN_CUDA(cudaMemcpyAsync(dev, host, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->c.stream)); GN_CUDA(cudaStreamSynchronize(ctx->c.stream)); return GN_OK;
}
int gn_device_download(gn_ctx* ctx, float* host, const float* dev, int64_t n) {
  if (!ctx || !ctx->alive || !dev || !host) return fail(GN_ERR_INVALID_ARG, "device_download: bad argument");
  GN_CUDA(cudaSetDevice(ctx->c.device)); GN_CUDA(cudaMemcpyAsync(host, dev, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->c.stream)); GN_CUDA(cudaStreamSynchronize(ctx->c.stream)); return GN_OK;
}

int gn_model_last_stats(gn_model* m, gn_step_stats* out) { CHECK_MODEL(m); if (!out) return fail(GN_ERR_INVALID_ARG, "out is null"); *out = m->stats; return GN_OK; }
int gn_model_set_profiling(gn_model* m, int level) { CHECK_MODEL(m); m->ctx->c.profile = level; return GN_OK; }

int gn_op_gemm_nt(gn_ctx* ctx, int engine, int M, int N, int K, const float* A, const float* B, const float* bias, float* C) {
  if (!ctx || !ctx->alive || !A || !B || !C || M <= 0 || N <= 0 || K <= 0) return fail(GN_ERR_INVALID_ARG, "op_gemm_nt: bad argument");
  Ctx* c = &ctx->c; std::lock_guard<std::mutex> run_lk(c->run_mu); GN_CUDA(cudaSetDevice(c->device));
  DevBuf dA, dB, dC, db; GN_TRY(dA.alloc((size_t)M * K)); GN_TRY(dB.alloc((size_t)N * K)); GN_TRY(dC.alloc((size_t)M * N)); if (bias) GN_TRY(db.alloc(N));
  GN_CUDA(cudaMemcpyAsync(dA.p, A, (size_t)M * K * 4, cudaMemcpyHostToDevice, c->stream)); GN_CUDA(cudaMemcpyAsync(dB.p, B, (size_t)N * K * 4, cudaMemcpyHostToDevice, c->stream));
  if (bias) GN_CUDA(cudaMemcpyAsync(db.p, bias, (size_t)N * 4, cudaMemcpyHostToDevice, c->stream));
  GemmDesc g; g.M = M; g.N = N; g.K = K; g.A = dA.p; g.sa_m = K; g.sa_k = 1; g.B = dB.p; g.sb_k = 1; g.sb_n = K; g.C = dC.p; g.ldc = N; g.bias = bias ? db.p : nullptr;
  if (engine == 1) { if (!gemm_tc_supported(c, g)) return fail(GN_ERR_UNSUPPORTED, "tcgen05 engine cannot run this shape (M=%d N=%d K=%d)", M, N, K); GN_TRY(gemm_tc(c, g)); }
  else GN_TRY(gemm_simt(c, g));
  GN_CUDA(cudaMemcpyAsync(C, dC.p, (size_t)M * N * 4, cudaMemcpyDeviceToHost, c->stream)); GN_CUDA(cudaStreamSynchronize(c->stream));
  return check_status_word(c);
}

int gn_op_adam(gn_ctx* ctx, float* params, const float* grads, float* m1, float* v, int64_t n, float lr, float beta1, float beta2, float eps, int t, float grad_scale) {
  if (!ctx || !ctx->alive || !params || !grads || !m1 || !v || n <= 0) return fail(GN_ERR_INVALID_ARG, "op_adam: bad argument");
  Ctx* c = &ctx->c; std::lock_guard<std::mutex> run_lk(c->run_mu); GN_CUDA(cudaSetDevice(c->device));
  DevBuf dp, dg, dm, dv; size_t nn = (size_t)n; GN_TRY(dp.alloc(nn + 4)); GN_TRY(dg.alloc(nn + 4)); GN_TRY(dm.alloc(nn + 4)); GN_TRY(dv.alloc(nn + 4));
  GN_CUDA(copy_h2d(c, dp.p, params, nn * 4)); GN_CUDA(copy_h2d(c, dg.p, grads, nn * 4));
  GN_CUDA(copy_h2d(c, dm.p, m1, nn * 4)); GN_CUDA(copy_h2d(c, dv.p, v, nn * 4));
  GN_TRY(adam_launch(c, dp.p, dg.p, dm.p, dv.p, n, lr, beta1, beta2, eps, t, grad_scale));
  GN_CUDA(cudaStreamSynchronize(c->stream));
  GN_CUDA(copy_d2h(c, params, dp.p, nn * 4)); GN_CUDA(copy_d2h(c, m1, dm.p, nn * 4)); GN_CUDA(copy_d2h(c, v, dv.p, nn * 4));
  return GN_OK;
}

int gn_op_attention(gn_ctx* ctx, int engine, int B, int T, int D, int H, int causal, const float* Q, const float* K, const float* V, const float* dO,
                    float* O, float* M, float* L, float* dQ, float* dK, float* dV) {
  if (!ctx || !ctx->alive || !Q || !K || !V || !O || B <= 0 || T <= 0 || D <= 0 || H <= 0 || D % H) return fail(GN_ERR_INVALID_ARG, "op_attention: bad argument");
  if (dO && (!dQ || !dK || !dV)) return fail(GN_ERR_INVALID_ARG, "op_attention: dO given without dQ, dK, dV");
  Ctx* c = &ctx->c; std::lock_guard<std::mutex> run_lk(c->run_mu); GN_CUDA(cudaSetDevice(c->device));
  const int hd = D / H; const size_t n = (size_t)B * T * D, ns = (size_t)B * H * T;
  if (!attn_fused_supported(hd, D)) return fail(GN_ERR_UNSUPPORTED, "op_attention: head size %d", hd);
  if (engine == 1 && !attn_tc_supported(c, hd, T, B, H, D)) return fail(GN_ERR_UNSUPPORTED, "tcgen05 attention cannot run this shape (head size %d, T=%d)", hd, T);
  DevBuf q, k, v, o, m, l, g, dv_, dq, dk, dvv;
  GN_TRY(q.alloc(n)); GN_TRY(k.alloc(n)); GN_TRY(v.alloc(n)); GN_TRY(o.alloc(n)); GN_TRY(m.alloc(ns)); GN_TRY(l.alloc(ns));
  GN_CUDA(copy_h2d(c, q.p, Q, n * 4)); GN_CUDA(copy_h2d(c, k.p, K, n * 4)); GN_CUDA(copy_h2d(c, v.p, V, n * 4));
  if (engine == 1) GN_TRY(attn_tc_fwd(c, q.p, k.p, v.p, o.p, m.p, l.p, B, T, D, H, causal));
  else GN_TRY(attn_fwd(c, hd, q.p, k.p, v.p, o.p, m.p, l.p, B, T, D, H, causal));
  if (dO) {
    GN_TRY(g.alloc(n)); GN_TRY(dv_.alloc(ns)); GN_TRY(dq.alloc(n)); GN_TRY(dk.alloc(n)); GN_TRY(dvv.alloc(n));
    GN_CUDA(copy_h2d(c, g.p, dO, n * 4));
    if (engine == 1) GN_TRY(attn_tc_bwd(c, q.p, k.p, v.p, o.p, g.p, m.p, l.p, dv_.p, dq.p, dk.p, dvv.p, B, T, D, H, causal));
    else GN_TRY(attn_bwd(c, hd, q.p, k.p, v.p, o.p, g.p, m.p, l.p, dv_.p, dq.p, dk.p, dvv.p, B, T, D, H, causal));
    GN_CUDA(copy_d2h(c, dQ, dq.p, n * 4)); GN_CUDA(copy_d2h(c, dK, dk.p, n * 4)); GN_CUDA(copy_d2h(c, dV, dvv.p, n * 4));
  }
  GN_CUDA(copy_d2h(c, O, o.p, n * 4));
  if (M) GN_CUDA(copy_d2h(c, M, m.p, ns * 4));
  if (L) GN_CUDA(copy_d2h(c, L, l.p, ns * 4));
  return check_status_word(c);
}

}  // extern "C"

#include "gemm_static.cuh"
#include "ops_tier.cuh"
