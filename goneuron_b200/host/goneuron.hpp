// goneuron.hpp -- header-only C++ mirror of GoNeuron's Sequential API over the C ABI of libgoneuron_cuda.so.
// Names follow the reference: goneuron.NewSequential / Compile / Fit / TrainBatch / Predict / PredictBatch
// (internal/net/sequential.go:26-37, 102-122, 133-164) and the layer constructors of goneuron/goneuron.go.
// Errors that the reference returns as `error` are thrown as std::runtime_error.
#pragma once
#include <cstring>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/goneuron_cuda.h"

namespace goneuron {

inline void check(int rc) { if (rc != GN_OK) throw std::runtime_error(std::string("goneuron_cuda: ") + gn_last_error()); }

inline gn_layer_desc Dense(int in, int out, gn_activation act = GN_ACT_LINEAR) { gn_layer_desc d{}; d.kind = GN_LAYER_DENSE; d.in_size = in; d.out_size = out; d.activation = act; return d; }
inline gn_layer_desc Conv2D(int inC, int outC, int k, int stride, int pad, gn_activation act, int h, int w) {
  gn_layer_desc d{}; d.kind = GN_LAYER_CONV2D; d.in_size = inC; d.out_size = outC; d.kernel = k; d.stride = stride; d.padding = pad; d.activation = act; d.in_h = h; d.in_w = w; return d; }
inline gn_layer_desc Conv1D(int inC, int outC, int k, int stride, int pad, int act, int length) { gn_layer_desc d{}; d.kind = GN_LAYER_CONV1D; d.in_size = inC; d.out_size = outC; d.kernel = k; d.stride = stride; d.padding = pad; d.activation = act; d.in_w = length; return d; }
inline gn_layer_desc RMSNorm(int dim, float eps = 1e-5f) { gn_layer_desc d{}; d.kind = GN_LAYER_RMSNORM; d.dim = dim; memcpy(&d.reserved, &eps, 4); return d; }
inline gn_layer_desc Dropout(float p, int inSize) { gn_layer_desc d{}; d.kind = GN_LAYER_DROPOUT; d.in_size = inSize; memcpy(&d.dim, &p, 4); return d; }
inline gn_layer_desc AvgPool2D(int inC, int k, int stride, int pad, int h, int w) { gn_layer_desc d{}; d.kind = GN_LAYER_AVGPOOL2D; d.in_size = inC; d.kernel = k; d.stride = stride; d.padding = pad; d.in_h = h; d.in_w = w; return d; }
inline gn_layer_desc MaxPool2D(int inC, int k, int stride, int pad, int h, int w) { gn_layer_desc d{}; d.kind = GN_LAYER_MAXPOOL2D; d.in_size = inC; d.kernel = k; d.stride = stride; d.padding = pad; d.in_h = h; d.in_w = w; return d; }
inline gn_layer_desc Flatten() { gn_layer_desc d{}; d.kind = GN_LAYER_FLATTEN; return d; }
inline gn_layer_desc SequenceUnrollerLSTM(int in, int hidden, int T, bool returnSeq = false) { gn_layer_desc d{}; d.kind = GN_LAYER_LSTM_UNROLLED; d.in_size = in; d.out_size = hidden; d.seq_len = T; d.return_seq = returnSeq; return d; }
// layer.NewSequenceUnroller(layer.NewGRU(in, hidden), T, returnSeq) -- unroller.go:57, gru.go:81
inline gn_layer_desc SequenceUnrollerGRU(int in, int hidden, int T, bool returnSeq = false) { gn_layer_desc d{}; d.kind = GN_LAYER_GRU_UNROLLED; d.in_size = in; d.out_size = hidden; d.seq_len = T; d.return_seq = returnSeq; return d; }
inline gn_layer_desc Embedding(int vocab, int dim, int T = 0) { gn_layer_desc d{}; d.kind = GN_LAYER_EMBEDDING; d.in_size = vocab; d.out_size = dim; d.seq_len = T; return d; }
inline gn_layer_desc PositionalEncoding(int T, int dim) { gn_layer_desc d{}; d.kind = GN_LAYER_POSENC; d.seq_len = T; d.dim = dim; return d; }
inline gn_layer_desc TransformerBlock(int dim, int heads, int T, int ff, bool causal) { gn_layer_desc d{}; d.kind = GN_LAYER_TRANSFORMER_BLOCK; d.dim = dim; d.heads = heads; d.seq_len = T; d.ff_dim = ff; d.causal = causal; return d; }
// layer.NewTransformerBlockExt(dim, heads, T, ff, causal, actType, normType, useRoPE) -- transformer.go:899-957: ffAct is
// GN_ACT_RELU (ActReLU), GN_ACT_GELU (ActGELU) or GN_ACT_SILU (ActSwiGLU); the descriptor carries them in activation / kernel / stride
inline gn_layer_desc TransformerBlockExt(int dim, int heads, int T, int ff, bool causal, gn_activation ffAct, bool rmsNorm, bool useRoPE) {
  gn_layer_desc d = TransformerBlock(dim, heads, T, ff, causal); d.activation = ffAct == GN_ACT_RELU ? 0 : ffAct; d.kernel = rmsNorm ? 1 : 0; d.stride = useRoPE ? 1 : 0; return d; }
// layer.NewBatchNorm2D(C, eps, momentum, true) + SetInputDimensions(h, w) -- batchnorm2d.go:67-160
inline gn_layer_desc BatchNorm2D(int numFeatures, int h, int w, float eps = 1e-5f, float momentum = 0.1f) {
  gn_layer_desc d{}; d.kind = GN_LAYER_BATCHNORM2D; d.in_size = numFeatures; d.in_h = h; d.in_w = w; memcpy(&d.dim, &momentum, 4); memcpy(&d.reserved, &eps, 4); return d; }
inline gn_layer_desc CLSPooling(int T, int dim) { gn_layer_desc d{}; d.kind = GN_LAYER_CLS_POOLING; d.seq_len = T; d.dim = dim; return d; }
inline gn_layer_desc LayerNorm(int dim) { gn_layer_desc d{}; d.kind = GN_LAYER_LAYERNORM; d.dim = dim; return d; }

struct Adam { float LearningRate, Beta1 = 0.9f, Beta2 = 0.999f, Epsilon = 1e-8f; explicit Adam(float lr) : LearningRate(lr) {} };

class Device {
 public:
  explicit Device(int index = 0) { check(gn_init(index, &ctx_)); }
  ~Device() { gn_shutdown(ctx_); }
  Device(const Device&) = delete; Device& operator=(const Device&) = delete;
  gn_ctx* handle() const { return ctx_; }
 private:
  gn_ctx* ctx_ = nullptr;
};

class Sequential {
 public:
  Sequential(Device& dev, std::vector<gn_layer_desc> layers, int virtual_workers = 1) : dev_(dev), layers_(std::move(layers)), workers_(virtual_workers) {}
  ~Sequential() { Close(); }
  void Compile(Adam* opt, gn_loss_kind loss) {
    opt_ = opt; check(gn_model_create(dev_.handle(), layers_.data(), (int)layers_.size(), loss, workers_, &m_));
    check(gn_model_param_count(m_, &n_params_)); check(gn_model_in_size(m_, &in_)); check(gn_model_out_size(m_, &out_));
  }
  int64_t NumParams() const { return n_params_; }
  void SetParams(const std::vector<float>& p) { check(gn_model_set_params(m_, p.data(), (int64_t)p.size())); }
  std::vector<float> Params() { std::vector<float> p(n_params_); check(gn_model_get_params(m_, p.data(), n_params_)); return p; }
  std::vector<float> Gradients() { std::vector<float> g(n_params_); check(gn_model_get_grads(m_, g.data(), n_params_)); return g; }
  // batchX: [batch * in], batchY: [batch * out], row-major
  float TrainBatch(const std::vector<float>& batchX, const std::vector<float>& batchY) {
    int batch = (int)(batchX.size() / in_);
    if ((int64_t)batch * in_ != (int64_t)batchX.size() || (int64_t)batch * out_ != (int64_t)batchY.size()) throw std::runtime_error("TrainBatch: size mismatch");
    check(gn_adam_set(m_, opt_->LearningRate, opt_->Beta1, opt_->Beta2, opt_->Epsilon, -1));
    float loss = 0.f; check(gn_train_batch(m_, batchX.data(), batchY.data(), batch, 0, 0, &loss)); return loss;
  }
  // Network.Fit: consecutive slices, no shuffling, short last batch; returns the last epoch's mean batch loss.
  float Fit(const std::vector<float>& x, const std::vector<float>& y, int epochs, int batchSize) {
    int64_t n = (int64_t)x.size() / in_; float epochLoss = 0.f;
    for (int e = 0; e < epochs; e++) {
      double sum = 0; int cnt = 0;
      for (int64_t s = 0; s < n; s += batchSize) {
        int64_t b = std::min<int64_t>(batchSize, n - s);
        std::vector<float> bx(x.begin() + s * in_, x.begin() + (s + b) * in_), by(y.begin() + s * out_, y.begin() + (s + b) * out_);
        sum += TrainBatch(bx, by); cnt++;
      }
      epochLoss = cnt ? (float)(sum / cnt) : 0.f;
    }
    return epochLoss;
  }
  std::vector<float> PredictBatch(const std::vector<float>& x) {
    int batch = (int)(x.size() / in_); std::vector<float> out((size_t)batch * out_);
    check(gn_forward_batch(m_, x.data(), batch, out.data())); return out;
  }
  std::vector<float> Predict(const std::vector<float>& x) { return PredictBatch(x); }
  void Close() { if (m_) { gn_model_destroy(m_); m_ = nullptr; } }
 private:
  Device& dev_; std::vector<gn_layer_desc> layers_; int workers_; gn_model* m_ = nullptr; Adam* opt_ = nullptr;
  int64_t n_params_ = 0, in_ = 0, out_ = 0;
};

}  // namespace goneuron
