/*
 * goneuron_cuda.h -- C ABI of libgoneuron_cuda.so, the B200 (sm_100a) training
 * backend for GoNeuron models.
 *
 * The library takes over one whole training step (forward, loss, backward,
 * gradient all-reduce, Adam) and batched inference of a goneuron Sequential
 * model.  A Go host binds these entry points 1:1 through cgo in a package
 * `internal/cuda` that takes the place of the reference's per-op Metal
 * dispatch (reference: internal/layer/metal.go:6-50 declares the cgo surface
 * that is replaced; internal/layer/device.go:27-30 is the Device interface
 * that selects it; internal/net/net.go:412-436 TrainBatch is the caller).
 *
 * Conventions (same as the reference's cgo surface, metal.go:117,153,170):
 *   - every pointer argument is borrowed for the duration of the call only;
 *   - host tensors are dense row-major float32, one row per sample;
 *   - handles are opaque; device memory is owned by the handle;
 *   - every function returns GN_OK (0) or a negative gn_status and never
 *     aborts the process; gn_last_error() returns a message for the calling
 *     thread's most recent failure.
 * Calls on one gn_model are serialised by an internal mutex (the reference
 * serialises on MetalDevice.mu, metal.go:70).
 */
#ifndef GONEURON_CUDA_H
#define GONEURON_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum gn_status {
  GN_OK = 0,
  GN_ERR_INVALID_ARG = -1,   /* bad pointer, size or descriptor              */
  GN_ERR_CUDA = -2,          /* a CUDA runtime/driver call failed             */
  GN_ERR_NO_DEVICE = -3,     /* no usable sm_100 device                       */
  GN_ERR_NCCL = -4,          /* NCCL missing or a collective failed           */
  GN_ERR_UNSUPPORTED = -5,   /* layer kind / option not built                 */
  GN_ERR_TIMEOUT = -6,       /* a bounded device-side wait gave up            */
  GN_ERR_OOM = -7            /* device memory exhausted                       */
} gn_status;

/* Layer kinds on the hot path (reference constructors in goneuron/goneuron.go:59-340). */
typedef enum gn_layer_kind {
  GN_LAYER_DENSE = 1,          /* layer.NewDense(in,out,act)            internal/layer/layer.go:224-340   */
  GN_LAYER_CONV2D = 2,         /* layer.NewConv2D(inC,outC,k,s,p,act)   internal/layer/conv2d.go:60-140   */
  GN_LAYER_MAXPOOL2D = 3,      /* layer.NewMaxPool2D(inC,k,s,p)         internal/layer/maxpool2d.go:46    */
  GN_LAYER_FLATTEN = 4,        /* layer.NewFlatten()                    internal/layer/reshape.go:64-96   */
  GN_LAYER_LSTM_UNROLLED = 5,  /* NewSequenceUnroller(NewLSTM(in,H),T,returnSeq) unroller.go:57, lstm.go:276 */
  GN_LAYER_EMBEDDING = 6,      /* layer.NewEmbedding(vocab,dim)         internal/layer/embedding.go:30-60 */
  GN_LAYER_POSENC = 7,         /* layer.NewPositionalEncoding(T,dim)    internal/layer/transformer.go:12-84 */
  GN_LAYER_TRANSFORMER_BLOCK = 8, /* NewTransformerBlock(dim,heads,T,ff,causal) transformer.go:859-1279 */
  GN_LAYER_CLS_POOLING = 9,    /* layer.NewCLSPooling(T,dim)            internal/layer/transformer.go:1647-1777 */
  GN_LAYER_LAYERNORM = 10,     /* layer.NewLayerNorm(dim,eps,true) applied row-wise  layernorm.go:193-441 */
  GN_LAYER_BATCHNORM2D = 11,   /* layer.NewBatchNorm2D(C,eps,momentum,true) + SetInputDimensions  batchnorm2d.go:67-665 */
  GN_LAYER_AVGPOOL2D = 12,     /* layer.NewAvgPool2D(inC,k,s,p) + input dimensions   internal/layer/avgpool2d.go:43-228, 401-468 */
  GN_LAYER_DROPOUT = 13,       /* layer.NewDropout(p, inSize): in_size = inSize, dim = bits of float p;  internal/layer/dropout.go:36-155, 241-293.
                                  State: two floats = number of random draws consumed so far (low 20 bits | the rest). */
  GN_LAYER_RMSNORM = 14,       /* layer.NewRMSNorm(dim, eps) applied row-wise: dim = dim, reserved = bits of eps (0 selects 1e-5)  rmsnorm.go:157-336 */
  GN_LAYER_CONV1D = 15,        /* layer.NewConv1D(inC,outC,k,stride,pad,act): in_size = inC, out_size = outC, in_w = input length;
                                  the backward pass does not apply the activation's derivative  conv1d.go:128-288 */
  GN_LAYER_GRU_UNROLLED = 16   /* NewSequenceUnroller(NewGRU(in,H),T,returnSeq): in_size = in, out_size = H; parameters Wx [3H,in] |
                                  Wh [2H,H] | b [3H], gates update, reset, candidate  gru.go:81-534, unroller.go:57-213 */
} gn_layer_kind;

/* Activations (reference: internal/activations/activations.go:22-236,342-352). */
typedef enum gn_activation {
  GN_ACT_LINEAR = 0,
  GN_ACT_RELU = 1,
  GN_ACT_SIGMOID = 2,
  GN_ACT_TANH = 3,
  GN_ACT_SOFTMAX = 4,      /* the ActTypeSoftmax branch, layer.go:504-529 (reached with &activations.Softmax{}) */
  GN_ACT_LOGSOFTMAX = 5,   /* the ActTypeLogSoftmax branch, layer.go:530-560 */
  GN_ACT_GELU = 6,         /* activations.GELU (tanh form), activations.go:241-275 */
  GN_ACT_SILU = 7,         /* activations.SiLU, activations.go:277-309 */
  GN_ACT_LEAKY_RELU = 8,   /* activations.NewLeakyReLU(alpha), activations.go:62-82; alpha = bits of `reserved` (0 selects 0.01) */
  GN_ACT_ELU = 9           /* activations.NewELU(alpha), activations.go:311-340; alpha = bits of `reserved` (0 selects 1, as NewELU) */
} gn_activation;

/* Losses (reference: internal/loss/loss.go:53-105 MSE, :120-178 CrossEntropy). */
typedef enum gn_loss_kind { GN_LOSS_MSE = 0, GN_LOSS_CROSS_ENTROPY = 1 } gn_loss_kind;

/* One layer of a Sequential model.  Unused fields are 0. */
typedef struct gn_layer_desc {
  int32_t kind;        /* gn_layer_kind */
  int32_t activation;  /* gn_activation (Dense, Conv2D) */
  int32_t in_size;     /* Dense in; Conv2D/MaxPool in-channels; LSTM input size; Embedding vocab */
  int32_t out_size;    /* Dense out; Conv2D out-channels; LSTM hidden size; Embedding dim */
  int32_t kernel;      /* Conv2D / MaxPool2D / AvgPool2D window */
  int32_t stride;
  int32_t padding;
  int32_t in_h;        /* Conv2D / MaxPool2D input height (SetInputDimensions, conv2d.go:686-691) */
  int32_t in_w;
  int32_t seq_len;     /* unroller time steps; PosEnc / TransformerBlock / CLSPooling sequence length */
  int32_t dim;         /* PosEnc / TransformerBlock / CLSPooling / LayerNorm model width; BatchNorm2D: momentum as float bits (0 = 0.1) */
  int32_t heads;       /* TransformerBlock */
  int32_t ff_dim;      /* TransformerBlock */
  int32_t causal;      /* TransformerBlock */
  int32_t return_seq;  /* unroller: 0 = last hidden state only */
  int32_t reserved;    /* BatchNorm2D: eps as float bits (0 = 1e-5); Dense / Conv2D: alpha of LEAKY_RELU / ELU as float bits */
} gn_layer_desc;

typedef struct gn_ctx gn_ctx;
typedef struct gn_model gn_model;

#define GN_UNIQUE_ID_BYTES 128

/* ---- context ---------------------------------------------------------- */

/* Creates a single-GPU context on CUDA device `device`.
 * Replaces layer.GetDefaultDevice / NewMetalDevice (device.go:33-48, metal.go:76-98). */
int gn_init(int device, gn_ctx** out);

/* Multi-GPU: one context per GPU (one per process or per host thread).  Rank 0
 * obtains an id with gn_get_unique_id and hands the 128 bytes to every rank
 * (any host channel); each rank then calls gn_init_rank.  The ranks form one
 * NCCL communicator; the batch passed to gn_train_batch on each rank is that
 * rank's contiguous shard (same chunking rule as the worker pool,
 * internal/net/net.go:621-633).  No counterpart in the reference beyond the
 * goroutine pool (net.go:588-717), which this replaces. */
int gn_get_unique_id(unsigned char id[GN_UNIQUE_ID_BYTES]);
int gn_init_rank(int device, int rank, int world_size,
                 const unsigned char id[GN_UNIQUE_ID_BYTES], gn_ctx** out);
int gn_shutdown(gn_ctx* ctx);                 /* idempotent; mirrors MetalDevice.Close */
int gn_ctx_world_size(gn_ctx* ctx, int* world_size, int* rank);
int gn_synchronize(gn_ctx* ctx);              /* drains the context's stream (metal.go:199 waitForMetal) */
/* Number of polls a device-side wait (on an mbarrier of the tensor-core kernels) makes before it gives up; 0 restores
 * the default (2^24).  A wait that gives up stops its kernel's pipeline, the call returns GN_ERR_TIMEOUT, and
 * gn_train_batch leaves parameters and optimiser state unchanged; the context stays usable.  The failure-detection
 * tests set a limit of 1 to make a wait run out without faulting the GPU.  No counterpart in the reference, whose
 * Metal dispatch blocks without a bound (metal.go:199). */
int gn_ctx_set_spin_limit(gn_ctx* ctx, unsigned int polls);
/* CUDA-event stopwatch on the stream every kernel of this context is launched on: start records an
 * event, stop records a second one, waits for it and returns the device time between the two. */
int gn_timer_start(gn_ctx* ctx);
int gn_timer_stop(gn_ctx* ctx, float* ms);
const char* gn_last_error(void);

/* ---- model ------------------------------------------------------------- */

/* Compiles a layer list + loss into a device-resident execution plan with one
 * flat parameter buffer, one flat gradient buffer and Adam moments, in the
 * reference's flat layout (Network.initBuffers, net.go:91-127).
 * `virtual_workers` (>=1) selects which of the reference's worker layouts is
 * reproduced for the two order-dependent behaviours (embedding gradient of the
 * last sample per worker chunk, embedding.go:151-154; per-timestep LSTM gradient
 * clipping, lstm.go:694,725-751); 1 = trainBatchSequential (net.go:721-784). */
int gn_model_create(gn_ctx* ctx, const gn_layer_desc* layers, int n_layers,
                    int loss_kind, int virtual_workers, gn_model** out);
int gn_model_destroy(gn_model* m);            /* idempotent; mirrors Layer.Close (layer.go:805-845) */
int gn_model_param_count(gn_model* m, int64_t* n);
int gn_model_in_size(gn_model* m, int64_t* n);   /* floats per input sample  */
int gn_model_out_size(gn_model* m, int64_t* n);  /* floats per output sample */

/* Network.SetParams / Params / Gradients (net.go:549-571, 787-810). */
int gn_model_set_params(gn_model* m, const float* host, int64_t n);
int gn_model_get_params(gn_model* m, float* host, int64_t n);
/* Gradients exactly as fed to Adam by the last gn_train_batch: batch-summed,
 * all-reduced, multiplied by float32(1/global_batch) (net.go:702-706, 764-770). */
int gn_model_get_grads(gn_model* m, float* host, int64_t n);

/* opt.NewAdam + field updates (opt.go:93-121).  `timestep` is the number of
 * optimiser steps already taken (Adam.timestep, opt.go:113); pass -1 to keep it.
 * Re-read before every step so host-side LR schedulers keep working. */
int gn_adam_set(gn_model* m, float lr, float beta1, float beta2, float eps, int timestep);
int gn_adam_get_state(gn_model* m, float* m1, float* v, int64_t n, int* timestep);
int gn_adam_set_state(gn_model* m, const float* m1, const float* v, int64_t n, int timestep);

/* Network.TrainBatch (net.go:412-436): forward + loss + backward over `batch`
 * samples, gradients * 1/global_batch, NCCL all-reduce when world_size > 1, one
 * Adam step (Network.Step, net.go:260-284).  x: [batch, in_size], y: [batch,
 * out_size], host memory.  *mean_loss = sum of per-sample losses / global_batch.
 * With world_size > 1 `batch` is this rank's shard and `global_batch`/
 * `first_sample` place it in the global batch; pass global_batch = 0 for the
 * single-GPU meaning (global_batch = batch, first_sample = 0). */
int gn_train_batch(gn_model* m, const float* x, const float* y, int batch,
                   int global_batch, int first_sample, float* mean_loss);
/* Same step with x and y already resident in this context's device memory. */
int gn_train_batch_device(gn_model* m, const float* x_dev, const float* y_dev, int batch,
                          int global_batch, int first_sample, float* mean_loss);

/* Network.ForwardBatch / Predict / PredictBatch (net.go:439-457, sequential.go:118-164):
 * forward only.  out: [batch, out_size] host memory. */
int gn_forward_batch(gn_model* m, const float* x, int batch, float* out);

/* Device scratch the caller may fill (bench: inputs resident in HBM). */
int gn_device_alloc(gn_ctx* ctx, int64_t n_floats, float** dev);
int gn_device_free(gn_ctx* ctx, float* dev);
int gn_device_upload(gn_ctx* ctx, float* dev, const float* host, int64_t n_floats);
int gn_device_download(gn_ctx* ctx, float* host, const float* dev, int64_t n_floats);

/* Layer state that is not a parameter: BatchNorm2D running mean and variance (runningMean[C] | runningVar[C] per
 * BatchNorm2D layer, in layer order; batchnorm2d.go:124-128, GetRunningMean/GetRunningVar :837-838).  Updated by
 * gn_train_batch sample by sample in batch order, used by gn_forward_batch (inference mode, :472-509). */
int gn_model_state_count(gn_model* m, int64_t* n);
int gn_model_get_state(gn_model* m, float* host, int64_t n);
int gn_model_set_state(gn_model* m, const float* host, int64_t n);

/* Counters of the last gn_train_batch: kernels launched by this library, and
 * device time in ms of the whole step / of the part of the gradient all-reduce that
 * the compute stream had to wait for (the per-layer all-reduces run on a second
 * stream under the rest of the backward pass); CUDA events on the context's stream. */
typedef struct gn_step_stats {
  int64_t kernel_launches;
  float step_ms;
  float allreduce_ms;
  float gemm_ms;          /* sum over the step's dense-contraction launches */
  int64_t gemm_launches;
  double gemm_flops;      /* 2*M*N*K summed over those launches */
  double gemm_bytes;      /* bytes those launches must move: operand planes (4 B per element) + output (+ residual) */
  double split_bytes;     /* bytes the operand split passes of the step move: 4 B read + 4 B written per element */
} gn_step_stats;
int gn_model_last_stats(gn_model* m, gn_step_stats* out);
/* 0 = off (default); 1 = time every contraction launch with CUDA events. */
int gn_model_set_profiling(gn_model* m, int level);

/* ---- per-kernel entry points (parity tests diff each kernel against the CPU
 *      restatement; all pointers are HOST memory, copied in and out) --------- */

/* C[M,N] = A[M,K] * B[N,K]^T (+ bias[N]) ; row-major, fp32 in/out.
 * engine: 0 = SIMT fp32, 1 = tcgen05 split-operand (three BF16 products per fp32 product, fp32-level accuracy).  (Dense forward, layer.go:406 /
 * matmul_optimized.go:18-152 at batch level.) */
int gn_op_gemm_nt(gn_ctx* ctx, int engine, int M, int N, int K,
                  const float* A, const float* B, const float* bias, float* C);
/* Adam.StepInPlace on host arrays with explicit bias-correction exponent t
 * (opt.go:207-252). */
int gn_op_adam(gn_ctx* ctx, float* params, const float* grads, float* m1, float* v,
               int64_t n, float lr, float beta1, float beta2, float eps, int t, float grad_scale);

/* Multi-head attention of one TransformerBlock on host arrays: Q, K, V, O, dO, dQ, dK, dV are [B*T, D]
 * row-major with head h in columns [h*D/H, (h+1)*D/H); M and L (may be NULL) receive the row maximum and the
 * row sum of the softmax, [B*H*T].  Forward: scores q.k/sqrt(hd), causal mask, softmax, weighted sum of v
 * (transformer.go:470-503); with dO != NULL also the backward pass (transformer.go:589-657).
 * engine: 0 = warp-level tensor-core kernels, 1 = tcgen05 kernels (head size 64, T a multiple of 128). */
int gn_op_attention(gn_ctx* ctx, int engine, int B, int T, int D, int H, int causal,
                    const float* Q, const float* K, const float* V, const float* dO,
                    float* O, float* M, float* L, float* dQ, float* dK, float* dV);

/* One LayerNorm over `rows` rows of width n on host arrays: y = gamma * (x - mean) / sqrt(var + 1e-5) + beta
 * (layernorm.go:193-304); with dy != NULL also the backward pass with the reference's second term divided by
 * N * std^2 (layernorm.go:385-441): dx [rows, n], dgamma [n], dbeta [n] (sums over the rows). */
int gn_op_layernorm(gn_ctx* ctx, int64_t rows, int n, const float* x, const float* gamma, const float* beta, const float* dy,
                    float* y, float* dx, float* dgamma, float* dbeta);

/* One Conv2D layer (NCHW, zero padding) on host arrays: y = act(conv(x, w) + bias) (conv2d.go:716-959); with dy != NULL
 * (gradient with respect to y) also dx, dw, db of one batch (conv2d.go:997-1174).  engine: 0 = direct CUDA-core kernels,
 * 1 = implicit GEMM on the tensor-core engine (all three directions; the input gradient for stride 1). */
int gn_op_conv2d(gn_ctx* ctx, int engine, int B, int in_c, int out_c, int kernel, int stride, int pad, int H, int W, int activation,
                 const float* x, const float* w, const float* bias, const float* dy, float* y, float* dx, float* dw, float* db);

/* The classification head after its Dense product, on host arrays [B, V]: out = softmax(z) or log-softmax(z)
 * (activations.go:146-236); loss[B] = CrossEntropy(out, y) per sample (loss.go:120-138, probabilities clipped at 1e-10);
 * dz = the gradient that reaches the pre-activations: CrossEntropy's (out - y) pushed through the head's Jacobian
 * (loss.go:165-178, layer.go:504-560).  loss and dz may be NULL. */
int gn_op_softmax_ce(gn_ctx* ctx, int B, int V, int log_softmax, const float* z, const float* y, float* out, float* loss, float* dz);

/* The LSTM recurrence of SequenceUnroller(LSTM(in, H), T, returnSeq = false) on host arrays: x [B, T*in], wx [4H, in],
 * wh [4H, H], bias [4H] (gate order i, f, g, o); h_all, c_all [B, T, H] receive every step's hidden and cell state
 * (lstm.go:276-407: only the input-gate rows receive wx x + wh h).  With dh_last != NULL ([B, H], gradient of the last
 * hidden state) also the gate deltas of back-propagation through time, dgate [B, T, 4H] (lstm.go:476-691).
 * engine: 0 = input projection inside the recurrence kernel, 1 = as one tensor-core contraction over all B*T rows. */
int gn_op_lstm(gn_ctx* ctx, int engine, int B, int T, int in_size, int H, const float* x, const float* wx, const float* wh, const float* bias,
               const float* dh_last, float* h_all, float* c_all, float* dgate);

/* The same product as gn_op_gemm_nt with engine 1 (C = A B^T + bias on the tensor cores), for callers that
 * must not allocate device memory: hosts whose own pool already owns all of HBM, and hosts with a per-step
 * latency budget (cudaMalloc / cudaFree lock the allocator, cudaFree waits for the device).  It has no
 * counterpart in the reference.  A, B, bias (may be NULL) and C are DEVICE pointers supplied by the caller
 * (A [M,K], B [N,K], C [M,N], row-major, dense); the operand planes live in a fixed 16 MiB array inside the
 * library image, which every GPU that loads the library holds until the process exits.  Limit:
 * (M+N)*roundup8(K) <= 4 Mi floats, else GN_ERR_INVALID_ARG.  The entry point calls no cudaMalloc / cudaFree.
 * The first call on each device resolves the array's device address; make it before any stream capture.
 * All calls on one GPU share the array (it keeps the last call's planes; each call rewrites what it reads):
 * calls that overlap on the GPU race, so issue them one after the other. */
int gn_op_gemm_nt_static(gn_ctx* ctx, int M, int N, int K, const float* A_dev, const float* B_dev,
                         const float* bias_dev, float* C_dev);

#ifdef __cplusplus
}
#endif
#endif /* GONEURON_CUDA_H */
