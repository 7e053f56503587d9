/* souffle_b200.h -- C ABI of libsouffle_b200.so (sm_100a).
 *
 * Drop-in boundary for the reference's fused global-sync kernels.  Every entry point takes
 * plain device pointers and sizes (no torch types), is asynchronous on the given CUDA stream
 * unless stated otherwise, returns 0 on success or a SouffleStatus code, and leaves a
 * human-readable message in souffle_last_error() (thread-local).
 *
 * Reference interfaces replaced (paths relative to the reference project root):
 *   cpp/bert/bert_binding.cu:23-535          souffle_bert_layer<1,12,384,64,3072>      -> souffle_bert_*
 *   cpp/bert/bert_base_impl.cu:277-308       souffle_bert_base() (12-layer loop)       -> souffle_bert_* with n_layers=12
 *   cpp/lstm/lstm_binding.cu:30-72           fused_lstm<1,10,256,100>                  -> souffle_lstm_*
 *   cpp/swin_transformer/swin_transformer_binding.cu:155-209  swin_fused_feed_mlp      -> souffle_swin_mlp_forward
 *   cpp/swin_transformer/swin_transformer_binding.cu:62-100   swin_ffn                 -> souffle_gemm_f16
 *   cpp/swin_transformer/swin_trans_fc2_binding.cu:19-55      swin_trans_fc2           -> souffle_gemm_f16
 *   cpp/efficientnet/efficientnet_se_module_binding.cu:164-227  SE module (opt_level 2)  -> souffle_se_module_forward
 *   cpp/souffle_utils/cuda_utils.h:11-19,86-98  checkCuda / check_compatability        -> status codes + souffle_last_error
 */
#ifndef SOUFFLE_B200_H_
#define SOUFFLE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* souffle_stream_t; /* a cudaStream_t */

typedef enum SouffleStatus {
  SOUFFLE_OK = 0,
  SOUFFLE_BAD_SHAPE = 1,       /* a dimension is unsupported (see each function) */
  SOUFFLE_BAD_POINTER = 2,     /* null or misaligned (16 B) pointer */
  SOUFFLE_BAD_DEVICE = 3,      /* not an sm_100 device, or no device */
  SOUFFLE_NOT_CORESIDENT = 4,  /* the persistent grid would not be co-resident */
  SOUFFLE_CUDA_ERROR = 5,      /* a CUDA runtime/driver call failed; message has the detail */
  SOUFFLE_DEVICE_TIMEOUT = 6,  /* a bounded device-side wait expired (reported by souffle_*_status) */
  SOUFFLE_BAD_ARGUMENT = 7
} SouffleStatus;

/* Message of the last failing call on this thread ("" if none). */
const char* souffle_last_error(void);
/* ABI version of this library (bumped on incompatible changes). */
int souffle_abi_version(void);

/* ------------------------------------------------------------------------------------------
 * BERT encoder layers.  Replaces cpp/bert/bert_binding.cu:23-535 (one layer, compile-time
 * 1x384x768) and the 12-layer loop of cpp/bert/bert_base_impl.cu:590-678 with one persistent
 * launch over runtime shapes.
 * ------------------------------------------------------------------------------------------ */
typedef enum SouffleBertVariant {
  SOUFFLE_BERT_STD = 0,        /* scale 1/sqrt(head_dim), additive length mask, tanh-GELU, biases, vector gamma/beta */
  SOUFFLE_BERT_REF_COMPAT = 1  /* what the reference's fused kernel computes: scale 1/sqrt(hidden), ReLU,
                                  no proj/FFN bias, LayerNorm without affine (fused_sqq_bert.cu:2934,
                                  fused_sqq_feedforward.cu:2120-2133, bert_binding.cu:115) */
} SouffleBertVariant;

typedef struct SouffleBertDesc {
  int32_t batch;      /* sequences per call */
  int32_t seq;        /* tokens per sequence: multiple of 16, <= 128, or 256 / 384 */
  int32_t heads;      /* 2, 4, 8, 12 or 16 (hidden = heads * 64 in {128, 256, 512, 768, 1024}) */
  int32_t head_dim;   /* 64 */
  int32_t ffn;        /* intermediate size, multiple of 64 */
  int32_t n_layers;   /* >= 1: layers chained inside one launch */
  int32_t variant;    /* SouffleBertVariant */
  int32_t keep_probs; /* 1: parity mode: the softmax probabilities of the LAST layer are materialised and that layer's
                         stage outputs stay readable (souffle_bert_plan_buffer); 0: intermediates are dropped from L2
                         as soon as their last reader has run and are never written to DRAM */
  float eps;          /* LayerNorm epsilon (applied in fp32) */
  /* Optional tiling overrides, 0 = choose automatically. */
  int32_t bn_qkv, bn_fc1, bn_proj, split_proj, bn_fc2, split_fc2;
  int32_t max_ctas;   /* 0 = one CTA per SM */
  int32_t timeout_ms; /* device-side wait limit, 0 = 2000 ms */
  int32_t profile;    /* 1: record per-stage, per-CTA SM clock stamps (souffle_bert_plan_read_profile) */
  int32_t bm_qkv, bm_fc1, bm_proj, bm_fc2; /* tile heights (128 or 256), 0 = choose automatically */
  int32_t debug_max_slots;    /* experiment knob: cap on operand ring slots per CTA, 0 = as many as fit */
  int32_t debug_skip_arrival; /* failure-detection test hook, 0 = off: CTA (value-1) leaves at the first grid
                                 barrier without arriving, so the others run into the wait limit and the
                                 launch ends with SOUFFLE_DEVICE_TIMEOUT (nothing is in flight at that point) */
  int32_t autotune;   /* 1: plan creation times the likeliest tilings of every GEMM stage on the device (a few
                         launches each on the plan's own buffers, tens of milliseconds in all) and keeps the
                         fastest; stages with an explicit bm_ / bn_ / split_ setting are left alone.  0: tiles come
                         from the cycle model alone.  Two plans of one shape may then differ in summation order. */
  int32_t pair_mma;   /* 1: run on CTA pairs where the shape qualifies (seq <= 128, an even number of heads, more
                         (sequence, head) items than CTAs, at least 2048 rows): clusters of two CTAs share every
                         tensor-core instruction (cta_group::2), each CTA loads half of every weight tile and the
                         attention stage takes two heads per pair.  0 (default): single-CTA MMAs, which measure
                         3 % faster at batch 64 because the epilogues, not the operand traffic, bound the GEMM stages
                         once the main loops speed up.  souffle_bert_plan_uses_pairs reports what a plan uses. */
} SouffleBertDesc;

/* Device pointers to one layer's parameters, fp16.  Matrices use the reference's [K][N]
 * row-major layout (cpp/bert/test_souffle_bert_layer.py:139-143).  Vectors may be null
 * (bias = 0, gamma = 1, beta = 0). */
typedef struct SouffleBertLayerWeights {
  const void* qkv_w;  /* [3][H][H]  */
  const void* qkv_b;  /* [3][H]     */
  const void* proj_w; /* [H][H]     */
  const void* proj_b; /* [H]        */
  const void* ln1_g;  /* [H]        */
  const void* ln1_b;  /* [H]        */
  const void* fc1_w;  /* [H][F]     */
  const void* fc1_b;  /* [F]        */
  const void* fc2_w;  /* [F][H]     */
  const void* fc2_b;  /* [H]        */
  const void* ln2_g;  /* [H]        */
  const void* ln2_b;  /* [H]        */
} SouffleBertLayerWeights;

/* The packed parameter block of the reference's 12-layer entry (cpp/bert/bert_base_impl.cu:536-572; 7,235,328
 * fp16 values for batch 1, seq 384, :279): the attention mask [batch][seq][seq] (1 = attend), the Q, K, V and
 * output matrices (H x H each), the FFN matrices (H x F, F x H), then thirteen vectors: q, k, v, output bias, LN1
 * gamma, beta, FFN bias (F), FFN output bias, LN2 gamma, beta.  The reference runs all twelve layers on this one
 * set (:590-678).  Fills `out` with pointers into `blob` -- nothing is copied, the addresses keep the 16-byte
 * alignment of `blob` -- `mask_out` with the mask's address and `blob_bytes` with the block's size; any of the
 * three may be null.  Host-only arithmetic: works on any address, also without a GPU. */
int souffle_bert_packed_weights(const void* blob, int32_t batch, int32_t seq, int32_t hidden, int32_t ffn,
                                SouffleBertLayerWeights* out, const void** mask_out, size_t* blob_bytes);

typedef struct SouffleBertPlan SouffleBertPlan;

/* Set-up (allocates the plan's device workspace, repacks the weights for the tensor cores and
 * builds the stage program; synchronous, not on the hot path).  `layers` is a host array of
 * desc->n_layers records.  The caller's weight buffers are not referenced afterwards. */
int souffle_bert_plan_create(const SouffleBertDesc* desc, const SouffleBertLayerWeights* layers,
                             SouffleBertPlan** plan_out);
int souffle_bert_plan_destroy(SouffleBertPlan* plan);

/* y[B*S][H] = encoder(x[B*S][H]); fp16 device buffers, 16-byte aligned.  `seq_lens` (device
 * int32[B]) is optional: keys at positions >= len get the additive -10000 mask
 * (cpp/bert/kernels/softmax.cu:22-24).  Asynchronous on `stream`; calls on one plan must not
 * overlap. */
int souffle_bert_forward(SouffleBertPlan* plan, const void* x, const int32_t* seq_lens, void* y,
                         souffle_stream_t stream);
/* Same with HOST buffers (pinned or pageable): copies x in, runs, copies y out, synchronises. */
int souffle_bert_forward_host(SouffleBertPlan* plan, const void* x_host, const int32_t* seq_lens_host,
                              void* y_host, souffle_stream_t stream);
/* The same without the final synchronisation: y_host is complete once `stream` has caught up (the call makes
 * `stream` wait for the copy-out).  Consecutive calls are pipelined over the plan's own copy-in, compute and
 * copy-out streams and two sets of device buffers: the copy-in of call i+1 and the copy-out of call i-1 run while
 * the kernel of call i does.  x_host must be ready when the call is made (the copy-in does not wait for `stream`)
 * and stay unchanged, and y_host untouched, until `stream` has caught up;
 * pinned buffers are needed for the copies to overlap.  (The reference's entry points take device tensors only.) */
int souffle_bert_forward_host_async(SouffleBertPlan* plan, const void* x_host, const int32_t* seq_lens_host,
                                    void* y_host, souffle_stream_t stream);

/* The stage outputs the reference binding returns (cpp/bert/bert_binding.cu:534), for the
 * LAST layer of a plan created with keep_probs = 1 (other plans do not keep them).  Valid after a forward call
 * has completed. */
typedef enum SouffleBertBuffer {
  SOUFFLE_BUF_QKV = 0,   /* fp16 [3][B][heads][S][d]            */
  SOUFFLE_BUF_PROBS = 1, /* fp16 [B*heads][S][S] (keep_probs=1) */
  SOUFFLE_BUF_CTX = 2,   /* fp16 [B*S][H]  attention value output, heads merged */
  SOUFFLE_BUF_LN1 = 3,   /* fp16 [B*S][H]  post-LayerNorm attention block output */
  SOUFFLE_BUF_FC1 = 4    /* fp16 [B*S][F]  post-activation FFN hidden */
} SouffleBertBuffer;
int souffle_bert_plan_buffer(SouffleBertPlan* plan, int which, void** ptr_out, size_t* bytes_out);
/* Copies one of those buffers into caller memory (device pointer, `dst_bytes` >= its size) on `stream`. */
int souffle_bert_plan_copy_buffer(SouffleBertPlan* plan, int which, void* dst, size_t dst_bytes,
                                  souffle_stream_t stream);

/* Synchronises the plan's device and reports the device-side status of the last launch:
 * SOUFFLE_OK, or SOUFFLE_DEVICE_TIMEOUT with the stage/CTA in souffle_last_error(). */
int souffle_bert_plan_status(SouffleBertPlan* plan);
/* Per-stage stamps of the last launch (desc.profile=1): out[n_stages + 1][cta][16] int64 SM-clock values (the last
 * record holds {kernel entry, prologue done, last stage done}); for the stages
 * {stage start, this CTA's work done, barrier left} and, for GEMM stages, cycle totals {MMA issuer waiting
 * for operands, MMA issuer waiting for a free accumulator, producer waiting for a free ring slot, epilogue
 * waiting for an accumulator, epilogue busy} and, in words 8..15 of a GEMM record, the first epilogue warp's cycles in
 * {TMEM loads, arithmetic, stores} and the stamps {first operand copy issued, first operand chunk landed, last
 * accumulator committed, first accumulator seen by the epilogue, epilogue finished}; differences within one CTA
 * are cycles.
 * The in-kernel counterpart of the reference's profile_grid_clock buffers
 * (cpp/bert/kernels/fused_sqq_bert.cu:2330,2770; cpp/bert/bert_binding.cu:67-76).  Synchronises. */
int souffle_bert_plan_read_profile(SouffleBertPlan* plan, int64_t* out, size_t capacity_elems);
/* Number of kernels launched by the last forward call and the persistent grid size. */
int souffle_bert_plan_info(SouffleBertPlan* plan, int* launches_out, int* grid_out, int* n_stages_out);
/* 1 if the plan's launch runs on CTA pairs (see SouffleBertDesc.pair_mma), else 0. */
int souffle_bert_plan_uses_pairs(SouffleBertPlan* plan);
/* The tiling chosen for stage `index` of the program: out[0..5] = {stage type (0 GEMM, 1 attention, 2 LayerNorm),
 * tile rows, tile columns, split-K factor, work items, ring slots}.  The reference fixes these at compile time
 * (cpp/bert/kernels/bert.h:18-52); here they depend on the shape and on the SM count. */
int souffle_bert_plan_stage_info(SouffleBertPlan* plan, int index, int out[6]);

/* ------------------------------------------------------------------------------------------
 * Stacked LSTM, batch 1, as one wavefront launch.  Replaces fused_lstm<1,10,256,100>
 * (cpp/lstm/lstm_binding.cu:30-72).  Gate order i, j, f, o with the forget bias of +1
 * (cpp/lstm/lstm_reuse_shared_memory.cu:309-318).
 * ------------------------------------------------------------------------------------------ */
typedef struct SouffleLstmDesc {
  int32_t layers;          /* 1..18 (one thread-block cluster of 8 CTAs per layer; all clusters must be co-resident) */
  int32_t hidden;          /* 64, 128 or 256 (input width == hidden) */
  int32_t steps;           /* >= 1 */
  int32_t ref_input_delay; /* 1: feed x one step late like the reference kernel (step 0 sees zeros, the last
                              x is never consumed: lstm_reuse_shared_memory.cu:324-326); 0: standard */
  int32_t timeout_ms;      /* device-side wait limit, 0 = 2000 ms */
} SouffleLstmDesc;
typedef struct SouffleLstmPlan SouffleLstmPlan;
/* w_in / w_state: fp16 device [4*layers][hidden][hidden], index [4*layer + gate][out][in] (the reference's
 * layout with fp16 storage); bias: fp32 device [layers][hidden] or null.  The plan keeps its own copies. */
int souffle_lstm_plan_create(const SouffleLstmDesc* desc, const void* w_in, const void* w_state, const float* bias,
                             SouffleLstmPlan** plan_out);
int souffle_lstm_plan_destroy(SouffleLstmPlan* plan);
/* y[steps][hidden] (fp32, top layer's h per step) from x[steps][hidden] (fp32); zero initial state. */
int souffle_lstm_forward(SouffleLstmPlan* plan, const float* x, float* y, souffle_stream_t stream);
int souffle_lstm_plan_status(SouffleLstmPlan* plan);
/* 0: LSTM launches carry the cluster dimension alone (the default: residency of all clusters rests on the occupancy
 * check made at plan creation, every device-side wait is bounded, and Nsight Compute can capture the launch);
 * 1: SOUFFLE_LSTM_COOPERATIVE=1 was set when the library was loaded and the driver has so far accepted the
 * cooperative attribute on top of the cluster dimension. */
int souffle_lstm_launch_mode(void);

/* Has no counterpart in the reference.  The same stacked-LSTM forward for callers that must not allocate
 * device memory (a server whose memory pool owns the whole GPU, a plugin inside someone else's process, a
 * loop that cannot take the device-wide synchronisation cudaMalloc/cudaFree imply): no plan, no cudaMalloc,
 * cudaFree or other allocating call.  The kernel's scratch -- every published hidden state, the per-layer
 * arrival counters, the status words -- sits in a fixed array inside the library image (about 1.5 MB held
 * by every GPU that loads the library, until the process exits), so layers * steps * hidden must not exceed
 * 12 * 128 * 256 = 393,216; larger shapes are rejected with SOUFFLE_BAD_SHAPE (use a plan for those).
 * w_in / w_state (fp16 [4*layers][hidden][hidden]), bias (fp32 [layers][hidden] or null), x and y (fp32
 * [steps][hidden]) are device pointers and are used in place, so they must stay valid until the work on
 * `stream` has run.  `device_status` is optional: 4 device ints that receive {code, where, cta, 0}, code 0
 * meaning every bounded wait was satisfied.  The first call on a device also looks up the array's device
 * address and sets the kernel's attributes; make that first call before any stream capture begins.
 * All calls share the one array and it keeps the previous call's contents: the counters and status words
 * are cleared on `stream` at the start of each call, and two calls that overlap on the GPU (different
 * streams, or different host threads) would race on it -- serialise them. */
int souffle_lstm_forward_static(const SouffleLstmDesc* desc, const void* w_in, const void* w_state, const float* bias,
                                const float* x, float* y, int32_t* device_status, souffle_stream_t stream);
/* Has no counterpart in the reference.  For callers of souffle_lstm_forward_static that passed no
 * `device_status`: waits until `stream` is idle, then reads the status words the last such call on the current
 * device left in the built-in array (one device-to-host copy, no allocation) and returns SOUFFLE_OK or
 * SOUFFLE_DEVICE_TIMEOUT.  A call that did pass `device_status` reports there, not here. */
int souffle_lstm_static_status(souffle_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Plain fp16 GEMM with fp32 accumulation: c[M][N] = a[M][K] . w[K][N].
 * Replaces swin_ffn (swin_transformer_binding.cu:62-100, shapes (256,2048,512),(256,512,2048))
 * and swin_trans_fc2 (swin_trans_fc2_binding.cu:19-55) for any K % 64 == 0, N % 64 == 0.
 * `workspace` must hold souffle_gemm_workspace_bytes() bytes and is reusable across calls
 * that do not overlap.  The library clears it the first time it sees the address and keeps the barrier words
 * consistent from call to call; nobody else may write its first 128 bytes in between.  A caller that frees a
 * workspace, or hands its memory to another use, tells the library with souffle_workspace_forget() before the
 * address can come back with other contents: barrier words the library believes consistent but that were
 * overwritten make the next call's result undefined (the barriers may pass at once), not merely a timeout.
 * ------------------------------------------------------------------------------------------ */
size_t souffle_gemm_workspace_bytes(void);
int souffle_gemm_f16(const void* a, const void* w_kn, void* c, int32_t M, int32_t N, int32_t K,
                     void* workspace, size_t workspace_bytes, souffle_stream_t stream);

/* fc1 -> grid barrier -> fc2 in one launch, no bias/activation, both results returned:
 * hidden[M][F] = src[M][C] . fc1_w[C][F];  out[M][C] = hidden . fc2_w[F][C]
 * (cpp/swin_transformer/swin_transformer_binding.cu:155-209).  With a workspace of
 * souffle_swin_mlp_workspace_bytes(M, C, F) bytes fc2 is cut along K into fp32 planes that a third stage of the
 * same launch sums (the reference's fc2 runs its long K loop on 32 blocks, kernels/swin_fused_ffn_*.cu:393);
 * with only souffle_gemm_workspace_bytes() it runs unsplit. */
size_t souffle_swin_mlp_workspace_bytes(int32_t M, int32_t C, int32_t F);
int souffle_swin_mlp_forward(const void* src, const void* fc1_w, const void* fc2_w, void* hidden, void* out,
                             int32_t M, int32_t C, int32_t F, void* workspace, size_t workspace_bytes,
                             souffle_stream_t stream);

/* out[M][N] (fp16) = LayerNorm(sum_p partial[p][M][N] (fp32) + bias[N] + resid[M][N]) * gamma + beta, statistics
 * in fp32 over each row; bias, resid, gamma/beta (fp16) may be null.  N in {128, 256, 512, 768, 1024}.  This is the
 * normalisation stage of the fused layer (cpp/bert/kernels/fused_sqq_bert.cu:3690-3782) as a call of its own. */
int souffle_layernorm_forward(const float* partial, int32_t n_partial, const void* bias, const void* resid,
                              const void* gamma, const void* beta, void* out, int32_t M, int32_t N, float eps,
                              void* workspace, size_t workspace_bytes, souffle_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Swin transformer blocks (pre-LN, shifted-window attention with relative-position bias, MLP with tanh-GELU)
 * as one persistent launch of eight stages per block: LN1, QKV (+roll, window partition), window attention, proj
 * (+window reverse, roll back, residual), LN2, FC1+GELU, FC2 cut along K into fp32 planes, and the sum of the
 * planes + bias + residual.  `n_blocks` blocks are chained inside the launch (a stage of the network: the
 * reference needs 226 kernels for the model, python/models/tee:1); even-numbered blocks use `shift`, odd-numbered
 * ones `shift_alt` (the usual pair: 0 and window / 2).  The reference has the block only as TVM operator
 * definitions (python/models/swin_transformer/swin_transformer_main.py:11-86) and, in C++, its MLP GEMM pair; the
 * relative-position bias and the shift mask follow the benchmark config.
 * ------------------------------------------------------------------------------------------ */
typedef struct SouffleSwinDesc {
  int32_t batch;      /* images per call */
  int32_t res;        /* token grid side (14); res % window == 0 */
  int32_t dim;        /* channels: 128, 256, 512, 768 or 1024 */
  int32_t heads;      /* dim / heads must be 32, heads even */
  int32_t window;     /* 7 or 8 */
  int32_t shift;      /* cyclic shift of blocks 0, 2, ...; 0 <= shift < window */
  int32_t mlp_ratio;  /* hidden = dim * mlp_ratio */
  float eps;          /* LayerNorm epsilon */
  int32_t timeout_ms; /* device-side wait limit, 0 = 2000 ms */
  int32_t n_blocks;   /* blocks chained in one launch, 1..18; 0 = 1 */
  int32_t shift_alt;  /* cyclic shift of blocks 1, 3, ... */
} SouffleSwinDesc;
/* fp16 device pointers; matrices [K][N] row-major; rel_bias is [(2*window-1)^2][heads]. */
typedef struct SouffleSwinWeights {
  const void *ln1_g, *ln1_b, *qkv_w, *qkv_b, *rel_bias, *proj_w, *proj_b, *ln2_g, *ln2_b, *fc1_w, *fc1_b, *fc2_w, *fc2_b;
} SouffleSwinWeights;
typedef struct SouffleSwinPlan SouffleSwinPlan;
/* `weights` is a host array of n_blocks records. */
int souffle_swin_block_plan_create(const SouffleSwinDesc* desc, const SouffleSwinWeights* weights,
                                   SouffleSwinPlan** plan_out);
/* The same with the patch merging that ends a stage of the network run inside the launch
 * (python/models/swin_transformer/swin_patch_merge.py:1-17: tokens (2h,2w), (2h+1,2w), (2h,2w+1), (2h+1,2w+1)
 * concatenated to 4*dim channels, LayerNorm over them, reduction to 2*dim without bias): three more stages, the
 * gather done by the LayerNorm stage's copies.  `merge` null = blocks only; dim <= 512 and res even with it.
 * y is then [batch*(res/2)^2][2*dim]. */
typedef struct SouffleSwinMerge {
  const void *norm_g, *norm_b; /* fp16 [4*dim], both or neither */
  const void* reduction_w;     /* fp16 [4*dim][2*dim], [K][N] row-major */
} SouffleSwinMerge;
int souffle_swin_stage_plan_create(const SouffleSwinDesc* desc, const SouffleSwinWeights* weights,
                                   const SouffleSwinMerge* merge, SouffleSwinPlan** plan_out);
int souffle_swin_block_plan_destroy(SouffleSwinPlan* plan);
/* y[batch*res*res][dim] = block_{n-1}(... block_0(x)); fp16 device buffers; asynchronous on `stream`. */
int souffle_swin_block_forward(SouffleSwinPlan* plan, const void* x, void* y, souffle_stream_t stream);
int souffle_swin_block_plan_status(SouffleSwinPlan* plan);

/* ------------------------------------------------------------------------------------------
 * Squeeze-and-excite module, fp32, NCHW, one launch with one grid barrier.  Replaces
 * torch_dispatch_efficientnet_se_module_v2_short_cut_fused at its opt_level 2
 * (cpp/efficientnet/efficientnet_se_module_binding.cu:164-227; kernel
 * cpp/efficientnet/kernels/se_module_global_fused.cu:316-444) for any shape:
 *   pooled[c] = mean_hw input[b][c][:];  r[j] = s * sigmoid(s), s = sum_c pooled[c] * w_reduce[j][c];
 *   gate[c] = sigmoid(sum_j r[j] * w_expand[c][j]);  out[b][c][hw] = input[b][c][hw] + gate[c]
 * (the reference ADDS the gate to the input, :434-436).  `pooled` (optional, [batch][channels]) receives the channel
 * means, which the reference returns as well (:160).  `workspace`: souffle_se_module_workspace_bytes() bytes,
 * same rules as for souffle_gemm_f16.  Asynchronous on `stream`.
 * ------------------------------------------------------------------------------------------ */
size_t souffle_se_module_workspace_bytes(int32_t batch, int32_t channels, int32_t height, int32_t width);
int souffle_se_module_forward(const float* input, const float* w_reduce, const float* w_expand, float* out, float* pooled,
                              int32_t batch, int32_t channels, int32_t height, int32_t width, int32_t reduce, void* workspace,
                              size_t workspace_bytes, souffle_stream_t stream);

/* Blocks until `stream` is idle, then decodes the status words in `workspace`. */
int souffle_workspace_status(void* workspace, souffle_stream_t stream);
/* Drops what the library remembers about a caller-owned workspace address (to be called before the memory is
 * freed or re-used for something else); the next call that is given the address clears it again. */
int souffle_workspace_forget(void* workspace);

#ifdef __cplusplus
}
#endif
#endif /* SOUFFLE_B200_H_ */
