// Test/bench infrastructure: builds the reference's own fused BERT kernels for sm_100a from the
// sources where they lie (-I<reference>/cpp -I<reference>/cpp/bert) and exposes them through a
// small C ABI, without torch.  Launch configuration follows cpp/bert/bert_binding.cu:395-528
// (opt_level 3 and 4: fused_sqq_bert_attn, then fused_sqq_feedforward[_pipelined_v2]).
// Nothing here is part of the shipped library.
#include <cuda.h>
#include <cuda/pipeline>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mma.h>
#include <stdint.h>
#include <stdio.h>

#include "souffle_utils/cuda_utils.h"
#include "kernels/gemm.cu"

using namespace fuselage::experiments::networks::bert;

namespace {
struct Scratch {
  half *bias_qkv, *mask;
  float *softmax_sum, *ln1_sum, *ln1_var, *ln2_sum, *ln2_var;
  int64_t *attn_clock, *ff_clock;
  bool ready = false;
} g;
const int S = 384, H = 768, NH = 12, F = 3072;

int prepare() {
  if (g.ready) return 0;
  if (cudaMalloc(&g.bias_qkv, 3 * H * 2) || cudaMalloc(&g.mask, (size_t)NH * S * S * 2) ||
      cudaMalloc(&g.softmax_sum, NH * S * 4) || cudaMalloc(&g.ln1_sum, S * 4) || cudaMalloc(&g.ln1_var, S * 4) ||
      cudaMalloc(&g.ln2_sum, S * 4) || cudaMalloc(&g.ln2_var, S * 4) || cudaMalloc(&g.attn_clock, 9 * 108 * 4 * 8) ||
      cudaMalloc(&g.ff_clock, 5 * 96 * 4 * 8))
    return 1;
  cudaMemset(g.bias_qkv, 0, 3 * H * 2);
  cudaMemset(g.mask, 0, (size_t)NH * S * S * 2);
  g.ready = true;
  return 0;
}
}  // namespace

// One encoder layer at the reference's native shape [1,384,768]; outputs are the six tensors of
// bert_binding.cu:534.  Runs `iters` times and returns the mean device time of the two fused
// kernels in microseconds (the accumulators they add into are re-zeroed before each run, outside
// the timed region, as torch::zeros does in the binding).
extern "C" int ref_bert_layer_s384(half* src, half* qkv_w, half* fc_w, half* ff1_w, half* ff2_w, int opt_level,
                                   half* out_qkv, half* out_probs, half* out_ctx, half* out_ln1, half* out_fc1,
                                   half* out_final, int iters, float* mean_us) {
  if (opt_level != 3 && opt_level != 4) return 2;
  if (prepare()) return 1;
  half eps = 0.00001, gama = 1, beta = 0;
  const size_t smem = 108 * 1024;
  void* attn_args[] = {&qkv_w, &src, &g.bias_qkv, &out_qkv, &out_probs, &g.mask, &g.softmax_sum, &out_ctx,
                       &fc_w, &out_ln1, &g.ln1_sum, &g.ln1_var, &eps, &gama, &beta, &g.attn_clock};
  void* ff_args[] = {&out_ln1, &eps, &gama, &beta, &ff1_w, &out_fc1, &ff2_w, &out_final,
                     &g.ln2_sum, &g.ln2_var, &g.ff_clock, &out_final};
  const int gemm_k5_blocks = (F / (kBlockRowWarps * kGemmK5WarpRowTiles * kWmmaM)) *
                             (S / (kBlockColWarps * kGemmK5WarpColTiles * kWmmaN));
  const int gemm_k5_shared_mem =
      (kStage * (kChunkK * kWmmaK * (kBlockRowWarps * kGemmK5WarpRowTiles * kWmmaM + kInputSkew) +
                 kBlockColWarps * kGemmK5WarpColTiles * kWmmaN * (kChunkK * kWmmaK + kInputSkew))) * sizeof(half);
  const size_t ff_smem_o3 = gemm_k5_shared_mem +
      kStage * (kGemmK6BlockSliceKTiles * kWmmaK * (kGemmK6BlockRowTiles * kWmmaM + kInputSkew)) * sizeof(half2);
  const void* ff_kernel = opt_level == 3 ? (const void*)fused_sqq_feedforward : (const void*)fused_sqq_feedforward_pipelined_v2;
  const size_t ff_smem = opt_level == 3 ? ff_smem_o3 : smem;
  if (cudaFuncSetAttribute((const void*)fused_sqq_bert_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) return 3;
  if (cudaFuncSetAttribute(ff_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ff_smem)) return 3;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float total = 0.f;
  for (int it = 0; it < iters; ++it) {
    cudaMemset(g.softmax_sum, 0, NH * S * 4);
    cudaMemset(g.ln1_sum, 0, S * 4);
    cudaMemset(g.ln1_var, 0, S * 4);
    cudaMemset(g.ln2_sum, 0, S * 4);
    cudaMemset(g.ln2_var, 0, S * 4);
    cudaEventRecord(e0);
    if (cudaLaunchCooperativeKernel((const void*)fused_sqq_bert_attn, dim3(108), dim3(128), attn_args, smem)) return 4;
    if (cudaLaunchCooperativeKernel(ff_kernel, dim3(gemm_k5_blocks), dim3(128), ff_args, ff_smem)) return 5;
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) return 6;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    total += ms;
  }
  if (mean_us) *mean_us = total * 1000.f / (iters > 0 ? iters : 1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return cudaGetLastError() == cudaSuccess ? 0 : 7;
}
