// Test/bench infrastructure: the reference's fused squeeze-and-excite kernel built for sm_100a from its
// source file (cpp/efficientnet/kernels/se_module_global_fused.cu:316-444) and launched as
// cpp/efficientnet/efficientnet_se_module_binding.cu:136-156 does at opt_level 2 (one block of 256 threads
// per channel tile, the binding's dynamic shared-memory size per shape, cooperative).
// Only shapes the binding dispatches with ONE channel per block are offered: with more channels per block
// the kernel's final stage reads its shared-memory copy at stride H*W although it was written at the padded
// stride (:431-436 against :344-352), so its output for those shapes is not the module's.
// Not part of the shipped library.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "souffle_utils/cuda_kernel_utils.h"
#include "efficientnet/kernels/se_module_global_fused.cu"

template <int64_t H, int64_t W, int64_t C, int64_t R>
static int run_se(float* input, float* w_reduce, float* w_expand, float* pooled, float* out, size_t smem, int iters,
                  float* mean_us) {
  float *reduce_out = nullptr, *expand_out = nullptr;
  int64_t* prof = nullptr;
  if (cudaMalloc(&reduce_out, R * 4) || cudaMalloc(&expand_out, C * 4) || cudaMalloc(&prof, 6 * C * 8 * 8)) return 1;
  void* args[] = {&input, &pooled, &w_reduce, &reduce_out, &w_expand, &expand_out, &out, &prof};
  const void* k = (const void*)efficientnet_se_module_v2_short_cut_fused<1, H, W, C, R, 1>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) return 3;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float total = 0.f;
  int rc = 0;
  for (int it = 0; it < iters && !rc; ++it) {
    cudaEventRecord(e0);
    if (cudaLaunchCooperativeKernel(k, dim3((unsigned)C), dim3(kBlockSize), args, smem)) rc = 4;
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = 6;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    total += ms;
  }
  if (mean_us) *mean_us = total * 1000.f / (iters > 0 ? iters : 1);
  cudaFree(reduce_out); cudaFree(expand_out); cudaFree(prof);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  return rc;
}

// input [1][C][H][W], w_reduce [R][C], w_expand [C][R], pooled [C], out [1][C][H][W], all fp32 on the device.
// Returns 2 for a shape that is not offered.
extern "C" int ref_se_module(int height, int channels, int reduce, float* input, float* w_reduce, float* w_expand,
                             float* pooled, float* out, int iters, float* mean_us) {
  if (height == 56 && channels == 96 && reduce == 4)
    return run_se<56, 56, 96, 4>(input, w_reduce, w_expand, pooled, out, 48 * 1024, iters, mean_us);
  if (height == 28 && channels == 144 && reduce == 6)
    return run_se<28, 28, 144, 6>(input, w_reduce, w_expand, pooled, out, 48 * 1024, iters, mean_us);
  if (height == 14 && channels == 240 && reduce == 10)
    return run_se<14, 14, 240, 10>(input, w_reduce, w_expand, pooled, out, 32 * 1024, iters, mean_us);
  if (height == 14 && channels == 480 && reduce == 20)
    return run_se<14, 14, 480, 20>(input, w_reduce, w_expand, pooled, out, 24 * 1024, iters, mean_us);
  return 2;
}
