// Test/bench infrastructure: the reference's fused Swin fc1->fc2 kernel built for sm_100a from
// its source file, launched as cpp/swin_transformer/swin_transformer_binding.cu:176-206 does
// (grid (16,4) x 128 threads, 138,240 B, cooperative).  Not part of the shipped library.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include "swin_transformer/kernels/swin_fused_ffn_m256n2048k512_m256n512k2048.cu"

extern "C" int ref_swin_mlp_256x512x2048(half* src, half* fc1_w, half* fc2_w, half* fc1_out, half* fc2_out, int iters,
                                         float* mean_us) {
  const size_t smem = 138240;
  void* args[] = {&fc1_w, &src, &fc1_out, &fc2_w, &fc2_out};
  const void* k = (const void*)swin_transformer_fused_fc1_fc2;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) return 3;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float total = 0.f;
  int rc = 0;
  for (int it = 0; it < iters && !rc; ++it) {
    cudaEventRecord(e0);
    if (cudaLaunchCooperativeKernel(k, dim3(16, 4), dim3(128), args, smem)) rc = 4;
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = 6;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    total += ms;
  }
  if (mean_us) *mean_us = total * 1000.f / (iters > 0 ? iters : 1);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  return rc;
}
