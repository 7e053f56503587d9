// Test/bench infrastructure: the reference's LSTM wavefront kernel built for sm_100a from its
// source file, launched as cpp/lstm/lstm_binding.cu:44-70 does (320 blocks x (32,8), 48 KiB,
// cooperative).  Not part of the shipped library.
#include <cuda_runtime.h>
#include <stdio.h>

#include "lstm/lstm_reuse_shared_memory.cu"

extern "C" int ref_lstm_10x256x100(float* x, float* w_in, float* w_state, float* y, int iters, float* mean_us) {
  const int L = 10, Hd = 256, T = 100;
  float *c, *h, *obuf, *bias, *inw;
  if (cudaMalloc(&c, T * Hd * 4) || cudaMalloc(&h, T * Hd * 4) || cudaMalloc(&obuf, 8 * L * Hd * 4) ||
      cudaMalloc(&bias, L * Hd * 4) || cudaMalloc(&inw, L * Hd * 4))
    return 1;
  void* args[] = {&x, &y, &c, &h, &inw, &w_in, &w_state, &bias, &obuf};
  const void* k = (const void*)lstm_reuse_shared_memory_v10_vec<1, 10, 256, 100>;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float total = 0.f;
  int rc = 0;
  for (int it = 0; it < iters && !rc; ++it) {
    cudaMemset(y, 0, T * Hd * 4);
    cudaMemset(c, 0, T * Hd * 4);
    cudaMemset(h, 0, T * Hd * 4);
    cudaMemset(obuf, 0, 8 * L * Hd * 4);
    cudaMemset(bias, 0, L * Hd * 4);
    cudaMemset(inw, 0, L * Hd * 4);
    cudaEventRecord(e0);
    if (cudaLaunchCooperativeKernel(k, dim3(320), dim3(32, 8), args, 48 * 1024)) rc = 4;
    cudaEventRecord(e1);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = 6;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    total += ms;
  }
  if (mean_us) *mean_us = total * 1000.f / (iters > 0 ? iters : 1);
  cudaFree(c); cudaFree(h); cudaFree(obuf); cudaFree(bias); cudaFree(inw);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  return rc;
}
