// Allocation-free LSTM entry point.
//
// Some hosts must not call cudaMalloc once they are running: an inference server that has handed
// all device memory to its own pool, a plugin loaded into a process whose allocator it does not
// own, or a latency-critical loop where the implicit device synchronisation of cudaMalloc/cudaFree
// is not acceptable.  For them the wavefront kernel's scratch (the published hidden states of every
// (layer, step), the per-layer arrival counters and the status words) lives in a fixed array that
// is part of the library image.  Every GPU that loads the library holds these kStaticScratchBytes
// until the process exits.
#pragma once
#include <cuda_runtime.h>

#include "lstm_kernel.cu"

namespace souffle {

constexpr size_t kStaticHiddenFloats = (size_t)12 * 128 * 256;      // layers * steps * hidden <= this
constexpr size_t kStaticCtlBytes = 512;                              // counters (2 x 32 x 4 B) + status
constexpr size_t kStaticScratchBytes = kStaticHiddenFloats * 4 + kStaticCtlBytes;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_lstm_static_scratch[kStaticScratchBytes];

struct StaticLstmDevice {
  unsigned char* scratch = nullptr;   // device address of g_lstm_static_scratch on this device
  int sms = 0;
  bool ready = false;
};
static StaticLstmDevice g_static_lstm[16];

}  // namespace souffle
