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

#include <mutex>

#include "lstm_kernel.cu"

namespace souffle {

constexpr size_t kStaticHiddenFloats = (size_t)12 * 128 * 256;      // layers * steps * hidden <= this
constexpr size_t kStaticStatusOffset = 2 * kLstmDoneWords * sizeof(unsigned);   // two sets of counters, then the status words
constexpr size_t kStaticCtlBytes = kStaticStatusOffset + 256;
constexpr size_t kStaticScratchBytes = kStaticHiddenFloats * 4 + kStaticCtlBytes;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_lstm_static_scratch[kStaticScratchBytes];

struct StaticLstmDevice {
  std::mutex mutex;                   // guards the first-call set-up and the residency cache
  unsigned char* scratch = nullptr;   // device address of g_lstm_static_scratch on this device
  int sms = 0;
  bool ready = false;
  unsigned resident_ok[3] = {0u, 0u, 0u};   // per hidden size (64, 128, 256): bit L set = L layers were found resident
};
static StaticLstmDevice g_static_lstm[16];

}  // namespace souffle
