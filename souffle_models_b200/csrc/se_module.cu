// Squeeze-and-excite module as one global-sync launch (fp32, NCHW).
//
// The reference's fused kernel (cpp/efficientnet/kernels/se_module_global_fused.cu:316-444) runs four phases
// separated by three grid.sync(): per-channel average pool (the channel's image kept in shared memory), the
// reduce GEMV with x*sigmoid(x), the expand GEMV with sigmoid, and the broadcast add of the gate onto the image.
// Here a channel's image is cut into slices handed out per warp, so that small channel counts still fill the GPU
// and small images cost no CTA-wide synchronisation; every warp keeps its slices in shared memory across the one
// grid barrier, and both tiny GEMVs are recomputed by every CTA that needs them instead of being exchanged through
// two more barriers: the input is read from HBM once and the output written once.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace souffle {

constexpr int kSeThreads = 512;
constexpr int kSeCacheFloats = 49152;         // 192 KiB of image slices per CTA
constexpr int kSeMaxReduce = 64;              // reduce channels
constexpr int kSeMaxChannels = 4096;          // channels (their means are staged in shared memory)

struct SeParams {
  const float* input;      // [batch][channels][hw]
  const float* w_reduce;   // [reduce][channels]
  const float* w_expand;   // [channels][reduce]
  float* out;              // [batch][channels][hw]
  float* pooled;           // optional [batch][channels] channel means (the reference returns them)
  float* partial;          // [batch*channels][slices] partial sums of the pool
  unsigned* sync;          // arrival counter of the grid barrier (zero at launch, left zero by the last CTA out)
  int* status;             // [0] code, [1] where, [2] cta
  int batch, channels, hw, reduce;
  int slices, slice_len;   // a channel image = slices pieces of slice_len floats (the last one shorter)
  int items;               // batch * channels * slices
  int cache;               // 1: the CTA's slices fit its shared memory
  unsigned long long timeout_ns;
};

__device__ __forceinline__ float se_sigmoid(float x) { return 1.0f / (1.0f + __expf(-x)); }

// Work is handed out per WARP: an item is one slice of one channel image; warp w of CTA b takes items
// (b * 16 + w), + gridDim.x * 16, ...  Everything but the grid barrier and the per-image reduce GEMV is
// warp-local, so a 7 x 7 image costs no CTA-wide synchronisation.
__global__ void __launch_bounds__(kSeThreads, 1) souffle_se_module(const SeParams p) {
  extern __shared__ float se_smem[];
  constexpr int kWarps = kSeThreads / 32;
  float* cache = se_smem;                                  // image slices of this CTA, kSeCacheFloats / kWarps per warp
  float* pooled_s = se_smem + kSeCacheFloats;              // channel means of one image [channels <= kSeMaxChannels]
  float* gate_in = pooled_s + kSeMaxChannels;              // reduce GEMV outputs of one image [reduce]
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * kWarps + warp, total_warps = gridDim.x * kWarps;
  float* my_cache = cache + warp * (kSeCacheFloats / kWarps);
  if (threadIdx.x == 0) abort_flag = 0;
  __syncthreads();

  // ---- phase 1: load this warp's slices (kept in shared memory when they fit) and their partial sums ----
  int slot = 0;
  for (int item = gw; item < p.items; item += total_warps, ++slot) {
    const int ch = item / p.slices, sl = item - ch * p.slices;          // ch = image * channels + channel
    const int begin = sl * p.slice_len;
    const int len = min(p.slice_len, p.hw - begin);
    const float* src = p.input + (size_t)ch * p.hw + begin;
    float* dst = my_cache + (size_t)slot * p.slice_len;
    float s = 0.0f;
    for (int i = lane; i < len; i += 32) {
      const float v = __ldg(src + i);
      if (p.cache) dst[i] = v;
      s += v;
    }
    s = warp_sum(s);
    if (lane == 0) p.partial[(size_t)ch * p.slices + sl] = s;
  }

  // ---- the one grid barrier: every partial sum is published ----
  __syncthreads();
  if (threadIdx.x == 0) {
    red_add_release_u32(p.sync, 1u);
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (ld_acquire_u32(p.sync) < gridDim.x) {
      if (((++spins) & 0x3F) == 0 && globaltimer_ns() - t0 > p.timeout_ns) {
        if (atomicCAS(p.status, (int)DEV_OK, (int)DEV_TIMEOUT_GRID) == (int)DEV_OK) {   // first CTA to give up records where
          p.status[1] = 900;
          p.status[2] = (int)blockIdx.x;
        }
        abort_flag = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (abort_flag) return;

  // ---- phases 2-4: per image the channel means and the reduce GEMV (x * sigmoid x) once per CTA, then per
  //      item this channel's gate (expand GEMV row, sigmoid) and the add ----
  const float inv_hw = 1.0f / (float)p.hw;
  const int items_per_img = p.channels * p.slices;
  // the images this CTA's warps touch: items [blockIdx.x * kWarps, ...) stride total_warps -> a CTA-uniform sequence
  const int rounds = (p.items + total_warps - 1) / total_warps;
  int cur_img = -1;
  slot = 0;
  for (int rd = 0; rd < rounds; ++rd, ++slot) {
    const int first = rd * total_warps + blockIdx.x * kWarps;          // item of warp 0 in this round
    const int last = min(first + kWarps - 1, p.items - 1);
    if (first >= p.items) break;
    for (int img = first / items_per_img; img <= last / items_per_img; ++img) {
      // a round of one CTA spans at most a few images; (re)build the image's reduce outputs when it changes
      if (img != cur_img) {
        __syncthreads();
        for (int k = threadIdx.x; k < p.channels; k += kSeThreads) {
          const float* pp = p.partial + (size_t)(img * p.channels + k) * p.slices;
          float s = 0.0f;
          for (int s2 = 0; s2 < p.slices; ++s2) s += __ldcg(pp + s2);       // written by other CTAs: read at L2
          pooled_s[k] = s * inv_hw;
        }
        __syncthreads();
        for (int j = warp; j < p.reduce; j += kWarps) {
          float acc = 0.0f;
          for (int k = lane; k < p.channels; k += 32) acc = fmaf(pooled_s[k], __ldg(p.w_reduce + (size_t)j * p.channels + k), acc);
          acc = warp_sum(acc);
          if (lane == 0) gate_in[j] = acc * se_sigmoid(acc);
        }
        __syncthreads();
        cur_img = img;
      }
      const int item = first + warp;
      if (item < p.items && item / items_per_img == img) {
        const int ch = item / p.slices, sl = item - ch * p.slices;
        const int c = ch - img * p.channels;
        float g = 0.0f;                                      // expand GEMV row of this channel: lanes over the reduce outputs
        for (int j = lane; j < p.reduce; j += 32) g = fmaf(gate_in[j], __ldg(p.w_expand + (size_t)c * p.reduce + j), g);
        g = se_sigmoid(warp_sum(g));
        if (p.pooled && sl == 0 && lane == 0) p.pooled[ch] = pooled_s[c];
        const int begin = sl * p.slice_len;
        const int len = min(p.slice_len, p.hw - begin);
        const float* src = p.cache ? my_cache + (size_t)slot * p.slice_len : p.input + (size_t)ch * p.hw + begin;
        float* dst = p.out + (size_t)ch * p.hw + begin;
        for (int i = lane; i < len; i += 32) dst[i] = src[i] + g;
      }
    }
  }

  // ---- leave the barrier word clean for the next launch: the last CTA out resets it ----
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned old = atomicAdd(p.sync + 1, 1u);
    if (old == gridDim.x - 1) {
      p.sync[0] = 0u;
      p.sync[1] = 0u;
    }
  }
}

}  // namespace souffle
