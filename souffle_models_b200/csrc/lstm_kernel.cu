// Stacked-LSTM wavefront megakernel for sm_100a (batch 1).
//
// Replaces cpp/lstm/lstm_reuse_shared_memory.cu:179-337 (lstm_reuse_shared_memory_v10_vec: 320
// blocks, 109 grid.sync(), fp32 weights partly in registers).  Cell semantics are the
// reference's (python/models/lstm/tf_lstm.py:59-70; cpp/lstm/lstm_reuse_shared_memory.cu:309-318):
// gates i, j, f, o;  c' = c*sigmoid(f+1) + sigmoid(i)*tanh(j);  h' = tanh(c')*sigmoid(o).
//
// Design: every layer is owned by kLstmParts CTAs; a CTA keeps its 4*U gate rows of both weight
// matrices (fp16, [x;h] concatenated along K) in shared memory for the whole sequence and its
// units' cell state in registers.  There is no grid-wide barrier: a cell (layer l, step t)
// starts as soon as h(l-1,t) and h(l,t-1) are published, which is signalled by per-layer
// arrival counters (release/acquire).  Hidden states of every (layer, step) have their own slot
// in global memory, so a producer never overwrites data a slower consumer still needs (the
// reference re-uses one slot per layer with no ordering between its readers and writers).
// All waits are bounded; on expiry the CTA records a status word and leaves.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace souffle {

constexpr int kLstmThreads = 512;
constexpr int kLstmParts = 8;              // CTAs per layer
constexpr int kLstmMaxHidden = 256;

struct LstmParams {
  const __half* w_in;     // [4*L][H][H], row = output unit, col = input
  const __half* w_state;  // [4*L][H][H]
  const float* bias;      // [L][H] or null; added to all four gates of a unit (reference layout)
  const float* x;         // [T][H]
  float* y;               // [T][H]: top layer's h per step
  float* h_all;           // [L][T][H] scratch: every published hidden state
  unsigned* done;         // [L] arrival counters of this launch
  unsigned* done_next;    // [L] counters the next launch will use (cleared here)
  int* status;
  int layers, hidden, steps, ref_input_delay;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + __expf(-v)); }

__device__ __forceinline__ bool wait_count(const unsigned* ctr, unsigned target, const WaitCtl& c, int where) {
  uint32_t spins = 0;
  while (ld_acquire_u32(ctr) < target) {
    if (((++spins) & 0x3F) == 0) {
      if (*c.abort_smem) return false;
      if (globaltimer_ns() > c.deadline_ns) {
        record_timeout(c, DEV_TIMEOUT_FLAG, where);
        return false;
      }
    }
  }
  return true;
}

// Shared-memory layout: weights [rows = 4*U][2H halves] with a 64-byte pad per row, then the
// fp32 input vector [2H], the gate pre-activations [4*U] and an abort word.
__global__ void __launch_bounds__(kLstmThreads, 1) souffle_lstm_wavefront(const LstmParams p) {
  extern __shared__ __align__(16) uint8_t lsm[];
  const int H = p.hidden, L = p.layers, T = p.steps;
  const int U = H / kLstmParts;                 // units owned by this CTA
  const int rows = 4 * U;                       // gate rows, row = unit*4 + gate
  const int row_bytes = 2 * H * 2 + 64;
  __half* w_s = reinterpret_cast<__half*>(lsm);
  float* v_s = reinterpret_cast<float*>(lsm + (size_t)rows * row_bytes);
  float* g_s = v_s + 2 * H;
  int* abort_s = reinterpret_cast<int*>(g_s + rows);
  const int layer = blockIdx.x / kLstmParts, part = blockIdx.x % kLstmParts;
  const int tid = threadIdx.x;

  if (tid == 0) *abort_s = 0;
  if (blockIdx.x == 0 && tid < L) p.done_next[tid] = 0u;
  // ---- weights -> shared memory (once) ----
  {
    const int chunks_per_row = 2 * H / 8;       // 16-byte chunks: first H/8 from w_in, rest from w_state
    for (int i = tid; i < rows * chunks_per_row; i += kLstmThreads) {
      const int r = i / chunks_per_row, ch = i % chunks_per_row;
      const int unit = part * U + r / 4, gate = r % 4;
      const bool st = ch >= H / 8;
      const __half* src = (st ? p.w_state : p.w_in) + ((size_t)(layer * 4 + gate) * H + unit) * H + (st ? ch - H / 8 : ch) * 8;
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(w_s) + (size_t)r * row_bytes + ch * 16) =
          __ldg(reinterpret_cast<const uint4*>(src));
    }
  }
  __syncthreads();

  WaitCtl ctl;
  ctl.abort_smem = abort_s;
  ctl.status_g = p.status;
  ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;

  // thread -> (row, quarter): 4 threads share a row and interleave its 16-byte chunks
  const int tpr = kLstmThreads / rows;          // threads per row (4 for H=256)
  const int row = tid / tpr, q = tid % tpr;
  const int n_chunks = 2 * H / 8 / tpr;         // chunks per thread
  float c_state = 0.0f;                         // cell state of unit `tid` (tid < U)
  const float bias_u = (p.bias && tid < U) ? p.bias[layer * H + part * U + tid] : 0.0f;

  for (int t = 0; t < T; ++t) {
    // ---- wait for h(layer-1, t) and h(layer, t-1) ----
    if (tid == 0) {
      bool ok = true;
      if (layer > 0) ok = wait_count(p.done + layer - 1, (unsigned)kLstmParts * (t + 1), ctl, 700 + layer);
      if (ok && t > 0) wait_count(p.done + layer, (unsigned)kLstmParts * t, ctl, 800 + layer);
    }
    __syncthreads();
    if (*abort_s) break;
    // ---- [x ; h_prev] -> shared memory (L2-coherent loads: written by other SMs) ----
    for (int i = tid; i < 2 * H / 4; i += kLstmThreads) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      const int e = i * 4;
      if (e < H) {
        if (layer == 0) {
          const int tx = p.ref_input_delay ? t - 1 : t;
          if (tx >= 0) v = __ldcg(reinterpret_cast<const float4*>(p.x + (size_t)tx * H + e));
        } else {
          v = __ldcg(reinterpret_cast<const float4*>(p.h_all + ((size_t)(layer - 1) * T + t) * H + e));
        }
      } else if (t > 0) {
        v = __ldcg(reinterpret_cast<const float4*>(p.h_all + ((size_t)layer * T + t - 1) * H + (e - H)));
      }
      *reinterpret_cast<float4*>(v_s + e) = v;
    }
    __syncthreads();
    // ---- gate pre-activations: fp16 weights x fp32 vector, fp32 accumulate ----
    if (row < rows) {
      const uint8_t* wr = reinterpret_cast<const uint8_t*>(w_s) + (size_t)row * row_bytes;
      float acc = 0.0f;
#pragma unroll 4
      for (int j = 0; j < n_chunks; ++j) {
        const int ch = j * tpr + q;
        const uint4 u = *reinterpret_cast<const uint4*>(wr + ch * 16);
        const float4 a = *reinterpret_cast<const float4*>(v_s + ch * 8);
        const float4 b = *reinterpret_cast<const float4*>(v_s + ch * 8 + 4);
        const __half2* h2 = reinterpret_cast<const __half2*>(&u);
        const float2 w0 = __half22float2(h2[0]), w1 = __half22float2(h2[1]), w2 = __half22float2(h2[2]),
                     w3 = __half22float2(h2[3]);
        acc = fmaf(w0.x, a.x, acc); acc = fmaf(w0.y, a.y, acc); acc = fmaf(w1.x, a.z, acc); acc = fmaf(w1.y, a.w, acc);
        acc = fmaf(w2.x, b.x, acc); acc = fmaf(w2.y, b.y, acc); acc = fmaf(w3.x, b.z, acc); acc = fmaf(w3.y, b.w, acc);
      }
      for (int o = tpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (q == 0) g_s[row] = acc;
    }
    __syncthreads();
    // ---- cell update for the U owned units, publish h ----
    if (tid < U) {
      const float gi = g_s[tid * 4 + 0] + bias_u, gj = g_s[tid * 4 + 1] + bias_u, gf = g_s[tid * 4 + 2] + bias_u,
                  go = g_s[tid * 4 + 3] + bias_u;
      c_state = c_state * sigmoid_f(gf + 1.0f) + sigmoid_f(gi) * tanhf(gj);
      const float h = tanhf(c_state) * sigmoid_f(go);
      const int unit = part * U + tid;
      __stcg(p.h_all + ((size_t)layer * T + t) * H + unit, h);
      if (layer == L - 1) p.y[(size_t)t * H + unit] = h;
      __threadfence();
    }
    __syncthreads();
    if (tid == 0) atom_add_release_u32(p.done + layer, 1u);
  }
}

}  // namespace souffle
