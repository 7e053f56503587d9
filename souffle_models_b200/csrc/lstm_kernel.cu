// Stacked-LSTM wavefront megakernel for sm_100a (batch 1).
//
// Replaces cpp/lstm/lstm_reuse_shared_memory.cu:179-337 (lstm_reuse_shared_memory_v10_vec: 320
// blocks, 109 grid.sync(), fp32 weights partly in registers).  Cell semantics are the
// reference's (python/models/lstm/tf_lstm.py:59-70; cpp/lstm/lstm_reuse_shared_memory.cu:309-318):
// gates i, j, f, o;  c' = c*sigmoid(f+1) + sigmoid(i)*tanh(j);  h' = tanh(c')*sigmoid(o).
//
// Design: every layer is owned by one thread-block cluster of kLstmParts CTAs; a CTA keeps its
// 4*U gate rows of both weight matrices (fp16, [x;h] concatenated along K) on chip for the whole
// sequence -- three quarters in the registers of its 512 cell threads (48 each at hidden 256: what 18
// warps leave room for), the rest in shared memory -- and its units' cell state.  Every path through the (layer, step)
// grid has steps-1 hops along time and layers-1 hops across layers, so the hop along time is the one
// that has to be short: a CTA writes its units' new hidden state straight into the shared memory of
// the eight CTAs of its cluster (distributed shared memory, st.async: the store itself counts as a
// transfer on the receiver's mbarrier, no fence on either side) -- no trip through L2.  Only the hop to
// the next layer goes through global memory: one slot per (layer, step) and per-layer arrival counters.
// Every CTA of a layer publishes its own count of finished steps; the consumer checks all eight, so a CTA whose
// publication lags cannot be covered by its peers running ahead.
// Two more warps keep that hop off the cell arithmetic's path: a fetch warp brings the layer's input
// vectors into shared memory up to four steps ahead, and a publish warp pays for the release fence
// behind the hidden states the cell warps have stored.
// There is no grid-wide barrier.  All waits in the step loop are bounded; on expiry the CTA records a
// status word, leaves the loop and waits for its cluster at the final cluster barrier (shared
// memory must outlive the peers' remote stores).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace souffle {

constexpr int kLstmThreads = 512;                  // threads of the cell arithmetic
constexpr int kLstmBlock = kLstmThreads + 64;      // + the fetch warp and the publish warp
constexpr int kLstmParts = 8;                      // CTAs per layer = cluster size
constexpr int kLstmMaxHidden = 256;
constexpr int kLstmXBufs = 4;                      // input vectors the fetch warp may run ahead
constexpr int kLstmRegChunks = 3;                  // of a thread's (up to 4) weight chunks per gate row, those kept in registers
constexpr int kLstmMaxLayers = 18;
constexpr int kLstmDoneWords = 256;                // one set of published-step counters: kLstmMaxLayers * kLstmParts, rounded up
static_assert(kLstmMaxLayers * kLstmParts <= kLstmDoneWords, "counter block too small");

struct LstmParams {
  const __half* w_in;     // [4*L][H][H], row = output unit, col = input
  const __half* w_state;  // [4*L][H][H]
  const float* bias;      // [L][H] or null; added to all four gates of a unit (reference layout)
  const float* x;         // [T][H]
  float* y;               // [T][H]: top layer's h per step
  float* h_all;           // [L][T][H] scratch: every published hidden state
  unsigned* done;         // [L][kLstmParts] published-step counters of this launch, one per (layer, CTA of its cluster)
  unsigned* done_next;    // the counters the next launch will use (cleared here)
  int* status;
  int layers, hidden, steps, ref_input_delay;
  unsigned long long timeout_ns;
};

// ex2-based forms: absolute error of a few 1e-7 on values in [-1, 1], far inside the 5e-3 bar on hidden states
__device__ __forceinline__ float sigmoid_f(float v) { return __fdividef(1.0f, 1.0f + __expf(-v)); }
__device__ __forceinline__ float tanh_f(float v) { return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * v)); }

// Bounded wait on an mbarrier whose arrivals come from other CTAs of the cluster.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, const WaitCtl& c, int where) {
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if (((++spins) & 0xFF) == 0) {
      if (*c.abort_smem) return false;
      if (globaltimer_ns() > c.deadline_ns) {
        record_timeout(c, DEV_TIMEOUT_MBAR, where);
        return false;
      }
    }
  }
  return true;
}

// Position of element e of an input or hidden vector in shared memory: the vector is cut into chunks of eight
// elements (the columns one 16-byte chunk of fp16 weights multiplies); the first halves of all chunks come first, the
// second halves after them, so that the sixteen threads of a unit read 16 contiguous bytes each.
__host__ __device__ inline int lstm_vec_index(int e, int H) { return ((e >> 3) << 2) + (e & 3) + ((e & 4) ? H / 2 : 0); }

// Shared memory of a CTA, in this order: weights [rows = 4*U][2H halves, 64-byte pad per row] (only the chunks the
// cell threads do not keep in registers are read from it); input vectors
// [kLstmXBufs][H] fp32; hidden vectors [2][H] fp32 (written by the whole cluster); gate pre-activations
// [2][rows] fp32; mbarriers xfull[kLstmXBufs], xempty[kLstmXBufs], hfull[2]; abort, verdict (two, by step parity)
// and produced words.
__host__ __device__ inline size_t lstm_smem_bytes(int H) {
  const int rows = 4 * (H / kLstmParts);
  return (kLstmRegChunks < 4 ? (size_t)rows * (2 * H * 2 + 64) : 0) + (size_t)(kLstmXBufs * H + 2 * H + 2 * rows) * 4 + (2 * kLstmXBufs + 2) * 8 + 32;
}

__global__ void __launch_bounds__(kLstmBlock, 1) souffle_lstm_wavefront(const LstmParams p) {
  extern __shared__ __align__(16) uint8_t lsm[];
  const int H = p.hidden, L = p.layers, T = p.steps;
  const int U = H / kLstmParts;                 // units owned by this CTA
  const int rows = 4 * U;                       // gate rows, row = unit*4 + gate
  const int row_bytes = 2 * H * 2 + 64;
  __half* w_s = reinterpret_cast<__half*>(lsm);
  float* x_s = reinterpret_cast<float*>(lsm + (kLstmRegChunks < 4 ? (size_t)rows * row_bytes : 0));   // [kLstmXBufs][H]
  float* h_s = x_s + kLstmXBufs * H;                                          // [2][H]
  float* g_s = h_s + 2 * H;                                                   // [2][rows]
  uint64_t* bars = reinterpret_cast<uint64_t*>(g_s + 2 * rows);
  int* abort_s = reinterpret_cast<int*>(bars + 2 * kLstmXBufs + 2);
  // verdict of step t lives in slot t & 1: thread 0 can only write step t+2's after everyone has read step t's
  // (it has to pass the barrier of step t+1 first), so all threads leave the loop at the same iteration
  volatile int* verdict_s = abort_s + 4;
  const uint32_t produced_a = smem_u32(abort_s + 2);       // steps whose hidden states this CTA has stored to global memory
  const uint32_t xfull0 = smem_u32(bars), xempty0 = smem_u32(bars + kLstmXBufs), hfull0 = smem_u32(bars + 2 * kLstmXBufs);
  const int layer = blockIdx.x / kLstmParts;
  const int part = (int)cluster_cta_rank();     // == blockIdx.x % kLstmParts for clusters along x
  const int tid = threadIdx.x;

  if (tid == 0) {
    *abort_s = 0;
    verdict_s[0] = 1;
    verdict_s[1] = 1;
    abort_s[2] = 0;
    for (int i = 0; i < kLstmXBufs; ++i) {
      mbar_init(xfull0 + 8 * i, 32);            // the 32 lanes of the fetch warp
      mbar_init(xempty0 + 8 * i, (uint32_t)(16 * U));   // every thread of the cell arithmetic
    }
    for (int i = 0; i < 2; ++i) {               // h(0) and h(1): one local arrival that announces H * 4 bytes
      mbar_init(hfull0 + 8 * i, 1);
      mbar_expect_tx(hfull0 + 8 * i, (uint32_t)H * 4u);
    }
    fence_mbar_init();
  }
  if (blockIdx.x == 0)
    for (int i = tid; i < L * kLstmParts; i += kLstmBlock) p.done_next[i] = 0u;
  for (int i = tid; i < 2 * H; i += kLstmBlock) h_s[i] = 0.0f;               // h before the first step
  // ---- weights -> shared memory (once), unless the cell threads keep all of them in registers ----
  if (kLstmRegChunks < 4) {
    const int chunks_per_row = 2 * H / 8;       // 16-byte chunks: first H/8 from w_in, rest from w_state
    for (int i = tid; i < rows * chunks_per_row; i += kLstmBlock) {
      const int r = i / chunks_per_row, ch = i % chunks_per_row;
      const int unit = part * U + r / 4, gate = r % 4;
      const bool st = ch >= H / 8;
      const __half* src = (st ? p.w_state : p.w_in) + ((size_t)(layer * 4 + gate) * H + unit) * H + (st ? ch - H / 8 : ch) * 8;
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(w_s) + (size_t)r * row_bytes + ch * 16) =
          __ldg(reinterpret_cast<const uint4*>(src));
    }
  }
  __syncthreads();
  cluster_sync_all();                           // every CTA's barriers exist before anyone arrives on them

  WaitCtl ctl;
  ctl.abort_smem = abort_s;
  ctl.status_g = p.status;
  ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;

  if (tid >= kLstmThreads + 32) {
    // ---------------- publish warp: makes the stored hidden states visible to the next layer ----------------
    if (tid == kLstmThreads + 32) {
      uint32_t published = 0, spins = 0;
      while (published < (uint32_t)T) {
        const uint32_t n = ld_acquire_cta_shared_u32(produced_a) / (uint32_t)U;     // whole steps only
        if (n > published) {
          st_release_u32(p.done + layer * kLstmParts + part, n);      // this CTA's units of steps < n are in h_all
          published = n;
        } else if (((++spins) & 0xFF) == 0) {
          if (*ctl.abort_smem) break;
          if (globaltimer_ns() > ctl.deadline_ns) {
            record_timeout(ctl, DEV_TIMEOUT_FLAG, 950);
            break;
          }
        }
      }
    }
    __syncwarp();
  } else if (tid >= kLstmThreads) {
    // ---------------- fetch warp: the layer's input vector of every step -> shared memory ----------------
    const int lane = tid - kLstmThreads;
    for (int t = 0; t < T; ++t) {
      const int xb = t % kLstmXBufs, use = t / kLstmXBufs;
      int ok = 1;
      if (lane == 0 && use > 0) ok = mbar_wait(xempty0 + 8 * xb, (uint32_t)(use - 1) & 1u, ctl, 900) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (ok && layer > 0) {
        // lane k < 8 waits until CTA k of the layer below has published step t; the warp-wide vote (which also orders
        // the other lanes' loads behind these acquires) says when all eight have
        const unsigned* ctr = p.done + (layer - 1) * kLstmParts + (lane & (kLstmParts - 1));
        bool mine = lane >= kLstmParts;
        uint32_t spins = 0;
        for (;;) {
          if (!mine) mine = ld_acquire_u32(ctr) >= (unsigned)(t + 1);
          if (__all_sync(0xffffffffu, mine)) break;
          if (((++spins) & 0x3F) == 0) {
            int give_up = 0;
            if (lane == 0) {
              if (*ctl.abort_smem) {
                give_up = 1;
              } else if (globaltimer_ns() > ctl.deadline_ns) {
                record_timeout(ctl, DEV_TIMEOUT_FLAG, 700 + layer);
                give_up = 1;
              }
            }
            if (__shfl_sync(0xffffffffu, give_up, 0)) {
              ok = 0;
              break;
            }
          }
        }
      }
      if (!ok) {
        if (lane == 0) *abort_s = 1;
        break;
      }
      const float* src = nullptr;
      if (layer == 0) {
        const int tx = p.ref_input_delay ? t - 1 : t;
        if (tx >= 0) src = p.x + (size_t)tx * H;
      } else {
        src = p.h_all + ((size_t)(layer - 1) * T + t) * H;
      }
      for (int i = lane; i < H / 4; i += 32) {     // elements 4i .. 4i+3 = one half of chunk i / 2 (see lstm_vec_index)
        const float4 v = src ? __ldcg(reinterpret_cast<const float4*>(src) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(x_s + xb * H + (i & 1) * (H / 2) + (i >> 1) * 4) = v;
      }
      mbar_arrive(xfull0 + 8 * xb);             // release: this lane's stores are visible to whoever waits
    }
  } else {
    // ---------------- cell arithmetic ----------------
    // Sixteen threads share a unit: thread (u, q) multiplies the four gate rows of unit u with the 16-byte chunks
    // q, q + 16, ... of [x ; h], so a chunk of the vector is read once for four rows; the sixteen partial sums meet
    // by shuffles, and lane q = 0 ends up with the unit's four gate pre-activations in registers -- no second trip
    // through shared memory, no barrier between the products and the cell update.
    const int n_act = 16 * U;                   // 128, 256 or 512 threads
    if (tid < n_act) {
      const int u = tid >> 4, q = tid & 15;
      const int nj = H / 64;                    // chunks per thread: 1, 2 or 4
      float c_state = 0.0f;                     // cell state of unit u (the same value in all sixteen lanes)
      const int unit = part * U + u;
      const float bias_u = p.bias ? p.bias[layer * H + unit] : 0.0f;
      const uint32_t h_s_a = smem_u32(h_s);
      const uint8_t* wu = reinterpret_cast<const uint8_t*>(w_s) + (size_t)(4 * u) * row_bytes;
      // this thread's weights: chunk j * 16 + q of the four gate rows of unit u, straight from global memory
      uint4 wreg[kLstmRegChunks > 0 ? kLstmRegChunks : 1][4];
#pragma unroll
      for (int j = 0; j < kLstmRegChunks; ++j) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          wreg[j][g] = make_uint4(0u, 0u, 0u, 0u);
          if (j < nj) {
            const int ch = j * 16 + q;
            const bool st = ch >= H / 8;
            const __half* src = (st ? p.w_state : p.w_in) + ((size_t)(layer * 4 + g) * H + unit) * H + (st ? ch - H / 8 : ch) * 8;
            wreg[j][g] = __ldg(reinterpret_cast<const uint4*>(src));
          }
        }
      }
      for (int t = 0; t < T; ++t) {
        const int xb = t % kLstmXBufs, hb = t & 1;          // h(t) goes to h_s[hb]; h(t-1) is in h_s[hb ^ 1]
        // ---- one thread waits for x(t) and h(t-1); its verdict is the CTA's ----
        if (tid == 0) {
          bool ok = mbar_wait(xfull0 + 8 * xb, (uint32_t)(t / kLstmXBufs) & 1u, ctl, 910);
          if (ok && t > 0) {
            ok = mbar_wait_cluster(hfull0 + 8 * (hb ^ 1), (uint32_t)((t - 1) >> 1) & 1u, ctl, 800 + layer);
            // that barrier's next phase receives h(t+1); nobody sends it before having this CTA's h(t)
            if (ok && t + 1 < T) mbar_expect_tx(hfull0 + 8 * (hb ^ 1), (uint32_t)H * 4u);
          }
          if (!ok) *abort_s = 1;
          verdict_s[t & 1] = ok ? 1 : 0;
        }
        named_barrier_sync(1, n_act);
        if (verdict_s[t & 1] == 0) break;
        // ---- gate pre-activations: fp16 weights x fp32 vector, fp32 accumulate ----
        const float* xv = x_s + xb * H;
        const float* hv = h_s + (hb ^ 1) * H;
        float acc[4][2];
#pragma unroll
        for (int g = 0; g < 4; ++g) acc[g][0] = acc[g][1] = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < nj) {
            const int ch = j * 16 + q;                      // chunk of [x ; h]
            const bool is_h = ch >= H / 8;
            const float* vec = is_h ? hv : xv;
            const int cl = is_h ? ch - H / 8 : ch;
            const float4 a = *reinterpret_cast<const float4*>(vec + cl * 4);
            const float4 b = *reinterpret_cast<const float4*>(vec + H / 2 + cl * 4);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w;
              if (j < kLstmRegChunks) {
                uint4& wr = wreg[j < kLstmRegChunks ? j : 0][g];
                // opaque to the optimiser: otherwise the fp16 -> fp32 conversions are hoisted out of the step loop
                // and the weights occupy twice the registers
                asm volatile("" : "+r"(wr.x), "+r"(wr.y), "+r"(wr.z), "+r"(wr.w));
                w = wr;
              } else {
                w = *reinterpret_cast<const uint4*>(wu + (size_t)g * row_bytes + ch * 16);
              }
              const __half2* h2 = reinterpret_cast<const __half2*>(&w);
              const float2 w0 = __half22float2(h2[0]), w1 = __half22float2(h2[1]), w2 = __half22float2(h2[2]),
                           w3 = __half22float2(h2[3]);
              acc[g][0] = fmaf(w0.x, a.x, acc[g][0]); acc[g][1] = fmaf(w0.y, a.y, acc[g][1]);
              acc[g][0] = fmaf(w1.x, a.z, acc[g][0]); acc[g][1] = fmaf(w1.y, a.w, acc[g][1]);
              acc[g][0] = fmaf(w2.x, b.x, acc[g][0]); acc[g][1] = fmaf(w2.y, b.y, acc[g][1]);
              acc[g][0] = fmaf(w3.x, b.z, acc[g][0]); acc[g][1] = fmaf(w3.y, b.w, acc[g][1]);
            }
          }
        }
        mbar_arrive(xempty0 + 8 * xb);                      // this thread has read x(t)
        float gsum[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float v = acc[g][0] + acc[g][1];
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          gsum[g] = v;
        }
        // ---- cell update of unit u; h(t) -> the whole cluster and the next layer ----
        // All sixteen lanes hold the four sums.  Lanes 0..3 of the group take one gate's nonlinearity each (f, i, j, o),
        // the four results come back by shuffle, and every lane then carries the same cell state and h: the sends to
        // the eight CTAs of the cluster are issued by eight lanes at once.
        {
          const int q4 = q & 3;
          const float pre = (q4 == 0 ? gsum[2] + 1.0f : q4 == 1 ? gsum[0] : q4 == 2 ? gsum[1] : gsum[3]) + bias_u;
          const float act = q4 == 2 ? tanh_f(pre) : sigmoid_f(pre);
          const int base = tid & 16;                        // lane of q == 0 within the warp
          const float sf = __shfl_sync(0xffffffffu, act, base), si = __shfl_sync(0xffffffffu, act, base + 1);
          const float tj = __shfl_sync(0xffffffffu, act, base + 2), so = __shfl_sync(0xffffffffu, act, base + 3);
          c_state = c_state * sf + si * tj;
          const float h = tanh_f(c_state) * so;
          const uint32_t off = (uint32_t)(hb * H + lstm_vec_index(unit, H)) * 4u;
          if (q < kLstmParts)
            st_async_b32(map_shared_rank(h_s_a + off, (uint32_t)q), __float_as_uint(h), map_shared_rank(hfull0 + 8u * (uint32_t)hb, (uint32_t)q));
          if (q == 0) {
            __stcg(p.h_all + ((size_t)layer * T + t) * H + unit, h);
            if (layer == L - 1) p.y[(size_t)t * H + unit] = h;
            red_add_release_cta_shared_u32(produced_a, 1u);   // the publish warp takes it from here
          }
        }
      }
    }
  }
  // Nobody leaves while a peer may still store into its shared memory.
  __syncthreads();
  cluster_sync_all();
}

}  // namespace souffle
