// Stage program: the host-built description a persistent megakernel interprets.
//
// The reference fuses an encoder layer into one cooperative launch whose stages are separated
// by grid.sync() (cpp/bert/kernels/fused_sqq_bert.cu:34-2305: nine stages, compile-time shapes
// from cpp/bert/kernels/bert.h:8-52).  Here the stage list is data: every stage is a record in
// global memory, shapes are runtime values, and the same kernel runs a BERT layer, a chain of
// layers, the Swin MLP pair or a single GEMM.
#pragma once
#include <stdint.h>

namespace souffle {

enum StageType : int {
  STAGE_GEMM = 0,   // C = A . B with a fused epilogue
  STAGE_ATTN = 1,   // per (sequence, head, query tile): softmax(Q K^T * scale + mask) V
  STAGE_LN = 2,     // z = sum_p partial[p] + bias + resid ; y = LayerNorm(z)
  STAGE_ATTN_SWIN = 3,  // per (window, head): softmax(Q K^T * scale + relative-position bias + shift mask) V
};

enum EpilogueKind : int {
  EPI_F16 = 0,      // out[row, col] = f16(act(acc + bias)) (+ resid)
  EPI_QKV = 1,      // like EPI_F16 but scattered head-split to [3][B][heads][S][d]
  EPI_PARTIAL = 2,  // raw fp32 accumulators to partial[split][row][col]
  EPI_SWIN_QKV = 3, // rows (tokens) are rolled by -shift and scattered window-major: [3][windows][64][C]
  EPI_SWIN_PROJ = 4,// rows arrive window-major, are rolled back to token order; + bias + residual[token]
};

enum Activation : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2 };

// Pointer selectors: a stage either carries a plan-owned pointer or names a per-call argument.
enum PtrSel : int { PTR_PLAN = 0, PTR_CALL_X = 1, PTR_CALL_Y = 2 };

struct alignas(16) Stage {      // 16-byte multiples: records are fetched with bulk copies
  int type;
  // ---- GEMM ----
  int tm_a;          // tensor-map index of the A operand ([M][K], box 64 x bm); negative = per-call map
  int tm_b;          // tensor-map index of the B operand
  int tm_out;        // EPI_PARTIAL with out_tma: tensor-map index of the fp32 planes viewed as [splitk][M][N] (box 16 columns x
  int out_tma;       // 32 rows x 1 plane, 64B swizzle) through which the epilogue stores them; out_tma = 0: plain stores
  int M, N, K;
  int bm;            // tile height: 128, or 256 (two 128-row halves that share each B tile)
  int bn;            // tile width in N (multiple of 16, <= 256, divides N)
  int splitk;        // K is cut into this many independent partial products
  int b_mn_major;    // 0: B stored [N][K] (K contiguous); 1: B stored [K][N] (N contiguous, bn % 64 == 0)
  int epi;           // EpilogueKind
  int act;           // Activation
  int out_sel;       // PtrSel for `out`
  int resid_sel;     // PtrSel for `resid`
  int ldo;           // leading dimension of out / resid (elements)
  const void* bias;  // fp16 [N] or null
  const void* resid; // fp16 [M][ldo] or null
  void* out;         // fp16 output
  float* partial;    // fp32 [splitk][M][N] (EPI_PARTIAL and STAGE_LN)
  // ---- attention / head split ----
  int batch, heads, seq, head_dim;
  float scale;       // softmax scale applied to Q.K
  const int* lens;   // per-sequence valid length or null (selected at call time when lens_from_call)
  int lens_from_call;
  int tm_qkv;        // tensor map over the head-split buffer viewed as [3*B*heads*S][d], box 64 x 128
  int win, shift;    // Swin: window size (7) and cyclic shift; `seq` is then the side of the token grid
  const void* rel_bias;  // Swin: fp16 [(2*win-1)^2][heads] relative-position bias table
  void* probs;       // optional fp16 [B*heads][S][S] normalised probabilities (debug / parity output)
  // ---- layer norm ----
  const void* gamma; // fp16 [N] or null
  const void* beta;  // fp16 [N] or null
  float eps;
  int n_partial;     // number of fp32 partial planes to sum
  int prof_index;    // position of this stage in the program (set by the host when the program is built)
  // ---- weight prefetch: the B matrix of the GEMM stage two stages further on, pulled into L2 by all CTAs while
  //      they wait at the barrier that ends this stage (weights never depend on an earlier stage) ----
  uint32_t pf_bytes;
  const void* pf_ptr;
  // ---- buffers whose last reader was the stage before this one (multiples of 128 bytes, 128-byte aligned): their
  //      lines are dropped from L2 at the start of this stage, so that dead intermediates are never written to DRAM ----
  uint32_t dead_bytes[2];
  const void* dead_ptr[2];
  // ---- derived on the host by finalize_stage(): the kernel's lone producer / MMA lanes would otherwise
  //      spend a few thousand cycles per stage in integer divisions ----
  int tiles_n, kchunks, items, slot_bytes, nslots;
  uint32_t mg_splitk, mg_tiles_n, mg_kchunks;   // magic multipliers, see fast_div()
  uint32_t mg_seq, mg_head_dim, mg_heads;
};

// q = n / d for n * d < 2^32 as one multiply-high: mg = ceil(2^32 / d); d == 1 has no 32-bit multiplier.
inline uint32_t fast_div_magic(uint32_t d) { return d <= 1 ? 0u : (uint32_t)((0x100000000ull + d - 1) / d); }

constexpr int kMaxTensorMaps = 96;
constexpr int kMaxStages = 160;
constexpr int kProfSlots = 16;   // int64 words per (stage, CTA) record of the in-kernel profile

}  // namespace souffle
