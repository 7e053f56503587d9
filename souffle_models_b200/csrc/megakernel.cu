// Persistent global-sync megakernel for sm_100a.
//
// One CTA per SM interprets a stage program (stage_program.h).  Dense contractions run on
// tcgen05.mma with fp32 accumulators in tensor memory, operands arrive by TMA into a
// 128B-swizzled shared-memory ring, and the softmax / LayerNorm / GELU epilogues read the
// accumulators straight out of TMEM.  Stages are separated by a bounded grid barrier.
//
// Reference behaviour covered (paths relative to the reference project root):
//   cpp/bert/kernels/fused_sqq_bert.cu:34-2305   whole encoder layer in one cooperative launch
//   cpp/bert/kernels/fused_sqq_bert.cu:2308-3785 attention half (QKV, QK^T, softmax, PV, proj, LN)
//   cpp/bert/kernels/fused_sqq_feedforward.cu:1728-2617 FFN half (FC1+act, FC2+residual, LN)
//   cpp/swin_transformer/kernels/swin_fused_ffn_m256n2048k512_m256n512k2048.cu:9-769 fc1 -> fc2
//   cpp/swin_transformer/kernels/gemm_three_stages.h:8-379 and kernels/gemm_k6.cu:9-339 single GEMMs
//
// Warp roles (384 threads): warp 0 = TMA producer (one elected lane), warp 1 = MMA issuer and
// TMEM owner, warps 2..9 = epilogue (warp w reads TMEM lanes 32*(w%4) .. +31; two warps share a
// lane quarter and take alternate 32-column chunks) and attention softmax warps; warps 10..11 are spare:
// they take LayerNorm rows like every other warp and drop dead buffers from L2 in front of the other stages.
// Every wait (mbarrier, grid barrier) is bounded by a wall-clock deadline; on expiry the CTA
// records a status word, drains and returns, so a fault never leaves the GPU spinning.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"
#include "stage_program.h"

namespace souffle {

constexpr int kThreads = 384;               // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue / softmax, warps 10..11 take rows of
                                            // the LayerNorm stages only (registers are handed out per four warps: a block of
                                            // ten warps is charged for twelve, so the two extra warps cost nothing)
constexpr int kEpiWarps = 8, kEpiThreads = kEpiWarps * 32;
constexpr int kRingBytes = 196608;          // 192 KiB operand ring (4 x 48 KiB, 3 x 64 KiB or 6 x 32 KiB slots)
constexpr int kCtlBytes = 1024;             // barriers + control words
constexpr int kVecBytes = 16384;             // per-stage vectors staged in shared memory (a GEMM's bias as fp32: N <= 4096)
constexpr int kStageRow = 64;                // bytes per staged row; the 16-byte pieces of a row are XOR-swizzled (see below)
constexpr int kStageWarp = 32 * kStageRow;   // one epilogue warp's transpose buffer
constexpr int kStageBytes = 8 * kStageWarp;  // 16 KiB
// Layout after the control block: ring | bias vector | store staging.  The attention stage with three
// key blocks needs 208 KiB and simply runs over all three regions (it uses neither of the other two).
constexpr int kSmemBytes = kCtlBytes + kRingBytes + kVecBytes + kStageBytes + 1024;  // + alignment slack
constexpr int kMaxSlots = 8;
constexpr uint32_t kTmemCols = 512;
constexpr int kATileBytes = 128 * 64 * 2;   // 128 rows x 64 halves
constexpr int kAccStride = 256;             // TMEM columns between the two accumulator buffers
constexpr int kOCol = 384;                  // TMEM column of the attention output accumulator

struct MegaParams {
  const Stage* stages;        // plan-owned stage list, or null to use the inline stages
  int n_stages;
  const CUtensorMap* maps;    // plan-owned tensor maps (indices >= 0)
  int n_maps;
  const void* x;
  void* y;
  const int* lens;
  unsigned* sync;       // [0] arrival count, [1] generation used by this launch
  unsigned* sync_next;  // the pair the next launch will use; cleared by this launch
  int* status;        // [0] code, [1] where, [2] cta
  unsigned long long timeout_ns;
  int max_slots;      // experiment knob: cap on operand ring slots, 0 = as many as fit
  int skip_arrival;   // test hook: CTA (skip_arrival-1) leaves at barrier 0 without arriving; 0 = off
  long long* prof;    // optional [n_stages][grid][8]: clock64 at stage start, work done, barrier left, then GEMM
                      // role cycles: MMA waiting for operands, MMA waiting for a free accumulator, producer
                      // waiting for a free slot, epilogue waiting for an accumulator, epilogue busy
};

// Everything a launch needs, passed in parameter space: per-call tensor maps (negative map
// indices: -1 -> call_maps[0], -2 -> call_maps[1], ...), up to two inline stages for the
// plan-less entry points, and the pointers above.
constexpr int kCallMaps = 4;
struct CallArgs {
  CUtensorMap call_maps[kCallMaps];
  Stage inline_stages[3];
  MegaParams p;
};
__device__ __forceinline__ const CUtensorMap* map_ptr(const CallArgs& a, int idx) {
  return idx < 0 ? &a.call_maps[-idx - 1] : a.p.maps + idx;
}

struct __align__(8) SmemCtl {
  uint64_t full[kMaxSlots];
  uint64_t empty[kMaxSlots];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t qk_full, qk_empty, v_full, v_empty, s_full, p_full, o_full;   // attention, pipeline 0
  uint64_t attn1[7];                                                     // attention, pipeline 1 (same order)
  uint64_t o_empty[2];                                                   // pair attention: output accumulator read out
  uint64_t ln_full[4], ln_empty[4];
  uint64_t rec_full;                // the next stage's record has landed (bulk copy issued inside the grid barrier)
  uint32_t tmem_base;
  int abort;
  unsigned long long deadline_ns;   // read from the global timer once per CTA
  alignas(16) Stage stage;   // current stage; plan-owned programs fetch the next record while the CTA waits at the barrier
};
static_assert(sizeof(SmemCtl) <= kCtlBytes, "control block too large");

// Per-thread view of the pipelines; identical arithmetic in every role keeps them in step.
struct RoleState {
  uint32_t slot = 0;       // next ring slot
  uint32_t slot_bits = 0;  // phase bit per ring slot
  uint32_t acc = 0;        // next accumulator buffer
  uint32_t acc_bits = 0;   // phase bit per accumulator buffer
  uint32_t attn_bit = 0;   // phase bit of the attention barriers, pipeline 0
  uint32_t attn_bit1 = 0;  // phase bit of the attention barriers, pipeline 1
  uint32_t ln_bits = 0;    // phase bit per LayerNorm batch buffer
  uint32_t o_bits = 0;     // pair attention: phase bit of the o_empty barrier of each pipeline (MMA lane)
};

// SM clock for the stage-level stamps of the in-kernel profile.  The memory clobber keeps the read where it is
// written: a plain clock64() may be scheduled above a preceding barrier, which charges a stage's work to the wait
// that follows it.
__device__ __forceinline__ long long clock_now() {
  long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t) :: "memory");
  return t;
}

__device__ __forceinline__ const void* sel_ptr(int sel, const void* plan, const MegaParams& p) {
  return sel == PTR_CALL_X ? p.x : (sel == PTR_CALL_Y ? (const void*)p.y : plan);
}

// ------------------------------------------------------------------------------------
// grid barrier: one monotonic arrival counter per launch, bounded spin
// ------------------------------------------------------------------------------------
__device__ bool grid_barrier(const MegaParams& p, const WaitCtl& ctl, int where, SmemCtl& cs) {
  // The CTA barrier orders every thread's global writes before thread 0, whose gpu-scope release is
  // cumulative and publishes them to the other CTAs.  On the way out thread 0's acquire, the second CTA
  // barrier and a proxy fence order the other CTAs' writes before this CTA's TMA and bulk-copy reads.
  __syncthreads();
  if (threadIdx.x == 0) {
    if (p.prof) p.prof[((size_t)where * gridDim.x + blockIdx.x) * kProfSlots + 1] = clock_now();
    // The counter only grows during a launch: barrier number `where` is passed once every CTA
    // has added 1 for it.  (The launch that runs next clears the other counter, see the prologue.)
    unsigned* count = p.sync;
    const unsigned target = (unsigned)(where + 1) * gridDim.x;
    const bool skip = p.skip_arrival > 0 && where == 0 && (int)blockIdx.x == p.skip_arrival - 1;
    if (skip) *ctl.abort_smem = 1; else red_add_release_u32(count, 1u);
    // Nobody reads the current stage record any more (the CTA barrier above): the next one is fetched by a bulk
    // copy while this thread waits for the other CTAs, so its round trip to L2 costs the stage nothing.
    const bool fetch = p.stages != nullptr;
    if (fetch) {
      // first this CTA's slice of the weights of the GEMM stage after next -> L2 (they come from HBM when the program's
      // weights exceed L2; without this every GEMM stage starts with all CTAs waiting on the same DRAM rows)
      const uint32_t pf_bytes = cs.stage.pf_bytes;
      if (pf_bytes) {
        const uint32_t per = ((pf_bytes + gridDim.x - 1) / gridDim.x + 15u) & ~15u, off = blockIdx.x * per;
        if (off < pf_bytes)
          bulk_prefetch_l2(reinterpret_cast<const char*>(cs.stage.pf_ptr) + off, off + per <= pf_bytes ? per : pf_bytes - off);
      }
      mbar_expect_tx(smem_u32(&cs.rec_full), (uint32_t)sizeof(Stage));
      bulk_load(smem_u32(&cs.stage), p.stages + where + 1, (uint32_t)sizeof(Stage), smem_u32(&cs.rec_full));
    }
    uint32_t spins = 0;
    while (!skip && ld_acquire_u32(count) < target) {
      if (((++spins) & 0x3F) == 0) {
        if (*ctl.abort_smem) break;
        if (globaltimer_ns() > ctl.deadline_ns) {
          record_timeout(ctl, DEV_TIMEOUT_GRID, where);
          break;
        }
      }
    }
    if (fetch) mbar_wait(smem_u32(&cs.rec_full), (uint32_t)where & 1u, ctl, 50);
  }
  __syncthreads();
  fence_proxy_async_global();     // the other CTAs' global writes (acquired above) before this CTA's TMA and bulk-copy reads
  fence_proxy_async_smem();       // this thread's accesses to shared memory before the next stage's copies into it
  return *ctl.abort_smem == 0;
}

// ------------------------------------------------------------------------------------
// GEMM stage
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint32_t d, uint32_t mg) {
  return d == 1u ? n : __umulhi(n, mg);
}

struct GemmGeom {
  int tiles_n, splitk, items, kchunks, bn, bm, nh, slot_bytes, nslots;
};
__device__ __forceinline__ GemmGeom gemm_geom(const Stage& st) {
  GemmGeom g;
  g.bn = st.bn;
  g.bm = st.bm;
  g.nh = st.bm >> 7;                       // 128-row halves per tile, each with its own accumulator
  g.tiles_n = st.tiles_n;
  g.splitk = st.splitk;
  g.items = st.items;
  g.kchunks = st.kchunks;
  g.slot_bytes = st.slot_bytes;
  g.nslots = st.nslots;
  return g;
}
// work item -> (m tile, n tile, k split)
__device__ __forceinline__ void gemm_item(const Stage& st, int item, int& mt, int& nt, int& ks) {
  const uint32_t q = fast_div((uint32_t)item, (uint32_t)st.splitk, st.mg_splitk);
  ks = item - (int)q * st.splitk;
  const uint32_t m = fast_div(q, (uint32_t)st.tiles_n, st.mg_tiles_n);
  nt = (int)q - (int)m * st.tiles_n;
  mt = (int)m;
}

// Epilogue parameters of a stage, copied into registers once (the stage record itself lives in
// shared memory and would otherwise be re-read around every asm statement).
struct EpiCtx {
  int epi, act, M, N, ldo;
  const float* bias_s;     // bias staged in shared memory as fp32 (converted once per stage), or null
  const __half* resid;
  __half* out;
  float* partial;
  const CUtensorMap* tm_out;   // store map of the fp32 planes, or null: plain stores
  bool prof;
};
constexpr uint32_t kNoRow = 0xFFFFFFFFu;      // "this row is outside the matrix"

// A thread that owns one row of a 32-row block holds 64 bytes of that row.  Written straight to global
// memory, one store instruction would touch 32 different lines with 16 bytes each.  Going through the
// warp's staging buffer turns that around: afterwards lanes 4j..4j+3 hold the 64 bytes of row j (+8, +16,
// +24), so every store instruction writes eight rows with 64 contiguous bytes each.
// `rowptr[i]` is the global byte address of row (8*i + lane/4) at this chunk's first column, or null.
__device__ __forceinline__ void staged_store_64B(uint8_t* sbuf, const uint32_t (&w)[16], uint8_t* const (&rowptr)[4], int lane) {
  // Piece i (16 bytes) of row r sits at r * 64 + ((i ^ (r >> 1)) & 3) * 16: the eight lanes of a quarter warp then hit
  // distinct banks both when every lane writes piece i of its own row and when four lanes read one row each of two
  // neighbouring rows (padded rows avoided the conflicts of the writes only: two thirds of the reads were replays).
  const int sw_w = (lane >> 1) & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(sbuf + lane * kStageRow + ((i ^ sw_w) << 4)) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
  __syncwarp();
  uint4 v[4];                    // all four loads are issued before the first store waits for its data
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 8 * i + (lane >> 2);
    v[i] = *reinterpret_cast<const uint4*>(sbuf + r * kStageRow + ((((lane & 3) ^ (r >> 1)) & 3) << 4));
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (rowptr[i]) *reinterpret_cast<uint4*>(rowptr[i] + (lane & 3) * 16) = v[i];
  __syncwarp();
}

// Swin row maps.  Tokens of an R x R grid are rolled by -shift and cut into (R/win)^2 windows of win*win
// tokens; the window-major buffers give every window 64 row slots (49 used for win = 7).
// token row (b*R*R + ty*R + tx)  ->  window-major row (global window)*64 + position
__device__ __forceinline__ int swin_token_to_slot(int row, int R, int win, int shift) {
  const int img = row / (R * R), t = row - img * R * R;
  const int ty = t / R, tx = t - ty * R;
  int sy = ty - shift, sx = tx - shift;
  if (sy < 0) sy += R;
  if (sx < 0) sx += R;
  const int nwr = R / win;
  const int w = (sy / win) * nwr + sx / win, pos = (sy % win) * win + sx % win;
  return (img * nwr * nwr + w) * 64 + pos;
}
// window-major row -> token row, or -1 for a padding slot
__device__ __forceinline__ int swin_slot_to_token(int slot, int R, int win, int shift, int n_windows) {
  const int wg = slot >> 6, pos = slot & 63;
  if (pos >= win * win || wg >= n_windows) return -1;
  const int nwr = R / win, img = wg / (nwr * nwr), w = wg - img * nwr * nwr;
  int ty = (w / nwr) * win + pos / win + shift, tx = (w % nwr) * win + pos % win + shift;
  if (ty >= R) ty -= R;
  if (tx >= R) tx -= R;
  return img * R * R + ty * R + tx;
}

// Output addressing is split into a row part, computed once per tile, and a column part, computed once
// per chunk; both are element offsets that fit 32 bits (the host rejects larger buffers).
// Row part: offset of matrix row `row` in the stage's output (kNoRow past the end).  The residual, where a
// stage has one, is laid out like the output, so the same offset addresses it.
template <bool kSwin>
__device__ __forceinline__ uint32_t epi_row_offset(const Stage& st, const EpiCtx& e, int row, int ks) {
  if (row >= e.M) return kNoRow;
  if (e.epi == EPI_PARTIAL) return (uint32_t)(ks * e.M + row) * (uint32_t)e.N;
  if (e.epi == EPI_QKV) {
    // [3][B][heads][S][d]: row -> (sequence, token)
    const uint32_t b = fast_div((uint32_t)row, (uint32_t)st.seq, st.mg_seq), sq = (uint32_t)row - b * (uint32_t)st.seq;
    return (b * (uint32_t)(st.heads * st.seq) + sq) * (uint32_t)st.head_dim;
  }
  if constexpr (kSwin) {
    if (e.epi == EPI_SWIN_QKV) return (uint32_t)swin_token_to_slot(row, st.seq, st.win, st.shift) * (uint32_t)e.ldo;
    if (e.epi == EPI_SWIN_PROJ) {
      const int t = swin_slot_to_token(row, st.seq, st.win, st.shift, e.M >> 6);
      return t >= 0 ? (uint32_t)t * (uint32_t)e.ldo : kNoRow;
    }
  }
  return (uint32_t)row * (uint32_t)e.ldo;
}
// Column part: offset of column `col` (a multiple of 16; a chunk never straddles a head or a q/k/v plane).
template <bool kSwin>
__device__ __forceinline__ uint32_t epi_col_offset(const Stage& st, const EpiCtx& e, int col) {
  if (e.epi == EPI_QKV) {
    const uint32_t g = fast_div((uint32_t)col, (uint32_t)st.head_dim, st.mg_head_dim), dd = (uint32_t)col - g * (uint32_t)st.head_dim;
    const uint32_t which = fast_div(g, (uint32_t)st.heads, st.mg_heads), hh = g - which * (uint32_t)st.heads;
    const uint32_t head_plane = (uint32_t)(st.seq * st.head_dim);
    return (which * (uint32_t)(st.batch * st.heads) + hh) * head_plane + dd;
  }
  if constexpr (kSwin) {
    if (e.epi == EPI_SWIN_QKV) {
      // [3][windows][64][C]: the column picks q/k/v and the channel
      const int which = col / e.ldo, ch = col - which * e.ldo;
      const uint32_t plane = (uint32_t)((e.M + st.seq * st.seq - 1) / (st.seq * st.seq)) * (uint32_t)((st.seq / st.win) * (st.seq / st.win) * 64) * (uint32_t)e.ldo;
      return (uint32_t)which * plane + (uint32_t)ch;
    }
  }
  return (uint32_t)col;
}

// One 32-column chunk of the accumulator block: r[i] = column col+i of this thread's own row, whose output
// offset is `own`; `so[i]` = output offset of row (8*i + lane/4) of the same 32-row block (staged stores).
template <bool kSwin>
__device__ __forceinline__ void epilogue_chunk32(const Stage& st, const EpiCtx& e, uint8_t* sbuf, const uint32_t (&r)[32],
                                                 uint32_t own, const uint32_t (&so)[4], int col, int lane, unsigned& t_mid,
                                                 uint32_t tma_row, int tma_plane, int& box, int nbox) {
  if (e.epi == EPI_PARTIAL) {
    // fp32 planes: two halves of 16 columns = 64 bytes per row each.  (Storing each thread's own 128-byte
    // row segment directly measured twice as slow: an instruction's cost grows with the lines it touches.)
    if (e.prof) t_mid = (unsigned)clock64();
    if (e.tm_out) {
      // Through the TMA: the thread writes its row's 64 bytes into a staging box (the layout of a 64B-swizzled box of
      // 16 columns x 32 rows) and one lane hands the box to the copy engine.  A warp has `nbox` boxes, used round
      // robin: two beside the operand ring while the main loop runs, twelve inside the ring for the CTA's last tile
      // (whose operands have all been consumed) -- a box is rewritten once the copy issued from it has read it.
      const int sw_w = (lane >> 1) & 3;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint8_t* buf = sbuf + box * kStageWarp;
        if (lane == 0) {
          if (nbox == 2) bulk_wait_group_read<1>(); else bulk_wait_group_read<11>();
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(buf + lane * kStageRow + ((i ^ sw_w) << 4)) =
              make_uint4(r[16 * half + 4 * i], r[16 * half + 4 * i + 1], r[16 * half + 4 * i + 2], r[16 * half + 4 * i + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && tma_row != kNoRow) {
          tma_store_3d(e.tm_out, smem_u32(buf), col + 16 * half, (int)tma_row, tma_plane);
          bulk_commit_group();
        }
        box = box + 1 == nbox ? 0 : box + 1;
      }
      return;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint8_t* rowptr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        rowptr[i] = so[i] != kNoRow ? reinterpret_cast<uint8_t*>(e.partial + (so[i] + (uint32_t)(col + 16 * half))) : nullptr;
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) w[i] = r[16 * half + i];
      staged_store_64B(sbuf, w, rowptr, lane);
    }
    return;
  }
  // The arithmetic below is written phase by phase over the whole chunk -- every loop is 16 or 32 independent
  // operations -- instead of element by element: an epilogue warp has at most one other warp on its scheduler, so
  // a dependent chain per element (conversion, add, pack, seven GELU steps) runs at one instruction per ALU latency.
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  if (e.bias_s) {               // fp32 in shared memory: no conversions here (they run on the narrow XU pipe)
    const float4* b4 = reinterpret_cast<const float4*>(e.bias_s + col);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 b = b4[i];
      v[4 * i] += b.x; v[4 * i + 1] += b.y; v[4 * i + 2] += b.z; v[4 * i + 3] += b.w;
    }
  }
  const bool gelu_packed = e.act == ACT_GELU && e.resid == nullptr;   // GELU on fp16 pairs after packing (below)
  if (e.act == ACT_RELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.0f);
  } else if (e.act == ACT_GELU && !gelu_packed) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
  }
  if (e.resid && own != kNoRow) {
    const uint4* r4 = reinterpret_cast<const uint4*>(e.resid + own + col);
    float2 fr[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 u = r4[i];
      const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) fr[4 * i + j] = __half22float2(h[j]);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      v[2 * i] += fr[i].x;
      v[2 * i + 1] += fr[i].y;
    }
  }
  const uint32_t coff = epi_col_offset<kSwin>(st, e, col);
  uint8_t* rowptr[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) rowptr[i] = so[i] != kNoRow ? reinterpret_cast<uint8_t*>(e.out + (so[i] + coff)) : nullptr;
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = pack_h2(v[2 * i], v[2 * i + 1]);
  if (gelu_packed) gelu_tanh_h2x16(w);
  if (e.prof) t_mid = (unsigned)clock64();
  staged_store_64B(sbuf, w, rowptr, lane);
}

// 16-column tail chunk (tile widths that are an odd multiple of 16): direct stores.
template <bool kSwin>
__device__ __forceinline__ void epilogue_chunk16(const Stage& st, const EpiCtx& e, const uint32_t (&r)[16], uint32_t own, int col) {
  if (own == kNoRow) return;
  if (e.epi == EPI_PARTIAL) {
    float4* dst = reinterpret_cast<float4*>(e.partial + own + col);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      dst[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                           __uint_as_float(r[4 * i + 3]));
    return;
  }
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
  if (e.bias_s) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] += e.bias_s[col + i];
  }
  if (e.act == ACT_RELU) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.0f);
  } else if (e.act == ACT_GELU) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = gelu_tanh(v[i]);
  }
  if (e.resid) {
    const uint4* r4 = reinterpret_cast<const uint4*>(e.resid + own + col);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 u = r4[i];
      const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        v[8 * i + 2 * j] += f.x;
        v[8 * i + 2 * j + 1] += f.y;
      }
    }
  }
  uint4* d4 = reinterpret_cast<uint4*>(e.out + (own + epi_col_offset<kSwin>(st, e, col)));
  d4[0] = make_uint4(pack_h2(v[0], v[1]), pack_h2(v[2], v[3]), pack_h2(v[4], v[5]), pack_h2(v[6], v[7]));
  d4[1] = make_uint4(pack_h2(v[8], v[9]), pack_h2(v[10], v[11]), pack_h2(v[12], v[13]), pack_h2(v[14], v[15]));
}

// Tiles are bm x bn with bm = 128 (two accumulators used alternately, so the epilogue of one tile
// overlaps the main loop of the next) or bm = 256 (two 128-row halves share every B tile, which
// halves the B traffic per FLOP; each half has its own accumulator and hand-shake).
// kPair: the two CTAs of a cluster work on one 256 x bn tile with pair MMAs (see sm100_ptx.cuh).  CTA r loads rows
// 128 r .. 128 r + 127 of the A tile and rows bn/2 * r .. of the B tile (the weights' output columns) into its own
// shared memory -- half the B traffic per FLOP of the single-CTA form -- with every copy's completion counted on the
// leader's full barrier; the leader's MMA lane issues for both and its commits arrive on the barriers of both CTAs;
// each CTA's epilogue warps drain their own 128 rows and report to the leader's accumulator-free barrier.
template <bool kSwin, bool kPair = false>
__device__ __forceinline__ void gemm_stage(const Stage& st, const CallArgs& ca, SmemCtl& ctl_s, uint32_t ring, __half* vec_s,
                           uint8_t* stage_s, RoleState& rs, const WaitCtl& ctl, int warp, int lane) {
  const MegaParams& p = ca.p;
  GemmGeom g = gemm_geom(st);
  if constexpr (kPair) g.nh = 1;                                       // per CTA: one 128-row half of the pair's tile
  if (rs.slot >= (uint32_t)g.nslots) rs.slot = 0;
  const uint32_t full0 = smem_u32(&ctl_s.full[0]), empty0 = smem_u32(&ctl_s.empty[0]);
  const uint32_t tfull0 = smem_u32(&ctl_s.tmem_full[0]), tempty0 = smem_u32(&ctl_s.tmem_empty[0]);
  const uint32_t a_bytes = (uint32_t)(g.nh * kATileBytes);
  const uint32_t rank = kPair ? cluster_cta_rank() : 0u;               // 0 = the pair's leader
  const int first_item = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int item_step = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // the stage's bias vector -> shared memory (one global read per CTA instead of one per tile chunk)
  // (done by the epilogue warps alone; the producer and MMA warps start the main loop meanwhile)
  const float* bias_s = nullptr;
  if (warp >= 2 && warp < 2 + kEpiWarps && st.bias && st.epi != EPI_PARTIAL && st.N * 4 <= kVecBytes) {
    const uint4* src = reinterpret_cast<const uint4*>(st.bias);
    float4* dst = reinterpret_cast<float4*>(vec_s);
    for (int i = threadIdx.x - 64; i < st.N / 8; i += kEpiThreads) {
      const uint4 u = __ldg(src + i);
      const __half2* h = reinterpret_cast<const __half2*>(&u);
      const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
      dst[2 * i] = make_float4(f0.x, f0.y, f1.x, f1.y);
      dst[2 * i + 1] = make_float4(f2.x, f2.y, f3.x, f3.y);
    }
    bias_s = reinterpret_cast<const float*>(vec_s);
    named_barrier_sync(1, kEpiThreads);
  }

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const CUtensorMap* tmA = map_ptr(ca, st.tm_a);
      const CUtensorMap* tmB = map_ptr(ca, st.tm_b);
      bool ok = true;
      long long t_wait = 0, t_first = 0;
      const bool prof = p.prof != nullptr;
      uint32_t s = rs.slot, bits = rs.slot_bits;
      for (int item = first_item; ok && item < g.items; item += item_step) {
        int mt, nt, ks;
        gemm_item(st, item, mt, nt, ks);
        const int m0 = mt * g.bm + (int)rank * 128, n0 = nt * g.bn + (int)rank * (g.bn >> 1), kbase = ks * g.kchunks;
        // CTAs start at different K chunks so they do not all pull the same A tile at once
        const uint32_t rot = (uint32_t)first_item + (uint32_t)item;
        int kk = (int)(rot - fast_div(rot, (uint32_t)g.kchunks, st.mg_kchunks) * (uint32_t)g.kchunks);
        for (int kc = 0; kc < g.kchunks; ++kc) {
          const long long tw = prof ? clock64() : 0;
          if (!mbar_wait(empty0 + 8 * s, ((bits >> s) & 1u) ^ 1u, ctl, 100 + (int)s)) { ok = false; break; }
          if (prof) t_wait += clock64() - tw;
          const uint32_t fb = full0 + 8 * s;
          const uint32_t a_dst = ring + s * g.slot_bytes, b_dst = a_dst + a_bytes;
          const int k0 = (kbase + kk) * 64;
          if (prof && !t_first) t_first = clock64();
          if constexpr (kPair) {
            // both CTAs' bytes are counted on the leader's barrier, which only the leader arms
            if (rank == 0) mbar_expect_tx(fb, 2u * (uint32_t)g.slot_bytes);
            const uint32_t fbl = map_shared_rank(fb, 0);
            tma_load_2d_pair(a_dst, tmA, fbl, k0, m0);          // box rows = 128: this CTA's half of the rows
            tma_load_2d_pair(b_dst, tmB, fbl, k0, n0);          // box rows = bn / 2: this CTA's half of the columns
          } else {
            mbar_expect_tx(fb, (uint32_t)g.slot_bytes);
            tma_load_2d(a_dst, tmA, fb, k0, m0);                // box rows = bm: both halves in one copy
            if (!st.b_mn_major) {
              tma_load_2d(b_dst, tmB, fb, k0, n0);
            } else {
              for (int j = 0; j < g.bn / 64; ++j) tma_load_2d(b_dst + j * 8192, tmB, fb, n0 + j * 64, k0);
            }
          }
          bits ^= 1u << s;
          s = (s + 1 == (uint32_t)g.nslots) ? 0 : s + 1;
          kk = (kk + 1 == g.kchunks) ? 0 : kk + 1;
        }
      }
      rs.slot = s;
      rs.slot_bits = bits;
      if (p.prof) {
        long long* pr = p.prof + ((size_t)st.prof_index * gridDim.x + blockIdx.x) * kProfSlots;
        pr[5] = t_wait;
        pr[11] = t_first;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (of a pair: the leader's) ----------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = kPair ? umma_idesc_f16_pair((uint32_t)g.bn, (uint32_t)st.b_mn_major)
                                   : umma_idesc_f16((uint32_t)g.bn, (uint32_t)st.b_mn_major);
      const uint32_t tmem = ctl_s.tmem_base;
      // descriptor low words of slot 0; a slot further on adds slot_bytes/16 to both
      const uint32_t a_lo0 = umma_desc_lo(ring, 16);
      const uint32_t b_lo0 = umma_desc_lo(ring + a_bytes, st.b_mn_major ? 8192u : 16u);
      const uint32_t slot16 = (uint32_t)g.slot_bytes >> 4;
      const uint32_t bstep = st.b_mn_major ? 128u : 2u;       // 16 K-rows = 2048 B, or 16 halves = 32 B
      const bool prof = p.prof != nullptr;
      bool ok = true;
      long long t_full = 0, t_acc = 0, t_first = 0, t_last = 0;
      for (int item = first_item; ok && item < g.items; item += item_step) {
        const uint32_t acc0 = g.nh == 2 ? 0u : rs.acc;       // accumulator of half 0; half 1 uses buffer 1
        const uint32_t d0 = tmem + acc0 * kAccStride, d1 = d0 + kAccStride;
        {                                                      // the epilogue must have drained the buffers
          const long long ta = prof ? clock64() : 0;
          for (int h = 0; h < g.nh; ++h) {
            const uint32_t acc = acc0 + (uint32_t)h;
            if (!mbar_wait(tempty0 + 8 * acc, ((rs.acc_bits >> acc) & 1u) ^ 1u, ctl, 200 + (int)acc)) { ok = false; break; }
          }
          tc_fence_after_sync();
          if (prof) t_acc += clock64() - ta;
        }
        for (int kc = 0; ok && kc < g.kchunks; ++kc) {
          const uint32_t s = rs.slot;
          const long long tw = prof ? clock64() : 0;
          if (!mbar_wait(full0 + 8 * s, (rs.slot_bits >> s) & 1u, ctl, 300 + (int)s)) { ok = false; break; }
          if (prof) {
            const long long tn = clock64();
            t_full += tn - tw;
            if (!t_first) t_first = tn;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + s * slot16, b_lo = b_lo0 + s * slot16;
          if constexpr (kPair) {
            umma_f16_k64_pair(d0, a_lo, b_lo, bstep, idesc, (uint32_t)(kc != 0));
            umma_commit_pair(empty0 + 8 * s);
          } else {
            if (g.nh == 2) umma_f16_k64_x2(d0, d1, a_lo, b_lo, bstep, idesc, (uint32_t)(kc != 0));
            else umma_f16_k64(d0, a_lo, b_lo, bstep, idesc, (uint32_t)(kc != 0));
            umma_commit(empty0 + 8 * s);
          }
          rs.slot_bits ^= 1u << s;
          rs.slot = (s + 1 == (uint32_t)g.nslots) ? 0 : s + 1;
        }
        if (!ok) break;
        for (int h = 0; h < g.nh; ++h) {
          const uint32_t acc = acc0 + (uint32_t)h;
          if constexpr (kPair) umma_commit_pair(tfull0 + 8 * acc);
          else umma_commit(tfull0 + 8 * acc);
          rs.acc_bits ^= 1u << acc;
        }
        if (prof) t_last = clock64();
        if (g.nh == 1) rs.acc ^= 1u;
      }
      if (p.prof) {
        long long* pr = p.prof + ((size_t)st.prof_index * gridDim.x + blockIdx.x) * kProfSlots;
        pr[3] = t_full;
        pr[4] = t_acc;
        pr[12] = t_first;
        pr[13] = t_last;
      }
    }
    __syncwarp();
  } else if (warp < 2 + kEpiWarps) {
    // ---------------- epilogue: TMEM -> registers -> global (8 warps: lane quarter x column parity) --
    const int q = warp & 3, cpar = (warp - 2) >> 2;
    const uint32_t tmem = ctl_s.tmem_base + ((uint32_t)(q * 32) << 16);
    const int full_chunks = g.bn >> 5;
    EpiCtx e;
    e.epi = st.epi; e.act = st.act; e.M = st.M; e.N = st.N; e.ldo = st.ldo;
    e.bias_s = bias_s;
    e.resid = reinterpret_cast<const __half*>(sel_ptr(st.resid_sel, st.resid, p));
    e.out = reinterpret_cast<__half*>(const_cast<void*>(sel_ptr(st.out_sel, st.out, p)));
    e.partial = st.partial;
    e.tm_out = (st.epi == EPI_PARTIAL && st.out_tma) ? map_ptr(ca, st.tm_out) : nullptr;
    const bool prof = p.prof != nullptr;
    e.prof = prof;
    // a warp's staging: 2 KB of the staging area, or -- for the boxes of TMA stores, which want two buffers -- 4 KB of
    // the vector area and the staging area taken together (a stage that writes planes stages no bias)
    uint8_t* sbuf = e.tm_out ? reinterpret_cast<uint8_t*>(vec_s) + (warp - 2) * 2 * kStageWarp : stage_s + (warp - 2) * kStageWarp;
    unsigned t_wait = 0, t_busy = 0, t_tmem = 0, t_math = 0, t_store = 0;   // cycle totals (32 bits are plenty)
    long long t_first = 0;
    int box = 0;
    for (int item = first_item; item < g.items; item += item_step) {
      int mt, nt, ks;
      gemm_item(st, item, mt, nt, ks);
      const uint32_t acc0 = g.nh == 2 ? 0u : rs.acc;
      bool ok = true;
      // TMA-store boxes of the CTA's last tile live in the operand ring: once its accumulator is complete every operand
      // tile of the stage has been consumed, and nothing is loaded before the next stage
      const bool last_tile = e.tm_out != nullptr && item + item_step >= g.items;
      uint8_t* tile_sbuf = last_tile ? stage_s - kVecBytes - kRingBytes + (warp - 2) * 12 * kStageWarp : sbuf;
      const int nbox = last_tile ? 12 : 2;
      if (last_tile) box = 0;
      for (int h = 0; h < g.nh; ++h) {
        const uint32_t acc = acc0 + (uint32_t)h;
        const unsigned tw = prof ? (unsigned)clock64() : 0u;
        ok = mbar_wait_warp(tfull0 + 8 * acc, (rs.acc_bits >> acc) & 1u, ctl, 400 + (int)acc, lane);
        if (!ok) break;
        unsigned tb = 0;
        if (prof) {
          const long long now = clock64();
          tb = (unsigned)now;
          t_wait += tb - tw;
          if (!t_first) t_first = now;
        }
        tc_fence_after_sync();
        const int row0 = mt * g.bm + (kPair ? (int)rank : h) * 128 + q * 32;
        const uint32_t own = epi_row_offset<kSwin>(st, e, row0 + lane, ks);
        uint32_t so[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) so[i] = epi_row_offset<kSwin>(st, e, row0 + 8 * i + (lane >> 2), ks);
        const uint32_t t0 = tmem + acc * kAccStride;
        const int colbase = nt * g.bn;
        // this warp takes chunks cpar, cpar+2, ... (its partner warp on the same lane quarter the others)
        for (int c = cpar; c < full_chunks; c += 2) {
          uint32_t r[32];
          const unsigned tl = prof ? (unsigned)clock64() : 0u;
          tmem_ld32(t0 + c * 32, r);
          tmem_ld_wait(r);
          unsigned tm = 0, tmid = 0;
          if (prof) {
            tm = (unsigned)clock64();
            t_tmem += tm - tl;
          }
          epilogue_chunk32<kSwin>(st, e, tile_sbuf, r, own, so, colbase + c * 32, lane, tmid,
                                  row0 < e.M ? (uint32_t)row0 : kNoRow, ks, box, nbox);
          if (prof) {
            t_math += tmid - tm;
            t_store += (unsigned)clock64() - tmid;
          }
        }
        if ((g.bn & 16) && (full_chunks & 1) == cpar) {
          uint32_t r[16];
          tmem_ld16(t0 + full_chunks * 32, r);
          tmem_ld_wait(r);
          epilogue_chunk16<kSwin>(st, e, r, own, colbase + full_chunks * 32);
        }
        tc_fence_before_sync();
        if constexpr (kPair) {                      // one arrival per warp on the leader's barrier (16 in all)
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(map_shared_rank(tempty0 + 8 * acc, 0));
        } else {
          mbar_arrive(tempty0 + 8 * acc);
        }
        rs.acc_bits ^= 1u << acc;
        if (prof) t_busy += (unsigned)clock64() - tb;
      }
      if (!ok) break;
      if (g.nh == 1) rs.acc ^= 1u;
    }
    if (e.tm_out && lane == 0) {          // the planes are complete before the CTA reports the stage done
      bulk_wait_group_all();
      fence_proxy_async_global();
    }
    __syncwarp();
    if (p.prof && warp == 2 && lane == 0) {
      long long* pr = p.prof + ((size_t)st.prof_index * gridDim.x + blockIdx.x) * kProfSlots;
      pr[6] = t_wait;
      pr[7] = t_busy;
      pr[8] = t_tmem;
      pr[9] = t_math;
      pr[10] = t_store;
      pr[14] = t_first;
      pr[15] = clock64();
    }
  }
}

// Parity output of the attention stages: normalised probabilities of one query row per thread, recomputed from the
// scores in TMEM.  Out of line: only the parity configurations call them, and inlined their registers would be charged
// to every attention item.
// Tile form (the cooperative attention stage): the unnormalised probabilities already sit in shared memory as the
// fp16 A-operand tiles of P.V ([128 rows][64 keys] per tile, 128-byte rows with the 16-byte pieces XOR-swizzled by
// row & 7); the 256 softmax threads copy them out scaled by 1 / rowsum: eight threads per row, 32 rows per pass, so a
// store instruction writes four rows of 128 contiguous bytes.  `sums` = the two groups' partial row sums [2][128].
__device__ __noinline__ void attn_copy_probs_tiles(const uint8_t* ptiles, const float* sums, __half* mat, int S, int rows, int t8) {
  const int sub = t8 & 7, rsub = t8 >> 3;
  for (int r = rsub; r < rows; r += 32) {
    const float inv = 1.0f / (sums[r] + sums[128 + r]);
    const uint8_t* src = ptiles + r * 128 + ((sub ^ (r & 7)) << 4);
    __half* dst = mat + (size_t)r * S + sub * 8;
    for (int tile = 0; tile * 64 + sub * 8 + 8 <= S; ++tile) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + tile * kATileBytes);
      const uint32_t in[4] = {v.x, v.y, v.z, v.w};
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&in[i]));
        w[i] = pack_h2(f.x * inv, f.y * inv);
      }
      *reinterpret_cast<uint4*>(dst + tile * 64) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// Staged form (S <= 128, a warp owns rows row0 .. row0 + 31 of the [S][S] matrix at `mat`): whole 64-byte row pieces
// go through the warp's staging buffer, so that a store instruction writes eight rows of 64 contiguous bytes.
__device__ __noinline__ void attn_store_probs_staged(uint32_t ts, uint8_t* sbuf, __half* mat, int row0, int S, int kv_len,
                                                     float sl2, float mask_l2, float mx, float inv, int lane) {
  for (int c = 0; c * 32 < S; ++c) {
    uint32_t r[32];
    tmem_ld32(ts + c * 32, r);
    tmem_ld_wait(r);
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int key = c * 32 + 2 * i;
      const float ta = __uint_as_float(r[2 * i]) * sl2 + (key >= kv_len ? mask_l2 : 0.0f);
      const float tb = __uint_as_float(r[2 * i + 1]) * sl2 + (key + 1 >= kv_len ? mask_l2 : 0.0f);
      w[i] = pack_h2(ex2_fast(ta - mx) * inv, ex2_fast(tb - mx) * inv);
    }
    if (c * 32 + 32 <= S) {
      uint8_t* rowptr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rr = row0 + 8 * i + (lane >> 2);
        rowptr[i] = rr < S ? reinterpret_cast<uint8_t*>(mat + (size_t)rr * S + c * 32) : nullptr;
      }
      staged_store_64B(sbuf, w, rowptr, lane);
    } else if (row0 + lane < S) {                     // the last 16 keys of a row (S is a multiple of 16)
      uint4* dst = reinterpret_cast<uint4*>(mat + (size_t)(row0 + lane) * S + c * 32);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  }
}

// ------------------------------------------------------------------------------------
// attention stage: one work item = (sequence, head, 128-query tile); S <= 384, head_dim 64
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void attn_stage(const Stage& st, const CallArgs& ca, SmemCtl& ctl_s, uint32_t ring, uint8_t* ring_ptr,
                                           uint8_t* stage_s, RoleState& rs, const WaitCtl& ctl, int warp, int lane) {
  const MegaParams& p = ca.p;
  const int S = st.seq, B = st.batch, H = st.heads;
  const int n_kb = (S + 127) / 128;
  const int items = B * H * n_kb;
  const uint32_t q_off = 0, k_off = kATileBytes, v_off = k_off + n_kb * kATileBytes,
                 p_off = v_off + n_kb * kATileBytes;
  const uint32_t qk_full = smem_u32(&ctl_s.qk_full), qk_empty = smem_u32(&ctl_s.qk_empty);
  const uint32_t v_full = smem_u32(&ctl_s.v_full), v_empty = smem_u32(&ctl_s.v_empty);
  const uint32_t s_full = smem_u32(&ctl_s.s_full), p_full = smem_u32(&ctl_s.p_full),
                 o_full = smem_u32(&ctl_s.o_full);
  const CUtensorMap* tm = map_ptr(ca, st.tm_qkv);

  if (warp == 0) {
    if (lane == 0) {
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int qt = item % n_kb, h = (item / n_kb) % H, b = item / (n_kb * H);
        const int rq = ((0 * B + b) * H + h) * S, rk = ((1 * B + b) * H + h) * S, rv = ((2 * B + b) * H + h) * S;
        if (!mbar_wait(qk_empty, rs.attn_bit ^ 1u, ctl, 500)) break;
        mbar_expect_tx(qk_full, (uint32_t)(kATileBytes * (1 + n_kb)));
        tma_load_2d(ring + q_off, tm, qk_full, 0, rq + qt * 128);
        for (int kb = 0; kb < n_kb; ++kb) tma_load_2d(ring + k_off + kb * kATileBytes, tm, qk_full, 0, rk + kb * 128);
        if (!mbar_wait(v_empty, rs.attn_bit ^ 1u, ctl, 501)) break;
        mbar_expect_tx(v_full, (uint32_t)(kATileBytes * n_kb));
        for (int kb = 0; kb < n_kb; ++kb) tma_load_2d(ring + v_off + kb * kATileBytes, tm, v_full, 0, rv + kb * 128);
        rs.attn_bit ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_f16(128u, 0u);
      const uint32_t idesc_o = umma_idesc_f16(64u, 1u);
      const uint32_t tmem = ctl_s.tmem_base;
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        if (!mbar_wait(qk_full, rs.attn_bit, ctl, 510)) break;
        tc_fence_after_sync();
        const uint64_t qd = umma_desc_sw128(ring + q_off, 16, 1024);
        for (int kb = 0; kb < n_kb; ++kb) {
          const uint64_t kd = umma_desc_sw128(ring + k_off + kb * kATileBytes, 16, 1024);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) umma_f16(tmem + kb * 128, qd + 2u * k, kd + 2u * k, idesc_s, (uint32_t)(k != 0));
        }
        umma_commit(s_full);
        umma_commit(qk_empty);
        if (!mbar_wait(p_full, rs.attn_bit, ctl, 511)) break;
        if (!mbar_wait(v_full, rs.attn_bit, ctl, 512)) break;
        tc_fence_after_sync();
        for (int kk = 0; kk < n_kb * 8; ++kk) {
          const uint64_t pd = umma_desc_sw128(ring + p_off + (kk >> 2) * kATileBytes, 16, 1024) + 2u * (kk & 3);
          const uint64_t vd = umma_desc_sw128(ring + v_off + (kk >> 3) * kATileBytes, 8192, 1024) + 128u * (kk & 7);
          umma_f16(tmem + kOCol, pd, vd, idesc_o, (uint32_t)(kk != 0));
        }
        umma_commit(o_full);
        umma_commit(v_empty);
        rs.attn_bit ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp < 2 + kEpiWarps) {
    // Both groups of four warps work on the same item: group 0 takes the first half of the 16-key blocks, group 1
    // the second half (a thread of each group owns query row r_in); row maxima and row sums are exchanged through
    // shared memory around two 256-thread barriers.  The output columns are split 32 / 32 likewise.
    const int grp = (warp - 2) >> 2, q = warp & 3;
    const int r_in = q * 32 + lane;
    const uint32_t tmem = ctl_s.tmem_base + ((uint32_t)(q * 32) << 16);
    const float sl2 = st.scale * 1.4426950408889634f;
    const int* lens = st.lens_from_call ? p.lens : st.lens;
    __half* ctx = reinterpret_cast<__half*>(st.out);
    __half* probs = reinterpret_cast<__half*>(st.probs);
    const int hidden = H * st.head_dim;
    // At S = 384 the tiles of this stage (Q, 3 K, 3 V, 6 P = 208 KB) run past the 192 KB ring into the vector and
    // staging areas behind it, which no one else uses during attention; the exchange buffer sits at their very end.
    static_assert(13 * kATileBytes <= kRingBytes + kVecBytes + kStageBytes - 2048, "attention tiles overlap the exchange buffer");
    float* red = reinterpret_cast<float*>(stage_s + kStageBytes - 2048);   // [2 groups][128 rows] maxima, then [2][128] sums
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int qt = item % n_kb, h = (item / n_kb) % H, b = item / (n_kb * H);
      const int kv_len = lens ? lens[b] : S;
      bool ok = mbar_wait_warp(s_full, rs.attn_bit, ctl, 520, lane);
      if (!ok) break;
      tc_fence_after_sync();
      // Keys >= kv_len carry the additive -1e4 mask: probability 0 in fp32, never the maximum -> only the blocks
      // with valid keys are visited; the other P blocks are written as zeros.
      const int kvl = kv_len < 1 ? 1 : (kv_len > S ? S : kv_len);
      const int nb = (kvl + 15) >> 4, nb_all = n_kb * 8;
      const int nb_half = (nb + 1) >> 1;
      const int blk0 = grp ? nb_half : 0, blk1 = grp ? nb : nb_half;       // this group's valid blocks
      uint32_t ra[16], rb[16];
      // ---- pass 1: maximum of the raw scores of the valid keys (the scale is positive) ----
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
      auto max16 = [&](const uint32_t (&r)[16], int blk) {
        const int key0 = blk * 16;
        if (key0 + 16 <= kvl) {
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(r[i])); m1 = fmaxf(m1, __uint_as_float(r[i + 1]));
            m2 = fmaxf(m2, __uint_as_float(r[i + 2])); m3 = fmaxf(m3, __uint_as_float(r[i + 3]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) m0 = fmaxf(m0, key0 + i < kvl ? __uint_as_float(r[i]) : -INFINITY);
        }
      };
      if (blk0 < blk1) {
        tmem_ld16(tmem + blk0 * 16, ra);
        tmem_ld_wait(ra);
      }
      for (int blk = blk0; blk < blk1; blk += 2) {
        if (blk + 1 < blk1) tmem_ld16(tmem + (blk + 1) * 16, rb);
        max16(ra, blk);
        if (blk + 1 < blk1) {
          tmem_ld_wait(rb);
          if (blk + 2 < blk1) tmem_ld16(tmem + (blk + 2) * 16, ra);
          max16(rb, blk + 1);
          if (blk + 2 < blk1) tmem_ld_wait(ra);
        }
      }
      red[grp * 128 + r_in] = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      named_barrier_sync(3, 256);
      const float mx = fmaxf(red[r_in], red[128 + r_in]) * sl2;
      // ---- pass 2: unnormalised probabilities -> fp16 A-operand tiles (128B-swizzled rows, 64 keys per tile) ----
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      uint8_t* pbase = ring_ptr + p_off + r_in * 128;
      auto exp16 = [&](const uint32_t (&r)[16], int blk) {
        const int key0 = blk * 16;
        uint32_t w[8];
        if (key0 + 16 <= kvl) {
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            const float p0 = ex2_fast(fmaf(__uint_as_float(r[i]), sl2, -mx)), p1 = ex2_fast(fmaf(__uint_as_float(r[i + 1]), sl2, -mx));
            const float p2 = ex2_fast(fmaf(__uint_as_float(r[i + 2]), sl2, -mx)), p3 = ex2_fast(fmaf(__uint_as_float(r[i + 3]), sl2, -mx));
            s0 += p0; s1 += p1; s2 += p2; s3 += p3;
            w[i >> 1] = pack_h2(p0, p1);
            w[(i >> 1) + 1] = pack_h2(p2, p3);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float p0 = key0 + i < kvl ? ex2_fast(fmaf(__uint_as_float(r[i]), sl2, -mx)) : 0.f;
            const float p1 = key0 + i + 1 < kvl ? ex2_fast(fmaf(__uint_as_float(r[i + 1]), sl2, -mx)) : 0.f;
            s0 += p0; s1 += p1;
            w[i >> 1] = pack_h2(p0, p1);
          }
        }
        uint8_t* base = pbase + (blk >> 2) * kATileBytes;
        const int j = (blk & 3) * 2;
        *reinterpret_cast<uint4*>(base + ((j ^ (r_in & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(base + (((j + 1) ^ (r_in & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
      };
      if (blk0 < blk1) {
        tmem_ld16(tmem + blk0 * 16, ra);
        tmem_ld_wait(ra);
      }
      for (int blk = blk0; blk < blk1; blk += 2) {
        if (blk + 1 < blk1) tmem_ld16(tmem + (blk + 1) * 16, rb);
        exp16(ra, blk);
        if (blk + 1 < blk1) {
          tmem_ld_wait(rb);
          if (blk + 2 < blk1) tmem_ld16(tmem + (blk + 2) * 16, ra);
          exp16(rb, blk + 1);
          if (blk + 2 < blk1) tmem_ld_wait(ra);
        }
      }
      // keys past the valid ones: probability 0 (the two groups share the blocks alternately)
      for (int blk = nb + grp; blk < nb_all; blk += 2) {
        uint8_t* base = pbase + (blk >> 2) * kATileBytes;
        const int j = (blk & 3) * 2;
        *reinterpret_cast<uint4*>(base + ((j ^ (r_in & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(base + (((j + 1) ^ (r_in & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
      }
      red[256 + grp * 128 + r_in] = (s0 + s1) + (s2 + s3);
      fence_proxy_async_smem();                               // this thread's P rows -> visible to the MMA
      named_barrier_sync(3, 256);
      const float inv = 1.0f / (red[256 + r_in] + red[384 + r_in]);
      const int qrow = qt * 128 + r_in;
      tc_fence_before_sync();
      if (grp == 0) mbar_arrive(p_full);                      // 128 arrivals: group 1's rows are behind the barrier above
      if (probs) {
        // parity output: normalised probabilities [B*heads][S][S], copied from the P tiles while P.V runs; nobody may
        // start the next item's P rows or row sums before every thread has copied
        attn_copy_probs_tiles(ring_ptr + p_off, red + 256, probs + ((size_t)(b * H + h) * S + qt * 128) * S, S,
                              S - qt * 128 < 128 ? S - qt * 128 : 128, (int)threadIdx.x - 64);
        named_barrier_sync(3, 256);
      }
      ok = mbar_wait_warp(o_full, rs.attn_bit, ctl, 521, lane);
      if (!ok) break;
      tc_fence_after_sync();
      {
        uint32_t r0[32];
        tmem_ld32(tmem + kOCol + grp * 32, r0);               // this group's 32 of the 64 output columns
        tmem_ld_wait(r0);
        if (qrow < S) {
          uint4* dst = reinterpret_cast<uint4*>(ctx + ((size_t)b * S + qrow) * hidden + h * st.head_dim + grp * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[i] = make_uint4(pack_h2(__uint_as_float(r0[8 * i]) * inv, __uint_as_float(r0[8 * i + 1]) * inv),
                                pack_h2(__uint_as_float(r0[8 * i + 2]) * inv, __uint_as_float(r0[8 * i + 3]) * inv),
                                pack_h2(__uint_as_float(r0[8 * i + 4]) * inv, __uint_as_float(r0[8 * i + 5]) * inv),
                                pack_h2(__uint_as_float(r0[8 * i + 6]) * inv, __uint_as_float(r0[8 * i + 7]) * inv));
        }
      }
      tc_fence_before_sync();
      rs.attn_bit ^= 1u;
    }
  }
}

// ------------------------------------------------------------------------------------
// attention stage for S <= 128: two independent pipelines ("ping" and "pong").  The CTA's work items
// alternate between them; each pipeline has its own Q/K/V/P tiles in shared memory, its own score and
// output accumulators in TMEM, its own barriers and its own group of four softmax warps (warps 2..5
// and 6..9).  While one group runs the softmax of item i, the tensor core already holds the scores of
// item i+1 for the other group, and the loads of item i+2 are in flight.
// ------------------------------------------------------------------------------------
enum AttnBar : int { AB_QK_FULL = 0, AB_QK_EMPTY, AB_V_FULL, AB_V_EMPTY, AB_S_FULL, AB_P_FULL, AB_O_FULL };
constexpr int kPipeBytes = 5 * kATileBytes;      // Q 16 KiB, K 16, V 16, P 32
constexpr int kPipeOCol = 256;                   // TMEM: scores at 0 / 128, outputs at 256 / 320

template <bool kPair>
__device__ __forceinline__ void attn_stage_pp(const Stage& st, const CallArgs& ca, SmemCtl& ctl_s, uint32_t ring, uint8_t* ring_ptr,
                              uint8_t* stage_s, RoleState& rs, const WaitCtl& ctl, int warp, int lane) {
  const MegaParams& p = ca.p;
  const int S = st.seq, B = st.batch, H = st.heads;
  // kPair: the two CTAs of a pair take the two heads 2c, 2c + 1 of one sequence (same valid length) and the leader
  // issues ONE pair MMA for both: A = [Q_0; Q_1] (M = 256), B = [K_0; K_1] (N = 256), so CTA r finds Q_r K_r^T in
  // columns 128 r .. of its accumulator (the off-diagonal blocks are waste the tensor core has time for); then
  // A = [P_0; P_1], B = [V_0 | V_1] (N = 128) leaves O_r in columns 64 r ...  Every CTA loads exactly its own Q, K, V.
  // The output accumulator re-uses the columns of the scores (512 columns hold two pipelines of 256), so the scores
  // of a pipeline's next item wait until its output has been read (o_empty).
  const uint32_t rank = kPair ? cluster_cta_rank() : 0u;
  const int units = kPair ? (B * H) >> 1 : B * H;                      // couples of heads, or single (sequence, head) items
  const int first = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, step = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int my_items = units > first ? (units - 1 - first) / step + 1 : 0;
  auto item_of = [&](int k) -> int { const int u = first + k * step; return kPair ? 2 * u + (int)rank : u; };
  const uint32_t bar0 = smem_u32(&ctl_s.qk_full), bar1 = smem_u32(&ctl_s.attn1[0]);
  auto bar = [&](int g, int which) -> uint32_t { return (g ? bar1 : bar0) + 8u * (uint32_t)which; };
  const uint32_t oempty0 = smem_u32(&ctl_s.o_empty[0]);
  const CUtensorMap* tm = map_ptr(ca, st.tm_qkv);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t bits = rs.attn_bit | (rs.attn_bit1 << 1);
      for (int k = 0; k < my_items; ++k) {
        const int item = item_of(k), g = k & 1;
        const int h = item % H, b = item / H;
        const int rq = ((0 * B + b) * H + h) * S, rk = ((1 * B + b) * H + h) * S, rv = ((2 * B + b) * H + h) * S;
        const uint32_t base = ring + g * kPipeBytes, bit = (bits >> g) & 1u;
        if (!mbar_wait(bar(g, AB_QK_EMPTY), bit ^ 1u, ctl, 500 + g)) break;
        if constexpr (kPair) {            // both CTAs' tiles are counted on the leader's barriers
          if (rank == 0) mbar_expect_tx(bar(g, AB_QK_FULL), 4u * kATileBytes);
          const uint32_t fl = map_shared_rank(bar(g, AB_QK_FULL), 0);
          tma_load_2d_pair(base, tm, fl, 0, rq);
          tma_load_2d_pair(base + kATileBytes, tm, fl, 0, rk);
        } else {
          mbar_expect_tx(bar(g, AB_QK_FULL), 2u * kATileBytes);
          tma_load_2d(base, tm, bar(g, AB_QK_FULL), 0, rq);
          tma_load_2d(base + kATileBytes, tm, bar(g, AB_QK_FULL), 0, rk);
        }
        if (!mbar_wait(bar(g, AB_V_EMPTY), bit ^ 1u, ctl, 502 + g)) break;
        if constexpr (kPair) {
          if (rank == 0) mbar_expect_tx(bar(g, AB_V_FULL), 2u * kATileBytes);
          tma_load_2d_pair(base + 2 * kATileBytes, tm, map_shared_rank(bar(g, AB_V_FULL), 0), 0, rv);
        } else {
          mbar_expect_tx(bar(g, AB_V_FULL), (uint32_t)kATileBytes);
          tma_load_2d(base + 2 * kATileBytes, tm, bar(g, AB_V_FULL), 0, rv);
        }
        bits ^= 1u << g;
      }
      rs.attn_bit = bits & 1u;
      rs.attn_bit1 = (bits >> 1) & 1u;
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc_s = kPair ? umma_idesc_f16_pair(256u, 0u) : umma_idesc_f16(128u, 0u);
      const uint32_t idesc_o = kPair ? umma_idesc_f16_pair(128u, 1u) : umma_idesc_f16(64u, 1u);
      const uint32_t tmem = ctl_s.tmem_base;
      uint32_t bits = rs.attn_bit | (rs.attn_bit1 << 1);
      uint32_t obits = rs.o_bits;                              // pair form: phase bit of the o_empty barrier of each pipeline
      bool ok = true;
      auto issue_s = [&](int k) {                              // scores of item k: S = Q K^T
        const int g = k & 1;
        const uint32_t base = ring + g * kPipeBytes;
        if (!mbar_wait(bar(g, AB_QK_FULL), (bits >> g) & 1u, ctl, 510 + g)) { ok = false; return; }
        tc_fence_after_sync();
        if constexpr (kPair) {
          umma_f16_k64_pair(tmem + g * 256, umma_desc_lo(base, 16), umma_desc_lo(base + kATileBytes, 16), 2u, idesc_s, 0u);
          umma_commit_pair(bar(g, AB_S_FULL));
          umma_commit_pair(bar(g, AB_QK_EMPTY));
        } else {
          umma_f16_k64(tmem + g * 128, umma_desc_lo(base, 16), umma_desc_lo(base + kATileBytes, 16), 2u, idesc_s, 0u);
          umma_commit(bar(g, AB_S_FULL));
          umma_commit(bar(g, AB_QK_EMPTY));
        }
      };
      if (my_items > 0) issue_s(0);
      if (ok && my_items > 1) issue_s(1);
      for (int k = 0; ok && k < my_items; ++k) {
        const int g = k & 1;
        const uint32_t base = ring + g * kPipeBytes, bit = (bits >> g) & 1u;
        if (!mbar_wait(bar(g, AB_P_FULL), bit, ctl, 512 + g)) break;
        if (!mbar_wait(bar(g, AB_V_FULL), bit, ctl, 514 + g)) break;
        tc_fence_after_sync();
        // O = P V: K = 128 keys = two chunks of 64; V is an MN-major B operand (16 keys = 2048 B per step)
        if constexpr (kPair) {
          const uint32_t d = tmem + g * 256;                   // over the scores, which the softmax has consumed
          umma_f16_k64_pair(d, umma_desc_lo(base + 3 * kATileBytes, 16), umma_desc_lo(base + 2 * kATileBytes, 8192), 128u, idesc_o, 0u);
          umma_f16_k64_pair(d, umma_desc_lo(base + 4 * kATileBytes, 16), umma_desc_lo(base + 2 * kATileBytes + 8192, 8192), 128u,
                            idesc_o, 1u);
          umma_commit_pair(bar(g, AB_O_FULL));
          umma_commit_pair(bar(g, AB_V_EMPTY));
        } else {
          const uint32_t d = tmem + kPipeOCol + g * 64;
          umma_f16_k64(d, umma_desc_lo(base + 3 * kATileBytes, 16), umma_desc_lo(base + 2 * kATileBytes, 8192), 128u, idesc_o, 0u);
          umma_f16_k64(d, umma_desc_lo(base + 4 * kATileBytes, 16), umma_desc_lo(base + 2 * kATileBytes + 8192, 8192), 128u,
                       idesc_o, 1u);
          umma_commit(bar(g, AB_O_FULL));
          umma_commit(bar(g, AB_V_EMPTY));
        }
        bits ^= 1u << g;
        if (k + 2 < my_items) {
          if constexpr (kPair) {          // the next scores of this pipeline overwrite the output just issued: wait for its readers
            if (!mbar_wait(oempty0 + 8 * g, (obits >> g) & 1u, ctl, 516 + g)) break;
            tc_fence_after_sync();
          }
          issue_s(k + 2);
        }
        obits ^= 1u << g;                 // one phase of o_empty per item, waited for or not
      }
      rs.attn_bit = bits & 1u;
      rs.attn_bit1 = (bits >> 1) & 1u;
      rs.o_bits = obits;
    }
    __syncwarp();
  } else if (warp < 2 + kEpiWarps) {
    const int g = (warp - 2) >> 2, q = warp & 3;
    const int r_in = q * 32 + lane;
    const uint32_t tmem = ctl_s.tmem_base + ((uint32_t)(q * 32) << 16);
    const float sl2 = st.scale * 1.4426950408889634f;
    const float mask_l2 = -10000.0f * 1.4426950408889634f;
    const int* lens = st.lens_from_call ? p.lens : st.lens;
    __half* ctx = reinterpret_cast<__half*>(st.out);
    __half* probs = reinterpret_cast<__half*>(st.probs);
    const int hd = st.head_dim, hidden = H * hd;
    uint8_t* sbuf = stage_s + (warp - 2) * kStageWarp;
    uint8_t* pbase = ring_ptr + g * kPipeBytes + 3 * kATileBytes + r_in * 128;
    uint32_t bit = g ? rs.attn_bit1 : rs.attn_bit;
    const bool prof = p.prof != nullptr;
    long long t_ws = 0, t_sm = 0, t_wo = 0, t_ep = 0, t_p1 = 0;
    for (int k = g; k < my_items; k += 2) {
      const int item = item_of(k);
      const int h = item % H, b = item / H;
      const int kv_len = lens ? lens[b] : S;
      const long long c0 = prof ? clock64() : 0;
      if (!mbar_wait_warp(bar(g, AB_S_FULL), bit, ctl, 520 + g, lane)) break;
      const long long c1 = prof ? clock64() : 0;
      tc_fence_after_sync();
      const uint32_t ts = kPair ? tmem + g * 256 + rank * 128 : tmem + g * 128;
      // Masked keys (>= kv_len) get -10000 added, which underflows to probability 0 in fp32 and never wins
      // the maximum, so both passes only visit the 16-column blocks that hold valid keys.  TMEM loads are
      // double-buffered 16 columns at a time: the next block is in flight while this one is processed.
      const int kvl = kv_len < 1 ? 1 : (kv_len > S ? S : kv_len);
      const int nb = (kvl + 15) >> 4;
      uint32_t ra[16], rb[16];
      // ---- pass 1: row maximum of the raw scores of the valid keys (the scale is positive) ----
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
      auto max16 = [&](const uint32_t (&r)[16], int blk) {
        const int key0 = blk * 16;
        if (key0 + 16 <= kvl) {
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(r[i])); m1 = fmaxf(m1, __uint_as_float(r[i + 1]));
            m2 = fmaxf(m2, __uint_as_float(r[i + 2])); m3 = fmaxf(m3, __uint_as_float(r[i + 3]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) m0 = fmaxf(m0, key0 + i < kvl ? __uint_as_float(r[i]) : -INFINITY);
        }
      };
      tmem_ld16(ts, ra);
      tmem_ld_wait(ra);
      for (int blk = 0; blk < nb; blk += 2) {
        if (blk + 1 < nb) tmem_ld16(ts + (blk + 1) * 16, rb);
        max16(ra, blk);
        if (blk + 1 < nb) {
          tmem_ld_wait(rb);
          if (blk + 2 < nb) tmem_ld16(ts + (blk + 2) * 16, ra);
          max16(rb, blk + 1);
          if (blk + 2 < nb) tmem_ld_wait(ra);
        }
      }
      const float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * sl2;
      const long long c1a = prof ? clock64() : 0;
      // ---- pass 2: unnormalised probabilities -> fp16 A-operand tile (128B-swizzled rows) ----
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      auto exp16 = [&](const uint32_t (&r)[16], int blk) {
        const int key0 = blk * 16;
        uint32_t w[8];
        if (key0 + 16 <= kvl) {
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            const float p0 = ex2_fast(fmaf(__uint_as_float(r[i]), sl2, -mx)), p1 = ex2_fast(fmaf(__uint_as_float(r[i + 1]), sl2, -mx));
            const float p2 = ex2_fast(fmaf(__uint_as_float(r[i + 2]), sl2, -mx)), p3 = ex2_fast(fmaf(__uint_as_float(r[i + 3]), sl2, -mx));
            s0 += p0; s1 += p1; s2 += p2; s3 += p3;
            w[i >> 1] = pack_h2(p0, p1);
            w[(i >> 1) + 1] = pack_h2(p2, p3);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float p0 = key0 + i < kvl ? ex2_fast(fmaf(__uint_as_float(r[i]), sl2, -mx)) : 0.f;
            const float p1 = key0 + i + 1 < kvl ? ex2_fast(fmaf(__uint_as_float(r[i + 1]), sl2, -mx)) : 0.f;
            s0 += p0; s1 += p1;
            w[i >> 1] = pack_h2(p0, p1);
          }
        }
        uint8_t* base = pbase + (blk >> 2) * kATileBytes;
        const int j = (blk & 3) * 2;
        *reinterpret_cast<uint4*>(base + ((j ^ (r_in & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(base + (((j + 1) ^ (r_in & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
      };
      tmem_ld16(ts, ra);
      tmem_ld_wait(ra);
      for (int blk = 0; blk < nb; blk += 2) {
        if (blk + 1 < nb) tmem_ld16(ts + (blk + 1) * 16, rb);
        exp16(ra, blk);
        if (blk + 1 < nb) {
          tmem_ld_wait(rb);
          if (blk + 2 < nb) tmem_ld16(ts + (blk + 2) * 16, ra);
          exp16(rb, blk + 1);
          if (blk + 2 < nb) tmem_ld_wait(ra);
        }
      }
      for (int blk = nb; blk < 8; ++blk) {                    // keys past the valid ones: probability 0
        uint8_t* base = pbase + (blk >> 2) * kATileBytes;
        const int j = (blk & 3) * 2;
        *reinterpret_cast<uint4*>(base + ((j ^ (r_in & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(base + (((j + 1) ^ (r_in & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
      }
      const float inv = 1.0f / ((s0 + s1) + (s2 + s3));
      if (probs) {                                            // parity output: normalised probabilities
        attn_store_probs_staged(ts, sbuf, probs + (size_t)(b * H + h) * S * S, q * 32, S, kv_len, sl2, mask_l2, mx, inv, lane);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      if constexpr (kPair) {                                  // one arrival per warp on the leader's barrier (8 in all)
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_shared_rank(bar(g, AB_P_FULL), 0));
      } else {
        mbar_arrive(bar(g, AB_P_FULL));
      }
      const long long c2 = prof ? clock64() : 0;
      if (!mbar_wait_warp(bar(g, AB_O_FULL), bit, ctl, 522 + g, lane)) break;
      const long long c3 = prof ? clock64() : 0;
      tc_fence_after_sync();
      {
        // O rows are 128 bytes: two staged stores of 64 bytes per row
        const int row0 = q * 32;
        uint8_t* rowptr[4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld32((kPair ? tmem + g * 256 + rank * 64 : tmem + kPipeOCol + g * 64) + half * 32, r);
          tmem_ld_wait(r);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int rr = row0 + 8 * i + (lane >> 2);
            rowptr[i] = rr < S ? reinterpret_cast<uint8_t*>(ctx + ((size_t)b * S + rr) * hidden + h * hd + half * 32) : nullptr;
          }
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = pack_h2(__uint_as_float(r[2 * i]) * inv, __uint_as_float(r[2 * i + 1]) * inv);
          staged_store_64B(sbuf, w, rowptr, lane);
        }
      }
      tc_fence_before_sync();
      if constexpr (kPair) {                                  // this warp has read its rows of the output accumulator
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(map_shared_rank(oempty0 + 8 * g, 0));
      }
      bit ^= 1u;
      if (prof) { const long long c4 = clock64(); t_ws += c1 - c0; t_sm += c2 - c1; t_wo += c3 - c2; t_ep += c4 - c3; t_p1 += c1a - c1; }
    }
    if (prof && warp == 2 && lane == 0) {  // [3] waiting for scores, [4] softmax, [5] waiting for P.V, [6] output
      long long* pr = p.prof + ((size_t)st.prof_index * gridDim.x + blockIdx.x) * kProfSlots;
      pr[3] = t_ws; pr[4] = t_sm; pr[5] = t_wo; pr[6] = t_ep; pr[7] = t_p1;
    }
    if (g) rs.attn_bit1 = bit; else rs.attn_bit = bit;
    // the other pipeline's bit advances with that pipeline's item count
    const int n_other = (my_items + (g ? 1 : 0)) >> 1;        // items handled by pipeline 1-g
    if (g) rs.attn_bit ^= (uint32_t)(n_other & 1); else rs.attn_bit1 ^= (uint32_t)(n_other & 1);
  }
}

// ------------------------------------------------------------------------------------
// Swin window attention: one work item = (window, head).  Q/K/V live window-major as [3][windows][64][C]
// with the heads side by side in C, so one 64-column TMA box holds a PAIR of 32-wide heads; the MMAs of
// head h read their half of every 128-byte row (K-major operands: descriptor start +64 B for odd heads)
// or their half of the output columns (P.V is computed for the pair, the other half is dropped).
// Scores get the relative-position bias of the (query, key) offset and, for shifted windows, -100 where
// query and key come from different sides of the wrap-around.  Slots >= win*win are padding.
// ------------------------------------------------------------------------------------
// Softmax of one query row of a WS x WS window (thread = row): reads the 64 score columns from TMEM,
// adds bias and shift mask, writes the unnormalised probabilities as an fp16 A-operand row (128B swizzle)
// and returns their sum.  Rows and keys >= WS*WS are padding (probability 0).
template <int WS>
__device__ __forceinline__ float swin_softmax_row(uint32_t tmem, const float* bias_s, uint8_t* prow, int r_in, int wy, int wx,
                                                  int R, int shift, float sl2) {
  constexpr int NT = WS * WS, TBL = 2 * WS - 1;
  const bool rowok = r_in < NT;
  const int qy = rowok ? r_in / WS : 0, qx = rowok ? r_in - qy * WS : 0;
  // region of a shifted coordinate along one axis: 0 | 1 | 2 (only the last window row/column mixes regions)
  int regy[WS], regx[WS];
#pragma unroll
  for (int i = 0; i < WS; ++i) {
    const int sy = wy + i, sx = wx + i;
    regy[i] = shift ? (sy < R - WS ? 0 : (sy < R - shift ? 1 : 2)) : 0;
    regx[i] = shift ? (sx < R - WS ? 0 : (sx < R - shift ? 1 : 2)) : 0;
  }
  int qreg = 0;
#pragma unroll
  for (int i = 0; i < WS; ++i) {
    if (i == qy) qreg += regy[i] * 3;
    if (i == qx) qreg += regx[i];
  }
  const float* brow = bias_s + (qy + WS - 1) * TBL + (qx + WS - 1);   // bias index = brow[-(ky*TBL + kx)]
  const float mask = -100.0f * 1.4426950408889634f;
  uint32_t r0[32], r1[32];
  tmem_ld32(tmem, r0);
  tmem_ld32(tmem + 32, r1);
  tmem_ld_wait(r0);
  tmem_ld_wait(r1);
  float mx = -INFINITY;
#pragma unroll
  for (int k = 0; k < 64; ++k) {
    if (k < NT) {
      constexpr int dummy = 0; (void)dummy;
      const int ky = k / WS, kx = k % WS;
      float v = __uint_as_float(k < 32 ? r0[k & 31] : r1[k & 31]) * sl2 + brow[-(ky * TBL + kx)];
      if (regy[ky] * 3 + regx[kx] != qreg) v += mask;
      if (k < 32) r0[k & 31] = __float_as_uint(v); else r1[k & 31] = __float_as_uint(v);
      mx = fmaxf(mx, v);
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t wv[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const int k = half * 32 + i;
      const float p0 = (k < NT && rowok) ? ex2_fast(__uint_as_float(half ? r1[i] : r0[i]) - mx) : 0.f;
      const float p1 = (k + 1 < NT && rowok) ? ex2_fast(__uint_as_float(half ? r1[i + 1] : r0[i + 1]) - mx) : 0.f;
      sum += p0 + p1;
      wv[i >> 1] = pack_h2(p0, p1);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(prow + (((half * 4 + j) ^ (r_in & 7)) << 4)) = make_uint4(wv[4 * j], wv[4 * j + 1], wv[4 * j + 2], wv[4 * j + 3]);
  }
  return rowok ? sum : 1.0f;
}

__device__ __noinline__ void attn_swin_stage(const Stage& st, const CallArgs& ca, SmemCtl& ctl_s, uint32_t ring, uint8_t* ring_ptr,
                                uint8_t* stage_s, RoleState& rs, const WaitCtl& ctl, int warp, int lane) {
  const int R = st.seq, ws = st.win, shift = st.shift, H = st.heads, C = st.ldo;
  const int nwr = R / ws, nw_img = nwr * nwr, n_windows = st.batch * nw_img, n_tok = ws * ws;
  const int items = n_windows * H;
  const uint32_t qk_full = smem_u32(&ctl_s.qk_full), qk_empty = smem_u32(&ctl_s.qk_empty);
  const uint32_t v_full = smem_u32(&ctl_s.v_full), v_empty = smem_u32(&ctl_s.v_empty);
  const uint32_t s_full = smem_u32(&ctl_s.s_full), p_full = smem_u32(&ctl_s.p_full), o_full = smem_u32(&ctl_s.o_full);
  const CUtensorMap* tm = map_ptr(ca, st.tm_qkv);
  // shared memory: Q 16 KiB | K 16 KiB | V 16 KiB | P 16 KiB
  if (warp == 0) {
    if (lane == 0) {
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int h = item % H, w = item / H;
        const int col = (h >> 1) * 64;
        if (!mbar_wait(qk_empty, rs.attn_bit ^ 1u, ctl, 530)) break;
        mbar_expect_tx(qk_full, 2u * kATileBytes);
        tma_load_2d(ring, tm, qk_full, col, (0 * n_windows + w) * 64);
        tma_load_2d(ring + kATileBytes, tm, qk_full, col, (1 * n_windows + w) * 64);
        if (!mbar_wait(v_empty, rs.attn_bit ^ 1u, ctl, 531)) break;
        mbar_expect_tx(v_full, (uint32_t)kATileBytes);
        tma_load_2d(ring + 2 * kATileBytes, tm, v_full, col, (2 * n_windows + w) * 64);
        rs.attn_bit ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_f16(64u, 0u), idesc_o = umma_idesc_f16(64u, 1u);
      const uint32_t tmem = ctl_s.tmem_base;
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int h = item % H;
        const uint32_t half = (uint32_t)(h & 1) * 4u;                  // 64 bytes into every 128-byte row
        if (!mbar_wait(qk_full, rs.attn_bit, ctl, 532)) break;
        tc_fence_after_sync();
        {
          // S[128 x 64] = Q_h K_h^T, K = 32: two K=16 steps
          const uint64_t hi = (uint64_t)kDescHiSw128 << 32;
          const uint64_t qd = hi | (umma_desc_lo(ring, 16) + half), kd = hi | (umma_desc_lo(ring + kATileBytes, 16) + half);
          umma_f16(tmem, qd, kd, idesc_s, 0u);
          umma_f16(tmem, qd + 2u, kd + 2u, idesc_s, 1u);
        }
        umma_commit(s_full);
        umma_commit(qk_empty);
        if (!mbar_wait(p_full, rs.attn_bit, ctl, 533)) break;
        if (!mbar_wait(v_full, rs.attn_bit, ctl, 534)) break;
        tc_fence_after_sync();
        // O[128 x 64] = P[128 x 64 keys] V_pair[64 keys x 64]: one K chunk of 64
        umma_f16_k64(tmem + 128, umma_desc_lo(ring + 3 * kATileBytes, 16), umma_desc_lo(ring + 2 * kATileBytes, 8192), 128u,
                     idesc_o, 0u);
        umma_commit(o_full);
        umma_commit(v_empty);
        rs.attn_bit ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    const int q = warp & 3, r_in = q * 32 + lane;
    const uint32_t tmem = ctl_s.tmem_base + ((uint32_t)(q * 32) << 16);
    const float sl2 = st.scale * 1.4426950408889634f, l2e = 1.4426950408889634f;
    const __half* table = reinterpret_cast<const __half*>(st.rel_bias);
    __half* ctx = reinterpret_cast<__half*>(st.out);
    const int tbl = 2 * ws - 1;
    float* bias_s = reinterpret_cast<float*>(stage_s);               // this head's column of the bias table (x log2 e)
    uint8_t* prow = ring_ptr + 3 * kATileBytes + r_in * 128;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int h = item % H, wg = item / H, w = wg % nw_img;
      const int wy = (w / nwr) * ws, wx = (w % nwr) * ws;
      named_barrier_sync(2, 128);                                    // previous item's readers are done with bias_s
      for (int i = r_in; i < tbl * tbl; i += 128) bias_s[i] = __half2float(table[i * H + h]) * l2e;
      named_barrier_sync(2, 128);
      if (!mbar_wait_warp(s_full, rs.attn_bit, ctl, 535, lane)) break;
      tc_fence_after_sync();
      float sum = 1.0f;
      if (ws == 7) sum = swin_softmax_row<7>(tmem, bias_s, prow, r_in, wy, wx, R, shift, sl2);
      else sum = swin_softmax_row<8>(tmem, bias_s, prow, r_in, wy, wx, R, shift, sl2);
      const float inv = 1.0f / sum;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_full);
      if (!mbar_wait_warp(o_full, rs.attn_bit, ctl, 536, lane)) break;
      tc_fence_after_sync();
      {
        uint32_t o[32];
        tmem_ld32(tmem + 128 + (h & 1) * 32, o);
        tmem_ld_wait(o);
        if (r_in < n_tok) {
          uint4* dst = reinterpret_cast<uint4*>(ctx + ((size_t)wg * 64 + r_in) * C + h * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[i] = make_uint4(pack_h2(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv),
                                pack_h2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv),
                                pack_h2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv),
                                pack_h2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv));
        }
      }
      tc_fence_before_sync();
      rs.attn_bit ^= 1u;
    }
  }
}

// ------------------------------------------------------------------------------------
// LayerNorm stage.  Rows stream through shared memory in batches fetched by bulk copies (all
// split-K planes plus the residual of a batch are in flight together, several batches deep), so
// the stage is bound by memory bandwidth rather than by per-warp load latency.  A warp owns a
// row: z = sum of planes + bias + residual, two-pass statistics in fp32, fp16 output.
// ------------------------------------------------------------------------------------
constexpr int kLnMaxBufs = 4;

// Two rows per call (the second optional): their instruction streams interleave, which hides the
// shared-memory, shuffle and MUFU latencies a single row's dependent chain exposes.
// kCg: the rows are read straight from global memory (L2: they were written by other SMs a stage ago).
template <bool kCg>
__device__ __forceinline__ float4 ln_ld4(const float* p) {
  if constexpr (kCg) return __ldcg(reinterpret_cast<const float4*>(p));
  else return *reinterpret_cast<const float4*>(p);
}
template <bool kCg>
__device__ __forceinline__ uint2 ln_ld2(const __half* p) {
  if constexpr (kCg) return __ldcg(reinterpret_cast<const uint2*>(p));
  else return *reinterpret_cast<const uint2*>(p);
}

template <int NJ, bool kCg = false>
__device__ __forceinline__ void ln_rows2(const float* pl0, const float* pl1, int n_partial, int plane_stride,
                                         const __half* res0, const __half* res1, const __half* bias,
                                         const __half* gamma, const __half* beta, float eps, __half* out0, __half* out1,
                                         int lane) {
  const bool two = out1 != nullptr;
  float z[2][NJ][4];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 a = n_partial > 0 ? ln_ld4<kCg>(pl0 + (lane + 32 * j) * 4) : zero4;
    const float4 b = (two && n_partial > 0) ? ln_ld4<kCg>(pl1 + (lane + 32 * j) * 4) : zero4;
    z[0][j][0] = a.x; z[0][j][1] = a.y; z[0][j][2] = a.z; z[0][j][3] = a.w;
    z[1][j][0] = b.x; z[1][j][1] = b.y; z[1][j][2] = b.z; z[1][j][3] = b.w;
  }
  for (int pl = 1; pl < n_partial; ++pl) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const float4 a = ln_ld4<kCg>(pl0 + (size_t)pl * plane_stride + (lane + 32 * j) * 4);
      z[0][j][0] += a.x; z[0][j][1] += a.y; z[0][j][2] += a.z; z[0][j][3] += a.w;
      if (two) {
        const float4 b = ln_ld4<kCg>(pl1 + (size_t)pl * plane_stride + (lane + 32 * j) * 4);
        z[1][j][0] += b.x; z[1][j][1] += b.y; z[1][j][2] += b.z; z[1][j][3] += b.w;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    float add[4] = {0.f, 0.f, 0.f, 0.f};
    if (bias) {
      const uint2 u = *reinterpret_cast<const uint2*>(bias + (lane + 32 * j) * 4);
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
      const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
      add[0] = f0.x; add[1] = f0.y; add[2] = f1.x; add[3] = f1.y;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const __half* res = r ? res1 : res0;
      float rr[4] = {0.f, 0.f, 0.f, 0.f};
      if (res && (r == 0 || two)) {
        const uint2 u = ln_ld2<kCg>(res + (lane + 32 * j) * 4);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        rr[0] = f0.x; rr[1] = f0.y; rr[2] = f1.x; rr[3] = f1.y;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) z[r][j][i] += add[i] + rr[i];
    }
  }
  if (eps < 0.0f) {                     // sum only: the split-K reduction of a GEMM whose consumer reads fp16
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      *reinterpret_cast<uint2*>(out0 + (lane + 32 * j) * 4) = make_uint2(pack_h2(z[0][j][0], z[0][j][1]), pack_h2(z[0][j][2], z[0][j][3]));
      if (two) *reinterpret_cast<uint2*>(out1 + (lane + 32 * j) * 4) = make_uint2(pack_h2(z[1][j][0], z[1][j][1]), pack_h2(z[1][j][2], z[1][j][3]));
    }
    return;
  }
  const float inv_n = 1.0f / (float)(NJ * 128);
  float sa = 0.0f, sb = 0.0f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    sa += (z[0][j][0] + z[0][j][1]) + (z[0][j][2] + z[0][j][3]);
    sb += (z[1][j][0] + z[1][j][1]) + (z[1][j][2] + z[1][j][3]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sa += __shfl_xor_sync(0xffffffffu, sa, o);
    sb += __shfl_xor_sync(0xffffffffu, sb, o);
  }
  const float mean0 = sa * inv_n, mean1 = sb * inv_n;
  float va = 0.0f, vb = 0.0f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float d0 = z[0][j][i] - mean0, d1 = z[1][j][i] - mean1;
      va = fmaf(d0, d0, va);
      vb = fmaf(d1, d1, vb);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    va += __shfl_xor_sync(0xffffffffu, va, o);
    vb += __shfl_xor_sync(0xffffffffu, vb, o);
  }
  const float rstd0 = rsqrtf(va * inv_n + eps), rstd1 = rsqrtf(vb * inv_n + eps);
  // (z - mean) * rstd in fp32 (one FMA), rounded to fp16 pairs; gamma and beta are applied on the pairs (one packed
  // FMA per two elements, no conversions).  With gamma = 1, beta = 0 that last step is exact.
  const float nm0 = -mean0 * rstd0, nm1 = -mean1 * rstd1;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    uint2 ug = make_uint2(0u, 0u), ub = make_uint2(0u, 0u);
    if (gamma) {
      ug = *reinterpret_cast<const uint2*>(gamma + (lane + 32 * j) * 4);
      ub = *reinterpret_cast<const uint2*>(beta + (lane + 32 * j) * 4);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (r == 1 && !two) break;
      const float rs_ = r ? rstd1 : rstd0, nm = r ? nm1 : nm0;
      uint32_t w0 = pack_h2(fmaf(z[r][j][0], rs_, nm), fmaf(z[r][j][1], rs_, nm));
      uint32_t w1 = pack_h2(fmaf(z[r][j][2], rs_, nm), fmaf(z[r][j][3], rs_, nm));
      if (gamma) {
        const __half2 y0 = __hfma2(*reinterpret_cast<const __half2*>(&w0), *reinterpret_cast<const __half2*>(&ug.x),
                                   *reinterpret_cast<const __half2*>(&ub.x));
        const __half2 y1 = __hfma2(*reinterpret_cast<const __half2*>(&w1), *reinterpret_cast<const __half2*>(&ug.y),
                                   *reinterpret_cast<const __half2*>(&ub.y));
        w0 = *reinterpret_cast<const uint32_t*>(&y0);
        w1 = *reinterpret_cast<const uint32_t*>(&y1);
      }
      *reinterpret_cast<uint2*>((r ? out1 : out0) + (lane + 32 * j) * 4) = make_uint2(w0, w1);
    }
  }
}

// Patch-merging gather (one lane): row (img, h, w) of the merged matrix = tokens (2h, 2w), (2h+1, 2w), (2h, 2w+1),
// (2h+1, 2w+1) of a [batch][R][R][N/4] fp16 grid side by side, one bulk copy each.
__device__ __noinline__ void ln_gather_rows(uint32_t dst, const __half* src, int row0, int rows, int N, int R, uint32_t bar) {
  const int R2 = R >> 1, Cq = N >> 2;
  for (int r = 0; r < rows; ++r) {
    const int gr = row0 + r, img = gr / (R2 * R2), rem = gr - img * R2 * R2, h2 = rem / R2, w2 = rem - h2 * R2;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const size_t token = (size_t)img * R * R + (size_t)(2 * h2 + (q & 1)) * R + (2 * w2 + (q >> 1));
      bulk_load(dst + (uint32_t)(r * N + q * Cq) * 2u, src + token * Cq, (uint32_t)(Cq * 2), bar);
    }
  }
}

// LayerNorm of one fp16 row of 2048 columns held in shared memory (the merged rows of a C = 512 stage): too wide
// for the two-rows-per-warp routine's registers.  Same arithmetic: two-pass fp32 statistics, packed-half affine.
__device__ __noinline__ void ln_row_wide(const __half* row, const __half* gamma, const __half* beta, float eps, __half* out, int lane) {
  constexpr int NJ = 16;
  float z[NJ][4];
  float sa = 0.0f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const uint2 u = *reinterpret_cast<const uint2*>(row + (lane + 32 * j) * 4);
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    z[j][0] = f0.x; z[j][1] = f0.y; z[j][2] = f1.x; z[j][3] = f1.y;
    sa += (f0.x + f0.y) + (f1.x + f1.y);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sa += __shfl_xor_sync(0xffffffffu, sa, o);
  const float inv_n = 1.0f / (float)(NJ * 128), mean = sa * inv_n;
  float va = 0.0f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float d0 = z[j][i] - mean;
      va = fmaf(d0, d0, va);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) va += __shfl_xor_sync(0xffffffffu, va, o);
  const float rstd = rsqrtf(va * inv_n + eps), nm = -mean * rstd;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    uint32_t w0 = pack_h2(fmaf(z[j][0], rstd, nm), fmaf(z[j][1], rstd, nm));
    uint32_t w1 = pack_h2(fmaf(z[j][2], rstd, nm), fmaf(z[j][3], rstd, nm));
    if (gamma) {
      // plain loads: the vectors may have been staged in shared memory by the caller
      const uint2 ug = *reinterpret_cast<const uint2*>(gamma + (lane + 32 * j) * 4);
      const uint2 ub = *reinterpret_cast<const uint2*>(beta + (lane + 32 * j) * 4);
      const __half2 y0 = __hfma2(*reinterpret_cast<const __half2*>(&w0), *reinterpret_cast<const __half2*>(&ug.x),
                                 *reinterpret_cast<const __half2*>(&ub.x));
      const __half2 y1 = __hfma2(*reinterpret_cast<const __half2*>(&w1), *reinterpret_cast<const __half2*>(&ug.y),
                                 *reinterpret_cast<const __half2*>(&ub.y));
      w0 = *reinterpret_cast<const uint32_t*>(&y0);
      w1 = *reinterpret_cast<const uint32_t*>(&y1);
    }
    *reinterpret_cast<uint2*>(out + (lane + 32 * j) * 4) = make_uint2(w0, w1);
  }
}

// One row of the direct form: the lanes of a warp read the row straight from L2.  Every round trip costs ~800 cycles,
// so the loads are issued in as few dependent rounds as the registers allow: bias, residual and the first planes
// together, further planes kG at a time, gamma and beta just before the statistics (they land while the shuffles run).
// With the loads strung one behind the other a row of six planes took 6.2 k cycles.
template <int NJ>
__device__ __forceinline__ void ln_row_direct(const float* pl, int n_partial, int plane_stride, const __half* res,
                                              const __half* bias, const __half* gamma, const __half* beta, float eps,
                                              __half* out, int lane) {
  constexpr int kG = NJ <= 4 ? 4 : (NJ <= 6 ? 3 : 2);      // planes in flight at once
  float z[NJ][4];
  {
    uint2 ub[NJ], ur[NJ];
    float4 v[kG][NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      ub[j] = bias ? __ldg(reinterpret_cast<const uint2*>(bias + (lane + 32 * j) * 4)) : make_uint2(0u, 0u);
      ur[j] = res ? __ldcg(reinterpret_cast<const uint2*>(res + (lane + 32 * j) * 4)) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int g = 0; g < kG; ++g)
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        v[g][j] = g < n_partial ? __ldcg(reinterpret_cast<const float4*>(pl + (size_t)g * plane_stride + (lane + 32 * j) * 4))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(&ub[j].x)), b1 = __half22float2(*reinterpret_cast<const __half2*>(&ub[j].y));
      const float2 r0 = __half22float2(*reinterpret_cast<const __half2*>(&ur[j].x)), r1 = __half22float2(*reinterpret_cast<const __half2*>(&ur[j].y));
      z[j][0] = b0.x + r0.x; z[j][1] = b0.y + r0.y; z[j][2] = b1.x + r1.x; z[j][3] = b1.y + r1.y;
#pragma unroll
      for (int g = 0; g < kG; ++g) { z[j][0] += v[g][j].x; z[j][1] += v[g][j].y; z[j][2] += v[g][j].z; z[j][3] += v[g][j].w; }
    }
    for (int p0 = kG; p0 < n_partial; p0 += kG) {
#pragma unroll
      for (int g = 0; g < kG; ++g)
#pragma unroll
        for (int j = 0; j < NJ; ++j)
          v[g][j] = p0 + g < n_partial ? __ldcg(reinterpret_cast<const float4*>(pl + (size_t)(p0 + g) * plane_stride + (lane + 32 * j) * 4))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int g = 0; g < kG; ++g) { z[j][0] += v[g][j].x; z[j][1] += v[g][j].y; z[j][2] += v[g][j].z; z[j][3] += v[g][j].w; }
    }
  }
  if (eps < 0.0f) {                     // sum only
#pragma unroll
    for (int j = 0; j < NJ; ++j)
      *reinterpret_cast<uint2*>(out + (lane + 32 * j) * 4) = make_uint2(pack_h2(z[j][0], z[j][1]), pack_h2(z[j][2], z[j][3]));
    return;
  }
  uint2 ug[NJ], ubt[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    ug[j] = gamma ? __ldg(reinterpret_cast<const uint2*>(gamma + (lane + 32 * j) * 4)) : make_uint2(0u, 0u);
    ubt[j] = gamma ? __ldg(reinterpret_cast<const uint2*>(beta + (lane + 32 * j) * 4)) : make_uint2(0u, 0u);
  }
  const float inv_n = 1.0f / (float)(NJ * 128);
  float sa = 0.0f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) sa += (z[j][0] + z[j][1]) + (z[j][2] + z[j][3]);
  sa = warp_sum(sa);
  const float mean = sa * inv_n;
  float va = 0.0f;
#pragma unroll
  for (int j = 0; j < NJ; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float d0 = z[j][i] - mean;
      va = fmaf(d0, d0, va);
    }
  va = warp_sum(va);
  const float rstd = rsqrtf(va * inv_n + eps), nm = -mean * rstd;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    uint32_t w0 = pack_h2(fmaf(z[j][0], rstd, nm), fmaf(z[j][1], rstd, nm));
    uint32_t w1 = pack_h2(fmaf(z[j][2], rstd, nm), fmaf(z[j][3], rstd, nm));
    if (gamma) {
      const __half2 y0 = __hfma2(*reinterpret_cast<const __half2*>(&w0), *reinterpret_cast<const __half2*>(&ug[j].x),
                                 *reinterpret_cast<const __half2*>(&ubt[j].x));
      const __half2 y1 = __hfma2(*reinterpret_cast<const __half2*>(&w1), *reinterpret_cast<const __half2*>(&ug[j].y),
                                 *reinterpret_cast<const __half2*>(&ubt[j].y));
      w0 = *reinterpret_cast<const uint32_t*>(&y0);
      w1 = *reinterpret_cast<const uint32_t*>(&y1);
    }
    *reinterpret_cast<uint2*>(out + (lane + 32 * j) * 4) = make_uint2(w0, w1);
  }
}

// Direct form of the LayerNorm stage (the host picks it when a CTA has at most one row per normalising warp): every
// warp reads its row from global memory itself -- no copy issue, copy latency and barrier wait of the staging ring.
// Out of line: its registers are not charged to the stage interpreter.
__device__ __noinline__ void ln_stage_direct(const Stage& st, const MegaParams& p, int warp, int lane) {
  const int N = st.N, M = st.M, P = st.n_partial, rb = st.bm, n_batches = st.items;
  if (warp >= rb) return;
  const __half* resid = reinterpret_cast<const __half*>(sel_ptr(st.resid_sel, st.resid, p));
  __half* out = reinterpret_cast<__half*>(const_cast<void*>(sel_ptr(st.out_sel, st.out, p)));
  const __half* bias = reinterpret_cast<const __half*>(st.bias);
  const __half* gamma = reinterpret_cast<const __half*>(st.gamma);
  const __half* beta = reinterpret_cast<const __half*>(st.beta);
  for (int blk = blockIdx.x; blk < n_batches; blk += gridDim.x) {
    const int row = blk * rb + warp;
    if (row >= M) break;
    const float* pl0 = st.partial + (size_t)row * N;
    const __half* ra = resid ? resid + (size_t)row * N : nullptr;
    __half* o0 = out + (size_t)row * N;
    switch (N >> 7) {
      case 1: ln_row_direct<1>(pl0, P, M * N, ra, bias, gamma, beta, st.eps, o0, lane); break;
      case 2: ln_row_direct<2>(pl0, P, M * N, ra, bias, gamma, beta, st.eps, o0, lane); break;
      case 4: ln_row_direct<4>(pl0, P, M * N, ra, bias, gamma, beta, st.eps, o0, lane); break;
      case 6: ln_row_direct<6>(pl0, P, M * N, ra, bias, gamma, beta, st.eps, o0, lane); break;
      default: ln_row_direct<8>(pl0, P, M * N, ra, bias, gamma, beta, st.eps, o0, lane); break;
    }
  }
}

// kMerge builds add the patch-merging form (Swin, python/models/swin_transformer/swin_patch_merge.py:1-17): with
// st.seq = R > 0 the fp16 input is a [batch][R][R][N/4] token grid and row (b, h, w) of the normalised matrix is the
// concatenation of tokens (2h, 2w), (2h+1, 2w), (2h, 2w+1), (2h+1, 2w+1), fetched as four bulk copies; rows of 2048
// columns are normalised one per warp and call.
template <bool kMerge>
__device__ __forceinline__ void ln_stage(const Stage& st, const MegaParams& p, SmemCtl& cs, uint32_t ring, uint8_t* ring_ptr,
                                         __half* vec_s, RoleState& rs, const WaitCtl& ctl, int warp, int lane) {
  const int N = st.N, M = st.M, P = st.n_partial;
  const __half* resid = reinterpret_cast<const __half*>(sel_ptr(st.resid_sel, st.resid, p));
  __half* out = reinterpret_cast<__half*>(const_cast<void*>(sel_ptr(st.out_sel, st.out, p)));
  const __half* bias = reinterpret_cast<const __half*>(st.bias);
  const __half* gamma = reinterpret_cast<const __half*>(st.gamma);
  const __half* beta = reinterpret_cast<const __half*>(st.beta);
  // Warp 0 only feeds the ring (issuing a bulk copy of tens of KB stalls the issuing thread until the copy
  // engine has taken the previous ones); the other warps normalise rows, two per warp and round.
  constexpr int kComp = kThreads / 32 - 1;
  // Batch geometry comes from the host (finalize_stage): rows per batch -- up to 96 KB so that two batches are
  // in flight, at most two rows per warp, and few enough that every CTA gets work -- buffers, batch count.
  const int row_bytes = (P * 4 + (resid ? 2 : 0)) * N;
  const int rb = st.bm, batch_bytes = st.slot_bytes, nbuf = st.nslots, n_batches = st.items;
  if (nbuf == 0) {          // direct form: see ln_stage_direct
    ln_stage_direct(st, p, warp, lane);
    return;
  }
  const bool stage_vecs = st.kchunks != 0;   // bias | gamma | beta side by side in shared memory
  const int my_batches = n_batches > (int)blockIdx.x ? (n_batches - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const uint32_t full0 = smem_u32(&cs.ln_full[0]), empty0 = smem_u32(&cs.ln_empty[0]);
  uint32_t bits = rs.ln_bits;
  const bool prof = p.prof != nullptr;

  if (warp == 0) {
    if (lane == 0) {
      if (prof) p.prof[((size_t)st.prof_index * gridDim.x + blockIdx.x) * kProfSlots + 9] = clock64();
      int buf = 0;
      for (int k = 0; k < my_batches; ++k) {
        const int batch = blockIdx.x + k * gridDim.x;
        if (!mbar_wait(empty0 + 8 * buf, ((bits >> buf) & 1u) ^ 1u, ctl, 610 + buf)) break;
        const int row0 = batch * rb;
        const int rows = (M - row0) < rb ? (M - row0) : rb;
        const uint32_t bar = full0 + 8 * buf;
        const uint32_t dst = ring + buf * batch_bytes;
        mbar_expect_tx(bar, (uint32_t)(rows * row_bytes));
        if (kMerge && st.seq > 0) {
          ln_gather_rows(dst, resid, row0, rows, N, st.seq, bar);
          bits ^= 1u << buf;
          buf = buf + 1 == nbuf ? 0 : buf + 1;
          continue;
        }
        for (int pl = 0; pl < P; ++pl)
          bulk_load(dst + pl * rb * N * 4, st.partial + ((size_t)pl * M + row0) * N, (uint32_t)(rows * N * 4), bar);
        if (resid) bulk_load(dst + P * rb * N * 4, resid + (size_t)row0 * N, (uint32_t)(rows * N * 2), bar);
        bits ^= 1u << buf;
        buf = buf + 1 == nbuf ? 0 : buf + 1;
      }
      if (prof) p.prof[((size_t)st.prof_index * gridDim.x + blockIdx.x) * kProfSlots + 10] = clock64();
    }
    __syncwarp();
  } else {
    const int cw = warp - 1;
    // The per-column vectors go to shared memory once (while the first batches are in flight): read from global
    // memory inside the row loop, a miss in the small L1 costs an L2 round trip in the middle of every row.
    if (stage_vecs) {
      const __half* srcs[3] = {bias, gamma, beta};
#pragma unroll
      for (int v = 0; v < 3; ++v) {
        if (!srcs[v]) continue;
        const uint2* src = reinterpret_cast<const uint2*>(srcs[v]);
        uint2* dst = reinterpret_cast<uint2*>(vec_s + v * N);
        for (int i = threadIdx.x - 32; i < N / 4; i += kThreads - 32) dst[i] = __ldg(src + i);
      }
      named_barrier_sync(2, kThreads - 32);
      if (bias) bias = vec_s;
      if (gamma) { gamma = vec_s + N; beta = vec_s + 2 * N; }
    }
    unsigned t_wait = 0, t_comp = 0;
    int buf = 0;
    for (int k = 0; k < my_batches; ++k) {
      const int batch = blockIdx.x + k * gridDim.x;
      const unsigned tw = prof ? (unsigned)clock64() : 0u;
      const bool ok = mbar_wait_warp(full0 + 8 * buf, (bits >> buf) & 1u, ctl, 600 + buf, lane);
      const unsigned tc = prof ? (unsigned)clock64() : 0u;
      t_wait += tc - tw;
      bits ^= 1u << buf;
      if (!ok) break;
      const int row0 = batch * rb;
      const int rows = (M - row0) < rb ? (M - row0) : rb;
      const float* base = reinterpret_cast<const float*>(ring_ptr + buf * batch_bytes);
      const __half* rbase = reinterpret_cast<const __half*>(ring_ptr + buf * batch_bytes + P * rb * N * 4);
      for (int r = cw; r < rows; r += 2 * kComp) {
        const int r2 = r + kComp;
        const bool two = r2 < rows;
        const float* pl0 = base + (size_t)r * N;
        const float* pl1 = two ? base + (size_t)r2 * N : nullptr;
        const __half* ra = resid ? rbase + (size_t)r * N : nullptr;
        const __half* rb2 = (resid && two) ? rbase + (size_t)r2 * N : nullptr;
        __half* o0 = out + (size_t)(row0 + r) * N;
        __half* o1 = two ? out + (size_t)(row0 + r2) * N : nullptr;
        switch (N >> 7) {
          case 1: ln_rows2<1>(pl0, pl1, P, rb * N, ra, rb2, bias, gamma, beta, st.eps, o0, o1, lane); break;
          case 2: ln_rows2<2>(pl0, pl1, P, rb * N, ra, rb2, bias, gamma, beta, st.eps, o0, o1, lane); break;
          case 4: ln_rows2<4>(pl0, pl1, P, rb * N, ra, rb2, bias, gamma, beta, st.eps, o0, o1, lane); break;
          case 6: ln_rows2<6>(pl0, pl1, P, rb * N, ra, rb2, bias, gamma, beta, st.eps, o0, o1, lane); break;
          case 16:
            if constexpr (kMerge) {
              ln_row_wide(ra, gamma, beta, st.eps, o0, lane);
              if (two) ln_row_wide(rb2, gamma, beta, st.eps, o1, lane);
            }
            break;
          default: ln_rows2<8>(pl0, pl1, P, rb * N, ra, rb2, bias, gamma, beta, st.eps, o0, o1, lane); break;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * buf);    // this warp is done with the buffer
      if (prof) t_comp += (unsigned)clock64() - tc;
      buf = buf + 1 == nbuf ? 0 : buf + 1;
    }
    if (prof && lane == 0)
      atomicMax(reinterpret_cast<unsigned long long*>(p.prof + ((size_t)st.prof_index * gridDim.x + blockIdx.x) * kProfSlots + 11),
                (unsigned long long)clock64());
    if (prof && warp == 2 && lane == 0) {    // [3] waiting for a batch, [7] normalising
      long long* pr = p.prof + ((size_t)st.prof_index * gridDim.x + blockIdx.x) * kProfSlots;
      pr[3] = t_wait;
      pr[4] = 0;
      pr[5] = rb;
      pr[6] = nbuf;
      pr[7] = t_comp;
      pr[8] = my_batches;
    }
  }
  // every thread leaves with the same view of the buffers' phase bits
  {
    const int q = my_batches / nbuf, rem = my_batches - q * nbuf;     // buffers 0..rem-1 were used q+1 times
    uint32_t flip = (q & 1) ? (1u << nbuf) - 1u : 0u;
    if (rem) flip ^= (1u << rem) - 1u;
    rs.ln_bits ^= flip;
  }
}

// ------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------
// 384 threads leave 168 registers per thread (the register file is handed out per four warps, so ten warps would
// leave no more); the epilogue is written to stay below that without spilling.
// The kernel exists in four builds, so that each fits 168 registers with its stages inlined where that matters:
//   kFamilyBert      BERT layers whose attention items outnumber the CTAs (two-pipeline attention), plain GEMMs,
//                    LayerNorm; every stage inlined into one register allocation (fastest).
//   kFamilyBertCoop  the same with the attention stage in which all eight softmax warps share one item: S up to
//                    384, and short sequences at small batch, where a CTA has at most one item anyway.
//   kFamilySwin      adds the Swin row-permuting epilogues and the window-attention stage; its stages stay out
//                    of line (inlined as well, the allocation would no longer fit).
//   kFamilyBertPair  kFamilyBert on CTA pairs: a cluster of two CTAs shares every MMA (cta_group::2), which halves the
//                    weight-tile traffic per FLOP of the GEMM stages; the attention stage takes two heads per pair.
//                    Launched with a cluster dimension of two.
constexpr int kFamilyBert = 0, kFamilyBertCoop = 1, kFamilySwin = 2, kFamilyBertPair = 3;
__device__ __noinline__ void gemm_stage_ool(const Stage& st, const CallArgs& ca, SmemCtl& ctl_s, uint32_t ring, __half* vec_s,
                                            uint8_t* stage_s, RoleState& rs, const WaitCtl& ctl, int warp, int lane) {
  gemm_stage<true>(st, ca, ctl_s, ring, vec_s, stage_s, rs, ctl, warp, lane);
}
__device__ __noinline__ void ln_stage_ool(const Stage& st, const MegaParams& p, SmemCtl& cs, uint32_t ring, uint8_t* ring_ptr,
                                          __half* vec_s, RoleState& rs, const WaitCtl& ctl, int warp, int lane) {
  ln_stage<true>(st, p, cs, ring, ring_ptr, vec_s, rs, ctl, warp, lane);
}

// Intermediates that the previous stage read for the last time (the barrier behind it has been passed by every CTA):
// this CTA's share of their lines is dropped from L2 before anything evicts them to DRAM.  Out of line: a few
// instructions per thread and stage, whose registers are not charged to the stages.
// Threads tid0 .. kThreads - 1 of every CTA share the work: all of them in front of a LayerNorm stage, the two spare
// warps alone in front of the other stages, whose roles then start without it.
__device__ __noinline__ void drop_dead_buffers(const Stage& st, int tid0) {
  const int nthr = kThreads - tid0, tid = (int)threadIdx.x - tid0;
#pragma unroll 1
  for (int b = 0; b < 2; ++b) {
    const uint32_t lines = st.dead_bytes[b] >> 7;
    if (!lines) continue;
    const char* base = reinterpret_cast<const char*>(st.dead_ptr[b]);
    for (uint32_t i = blockIdx.x * nthr + tid; i < lines; i += gridDim.x * nthr) discard_l2_128(base + ((size_t)i << 7));
  }
}

template <int kFamily>
__global__ void __launch_bounds__(kThreads, 1)
souffle_megakernel(const __grid_constant__ CallArgs ca) {
  const MegaParams& p = ca.p;
  extern __shared__ uint8_t smem_raw[];
  if (p.prof && threadIdx.x == 0) {
    long long* pr = p.prof + ((size_t)p.n_stages * gridDim.x + blockIdx.x) * kProfSlots;
    pr[0] = clock64();
    pr[3] = (long long)globaltimer_ns();        // wall clock shared by all SMs: launch skew between CTAs
  }
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;      // 1024-byte alignment for swizzled tiles
  SmemCtl& cs = *reinterpret_cast<SmemCtl*>(smem_raw + pad);
  uint8_t* ring_ptr = smem_raw + pad + kCtlBytes;
  __half* vec_s = reinterpret_cast<__half*>(ring_ptr + kRingBytes);
  uint8_t* stage_s = ring_ptr + kRingBytes + kVecBytes;
  const uint32_t ring = raw + pad + kCtlBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxSlots; ++i) {
      mbar_init(smem_u32(&cs.full[i]), 1);
      mbar_init(smem_u32(&cs.empty[i]), 1);
    }
    constexpr bool kPairK = kFamily == kFamilyBertPair;
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&cs.tmem_full[i]), 1);
      // arrivals of the epilogue: every thread, or (pairs) one per epilogue warp of both CTAs on the leader's barrier
      mbar_init(smem_u32(&cs.tmem_empty[i]), kPairK ? 2 * kEpiWarps : kEpiThreads);
      mbar_init(smem_u32(&cs.o_empty[i]), 8);
    }
    mbar_init(smem_u32(&cs.rec_full), 1);
    mbar_init(smem_u32(&cs.qk_full), 1);
    mbar_init(smem_u32(&cs.qk_empty), 1);
    mbar_init(smem_u32(&cs.v_full), 1);
    mbar_init(smem_u32(&cs.v_empty), 1);
    mbar_init(smem_u32(&cs.s_full), 1);
    mbar_init(smem_u32(&cs.p_full), kPairK ? 8 : 128);         // softmax threads, or (pairs) the softmax warps of both CTAs
    mbar_init(smem_u32(&cs.o_full), 1);
    for (int i = 0; i < 7; ++i) mbar_init(smem_u32(&cs.attn1[i]), i == 5 ? (kPairK ? 8 : 128) : 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&cs.ln_full[i]), 1);
      mbar_init(smem_u32(&cs.ln_empty[i]), kThreads / 32 - 1);
    }
    cs.abort = 0;
    cs.deadline_ns = globaltimer_ns() + p.timeout_ns;
    fence_mbar_init();
    if (blockIdx.x == 0) {          // the other launch parity's barrier words start clean
      p.sync_next[0] = 0u;
      p.sync_next[1] = 0u;
    }
  }
  if constexpr (kFamily == kFamilyBertPair) {
    if (warp == 1) tmem_alloc_pair(smem_u32(&cs.tmem_base), kTmemCols);
  } else {
    if (warp == 1) tmem_alloc(smem_u32(&cs.tmem_base), kTmemCols);
  }
  if (warp >= 2 && p.maps) {               // warm the descriptor cache while the CTA sets up
    for (int i = (int)threadIdx.x - 64; i < p.n_maps; i += kThreads - 64) tma_prefetch_desc(p.maps + i);
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kFamily == kFamilyBertPair) cluster_sync_all();     // the peer's barriers exist before anything arrives on them
  tc_fence_after_sync();

  WaitCtl ctl;
  ctl.abort_smem = &cs.abort;
  ctl.status_g = p.status;
  ctl.deadline_ns = cs.deadline_ns;
  if (p.prof && threadIdx.x == 0) {          // one record past the stages: kernel entry, prologue done, ...
    long long* pr = p.prof + ((size_t)p.n_stages * gridDim.x + blockIdx.x) * kProfSlots;
    pr[1] = clock64();
  }

  RoleState rs;
  for (int si = 0; si < p.n_stages; ++si) {
    // stage record -> shared memory (uniform, read-only afterwards).  Records of a plan-owned program arrive during
    // the barrier before the stage (grid_barrier), except the first; the stages of the plan-less entry points travel
    // in the launch parameters and are copied here.
    if (si == 0 || !p.stages) {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(p.stages ? p.stages + si : &ca.inline_stages[si]);
      uint32_t* dst = reinterpret_cast<uint32_t*>(&cs.stage);
      for (int i = threadIdx.x; i < (int)(sizeof(Stage) / 4); i += kThreads) dst[i] = src[i];
    }
    __syncthreads();
    if (p.prof && threadIdx.x == 0) p.prof[((size_t)si * gridDim.x + blockIdx.x) * kProfSlots + 0] = clock_now();
    const Stage& st = cs.stage;
    if (st.type == STAGE_LN) drop_dead_buffers(st, 0);
    else if (warp >= 2 + kEpiWarps) drop_dead_buffers(st, (2 + kEpiWarps) * 32);
    if constexpr (kFamily == kFamilySwin) {
      if (st.type == STAGE_GEMM) gemm_stage_ool(st, ca, cs, ring, vec_s, stage_s, rs, ctl, warp, lane);
      else if (st.type == STAGE_ATTN_SWIN) attn_swin_stage(st, ca, cs, ring, ring_ptr, stage_s, rs, ctl, warp, lane);
      else if (st.type == STAGE_LN) ln_stage_ool(st, p, cs, ring, ring_ptr, vec_s, rs, ctl, warp, lane);
    } else {
      if (st.type == STAGE_GEMM) {
        gemm_stage<false, kFamily == kFamilyBertPair>(st, ca, cs, ring, vec_s, stage_s, rs, ctl, warp, lane);
      } else if (st.type == STAGE_ATTN) {
        if constexpr (kFamily == kFamilyBert) attn_stage_pp<false>(st, ca, cs, ring, ring_ptr, stage_s, rs, ctl, warp, lane);
        else if constexpr (kFamily == kFamilyBertPair) attn_stage_pp<true>(st, ca, cs, ring, ring_ptr, stage_s, rs, ctl, warp, lane);
        else attn_stage(st, ca, cs, ring, ring_ptr, stage_s, rs, ctl, warp, lane);
      } else if (st.type == STAGE_LN) {
        ln_stage<false>(st, p, cs, ring, ring_ptr, vec_s, rs, ctl, warp, lane);
      }
    }
    if (si + 1 < p.n_stages) {
      if (!grid_barrier(p, ctl, si, cs)) break;
    } else {
      __syncthreads();
      if (p.prof && threadIdx.x == 0) p.prof[((size_t)si * gridDim.x + blockIdx.x) * kProfSlots + 1] = clock_now();
    }
    if (p.prof && threadIdx.x == 0) p.prof[((size_t)si * gridDim.x + blockIdx.x) * kProfSlots + 2] = clock_now();
    if (cs.abort) break;
  }

  __syncthreads();
  if (p.prof && threadIdx.x == 0) {
    long long* pr = p.prof + ((size_t)p.n_stages * gridDim.x + blockIdx.x) * kProfSlots;
    pr[2] = clock64();
    pr[4] = (long long)globaltimer_ns();
  }
  if (cs.abort) {
    // let copies that were already issued land before the CTA's shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kFamily == kFamilyBertPair) {
    cluster_sync_all();                    // both CTAs are done with the pair's tensor memory and with each other's barriers
    if (warp == 1) tmem_dealloc_pair(cs.tmem_base, kTmemCols);
  } else {
    if (warp == 1) tmem_dealloc(cs.tmem_base, kTmemCols);
  }
}

}  // namespace souffle
