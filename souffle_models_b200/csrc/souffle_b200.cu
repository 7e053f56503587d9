// Host side of libsouffle_b200.so: plan construction, tensor maps, launches, C ABI.
//
// Mirrors the host half of the reference bindings -- cpp/bert/bert_binding.cu:23-535 (allocate
// intermediates, pack kernel arguments, cooperative launch), cpp/swin_transformer/
// swin_transformer_binding.cu:62-209 and cpp/souffle_utils/cuda_utils.h:11-19,86-98 (error
// check, co-residency check) -- with set-up split from the call: buffers, repacked weights and
// the stage program are built once per plan; a forward call is one cooperative launch.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/souffle_b200.h"
#include "megakernel.cu"
#include "lstm_kernel.cu"
#include "lstm_static.cu"
#include "se_module.cu"

namespace souffle {

// ------------------------------------------------------------------------------------
// errors
// ------------------------------------------------------------------------------------
static thread_local std::string g_last_error;

static int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}
#define SF_CUDA(call)                                                                          \
  do {                                                                                         \
    cudaError_t e_ = (call);                                                                   \
    if (e_ != cudaSuccess)                                                                     \
      return fail(SOUFFLE_CUDA_ERROR, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_),  \
                  __FILE__, __LINE__);                                                         \
  } while (0)

static bool aligned16(const void* p) { return p && (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------------------------
// tensor maps (driver entry point fetched at run time: no link-time libcuda dependency)
// ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// fp16 matrix [rows][cols] (cols contiguous), box = 64 columns x box_rows rows, 128B swizzle,
// out-of-range elements read as zero.
static int make_map_uncached(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows);

// A tensor map is a pure function of (address, extents, box): the plan-less entry points, which encode four of
// them per call, keep the last few per thread.
static int make_map(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  struct Entry { const void* ptr; uint64_t rows, cols; uint32_t box; CUtensorMap map; };
  constexpr int kEntries = 16;
  static thread_local Entry cache[kEntries];
  static thread_local int used = 0, next = 0;
  for (int i = 0; i < used; ++i) {
    const Entry& e = cache[i];
    if (e.ptr == ptr && e.rows == rows && e.cols == cols && e.box == box_rows) {
      *m = e.map;
      return SOUFFLE_OK;
    }
  }
  const int rc = make_map_uncached(m, ptr, rows, cols, box_rows);
  if (rc) return rc;
  Entry& e = cache[next];
  e.ptr = ptr; e.rows = rows; e.cols = cols; e.box = box_rows; e.map = *m;
  next = (next + 1) % kEntries;
  if (used < kEntries) ++used;
  return SOUFFLE_OK;
}

static int make_map_uncached(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(SOUFFLE_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
  if (!aligned16(ptr) || (cols * 2) % 16 != 0) return fail(SOUFFLE_BAD_POINTER, "tensor map needs 16-byte alignment");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SOUFFLE_CUDA_ERROR, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SOUFFLE_OK;
}

// fp32 planes [planes][rows][cols] as a store target: box = 16 columns x 32 rows x 1 plane (64-byte rows in shared
// memory, 64B swizzle); rows of a box past `rows` are not written.
static int make_plane_map(CUtensorMap* m, const void* ptr, uint64_t planes, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(SOUFFLE_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
  if (!aligned16(ptr) || (cols * 4) % 16 != 0) return fail(SOUFFLE_BAD_POINTER, "tensor map needs 16-byte alignment");
  cuuint64_t dims[3] = {cols, rows, planes};
  cuuint64_t strides[2] = {cols * 4, rows * cols * 4};
  cuuint32_t box[3] = {16, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SOUFFLE_CUDA_ERROR, "cuTensorMapEncodeTiled (planes) failed with CUresult %d", (int)r);
  return SOUFFLE_OK;
}

// ------------------------------------------------------------------------------------
// weight repack: [K][N] (reference layout) -> [N][K] so the B operand is K-major and any
// tile width that is a multiple of 16 can be fed to the tensor cores.  Set-up only.
// ------------------------------------------------------------------------------------
__global__ void transpose_kn_to_nk(const __half* __restrict__ src, __half* __restrict__ dst, int K, int N) {
  __shared__ __half tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int k = k0 + i, n = n0 + threadIdx.x;
    if (k < K && n < N) tile[i][threadIdx.x] = src[(size_t)k * N + n];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int n = n0 + i, k = k0 + threadIdx.x;
    if (k < K && n < N) dst[(size_t)n * K + k] = tile[threadIdx.x][i];
  }
}

// ------------------------------------------------------------------------------------
// tiling choice: a small cycle model of one CTA, fitted to the in-kernel stage profile on a B200.
// A K chunk costs the larger of its tensor-core time (bm*bn/64 cycles) and its shared-memory traffic
// (operands written once by TMA and read by the tensor core, B once per 128-row half, at 128 B/clk).
// The epilogue of a 128-row tile overlaps the next tile's main loop but competes with it; with
// 256-row tiles it is exposed.  Tiles run in waves over the SMs; split-K pays for its fp32 planes
// (written by the GEMM, re-read by the LayerNorm stage).
// ------------------------------------------------------------------------------------
struct TileChoice {
  int bm = 128, bn = 0, split = 1;
};
struct RankedTile {
  double cost;
  TileChoice t;
};
static TileChoice choose_tiles(int M, int N, int K, int sms, bool allow_split, bool b_mn, int head_split = 0,
                               std::vector<RankedTile>* ranked = nullptr) {
  const int kch = K / 64;
  double best = 1e300;
  TileChoice bt;
  const int cands[8] = {256, 192, 128, 96, 64, 48, 32, 16};
  for (int bm = 128; bm <= 256; bm += 128) {
    if (bm == 256 && M <= 128) continue;
    for (int ci = 0; ci < 8; ++ci) {
      const int bn = cands[ci];
      if (N % bn) continue;
      if (b_mn && bn % 64) continue;
      if (head_split == 1 && bn != 16 && bn % 32) continue;   // 32-column epilogue chunks must not straddle a head
      if (head_split == 2 && bn % 32) continue;               // row-permuting epilogues have no 16-column path
      if (196608 / ((bm + bn) * 128) < 2) continue;
      for (int split = 1; split <= (allow_split ? 16 : 1); ++split) {
        if (kch % split) continue;
        const long items = (long)((M + bm - 1) / bm) * (N / bn) * split;
        const long waves = (items + sms - 1) / sms;
        const double smem = 2.0 * bm + (bm / 128 + 1.0) * bn, mma = bm * bn / 64.0;
        const double chunk = 1.1 * (smem > mma ? smem : mma);
        const double epilogue = bm * bn * (allow_split ? 0.2 : 0.35);      // fp32 planes need no math
        const double tile = (kch / split) * chunk + (bm == 256 ? 0.7 : 0.45) * epilogue + 1500.0;
        double cost = waves * tile;
        if (allow_split) cost += (double)split * M * N * 8.0 / sms / 12.0;
        if (ranked) {
          RankedTile r;
          r.cost = cost; r.t.bm = bm; r.t.bn = bn; r.t.split = split;
          ranked->push_back(r);
        }
        if (cost < best - 1e-9) {
          best = cost;
          bt.bm = bm; bt.bn = bn; bt.split = split;
        }
      }
    }
  }
  if (ranked) std::stable_sort(ranked->begin(), ranked->end(), [](const RankedTile& a, const RankedTile& b) { return a.cost < b.cost; });
  return bt;
}

// The same for a plan on CTA pairs: a pair owns a 256 x bn tile, each CTA loads 128 rows of A and bn/2 rows of B per
// K chunk and runs MMAs of bn/2 cycles; both accumulator buffers of a CTA alternate, so the epilogue overlaps.
static TileChoice choose_tiles_pair(int M, int N, int K, int npairs, bool allow_split, std::vector<RankedTile>* ranked = nullptr) {
  const int kch = K / 64;
  double best = 1e300;
  TileChoice bt;
  bt.bm = 256;
  const int cands[6] = {256, 192, 128, 96, 64, 32};
  for (int ci = 0; ci < 6; ++ci) {
    const int bn = cands[ci];
    if (N % bn) continue;
    for (int split = 1; split <= (allow_split ? 16 : 1); ++split) {
      if (kch % split) continue;
      const long items = (long)((M + 255) / 256) * (N / bn) * split;
      const long waves = (items + npairs - 1) / npairs;
      const double load = (16384.0 + 64.0 * bn) / 55.0, mma = 2.0 * bn;
      const double chunk = 1.05 * (load > mma ? load : mma);
      const double epilogue = 128.0 * bn * (allow_split ? 0.2 : 0.35);
      const double tile = (kch / split) * chunk + 0.45 * epilogue + 1500.0;
      double cost = waves * tile;
      if (allow_split) cost += (double)split * M * N * 8.0 / (2.0 * npairs) / 12.0;
      if (ranked) {
        RankedTile r;
        r.cost = cost; r.t.bm = 256; r.t.bn = bn; r.t.split = split;
        ranked->push_back(r);
      }
      if (cost < best - 1e-9) {
        best = cost;
        bt.bn = bn; bt.split = split;
      }
    }
  }
  if (ranked) std::stable_sort(ranked->begin(), ranked->end(), [](const RankedTile& a, const RankedTile& b) { return a.cost < b.cost; });
  return bt;
}

// ------------------------------------------------------------------------------------
// launch helper shared by every entry point
// ------------------------------------------------------------------------------------
struct DeviceInfo {
  int device = -1, sms = 0, cc_major = 0, max_ctas = 0;
  int max_pairs = 0;             // clusters of two CTAs of the pair build that can be resident at once
  int pair_coop = 1;             // the pair launch still carries the cooperative attribute on top of the cluster dimension
  bool attr_set = false;
};
static DeviceInfo g_dev[16];

static int device_info(DeviceInfo** out) {
  int dev = 0;
  SF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return fail(SOUFFLE_BAD_DEVICE, "device index %d out of range", dev);
  DeviceInfo& d = g_dev[dev];
  if (d.device < 0) {
    SF_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
    SF_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    if (d.cc_major != 10)
      return fail(SOUFFLE_BAD_DEVICE, "device %d has compute capability %d.x; this library needs sm_100", dev, d.cc_major);
    const void* fns[3] = {(const void*)souffle_megakernel<kFamilyBert>, (const void*)souffle_megakernel<kFamilyBertCoop>,
                          (const void*)souffle_megakernel<kFamilySwin>};
    int per_sm = 1 << 30;
    for (const void* fn : fns) {
      SF_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      int n = 0;
      SF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, kThreads, kSmemBytes));
      if (n < per_sm) per_sm = n;
    }
    d.max_ctas = per_sm * d.sms;
    if (d.max_ctas < 1) return fail(SOUFFLE_NOT_CORESIDENT, "megakernel does not fit on an SM of device %d", dev);
    {   // the build that runs on CTA pairs: how many clusters of two fit the device at once
      const void* pf = (const void*)souffle_megakernel<kFamilyBertPair>;
      SF_CUDA(cudaFuncSetAttribute(pf, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
      cudaLaunchConfig_t cfg;
      cudaLaunchAttribute at[1];
      memset(&cfg, 0, sizeof(cfg));
      cfg.gridDim = dim3(2 * d.sms);
      cfg.blockDim = dim3(kThreads);
      cfg.dynamicSmemBytes = kSmemBytes;
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      cfg.attrs = at;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, pf, &cfg) != cudaSuccess) {
        cudaGetLastError();
        clusters = 0;
      }
      d.max_pairs = clusters;
    }
    d.device = dev;
  }
  *out = &d;
  return SOUFFLE_OK;
}

// `family` selects the build of the kernel (see souffle_megakernel).
static int launch_mega(const CallArgs& args_in, int grid, cudaStream_t stream, int family = kFamilyBert) {
  CallArgs args = args_in;
  for (int i = 0; i < 3; ++i) args.inline_stages[i].prof_index = i;      // stages that travel in the launch parameters
  void* kargs[] = {&args};
  if (family == kFamilyBertPair) {
    // Clusters of two CTAs.  All CTAs must be resident at once (the grid barrier): the grid never exceeds what
    // cudaOccupancyMaxActiveClusters reported, every device-side wait is bounded, and the cooperative attribute
    // adds the driver's own check where it accepts the combination (SOUFFLE_PAIR_COOPERATIVE=0 leaves it out:
    // Nsight Compute cannot capture a launch that carries both attributes).
    DeviceInfo* di = nullptr;
    int rc = device_info(&di);
    if (rc) return rc;
    static const bool env_coop = []() { const char* e = getenv("SOUFFLE_PAIR_COOPERATIVE"); return !(e && e[0] == '0'); }();
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeCooperative;
    at[1].val.cooperative = 1;
    cfg.attrs = at;
    const void* fn = (const void*)souffle_megakernel<kFamilyBertPair>;
    if (env_coop && di->pair_coop) {
      cfg.numAttrs = 2;
      if (cudaLaunchKernelExC(&cfg, fn, kargs) == cudaSuccess) return SOUFFLE_OK;
      cudaGetLastError();          // a refused launch configuration is not sticky
      di->pair_coop = 0;
    }
    cfg.numAttrs = 1;
    SF_CUDA(cudaLaunchKernelExC(&cfg, fn, kargs));
    return SOUFFLE_OK;
  }
  const void* fn = family == kFamilySwin ? (const void*)souffle_megakernel<kFamilySwin>
                   : family == kFamilyBertCoop ? (const void*)souffle_megakernel<kFamilyBertCoop>
                                               : (const void*)souffle_megakernel<kFamilyBert>;
  SF_CUDA(cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), kargs, (size_t)kSmemBytes, stream));
  return SOUFFLE_OK;
}

// Work items of a stage; for a plan on CTA pairs GEMM tiles and attention couples are per PAIR (bm = 256).
static int stage_items(const Stage& s, bool pair = false) {
  if (s.type == STAGE_GEMM) return ((s.M + s.bm - 1) / s.bm) * (s.N / s.bn) * s.splitk;
  if (s.type == STAGE_ATTN && pair) return s.batch * s.heads / 2;
  if (s.type == STAGE_ATTN) return s.batch * s.heads * ((s.seq + 127) / 128);
  if (s.type == STAGE_ATTN_SWIN) return s.batch * (s.seq / s.win) * (s.seq / s.win) * s.heads;
  return (s.M + kThreads / 32 - 2) / (kThreads / 32 - 1);       // one row per normalising warp (all warps but the first)
}

// Fills the derived fields of a GEMM stage (tile counts, ring geometry, magic divisors) and checks that its
// output fits the kernel's 32-bit element offsets.
static int finalize_stage(Stage& s, int max_slots, int grid, bool pair = false) {
  if (s.type == STAGE_LN) {
    // Rows per batch: up to 96 KB (two batches in flight), at most two rows per normalising warp, and few
    // enough that every CTA gets work.  The per-column vectors are staged in shared memory when a CTA
    // normalises enough rows to pay for the copy.
    const int comp = kThreads / 32 - 1;
    const bool has_resid = s.resid != nullptr || s.resid_sel != PTR_PLAN;
    const int row_bytes = (s.n_partial * 4 + (has_resid ? 2 : 0)) * s.N;
    int rb = 98304 / row_bytes;
    rb = rb > 2 * comp ? 2 * comp : (rb < 1 ? 1 : rb);
    int per_cta = (s.M + grid - 1) / grid;
    if (rb > per_cta) rb = per_cta;
    if (rb > comp) rb -= rb % comp;
    s.bm = rb;
    s.slot_bytes = rb * row_bytes;
    s.nslots = 196608 / s.slot_bytes > 4 ? 4 : 196608 / s.slot_bytes;
    s.items = (s.M + rb - 1) / rb;
    s.kchunks = (3 * s.N * 2 <= kVecBytes) ? 1 : 0;
    // Rows of up to 1024 columns that need no gather: the warps read their rows from L2 themselves, one row per
    // normalising warp and pass (no staging ring).  Measured faster than the ring at every batch size: twelve layers
    // at 16 sequences 0.87 against 0.93 ms, equal at 64.
    if (s.seq == 0 && s.N <= 1024) {
      if (per_cta > comp + 1) per_cta = comp + 1;       // every warp takes a row
      s.bm = per_cta;
      s.items = (s.M + per_cta - 1) / per_cta;
      s.nslots = 0;
      s.kchunks = 0;
      return SOUFFLE_OK;
    }
    if (s.nslots < 1) return fail(SOUFFLE_BAD_SHAPE, "LayerNorm rows of %d bytes do not fit the staging ring", row_bytes);
    return SOUFFLE_OK;
  }
  if (s.type == STAGE_ATTN_SWIN) {
    // The extents the window-attention stage relies on: a window's tokens fit the 64 rows of its Q/K/V/P tiles,
    // one head's column of the relative-position table fits the staging area as fp32, the two heads of a
    // 64-column pair exist, and the window-major buffers hold whole 64-row windows.
    const int tbl = 2 * s.win - 1;
    if (s.win < 1 || s.win * s.win > 64 || s.seq % s.win || tbl * tbl * 4 > kStageBytes || s.head_dim != 32 || (s.heads & 1) ||
        s.heads * 32 != s.ldo || s.shift < 0 || s.shift >= s.win)
      return fail(SOUFFLE_BAD_SHAPE, "window attention: window %d, grid %d, heads %d, row length %d are outside what the stage addresses",
                  s.win, s.seq, s.heads, s.ldo);
    return SOUFFLE_OK;
  }
  if (s.type != STAGE_GEMM) return SOUFFLE_OK;
  if ((s.epi == EPI_SWIN_QKV || s.epi == EPI_SWIN_PROJ) &&
      (s.win < 1 || s.win * s.win > 64 || s.seq % s.win || s.heads * 32 != s.ldo ||
       s.M != (s.epi == EPI_SWIN_QKV ? s.batch * s.seq * s.seq : s.batch * (s.seq / s.win) * (s.seq / s.win) * 64)))
    return fail(SOUFFLE_BAD_SHAPE, "window-major epilogue: %d rows do not match batch %d, grid %d, window %d", s.M, s.batch, s.seq, s.win);
  if (s.bias && s.epi != EPI_PARTIAL && s.N * 4 > kVecBytes)
    return fail(SOUFFLE_BAD_SHAPE, "a GEMM stage with a bias vector is limited to %d output columns (got %d)", kVecBytes / 4, s.N);
  s.tiles_n = s.N / s.bn;
  s.kchunks = s.K / 64 / s.splitk;
  s.items = stage_items(s);
  // per CTA and K chunk: the A rows (all of the tile's, or one 128-row half of a pair's) and the B rows (all, or half)
  s.slot_bytes = pair ? 16384 + s.bn * 64 : (s.bm / 128) * 16384 + s.bn * 128;
  int n = 196608 / s.slot_bytes;
  if (n > 8) n = 8;
  if (max_slots > 0 && n > max_slots) n = max_slots;
  s.nslots = n;
  s.mg_splitk = fast_div_magic((uint32_t)s.splitk);
  s.mg_tiles_n = fast_div_magic((uint32_t)s.tiles_n);
  s.mg_kchunks = fast_div_magic((uint32_t)s.kchunks);
  s.mg_seq = fast_div_magic((uint32_t)(s.seq > 0 ? s.seq : 1));
  s.mg_head_dim = fast_div_magic((uint32_t)(s.head_dim > 0 ? s.head_dim : 1));
  s.mg_heads = fast_div_magic((uint32_t)(s.heads > 0 ? s.heads : 1));
  const unsigned long long out_elems = (unsigned long long)s.M * (unsigned long long)s.N * (s.epi == EPI_PARTIAL ? s.splitk : 1);
  // 2^20 rows keep every multiply-high division exact (numerator * divisor < 2^32)
  if (s.M > (1 << 20) || out_elems * (s.epi == EPI_SWIN_QKV ? 2 : 1) >= 0xFFFF0000ull || (long long)s.items * 16 >= (1ll << 32))
    return fail(SOUFFLE_BAD_SHAPE, "GEMM stage %d x %d (split %d) is too large for 32-bit output offsets", s.M, s.N, s.splitk);
  return SOUFFLE_OK;
}

static int decode_status(const int* h, const char* what) {
  if (h[0] == DEV_OK) return SOUFFLE_OK;
  return fail(SOUFFLE_DEVICE_TIMEOUT, "%s: device wait expired (code %d, where %d, cta %d)", what, h[0], h[1], h[2]);
}

}  // namespace souffle

using namespace souffle;

// ======================================================================================
// BERT plan
// ======================================================================================
struct SouffleBertPlan {
  SouffleBertDesc desc;
  int device = 0, grid = 0, launches = 0;
  int family = 0;                // which build of the kernel runs this plan (kFamilyBert / kFamilyBertCoop / kFamilyBertPair)
  bool pair = false;             // the plan runs on CTA pairs: 256-row tiles, half a B tile per CTA
  unsigned launch_id = 0;
  std::vector<Stage> stages;
  std::vector<const void*> stage_weights;   // per stage: the repacked [N][K] weight matrix of a GEMM stage, else null
  struct Dead { size_t after_stage; const void* ptr; uint32_t bytes; };
  std::vector<Dead> dead_after;             // buffers nobody reads again once stage `after_stage` has run
  std::vector<CUtensorMap> maps;
  std::vector<void*> allocs;
  Stage* d_stages = nullptr;
  CUtensorMap* d_maps = nullptr;
  unsigned* d_sync = nullptr;   // two (count, generation) pairs
  int* d_status = nullptr;
  long long* d_prof = nullptr;
  // plan-owned activations
  __half *qkv = nullptr, *ctx = nullptr, *ln1 = nullptr, *fc1 = nullptr, *probs = nullptr, *act[2] = {nullptr, nullptr};
  float* partial = nullptr;
  // host-buffer path
  // host-buffer path: two sets of device buffers and three streams, so that consecutive calls overlap their
  // copies with one another's compute (copy-in of call i+1 and copy-out of call i-1 run under the kernel of call i)
  __half *x_dev[2] = {nullptr, nullptr}, *y_dev[2] = {nullptr, nullptr};
  int* lens_dev[2] = {nullptr, nullptr};
  cudaStream_t s_in = nullptr, s_cmp = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_k[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
  unsigned host_calls = 0;
  // per-call map cache for x
  const void* last_x = nullptr;
  CUtensorMap x_map;
  int x_box_rows = 128;
};

namespace souffle {

static int plan_alloc(SouffleBertPlan* p, void** ptr, size_t bytes);

// Numbers the stages and copies the program and its tensor maps to the device.
static int upload_program(SouffleBertPlan* p) {
  int rc;
  for (size_t i = 0; i < p->stages.size(); ++i) {
    Stage& s = p->stages[i];
    s.prof_index = (int)i;
    // the weights of the GEMM stage after next are prefetched into L2 at the barrier that ends this stage
    s.pf_ptr = nullptr;
    s.pf_bytes = 0;
    if (i + 2 < p->stages.size() && p->stages[i + 2].type == STAGE_GEMM && p->stage_weights.size() > i + 2 && p->stage_weights[i + 2]) {
      const Stage& g = p->stages[i + 2];
      s.pf_ptr = p->stage_weights[i + 2];
      s.pf_bytes = (uint32_t)((size_t)g.N * g.K * 2) & ~15u;
    }
    s.dead_bytes[0] = s.dead_bytes[1] = 0;
    s.dead_ptr[0] = s.dead_ptr[1] = nullptr;
  }
  for (const SouffleBertPlan::Dead& dd : p->dead_after) {
    if (dd.after_stage + 1 >= p->stages.size()) continue;          // nothing runs after it inside the launch
    Stage& nx = p->stages[dd.after_stage + 1];
    const int k = nx.dead_bytes[0] ? 1 : 0;
    if (nx.dead_bytes[k]) continue;                                // both slots taken: the buffer is written back as before
    nx.dead_ptr[k] = dd.ptr;
    nx.dead_bytes[k] = dd.bytes;
  }
  if ((rc = plan_alloc(p, (void**)&p->d_stages, p->stages.size() * sizeof(Stage)))) return rc;
  if ((rc = plan_alloc(p, (void**)&p->d_maps, p->maps.size() * sizeof(CUtensorMap)))) return rc;
  SF_CUDA(cudaMemcpy(p->d_stages, p->stages.data(), p->stages.size() * sizeof(Stage), cudaMemcpyHostToDevice));
  SF_CUDA(cudaMemcpy(p->d_maps, p->maps.data(), p->maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice));
  SF_CUDA(cudaDeviceSynchronize());
  return SOUFFLE_OK;
}

static int plan_alloc(SouffleBertPlan* p, void** ptr, size_t bytes) {
  SF_CUDA(cudaMalloc(ptr, bytes));
  p->allocs.push_back(*ptr);
  return SOUFFLE_OK;
}

static int add_map(SouffleBertPlan* p, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, int* idx) {
  if ((int)p->maps.size() >= kMaxTensorMaps) return fail(SOUFFLE_BAD_SHAPE, "too many tensor maps");
  CUtensorMap m;
  int rc = make_map(&m, ptr, rows, cols, box_rows);
  if (rc) return rc;
  *idx = (int)p->maps.size();
  p->maps.push_back(m);
  return SOUFFLE_OK;
}

// The store map of a split-K GEMM stage's planes (see make_plane_map); sets the stage's tm_out / out_tma.
static int add_plane_map(SouffleBertPlan* p, Stage& s) {
  if ((int)p->maps.size() >= kMaxTensorMaps) return fail(SOUFFLE_BAD_SHAPE, "too many tensor maps");
  if (s.N % 16) return SOUFFLE_OK;                     // (cannot happen: tile widths are multiples of 16) plain stores
  CUtensorMap m;
  int rc = make_plane_map(&m, s.partial, (uint64_t)s.splitk, (uint64_t)s.M, (uint64_t)s.N);
  if (rc) return rc;
  s.out_tma = 1;
  for (size_t i = 0; i < p->maps.size(); ++i)          // the layers of a stack share their planes: one map serves them all
    if (memcmp(&p->maps[i], &m, sizeof(m)) == 0) {
      s.tm_out = (int)i;
      return SOUFFLE_OK;
    }
  s.tm_out = (int)p->maps.size();
  p->maps.push_back(m);
  return SOUFFLE_OK;
}

// Marks `ptr` (`bytes` long) as dead once the stage just appended has run: the stage appended NEXT drops its lines from
// L2.  Kept in a side table until the program is complete (see upload_program).
static void note_dead(SouffleBertPlan* p, const void* ptr, size_t bytes) {
  if (!ptr || bytes < 128 || bytes >= (1ull << 32) || (reinterpret_cast<uintptr_t>(ptr) & 127u)) return;
  p->dead_after.push_back({p->stages.size() - 1, ptr, (uint32_t)(bytes & ~(size_t)127)});
}

// Remembers the weight matrix of the stage just appended (for the L2 prefetch, see upload_program).
static void note_weights(SouffleBertPlan* p, const void* w) {
  p->stage_weights.resize(p->stages.size(), nullptr);
  p->stage_weights.back() = w;
}

static Stage blank_stage(int type) {
  Stage s;
  memset(&s, 0, sizeof(s));
  s.type = type;
  s.splitk = 1;
  s.bm = 128;
  s.n_partial = 0;
  return s;
}

// Times the likeliest tilings of one GEMM stage on the device and returns the fastest.  `proto` is the stage as
// the plan will build it (shape, epilogue, output pointers) without tile fields; its operands are read through
// per-call tensor maps over `a` ([M][K]) and `w` ([N][K]), whose contents do not matter for the timing.  A stage
// that writes split-K planes is timed together with the LayerNorm stage that sums them (`ln_proto`), since more
// planes make that one slower.  Failures of any kind leave `*choice` as the cycle model set it.
static void autotune_gemm(const Stage& proto, const Stage* ln_proto, const void* a, const void* w, int sms, bool allow_split,
                          int head_split, int max_split, void* tune_ws, TileChoice* choice, bool pair = false) {
  std::vector<RankedTile> ranked;
  if (pair) choose_tiles_pair(proto.M, proto.N, proto.K, sms / 2, allow_split, &ranked);
  else choose_tiles(proto.M, proto.N, proto.K, sms, allow_split, false, head_split, &ranked);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return;
  float best_ms = 1e30f;
  int measured = 0;
  for (size_t ci = 0; ci < ranked.size() && measured < 16; ++ci) {
    const TileChoice t = ranked[ci].t;
    if (t.split > max_split) continue;
    CallArgs args;
    memset(&args, 0, sizeof(args));
    Stage& g = args.inline_stages[0];
    g = proto;
    g.tm_a = -1; g.tm_b = -2; g.bm = t.bm; g.bn = t.bn; g.splitk = t.split;
    if (finalize_stage(g, 0, 1, pair)) continue;
    if (make_map_uncached(&args.call_maps[0], a, (uint64_t)proto.M, (uint64_t)proto.K, (uint32_t)(pair ? 128 : t.bm))) continue;
    if (make_map_uncached(&args.call_maps[1], w, (uint64_t)proto.N, (uint64_t)proto.K, (uint32_t)(pair ? t.bn / 2 : t.bn))) continue;
    if (g.epi == EPI_PARTIAL) {
      if (make_plane_map(&args.call_maps[2], g.partial, (uint64_t)t.split, (uint64_t)proto.M, (uint64_t)proto.N)) continue;
      g.tm_out = -3;
      g.out_tma = 1;
    }
    int items = stage_items(g) * (pair ? 2 : 1);                // CTAs that have work
    args.p.n_stages = 1;
    if (ln_proto) {
      Stage& ln = args.inline_stages[1];
      ln = *ln_proto;
      ln.n_partial = t.split;
      const int li = stage_items(ln);
      if (li > items) items = li;
      args.p.n_stages = 2;
    }
    const int grid = items < sms ? items : sms;                 // even for pairs: items and sms both are
    if (ln_proto && finalize_stage(args.inline_stages[1], 0, grid)) continue;
    args.p.sync = reinterpret_cast<unsigned*>(tune_ws);
    args.p.sync_next = args.p.sync + 2;
    args.p.status = reinterpret_cast<int*>(reinterpret_cast<char*>(tune_ws) + 64);
    args.p.timeout_ns = 200ull * 1000000ull;
    bool ok = true;
    for (int it = 0; it < 26 && ok; ++it) {                // two warm-up launches, twenty-four timed ones
      ok = cudaMemsetAsync(tune_ws, 0, 128, nullptr) == cudaSuccess;
      if (it == 2) ok = ok && cudaEventRecord(e0, nullptr) == cudaSuccess;
      ok = ok && launch_mega(args, grid, nullptr, pair ? kFamilyBertPair : kFamilyBert) == SOUFFLE_OK;
    }
    float ms = 0.0f;
    int h[4] = {0, 0, 0, 0};
    ok = ok && cudaEventRecord(e1, nullptr) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess &&
         cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess &&
         cudaMemcpy(h, reinterpret_cast<char*>(tune_ws) + 64, sizeof(h), cudaMemcpyDeviceToHost) == cudaSuccess && h[0] == DEV_OK;
    if (!ok) {
      cudaGetLastError();
      continue;
    }
    ++measured;
    if (ms < best_ms) {
      best_ms = ms;
      *choice = t;
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
}

static int build_bert_plan(SouffleBertPlan* p, const SouffleBertLayerWeights* layers) {
  const SouffleBertDesc& d = p->desc;
  DeviceInfo* di = nullptr;
  int rc = device_info(&di);
  if (rc) return rc;
  p->device = di->device;
  const int B = d.batch, S = d.seq, Hh = d.heads, hd = d.head_dim, H = Hh * hd, F = d.ffn, M = B * S, L = d.n_layers;
  const bool std_variant = d.variant == SOUFFLE_BERT_STD;
  const float scale = std_variant ? 1.0f / sqrtf((float)hd) : 1.0f / sqrtf((float)H);
  int sms = di->sms;
  if (d.max_ctas > 0 && d.max_ctas < sms) sms = d.max_ctas;
  if (sms > di->max_ctas) sms = di->max_ctas;
  // CTA pairs (opt-in): for shapes whose GEMM stages have many tiles per CTA and whose attention stage has more
  // (sequence, head) items than CTAs (its two-pipeline form, which the pair build has; the one-item form exists for
  // single CTAs only)
  int npairs = sms / 2 < di->max_pairs ? sms / 2 : di->max_pairs;
  const bool pair = d.pair_mma == 1 && npairs >= 1 && S <= 128 && Hh % 2 == 0 && B * Hh > sms && M >= 2048;
  p->pair = pair;
  if (pair) sms = 2 * npairs;

  // ---- buffers ----
  if ((rc = plan_alloc(p, (void**)&p->qkv, (size_t)3 * M * H * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&p->ctx, (size_t)M * H * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&p->ln1, (size_t)M * H * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&p->fc1, (size_t)M * F * 2))) return rc;
  if (L > 1) {
    if ((rc = plan_alloc(p, (void**)&p->act[0], (size_t)M * H * 2))) return rc;
    if (L > 2 && (rc = plan_alloc(p, (void**)&p->act[1], (size_t)M * H * 2))) return rc;
  }
  if (d.keep_probs) {
    if ((rc = plan_alloc(p, (void**)&p->probs, (size_t)B * Hh * S * S * 2))) return rc;
  }
  if ((rc = plan_alloc(p, (void**)&p->d_sync, 64))) return rc;
  if ((rc = plan_alloc(p, (void**)&p->d_status, 64))) return rc;
  SF_CUDA(cudaMemset(p->d_sync, 0, 64));
  SF_CUDA(cudaMemset(p->d_status, 0, 64));

  // ---- tiling ----
  TileChoice t_qkv = choose_tiles(M, 3 * H, H, sms, false, false, 1), t_fc1 = choose_tiles(M, F, H, sms, false, false),
             t_proj = choose_tiles(M, H, H, sms, true, false), t_fc2 = choose_tiles(M, H, F, sms, true, false);
  if (pair) {
    t_qkv = choose_tiles_pair(M, 3 * H, H, npairs, false);
    t_fc1 = choose_tiles_pair(M, F, H, npairs, false);
    t_proj = choose_tiles_pair(M, H, H, npairs, true);
    t_fc2 = choose_tiles_pair(M, H, F, npairs, true);
  }
  if (d.bm_qkv) t_qkv.bm = d.bm_qkv;
  if (d.bn_qkv) t_qkv.bn = d.bn_qkv;
  if (d.bm_fc1) t_fc1.bm = d.bm_fc1;
  if (d.bn_fc1) t_fc1.bn = d.bn_fc1;
  if (d.bm_proj) t_proj.bm = d.bm_proj;
  if (d.bn_proj) t_proj.bn = d.bn_proj;
  if (d.split_proj) t_proj.split = d.split_proj;
  if (d.bm_fc2) t_fc2.bm = d.bm_fc2;
  if (d.bn_fc2) t_fc2.bn = d.bn_fc2;
  if (d.split_fc2) t_fc2.split = d.split_fc2;
  if (d.autotune) {
    // Scratch for the measurements: a weight-shaped operand, as many fp32 planes as the deepest split tried
    // (capped at 256 MB), barrier words.  Activation-shaped operands are the plan's own buffers.
    const size_t w_bytes = (size_t)(3 * H > F ? 3 * H : F) * H * 2;
    int max_split = (int)((256ull << 20) / ((size_t)M * H * 4));
    max_split = max_split > 16 ? 16 : (max_split < 1 ? 1 : max_split);
    void *w_tmp = nullptr, *planes = nullptr, *tune_ws = nullptr;
    if (cudaMalloc(&w_tmp, w_bytes) == cudaSuccess && cudaMalloc(&planes, (size_t)max_split * M * H * 4) == cudaSuccess &&
        cudaMalloc(&tune_ws, 256) == cudaSuccess && cudaMemset(w_tmp, 0, w_bytes) == cudaSuccess) {
      Stage ln = blank_stage(STAGE_LN);
      ln.M = M; ln.N = H; ln.ldo = H; ln.partial = reinterpret_cast<float*>(planes); ln.resid = p->ctx; ln.out = p->ln1;
      ln.eps = d.eps;
      Stage g = blank_stage(STAGE_GEMM);
      g.M = M; g.batch = B; g.heads = Hh; g.seq = S; g.head_dim = hd;
      if (!d.bm_qkv && !d.bn_qkv) {
        Stage q = g;
        q.N = 3 * H; q.K = H; q.epi = EPI_QKV; q.out = p->qkv; q.ldo = H;
        autotune_gemm(q, nullptr, p->ln1, w_tmp, sms, false, 1, 1, tune_ws, &t_qkv, pair);
      }
      if (!d.bm_fc1 && !d.bn_fc1) {
        Stage f = g;
        f.N = F; f.K = H; f.epi = EPI_F16; f.act = std_variant ? ACT_GELU : ACT_RELU; f.out = p->fc1; f.ldo = F;
        autotune_gemm(f, nullptr, p->ln1, w_tmp, sms, false, 0, 1, tune_ws, &t_fc1, pair);
      }
      if (!d.bm_proj && !d.bn_proj && !d.split_proj) {
        Stage f = g;
        f.N = H; f.K = H; f.epi = EPI_PARTIAL; f.partial = reinterpret_cast<float*>(planes); f.ldo = H;
        autotune_gemm(f, &ln, p->ctx, w_tmp, sms, true, 0, max_split, tune_ws, &t_proj, pair);
      }
      if (!d.bm_fc2 && !d.bn_fc2 && !d.split_fc2) {
        Stage f = g;
        f.N = H; f.K = F; f.epi = EPI_PARTIAL; f.partial = reinterpret_cast<float*>(planes); f.ldo = H;
        autotune_gemm(f, &ln, p->fc1, w_tmp, sms, true, 0, max_split, tune_ws, &t_fc2, pair);
      }
    }
    cudaDeviceSynchronize();
    cudaGetLastError();
    if (w_tmp) cudaFree(w_tmp);
    if (planes) cudaFree(planes);
    if (tune_ws) cudaFree(tune_ws);
  }
  if (pair) t_qkv.bm = t_fc1.bm = t_proj.bm = t_fc2.bm = 256;      // a pair's tile is 256 rows: 128 per CTA
  auto bad_tile = [pair](const TileChoice& t, int N) {
    if (pair) return t.bn < 32 || t.bn > 256 || t.bn % 32 || N % t.bn;     // each CTA holds bn / 2 rows of the B tile
    return (t.bm != 128 && t.bm != 256) || t.bn < 16 || t.bn > 256 || t.bn % 16 || N % t.bn ||
           196608 / ((t.bm + t.bn) * 128) < 2;
  };
  if (t_qkv.bn != 16 && t_qkv.bn % 32) return fail(SOUFFLE_BAD_SHAPE, "bn_qkv must be 16 or a multiple of 32");
  if (bad_tile(t_qkv, 3 * H) || bad_tile(t_fc1, F) || bad_tile(t_proj, H) || bad_tile(t_fc2, H))
    return fail(SOUFFLE_BAD_SHAPE, "tile shapes (%dx%d, %dx%d, %dx%d, %dx%d) do not fit the layer", t_qkv.bm, t_qkv.bn,
                t_fc1.bm, t_fc1.bn, t_proj.bm, t_proj.bn, t_fc2.bm, t_fc2.bn);
  if (t_proj.split < 1 || t_fc2.split < 1 || t_proj.split > 16 || t_fc2.split > 16 || (H / 64) % t_proj.split ||
      (F / 64) % t_fc2.split)
    return fail(SOUFFLE_BAD_SHAPE, "split-K factors must be in 1..16 and divide K/64");
  const int bn_qkv = t_qkv.bn, bn_fc1 = t_fc1.bn, bn_proj = t_proj.bn, sp_proj = t_proj.split, bn_fc2 = t_fc2.bn,
            sp_fc2 = t_fc2.split;
  const int max_split = sp_proj > sp_fc2 ? sp_proj : sp_fc2;
  if ((rc = plan_alloc(p, (void**)&p->partial, (size_t)max_split * M * H * 4))) return rc;
  // rows of an A box: the tile's height, or one CTA's 128-row half of a pair's tile; rows of a B box: the tile's
  // width, or one CTA's half of it
  auto a_rows = [pair](const TileChoice& t) { return (uint32_t)(pair ? 128 : t.bm); };
  auto b_rows = [pair](int bn) { return (uint32_t)(pair ? bn / 2 : bn); };
  p->x_box_rows = (int)a_rows(t_qkv);

  // ---- activation maps (A operands, box 64 x 128) ----
  int m_ctx, m_ln1, m_fc1, m_act[2] = {-1, -1}, m_qkv;
  if ((rc = add_map(p, p->ctx, M, H, a_rows(t_proj), &m_ctx))) return rc;
  if ((rc = add_map(p, p->ln1, M, H, a_rows(t_fc1), &m_ln1))) return rc;
  if ((rc = add_map(p, p->fc1, M, F, a_rows(t_fc2), &m_fc1))) return rc;
  for (int i = 0; i < 2; ++i)
    if (p->act[i] && (rc = add_map(p, p->act[i], M, H, a_rows(t_qkv), &m_act[i]))) return rc;
  if ((rc = add_map(p, p->qkv, (uint64_t)3 * B * Hh * S, hd, 128, &m_qkv))) return rc;

  // ---- per layer: repack weights, maps, stages ----
  for (int l = 0; l < L; ++l) {
    const SouffleBertLayerWeights& w = layers[l];
    if (!aligned16(w.qkv_w) || !aligned16(w.proj_w) || !aligned16(w.fc1_w) || !aligned16(w.fc2_w))
      return fail(SOUFFLE_BAD_POINTER, "layer %d: weight matrices must be non-null and 16-byte aligned", l);
    __half *wqkv_t, *wo_t, *w1_t, *w2_t;
    if ((rc = plan_alloc(p, (void**)&wqkv_t, (size_t)3 * H * H * 2))) return rc;
    if ((rc = plan_alloc(p, (void**)&wo_t, (size_t)H * H * 2))) return rc;
    if ((rc = plan_alloc(p, (void**)&w1_t, (size_t)H * F * 2))) return rc;
    if ((rc = plan_alloc(p, (void**)&w2_t, (size_t)F * H * 2))) return rc;
    const dim3 tb(32, 8);
    for (int j = 0; j < 3; ++j)
      transpose_kn_to_nk<<<dim3(H / 32, H / 32), tb>>>(reinterpret_cast<const __half*>(w.qkv_w) + (size_t)j * H * H,
                                                        wqkv_t + (size_t)j * H * H, H, H);
    transpose_kn_to_nk<<<dim3(H / 32, H / 32), tb>>>(reinterpret_cast<const __half*>(w.proj_w), wo_t, H, H);
    transpose_kn_to_nk<<<dim3(F / 32, H / 32), tb>>>(reinterpret_cast<const __half*>(w.fc1_w), w1_t, H, F);
    transpose_kn_to_nk<<<dim3(H / 32, F / 32), tb>>>(reinterpret_cast<const __half*>(w.fc2_w), w2_t, F, H);
    SF_CUDA(cudaGetLastError());
    // vectors are copied so the plan does not alias caller memory
    auto copy_vec = [&](const void* src, size_t n, const void** dst) -> int {
      *dst = nullptr;
      if (!src) return SOUFFLE_OK;
      void* v;
      int r2 = plan_alloc(p, &v, n * 2);
      if (r2) return r2;
      if (cudaMemcpy(v, src, n * 2, cudaMemcpyDeviceToDevice) != cudaSuccess)
        return fail(SOUFFLE_CUDA_ERROR, "copying a parameter vector failed");
      *dst = v;
      return SOUFFLE_OK;
    };
    const void *qkv_b, *proj_b, *ln1_g, *ln1_b, *fc1_b, *fc2_b, *ln2_g, *ln2_b;
    if ((rc = copy_vec(w.qkv_b, 3 * H, &qkv_b))) return rc;
    if ((rc = copy_vec(std_variant ? w.proj_b : nullptr, H, &proj_b))) return rc;
    if ((rc = copy_vec(std_variant ? w.ln1_g : nullptr, H, &ln1_g))) return rc;
    if ((rc = copy_vec(std_variant ? w.ln1_b : nullptr, H, &ln1_b))) return rc;
    if ((rc = copy_vec(std_variant ? w.fc1_b : nullptr, F, &fc1_b))) return rc;
    if ((rc = copy_vec(std_variant ? w.fc2_b : nullptr, H, &fc2_b))) return rc;
    if ((rc = copy_vec(std_variant ? w.ln2_g : nullptr, H, &ln2_g))) return rc;
    if ((rc = copy_vec(std_variant ? w.ln2_b : nullptr, H, &ln2_b))) return rc;
    if ((ln1_g == nullptr) != (ln1_b == nullptr) || (ln2_g == nullptr) != (ln2_b == nullptr))
      return fail(SOUFFLE_BAD_ARGUMENT, "layer %d: gamma and beta must be given together", l);

    int m_wqkv, m_wo, m_w1, m_w2;
    if ((rc = add_map(p, wqkv_t, 3 * H, H, b_rows(bn_qkv), &m_wqkv))) return rc;
    if ((rc = add_map(p, wo_t, H, H, b_rows(bn_proj), &m_wo))) return rc;
    if ((rc = add_map(p, w1_t, F, H, b_rows(bn_fc1), &m_w1))) return rc;
    if ((rc = add_map(p, w2_t, H, F, b_rows(bn_fc2), &m_w2))) return rc;

    // layer input / output routing
    const bool first = l == 0, last = l == L - 1;
    const bool keep = last && d.keep_probs;      // the last layer's stage outputs stay readable for the host (parity mode)
    const int in_map = first ? -1 : m_act[(l - 1) & 1];
    const void* in_ptr = first ? nullptr : p->act[(l - 1) & 1];
    const int in_sel = first ? PTR_CALL_X : PTR_PLAN;
    void* out_ptr = last ? nullptr : p->act[l & 1];
    const int out_sel = last ? PTR_CALL_Y : PTR_PLAN;

    Stage s = blank_stage(STAGE_GEMM);                 // QKV projection, head-split store
    s.tm_a = in_map; s.tm_b = m_wqkv; s.M = M; s.N = 3 * H; s.K = H; s.bm = t_qkv.bm; s.bn = bn_qkv;
    s.epi = EPI_QKV; s.bias = qkv_b; s.out = p->qkv; s.batch = B; s.heads = Hh; s.seq = S; s.head_dim = hd;
    p->stages.push_back(s);
    note_weights(p, wqkv_t);

    s = blank_stage(STAGE_ATTN);                       // softmax(QK^T) V
    s.tm_qkv = m_qkv; s.batch = B; s.heads = Hh; s.seq = S; s.head_dim = hd; s.scale = scale;
    s.lens_from_call = 1; s.out = p->ctx; s.probs = (last && d.keep_probs) ? p->probs : nullptr;
    p->stages.push_back(s);
    if (!keep) note_dead(p, p->qkv, (size_t)3 * M * H * 2);            // Q, K, V: read by the attention stage only

    s = blank_stage(STAGE_GEMM);                       // output projection -> fp32 partials
    s.tm_a = m_ctx; s.tm_b = m_wo; s.M = M; s.N = H; s.K = H; s.bm = t_proj.bm; s.bn = bn_proj; s.splitk = sp_proj;
    s.epi = EPI_PARTIAL; s.partial = p->partial;
    if ((rc = add_plane_map(p, s))) return rc;
    p->stages.push_back(s);
    note_weights(p, wo_t);
    if (!keep) note_dead(p, p->ctx, (size_t)M * H * 2);               // attention output: read by the projection only

    s = blank_stage(STAGE_LN);                         // + bias + residual, LayerNorm 1
    s.M = M; s.N = H; s.ldo = H; s.partial = p->partial; s.n_partial = sp_proj; s.bias = proj_b;
    s.resid = in_ptr; s.resid_sel = in_sel; s.out = p->ln1; s.gamma = ln1_g; s.beta = ln1_b; s.eps = d.eps;
    p->stages.push_back(s);
    note_dead(p, p->partial, (size_t)sp_proj * M * H * 4);             // the projection's planes
    if (!first) note_dead(p, in_ptr, (size_t)M * H * 2);               // the previous layer's output: QKV and this residual were its readers

    s = blank_stage(STAGE_GEMM);                       // FC1 + bias + activation
    s.tm_a = m_ln1; s.tm_b = m_w1; s.M = M; s.N = F; s.K = H; s.bm = t_fc1.bm; s.bn = bn_fc1;
    s.epi = EPI_F16; s.act = std_variant ? ACT_GELU : ACT_RELU; s.bias = fc1_b; s.out = p->fc1; s.ldo = F;
    p->stages.push_back(s);
    note_weights(p, w1_t);

    s = blank_stage(STAGE_GEMM);                       // FC2 -> fp32 partials
    s.tm_a = m_fc1; s.tm_b = m_w2; s.M = M; s.N = H; s.K = F; s.bm = t_fc2.bm; s.bn = bn_fc2; s.splitk = sp_fc2;
    s.epi = EPI_PARTIAL; s.partial = p->partial;
    if ((rc = add_plane_map(p, s))) return rc;
    p->stages.push_back(s);
    note_weights(p, w2_t);
    if (!keep) note_dead(p, p->fc1, (size_t)M * F * 2);               // FFN hidden layer: read by FC2 only

    s = blank_stage(STAGE_LN);                         // + bias + residual, LayerNorm 2
    s.M = M; s.N = H; s.ldo = H; s.partial = p->partial; s.n_partial = sp_fc2; s.bias = fc2_b;
    s.resid = p->ln1; s.resid_sel = PTR_PLAN; s.out = out_ptr; s.out_sel = out_sel;
    s.gamma = ln2_g; s.beta = ln2_b; s.eps = d.eps;
    p->stages.push_back(s);
    if (!last) {
      note_dead(p, p->partial, (size_t)sp_fc2 * M * H * 4);            // FC2's planes
      note_dead(p, p->ln1, (size_t)M * H * 2);                         // LayerNorm 1 output: FC1 and this residual were its readers
    }
  }
  if ((int)p->stages.size() > kMaxStages) return fail(SOUFFLE_BAD_SHAPE, "too many stages (%zu)", p->stages.size());

  int max_items = 1;
  for (const Stage& s : p->stages) {
    const int it = stage_items(s, pair) * ((pair && s.type != STAGE_LN) ? 2 : 1);      // CTAs that have work
    if (it > max_items) max_items = it;
  }
  p->grid = max_items < sms ? max_items : sms;
  if (pair) p->grid &= ~1;

  if (d.profile) {
    const size_t pb = (p->stages.size() + 1) * (size_t)p->grid * kProfSlots * sizeof(long long);
    if ((rc = plan_alloc(p, (void**)&p->d_prof, pb))) return rc;
    SF_CUDA(cudaMemset(p->d_prof, 0, pb));
  }
  // one attention item per CTA at most, or a long sequence: the stage in which all softmax warps share an item
  p->family = pair ? kFamilyBertPair : (d.seq > 128 || d.batch * d.heads <= p->grid) ? kFamilyBertCoop : kFamilyBert;
  for (Stage& fs : p->stages)
    if ((rc = finalize_stage(fs, p->desc.debug_max_slots, p->grid, pair))) return rc;
  return upload_program(p);
}

}  // namespace souffle

extern "C" {

const char* souffle_last_error(void) { return g_last_error.c_str(); }
int souffle_abi_version(void) { return 1; }

int souffle_bert_plan_create(const SouffleBertDesc* desc, const SouffleBertLayerWeights* layers,
                             SouffleBertPlan** plan_out) {
  if (!desc || !layers || !plan_out) return fail(SOUFFLE_BAD_ARGUMENT, "null argument");
  *plan_out = nullptr;
  const SouffleBertDesc& d = *desc;
  if (d.batch < 1 || d.heads < 1 || d.n_layers < 1 || d.n_layers > 12)
    return fail(SOUFFLE_BAD_SHAPE, "batch, heads must be >= 1 and 1 <= n_layers <= 12");
  if (d.head_dim != 64) return fail(SOUFFLE_BAD_SHAPE, "head_dim must be 64 (got %d)", d.head_dim);
  const bool seq_ok = (d.seq >= 16 && d.seq <= 128 && d.seq % 16 == 0) || d.seq == 256 || d.seq == 384;
  if (!seq_ok) return fail(SOUFFLE_BAD_SHAPE, "seq must be a multiple of 16 up to 128, or 256, or 384 (got %d)", d.seq);
  const int H = d.heads * d.head_dim;
  if (H != 128 && H != 256 && H != 512 && H != 768 && H != 1024)
    return fail(SOUFFLE_BAD_SHAPE, "hidden size %d must be 128, 256, 512, 768 or 1024", H);
  if (d.ffn < 64 || d.ffn % 64) return fail(SOUFFLE_BAD_SHAPE, "ffn must be a positive multiple of 64 (got %d)", d.ffn);
  if (d.variant != SOUFFLE_BERT_STD && d.variant != SOUFFLE_BERT_REF_COMPAT)
    return fail(SOUFFLE_BAD_ARGUMENT, "unknown variant %d", d.variant);
  SouffleBertPlan* p = new SouffleBertPlan();
  p->desc = d;
  int rc = build_bert_plan(p, layers);
  if (rc) {
    const std::string keep = g_last_error;
    souffle_bert_plan_destroy(p);
    g_last_error = keep;
    return rc;
  }
  *plan_out = p;
  return SOUFFLE_OK;
}

int souffle_bert_plan_destroy(SouffleBertPlan* plan) {
  if (!plan) return SOUFFLE_OK;
  cudaDeviceSynchronize();
  for (void* a : plan->allocs) cudaFree(a);
  for (int i = 0; i < 2; ++i) {
    if (plan->x_dev[i]) cudaFree(plan->x_dev[i]);
    if (plan->y_dev[i]) cudaFree(plan->y_dev[i]);
    if (plan->lens_dev[i]) cudaFree(plan->lens_dev[i]);
    if (plan->ev_in[i]) cudaEventDestroy(plan->ev_in[i]);
    if (plan->ev_k[i]) cudaEventDestroy(plan->ev_k[i]);
    if (plan->ev_out[i]) cudaEventDestroy(plan->ev_out[i]);
  }
  if (plan->s_in) cudaStreamDestroy(plan->s_in);
  if (plan->s_cmp) cudaStreamDestroy(plan->s_cmp);
  if (plan->s_out) cudaStreamDestroy(plan->s_out);
  delete plan;
  return SOUFFLE_OK;
}

int souffle_bert_forward(SouffleBertPlan* plan, const void* x, const int32_t* seq_lens, void* y,
                         souffle_stream_t stream) {
  if (!plan) return fail(SOUFFLE_BAD_ARGUMENT, "null plan");
  if (!aligned16(x) || !aligned16(y)) return fail(SOUFFLE_BAD_POINTER, "x and y must be non-null and 16-byte aligned");
  const SouffleBertDesc& d = plan->desc;
  const int M = d.batch * d.seq, H = d.heads * d.head_dim;
  if (x != plan->last_x) {
    int rc = make_map(&plan->x_map, x, M, H, (uint32_t)plan->x_box_rows);
    if (rc) return rc;
    plan->last_x = x;
  }
  CallArgs args;
  memset(&args, 0, sizeof(args));
  args.call_maps[0] = plan->x_map;
  MegaParams& mp = args.p;
  mp.stages = plan->d_stages;
  mp.n_stages = (int)plan->stages.size();
  mp.maps = plan->d_maps;
  mp.n_maps = (int)plan->maps.size();
  mp.x = x;
  mp.y = y;
  mp.lens = seq_lens;
  const unsigned par = plan->launch_id & 1u;
  mp.sync = plan->d_sync + 2 * par;
  mp.sync_next = plan->d_sync + 2 * (par ^ 1u);
  mp.status = plan->d_status;
  mp.timeout_ns = (unsigned long long)(d.timeout_ms > 0 ? d.timeout_ms : 2000) * 1000000ull;
  mp.prof = plan->d_prof;
  mp.skip_arrival = d.debug_skip_arrival;
  mp.max_slots = d.debug_max_slots;
  int rc = launch_mega(args, plan->grid, reinterpret_cast<cudaStream_t>(stream), plan->family);
  if (rc) return rc;
  plan->launch_id++;
  plan->launches = 1;
  return SOUFFLE_OK;
}

int souffle_bert_forward_host_async(SouffleBertPlan* plan, const void* x_host, const int32_t* seq_lens_host,
                                    void* y_host, souffle_stream_t stream) {
  if (!plan || !x_host || !y_host) return fail(SOUFFLE_BAD_ARGUMENT, "null argument");
  const SouffleBertDesc& d = plan->desc;
  const size_t bytes = (size_t)d.batch * d.seq * d.heads * d.head_dim * 2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!plan->s_in) {
    for (int i = 0; i < 2; ++i) {
      SF_CUDA(cudaMalloc((void**)&plan->x_dev[i], bytes));
      SF_CUDA(cudaMalloc((void**)&plan->y_dev[i], bytes));
      SF_CUDA(cudaMalloc((void**)&plan->lens_dev[i], (size_t)d.batch * 4));
      SF_CUDA(cudaEventCreateWithFlags(&plan->ev_in[i], cudaEventDisableTiming));
      SF_CUDA(cudaEventCreateWithFlags(&plan->ev_k[i], cudaEventDisableTiming));
      SF_CUDA(cudaEventCreateWithFlags(&plan->ev_out[i], cudaEventDisableTiming));
    }
    SF_CUDA(cudaStreamCreateWithFlags(&plan->s_cmp, cudaStreamNonBlocking));
    SF_CUDA(cudaStreamCreateWithFlags(&plan->s_out, cudaStreamNonBlocking));
    SF_CUDA(cudaStreamCreateWithFlags(&plan->s_in, cudaStreamNonBlocking));
  }
  const int b = (int)(plan->host_calls++ & 1u);
  // copy-in: once the kernel of the call before last has read this input buffer (an event that was never
  // recorded does not block).  It does not wait for `stream`, which is itself waiting for earlier copy-outs:
  // x_host has to be ready when the call is made.
  SF_CUDA(cudaStreamWaitEvent(plan->s_in, plan->ev_k[b], 0));
  SF_CUDA(cudaMemcpyAsync(plan->x_dev[b], x_host, bytes, cudaMemcpyHostToDevice, plan->s_in));
  if (seq_lens_host)
    SF_CUDA(cudaMemcpyAsync(plan->lens_dev[b], seq_lens_host, (size_t)d.batch * 4, cudaMemcpyHostToDevice, plan->s_in));
  SF_CUDA(cudaEventRecord(plan->ev_in[b], plan->s_in));
  // compute: launches of one plan run one after the other on the plan's own stream; the output buffer must
  // have been copied out by the call before last
  SF_CUDA(cudaStreamWaitEvent(plan->s_cmp, plan->ev_in[b], 0));
  SF_CUDA(cudaStreamWaitEvent(plan->s_cmp, plan->ev_out[b], 0));
  int rc = souffle_bert_forward(plan, plan->x_dev[b], seq_lens_host ? plan->lens_dev[b] : nullptr, plan->y_dev[b],
                                reinterpret_cast<souffle_stream_t>(plan->s_cmp));
  if (rc) return rc;
  SF_CUDA(cudaEventRecord(plan->ev_k[b], plan->s_cmp));
  // copy-out, and the caller's stream waits for it
  SF_CUDA(cudaStreamWaitEvent(plan->s_out, plan->ev_k[b], 0));
  SF_CUDA(cudaMemcpyAsync(y_host, plan->y_dev[b], bytes, cudaMemcpyDeviceToHost, plan->s_out));
  SF_CUDA(cudaEventRecord(plan->ev_out[b], plan->s_out));
  SF_CUDA(cudaStreamWaitEvent(st, plan->ev_out[b], 0));
  return SOUFFLE_OK;
}

int souffle_bert_forward_host(SouffleBertPlan* plan, const void* x_host, const int32_t* seq_lens_host,
                              void* y_host, souffle_stream_t stream) {
  const int rc = souffle_bert_forward_host_async(plan, x_host, seq_lens_host, y_host, stream);
  if (rc) return rc;
  SF_CUDA(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  return SOUFFLE_OK;
}

int souffle_bert_plan_buffer(SouffleBertPlan* plan, int which, void** ptr_out, size_t* bytes_out) {
  if (!plan || !ptr_out) return fail(SOUFFLE_BAD_ARGUMENT, "null argument");
  const SouffleBertDesc& d = plan->desc;
  const size_t M = (size_t)d.batch * d.seq, H = (size_t)d.heads * d.head_dim;
  void* ptr = nullptr;
  size_t bytes = 0;
  switch (which) {
    case SOUFFLE_BUF_QKV: ptr = plan->qkv; bytes = 3 * M * H * 2; break;
    case SOUFFLE_BUF_PROBS: ptr = plan->probs; bytes = (size_t)d.batch * d.heads * d.seq * d.seq * 2; break;
    case SOUFFLE_BUF_CTX: ptr = plan->ctx; bytes = M * H * 2; break;
    case SOUFFLE_BUF_LN1: ptr = plan->ln1; bytes = M * H * 2; break;
    case SOUFFLE_BUF_FC1: ptr = plan->fc1; bytes = M * (size_t)d.ffn * 2; break;
    default: return fail(SOUFFLE_BAD_ARGUMENT, "unknown buffer id %d", which);
  }
  if (!ptr) return fail(SOUFFLE_BAD_ARGUMENT, "buffer %d was not requested at plan creation", which);
  if (!d.keep_probs)
    return fail(SOUFFLE_BAD_ARGUMENT, "stage outputs are kept readable only by plans created with keep_probs (others drop them from L2 once consumed)");
  *ptr_out = ptr;
  if (bytes_out) *bytes_out = bytes;
  return SOUFFLE_OK;
}

int souffle_bert_plan_copy_buffer(SouffleBertPlan* plan, int which, void* dst, size_t dst_bytes,
                                  souffle_stream_t stream) {
  void* src = nullptr;
  size_t bytes = 0;
  int rc = souffle_bert_plan_buffer(plan, which, &src, &bytes);
  if (rc) return rc;
  if (!dst || dst_bytes < bytes) return fail(SOUFFLE_BAD_ARGUMENT, "destination holds %zu bytes, buffer has %zu", dst_bytes, bytes);
  SF_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, reinterpret_cast<cudaStream_t>(stream)));
  return SOUFFLE_OK;
}

int souffle_bert_plan_status(SouffleBertPlan* plan) {
  if (!plan) return fail(SOUFFLE_BAD_ARGUMENT, "null plan");
  SF_CUDA(cudaDeviceSynchronize());
  int h[4] = {0, 0, 0, 0};
  SF_CUDA(cudaMemcpy(h, plan->d_status, sizeof(h), cudaMemcpyDeviceToHost));
  if (h[0] != DEV_OK) {
    // leave the plan usable: clear the status and both barrier pairs
    cudaMemset(plan->d_status, 0, 64);
    cudaMemset(plan->d_sync, 0, 64);
  }
  return decode_status(h, "souffle_bert_forward");
}

int souffle_bert_plan_read_profile(SouffleBertPlan* plan, int64_t* out, size_t capacity_elems) {
  if (!plan || !out) return fail(SOUFFLE_BAD_ARGUMENT, "null argument");
  if (!plan->d_prof) return fail(SOUFFLE_BAD_ARGUMENT, "the plan was created without desc.profile");
  const size_t n = (plan->stages.size() + 1) * (size_t)plan->grid * kProfSlots;
  if (capacity_elems < n) return fail(SOUFFLE_BAD_ARGUMENT, "profile needs %zu elements, got %zu", n, capacity_elems);
  SF_CUDA(cudaDeviceSynchronize());
  SF_CUDA(cudaMemcpy(out, plan->d_prof, n * sizeof(long long), cudaMemcpyDeviceToHost));
  return SOUFFLE_OK;
}

int souffle_bert_plan_info(SouffleBertPlan* plan, int* launches_out, int* grid_out, int* n_stages_out) {
  if (!plan) return fail(SOUFFLE_BAD_ARGUMENT, "null plan");
  if (launches_out) *launches_out = plan->launches;
  if (grid_out) *grid_out = plan->grid;
  if (n_stages_out) *n_stages_out = (int)plan->stages.size();
  return SOUFFLE_OK;
}

int souffle_bert_plan_uses_pairs(SouffleBertPlan* plan) { return plan && plan->pair ? 1 : 0; }

int souffle_bert_packed_weights(const void* blob, int32_t batch, int32_t seq, int32_t hidden, int32_t ffn,
                                SouffleBertLayerWeights* out, const void** mask_out, size_t* blob_bytes) {
  if (batch < 1 || seq < 1 || hidden < 8 || hidden % 8 || ffn < 8 || ffn % 8)
    return fail(SOUFFLE_BAD_SHAPE, "packed block needs batch, seq >= 1 and hidden, ffn multiples of 8 (got %d, %d, %d, %d)",
                batch, seq, hidden, ffn);
  if ((size_t)batch * seq * seq % 8) return fail(SOUFFLE_BAD_SHAPE, "mask of %d x %d x %d halves breaks the 16-byte alignment", batch, seq, seq);
  const size_t H = (size_t)hidden, F = (size_t)ffn;
  const __half* p = reinterpret_cast<const __half*>(blob);
  const __half* mask = p;
  p += (size_t)batch * seq * seq;
  SouffleBertLayerWeights w;
  w.qkv_w = p;  p += 3 * H * H;
  w.proj_w = p; p += H * H;
  w.fc1_w = p;  p += H * F;
  w.fc2_w = p;  p += F * H;
  w.qkv_b = p;  p += 3 * H;
  w.proj_b = p; p += H;
  w.ln1_g = p;  p += H;
  w.ln1_b = p;  p += H;
  w.fc1_b = p;  p += F;
  w.fc2_b = p;  p += H;
  w.ln2_g = p;  p += H;
  w.ln2_b = p;  p += H;
  if (out) *out = w;
  if (mask_out) *mask_out = mask;
  if (blob_bytes) *blob_bytes = (size_t)(reinterpret_cast<const char*>(p) - reinterpret_cast<const char*>(blob));
  return SOUFFLE_OK;
}

int souffle_bert_plan_stage_info(SouffleBertPlan* plan, int index, int out[6]) {
  if (!plan || !out) return fail(SOUFFLE_BAD_ARGUMENT, "null argument");
  if (index < 0 || index >= (int)plan->stages.size()) return fail(SOUFFLE_BAD_ARGUMENT, "stage index %d out of range", index);
  const Stage& s = plan->stages[index];
  out[0] = s.type; out[1] = s.bm; out[2] = s.bn; out[3] = s.splitk; out[4] = stage_items(s, plan->pair);
  out[5] = s.type == STAGE_GEMM ? s.nslots : 0;
  return SOUFFLE_OK;
}

// ======================================================================================
// plan-less GEMM / Swin MLP: tensor maps and stages travel in the launch parameters
// ======================================================================================
size_t souffle_gemm_workspace_bytes(void) { return 256; }

// The barrier words of a caller-owned workspace: two (count, spare) pairs used by alternate launches; the
// kernel clears the pair of the NEXT launch in its prologue (see souffle_megakernel), so the workspace needs a
// memset only the first time this library sees it, and a launch that ended in a device timeout leaves the
// other pair clean for the call after it.
static std::mutex g_ws_mutex;
static std::unordered_map<const void*, unsigned> g_ws_launches;

static int ws_prepare(void* workspace, size_t ws_bytes, cudaStream_t st, MegaParams* mp) {
  if (!aligned16(workspace) || ws_bytes < souffle_gemm_workspace_bytes())
    return fail(SOUFFLE_BAD_POINTER, "workspace must be 16-byte aligned and hold %zu bytes", souffle_gemm_workspace_bytes());
  unsigned launch = 0;
  {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    auto it = g_ws_launches.find(workspace);
    if (it == g_ws_launches.end()) {
      SF_CUDA(cudaMemsetAsync(workspace, 0, 128, st));
      g_ws_launches.emplace(workspace, 1u);
    } else {
      launch = it->second++;
    }
  }
  const unsigned par = launch & 1u;
  mp->sync = reinterpret_cast<unsigned*>(workspace) + 2 * par;
  mp->sync_next = reinterpret_cast<unsigned*>(workspace) + 2 * (par ^ 1u);
  mp->status = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + 64);
  mp->timeout_ns = 2000ull * 1000000ull;
  return SOUFFLE_OK;
}

static int fill_gemm_stage(Stage* s, int tm_a, int tm_b, const void* out, int M, int N, int K, int sms) {
  *s = blank_stage(STAGE_GEMM);
  const TileChoice t = choose_tiles(M, N, K, sms, false, true);
  if (!t.bn) return fail(SOUFFLE_BAD_SHAPE, "N=%d must be a multiple of 64", N);
  s->tm_a = tm_a; s->tm_b = tm_b; s->M = M; s->N = N; s->K = K; s->bm = t.bm; s->bn = t.bn; s->b_mn_major = 1;
  s->epi = EPI_F16; s->out = const_cast<void*>(out); s->ldo = N;
  return finalize_stage(*s, 0, 1);
}

int souffle_gemm_f16(const void* a, const void* w_kn, void* c, int32_t M, int32_t N, int32_t K, void* workspace,
                     size_t workspace_bytes, souffle_stream_t stream) {
  if (M < 1 || N < 64 || N % 64 || K < 64 || K % 64)
    return fail(SOUFFLE_BAD_SHAPE, "GEMM needs M >= 1, N %% 64 == 0, K %% 64 == 0 (got %d, %d, %d)", M, N, K);
  if (!aligned16(a) || !aligned16(w_kn) || !aligned16(c)) return fail(SOUFFLE_BAD_POINTER, "operands must be 16-byte aligned");
  DeviceInfo* di = nullptr;
  int rc = device_info(&di);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CallArgs args;
  memset(&args, 0, sizeof(args));
  if ((rc = ws_prepare(workspace, workspace_bytes, st, &args.p))) return rc;
  const int sms = di->sms < di->max_ctas ? di->sms : di->max_ctas;
  if ((rc = fill_gemm_stage(&args.inline_stages[0], -1, -2, c, M, N, K, sms))) return rc;
  if ((rc = make_map(&args.call_maps[0], a, M, K, (uint32_t)args.inline_stages[0].bm))) return rc;
  if ((rc = make_map(&args.call_maps[1], w_kn, K, N, 64))) return rc;     // [K][N]: box 64 (N) x 64 (K rows)
  args.p.n_stages = 1;
  const int items = stage_items(args.inline_stages[0]);
  return launch_mega(args, items < sms ? items : sms, st);
}

// FC2 of the MLP has few output tiles and a long K (256 x 512 outputs, K = 2048 in the reference's shape), so
// it is cut along K into fp32 planes and a third stage sums them: the LayerNorm stage in its sum-only mode.
// The planes live behind the barrier words of the workspace.
static int swin_mlp_split(int M, int C, int F, int sms) {
  const TileChoice t = choose_tiles(M, C, F, sms, true, true);
  return t.bn ? t.split : 1;
}

size_t souffle_swin_mlp_workspace_bytes(int32_t M, int32_t C, int32_t F) {
  if (M < 1 || C < 64 || F < 64) return souffle_gemm_workspace_bytes();
  return souffle_gemm_workspace_bytes() + (size_t)16 * M * C * sizeof(float);      // room for the deepest split
}

int souffle_swin_mlp_forward(const void* src, const void* fc1_w, const void* fc2_w, void* hidden, void* out, int32_t M,
                             int32_t C, int32_t F, void* workspace, size_t workspace_bytes, souffle_stream_t stream) {
  if (M < 1 || C < 64 || C % 64 || F < 64 || F % 64)
    return fail(SOUFFLE_BAD_SHAPE, "MLP needs M >= 1 and C, F multiples of 64 (got %d, %d, %d)", M, C, F);
  if (!aligned16(src) || !aligned16(fc1_w) || !aligned16(fc2_w) || !aligned16(hidden) || !aligned16(out))
    return fail(SOUFFLE_BAD_POINTER, "operands must be 16-byte aligned");
  DeviceInfo* di = nullptr;
  int rc = device_info(&di);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CallArgs args;
  memset(&args, 0, sizeof(args));
  if ((rc = ws_prepare(workspace, workspace_bytes, st, &args.p))) return rc;
  const int sms = di->sms < di->max_ctas ? di->sms : di->max_ctas;
  if ((rc = fill_gemm_stage(&args.inline_stages[0], -1, -2, hidden, M, F, C, sms))) return rc;
  // split FC2 when the caller's workspace has room for the planes and the reduction stage supports the width
  int split = swin_mlp_split(M, C, F, sms);
  const bool can_reduce = C == 128 || C == 256 || C == 512 || C == 768 || C == 1024;
  const size_t plane_bytes = (size_t)M * C * sizeof(float);
  if (!can_reduce || workspace_bytes < souffle_gemm_workspace_bytes() + (size_t)split * plane_bytes) split = 1;
  Stage& s2 = args.inline_stages[1];
  if (split > 1) {
    const TileChoice t = choose_tiles(M, C, F, sms, true, true);
    s2 = blank_stage(STAGE_GEMM);
    s2.tm_a = -3; s2.tm_b = -4; s2.M = M; s2.N = C; s2.K = F; s2.bm = t.bm; s2.bn = t.bn; s2.splitk = split; s2.b_mn_major = 1;
    s2.epi = EPI_PARTIAL; s2.ldo = C;
    s2.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + souffle_gemm_workspace_bytes());
    if ((rc = finalize_stage(s2, 0, 1))) return rc;
  } else if ((rc = fill_gemm_stage(&s2, -3, -4, out, M, C, F, sms))) {
    return rc;
  }
  if ((rc = make_map(&args.call_maps[0], src, M, C, (uint32_t)args.inline_stages[0].bm))) return rc;
  if ((rc = make_map(&args.call_maps[1], fc1_w, C, F, 64))) return rc;
  if ((rc = make_map(&args.call_maps[2], hidden, M, F, (uint32_t)s2.bm))) return rc;
  if ((rc = make_map(&args.call_maps[3], fc2_w, F, C, 64))) return rc;
  args.p.n_stages = split > 1 ? 3 : 2;
  int items = stage_items(args.inline_stages[0]);
  const int i2 = stage_items(s2);
  if (i2 > items) items = i2;
  const int grid = items < sms ? items : sms;
  if (split > 1) {
    Stage& s3 = args.inline_stages[2];
    s3 = blank_stage(STAGE_LN);
    s3.M = M; s3.N = C; s3.ldo = C; s3.partial = s2.partial; s3.n_partial = split; s3.out = out;
    s3.eps = -1.0f;                                    // sum only
    if ((rc = finalize_stage(s3, 0, grid))) return rc;
  }
  return launch_mega(args, grid, st);
}

int souffle_layernorm_forward(const float* partial, int32_t n_partial, const void* bias, const void* resid,
                              const void* gamma, const void* beta, void* out, int32_t M, int32_t N, float eps,
                              void* workspace, size_t workspace_bytes, souffle_stream_t stream) {
  if (M < 1 || (N != 128 && N != 256 && N != 512 && N != 768 && N != 1024) || n_partial < 1 || n_partial > 16)
    return fail(SOUFFLE_BAD_SHAPE, "LayerNorm needs M >= 1, N in {128, 256, 512, 768, 1024}, 1 <= n_partial <= 16 (got %d, %d, %d)", M, N, n_partial);
  if (!aligned16(partial) || !aligned16(out) || (bias && !aligned16(bias)) || (resid && !aligned16(resid)) ||
      (gamma && !aligned16(gamma)) || (beta && !aligned16(beta)))
    return fail(SOUFFLE_BAD_POINTER, "operands must be 16-byte aligned");
  if ((gamma == nullptr) != (beta == nullptr)) return fail(SOUFFLE_BAD_ARGUMENT, "gamma and beta must be given together");
  DeviceInfo* di = nullptr;
  int rc = device_info(&di);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CallArgs args;
  memset(&args, 0, sizeof(args));
  if ((rc = ws_prepare(workspace, workspace_bytes, st, &args.p))) return rc;
  Stage& s = args.inline_stages[0];
  s = blank_stage(STAGE_LN);
  s.M = M; s.N = N; s.ldo = N; s.partial = const_cast<float*>(partial); s.n_partial = n_partial; s.bias = bias;
  s.resid = resid; s.out = out; s.gamma = gamma; s.beta = beta; s.eps = eps;
  args.p.n_stages = 1;
  const int sms = di->sms < di->max_ctas ? di->sms : di->max_ctas;
  const int items = stage_items(s);
  const int grid = items < sms ? items : sms;
  if ((rc = finalize_stage(s, 0, grid))) return rc;
  return launch_mega(args, grid, st);
}

// ======================================================================================
// Swin block plan (shares the plan machinery of the encoder)
// ======================================================================================
struct SouffleSwinPlan {
  SouffleBertPlan base;
  SouffleSwinDesc desc;
  SouffleSwinMerge merge = {nullptr, nullptr, nullptr};
  bool has_merge = false;
};

static int launch_plan(SouffleBertPlan* plan, const void* x, void* y, const int32_t* lens, int timeout_ms, cudaStream_t st) {
  CallArgs args;
  memset(&args, 0, sizeof(args));
  args.call_maps[0] = plan->x_map;
  MegaParams& mp = args.p;
  mp.stages = plan->d_stages;
  mp.n_stages = (int)plan->stages.size();
  mp.maps = plan->d_maps;
  mp.n_maps = (int)plan->maps.size();
  mp.x = x;
  mp.y = y;
  mp.lens = lens;
  const unsigned par = plan->launch_id & 1u;
  mp.sync = plan->d_sync + 2 * par;
  mp.sync_next = plan->d_sync + 2 * (par ^ 1u);
  mp.status = plan->d_status;
  mp.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  int rc = launch_mega(args, plan->grid, st, kFamilySwin);
  if (rc) return rc;
  plan->launch_id++;
  plan->launches = 1;
  return SOUFFLE_OK;
}

static int finish_plan(SouffleBertPlan* p, int sms) {
  int rc;
  int max_items = 1;
  for (const Stage& s : p->stages) {
    const int it = stage_items(s);
    if (it > max_items) max_items = it;
  }
  p->grid = max_items < sms ? max_items : sms;
  for (Stage& fs : p->stages)
    if ((rc = finalize_stage(fs, p->desc.debug_max_slots, p->grid))) return rc;
  return upload_program(p);
}

static int build_swin_plan(SouffleSwinPlan* sp, const SouffleSwinWeights* blocks) {
  SouffleBertPlan* p = &sp->base;
  const SouffleSwinDesc& d = sp->desc;
  DeviceInfo* di = nullptr;
  int rc = device_info(&di);
  if (rc) return rc;
  p->device = di->device;
  const int sms = di->sms < di->max_ctas ? di->sms : di->max_ctas;
  const int R = d.res, C = d.dim, Hh = d.heads, ws = d.window, F = C * d.mlp_ratio;
  const int T = d.batch * R * R, nWt = d.batch * (R / ws) * (R / ws), Mw = nWt * 64;
  const int n_blocks = d.n_blocks > 0 ? d.n_blocks : 1;
  // FC2 has few output tiles and the longest K of the block: it is cut along K into fp32 planes, and a sum-only
  // LayerNorm stage adds them, the bias and the residual (the block's output).
  const TileChoice t_qkv = choose_tiles(T, 3 * C, C, sms, false, false, 2), t_proj = choose_tiles(Mw, C, C, sms, false, false, 2),
                   t_fc1 = choose_tiles(T, F, C, sms, false, false, 0), t_fc2 = choose_tiles(T, C, F, sms, true, false, 0);
  // activations, shared by all blocks of the chain (stages run one after the other)
  __half *y1, *qkvw, *ctxw, *x1, *y2, *hid, *xbuf[2] = {nullptr, nullptr};
  float* planes;
  if ((rc = plan_alloc(p, (void**)&y1, (size_t)T * C * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&qkvw, (size_t)3 * Mw * C * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&ctxw, (size_t)Mw * C * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&x1, (size_t)T * C * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&y2, (size_t)T * C * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&hid, (size_t)T * F * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&planes, (size_t)t_fc2.split * T * C * 4))) return rc;
  for (int i = 0; i < 2 && i < n_blocks - 1; ++i)
    if ((rc = plan_alloc(p, (void**)&xbuf[i], (size_t)T * C * 2))) return rc;
  __half* xlast = nullptr;          // output of the last block when patch merging follows inside the launch
  if (sp->has_merge && (rc = plan_alloc(p, (void**)&xlast, (size_t)T * C * 2))) return rc;
  if ((rc = plan_alloc(p, (void**)&p->d_sync, 64))) return rc;
  if ((rc = plan_alloc(p, (void**)&p->d_status, 64))) return rc;
  SF_CUDA(cudaMemset(p->d_sync, 0, 64));
  SF_CUDA(cudaMemset(p->d_status, 0, 64));
  SF_CUDA(cudaMemset(qkvw, 0, (size_t)3 * Mw * C * 2));     // padding slots stay zero for ever
  SF_CUDA(cudaMemset(ctxw, 0, (size_t)Mw * C * 2));
  int m_y1, m_ctx, m_y2, m_hid, m_qkv;
  if ((rc = add_map(p, y1, T, C, t_qkv.bm, &m_y1)) || (rc = add_map(p, ctxw, Mw, C, t_proj.bm, &m_ctx)) ||
      (rc = add_map(p, y2, T, C, t_fc1.bm, &m_y2)) || (rc = add_map(p, hid, T, F, t_fc2.bm, &m_hid)) ||
      (rc = add_map(p, qkvw, (uint64_t)3 * Mw, C, 128, &m_qkv)))
    return rc;
  auto copy_vec = [&](const void* src, size_t n, const void** dst) -> int {
    *dst = nullptr;
    if (!src) return SOUFFLE_OK;
    void* v;
    int r2 = plan_alloc(p, &v, n * 2);
    if (r2) return r2;
    if (cudaMemcpy(v, src, n * 2, cudaMemcpyDeviceToDevice) != cudaSuccess) return fail(SOUFFLE_CUDA_ERROR, "copying a parameter vector failed");
    *dst = v;
    return SOUFFLE_OK;
  };
  const int tbl = (2 * ws - 1) * (2 * ws - 1);
  const dim3 tb(32, 8);

  for (int bi = 0; bi < n_blocks; ++bi) {
    const SouffleSwinWeights& w = blocks[bi];
    const int shift = (bi & 1) ? d.shift_alt : d.shift;
    if (!w.qkv_w || !w.proj_w || !w.fc1_w || !w.fc2_w || !w.rel_bias)
      return fail(SOUFFLE_BAD_POINTER, "block %d: qkv_w, proj_w, fc1_w, fc2_w and rel_bias must be given", bi);
    // weights: repack [K][N] -> [N][K]
    __half *wqkv_t, *wo_t, *w1_t, *w2_t;
    if ((rc = plan_alloc(p, (void**)&wqkv_t, (size_t)3 * C * C * 2))) return rc;
    if ((rc = plan_alloc(p, (void**)&wo_t, (size_t)C * C * 2))) return rc;
    if ((rc = plan_alloc(p, (void**)&w1_t, (size_t)C * F * 2))) return rc;
    if ((rc = plan_alloc(p, (void**)&w2_t, (size_t)F * C * 2))) return rc;
    transpose_kn_to_nk<<<dim3(3 * C / 32, C / 32), tb>>>(reinterpret_cast<const __half*>(w.qkv_w), wqkv_t, C, 3 * C);
    transpose_kn_to_nk<<<dim3(C / 32, C / 32), tb>>>(reinterpret_cast<const __half*>(w.proj_w), wo_t, C, C);
    transpose_kn_to_nk<<<dim3(F / 32, C / 32), tb>>>(reinterpret_cast<const __half*>(w.fc1_w), w1_t, C, F);
    transpose_kn_to_nk<<<dim3(C / 32, F / 32), tb>>>(reinterpret_cast<const __half*>(w.fc2_w), w2_t, F, C);
    SF_CUDA(cudaGetLastError());
    const void *ln1_g, *ln1_b, *qkv_b, *relb, *proj_b, *ln2_g, *ln2_b, *fc1_b, *fc2_b;
    if ((rc = copy_vec(w.ln1_g, C, &ln1_g)) || (rc = copy_vec(w.ln1_b, C, &ln1_b)) || (rc = copy_vec(w.qkv_b, 3 * C, &qkv_b)) ||
        (rc = copy_vec(w.rel_bias, (size_t)tbl * Hh, &relb)) || (rc = copy_vec(w.proj_b, C, &proj_b)) ||
        (rc = copy_vec(w.ln2_g, C, &ln2_g)) || (rc = copy_vec(w.ln2_b, C, &ln2_b)) || (rc = copy_vec(w.fc1_b, F, &fc1_b)) ||
        (rc = copy_vec(w.fc2_b, C, &fc2_b)))
      return rc;
    if ((ln1_g == nullptr) != (ln1_b == nullptr) || (ln2_g == nullptr) != (ln2_b == nullptr))
      return fail(SOUFFLE_BAD_ARGUMENT, "gamma and beta must be given together");
    int m_wqkv, m_wo, m_w1, m_w2;
    if ((rc = add_map(p, wqkv_t, 3 * C, C, t_qkv.bn, &m_wqkv)) || (rc = add_map(p, wo_t, C, C, t_proj.bn, &m_wo)) ||
        (rc = add_map(p, w1_t, F, C, t_fc1.bn, &m_w1)) || (rc = add_map(p, w2_t, C, F, t_fc2.bn, &m_w2)))
      return rc;
    // the block's input (also the residual of its attention half) and output
    const int in_sel = bi == 0 ? PTR_CALL_X : PTR_PLAN;
    const __half* xin = bi == 0 ? nullptr : xbuf[(bi - 1) & 1];
    const bool last = bi == n_blocks - 1;

    Stage s = blank_stage(STAGE_LN);                       // LN1(x)
    s.M = T; s.N = C; s.ldo = C; s.n_partial = 0; s.resid_sel = in_sel; s.resid = xin; s.out = y1; s.gamma = ln1_g; s.beta = ln1_b;
    s.eps = d.eps;
    p->stages.push_back(s);
    s = blank_stage(STAGE_GEMM);                           // QKV, rolled and scattered window-major
    s.tm_a = m_y1; s.tm_b = m_wqkv; s.M = T; s.N = 3 * C; s.K = C; s.bm = t_qkv.bm; s.bn = t_qkv.bn; s.epi = EPI_SWIN_QKV;
    s.bias = qkv_b; s.out = qkvw; s.ldo = C; s.batch = d.batch; s.heads = Hh; s.head_dim = 32; s.seq = R; s.win = ws; s.shift = shift;
    p->stages.push_back(s);
    note_weights(p, wqkv_t);
    s = blank_stage(STAGE_ATTN_SWIN);                      // window attention
    s.tm_qkv = m_qkv; s.batch = d.batch; s.heads = Hh; s.head_dim = 32; s.seq = R; s.win = ws; s.shift = shift; s.ldo = C;
    s.scale = 1.0f / sqrtf(32.0f); s.rel_bias = relb; s.out = ctxw;
    p->stages.push_back(s);
    s = blank_stage(STAGE_GEMM);                           // proj, window reverse, roll back, + x
    s.tm_a = m_ctx; s.tm_b = m_wo; s.M = Mw; s.N = C; s.K = C; s.bm = t_proj.bm; s.bn = t_proj.bn; s.epi = EPI_SWIN_PROJ;
    s.bias = proj_b; s.resid_sel = in_sel; s.resid = xin; s.out = x1; s.ldo = C; s.batch = d.batch; s.heads = Hh; s.head_dim = 32;
    s.seq = R; s.win = ws; s.shift = shift;
    p->stages.push_back(s);
    note_weights(p, wo_t);
    s = blank_stage(STAGE_LN);                             // LN2(x1)
    s.M = T; s.N = C; s.ldo = C; s.n_partial = 0; s.resid = x1; s.out = y2; s.gamma = ln2_g; s.beta = ln2_b; s.eps = d.eps;
    p->stages.push_back(s);
    s = blank_stage(STAGE_GEMM);                           // FC1 + GELU
    s.tm_a = m_y2; s.tm_b = m_w1; s.M = T; s.N = F; s.K = C; s.bm = t_fc1.bm; s.bn = t_fc1.bn; s.epi = EPI_F16; s.act = ACT_GELU;
    s.bias = fc1_b; s.out = hid; s.ldo = F;
    p->stages.push_back(s);
    note_weights(p, w1_t);
    s = blank_stage(STAGE_GEMM);                           // FC2 -> fp32 planes
    s.tm_a = m_hid; s.tm_b = m_w2; s.M = T; s.N = C; s.K = F; s.bm = t_fc2.bm; s.bn = t_fc2.bn; s.splitk = t_fc2.split;
    s.epi = EPI_PARTIAL; s.partial = planes; s.ldo = C;
    if ((rc = add_plane_map(p, s))) return rc;
    p->stages.push_back(s);
    note_weights(p, w2_t);
    s = blank_stage(STAGE_LN);                             // planes + bias + x1 -> block output (no normalisation)
    s.M = T; s.N = C; s.ldo = C; s.partial = planes; s.n_partial = t_fc2.split; s.bias = fc2_b; s.resid = x1; s.eps = -1.0f;
    if (last && !sp->has_merge) s.out_sel = PTR_CALL_Y; else s.out = last ? xlast : xbuf[bi & 1];
    p->stages.push_back(s);
  }
  if (sp->has_merge) {
    // Patch merging (python/models/swin_transformer/swin_patch_merge.py:1-17): 2 x 2 neighbourhoods concatenated to
    // 4C channels (gathered by the LayerNorm stage's copies), LayerNorm, reduction 4C -> 2C without bias.  The
    // reduction has (R/2)^2 rows per image and K = 4C: it is cut along K, a sum-only stage adds the planes.
    const int Tm = d.batch * (R / 2) * (R / 2), C4 = 4 * C, C2 = 2 * C;
    const TileChoice t_red = choose_tiles(Tm, C2, C4, sms, true, false, 0);
    __half *merged, *wr_t;
    float* planes2;
    if ((rc = plan_alloc(p, (void**)&merged, (size_t)Tm * C4 * 2))) return rc;
    if ((rc = plan_alloc(p, (void**)&wr_t, (size_t)C4 * C2 * 2))) return rc;
    if ((rc = plan_alloc(p, (void**)&planes2, (size_t)t_red.split * Tm * C2 * 4))) return rc;
    transpose_kn_to_nk<<<dim3(C2 / 32, C4 / 32), tb>>>(reinterpret_cast<const __half*>(sp->merge.reduction_w), wr_t, C4, C2);
    SF_CUDA(cudaGetLastError());
    const void *mg, *mb;
    if ((rc = copy_vec(sp->merge.norm_g, C4, &mg)) || (rc = copy_vec(sp->merge.norm_b, C4, &mb))) return rc;
    if ((mg == nullptr) != (mb == nullptr)) return fail(SOUFFLE_BAD_ARGUMENT, "gamma and beta must be given together");
    int m_merged, m_wr;
    if ((rc = add_map(p, merged, Tm, C4, t_red.bm, &m_merged)) || (rc = add_map(p, wr_t, C2, C4, t_red.bn, &m_wr))) return rc;
    Stage s = blank_stage(STAGE_LN);                         // gather + LayerNorm over 4C
    s.M = Tm; s.N = C4; s.ldo = C4; s.n_partial = 0; s.resid = xlast; s.out = merged; s.gamma = mg; s.beta = mb; s.eps = d.eps;
    s.seq = R; s.batch = d.batch;
    p->stages.push_back(s);
    s = blank_stage(STAGE_GEMM);                             // reduction -> fp32 planes
    s.tm_a = m_merged; s.tm_b = m_wr; s.M = Tm; s.N = C2; s.K = C4; s.bm = t_red.bm; s.bn = t_red.bn; s.splitk = t_red.split;
    s.epi = EPI_PARTIAL; s.partial = planes2; s.ldo = C2;
    if ((rc = add_plane_map(p, s))) return rc;
    p->stages.push_back(s);
    note_weights(p, wr_t);
    s = blank_stage(STAGE_LN);                               // sum of the planes -> y
    s.M = Tm; s.N = C2; s.ldo = C2; s.partial = planes2; s.n_partial = t_red.split; s.eps = -1.0f; s.out_sel = PTR_CALL_Y;
    p->stages.push_back(s);
  }
  return finish_plan(p, sms);
}

int souffle_swin_block_plan_create(const SouffleSwinDesc* desc, const SouffleSwinWeights* weights, SouffleSwinPlan** plan_out) {
  return souffle_swin_stage_plan_create(desc, weights, nullptr, plan_out);
}

int souffle_swin_stage_plan_create(const SouffleSwinDesc* desc, const SouffleSwinWeights* weights, const SouffleSwinMerge* merge,
                                   SouffleSwinPlan** plan_out) {
  if (!desc || !weights || !plan_out) return fail(SOUFFLE_BAD_ARGUMENT, "null argument");
  *plan_out = nullptr;
  const SouffleSwinDesc& d = *desc;
  if (d.batch < 1 || d.res < 1) return fail(SOUFFLE_BAD_SHAPE, "batch and res must be >= 1");
  if (d.window != 7 && d.window != 8) return fail(SOUFFLE_BAD_SHAPE, "window must be 7 or 8 (got %d)", d.window);
  if (d.res % d.window) return fail(SOUFFLE_BAD_SHAPE, "res %d is not a multiple of the window %d", d.res, d.window);
  if (d.shift < 0 || d.shift >= d.window || d.shift_alt < 0 || d.shift_alt >= d.window)
    return fail(SOUFFLE_BAD_SHAPE, "shift and shift_alt must be in [0, window)");
  if (d.n_blocks < 0 || d.n_blocks > 18) return fail(SOUFFLE_BAD_SHAPE, "n_blocks must be in 1..18 (0 = 1), got %d", d.n_blocks);
  if (d.dim != 128 && d.dim != 256 && d.dim != 512 && d.dim != 768 && d.dim != 1024)
    return fail(SOUFFLE_BAD_SHAPE, "dim %d must be 128, 256, 512, 768 or 1024", d.dim);
  if (d.heads < 2 || d.heads % 2 || d.heads * 32 != d.dim) return fail(SOUFFLE_BAD_SHAPE, "heads must be even with dim / heads == 32");
  if (d.mlp_ratio < 1 || d.dim * d.mlp_ratio > 4096) return fail(SOUFFLE_BAD_SHAPE, "dim * mlp_ratio must be in (0, 4096]");
  for (int i = 0; i < (d.n_blocks > 0 ? d.n_blocks : 1); ++i)
    if (!aligned16(weights[i].qkv_w) || !aligned16(weights[i].proj_w) || !aligned16(weights[i].fc1_w) || !aligned16(weights[i].fc2_w))
      return fail(SOUFFLE_BAD_POINTER, "block %d: weight matrices must be non-null and 16-byte aligned", i);
  if (merge) {
    if (d.res % 2) return fail(SOUFFLE_BAD_SHAPE, "patch merging needs an even token grid (res %d)", d.res);
    if (d.dim > 512) return fail(SOUFFLE_BAD_SHAPE, "patch merging normalises 4 * dim columns: dim must be 128, 256 or 512 (got %d)", d.dim);
    if (!aligned16(merge->reduction_w)) return fail(SOUFFLE_BAD_POINTER, "reduction_w must be non-null and 16-byte aligned");
  }
  SouffleSwinPlan* sp = new SouffleSwinPlan();
  sp->desc = d;
  if (merge) {
    sp->merge = *merge;
    sp->has_merge = true;
  }
  int rc = build_swin_plan(sp, weights);
  if (rc) {
    const std::string keep = g_last_error;
    souffle_swin_block_plan_destroy(sp);
    g_last_error = keep;
    return rc;
  }
  *plan_out = sp;
  return SOUFFLE_OK;
}

int souffle_swin_block_plan_destroy(SouffleSwinPlan* sp) {
  if (!sp) return SOUFFLE_OK;
  cudaDeviceSynchronize();
  for (void* a : sp->base.allocs) cudaFree(a);
  delete sp;
  return SOUFFLE_OK;
}

int souffle_swin_block_forward(SouffleSwinPlan* sp, const void* x, void* y, souffle_stream_t stream) {
  if (!sp) return fail(SOUFFLE_BAD_ARGUMENT, "null plan");
  if (!aligned16(x) || !aligned16(y)) return fail(SOUFFLE_BAD_POINTER, "x and y must be non-null and 16-byte aligned");
  return launch_plan(&sp->base, x, y, nullptr, sp->desc.timeout_ms, reinterpret_cast<cudaStream_t>(stream));
}

int souffle_swin_block_plan_status(SouffleSwinPlan* sp) {
  if (!sp) return fail(SOUFFLE_BAD_ARGUMENT, "null plan");
  return souffle_bert_plan_status(&sp->base);
}

// ======================================================================================
// LSTM plan
// ======================================================================================
// One cluster of kLstmParts CTAs per layer.  lstm_check_resident() establishes at plan creation that all clusters fit
// the GPU at once, which the cross-layer waits assume, and every wait in the kernel is bounded.  The cooperative
// launch attribute would add the driver's own guarantee, but Nsight Compute cannot capture a launch that carries both
// attributes (it answers LaunchFailed), so it is asked for only when SOUFFLE_LSTM_COOPERATIVE=1 is set; a driver that
// refuses the combination gets the cluster launch alone from then on.
static int lstm_coop_default() {
  const char* e = getenv("SOUFFLE_LSTM_COOPERATIVE");
  return (e && e[0] == '1') ? 1 : 0;
}
static int g_lstm_coop = lstm_coop_default();
static void lstm_launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* at, int layers, size_t smem, cudaStream_t st, bool coop) {
  memset(cfg, 0, sizeof(*cfg));
  cfg->gridDim = dim3(layers * kLstmParts);
  cfg->blockDim = dim3(kLstmBlock);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = st;
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = kLstmParts;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeCooperative;
  at[1].val.cooperative = 1;
  cfg->attrs = at;
  cfg->numAttrs = coop ? 2 : 1;
}
static int lstm_check_resident(int layers, size_t smem) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute at[2];
  lstm_launch_config(&cfg, at, layers, smem, nullptr, false);
  int clusters = 0;
  SF_CUDA(cudaOccupancyMaxActiveClusters(&clusters, (const void*)souffle_lstm_wavefront, &cfg));
  if (clusters < layers)
    return fail(SOUFFLE_NOT_CORESIDENT, "%d clusters of %d CTAs needed, %d can be resident", layers, kLstmParts, clusters);
  return SOUFFLE_OK;
}
static int lstm_launch(const LstmParams& lp, size_t smem, cudaStream_t st) {
  void* kargs[] = {const_cast<LstmParams*>(&lp)};
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute at[2];
  if (g_lstm_coop) {
    lstm_launch_config(&cfg, at, lp.layers, smem, st, true);
    const cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*)souffle_lstm_wavefront, kargs);
    if (e == cudaSuccess) return SOUFFLE_OK;
    cudaGetLastError();          // a refused launch configuration is not sticky
    g_lstm_coop = 0;
  }
  lstm_launch_config(&cfg, at, lp.layers, smem, st, false);
  SF_CUDA(cudaLaunchKernelExC(&cfg, (const void*)souffle_lstm_wavefront, kargs));
  return SOUFFLE_OK;
}

struct SouffleLstmPlan {
  SouffleLstmDesc desc;
  __half *w_in = nullptr, *w_state = nullptr;
  float *bias = nullptr, *h_all = nullptr;
  unsigned* done = nullptr;   // two sets of kLstmDoneWords counters, used by alternate launches
  int* status = nullptr;
  unsigned launch_id = 0;
  size_t smem = 0;
};

int souffle_lstm_plan_create(const SouffleLstmDesc* desc, const void* w_in, const void* w_state, const float* bias,
                             SouffleLstmPlan** plan_out) {
  if (!desc || !plan_out) return fail(SOUFFLE_BAD_ARGUMENT, "null argument");
  *plan_out = nullptr;
  const SouffleLstmDesc& d = *desc;
  if (d.layers < 1 || d.layers > kLstmMaxLayers) return fail(SOUFFLE_BAD_SHAPE, "layers must be in 1..%d (got %d)", kLstmMaxLayers, d.layers);
  if (d.hidden != 64 && d.hidden != 128 && d.hidden != 256)
    return fail(SOUFFLE_BAD_SHAPE, "hidden must be 64, 128 or 256 (got %d)", d.hidden);
  if (d.steps < 1) return fail(SOUFFLE_BAD_SHAPE, "steps must be >= 1");
  if (!aligned16(w_in) || !aligned16(w_state)) return fail(SOUFFLE_BAD_POINTER, "weights must be non-null and 16-byte aligned");
  int dev = 0, cc = 0, sms = 0;
  SF_CUDA(cudaGetDevice(&dev));
  SF_CUDA(cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev));
  SF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (cc != 10) return fail(SOUFFLE_BAD_DEVICE, "device %d is not sm_100", dev);
  SouffleLstmPlan* p = new SouffleLstmPlan();
  p->desc = d;
  const int H = d.hidden;
  p->smem = lstm_smem_bytes(H);
  const size_t wbytes = (size_t)4 * d.layers * H * H * 2;
  cudaError_t e = cudaFuncSetAttribute(souffle_lstm_wavefront, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lstm_smem_bytes(kLstmMaxHidden));
  if (e == cudaSuccess && lstm_check_resident(d.layers, p->smem) != SOUFFLE_OK) {
    delete p;
    return SOUFFLE_NOT_CORESIDENT;
  }
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->w_in, wbytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->w_state, wbytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->h_all, (size_t)d.layers * d.steps * H * 4);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->done, 2 * kLstmDoneWords * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->status, 64);
  if (e == cudaSuccess && bias) e = cudaMalloc((void**)&p->bias, (size_t)d.layers * H * 4);
  if (e == cudaSuccess) e = cudaMemcpy(p->w_in, w_in, wbytes, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->w_state, w_state, wbytes, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess && bias) e = cudaMemcpy(p->bias, bias, (size_t)d.layers * H * 4, cudaMemcpyDeviceToDevice);
  if (e == cudaSuccess) e = cudaMemset(p->done, 0, 2 * kLstmDoneWords * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemset(p->status, 0, 64);
  if (e != cudaSuccess) {
    souffle_lstm_plan_destroy(p);
    return fail(SOUFFLE_CUDA_ERROR, "LSTM plan set-up failed: %s", cudaGetErrorString(e));
  }
  *plan_out = p;
  return SOUFFLE_OK;
}

int souffle_lstm_plan_destroy(SouffleLstmPlan* p) {
  if (!p) return SOUFFLE_OK;
  cudaDeviceSynchronize();
  cudaFree(p->w_in); cudaFree(p->w_state); cudaFree(p->bias); cudaFree(p->h_all); cudaFree(p->done); cudaFree(p->status);
  delete p;
  return SOUFFLE_OK;
}

int souffle_lstm_forward(SouffleLstmPlan* plan, const float* x, float* y, souffle_stream_t stream) {
  if (!plan) return fail(SOUFFLE_BAD_ARGUMENT, "null plan");
  if (!aligned16(x) || !aligned16(y)) return fail(SOUFFLE_BAD_POINTER, "x and y must be non-null and 16-byte aligned");
  const SouffleLstmDesc& d = plan->desc;
  LstmParams lp;
  lp.w_in = plan->w_in; lp.w_state = plan->w_state; lp.bias = plan->bias; lp.x = x; lp.y = y; lp.h_all = plan->h_all;
  const unsigned par = plan->launch_id & 1u;
  lp.done = plan->done + kLstmDoneWords * par;
  lp.done_next = plan->done + kLstmDoneWords * (par ^ 1u);
  lp.status = plan->status;
  lp.layers = d.layers; lp.hidden = d.hidden; lp.steps = d.steps; lp.ref_input_delay = d.ref_input_delay;
  lp.timeout_ns = (unsigned long long)(d.timeout_ms > 0 ? d.timeout_ms : 2000) * 1000000ull;
  const int rc = lstm_launch(lp, plan->smem, reinterpret_cast<cudaStream_t>(stream));
  if (rc) return rc;
  plan->launch_id++;
  return SOUFFLE_OK;
}

int souffle_lstm_launch_mode(void) { return g_lstm_coop; }

int souffle_lstm_plan_status(SouffleLstmPlan* plan) {
  if (!plan) return fail(SOUFFLE_BAD_ARGUMENT, "null plan");
  SF_CUDA(cudaDeviceSynchronize());
  int h[4] = {0, 0, 0, 0};
  SF_CUDA(cudaMemcpy(h, plan->status, sizeof(h), cudaMemcpyDeviceToHost));
  if (h[0] != DEV_OK) {
    cudaMemset(plan->status, 0, 64);
    cudaMemset(plan->done, 0, 2 * kLstmDoneWords * sizeof(unsigned));
  }
  return decode_status(h, "souffle_lstm_forward");
}

// Allocation-free variant (see lstm_static.cu).  The first call on a device looks up the scratch
// array's device address and sets the kernel attributes; make that call before any stream capture.
static int static_lstm_device(int* dev_out, StaticLstmDevice** sd_out) {
  int dev = 0;
  SF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return fail(SOUFFLE_BAD_DEVICE, "device index %d out of range", dev);
  StaticLstmDevice& sd = g_static_lstm[dev];
  std::lock_guard<std::mutex> lock(sd.mutex);             // host threads may race for the first call on a device
  if (!sd.ready) {
    int cc = 0;
    SF_CUDA(cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev));
    if (cc != 10) return fail(SOUFFLE_BAD_DEVICE, "device %d is not sm_100", dev);
    SF_CUDA(cudaDeviceGetAttribute(&sd.sms, cudaDevAttrMultiProcessorCount, dev));
    void* ptr = nullptr;
    SF_CUDA(cudaGetSymbolAddress(&ptr, g_lstm_static_scratch));
    // the largest shared-memory request any shape makes (plans ask for the same limit)
    SF_CUDA(cudaFuncSetAttribute(souffle_lstm_wavefront, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lstm_smem_bytes(kLstmMaxHidden)));
    sd.scratch = static_cast<unsigned char*>(ptr);
    sd.ready = true;
  }
  *dev_out = dev;
  *sd_out = &sd;
  return SOUFFLE_OK;
}

int souffle_lstm_forward_static(const SouffleLstmDesc* desc, const void* w_in, const void* w_state, const float* bias,
                                const float* x, float* y, int32_t* device_status, souffle_stream_t stream) {
  if (!desc) return fail(SOUFFLE_BAD_ARGUMENT, "null descriptor");
  const SouffleLstmDesc& d = *desc;
  if (d.layers < 1 || d.layers > kLstmMaxLayers) return fail(SOUFFLE_BAD_SHAPE, "layers must be in 1..%d (got %d)", kLstmMaxLayers, d.layers);
  if (d.hidden != 64 && d.hidden != 128 && d.hidden != 256)
    return fail(SOUFFLE_BAD_SHAPE, "hidden must be 64, 128 or 256 (got %d)", d.hidden);
  if (d.steps < 1) return fail(SOUFFLE_BAD_SHAPE, "steps must be >= 1");
  if ((size_t)d.layers * d.steps * d.hidden > kStaticHiddenFloats)
    return fail(SOUFFLE_BAD_SHAPE, "layers*steps*hidden = %zu exceeds the built-in scratch of %zu values; use a plan",
                (size_t)d.layers * d.steps * d.hidden, kStaticHiddenFloats);
  if (!aligned16(w_in) || !aligned16(w_state) || !aligned16(x) || !aligned16(y))
    return fail(SOUFFLE_BAD_POINTER, "w_in, w_state, x and y must be non-null and 16-byte aligned");
  int dev = 0;
  StaticLstmDevice* sdp = nullptr;
  int rc = static_lstm_device(&dev, &sdp);
  if (rc) return rc;
  StaticLstmDevice& sd = *sdp;
  const size_t smem = lstm_smem_bytes(d.hidden);
  {
    // all clusters must be resident at once: asked of the driver once per (device, layers, hidden)
    const int hi = d.hidden == 64 ? 0 : (d.hidden == 128 ? 1 : 2);
    std::lock_guard<std::mutex> lock(sd.mutex);
    if (!(sd.resident_ok[hi] & (1u << d.layers))) {
      rc = lstm_check_resident(d.layers, smem);
      if (rc) return rc;
      sd.resident_ok[hi] |= 1u << d.layers;
    }
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  unsigned char* ctl = sd.scratch + kStaticHiddenFloats * 4;
  // counters and status must start at zero; the hidden-state slots are all written before they are read
  SF_CUDA(cudaMemsetAsync(ctl, 0, kStaticCtlBytes, st));
  if (device_status) SF_CUDA(cudaMemsetAsync(device_status, 0, 16, st));
  LstmParams lp;
  lp.w_in = reinterpret_cast<const __half*>(w_in);
  lp.w_state = reinterpret_cast<const __half*>(w_state);
  lp.bias = bias; lp.x = x; lp.y = y;
  lp.h_all = reinterpret_cast<float*>(sd.scratch);
  lp.done = reinterpret_cast<unsigned*>(ctl);
  lp.done_next = reinterpret_cast<unsigned*>(ctl) + kLstmDoneWords;
  lp.status = device_status ? reinterpret_cast<int*>(device_status) : reinterpret_cast<int*>(ctl + kStaticStatusOffset);
  lp.layers = d.layers; lp.hidden = d.hidden; lp.steps = d.steps; lp.ref_input_delay = d.ref_input_delay;
  lp.timeout_ns = (unsigned long long)(d.timeout_ms > 0 ? d.timeout_ms : 2000) * 1000000ull;
  return lstm_launch(lp, smem, st);
}

// For callers that passed no device_status: waits for `stream`, then reads the status words the last
// allocation-free call on the current device left in the built-in array (a plain device-to-host copy).
int souffle_lstm_static_status(souffle_stream_t stream) {
  int dev = 0;
  StaticLstmDevice* sd = nullptr;
  int rc = static_lstm_device(&dev, &sd);
  if (rc) return rc;
  SF_CUDA(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  int h[4] = {0, 0, 0, 0};
  SF_CUDA(cudaMemcpy(h, sd->scratch + kStaticHiddenFloats * 4 + kStaticStatusOffset, sizeof(h), cudaMemcpyDeviceToHost));
  return decode_status(h, "souffle_lstm_forward_static");
}

// ======================================================================================
// squeeze-and-excite module
// ======================================================================================
static void se_geometry(int batch, int channels, int hw, int sms, SeParams* p) {
  // cut a channel image into slices until every warp of the grid has one, but not below 512 floats a slice
  const int warps = sms * (kSeThreads / 32);
  int slices = 1;
  const int chans = batch * channels;
  while (chans * slices < warps && hw / (slices * 2) >= 512) slices *= 2;
  int slice_len = (hw + slices - 1) / slices;
  slice_len = (slice_len + 3) & ~3;
  slices = (hw + slice_len - 1) / slice_len;
  p->slices = slices;
  p->slice_len = slice_len;
  p->items = chans * slices;
}

size_t souffle_se_module_workspace_bytes(int32_t batch, int32_t channels, int32_t height, int32_t width) {
  if (batch < 1 || channels < 1 || height < 1 || width < 1) return 256;
  const int hw = height * width;
  const int max_slices = hw / 512 > 1 ? hw / 512 : 1;        // whatever the SM count, a slice has >= 512 floats
  return 256 + (size_t)batch * channels * max_slices * sizeof(float);
}

int souffle_se_module_forward(const float* input, const float* w_reduce, const float* w_expand, float* out, float* pooled,
                              int32_t batch, int32_t channels, int32_t height, int32_t width, int32_t reduce, void* workspace,
                              size_t workspace_bytes, souffle_stream_t stream) {
  if (!input || !w_reduce || !w_expand || !out) return fail(SOUFFLE_BAD_ARGUMENT, "null argument");
  if (batch < 1 || channels < 1 || channels > kSeMaxChannels || height < 1 || width < 1 || reduce < 1 || reduce > kSeMaxReduce)
    return fail(SOUFFLE_BAD_SHAPE, "SE module needs batch, height, width >= 1, 1 <= channels <= %d and 1 <= reduce <= %d",
                kSeMaxChannels, kSeMaxReduce);
  if ((long long)batch * channels * height * width >= (1ll << 31)) return fail(SOUFFLE_BAD_SHAPE, "input too large");
  int dev = 0, sms = 0, cc = 0;
  SF_CUDA(cudaGetDevice(&dev));
  SF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  SF_CUDA(cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev));
  if (cc != 10) return fail(SOUFFLE_BAD_DEVICE, "device %d has compute capability %d.x; this library needs sm_100", dev, cc);
  SeParams p;
  memset(&p, 0, sizeof(p));
  se_geometry(batch, channels, height * width, sms, &p);
  const size_t need = 256 + (size_t)batch * channels * p.slices * sizeof(float);
  if (!aligned16(workspace) || workspace_bytes < need)
    return fail(SOUFFLE_BAD_POINTER, "workspace must be 16-byte aligned and hold %zu bytes", need);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  {
    std::lock_guard<std::mutex> lock(g_ws_mutex);          // first sight of this workspace: clear its control words
    if (g_ws_launches.find(workspace) == g_ws_launches.end()) {
      SF_CUDA(cudaMemsetAsync(workspace, 0, 128, st));
      g_ws_launches.emplace(workspace, 0u);
    }
  }
  const size_t smem = (size_t)(kSeCacheFloats + kSeMaxChannels + kSeMaxReduce) * sizeof(float);
  static bool attr_set[16] = {};
  if (dev < 16 && !attr_set[dev]) {
    SF_CUDA(cudaFuncSetAttribute(souffle_se_module, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set[dev] = true;
  }
  const int warps_per_cta = kSeThreads / 32;
  const int ctas = (p.items + warps_per_cta - 1) / warps_per_cta;
  const int grid = ctas < sms ? ctas : sms;
  const int per_warp = (p.items + grid * warps_per_cta - 1) / (grid * warps_per_cta);
  p.input = input; p.w_reduce = w_reduce; p.w_expand = w_expand; p.out = out; p.pooled = pooled;
  p.sync = reinterpret_cast<unsigned*>(workspace) + 8;        // words 8, 9: the SE barrier (the GEMM entries use 0..3)
  p.status = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + 64);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256);
  p.batch = batch; p.channels = channels; p.hw = height * width; p.reduce = reduce;
  p.cache = (long long)per_warp * p.slice_len <= kSeCacheFloats / warps_per_cta ? 1 : 0;
  p.timeout_ns = 2000ull * 1000000ull;
  void* kargs[] = {&p};
  SF_CUDA(cudaLaunchCooperativeKernel((const void*)souffle_se_module, dim3(grid), dim3(kSeThreads), kargs, smem, st));
  return SOUFFLE_OK;
}

int souffle_workspace_forget(void* workspace) {
  if (!workspace) return fail(SOUFFLE_BAD_ARGUMENT, "null workspace");
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  g_ws_launches.erase(workspace);
  return SOUFFLE_OK;
}

int souffle_workspace_status(void* workspace, souffle_stream_t stream) {
  if (!workspace) return fail(SOUFFLE_BAD_ARGUMENT, "null workspace");
  SF_CUDA(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  int h[4] = {0, 0, 0, 0};
  SF_CUDA(cudaMemcpy(h, reinterpret_cast<char*>(workspace) + 64, sizeof(h), cudaMemcpyDeviceToHost));
  if (h[0] != DEV_OK) {                 // start over: the next call on this workspace clears all of it
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    g_ws_launches.erase(workspace);
  }
  return decode_status(h, "souffle workspace");
}

}  // extern "C"
