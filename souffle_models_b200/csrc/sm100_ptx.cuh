// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, never multicast),
// tcgen05 (TMEM alloc / MMA / commit / load) and the bounded-wait helpers the megakernel
// uses.  It replaces the role of cpp/souffle_utils/cuda_kernel_utils.h:8-55 and
// cuda_utils.h:11-19 in the reference (warp reductions, error checks) for a Blackwell design.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace souffle {

// ------------------------------------------------------------------------------------
// error / abort bookkeeping shared by every bounded wait
// ------------------------------------------------------------------------------------
enum DeviceStatus : int {
  DEV_OK = 0,
  DEV_TIMEOUT_MBAR = 1,   // an mbarrier wait ran out of time
  DEV_TIMEOUT_GRID = 2,   // the grid barrier ran out of time
  DEV_TIMEOUT_FLAG = 3,   // a dataflow flag wait ran out of time
};

struct WaitCtl {
  volatile int* abort_smem;        // CTA-local flag: set once, every loop leaves when it is set
  int* status_g;                   // device status words: [0]=code, [1]=where, [2]=cta
  unsigned long long deadline_ns;  // globaltimer value after which waits give up
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __noinline__ void record_timeout(const WaitCtl& c, int code, int where) {
  *c.abort_smem = 1;
  if (atomicCAS(c.status_g, 0, code) == 0) {
    c.status_g[1] = where;
    c.status_g[2] = (int)blockIdx.x;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up when the CTA's abort flag is set or the deadline has passed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtl& c, int where) {
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
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

// Warp-collective bounded wait: one lane polls, the verdict is broadcast.  Keeps 31 lanes per warp
// from hammering the barrier word while the producer and MMA lanes work on its neighbours.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtl& c, int where, int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity, c, where) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// Named barrier among a subset of warps (id 1..15, thread count a multiple of 32).
__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------------------------------
// proxies and fences
// ------------------------------------------------------------------------------------
// Orders generic-proxy writes (st.global / st.shared) before later async-proxy reads (TMA, tcgen05).
// The form without a state space measured ~900 cycles on a B200, the two restricted forms 3 and 10: hot paths name
// the spaces they mean.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------------------------
// TMA: tiled 2-D loads into 128B-swizzled shared memory, completion on an mbarrier.
// The innermost coordinate is always a multiple of 8 halves (16 bytes).
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// Untiled bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Pulls `bytes` (a multiple of 16, 16-byte aligned) of global memory into L2; nothing is written anywhere else.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// Tells L2 that the 128 bytes at `p` (128-byte aligned) hold nothing anybody will read again: the line may be dropped
// without being written back.  Reading it afterwards, before it has been written again, gives unspecified values.
__device__ __forceinline__ void discard_l2_128(const void* p) {
  asm volatile("discard.global.L2 [%0], 128;" ::"l"(p) : "memory");
}
// Tiled 3-D store of a shared-memory box to global memory (rows or planes of the box that lie past the tensor's
// extents are not written).  The copy belongs to the issuing thread's current bulk group.
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(tmap), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most kPending of this thread's bulk groups have not yet READ their shared-memory source.
template <int kPending>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
// Waits until all of this thread's bulk groups are complete (their writes performed).
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ------------------------------------------------------------------------------------
// tcgen05: tensor memory + UMMA
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Shared-memory matrix descriptor for a 128B-swizzled tile whose 8-row groups are 1024 B apart.
//   bits [0,14) start>>4, [16,30) leading byte offset>>4, [32,46) stride byte offset>>4,
//   [46,48) version=1 (Blackwell), [61,64) layout type (2 = SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::f16, fp16 x fp16 -> fp32, A K-major, M=128.
//   [4,6) D format (1=f32), [7,10) A fmt (0=f16), [10,13) B fmt, [15] A major, [16] B major (1 = MN),
//   [17,23) N>>3, [24,29) M>>4.
__device__ __forceinline__ uint32_t umma_idesc_f16(uint32_t n, uint32_t b_mn_major) {
  return (1u << 4) | (b_mn_major << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// High word of a SW128 descriptor (stride byte offset 1024, version 1, layout SWIZZLE_128B) and the
// low word for a tile at `smem_addr` with leading byte offset `lbo_bytes`.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
// One K chunk of 64 (four K=16 steps) in a single instruction sequence.  The issuing thread is a
// lone lane whose every dependent instruction costs several cycles, so the descriptor arithmetic is
// kept to one 32-bit add per operand and step.  `acc0` = 0 makes the first step overwrite D.
__device__ __forceinline__ void umma_f16_k64(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t bstep,
                                             uint32_t idesc, uint32_t acc0) {
  asm volatile(
      "{\n\t.reg .pred p, pt;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"
      "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
      "mov.b64 da, {%1, %6};\n\tmov.b64 db, {%2, %6};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "add.u32 al, %1, 2;\n\tadd.u32 bl, %2, %3;\n\tmov.b64 da, {al, %6};\n\tmov.b64 db, {bl, %6};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 al, al, 2;\n\tadd.u32 bl, bl, %3;\n\tmov.b64 da, {al, %6};\n\tmov.b64 db, {bl, %6};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 al, al, 2;\n\tadd.u32 bl, bl, %3;\n\tmov.b64 da, {al, %6};\n\tmov.b64 db, {bl, %6};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(bstep), "r"(idesc), "r"(acc0), "r"(kDescHiSw128)
      : "memory");
}
// Same for a 256-row tile: two accumulators (d0, d1) and two A tiles 16 KB apart share every B step.
__device__ __forceinline__ void umma_f16_k64_x2(uint32_t d0, uint32_t d1, uint32_t a_lo, uint32_t b_lo, uint32_t bstep,
                                                uint32_t idesc, uint32_t acc0) {
  asm volatile(
      "{\n\t.reg .pred p, pt;\n\t.reg .b64 da, da2, db;\n\t.reg .b32 al, al2, bl;\n\t"
      "setp.ne.b32 p, %6, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
      "add.u32 al2, %2, 1024;\n\t"
      "mov.b64 da, {%2, %7};\n\tmov.b64 da2, {al2, %7};\n\tmov.b64 db, {%3, %7};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], da2, db, %5, p;\n\t"
      "add.u32 al, %2, 2;\n\tadd.u32 al2, al2, 2;\n\tadd.u32 bl, %3, %4;\n\t"
      "mov.b64 da, {al, %7};\n\tmov.b64 da2, {al2, %7};\n\tmov.b64 db, {bl, %7};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], da2, db, %5, pt;\n\t"
      "add.u32 al, al, 2;\n\tadd.u32 al2, al2, 2;\n\tadd.u32 bl, bl, %4;\n\t"
      "mov.b64 da, {al, %7};\n\tmov.b64 da2, {al2, %7};\n\tmov.b64 db, {bl, %7};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], da2, db, %5, pt;\n\t"
      "add.u32 al, al, 2;\n\tadd.u32 al2, al2, 2;\n\tadd.u32 bl, bl, %4;\n\t"
      "mov.b64 da, {al, %7};\n\tmov.b64 da2, {al2, %7};\n\tmov.b64 db, {bl, %7};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, pt;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], da2, db, %5, pt;\n\t}"
      ::"r"(d0), "r"(d1), "r"(a_lo), "r"(b_lo), "r"(bstep), "r"(idesc), "r"(acc0), "r"(kDescHiSw128)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ------------------------------------------------------------------------------------
// CTA pairs (cta_group::2): two CTAs of a cluster of two share every MMA.  An MMA of M = 256 takes 128 rows of A and
// N / 2 columns of B from the shared memory of each CTA (same offsets in both) and leaves rows 128 r .. 128 r + 127 of
// the 256 x N result in the tensor memory of CTA r, so each CTA stores only half of every B tile.  One thread of
// the leader CTA (cluster rank 0) issues for both.  All tcgen05 instructions of a kernel use one CTA group.
// ------------------------------------------------------------------------------------
// one warp of EACH CTA of the pair, the same shared-memory offset for the result in both
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {  // one warp of each CTA
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Instruction descriptor of a pair MMA: M = 256 over the two CTAs, N over both halves of B.
__device__ __forceinline__ uint32_t umma_idesc_f16_pair(uint32_t n, uint32_t b_mn_major) {
  return (1u << 4) | (b_mn_major << 16) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}
// One K chunk of 64 as four pair MMAs (see umma_f16_k64).
__device__ __forceinline__ void umma_f16_k64_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t bstep,
                                                  uint32_t idesc, uint32_t acc0) {
  asm volatile(
      "{\n\t.reg .pred p, pt;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"
      "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
      "mov.b64 da, {%1, %6};\n\tmov.b64 db, {%2, %6};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t"
      "add.u32 al, %1, 2;\n\tadd.u32 bl, %2, %3;\n\tmov.b64 da, {al, %6};\n\tmov.b64 db, {bl, %6};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 al, al, 2;\n\tadd.u32 bl, bl, %3;\n\tmov.b64 da, {al, %6};\n\tmov.b64 db, {bl, %6};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, pt;\n\t"
      "add.u32 al, al, 2;\n\tadd.u32 bl, bl, %3;\n\tmov.b64 da, {al, %6};\n\tmov.b64 db, {bl, %6};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, pt;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(bstep), "r"(idesc), "r"(acc0), "r"(kDescHiSw128)
      : "memory");
}
// Arrives, once every pair MMA issued so far by this thread has completed, on the mbarrier at this shared-memory
// offset in BOTH CTAs of the pair (the commit is multicast over the cluster; it carries no data).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
      ::"r"(bar) : "memory");
}
// Tiled 2-D load into this CTA's shared memory whose completion is counted on an mbarrier of the pair's leader
// (`bar` is a shared::cluster address, see map_shared_rank).  A plain load: nothing is multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// Arrival on an mbarrier of another CTA of the cluster (`bar` is a shared::cluster address).  The release form makes
// the thread's earlier writes visible to whoever sees the phase complete -- and so waits for ALL of them, global
// stores still in flight included (measured: ~1.7 k cycles after an epilogue's stores).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// The same arrival with the default (CTA-scope) release: for hand-shakes that only protect tensor memory, whose
// reads tcgen05.fence::before_thread_sync has already ordered before the arrival; it does not wait for global stores.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 columns of fp32: thread i of the warp receives lane (base+i), columns [col, col+32).
// The loads carry no memory clobber (they only write registers); the matching wait names the same
// registers as read-write operands so the compiler cannot move their uses above it.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]));
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]));
}

// ------------------------------------------------------------------------------------
// global-memory release/acquire for the grid barrier and dataflow flags
// ------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned atom_add_release_u32(unsigned* p, unsigned v) {
  unsigned old;
  asm volatile("atom.add.release.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void red_add_release_u32(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ------------------------------------------------------------------------------------
// thread-block clusters: distributed shared memory and cluster-scope barriers
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA's window) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_shared_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// 4-byte store into the shared memory of any CTA of the cluster that also counts 4 bytes as transferred on an
// mbarrier of that CTA: the value is visible to whoever sees the barrier's phase complete (no fence on either side)
__device__ __forceinline__ void st_async_b32(uint32_t cluster_addr, uint32_t v, uint32_t cluster_mbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
               ::"r"(cluster_addr), "r"(v), "r"(cluster_mbar) : "memory");
}
__device__ __forceinline__ void st_release_cta_shared_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_cta_shared_u32(uint32_t addr, uint32_t v) {
  asm volatile("red.release.cta.shared::cta.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_cta_shared_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// hardware barrier over all threads of the cluster (every warp executes both halves, converged)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ------------------------------------------------------------------------------------
// small math
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// tanh-form GELU (the reference's activate kernel, cpp/bert/bert_base_impl.cu:722-734).
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanh_fast(u));
}
// The same GELU on a pair of fp16 values (the result is stored as fp16 anyway): six packed operations and
// one packed tanh for two elements.  Overflow of x*x saturates tanh at +-1, which is the right limit.
__device__ __forceinline__ uint32_t gelu_tanh_h2(uint32_t xw) {
  const __half2 x = *reinterpret_cast<const __half2*>(&xw);
  const __half2 c0 = __float2half2_rn(0.7978845608028654f), c1 = __float2half2_rn(0.7978845608028654f * 0.044715f);
  const __half2 u = __hmul2(x, __hfma2(__hmul2(x, x), c1, c0));
  uint32_t uw = *reinterpret_cast<const uint32_t*>(&u), tw;
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(tw) : "r"(uw));
  const __half2 t = *reinterpret_cast<const __half2*>(&tw);
  const __half2 hx = __hmul2(x, __float2half2_rn(0.5f));
  const __half2 y = __hfma2(hx, t, hx);
  return *reinterpret_cast<const uint32_t*>(&y);
}
// Sixteen pairs at once, step by step: each loop is sixteen independent operations (see epilogue_chunk32).
__device__ __forceinline__ void gelu_tanh_h2x16(uint32_t (&w)[16]) {
  const __half2 c0 = __float2half2_rn(0.7978845608028654f), c1 = __float2half2_rn(0.7978845608028654f * 0.044715f);
  const __half2 half = __float2half2_rn(0.5f);
  __half2 x[16], t[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = *reinterpret_cast<const __half2*>(&w[i]);
#pragma unroll
  for (int i = 0; i < 16; ++i) t[i] = __hmul2(x[i], x[i]);
#pragma unroll
  for (int i = 0; i < 16; ++i) t[i] = __hfma2(t[i], c1, c0);
#pragma unroll
  for (int i = 0; i < 16; ++i) t[i] = __hmul2(x[i], t[i]);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    uint32_t uw = *reinterpret_cast<const uint32_t*>(&t[i]), tw;
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(tw) : "r"(uw));
    t[i] = *reinterpret_cast<const __half2*>(&tw);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = __hmul2(x[i], half);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const __half2 y = __hfma2(x[i], t[i], x[i]);
    w[i] = *reinterpret_cast<const uint32_t*>(&y);
  }
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace souffle
