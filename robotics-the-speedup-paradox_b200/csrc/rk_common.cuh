// Device-side building blocks for the sm_100a quantized-linear kernels:
// mbarrier, TMA (cp.async.bulk.tensor, never multicast), tcgen05 MMA / TMEM wrappers,
// UMMA shared-memory and instruction descriptors, and bounded waits.
//
// Every wait in these kernels is bounded.  When a wait gives up, the thread records a
// status code in the kernel's status word, raises a CTA-wide abort flag and the kernel
// drains and returns normally (TMEM freed, no trap), so the context stays usable.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace rk {

// Status codes written to the device status word (0 = ok).
enum : int {
  RK_DEV_OK = 0,
  RK_DEV_TIMEOUT_FULL = 101,      // consumer gave up waiting for a TMA stage
  RK_DEV_TIMEOUT_EMPTY = 102,     // producer gave up waiting for a free stage
  RK_DEV_TIMEOUT_ACC = 103,       // epilogue gave up waiting for the accumulator
  RK_DEV_TIMEOUT_XFORM = 104,     // MMA warp gave up waiting for unpacked operands
  RK_DEV_TIMEOUT_ACC_FREE = 105,  // MMA warp gave up waiting for a free accumulator buffer
  RK_DEV_TIMEOUT_RAW = 106,       // unpack warps gave up waiting for a TMA stage
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes, uint32_t on = 1u) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes), "r"(on) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Non-blocking probe of a phase: never parks the thread, so it does not disturb a thread that is
// parked on the same barrier with try_wait.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  `abort_flag` is a CTA-shared word: once any role has given up, every
// other wait returns immediately so that the CTA can drain.  Returns false on give-up.
constexpr uint32_t kWaitSpinFast = 2048;
constexpr uint32_t kWaitSpinMax = 1u << 21;  // with 256 ns sleeps: roughly half a second

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int code, uint32_t spin_max = kWaitSpinMax) {
  // In steady state most waits find their phase already complete.  The non-blocking probe answers
  // that case an order of magnitude faster than the potentially-blocking form (measured: a
  // try_wait that succeeds at once still costs a few hundred cycles), so probe first and park
  // only when there is something to wait for.
  if (mbar_test_wait(bar, parity)) return true;
  for (uint32_t it = 0; it < spin_max; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > kWaitSpinFast) {
      if (*abort_flag) return false;
      __nanosleep(256);
    }
  }
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
  return false;
}

// Warp-level wait by polling.  Lane 0 probes the barrier with the non-blocking form and sleeps a
// few tens of nanoseconds between probes, so several warps may watch one barrier without parking on
// it and without flooding the shared-memory pipe; the verdict reaches the other lanes by shuffle.
// There is no CTA-wide rendezvous: warps that share a role drift freely and the barrier arrival
// counts keep them honest.  Every lane of the warp must call this.  Returns false on give-up.
constexpr uint32_t kPollFast = 64;
__device__ __forceinline__ bool mbar_poll_lane(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               int code) {
  uint32_t it = 0;
  while (!mbar_test_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (++it > kWaitSpinMax) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
    __nanosleep(it < kPollFast ? 20 : 256);
  }
  return true;
}
__device__ __forceinline__ bool mbar_poll_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               int code) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_poll_lane(bar, parity, abort_flag, status, code) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Ring position: stage index plus the phase parity of that stage's barriers.  Advancing costs an
// add, a compare and a select; the single-thread roles (TMA producer, MMA issuer) are latency
// bound, so integer division by a run-time ring depth in their loops would dominate them.
struct Ring {
  int stage;
  uint32_t phase;
  __device__ __forceinline__ void advance(int depth) {
    if (++stage == depth) {
      stage = 0;
      phase ^= 1u;
    }
  }
};


// Group-wide bounded wait with ONE polling thread: the hardware parks a single waiter per
// barrier; further threads polling the same barrier return at once and spin at full issue rate,
// starving the warps that share their scheduler.  So one thread of the group waits on the
// mbarrier and a named hardware barrier (`bar.sync id, nthreads`) releases the rest.
// Every thread of the group must call this; `nthreads` is the group size (multiple of 32).
// `verdict` points at two shared words owned by the group; `iter` counts the group's calls.  The
// leader publishes its result in slot iter & 1 before the named barrier, so every thread of the
// group takes the same decision even if another role raises the abort flag meanwhile (threads
// leaving a loop at different iterations would strand the others on the hardware barrier).
__device__ __forceinline__ bool mbar_wait_group(uint32_t bar, uint32_t parity, bool is_leader, int named_id,
                                                int nthreads, int* abort_flag, int* status, int code,
                                                volatile int* verdict, uint32_t iter,
                                                uint32_t spin_max = kWaitSpinMax) {
  if (is_leader) verdict[iter & 1] = mbar_wait_bounded(bar, parity, abort_flag, status, code, spin_max) ? 1 : 0;
  asm volatile("bar.sync %0, %1;" ::"r"(named_id), "r"(nthreads) : "memory");
  return verdict[iter & 1] != 0;
}

// ---------------------------------------------------------------- TMA (bulk tensor copy, one CTA, no multicast)
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// Asks L2 to fetch one box of a tiled tensor; nothing is delivered to this kernel.  Used for
// weights and scales before the dependency wait: they are parameters, not outputs of the kernel
// that runs before this one, and L2 is the coherence point, so an early fetch can never be stale.
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y) : "memory");
}
// 2-D tile load global -> shared; completion is signalled on `bar` as transaction bytes.
// x (innermost coordinate) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tmap, int x, int y, uint32_t bar,
                                                 uint64_t policy, uint32_t on = 1u) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %6, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;\n\t}"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "l"(policy), "r"(on)
      : "memory");
}
// Three coordinates (innermost first); the x * element-size alignment rule is the same as in 2-D.
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const void* tmap, int x, int y, int z, uint32_t bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
// Tile store shared -> global; rows and columns outside the tensor are clipped by the hardware.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most `N` of this thread's store groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Full completion (writes performed).  A CTA about to exit only needs tma_store_wait_read<0>(): the
// grid's completion makes its bulk stores visible to whatever runs next.
// orders the async proxy's global-memory accesses against the generic proxy's
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// One lane of a converged warp, chosen by the hardware.  The single-thread tcgen05 instructions
// below take the flag as a predicate (`on`): the issuing role then runs as a warp-uniform loop
// whose tcgen05 instructions execute in the elected lane only, instead of as a divergent
// `if (lane == 0)` region (uniform control flow lets the compiler keep descriptors and loop state
// in uniform registers; measured 20-30% fewer cycles per K block for the issuing thread).
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred;
}
// Arrive once on `bar` when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar, uint32_t on = 1u) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar), "r"(on)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp receives lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns, registers -> TMEM (thread t of the warp writes lane base_lane + t)
__device__ __forceinline__ void tmem_st_32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_8(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t r4,
                                          uint32_t r5, uint32_t r6, uint32_t r7) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(r4), "r"(r5), "r"(r6), "r"(r7)
               : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// tcgen05.cp: 32 lanes x 128 bits from shared memory, replicated to the four 32-lane quadrants.
// Used to place block scale factors where the block-scaled MMA reads them.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc, uint32_t on = 1u) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t"
               "@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n\t}" ::"r"(taddr), "l"(sdesc), "r"(on) : "memory");
}

// ---------------------------------------------------------------- UMMA descriptors
// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes of K,
// stored with the 128-byte swizzle (what a SWIZZLE_128B TMA box of {128 B, rows} writes):
//   bits [0,14)  start address >> 4          bits [16,30) leading byte offset >> 4 (unused here)
//   bits [32,46) stride byte offset >> 4     bits [46,48) descriptor version = 1
//   bits [61,64) layout type: 2 = 128-byte swizzle
// Consecutive 8-row groups are 1024 bytes apart (stride byte offset).
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Un-swizzled descriptor (layout type 0) for the scale-factor staging area read by tcgen05.cp:
// 8-row x 16-byte core matrices, rows 16 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_noswizzle(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// Instruction descriptor fields (dense, non-block-scaled kinds):
//   [4,6) D format (0 f16, 1 f32, 2 s32)  [7,10) A format  [10,13) B format
//   [15] A major (0 = K)  [16] B major (0 = K)  [17,23) N>>3  [24,29) M>>4
enum : uint32_t { DFMT_F16 = 0, DFMT_F32 = 1, DFMT_S32 = 2 };
enum : uint32_t { FMT_F16 = 0, FMT_BF16 = 1, FMT_TF32 = 2 };   // kind::f16 / tf32
enum : uint32_t { FMT_U8 = 0, FMT_S8 = 1 };                     // kind::i8
enum : uint32_t { FMT_E4M3 = 0, FMT_E5M2 = 1, FMT_E2M1_IN_F8 = 5 };  // kind::f8f6f4 / mxf8f6f4
enum : uint32_t { FMT_E2M1_MXF4 = 1 };                          // kind::mxf4nvf4

__host__ __device__ constexpr uint32_t umma_idesc(uint32_t dfmt, uint32_t afmt, uint32_t bfmt, uint32_t m,
                                                  uint32_t n) {
  return (dfmt << 4) | (afmt << 7) | (bfmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Block-scaled kinds: [4,6) B scale-factor id, [23] scale format (0 = UE4M3, 1 = UE8M0),
// [29,31) A scale-factor id; D is always f32.
__host__ __device__ constexpr uint32_t umma_idesc_bs(uint32_t afmt, uint32_t bfmt, uint32_t m, uint32_t n,
                                                     uint32_t sf_ue8m0, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | (afmt << 7) | (bfmt << 10) | ((n >> 3) << 17) | (sf_ue8m0 << 23) | ((m >> 4) << 24) |
         (a_sf_id << 29);
}

// D[tmem] (+)= A[smem] * B[smem]^T; issued by one thread.
#define RK_DEFINE_MMA(NAME, KIND)                                                                           \
  __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,     \
                                       uint32_t accumulate, uint32_t on = 1u) {                             \
    asm volatile(                                                                                           \
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"                        \
        "@q tcgen05.mma.cta_group::1.kind::" KIND " [%0], %1, %2, %3, p;\n\t}"                              \
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(on)                         \
        : "memory");                                                                                        \
  }
RK_DEFINE_MMA(mma_i8, "i8")
RK_DEFINE_MMA(mma_f16, "f16")
RK_DEFINE_MMA(mma_f8f6f4, "f8f6f4")
#undef RK_DEFINE_MMA

// D[tmem] (+)= A[tmem] * B[smem]^T: the A operand is a TMEM tile (one row per lane, K along columns)
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate, uint32_t on = 1u) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(on)
      : "memory");
}

__device__ __forceinline__ void mma_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate, uint32_t on = 1u) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %6, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate), "r"(on)
      : "memory");
}
__device__ __forceinline__ void mma_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate, uint32_t on = 1u) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %6, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate), "r"(on)
      : "memory");
}

// Unpredicated forms for a straight-line issue block that only the elected lane enters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_np(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mma_mxf8_np(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_nvf4_np(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
#define RK_DEFINE_MMA_NP(NAME, KIND)                                                                        \
  __device__ __forceinline__ void NAME(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,     \
                                       uint32_t accumulate) {                                               \
    asm volatile(                                                                                           \
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                                  \
        "tcgen05.mma.cta_group::1.kind::" KIND " [%0], %1, %2, %3, p;\n\t}"                                 \
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)                                  \
        : "memory");                                                                                        \
  }
RK_DEFINE_MMA_NP(mma_i8_np, "i8")
RK_DEFINE_MMA_NP(mma_f8f6f4_np, "f8f6f4")
#undef RK_DEFINE_MMA_NP
__device__ __forceinline__ void tc_commit_np(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while its
// predecessor in the stream is still running.  `pdl_launch_dependents` lets the successor's CTAs
// be scheduled as soon as resources free up; `pdl_wait` blocks until the predecessor grid has
// completed and its memory is visible.  Everything before `pdl_wait` must touch on-chip state
// only (barrier init, TMEM allocation, descriptor prefetch) - with one exception: prefetches of
// weights into L2 (tma_prefetch_l2_2d), which deliver no data.  Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Host side: RK_B200_PDL=0 in the environment launches every kernel fully serialized (a debugging aid).
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("RK_B200_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

// Launch of a kernel without dynamic shared memory as a programmatic dependent of its predecessor in
// the stream.  Such a kernel must execute `pdl_wait()` in EVERY thread before it touches global
// memory or returns: then its completion implies its predecessor's, and the chain stays ordered.
// A launch failure surfaces through cudaGetLastError() like one of the <<< >>> form.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------- small numeric helpers
__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace rk
