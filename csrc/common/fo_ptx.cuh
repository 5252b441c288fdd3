// Inline-PTX wrappers for the Blackwell (sm_100a) features used by the kernels in this
// library: mbarrier, TMA tiled loads (each CTA fetches its own tiles), tcgen05 tensor-core
// MMA with TMEM accumulators, scoped acquire/release flag accesses for cross-GPU
// signalling, and bounded spin-waits that report a status instead of hanging.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "fo_status.h"

namespace fo {
namespace ptx {

#define FO_DEVICE __device__ __forceinline__

FO_DEVICE uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ thread-block clusters

FO_DEVICE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
FO_DEVICE void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
FO_DEVICE void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
FO_DEVICE uint32_t mapa_shared(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// Arrive on an mbarrier that may live in another CTA of the cluster (address from mapa_shared).
FO_DEVICE void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}

// ------------------------------------------------------------------ mbarrier

FO_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

FO_DEVICE void mbar_fence_init() {
  // Make barrier initialisation visible to the async proxy (TMA, tcgen05.commit).
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

FO_DEVICE void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

FO_DEVICE void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

FO_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// The same test with an explicit limit on how long the hardware may keep the thread suspended
// before it returns unsatisfied (it still resumes at once when the phase completes).
FO_DEVICE bool mbar_try_wait_suspend(uint64_t* bar, uint32_t parity, uint32_t suspend_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(suspend_ns)
      : "memory");
  return ok != 0;
}

// One lane of the (converged) warp, chosen by the hardware: true in that lane only.  Roles whose
// loops every lane walks use it to predicate the single-thread instructions (TMA, MMA, commits).
FO_DEVICE bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// Time base of the bounded waits: the SM cycle counter.  Reading %globaltimer costs on the
// order of a microsecond, which is ruinous inside a hand-off between warps that happens several
// times per tile; clock64 costs a few cycles.  Timeouts given in nanoseconds are converted
// with 2 cycles per nanosecond (the SM clock never exceeds 2 GHz), so a wait lasts at least
// as long as asked and at most about twice as long when the clock is throttled.
FO_DEVICE uint64_t cycles_now() { return static_cast<uint64_t>(clock64()); }

// Nanosecond clock shared by all SMs of a GPU (about a microsecond per read: tracing only).
FO_DEVICE uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
FO_DEVICE uint32_t sm_id() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
  return v;
}
FO_DEVICE uint64_t ns_to_cycles(uint64_t ns) { return ns * 2ull; }

// Bounded mbarrier wait.  `abort_flag` is a CTA-shared word any role sets when it gives
// up, so the other roles leave their own waits promptly instead of each running to
// its limit.  After 32 quick polls the thread lets the hardware suspend it for up to
// kMbarSuspendNs per poll; the abort flag and the cycle budget are looked at every 8 of those.
// Returns false on timeout or abort.
constexpr uint32_t kMbarDrainPolls = 1u << 20;  // poll bound used only while draining at exit
constexpr uint32_t kMbarSuspendNs = 4000;       // longest hardware suspension of one slow-path poll

// `sleep_ns` > 0: between the slow-path polls the thread also sleeps that long (an option for
// roles with slack; measured on the plain GEMM it changed neither the instruction count nor the
// time, so the callers' default is 0).
FO_DEVICE bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                 uint64_t timeout_ns, uint32_t sleep_ns = 0) {
  for (uint32_t it = 0; it < (sleep_ns ? 4u : 32u); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  // A wait that has not been satisfied by now is a long one (a role that runs ahead of the
  // pipeline, or an idle epilogue during a main loop): let the hardware park the thread for up
  // to kMbarSuspendNs per poll instead of spinning through the issue slots of a busy SM.
  const uint64_t t0 = cycles_now();
  const uint64_t budget = ns_to_cycles(timeout_ns);
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait_suspend(bar, parity, kMbarSuspendNs)) return true;
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((it & 7u) == 0u) {
      if (*abort_flag) return false;
      if (cycles_now() - t0 > budget) return false;
    }
  }
}

// ------------------------------------------------------------------ TMA (tiled; one CTA per copy)

FO_DEVICE void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
// c0 is the innermost (contiguous) coordinate; c0 * elem_size must be a multiple of 16 B.
// `l2_hint` is an L2 eviction-priority policy word (kL2EvictNormal / First / Last).
constexpr uint64_t kL2EvictNormal = 0x1000000000000000ull;
constexpr uint64_t kL2EvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kL2EvictLast = 0x14F0000000000000ull;

FO_DEVICE void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int32_t c0,
                           int32_t c1, uint64_t l2_hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1), "l"(l2_hint)
      : "memory");
}

// The same load issued by either CTA of a cta_group::2 pair: data lands in the issuing
// CTA's shared memory, the byte count is credited to the barrier at the same offset in the
// pair's leader CTA (bit 24 of a shared::cluster address selects the CTA of the pair).
// Each CTA fetches its own operand slice; nothing is broadcast to the peer.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
FO_DEVICE void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int32_t c0,
                                int32_t c1, uint64_t l2_hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)),
        "r"(smem_u32(bar) & kPeerBitMask), "r"(c0), "r"(c1), "l"(l2_hint)
      : "memory");
}

// 2-D tiled store shared -> global (local or peer memory), tracked by this thread's bulk
// async-group.  The store coordinate x * elem_size must be a multiple of 16 B and neither
// coordinate may be negative.
FO_DEVICE void tma_store_2d(const CUtensorMap* m, const void* smem_src, int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
FO_DEVICE void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// At most N of this thread's most recent bulk groups may still be pending afterwards.
template <int N>
FO_DEVICE void bulk_wait_group() {  // writes of older groups are complete
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
template <int N>
FO_DEVICE void bulk_wait_group_read() {  // sources of older groups have been read
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Orders this thread's generic-proxy shared-memory writes before later async-proxy reads.
FO_DEVICE void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
FO_DEVICE void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// One store, delivered by the NVSwitch to the same offset of every GPU bound to the multicast
// object that `mc_addr` maps.
FO_DEVICE void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

// One load, answered by the NVSwitch with the element-wise sum (accumulated in fp32) of the
// eight 16-bit values at the same offset of every GPU bound to the multicast object.
template <bool BF16>
FO_DEVICE uint4 multimem_ld_reduce_add_v4(const void* mc_addr) {
  uint4 v;
  if constexpr (BF16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
  } else {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
  }
  return v;
}

// ------------------------------------------------------------------ tcgen05 / TMEM

FO_DEVICE void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
FO_DEVICE void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
FO_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

FO_DEVICE void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {  // same warp id in both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
FO_DEVICE void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
FO_DEVICE void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

FO_DEVICE void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
FO_DEVICE void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 B
// (64 x 16-bit) with the 128-byte swizzle TMA applies: 8-row groups are 1024 B apart.
FO_DEVICE uint64_t make_smem_desc_sw128_kmajor(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);  // start address, 16 B units
  d |= static_cast<uint64_t>(1) << 16;                     // leading byte offset (unused for SW128 K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride byte offset: 8 rows * 128 B
  d |= static_cast<uint64_t>(1) << 46;                     // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                     // layout: 128-byte swizzle
  return d;
}

// Instruction descriptor for tcgen05.mma.kind::f16: A,B both K-major 16-bit, fp32 accumulate.
FO_DEVICE constexpr uint32_t make_idesc_f16(bool is_bf16, int umma_m, int umma_n) {
  uint32_t d = 0;
  d |= 1u << 4;                          // D format: F32
  d |= (is_bf16 ? 1u : 0u) << 7;         // A format
  d |= (is_bf16 ? 1u : 0u) << 10;        // B format
  d |= static_cast<uint32_t>(umma_n >> 3) << 17;
  d |= static_cast<uint32_t>(umma_m >> 4) << 24;
  return d;
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
FO_DEVICE void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Pair form: one thread of the leader CTA issues; the two SMs each compute their 128 rows of
// a 256-row tile, A rows and B columns are read from both CTAs' shared memory.
FO_DEVICE void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive (once the pair's MMAs issued so far have completed) on the barrier at this offset in
// every CTA of the cluster selected by `cta_mask`.  This multicast is a barrier signal, not a
// data load.
FO_DEVICE void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// Arrive on `bar` once all MMAs issued so far by this thread have completed.
FO_DEVICE void umma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row (lane base + i).
FO_DEVICE void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
FO_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ named barriers

FO_DEVICE void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------------ scoped flag accesses

FO_DEVICE uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
FO_DEVICE uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Cross-GPU signal: the caller issues ONE release fence for a batch of these (fence + relaxed
// atomic is a release pattern).  A chain of red.release operations would make every atomic
// wait for the previous one's NVLink round trip.
FO_DEVICE void red_relaxed_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
FO_DEVICE void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
FO_DEVICE void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
FO_DEVICE void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

// 16-byte global accesses that bypass L1 (data produced by other SMs or other GPUs).
FO_DEVICE uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
FO_DEVICE void st_v4(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// First writer records the failure; later failures keep the first diagnosis.
FO_DEVICE void report_status(int32_t* status, int32_t code, int32_t a0, int32_t a1, int32_t a2) {
  if (status == nullptr) return;
  if (atomicCAS(&status[kStatusWordCode], 0, code) == 0) {
    status[kStatusWordArg0] = a0;
    status[kStatusWordArg1] = a1;
    status[kStatusWordArg2] = a2;
    __threadfence_system();
  }
}

// Bounded acquire-spin on a 32-bit counter until it reaches `target` (wrap-safe compare).
// `timeout_ns` bounds the wait (see cycles_now); returns false when it gives up.
template <bool kSysScope>
FO_DEVICE bool wait_counter_ge(const uint32_t* p, uint32_t target, uint64_t timeout_ns,
                               volatile int* abort_flag, uint32_t* observed) {
  uint32_t v = 0;
  for (uint32_t it = 0; it < 16u; ++it) {
    v = kSysScope ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (static_cast<int32_t>(v - target) >= 0) {
      *observed = v;
      return true;
    }
  }
  const uint64_t t0 = cycles_now();
  const uint64_t budget = ns_to_cycles(timeout_ns);
  uint32_t it = 0;
  while (true) {
    v = kSysScope ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (static_cast<int32_t>(v - target) >= 0) {
      *observed = v;
      return true;
    }
    __nanosleep(32);
    if ((++it & 63u) == 0u) {
      if (abort_flag != nullptr && *abort_flag) break;
      if (cycles_now() - t0 > budget) break;
    }
  }
  *observed = v;
  return false;
}

}  // namespace ptx
}  // namespace fo
