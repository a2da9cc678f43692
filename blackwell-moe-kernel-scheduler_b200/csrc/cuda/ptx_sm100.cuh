// Inline-PTX building blocks for sm_100a: mbarriers with bounded waits, TMA
// (cp.async.bulk.tensor) loads and stores, tcgen05 tensor-core MMA with
// accumulators in Tensor Memory, and cluster launch control.
//
// Every wait in this file is bounded: it polls a CTA-wide abort word and a wall
// clock budget, and returns false instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cstdint>

namespace bmoe {
namespace ptx {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// True in exactly one lane of a fully converged warp (the same lane on every
// call), so the surrounding loop stays warp-uniform and addresses, descriptors
// and coordinates can live in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t elected;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(elected));
  return elected != 0;
}

// ---------------------------------------------------------------- mbarrier --

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals)
               : "memory");
}

// Makes mbarrier initialisation visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders generic-proxy shared-memory writes before later async-proxy reads.
__device__ __forceinline__ void fence_async_shared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Untiled bulk copies (TMA engine): addresses 16-byte aligned, size a multiple of 16.
// global -> shared, completion counted in bytes on an mbarrier of this CTA.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// shared -> global (local or peer memory), part of the thread's current bulk group.
__device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

// Orders this thread's earlier generic-proxy observations (all state spaces)
// before its later async-proxy operations such as TMA loads.
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Flag written by another GPU (peer stores over NVLink).
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Counter advanced by other CTAs of this GPU.
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
               "r"(bytes)
               : "memory");
}

// One try_wait: returns whether the phase has completed, after at most
// BMOE_TRY_WAIT_HINT_NS nanoseconds of hardware suspension (0 = the plain form with the
// hardware's own short window). With the long hint a waiting warp costs no issue slots
// and no power, which matters under the power cap; measured against the plain form it
// is as fast on latency-bound small launches and 1-4 % faster on the long tensor-bound
// ones. The bounded-wait loops re-check their abort word and time budget at this
// granularity.
#ifndef BMOE_TRY_WAIT_HINT_NS
#define BMOE_TRY_WAIT_HINT_NS 500000
#endif
constexpr uint32_t kSuspendHintNs = BMOE_TRY_WAIT_HINT_NS;

__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  if constexpr (kSuspendHintNs != 0) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return done != 0;
}

// Bounded wait. Returns true once the phase with `parity` has completed, false
// if *abort_word became non-zero or `budget_ns` elapsed (then *abort_word is
// set so that every other role of the CTA gives up as well).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_word,
                                          uint64_t budget_ns) {
  if (mbar_test(bar, parity)) return true;
  uint64_t start = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_test(bar, parity)) return true;
    if ((spin & 0x3f) == 0) {
      if (*abort_word != 0) return false;
      const uint64_t now = global_timer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > budget_ns) {
        *abort_word = 1;
        return false;
      }
    }
  }
}

// --------------------------------------------------------------------- TMA --

// Acquire on a tensor map that lives in global memory and was written by the
// host before the launch; required before the async proxy reads it.
__device__ __forceinline__ void tensormap_acquire(const void* tmap) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(tmap)
               : "memory");
}

__device__ __forceinline__ void tensormap_prefetch(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
// c0 is the innermost (contiguous) coordinate and must keep the start address
// 16-byte aligned.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tmap,
                                            uint32_t bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst_smem),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// 2-D tiled store shared -> global (bulk async group); rows / columns outside
// the tensor extent are clipped by the hardware.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src_smem,
                                             int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::
          "l"(tmap),
      "r"(src_smem), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Waits until at most N committed store groups still READ their shared source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Waits until all committed store groups have fully completed.
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ----------------------------------------------------------------- tcgen05 --

// Whole-warp: allocates `columns` (power of two, 32..512) TMEM columns and
// writes the base address to shared memory at `dst_smem`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   dst_smem),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major BF16 operand tile stored as
// rows of 64 elements (128 bytes) with the 128-byte swizzle, 8-row groups
// 1024 bytes apart (the layout a SWIZZLE_128B TMA box of 64 x rows produces).
//   bits  0-13  start address >> 4
//   bits 16-29  leading-dimension byte offset >> 4 (unused for this layout)
//   bits 32-45  stride byte offset >> 4 (1024 B between 8-row groups)
//   bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  swizzle mode (2 = 128-byte)
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t tile_smem) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((tile_smem & 0x3ffff) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}

// Instruction descriptor for kind::f16: BF16 x BF16 -> FP32, both operands
// K-major, dense, no negation.
//   bits 4-5 D format (1 = F32)   bits 7-9 A format (1 = BF16)
//   bits 10-12 B format (1 = BF16) bit 15/16 A/B major (0 = K-major)
//   bits 17-22 N >> 3              bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t make_bf16_idesc(uint32_t m, uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T for one K=16 slice; issued by one thread.
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t a_desc,
                                             uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor for kind::f8f6f4 with both operands FP8 E4M3 (format code 0),
// FP32 accumulation; the other fields as for kind::f16. One instruction covers K = 32
// elements (the same 32 bytes of a swizzle row as 16 BF16).
__host__ __device__ constexpr uint32_t make_e4m3_idesc(uint32_t m, uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T for one K=32 slice of FP8 E4M3 operands.
__device__ __forceinline__ void umma_e4m3_ss(uint32_t d_tmem, uint64_t a_desc,
                                             uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on `bar` once all tcgen05.mma issued so far by this thread finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          bar)
      : "memory");
}

// Warp-collective: 32 lanes x 32 consecutive FP32 columns starting at taddr
// (lane field = first lane of this warp's quadrant).
__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
      "[%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
        "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
        "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]),
        "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
        "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------- CTA pair (cluster) --
// Two CTAs of one cluster act as a pair ("cta_group::2"): the even-ranked CTA
// issues one 256-row MMA over both CTAs' operand tiles and accumulators.

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem), "r"(rank));
  return remote;
}

// All threads of every CTA in the cluster.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on an mbarrier given by a cluster-wide shared address (own or peer CTA).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}

__device__ __forceinline__ bool mbar_test_cluster(uint32_t bar, uint32_t parity) {
  uint32_t done;
  if constexpr (kSuspendHintNs != 0) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return done != 0;
}

// mbar_wait with cluster-scope acquire (arrivals may come from the peer CTA).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity,
                                                  volatile uint32_t* abort_word,
                                                  uint64_t budget_ns) {
  if (mbar_test_cluster(bar, parity)) return true;
  uint64_t start = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_test_cluster(bar, parity)) return true;
    if ((spin & 0x3f) == 0) {
      if (*abort_word != 0) return false;
      const uint64_t now = global_timer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > budget_ns) {
        *abort_word = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t value) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(value) : "memory");
}

// Pair form of tma_load_2d: the destination is this CTA's shared memory, the
// mbarrier may belong to the peer CTA (cluster-wide address). No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tmap,
                                                 uint32_t cluster_bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst_smem),
      "l"(tmap), "r"(cluster_bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   dst_smem),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr),
               "r"(columns)
               : "memory");
}

// 256 x N x 16 MMA over both CTAs of the pair; issued by one thread of the
// even-ranked CTA. Descriptors name the same offsets in both CTAs' memories.
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t d_tmem, uint64_t a_desc,
                                                  uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same for FP8 E4M3 operands (K = 32 per instruction).
__device__ __forceinline__ void umma_e4m3_ss_pair(uint32_t d_tmem, uint64_t a_desc,
                                                  uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on ONE mbarrier (cluster-wide address, own or peer CTA) once all
// pair MMAs issued so far by this thread have finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          cluster_bar)
      : "memory");
}

// ---------------------------------------------------- cluster launch control --

// Asks the hardware to cancel one not-yet-started CTA of this grid. The
// 16-byte answer lands at `response_smem` and completes 16 bytes on `bar`.
__device__ __forceinline__ void clc_try_cancel(uint32_t response_smem, uint32_t bar) {
  asm volatile(
      "clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128"
      " [%0], [%1];" ::"r"(response_smem),
      "r"(bar)
      : "memory");
}

// Decodes an answer: returns true and the cancelled CTA's blockIdx.x if a CTA
// was cancelled (its work now belongs to the caller), false if none was left.
__device__ __forceinline__ bool clc_query(uint32_t response_smem, uint32_t* cta_x) {
  uint32_t ok, x;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b128 r;\n\t"
      "ld.shared.b128 r, [%2];\n\t"
      "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, r;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "mov.u32 %1, 0;\n\t"
      "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %1, r;\n\t"
      "}"
      : "=r"(ok), "=r"(x)
      : "r"(response_smem)
      : "memory");
  *cta_x = x;
  return ok != 0;
}

// ---------------------------------------------------------------- numerics --

// Two FP32 -> packed BF16x2 with round-to-nearest-even; `lo` goes to the low
// half (lower address).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b,
                                             uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b),
               "r"(c), "r"(d)
               : "memory");
}

}  // namespace ptx
}  // namespace bmoe
