// Inline-PTX wrappers shared by the tensor-core kernels (GEMM, attention): mbarriers with bounded
// waits, TMA tile loads, tensor-memory allocation and loads, tcgen05.mma issue and commit, the
// shared-memory matrix descriptor, and the host-side entry to cuTensorMapEncodeTiled.
#pragma once

#include <cuda.h>

#include "common.h"

namespace tq {
namespace {

constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_address(const void* pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ void barrier_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void barrier_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void barrier_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool barrier_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Waits for the phase of `bar` with the given parity, for a bounded number of polls. When the
// bound runs out the device's sticky status word gets `code` (the first give-up wins; tq_status_poll
// reads and clears it) and the launch's abort word is set, which makes every other bounded wait of
// the same launch leave at its next look (every 1024 polls). The launch's first CTA clears the abort
// word when the kernel starts (WaitStatus::begin), so what an earlier launch left there does not
// make this one bail out. The caller must leave its loop on false.
__device__ __forceinline__ bool barrier_wait(uint32_t bar, uint32_t parity, const WaitStatus& status, int code) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (barrier_try_wait(bar, parity)) return true;
    if ((spin & 0x3ff) == 0x3ff && status.aborted()) return false;
  }
  atomicCAS(status.sticky(), 0, code);
  status.set_abort();
  return false;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], 128 x N x 16, issued by one thread. Each descriptor is given as
// its constant high word and its low word (start address and leading offset), so that stepping
// through a tile is one 32-bit add per operand (see descriptor_low for the bit layout).
__device__ __forceinline__ void mma_f16_split(uint32_t tmem_d, uint32_t a_low, uint32_t a_high, uint32_t b_low, uint32_t b_high,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(tmem_d), "r"(a_low), "r"(a_high), "r"(b_low), "r"(b_high), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand lies in tensor memory, one row per lane, two 16-bit
// elements of K per 32-bit column (16 elements of K = 8 columns).
__device__ __forceinline__ void mma_f16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_low, uint32_t b_high, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "r"(b_low), "r"(b_high), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The mbarrier gets one arrival when every tcgen05 operation this thread issued so far is done.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive columns of tensor memory: lane i of the warp gets row i.
__device__ __forceinline__ void tmem_load_32(uint32_t address, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(address)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// The reverse: lane i of the warp writes 32 consecutive columns of row i.
__device__ __forceinline__ void tmem_store_32(uint32_t address, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, as two 32-bit words.
//   low word:  [0,14) start address >> 4, [16,30) leading byte offset >> 4
//   high word: [0,14) stride byte offset >> 4, [14,16) version = 1, [29,32) layout = 2 (SWIZZLE_128B)
// For a K-major operand the stride offset is the distance between 8-row groups (8 x 128 B = 1024)
// and the leading offset is unused; for an MN-major operand the leading offset is the distance
// between 64-element chunks along M/N and the stride offset the distance between groups of 8
// K-rows (again 1024). Stepping 16 elements along K is +32 B (K-major) or +2048 B (MN-major) on the
// start address, i.e. +2 or +128 on the low word.
constexpr uint32_t kDescriptorHigh = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t descriptor_low(uint32_t address, uint32_t leading_bytes) {
  return ((address & 0x3ffff) >> 4) | ((leading_bytes >> 4) << 16);
}

__device__ __forceinline__ float exp2_ftz(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
__device__ __forceinline__ float rcp_ftz(float d) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  return r;
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

// The address, in the cluster's shared window, of the same shared-memory offset in CTA `rank`.
__device__ __forceinline__ uint32_t peer_address(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void remote_expect_tx(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void remote_arrive(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// A TMA load into this CTA's shared memory whose bytes are counted on a barrier that may live in
// the other CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

// The CTA-pair form (cta_group::2): one MMA over both CTAs' tiles, descriptors as (low, high) words.
__device__ __forceinline__ void mma_f16_pair_split(uint32_t tmem_d, uint32_t a_low, uint32_t a_high, uint32_t b_low, uint32_t b_high,
                                                   uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(tmem_d), "r"(a_low), "r"(a_high), "r"(b_low), "r"(b_high), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair, once every
// tcgen05 operation this thread issued so far is done.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both)
               : "memory");
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled function = [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &entry, 12000, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return static_cast<EncodeTiled>(nullptr);
    }
    return reinterpret_cast<EncodeTiled>(entry);
  }();
  return function;
}


}  // namespace
}  // namespace tq
