// Blackwell (sm_100a) building blocks shared by the tensor-core kernels:
// mbarriers with bounded waits, TMA tiled loads, tcgen05 MMA / TMEM access,
// shared-memory and instruction descriptors, and the host-side tensor-map
// encoder.  Everything is inline PTX; no CUTLASS / CuTe types are involved.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace b200 {
namespace tc {

// ---- status words in the caller's workspace -----------------------------
// word 0: sticky non-zero when a bounded wait gave up; word 1: the site id.
enum WaitSite : int {
  kSiteProducerEmpty = 1,
  kSiteMmaFull = 2,
  kSiteMmaTmemEmpty = 3,
  kSiteEpilogueTmemFull = 4,
  kSiteSoftmax = 5,
  kSiteCorrection = 6,
  kSiteDrain = 7,
  kSiteOther = 8,
  kSiteSelfTest = 9,
};

// About two seconds at 2 GHz; a wait that long means a lost arrival.
constexpr long long kWaitCycles = 4000000000ll;

__device__ __forceinline__ uint32_t smem_u32(const void *pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t predicate = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(predicate));
  return predicate != 0;
}

// ---- mbarrier ------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns false when the wait gave up or another role already
// aborted (`*abort_flag` non-zero, a shared-memory word); the first role to give
// up publishes the site in the workspace so the host can report it.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          int *status, int site, long long limit = kWaitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ffu) == 0) {
      if (*abort_flag) return false;
      if (clock64() - start > limit) {
        *abort_flag = 1;
        if (atomicCAS(status, 0, 1) == 0) status[1] = site;
        __threadfence();
        return false;
      }
    }
  }
  return true;
}

// ---- TMA -----------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// 2-D tiled load, completion counted in bytes on `bar`.  x is the innermost
// coordinate and must keep x * element_size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *smem, const CUtensorMap *map, uint64_t *bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem, const CUtensorMap *map, uint64_t *bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *smem, const CUtensorMap *map, uint64_t *bar, int x, int y, int z,
                                            int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// 2-D tiled store from shared memory (bulk async group).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, const void *smem, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int PENDING> __device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory");
}
template <int PENDING> __device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(PENDING) : "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store / UMMA)
__device__ __forceinline__ void fence_async_shared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMEM ------------------------------------------------------------------
// Whole-warp instructions.  `columns` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t *slot_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(slot_in_smem)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- descriptors -----------------------------------------------------------
// Shared-memory operand descriptor for a K-major tile whose rows are exactly
// one 128-byte swizzle span (64 16-bit elements), written by TMA with
// CU_TENSOR_MAP_SWIZZLE_128B at a 1024-byte aligned address: 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused.
// Stepping along K inside the span adds the byte offset to the start address.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(uint32_t smem_address) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);  // start address, 16-byte units
  desc |= static_cast<uint64_t>(1024u >> 4) << 32;               // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;                        // descriptor version (sm_100)
  desc |= static_cast<uint64_t>(2) << 61;                        // SWIZZLE_128B
  return desc;
}

// Shared-memory descriptor of an MN-major operand (the contiguous direction is
// M or N, not K) made of TMA boxes of [64 elements x rows] with 128-byte
// swizzle: inside a box, consecutive K rows are 128 bytes apart and groups of 8
// rows 1024 bytes apart (stride byte offset); boxes that continue the MN
// direction are `mn_chunk_bytes` apart (leading byte offset).  Stepping K by 16
// rows adds 2048 bytes to the start address.
__device__ __forceinline__ uint64_t smem_desc_mn_major_sw128(uint32_t smem_address, uint32_t mn_chunk_bytes) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);
  desc |= static_cast<uint64_t>((mn_chunk_bytes & 0x3ffffu) >> 4) << 16;  // leading byte offset
  desc |= static_cast<uint64_t>(1024u >> 4) << 32;                        // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}

// Instruction descriptor of tcgen05.mma.kind::f16: f32 accumulate, both
// operands K-major, no negation / sparsity / saturation.
// format: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t instr_desc_f16(int format, int m, int n, bool b_mn_major = false) {
  return (1u << 4) | (static_cast<uint32_t>(format) << 7) | (static_cast<uint32_t>(format) << 10) |
         (b_mn_major ? (1u << 16) : 0u) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] . B[smem]; one thread issues for the CTA.
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]  (A operand read from tensor memory).
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar)) : "memory");
}

// ---- CTA pairs (cta_group::2) ------------------------------------------------
// Two CTAs of a cluster on the two SMs of a TPC issue ONE MMA over a 256-row tile: each CTA
// holds its 128 rows of A, its half of B's N columns and its 128 lanes of the accumulator; the
// even CTA (rank 0, the "leader") issues for both.  Each CTA loads its own halves with plain
// (unicast) TMA copies whose completion bytes are counted on the LEADER's barrier; commits
// arrive on the barrier at the same shared-memory offset in both CTAs.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
// Every thread of every CTA of the cluster; also orders shared-memory accesses across the pair.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of this CTA's shared-memory location `smem_address` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_address(uint32_t smem_address, uint32_t rank) {
  uint32_t mapped;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(mapped) : "r"(smem_address), "r"(rank));
  return mapped;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void store_cluster_u32(uint32_t cluster_word, uint32_t value) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_word), "r"(value) : "memory");
}
// 2-D tiled load into THIS CTA's shared memory; the bytes complete on `cluster_bar`, a barrier
// of the pair's leader given as a cluster address.  Unicast: every CTA fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(void *smem, const CUtensorMap *map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
// Whole-warp, issued by the same warp of BOTH CTAs with the same shared-memory slot offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *slot_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(slot_in_smem)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
// D[tmem of both CTAs] (+)= A . B over the pair; issued by one thread of the leader.
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive, once the pair's MMAs issued so far have completed, on the barrier at `bar`'s offset in
// every CTA of `cta_mask` (bit i = CTA rank i).  This is a barrier arrival, not a data copy.
__device__ __forceinline__ void mma_commit_pair(uint64_t *bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(cta_mask) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane
// (base lane + i), columns [column, column + 32).
__device__ __forceinline__ void tmem_load_32x32(uint32_t address, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_store_32x32(uint32_t address, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(address),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_store_32x16(uint32_t address, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(address),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns (see tmem_load_32x32).
__device__ __forceinline__ void tmem_load_32x16(uint32_t address, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address)
      : "memory");
}
__device__ __forceinline__ void tmem_store_32x8(uint32_t address, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}

}  // namespace tc

// ---- host: tensor maps -----------------------------------------------------
// Encodes a tiled tensor map over 16-bit elements with 128-byte swizzle.
// dims/strides are innermost first; strides (in bytes) are given for
// dimensions 1.. and must be multiples of 16.  Returns a B200_* status.
int encode_tensor_map_16bit(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                            const uint64_t *strides_bytes, const uint32_t *box, bool swizzle128);

}  // namespace b200
