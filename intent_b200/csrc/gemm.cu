// Dense GEMM  C[M,N] = cast(A[M,K] . B[K,N])  on the tcgen05 tensor cores.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: A (128 x 64) and B (256 x 64) K-major tiles,
//               128-byte swizzled, into a kStages-deep shared-memory ring
//   warp 1      MMA issuer: tcgen05.mma 128x256x16 (kind::f16, f32 accumulate)
//               into one of two 256-column TMEM accumulators
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator, convert,
//               store C; runs while the next tile's main loop fills the
//               other accumulator
// mbarriers: full/empty per ring stage, full/empty per accumulator.  Every
// wait is bounded (see tc::mbar_wait); a wait that gives up raises the status
// word in the caller's workspace and the CTA drains and exits.
//
// Work per launch: 2*M*N*K flop; compulsory traffic (M*K + K*N + M*N)*2 bytes.
// Tiles are walked in groups of kGroupM row-tiles per B column-tile so the
// CTAs running together share A/B panels through L2.
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "tc.cuh"

namespace b200 {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;   // one 128-byte swizzle span of 16-bit elements
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kAccumulators = 2;
constexpr int kTmemColumns = kAccumulators * kBlockN;  // 512
constexpr int kGroupM = 16;
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;

constexpr uint32_t kBytesA = kBlockM * kBlockK * 2;
constexpr uint32_t kBytesB = kBlockN * kBlockK * 2;
constexpr uint32_t kStageBytes = kBytesA + kBytesB;
constexpr uint32_t kChunkBytesB = 64 * kBlockK * 2;  // one 64-column chunk of an N-major B stage

struct __align__(8) Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[kAccumulators];
  uint64_t tmem_empty[kAccumulators];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr size_t kSmemBytes = 1024 /* alignment slack */ + kStages * kStageBytes + sizeof(Barriers);

struct TileWalk {
  int tiles_m, tiles_n, total;
  __device__ void locate(int tile, int *m, int *n) const {
    const int group_span = kGroupM * tiles_n;
    const int group = tile / group_span;
    const int first_m = group * kGroupM;
    const int rows_in_group = min(kGroupM, tiles_m - first_m);
    const int within = tile - group * group_span;
    *m = first_m + within % rows_in_group;
    *n = within / rows_in_group;
  }
};

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// B_N_MAJOR: B is stored with N contiguous (row-major (K,N)); its stage is then four
// boxes of 64 N-columns x 64 K-rows (8 KB each) and the MMA reads it as an MN-major operand.
template <typename T, bool RELU, bool B_N_MAJOR = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            T *__restrict__ c, int64_t c_pitch, int m, int n, int k, int *status) {
  extern __shared__ unsigned char raw_smem[];
  unsigned char *tiles = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~static_cast<uintptr_t>(1023));
  Barriers *bars = reinterpret_cast<Barriers *>(tiles + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  TileWalk walk;
  walk.tiles_m = (m + kBlockM - 1) / kBlockM;
  walk.tiles_n = (n + kBlockN - 1) / kBlockN;
  walk.total = walk.tiles_m * walk.tiles_n;
  const int k_blocks = (k + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&bars->full[s], 1);
      tc::mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < kAccumulators; ++a) {
      tc::mbar_init(&bars->tmem_full[a], 1);
      tc::mbar_init(&bars->tmem_empty[a], kEpilogueThreads / 32);
    }
    bars->abort_flag = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_descriptor(&map_a);
    tc::tma_prefetch_descriptor(&map_b);
  }
  if (warp == 1) tc::tmem_alloc(&bars->tmem_base, kTmemColumns);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int *abort_flag = &bars->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (tc::elect_one()) {
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;  // ring slots handed to TMA (for the drain below)
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < walk.total; tile += gridDim.x) {
        int tm, tn;
        walk.locate(tile, &tm, &tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!tc::mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, status, tc::kSiteProducerEmpty)) {
            alive = false;
            break;
          }
          unsigned char *slot = tiles + stage * kStageBytes;
          tc::mbar_expect_tx(&bars->full[stage], kStageBytes);
          tc::tma_load_2d(slot, &map_a, &bars->full[stage], kb * kBlockK, tm * kBlockM);
          if (B_N_MAJOR) {
#pragma unroll
            for (int chunk = 0; chunk < kBlockN / 64; ++chunk)
              tc::tma_load_2d(slot + kBytesA + chunk * kChunkBytesB, &map_b, &bars->full[stage],
                              tn * kBlockN + chunk * 64, kb * kBlockK);
          } else {
            tc::tma_load_2d(slot + kBytesA, &map_b, &bars->full[stage], kb * kBlockK, tn * kBlockN);
          }
          ++issued;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!alive) {
        // Let copies already in flight land before the CTA's shared memory is released.
        const uint32_t pending = issued < (uint32_t)kStages ? issued : (uint32_t)kStages;
        for (uint32_t back = 1; back <= pending; ++back) {
          const uint32_t slot_index = issued - back;
          const uint32_t s = slot_index % kStages, ph = (slot_index / kStages) & 1;
          const long long start = clock64();
          while (!tc::mbar_try_wait(&bars->full[s], ph) && clock64() - start < tc::kWaitCycles / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer
    if (tc::elect_one()) {
      constexpr uint32_t idesc = tc::instr_desc_f16(sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0,
                                                    kBlockM, kBlockN, B_N_MAJOR);
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < walk.total; tile += gridDim.x) {
        if (!tc::mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1, abort_flag, status, tc::kSiteMmaTmemEmpty)) break;
        tc::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * kBlockN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!tc::mbar_wait(&bars->full[stage], phase, abort_flag, status, tc::kSiteMmaFull)) {
            alive = false;
            break;
          }
          tc::tc_fence_after_sync();
          const uint32_t a_address = tc::smem_u32(tiles + stage * kStageBytes);
          const uint64_t desc_a = tc::smem_desc_k_major_sw128(a_address);
          const uint64_t desc_b = tc::smem_desc_k_major_sw128(a_address + kBytesA);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            // +32 bytes per K step inside the swizzle span = +2 in 16-byte units
            if (B_N_MAJOR)  // 16 K-rows of 128 bytes further down every 64-column chunk
              tc::mma_f16_ss(tmem_d, desc_a + 2 * kk,
                             tc::smem_desc_mn_major_sw128(a_address + kBytesA + kk * 2048, kChunkBytesB), idesc,
                             (kb | kk) != 0);
            else
              tc::mma_f16_ss(tmem_d, desc_a + 2 * kk, desc_b + 2 * kk, idesc, (kb | kk) != 0);
          }
          tc::mma_commit(&bars->empty[stage]);  // frees the ring slot when these MMAs retire
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!alive) break;
        tc::mma_commit(&bars->tmem_full[acc]);
        if (++acc == kAccumulators) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    const int quadrant = warp & 3;  // TMEM lanes [32*quadrant, +32) belong to this warp
    uint32_t acc = 0, acc_phase = 0;
    for (int tile = blockIdx.x; tile < walk.total; tile += gridDim.x) {
      int tm, tn;
      walk.locate(tile, &tm, &tn);
      if (!tc::mbar_wait(&bars->tmem_full[acc], acc_phase, abort_flag, status, tc::kSiteEpilogueTmemFull)) break;
      tc::tc_fence_after_sync();
      const int row = tm * kBlockM + quadrant * 32 + lane;
      const int column0 = tn * kBlockN;
      T *destination = c + (int64_t)row * c_pitch + column0;
      const bool vector_ok = (c_pitch % 8 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
#pragma unroll 1
      for (int chunk = 0; chunk < kBlockN / 32; ++chunk) {
        uint32_t v[32];
        tc::tmem_load_32x32(tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + acc * kBlockN + chunk * 32, v);
        tc::tmem_load_wait();
        if (row < m) {
          const int column = column0 + chunk * 32;
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            f[i] = __uint_as_float(v[i]);
            if (RELU) f[i] = (f[i] != f[i]) ? f[i] : fmaxf(f[i], 0.0f);
          }
          if (vector_ok && column + 32 <= n) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 packed;
              packed.x = pack2<T>(f[q * 8 + 0], f[q * 8 + 1]);
              packed.y = pack2<T>(f[q * 8 + 2], f[q * 8 + 3]);
              packed.z = pack2<T>(f[q * 8 + 4], f[q * 8 + 5]);
              packed.w = pack2<T>(f[q * 8 + 6], f[q * 8 + 7]);
              *reinterpret_cast<uint4 *>(destination + chunk * 32 + q * 8) = packed;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (column + i < n) destination[chunk * 32 + i] = Element<T>::narrow(f[i]);
          }
        }
      }
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&bars->tmem_empty[acc]);
      if (++acc == kAccumulators) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemColumns);
  }
}

// ---------------------------------------------------------------------------
// CTA-pair kernel (cta_group::2).  Two CTAs on the two SMs of a TPC share one 256 x 256 tile:
// each loads its own 128 rows of A and its own 128 of B's 256 columns (plain unicast TMA, no
// multicast), the pair's leader issues tcgen05.mma over M = 256, and each CTA ends up with its
// 128 rows of the accumulator in its own TMEM.  Against the single-CTA 128 x 256 tile this
// halves the bytes of B an SM pulls from L2 and reads from shared memory per flop (32 KB per
// 64-deep K block and CTA instead of 48 KB).  The epilogue goes TMEM -> registers -> 128-byte
// swizzled shared memory -> cp.async.bulk.tensor store, so C leaves the SM as full 128-byte
// rows of a 128 x 64 box instead of 32 scattered 64-byte pieces per warp store.
//   warp 0      TMA producer (every CTA; completion bytes counted on the leader's barrier)
//   warp 1      MMA issuer (leader only); both CTAs' warp 1 allocate / free TMEM together
//   warps 2..5  epilogue, two staging buffers, one thread issues the stores
// Requires B K-major and a C that TMA can store (16-byte aligned base, pitch a multiple of 8).
// ---------------------------------------------------------------------------
namespace pair {

constexpr int kTileM = 256, kTileN = 256;      // per pair
constexpr int kCtaM = 128, kCtaN = 128;        // rows of A / columns of B each CTA loads
constexpr int kStages = 6;
constexpr uint32_t kBytesA = kCtaM * kBlockK * 2;
constexpr uint32_t kBytesB = kCtaN * kBlockK * 2;
constexpr uint32_t kStageBytes = kBytesA + kBytesB;             // 32 KB
constexpr int kStoreColumns = 64;                                // one 128-byte swizzle span of 16-bit elements
constexpr uint32_t kStoreBytes = kCtaM * kStoreColumns * 2;     // 16 KB
constexpr int kStoreBuffers = 2;
constexpr int kEpilogueBarrier = 1;                              // named barrier of the four epilogue warps

struct __align__(8) Barriers {
  uint64_t full[kStages];        // leader's: both CTAs' tiles of a stage have landed
  uint64_t empty[kStages];       // every CTA's own: the pair's MMAs have read the stage
  uint64_t tmem_full[kAccumulators];
  uint64_t tmem_empty[kAccumulators];   // leader's: both CTAs' epilogues have drained the accumulator
  uint32_t tmem_base;
  int abort_flag;
  int epilogue_abort;            // an epilogue warp gave up: the four warps leave together
};

constexpr size_t kSmemBytes = 1024 + kStages * kStageBytes + kStoreBuffers * kStoreBytes + sizeof(Barriers);

struct TileWalk {
  int tiles_m, tiles_n, total;
  __device__ void locate(int tile, int *m, int *n) const {
    const int group_rows = kGroupM / 2;                 // 8 pair tiles = the 16 row tiles of the single-CTA walk
    const int group_span = group_rows * tiles_n;
    const int group = tile / group_span;
    const int first_m = group * group_rows;
    const int rows_in_group = min(group_rows, tiles_m - first_m);
    const int within = tile - group * group_span;
    *m = first_m + within % rows_in_group;
    *n = within / rows_in_group;
  }
};

// A wait that gives up also raises the peer's abort flag, so the pair winds down together.
__device__ __forceinline__ bool wait(uint64_t *bar, uint32_t parity, Barriers *bars, uint32_t peer, int *status, int site) {
  if (tc::mbar_wait(bar, parity, &bars->abort_flag, status, site)) return true;
  tc::store_cluster_u32(tc::cluster_address(tc::smem_u32(&bars->abort_flag), peer), 1u);
  return false;
}

template <typename T, bool RELU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, int m, int n, int k, int *status) {
  extern __shared__ unsigned char raw_smem[];
  unsigned char *tiles = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char *staging = tiles + kStages * kStageBytes;
  Barriers *bars = reinterpret_cast<Barriers *>(staging + kStoreBuffers * kStoreBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_cta_rank();
  const bool leader = rank == 0;
  const int pairs = gridDim.x / 2, pair_id = blockIdx.x / 2;
  TileWalk walk;
  walk.tiles_m = (m + kTileM - 1) / kTileM;
  walk.tiles_n = (n + kTileN - 1) / kTileN;
  walk.total = walk.tiles_m * walk.tiles_n;
  const int k_blocks = (k + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&bars->full[s], 1);
      tc::mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < kAccumulators; ++a) {
      tc::mbar_init(&bars->tmem_full[a], 1);
      tc::mbar_init(&bars->tmem_empty[a], 2 * kEpilogueThreads / 32);   // four warps of each CTA
    }
    bars->abort_flag = 0;
    bars->epilogue_abort = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_descriptor(&map_a);
    tc::tma_prefetch_descriptor(&map_b);
    tc::tma_prefetch_descriptor(&map_c);
  }
  if (warp == 1) tc::tmem_alloc_pair(&bars->tmem_base, kTmemColumns);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::cluster_sync();            // the peer's barriers exist before anything arrives on them
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (tc::elect_one()) {
      uint32_t stage = 0, phase = 0;
      uint32_t issued = 0;
      bool alive = true;
      for (int tile = pair_id; alive && tile < walk.total; tile += pairs) {
        int tm, tn;
        walk.locate(tile, &tm, &tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!wait(&bars->empty[stage], phase ^ 1, bars, rank ^ 1, status, tc::kSiteProducerEmpty)) {
            alive = false;
            break;
          }
          unsigned char *slot = tiles + stage * kStageBytes;
          const uint32_t leader_full = tc::cluster_address(tc::smem_u32(&bars->full[stage]), 0);
          if (leader) tc::mbar_expect_tx(&bars->full[stage], 2 * kStageBytes);   // both CTAs' bytes
          tc::tma_load_2d_pair(slot, &map_a, leader_full, kb * kBlockK, tm * kTileM + (int)rank * kCtaM);
          tc::tma_load_2d_pair(slot + kBytesA, &map_b, leader_full, kb * kBlockK, tn * kTileN + (int)rank * kCtaN);
          ++issued;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!alive && leader) {
        // Let copies already in flight (the peer's too: they complete on these barriers) land
        // before the pair's shared memory is released.
        const uint32_t pending = issued < (uint32_t)kStages ? issued : (uint32_t)kStages;
        for (uint32_t back = 1; back <= pending; ++back) {
          const uint32_t slot_index = issued - back;
          const uint32_t s = slot_index % kStages, ph = (slot_index / kStages) & 1;
          const long long start = clock64();
          while (!tc::mbar_try_wait(&bars->full[s], ph) && clock64() - start < tc::kWaitCycles / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer
    if (leader && tc::elect_one()) {
      constexpr uint32_t idesc = tc::instr_desc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, kTileM, kTileN, false);
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool alive = true;
      for (int tile = pair_id; alive && tile < walk.total; tile += pairs) {
        if (!wait(&bars->tmem_empty[acc], acc_phase ^ 1, bars, 1, status, tc::kSiteMmaTmemEmpty)) break;
        tc::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * kTileN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!wait(&bars->full[stage], phase, bars, 1, status, tc::kSiteMmaFull)) {
            alive = false;
            break;
          }
          tc::tc_fence_after_sync();
          const uint32_t a_address = tc::smem_u32(tiles + stage * kStageBytes);
          const uint64_t desc_a = tc::smem_desc_k_major_sw128(a_address);
          const uint64_t desc_b = tc::smem_desc_k_major_sw128(a_address + kBytesA);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk)
            tc::mma_f16_ss_pair(tmem_d, desc_a + 2 * kk, desc_b + 2 * kk, idesc, (kb | kk) != 0);
          tc::mma_commit_pair(&bars->empty[stage], 3);   // frees the slot in both CTAs
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!alive) break;
        tc::mma_commit_pair(&bars->tmem_full[acc], 3);
        if (++acc == kAccumulators) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    const int quadrant = warp & 3;                      // TMEM lanes [32 * quadrant, +32) belong to this warp
    const int row_in_tile = quadrant * 32 + lane;       // of this CTA's 128 rows
    const bool issuer = warp == 2 && lane == 0;
    const uint32_t leader_empty0 = tc::cluster_address(tc::smem_u32(&bars->tmem_empty[0]), 0);
    const uint32_t leader_empty1 = tc::cluster_address(tc::smem_u32(&bars->tmem_empty[1]), 0);
    uint32_t acc = 0, acc_phase = 0;
    uint32_t buffer = 0;
    for (int tile = pair_id; tile < walk.total; tile += pairs) {
      int tm, tn;
      walk.locate(tile, &tm, &tn);
      // The four warps meet at named barriers below, so they must take the same way out: a warp
      // whose wait gave up says so in shared memory, and all of them decide after one barrier.
      if (!wait(&bars->tmem_full[acc], acc_phase, bars, rank ^ 1, status, tc::kSiteEpilogueTmemFull))
        bars->epilogue_abort = 1;
      asm volatile("bar.sync %0, %1;" ::"n"(kEpilogueBarrier), "n"(kEpilogueThreads) : "memory");
      if (*reinterpret_cast<volatile int *>(&bars->epilogue_abort)) break;
      tc::tc_fence_after_sync();
      const int row0 = tm * kTileM + (int)rank * kCtaM;
      const int column0 = tn * kTileN;
#pragma unroll 1
      for (int chunk = 0; chunk < kTileN / kStoreColumns; ++chunk) {
        // the store that read this staging buffer two chunks ago has finished reading it
        if (issuer) tc::tma_store_wait_read<kStoreBuffers - 1>();
        asm volatile("bar.sync %0, %1;" ::"n"(kEpilogueBarrier), "n"(kEpilogueThreads) : "memory");
        unsigned char *out = staging + buffer * kStoreBytes + row_in_tile * 128;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t v[32];
          tc::tmem_load_32x32(tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + acc * kTileN +
                                  chunk * kStoreColumns + half * 32, v);
          tc::tmem_load_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              f[i] = __uint_as_float(v[q * 8 + i]);
              if (RELU) f[i] = (f[i] != f[i]) ? f[i] : fmaxf(f[i], 0.0f);
            }
            uint4 packed;
            packed.x = pack2<T>(f[0], f[1]);
            packed.y = pack2<T>(f[2], f[3]);
            packed.z = pack2<T>(f[4], f[5]);
            packed.w = pack2<T>(f[6], f[7]);
            // 128-byte swizzle: the 16-byte piece c of row r sits at piece c ^ (r & 7)
            const int piece = (half * 4 + q) ^ (row_in_tile & 7);
            *reinterpret_cast<uint4 *>(out + piece * 16) = packed;
          }
        }
        if (chunk == kTileN / kStoreColumns - 1) {
          // the accumulator is in registers / shared memory: hand it back to the MMA issuer
          tc::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
        }
        tc::fence_async_shared();
        asm volatile("bar.sync %0, %1;" ::"n"(kEpilogueBarrier), "n"(kEpilogueThreads) : "memory");
        if (issuer) {
          tc::tma_store_2d(&map_c, staging + buffer * kStoreBytes, column0 + chunk * kStoreColumns, row0);
          tc::tma_store_commit();
        }
        buffer ^= 1;
      }
      if (++acc == kAccumulators) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) tc::tma_store_wait<0>();                // C is written before the CTA leaves
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  tc::cluster_sync();            // neither CTA frees TMEM or shared memory the other may still use
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc_pair(tmem_base, kTmemColumns);
  }
}

}  // namespace pair

// C = 0 for an empty reduction (K == 0).
template <typename T>
__global__ void zero_fill_kernel(T *c, int64_t c_pitch, int m, int n) {
  const int64_t total = (int64_t)m * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    c[(i / n) * c_pitch + i % n] = Element<T>::narrow(0.0f);
}

// ---- tensor-map cache -------------------------------------------------------
struct MapKey {
  const void *base;
  uint64_t d0, d1, stride;
  uint32_t b0, b1;
  bool operator==(const MapKey &o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && stride == o.stride && b0 == o.b0 && b1 == o.b1;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey &k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    for (uint64_t v : {k.d0, k.d1, k.stride, (uint64_t)k.b0, (uint64_t)k.b1}) h = h * 1000003u ^ v;
    return h;
  }
};

int cached_map_2d(CUtensorMap *out, const void *base, uint64_t inner, uint64_t outer, uint64_t stride_bytes,
                  uint32_t box_inner, uint32_t box_outer) {
  static std::mutex lock;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, inner, outer, stride_bytes, box_inner, box_outer};
  std::lock_guard<std::mutex> guard(lock);
  auto found = cache.find(key);
  if (found != cache.end()) {
    *out = found->second;
    return B200_OK;
  }
  const uint64_t dims[2] = {inner, outer};
  const uint64_t strides[1] = {stride_bytes};
  const uint32_t box[2] = {box_inner, box_outer};
  const int status = encode_tensor_map_16bit(out, base, 2, dims, strides, box, true);
  if (status != B200_OK) return status;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return B200_OK;
}

// CTA pairs the device runs at once (one CTA per SM; cached per device).
int resident_pairs(const void *kernel) {
  static std::mutex lock;
  static int known[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return sm_count() / 2;
  std::lock_guard<std::mutex> guard(lock);
  if (known[device] == 0) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(sm_count() / 2 * 2));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = pair::kSmemBytes;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters < 1) clusters = sm_count() / 2;
    known[device] = clusters < sm_count() / 2 ? clusters : sm_count() / 2;
  }
  return known[device];
}

template <typename T>
int gemm_pair_typed(const T *a, const T *b, T *c, int64_t m, int64_t n, int64_t k, int64_t a_pitch, int64_t b_pitch,
                    int64_t c_pitch, int relu, int *status, cudaStream_t stream) {
  CUtensorMap map_a, map_b, map_c;
  int result = cached_map_2d(&map_a, a, (uint64_t)k, (uint64_t)m, (uint64_t)a_pitch * 2, kBlockK, pair::kCtaM);
  if (result != B200_OK) return result;
  result = cached_map_2d(&map_b, b, (uint64_t)k, (uint64_t)n, (uint64_t)b_pitch * 2, kBlockK, pair::kCtaN);
  if (result != B200_OK) return result;
  result = cached_map_2d(&map_c, c, (uint64_t)n, (uint64_t)m, (uint64_t)c_pitch * 2, pair::kStoreColumns, pair::kCtaM);
  if (result != B200_OK) return result;
  auto kernel = relu ? pair::gemm_pair_kernel<T, true> : pair::gemm_pair_kernel<T, false>;
  B200_CUDA_TRY(opt_in_dynamic_smem(kernel, pair::kSmemBytes));
  const int64_t tiles = ((m + pair::kTileM - 1) / pair::kTileM) * ((n + pair::kTileN - 1) / pair::kTileN);
  const int64_t resident = resident_pairs(reinterpret_cast<const void *>(kernel));
  const int pairs = (int)(tiles < resident ? tiles : resident);
  kernel<<<2 * pairs, kThreads, pair::kSmemBytes, stream>>>(map_a, map_b, map_c, (int)m, (int)n, (int)k, status);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// INTENT_B200_GEMM_KERNEL = single | pair overrides the choice below (read at every call).
bool use_pair_kernel(bool eligible, int64_t m, int64_t n) {
  const char *choice = getenv("INTENT_B200_GEMM_KERNEL");
  if (choice && strcmp(choice, "single") == 0) return false;
  if (choice && strcmp(choice, "pair") == 0) return eligible;
  // a pair works on 256 x 256 tiles: worth it once the problem has a wave of them
  return eligible && ((m + 255) / 256) * ((n + 255) / 256) >= sm_count() / 2;
}

template <typename T>
int gemm_typed(const T *a, const T *b, T *c, int64_t m, int64_t n, int64_t k, int64_t a_pitch,
               int64_t b_pitch, int64_t c_pitch, int relu, bool b_n_major, int *status, cudaStream_t stream) {
  if (k == 0) {
    zero_fill_kernel<T><<<sm_count() * 4, 256, 0, stream>>>(c, c_pitch, (int)m, (int)n);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  const bool storable = aligned16(c) && c_pitch % 8 == 0 && c_pitch >= n;
  if (use_pair_kernel(!b_n_major && storable, m, n))
    return gemm_pair_typed<T>(a, b, c, m, n, k, a_pitch, b_pitch, c_pitch, relu, status, stream);
  CUtensorMap map_a, map_b;
  int result = cached_map_2d(&map_a, a, (uint64_t)k, (uint64_t)m, (uint64_t)a_pitch * 2, kBlockK, kBlockM);
  if (result != B200_OK) return result;
  result = b_n_major
      ? cached_map_2d(&map_b, b, (uint64_t)n, (uint64_t)k, (uint64_t)b_pitch * 2, 64, kBlockK)
      : cached_map_2d(&map_b, b, (uint64_t)k, (uint64_t)n, (uint64_t)b_pitch * 2, kBlockK, kBlockN);
  if (result != B200_OK) return result;
  auto kernel = b_n_major ? (relu ? gemm_kernel<T, true, true> : gemm_kernel<T, false, true>)
                          : (relu ? gemm_kernel<T, true, false> : gemm_kernel<T, false, false>);
  B200_CUDA_TRY(opt_in_dynamic_smem(kernel, kSmemBytes));
  const int64_t tiles = ((m + kBlockM - 1) / kBlockM) * ((n + kBlockN - 1) / kBlockN);
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, c, c_pitch, (int)m, (int)n, (int)k, status);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace

// ---- host: tensor-map encoder (driver entry point, no link-time libcuda) ----
int encode_tensor_map_16bit(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                            const uint64_t *strides_bytes, const uint32_t *box, bool swizzle128) {
  typedef CUresult (*Encode)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                             const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Encode encode = nullptr;
  static std::once_flag once;
  static cudaError_t lookup_error = cudaSuccess;
  std::call_once(once, [] {
    void *pointer = nullptr;
    cudaDriverEntryPointQueryResult query;
    lookup_error = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pointer, cudaEnableDefault, &query);
    if (lookup_error == cudaSuccess && query == cudaDriverEntryPointSuccess) encode = reinterpret_cast<Encode>(pointer);
  });
  if (!encode) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable (%s)", cudaGetErrorString(lookup_error));
  cuuint32_t element_strides[5] = {1, 1, 1, 1, 1};
  const CUresult result = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, (cuuint32_t)rank, const_cast<void *>(base),
                                 dims, strides_bytes, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "cuTensorMapEncodeTiled rejected the layout (CUresult %d)", (int)result);
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gemm(const void *a, int64_t a_d0, int64_t a_d1, int64_t a_s0, int64_t a_s1,
                         const void *b, int64_t b_d0, int64_t b_d1, int64_t b_s0, int64_t b_s1,
                         void *c, int64_t c_d0, int64_t c_d1, int64_t c_s0, int64_t c_s1,
                         void *workspace, int64_t ws_d0, int64_t ws_s0,
                         int32_t dtype, int32_t relu, void *stream) {
  const int64_t m = a_d0, k = a_d1, n = b_d1;
  if (m < 0 || n < 0 || k < 0 || b_d0 != k || c_d0 != m || c_d1 != n)
    return fail(B200_ERR_INVALID_ARGUMENT, "gemm: a is %lldx%lld, b is %lldx%lld, c is %lldx%lld",
                (long long)a_d0, (long long)a_d1, (long long)b_d0, (long long)b_d1, (long long)c_d0, (long long)c_d1);
  if (m == 0 || n == 0) return B200_OK;
  if (!c || (k > 0 && (!a || !b))) return fail(B200_ERR_INVALID_ARGUMENT, "gemm: null buffer");
  if (!workspace || ws_d0 < B200_WORKSPACE_WORDS || (ws_d0 > 1 && ws_s0 != 1))
    return fail(B200_ERR_INVALID_ARGUMENT, "gemm: workspace must hold %d contiguous int32 words", B200_WORKSPACE_WORDS);
  if (dtype != B200_F16 && dtype != B200_BF16)
    return fail(B200_ERR_INVALID_ARGUMENT, "gemm: element type %d is not f16/bf16", dtype);
  if (n > 1 && c_s1 != 1) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gemm: c must be row-major (c_s1 == 1)");
  if (k > 1 && a_s1 != 1) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gemm: a must be K-major (a_s1 == 1)");
  // B: K-major (b_s0 == 1, "column-major (K,N)") or N-major (b_s1 == 1, row-major (K,N))
  const bool b_k_major = k <= 1 || b_s0 == 1;
  const bool b_n_major = !b_k_major && (n <= 1 || b_s1 == 1);
  if (!b_k_major && !b_n_major)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gemm: b needs a unit stride along K (b_s0 == 1) or along N (b_s1 == 1)");
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gemm: extent exceeds int32");
  // a 1-row / 1-column operand has a free leading stride; give TMA a legal one
  const int64_t a_pitch = m > 1 ? a_s0 : (k + 7) / 8 * 8;
  const int64_t b_pitch = b_n_major ? (k > 1 ? b_s0 : (n + 7) / 8 * 8) : (n > 1 ? b_s1 : (k + 7) / 8 * 8);
  const int64_t b_inner = b_n_major ? n : k;
  if (k > 0 && (a_pitch % 8 || b_pitch % 8 || a_pitch < k || b_pitch < b_inner || !aligned16(a) || !aligned16(b)))
    return fail(B200_ERR_UNSUPPORTED_LAYOUT,
                "gemm: TMA needs 16-byte aligned bases and leading strides that are multiples of 8 elements and "
                "cover the contiguous extent");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == B200_F16)
    return gemm_typed<__half>((const __half *)a, (const __half *)b, (__half *)c, m, n, k, a_pitch, b_pitch, c_s0,
                              relu, b_n_major, (int *)workspace, s);
  return gemm_typed<__nv_bfloat16>((const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, (__nv_bfloat16 *)c, m, n, k,
                                   a_pitch, b_pitch, c_s0, relu, b_n_major, (int *)workspace, s);
}

// ---------------------------------------------------------------------------
// b200_gemm_static_scratch: the same GEMM for callers that cannot allocate.
//
// The kernel's only scratch is the pair of status words that the bounded waits
// write when they give up.  Here those words live in a file-scope device array
// that every GPU loading this library carries until the process exits, so the
// caller hands over nothing but its operands.
// ---------------------------------------------------------------------------
namespace b200 {
namespace {

// Fixed footprint: kStaticScratchWords int32 words (256 bytes) per GPU.  The
// kernel uses words 0 and 1 whatever the problem size, so the limit that a call
// can exceed is the extent limit stated at the entry, not the scratch itself.
constexpr int kStaticScratchWords = B200_WORKSPACE_WORDS;
static __device__ __align__(256) int static_scratch[kStaticScratchWords];

// `static_scratch` is only a stand-in for the device symbol in host code; the
// address a kernel may be given comes from cudaGetSymbolAddress, once per
// device, with that device current.
constexpr int kMaxDevices = 64;
int *static_scratch_address[kMaxDevices];
std::mutex static_scratch_lock;

int resolve_static_scratch(int **address) {
  int device = -1;
  B200_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices)
    return fail(B200_ERR_DEVICE, "gemm_static_scratch: device ordinal %d is outside [0, %d)", device, kMaxDevices);
  std::lock_guard<std::mutex> guard(static_scratch_lock);
  if (!static_scratch_address[device]) {
    void *pointer = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&pointer, static_scratch));
    static_scratch_address[device] = static_cast<int *>(pointer);
  }
  *address = static_scratch_address[device];
  return B200_OK;
}

template <typename T>
int gemm_static_scratch_typed(const T *a, const T *b, T *c, int64_t m, int64_t n, int64_t k, int64_t a_pitch,
                              int64_t b_pitch, int64_t c_pitch, int relu, int *status, cudaStream_t stream) {
  if (k == 0) {
    zero_fill_kernel<T><<<sm_count() * 4, 256, 0, stream>>>(c, c_pitch, (int)m, (int)n);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  // Tensor maps are encoded on the stack: no cache, no heap.
  CUtensorMap map_a, map_b;
  const uint64_t dims_a[2] = {(uint64_t)k, (uint64_t)m}, dims_b[2] = {(uint64_t)k, (uint64_t)n};
  const uint64_t stride_a[1] = {(uint64_t)a_pitch * 2}, stride_b[1] = {(uint64_t)b_pitch * 2};
  const uint32_t box_a[2] = {kBlockK, kBlockM}, box_b[2] = {kBlockK, kBlockN};
  int result = encode_tensor_map_16bit(&map_a, a, 2, dims_a, stride_a, box_a, true);
  if (result != B200_OK) return result;
  result = encode_tensor_map_16bit(&map_b, b, 2, dims_b, stride_b, box_b, true);
  if (result != B200_OK) return result;
  auto kernel = relu ? gemm_kernel<T, true> : gemm_kernel<T, false>;
  B200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
  const int64_t tiles = ((m + kBlockM - 1) / kBlockM) * ((n + kBlockN - 1) / kBlockN);
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, c, c_pitch, (int)m, (int)n, (int)k, status);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" int b200_gemm_static_scratch(const void *a, int64_t a_d0, int64_t a_d1, int64_t a_s0, int64_t a_s1,
                                        const void *b, int64_t b_d0, int64_t b_d1, int64_t b_s0, int64_t b_s1,
                                        void *c, int64_t c_d0, int64_t c_d1, int64_t c_s0, int64_t c_s1,
                                        int32_t dtype, int32_t relu, int32_t wait_and_check, void *stream) {
  const int64_t m = a_d0, k = a_d1, n = b_d1;
  if (m < 0 || n < 0 || k < 0 || b_d0 != k || c_d0 != m || c_d1 != n)
    return fail(B200_ERR_INVALID_ARGUMENT, "gemm_static_scratch: a is %lldx%lld, b is %lldx%lld, c is %lldx%lld",
                (long long)a_d0, (long long)a_d1, (long long)b_d0, (long long)b_d1, (long long)c_d0, (long long)c_d1);
  if (m > B200_STATIC_SCRATCH_MAX_EXTENT || n > B200_STATIC_SCRATCH_MAX_EXTENT || k > B200_STATIC_SCRATCH_MAX_EXTENT)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT,
                "gemm_static_scratch: extents %lld x %lld x %lld exceed the supported maximum of %lld per dimension",
                (long long)m, (long long)n, (long long)k, (long long)B200_STATIC_SCRATCH_MAX_EXTENT);
  if (m == 0 || n == 0) return B200_OK;
  if (!c || (k > 0 && (!a || !b))) return fail(B200_ERR_INVALID_ARGUMENT, "gemm_static_scratch: null buffer");
  if (dtype != B200_F16 && dtype != B200_BF16)
    return fail(B200_ERR_INVALID_ARGUMENT, "gemm_static_scratch: element type %d is not f16/bf16", dtype);
  if (n > 1 && c_s1 != 1) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gemm_static_scratch: c must be row-major (c_s1 == 1)");
  if (k > 1 && a_s1 != 1) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gemm_static_scratch: a must be K-major (a_s1 == 1)");
  if (k > 1 && b_s0 != 1)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gemm_static_scratch: b must be K-major (b_s0 == 1, column-major (K,N))");
  const int64_t a_pitch = m > 1 ? a_s0 : (k + 7) / 8 * 8;
  const int64_t b_pitch = n > 1 ? b_s1 : (k + 7) / 8 * 8;
  if (k > 0 && (a_pitch % 8 || b_pitch % 8 || a_pitch < k || b_pitch < k || !aligned16(a) || !aligned16(b)))
    return fail(B200_ERR_UNSUPPORTED_LAYOUT,
                "gemm_static_scratch: TMA needs 16-byte aligned bases and leading strides that are multiples of 8 "
                "elements and >= K");
  int *scratch = nullptr;
  int result = resolve_static_scratch(&scratch);
  if (result != B200_OK) return result;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left: the sticky status words must start at zero.
  B200_CUDA_TRY(cudaMemsetAsync(scratch, 0, 2 * sizeof(int), s));
  if (dtype == B200_F16)
    result = gemm_static_scratch_typed<__half>((const __half *)a, (const __half *)b, (__half *)c, m, n, k, a_pitch,
                                               b_pitch, c_s0, relu, scratch, s);
  else
    result = gemm_static_scratch_typed<__nv_bfloat16>((const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b,
                                                      (__nv_bfloat16 *)c, m, n, k, a_pitch, b_pitch, c_s0, relu,
                                                      scratch, s);
  if (result != B200_OK || !wait_and_check) return result;
  int words[2] = {0, 0};
  B200_CUDA_TRY(cudaMemcpyAsync(words, scratch, sizeof words, cudaMemcpyDeviceToHost, s));
  B200_CUDA_TRY(cudaStreamSynchronize(s));
  if (words[0] != 0)
    return fail(B200_ERR_DEVICE_TIMEOUT, "gemm_static_scratch: a bounded device-side wait gave up (site %d)", words[1]);
  return B200_OK;
}
