// Flash-attention forward on the tcgen05 tensor cores (bf16 / f16, head dim 64 or 128).
//
// One CTA per SM owns TWO tiles of 128 query rows (A and B, 256 consecutive rows
// of one (batch, head)) and streams the key/value sequence through them in tiles
// of 128 keys.  The single MMA-issuing thread interleaves the two tiles,
//
//     S_A(j)   P.V_B(j-1)   S_B(j)   P.V_A(j)   S_A(j+1)   ...
//
// so that while the softmax warps of one tile work on their scores the tensor
// pipe runs the other tile's two MMAs: each softmax has two MMA slots of cover.
//
//   warp 0       TMA producer: Q_A, Q_B once, then K_j, V_j, K_j+1, ... through a
//                ring of four 32 KB slots (128 rows x 128 B in two 64-column
//                halves, 128-byte swizzle)
//   warp 1       MMA issuer:  S = Q . K_j^T   (A, B from shared memory, K-major)
//                             O += P . V_j    (A = P from TMEM, B = V MN-major),
//                issued as two halves of 64 keys, each as soon as its P is ready.
//                The whole warp walks the loop (waits and descriptor arithmetic
//                stay warp-uniform, descriptors are built once and advanced by
//                adding byte offsets / 16); one elected lane issues a product per
//                branch.
//   warps 2..9   softmax of tile A, warps 10..17 softmax of tile B.  Two threads
//                share a query row: thread (row, h) owns the score columns
//                [32h, 32h+32) and [64+32h, 64+32h+32), handled 16 at a time with
//                the TMEM read (tcgen05.ld) of the next 16 in flight.  Pass 1
//                takes the row maximum, which the two threads exchange through
//                shared memory; pass 2 reads the scores again,
//                p = ex2.approx.ftz(s*scale*log2e - m), f32 partial row sum,
//                P rounded to the operand type and written over the first 16 of
//                the 32 score columns it came from (tcgen05.st), then the half's
//                barrier is signalled.  The running maximum is only replaced, and
//                O and the sums rescaled, when it grows by more than 2^8: the
//                accumulator stays exact in the usual online-softmax sense while
//                rescales stay rare.  Last: the two partial sums are added and
//                each thread writes its half of O * div.approx.ftz(1, sum).
//
// Measured timeline of one step (both tiles, 128 keys) at the heaviest CTA: about
// 3200 clocks, of which the tensor pipe is busy 2048; per tile the chain is
// softmax (about 2000: 480 to the maximum, 1500 for the exponentials at 12 clocks
// per 32 of them and sub-partition) -> P.V second half + S (768) -> hand-offs (380).
// Under sustained load the part runs at its power cap (about 1.7 GHz), so the step
// time in seconds follows the clock.
//
// TMEM (512 columns): S_A [0,128), S_B [128,256), O_A [256,384), O_B [384,512).
// Causal tiles that lie entirely above the diagonal are never visited (tile A
// stops one key tile before tile B); the diagonal tile and the ragged last key
// tile are masked element-wise.
// Work per launch: 4*B*H*D*S*(S+1)/2 flop (causal), 4*B*H*S*D*2 compulsory bytes.
#include <type_traits>

#include "tc.cuh"

namespace b200 {
namespace {

constexpr int kBlockM = 128;                     // query rows per tile (two tiles per CTA)
constexpr int kBlockN = 128;
constexpr int kMaxHeadDim = 128;                 // head dimension is a template parameter: 64 or 128
constexpr int kFirstSoftmaxWarp = 2;             // warp 0: TMA producer, warp 1: MMA issuer
constexpr int kThreads = (kFirstSoftmaxWarp + 16) * 32;     // + 2 tiles x 2 column halves x 4 warps
constexpr int kTmemColumns = 512;
constexpr int kRingSlots = 4;
constexpr uint32_t kTileBytes = 128 * 128 * 2;   // shared-memory slot of one Q / K / V tile (half used at head dim 64)
constexpr uint32_t kHalfBytes = kTileBytes / 2;  // 64-column half
constexpr float kRescaleThreshold = 8.0f;        // log2 units

struct __align__(8) Barriers {
  uint64_t q_full;
  uint64_t slot_full[kRingSlots], slot_empty[kRingSlots];
  uint64_t s_full[2], p_ready[2][2], o_full[2];   // p_ready: [tile][64-key half of the step]
  uint32_t tmem_base;
  int abort_flag;
  int softmax_abort[2][4];            // [tile][quadrant]: one of the two warps of these rows gave up
  // the two threads that share a query row (one per column half) exchange their maxima and sums here
  float exchange[2][2][2][kBlockM];   // maxima: [tile][step parity][column half][row]
  float sums[2][2][kBlockM];          // [tile][column half][row]
};

constexpr size_t kSmemBytes = 1024 + (2 + kRingSlots) * kTileBytes + sizeof(Barriers);

struct Shape {
  int batch, heads_q, seq_q, seq_k, head_group, causal;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  float scale_log2;
};

__device__ __forceinline__ float ex2_approx_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ float div_approx_ftz(float a, float b) {
  float y;
  asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(y) : "f"(a), "f"(b));
  return y;
}

template <typename T> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// Ring bookkeeping shared by producer and consumer: tile i of the K0,V0,K1,V1,.. stream
// lives in slot i % kRingSlots and completes that slot's barriers for the (i / kRingSlots)-th time.
struct RingPosition {
  int slot;
  uint32_t phase;
  __device__ explicit RingPosition(int index) : slot(index % kRingSlots), phase((index / kRingSlots) & 1) {}
};

// What the softmax warps of one query tile need: its barriers, exchange space and TMEM columns.
struct SoftmaxTile {
  uint64_t *s_full, *o_full, *p_ready;   // p_ready: the two 64-key halves of a step
  float (*exchange)[2][kBlockM];         // maxima: [step parity][column half][row]
  float (*sums)[kBlockM];                // [column half][row]
  int *gave_up;                          // of the two warps that own this thread's rows
  uint32_t tmem_s, tmem_o;
  int q0, key_tiles;                     // first query row of the tile, key tiles it walks
  int first_barrier;                     // named barriers first_barrier .. +3, one per quadrant
};

// How the softmax warps wait and arrive: bounded waits that report through the caller's workspace.
struct CtaSync {
  volatile int *abort_flag;
  int *status;
  __device__ bool wait(uint64_t *bar, uint32_t parity, int site) const {
    return tc::mbar_wait(bar, parity, abort_flag, status, site);
  }
  __device__ void arrive(uint64_t *bar) const { tc::mbar_arrive(bar); }
};

// The softmax of one thread's half row over all key tiles, then its half of the output row.  Two threads
// share a query row (`half` 0 / 1 owns score columns [32h, 32h+32) and [64+32h, 64+32h+32)); `quadrant`
// is the warp's TMEM lane quadrant.
template <typename T, int kHeadDim>
__device__ __forceinline__ void softmax_rows(const SoftmaxTile &tile, const CtaSync &sync, const Shape &shape,
                                             T *__restrict__ out, int head, int batch, int half, int quadrant,
                                             int lane) {
  const int row_in_tile = quadrant * 32 + lane;
  const int pair_barrier = tile.first_barrier + quadrant;   // the two warps that own the same 32 rows
  const int q_row = tile.q0 + row_in_tile;
  constexpr int kOutColumns = kHeadDim / 2;     // output columns per thread
  const uint32_t lane_base = static_cast<uint32_t>(quadrant * 32) << 16;
  float reference = -INFINITY;  // maximum the exponentials are taken against (scaled log2 units)
  float sum = 0.0f;             // of this thread's columns only; the halves are added at the end
  bool alive = true;
  for (int j = 0; j < tile.key_tiles; ++j) {
    const uint32_t phase = j & 1;
    // The two warps of a row meet at a named barrier below, so they must leave together: a warp whose
    // wait gave up says so in shared memory and both decide after the barrier.
    const bool ready = sync.wait(tile.s_full, phase, tc::kSiteSoftmax);
    if (!ready) *tile.gave_up = 1;
    tc::tc_fence_after_sync();
    // Two passes over this thread's 64 scores, 16 at a time (TMEM reads are cheap): the read of the next 16
    // is in flight while the current 16 are worked on, and the first read of pass 2 is issued before the
    // two threads of the row meet.  P only ever goes over columns this thread has already consumed.
    const uint32_t my_scores = tile.tmem_s + lane_base + half * 32;   // chunk c: + c * 64
    const int k0 = j * kBlockN + half * 32;                      // first key of chunk 0; chunk 1: + 64
    const bool masked_tile = (j * kBlockN + kBlockN > shape.seq_k) || (shape.causal && j * kBlockN + kBlockN - 1 > tile.q0);
    // score (c, i) holds no valid key when c*64 + i >= limit
    const int limit = shape.causal ? min(shape.seq_k - k0, q_row - k0 + 1) : shape.seq_k - k0;
    auto column_of = [&](int q) { return my_scores + (q >> 1) * 64 + (q & 1) * 16; };   // 16-column group q of 4
    auto mask = [&](uint32_t (&scores)[16], int q) {
      if (masked_tile) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if ((q >> 1) * 64 + (q & 1) * 16 + i >= limit) scores[i] = 0xff800000u;  // -inf
      }
    };
    uint32_t buffer[2][16];
    float partial_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    if (ready) {
      tc::tmem_load_32x16(column_of(0), buffer[0]);
      tc::tmem_load_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        tc::tmem_load_32x16(column_of((q + 1) & 3), buffer[(q + 1) & 1]);   // q = 3: group 0 again, for pass 2
        mask(buffer[q & 1], q);
#pragma unroll
        for (int i = 0; i < 16; ++i) partial_max[i & 3] = fmaxf(partial_max[i & 3], __uint_as_float(buffer[q & 1][i]));
        if (q < 3) tc::tmem_load_wait();
      }
    }
    float tile_max = fmaxf(fmaxf(partial_max[0], partial_max[1]), fmaxf(partial_max[2], partial_max[3]));
    tile.exchange[phase][half][row_in_tile] = tile_max;
    named_barrier_sync(pair_barrier, 64);
    if (*reinterpret_cast<volatile int *>(tile.gave_up)) {
      tc::tmem_load_wait();
      alive = false;
      break;
    }
    tile_max = fmaxf(tile_max, tile.exchange[phase][half ^ 1][row_in_tile]) * shape.scale_log2;
    // A row of the first key tile always holds key 0, so `reference` is finite from j = 0 on.
    const bool grow = tile_max > reference + kRescaleThreshold;
    tc::tmem_load_wait();       // group 0 of pass 2 is in buffer[0]
    if (__any_sync(0xffffffffu, grow)) {
      const float factor = grow ? ex2_approx_ftz(reference - tile_max) : 1.0f;  // 0 on the first tile
      if (grow) { reference = tile_max; sum *= factor; }
      if (j > 0) {
        // S(j) has completed, hence this tile's P.V(j-1) too: O is quiescent until p_ready is signalled
#pragma unroll 1
        for (int chunk = 0; chunk < kOutColumns / 32; ++chunk) {
          uint32_t raw[32];
          tc::tmem_load_32x32(tile.tmem_o + lane_base + half * kOutColumns + chunk * 32, raw);
          tc::tmem_load_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * factor);
          tc::tmem_store_32x32(tile.tmem_o + lane_base + half * kOutColumns + chunk * 32, raw);
        }
      }
    }
    const float offset = -reference;
    float partial_sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q < 3) tc::tmem_load_32x16(column_of(q + 1), buffer[(q + 1) & 1]);
      mask(buffer[q & 1], q);
      uint32_t packed[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float p0 = ex2_approx_ftz(fmaf(__uint_as_float(buffer[q & 1][2 * i]), shape.scale_log2, offset));
        const float p1 = ex2_approx_ftz(fmaf(__uint_as_float(buffer[q & 1][2 * i + 1]), shape.scale_log2, offset));
        partial_sum[(2 * i) & 3] += p0;
        partial_sum[(2 * i + 1) & 3] += p1;
        packed[i] = pack_pair<T>(p0, p1);
      }
      tc::tmem_store_32x8(my_scores + (q >> 1) * 64 + (q & 1) * 8, packed);
      if (q & 1) {           // 64 keys of P are complete
        tc::tmem_store_wait();
        tc::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) sync.arrive(tile.p_ready + (q >> 1));
      }
      if (q < 3) tc::tmem_load_wait();
    }
    sum += (partial_sum[0] + partial_sum[1]) + (partial_sum[2] + partial_sum[3]);
  }
  // the row sum is the sum of both halves (they share the reference maximum)
  tile.sums[half][row_in_tile] = sum;
  named_barrier_sync(pair_barrier, 64);
  sum += tile.sums[half ^ 1][row_in_tile];
  if (alive && sync.wait(tile.o_full, 0, tc::kSiteEpilogueTmemFull)) {
    tc::tc_fence_after_sync();
    const float inverse = div_approx_ftz(1.0f, sum);
    T *destination = out + batch * shape.o_stride_b + head * shape.o_stride_h + (int64_t)q_row * shape.o_stride_s +
                     half * kOutColumns;
    const bool vector_ok = ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && shape.o_stride_b % 8 == 0 &&
                           shape.o_stride_h % 8 == 0 && shape.o_stride_s % 8 == 0;
#pragma unroll 1
    for (int chunk = 0; chunk < kOutColumns / 32; ++chunk) {
      uint32_t raw[32];
      tc::tmem_load_32x32(tile.tmem_o + lane_base + half * kOutColumns + chunk * 32, raw);
      tc::tmem_load_wait();
      if (q_row < shape.seq_q) {
        if (vector_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_pair<T>(__uint_as_float(raw[q * 8 + 0]) * inverse, __uint_as_float(raw[q * 8 + 1]) * inverse);
            v.y = pack_pair<T>(__uint_as_float(raw[q * 8 + 2]) * inverse, __uint_as_float(raw[q * 8 + 3]) * inverse);
            v.z = pack_pair<T>(__uint_as_float(raw[q * 8 + 4]) * inverse, __uint_as_float(raw[q * 8 + 5]) * inverse);
            v.w = pack_pair<T>(__uint_as_float(raw[q * 8 + 6]) * inverse, __uint_as_float(raw[q * 8 + 7]) * inverse);
            *reinterpret_cast<uint4 *>(destination + chunk * 32 + q * 8) = v;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            destination[chunk * 32 + i] = Element<T>::narrow(__uint_as_float(raw[i]) * inverse);
        }
      }
    }
  }
}

template <typename T, int kHeadDim>
__global__ void __launch_bounds__(kThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, T *__restrict__ out, const Shape shape, int *status) {
  extern __shared__ unsigned char raw_smem[];
  unsigned char *tiles = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char *q_tiles = tiles;                       // Q_A, Q_B
  unsigned char *ring = tiles + 2 * kTileBytes;         // kRingSlots tiles
  Barriers *bars = reinterpret_cast<Barriers *>(tiles + (2 + kRingSlots) * kTileBytes);

  constexpr uint32_t kLoadBytes = 128 * kHeadDim * 2;  // bytes TMA delivers per tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heaviest query tiles (most key tiles under the causal mask) are scheduled first
  const int pairs = (shape.seq_q + 2 * kBlockM - 1) / (2 * kBlockM);
  const int pair = pairs - 1 - (int)blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / shape.head_group;
  const int q0 = pair * 2 * kBlockM;                    // first row of tile A; tile B starts at q0 + 128
  const int all_key_tiles = (shape.seq_k + kBlockN - 1) / kBlockN;
  int tiles_of[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    tiles_of[x] = all_key_tiles;
    if (shape.causal) tiles_of[x] = min(all_key_tiles, (q0 + x * kBlockM + kBlockM - 1) / kBlockN + 1);
  }
  const int key_tiles = max(tiles_of[0], tiles_of[1]);  // = tiles_of[1]

  if (threadIdx.x == 0) {
    tc::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kRingSlots; ++s) {
      tc::mbar_init(&bars->slot_full[s], 1);
      tc::mbar_init(&bars->slot_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) {
      tc::mbar_init(&bars->s_full[x], 1);
      tc::mbar_init(&bars->p_ready[x][0], 8);   // one arrival per softmax warp of the tile
      tc::mbar_init(&bars->p_ready[x][1], 8);
      tc::mbar_init(&bars->o_full[x], 1);
    }
    bars->abort_flag = 0;
    for (int i = 0; i < 8; ++i) (&bars->softmax_abort[0][0])[i] = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_descriptor(&map_q);
    tc::tma_prefetch_descriptor(&map_k);
    tc::tma_prefetch_descriptor(&map_v);
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
      tc::mbar_expect_tx(&bars->q_full, 2 * kLoadBytes);
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        tc::tma_load_4d(q_tiles + x * kTileBytes, &map_q, &bars->q_full, 0, q0 + x * kBlockM, head, batch);
        if (kHeadDim > 64)
          tc::tma_load_4d(q_tiles + x * kTileBytes + kHalfBytes, &map_q, &bars->q_full, 64, q0 + x * kBlockM, head, batch);
      }
      int issued = 0;
      bool alive = true;
      for (int index = 0; index < 2 * key_tiles; ++index) {  // K0, V0, K1, V1, ...
        const RingPosition at(index);
        if (!tc::mbar_wait(&bars->slot_empty[at.slot], at.phase ^ 1, abort_flag, status, tc::kSiteProducerEmpty)) {
          alive = false;
          break;
        }
        unsigned char *slot = ring + at.slot * kTileBytes;
        const CUtensorMap *map = (index & 1) ? &map_v : &map_k;
        const int key0 = (index >> 1) * kBlockN;
        tc::mbar_expect_tx(&bars->slot_full[at.slot], kLoadBytes);
        tc::tma_load_4d(slot, map, &bars->slot_full[at.slot], 0, key0, kv_head, batch);
        if (kHeadDim > 64) tc::tma_load_4d(slot + kHalfBytes, map, &bars->slot_full[at.slot], 64, key0, kv_head, batch);
        ++issued;
      }
      if (!alive) {
        // let copies in flight land before the shared memory goes away
        const long long start = clock64();
        while (!tc::mbar_try_wait(&bars->q_full, 0) && clock64() - start < tc::kWaitCycles / 8) {}
        for (int back = 1; back <= min(issued, kRingSlots); ++back) {
          const RingPosition at(issued - back);
          while (!tc::mbar_try_wait(&bars->slot_full[at.slot], at.phase) && clock64() - start < tc::kWaitCycles / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer
    // The whole warp walks the loop, so waits, slot and descriptor arithmetic stay warp-uniform; one
    // elected lane issues the tcgen05 instructions, a whole product per branch.  The issue order
    //   S_A(j), P.V_B(j-1), S_B(j), P.V_A(j), S_A(j+1), ...
    // keeps the two tiles in opposite phase: one tile's softmax runs while the other tile's products
    // occupy the tensor pipe.
    const bool issuer = tc::elect_one();
    constexpr int format = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr uint32_t idesc_s = tc::instr_desc_f16(format, kBlockM, kBlockN, false);
    constexpr uint32_t idesc_o = tc::instr_desc_f16(format, kBlockM, kHeadDim, true);
    // descriptors of the first 16-element slice; a slice further on adds its byte offset / 16
    const uint64_t desc_q = tc::smem_desc_k_major_sw128(tc::smem_u32(q_tiles));
    const uint64_t desc_k = tc::smem_desc_k_major_sw128(tc::smem_u32(ring));
    const uint64_t desc_v = tc::smem_desc_mn_major_sw128(tc::smem_u32(ring), kHalfBytes);

    auto wait_slot = [&](int index) {
      const RingPosition at(index);
      return tc::mbar_wait(&bars->slot_full[at.slot], at.phase, abort_flag, status, tc::kSiteMmaFull);
    };
    auto release_slot = [&](int index) {      // arrives once the products issued so far have read the slot
      if (issuer) tc::mma_commit(&bars->slot_empty[RingPosition(index).slot]);
    };
    // S_x(j) = Q_x . K_j^T into the score columns of tile x
    auto issue_scores = [&](int x, int j) {
      const uint64_t desc_qx = desc_q + ((x * kTileBytes) >> 4);
      const uint64_t desc_kj = desc_k + ((RingPosition(2 * j).slot * kTileBytes) >> 4);
      if (issuer) {
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk) {
          const uint32_t offset = ((kk / 4) * kHalfBytes + (kk % 4) * 32) >> 4;
          tc::mma_f16_ss(tmem_base + x * kBlockN, desc_qx + offset, desc_kj + offset, idesc_s, kk != 0);
        }
        tc::mma_commit(&bars->s_full[x]);
      }
    };
    // O_x += P_x(j) . V_j in two halves of 64 keys, each as soon as its part of P is in TMEM.  Key block kk
    // (16 keys, 8 packed columns) was written by column half (kk%4)/2 of the softmax warps into its own
    // score columns: (kk/4)*64 + ((kk%4)/2)*32 + (kk%2)*8.
    auto issue_values = [&](int x, int j) -> bool {
      const uint64_t desc_vj = desc_v + ((RingPosition(2 * j + 1).slot * kTileBytes) >> 4);
      const uint32_t tmem_s = tmem_base + x * kBlockN, tmem_o = tmem_base + 2 * kBlockN + x * kMaxHeadDim;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        if (!tc::mbar_wait(&bars->p_ready[x][part], j & 1, abort_flag, status, tc::kSiteMmaTmemEmpty)) return false;
        tc::tc_fence_after_sync();
        if (issuer) {
#pragma unroll
          for (int kk = part * 4; kk < part * 4 + 4; ++kk) {
            const uint32_t p_column = (kk / 4) * 64 + ((kk % 4) / 2) * 32 + (kk % 2) * 8;
            // B: 16 key rows = 2048 bytes further down the V tile
            tc::mma_f16_ts(tmem_o, tmem_s + p_column, desc_vj + ((kk * 2048) >> 4), idesc_o, (j | kk) != 0);
          }
          if (part == 1 && j == tiles_of[x] - 1) tc::mma_commit(&bars->o_full[x]);
        }
      }
      return true;
    };

    // Tile A's chain P_A(j) -> P.V_A(j) -> S_A(j+1) is the critical one: K_(j+1) and V_j are waited for
    // while softmax A(j) still runs, so that S_A(j+1) is queued right behind P.V_A(j).
    bool alive = tc::mbar_wait(&bars->q_full, 0, abort_flag, status, tc::kSiteMmaFull) && wait_slot(0);   // Q, K_0
    for (int j = 0; alive && j < key_tiles; ++j) {
      if (j < tiles_of[0]) issue_scores(0, j);
      if (j >= 1) {                                                   // P.V_B(j-1): covers softmax A(j)
        // V_(j-1) was already waited for before P.V_A(j-1) unless tile A had stopped by then
        if ((j - 1 >= tiles_of[0] && !wait_slot(2 * j - 1)) || !issue_values(1, j - 1)) { alive = false; break; }
        release_slot(2 * j - 1);                                      // V_(j-1): both tiles are done with it
      }
      issue_scores(1, j);                                             // tile B sees every key tile
      release_slot(2 * j);                                            // K_j
      if (j + 1 < key_tiles && !wait_slot(2 * j + 2)) { alive = false; break; }   // K_(j+1)
      if (j < tiles_of[0]) {                                          // P.V_A(j): covers softmax B(j)
        if (!wait_slot(2 * j + 1) || !issue_values(0, j)) { alive = false; break; }
      }
    }
    if (alive && (key_tiles - 1 < tiles_of[0] || wait_slot(2 * key_tiles - 1)) && issue_values(1, key_tiles - 1))
      release_slot(2 * key_tiles - 1);
  } else {
    // -------------------------------------------------------------- softmax
    const int x = (warp - kFirstSoftmaxWarp) >> 3;             // 0: tile A, 1: tile B
    SoftmaxTile tile;
    tile.s_full = &bars->s_full[x]; tile.o_full = &bars->o_full[x]; tile.p_ready = bars->p_ready[x];
    tile.exchange = bars->exchange[x]; tile.sums = bars->sums[x]; tile.gave_up = &bars->softmax_abort[x][warp & 3];
    tile.tmem_s = tmem_base + x * kBlockN; tile.tmem_o = tmem_base + 2 * kBlockN + x * kMaxHeadDim;
    tile.q0 = q0 + x * kBlockM; tile.key_tiles = tiles_of[x]; tile.first_barrier = 1 + x * 4;
    softmax_rows<T, kHeadDim>(tile, CtaSync{abort_flag, status}, shape, out, head, batch,
                              ((warp - kFirstSoftmaxWarp) >> 2) & 1, warp & 3, lane);
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemColumns);
  }
}

// Rows with no valid key (an empty key sequence) are zero.
template <typename T>
__global__ void zero_output_kernel(T *out, int64_t total_rows, int heads, int seq, int dv, int64_t sb, int64_t sh,
                                   int64_t ss) {
  const int64_t total = total_rows * dv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / dv, d = i % dv;
    const int64_t b = row / ((int64_t)heads * seq), h = (row / seq) % heads, s = row % seq;
    out[b * sb + h * sh + s * ss + d] = Element<T>::narrow(0.0f);
  }
}

int tensor_map_4d(CUtensorMap *map, const void *base, int64_t d0, int64_t d1, int64_t d2, int64_t d3, int64_t s0,
                  int64_t s1, int64_t s2) {
  // innermost first: (D, S, H, B); a size-1 dimension may carry any stride, give TMA a legal one
  const uint64_t dims[4] = {(uint64_t)d3, (uint64_t)d2, (uint64_t)d1, (uint64_t)d0};
  auto legal = [&](int64_t stride, int64_t extent, int64_t fallback) {
    return (uint64_t)((extent > 1 ? stride : fallback) * 2);
  };
  const int64_t row = (d3 + 7) / 8 * 8;
  const uint64_t strides[3] = {legal(s2, d2, row), legal(s1, d1, row * d2), legal(s0, d0, row * d2 * d1)};
  const uint32_t box[4] = {64, 128, 1, 1};
  return encode_tensor_map_16bit(map, base, 4, dims, strides, box, true);
}

template <typename T, int kHeadDim>
int attention_typed(const T *q, const T *k, const T *v, T *o, const int64_t *qd, const int64_t *qs,
                    const int64_t *kd, const int64_t *ks, const int64_t *vs, const int64_t *os, float scale,
                    int head_group, int causal, int *status, cudaStream_t stream) {
  const int64_t batch = qd[0], heads_q = qd[1], seq_q = qd[2], heads_k = kd[1], seq_k = kd[2];
  if (seq_k == 0) {
    zero_output_kernel<T><<<sm_count() * 4, 256, 0, stream>>>(o, batch * heads_q * seq_q, (int)heads_q, (int)seq_q,
                                                              kHeadDim, os[0], os[1], os[2]);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  CUtensorMap map_q, map_k, map_v;
  int result = tensor_map_4d(&map_q, q, batch, heads_q, seq_q, kHeadDim, qs[0], qs[1], qs[2]);
  if (result != B200_OK) return result;
  result = tensor_map_4d(&map_k, k, batch, heads_k, seq_k, kHeadDim, ks[0], ks[1], ks[2]);
  if (result != B200_OK) return result;
  result = tensor_map_4d(&map_v, v, batch, heads_k, seq_k, kHeadDim, vs[0], vs[1], vs[2]);
  if (result != B200_OK) return result;
  Shape shape;
  shape.batch = (int)batch; shape.heads_q = (int)heads_q; shape.seq_q = (int)seq_q; shape.seq_k = (int)seq_k;
  shape.head_group = head_group; shape.causal = causal;
  shape.o_stride_b = os[0]; shape.o_stride_h = os[1]; shape.o_stride_s = os[2];
  shape.scale_log2 = scale * (float)1.4426950408889634;  // scale * LOG2E, rounded to f32 like the kernel definition
  const dim3 grid((unsigned)((seq_q + 2 * kBlockM - 1) / (2 * kBlockM)), (unsigned)heads_q, (unsigned)batch);
  auto kernel = attention_kernel<T, kHeadDim>;
  B200_CUDA_TRY(opt_in_dynamic_smem(kernel, kSmemBytes));
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, o, shape, status);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_flash_attention(const void *q, int64_t q_d0, int64_t q_d1, int64_t q_d2, int64_t q_d3,
                                    int64_t q_s0, int64_t q_s1, int64_t q_s2, int64_t q_s3,
                                    const void *k, int64_t k_d0, int64_t k_d1, int64_t k_d2, int64_t k_d3,
                                    int64_t k_s0, int64_t k_s1, int64_t k_s2, int64_t k_s3,
                                    const void *v, int64_t v_d0, int64_t v_d1, int64_t v_d2, int64_t v_d3,
                                    int64_t v_s0, int64_t v_s1, int64_t v_s2, int64_t v_s3,
                                    void *o, int64_t o_d0, int64_t o_d1, int64_t o_d2, int64_t o_d3,
                                    int64_t o_s0, int64_t o_s1, int64_t o_s2, int64_t o_s3,
                                    float scale, void *workspace, int64_t ws_d0, int64_t ws_s0,
                                    int32_t dtype, int32_t head_group, int32_t causal, void *stream) {
  const int64_t qd[4] = {q_d0, q_d1, q_d2, q_d3}, qs[4] = {q_s0, q_s1, q_s2, q_s3};
  const int64_t kd[4] = {k_d0, k_d1, k_d2, k_d3}, ks[4] = {k_s0, k_s1, k_s2, k_s3};
  const int64_t vd[4] = {v_d0, v_d1, v_d2, v_d3}, vs[4] = {v_s0, v_s1, v_s2, v_s3};
  const int64_t od[4] = {o_d0, o_d1, o_d2, o_d3}, os[4] = {o_s0, o_s1, o_s2, o_s3};
  for (int i = 0; i < 4; ++i)
    if (qd[i] < 0 || kd[i] < 0 || vd[i] < 0 || od[i] < 0) return fail(B200_ERR_INVALID_ARGUMENT, "flash_attention: negative extent");
  if (head_group < 1 || kd[0] != qd[0] || vd[0] != qd[0] || od[0] != qd[0] || qd[1] != kd[1] * head_group ||
      vd[1] != kd[1] || od[1] != qd[1] || vd[2] != kd[2] || od[2] != qd[2] || kd[3] != qd[3] || od[3] != vd[3])
    return fail(B200_ERR_INVALID_ARGUMENT,
                "flash_attention: q (B,HQ,Q,D), k (B,HK,K,D), v (B,HK,K,DV), o (B,HQ,Q,DV) with HQ = HK * head_group");
  if (qd[0] == 0 || qd[1] == 0 || qd[2] == 0) return B200_OK;
  if (dtype != B200_F16 && dtype != B200_BF16)
    return fail(B200_ERR_INVALID_ARGUMENT, "flash_attention: element type %d is not f16/bf16", dtype);
  if (qd[3] != vd[3] || (qd[3] != 64 && qd[3] != 128))
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "flash_attention: head dimensions must be D == DV in {64, 128} (got D=%lld, DV=%lld)",
                (long long)qd[3], (long long)vd[3]);
  if (!q || !k || !v || !o) return fail(B200_ERR_INVALID_ARGUMENT, "flash_attention: null buffer");
  if (!workspace || ws_d0 < B200_WORKSPACE_WORDS || (ws_d0 > 1 && ws_s0 != 1))
    return fail(B200_ERR_INVALID_ARGUMENT, "flash_attention: workspace must hold %d contiguous int32 words", B200_WORKSPACE_WORDS);
  if (q_s3 != 1 || k_s3 != 1 || v_s3 != 1 || o_s3 != 1)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "flash_attention: innermost strides must be 1");
  const void *bases[3] = {q, k, v};
  const int64_t *strides[3] = {qs, ks, vs};
  const int64_t *extents[3] = {qd, kd, vd};
  for (int t = 0; t < 3; ++t) {
    if (!aligned16(bases[t])) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "flash_attention: TMA needs 16-byte aligned bases");
    for (int axis = 0; axis < 3; ++axis)
      if (extents[t][axis] > 1 && (strides[t][axis] % 8 || strides[t][axis] <= 0))
        return fail(B200_ERR_UNSUPPORTED_LAYOUT, "flash_attention: outer strides must be positive multiples of 8 elements");
  }
  if (qd[2] > INT32_MAX - 256 || kd[2] > INT32_MAX - 256 || qd[1] > 65535 || qd[0] > 65535)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "flash_attention: extent exceeds the launch limits");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200_ATTENTION(T, D)                                                                                    \
  attention_typed<T, D>((const T *)q, (const T *)k, (const T *)v, (T *)o, qd, qs, kd, ks, vs, os, scale, head_group, \
                        causal, (int *)workspace, s)
  if (dtype == B200_F16) return qd[3] == 64 ? B200_ATTENTION(__half, 64) : B200_ATTENTION(__half, 128);
  return qd[3] == 64 ? B200_ATTENTION(__nv_bfloat16, 64) : B200_ATTENTION(__nv_bfloat16, 128);
#undef B200_ATTENTION
}
