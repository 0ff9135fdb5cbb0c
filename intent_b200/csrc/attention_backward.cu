// Attention backward (f16 / bf16, head dim 64 or 128) on the tcgen05 tensor cores: the delta
// row-dot kernel, and ONE kernel template for both gradient kernels.
//
// dK/dV and dQ have the same shape of work.  A CTA keeps two "stationary" tiles X0, X1 (128 rows)
// in shared memory and streams pairs of tiles Y0, Y1 past them:
//
//                 stationary X0, X1     streamed Y0, Y1      TMEM lanes     per-column / per-row
//   MODE 0 dK,dV  K, V (128 keys)       Q, dO (128 queries)  keys           lse, delta per column
//   MODE 1 dQ     Q, dO (128 queries)   K, V (128 keys)      queries        lse, delta per row
//
// per step:   T0 = X0 . Y0^T,  T1 = X1 . Y1^T                    (two SS MMAs, f32 in TMEM)
//             P  = ex2(T0 * scale*log2e - lse*log2e), 0 where key > query (causal)
//             G  = P * (T1 - delta)
//             P, G rounded to 16 bits and written back over T0, T1  (compute warps, thread = lane)
//             acc1 += G . Y0      (dK += dS^T . Q   /  dQ += dS . K)   TS MMA, Y0 as MN-major B
//             acc0 += P . Y1      (dV += P^T . dO;  MODE 0 only)
// end:        out0 = acc1 * scale,  out1 = acc0.
//
// MODE 0 walks the HEAD_GROUP query heads of its key head and, when causal, only the query tiles
// at or after its key tile; MODE 1 walks the key tiles up to its query tile.  Rows beyond a
// sequence end are zero-filled by TMA; for queries beyond the end lse is taken as +inf so P = G = 0.
//
//   warp 0      TMA producer (X0, X1 once; Y0, Y1 through a ring)
//   warp 1      MMA issuer (one elected thread)
//   warps 2..9  compute: two threads per TMEM lane, 64 columns of T0 and T1 each (32 at a time); a
//               thread writes its packed P, G over the first 32 of its own 64 columns
// Every mbarrier wait is bounded; a wait that gives up raises the CTA's abort flag and reports
// its site in the caller's workspace words.
#include <mutex>
#include <type_traits>

#include "tc.cuh"

namespace b200 {
namespace {

constexpr int kTile = 128;
constexpr int kThreads = 320;      // producer warp, MMA warp, 2 column halves x 4 compute warps
constexpr int kTmemColumns = 512;
constexpr float kLog2e = 1.4426950408889634f;

template <int kHeadDim> struct Layout {
  static constexpr uint32_t kTileBytes = kTile * kHeadDim * 2;
  static constexpr uint32_t kHalfBytes = kTile * 64 * 2;          // one 64-column half of a tile
  static constexpr int kStages = kHeadDim == 64 ? 4 : 2;
};

struct __align__(16) Barriers {
  uint64_t x_full, y_full[4], y_empty[4], t0_full, t1_full, p_ready, g_ready, acc_full;
  uint32_t tmem_base;
  int abort_flag;
  __align__(16) float columns[8][2][kTile / 2];   // MODE 0: [compute warp][lse*log2e | delta][its 64 query columns] of the current step
};

struct Shape {
  int heads_q, heads_k, seq_q, seq_k, head_group, causal;
  float score_scale, scale;
  int64_t lse_stride[3], delta_stride[3], out0_stride[3], out1_stride[3];
};

__device__ __forceinline__ float ex2_approx_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// A load the compiler may not sink to its first use: issued here, it is in flight while the
// volatile statements that follow (barrier waits, TMEM traffic) run.
__device__ __forceinline__ float load_now(const float *pointer) {
  float value;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(value) : "l"(pointer));
  return value;
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

template <typename T, int kHeadDim, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
attention_backward_kernel(const __grid_constant__ CUtensorMap map_x0, const __grid_constant__ CUtensorMap map_x1,
                          const __grid_constant__ CUtensorMap map_y0, const __grid_constant__ CUtensorMap map_y1,
                          const float *__restrict__ lse, const float *__restrict__ delta, T *__restrict__ out0,
                          T *__restrict__ out1, const Shape shape, int *status) {
  using L = Layout<kHeadDim>;
  constexpr int kStages = L::kStages;
  extern __shared__ unsigned char raw_smem[];
  unsigned char *tiles = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char *x_tiles = tiles;                               // X0, X1
  unsigned char *ring = tiles + 2 * L::kTileBytes;              // kStages x (Y0, Y1)
  Barriers *bars = reinterpret_cast<Barriers *>(ring + kStages * 2 * L::kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heaviest tiles first: the first key tile (MODE 0) and the last query tile (MODE 1) walk the most steps
  const int tile_index = MODE == 1 ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int row0 = tile_index * kTile;                          // first key (MODE 0) / query (MODE 1) of the CTA
  const int streamed_extent = MODE == 0 ? shape.seq_q : shape.seq_k;
  const int streamed_tiles = (streamed_extent + kTile - 1) / kTile;
  // the streamed tiles this CTA visits: [first, first + per_head) for each of `heads` streamed heads
  int first = 0, per_head = streamed_tiles, heads = 1;
  if (MODE == 0) {
    heads = shape.head_group;
    if (shape.causal) { first = min(tile_index, streamed_tiles); per_head = streamed_tiles - first; }
  } else if (shape.causal) {
    per_head = min(streamed_tiles, tile_index + 1);
  }
  const int steps = heads * per_head;
  const int x_head = head;                                                  // head of the stationary tiles
  auto y_head = [&](int step) { return MODE == 0 ? head * shape.head_group + step / per_head : head / shape.head_group; };
  auto y_row0 = [&](int step) { return (first + step % per_head) * kTile; };

  if (threadIdx.x == 0) {
    tc::mbar_init(&bars->x_full, 1);
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&bars->y_full[s], 1);
      tc::mbar_init(&bars->y_empty[s], 1);
    }
    tc::mbar_init(&bars->t0_full, 1);
    tc::mbar_init(&bars->t1_full, 1);
    tc::mbar_init(&bars->p_ready, 8);
    tc::mbar_init(&bars->g_ready, 8);
    tc::mbar_init(&bars->acc_full, 1);
    bars->abort_flag = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_descriptor(&map_x0);
    tc::tma_prefetch_descriptor(&map_x1);
    tc::tma_prefetch_descriptor(&map_y0);
    tc::tma_prefetch_descriptor(&map_y1);
  }
  if (warp == 1) tc::tmem_alloc(&bars->tmem_base, kTmemColumns);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_t0 = tmem_base, tmem_t1 = tmem_base + kTile, tmem_acc0 = tmem_base + 2 * kTile,
                 tmem_acc1 = tmem_base + 3 * kTile;
  volatile int *abort_flag = &bars->abort_flag;

  // one [128 rows x kHeadDim] tile: one TMA box per 64-column half
  auto load_tile = [&](unsigned char *destination, const CUtensorMap *map, uint64_t *bar, int row, int h) {
    tc::tma_load_4d(destination, map, bar, 0, row, h, batch);
    if (kHeadDim > 64) tc::tma_load_4d(destination + L::kHalfBytes, map, bar, 64, row, h, batch);
  };

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (tc::elect_one() && steps > 0) {
      tc::mbar_expect_tx(&bars->x_full, 2 * L::kTileBytes);
      load_tile(x_tiles, &map_x0, &bars->x_full, row0, x_head);
      load_tile(x_tiles + L::kTileBytes, &map_x1, &bars->x_full, row0, x_head);
      int issued = 0;
      bool alive = true;
      for (int step = 0; step < steps; ++step) {
        const int stage = step % kStages;
        const uint32_t phase = (step / kStages) & 1;
        if (!tc::mbar_wait(&bars->y_empty[stage], phase ^ 1, abort_flag, status, tc::kSiteProducerEmpty)) {
          alive = false;
          break;
        }
        unsigned char *slot = ring + stage * 2 * L::kTileBytes;
        tc::mbar_expect_tx(&bars->y_full[stage], 2 * L::kTileBytes);
        load_tile(slot, &map_y0, &bars->y_full[stage], y_row0(step), y_head(step));
        load_tile(slot + L::kTileBytes, &map_y1, &bars->y_full[stage], y_row0(step), y_head(step));
        ++issued;
      }
      if (!alive) {
        // let copies in flight land before the shared memory goes away
        const long long start = clock64();
        while (!tc::mbar_try_wait(&bars->x_full, 0) && clock64() - start < tc::kWaitCycles / 8) {}
        for (int back = 1; back <= min(issued, kStages); ++back) {
          const int step = issued - back;
          while (!tc::mbar_try_wait(&bars->y_full[step % kStages], (step / kStages) & 1) &&
                 clock64() - start < tc::kWaitCycles / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- MMA issuer
    // The whole warp walks the loop (waits and descriptor arithmetic stay warp-uniform, descriptors are
    // built once and advanced by byte offsets / 16); one elected lane issues a whole product per branch.
    if (steps > 0) {
      const bool issuer = tc::elect_one();
      constexpr int format = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_t = tc::instr_desc_f16(format, kTile, kTile, false);
      constexpr uint32_t idesc_acc = tc::instr_desc_f16(format, kTile, kHeadDim, true);
      const uint64_t desc_x = tc::smem_desc_k_major_sw128(tc::smem_u32(x_tiles));
      const uint64_t desc_y = tc::smem_desc_k_major_sw128(tc::smem_u32(ring));
      const uint64_t desc_y_mn = tc::smem_desc_mn_major_sw128(tc::smem_u32(ring), L::kHalfBytes);
      bool alive = tc::mbar_wait(&bars->x_full, 0, abort_flag, status, tc::kSiteMmaFull);
      tc::tc_fence_after_sync();
      // T0 = X0 . Y0^T or T1 = X1 . Y1^T of one step
      auto issue_scores = [&](int which, int step) {
        const uint64_t desc_ys = desc_y + (((step % kStages) * 2 * L::kTileBytes) >> 4);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk) {
            const uint32_t offset = (which * L::kTileBytes + (kk / 4) * L::kHalfBytes + (kk % 4) * 32) >> 4;
            tc::mma_f16_ss(which ? tmem_t1 : tmem_t0, desc_x + offset, desc_ys + offset, idesc_t, kk != 0);
          }
          tc::mma_commit(which ? &bars->t1_full : &bars->t0_full);
        }
      };
      // acc += (P or G, 16 bits, in TMEM) . (Y1 or Y0 of the step, as an MN-major B operand)
      auto issue_gradient = [&](uint32_t accumulator, uint32_t operand, int which_y, int step) {
        const uint64_t desc_ys = desc_y_mn + ((((step % kStages) * 2 + which_y) * L::kTileBytes) >> 4);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            // key block kk (16 streamed rows, 8 packed columns) was written by column half kk/4 into its own
            // columns; B: the same 16 rows of Y, 2048 bytes apart
            tc::mma_f16_ts(accumulator, operand + (kk / 4) * 64 + (kk % 4) * 8, desc_ys + ((kk * 2048) >> 4), idesc_acc,
                           (step | kk) != 0);
          }
        }
      };
      auto wait_stage = [&](int step) {
        const bool ok = tc::mbar_wait(&bars->y_full[step % kStages], (step / kStages) & 1, abort_flag, status, tc::kSiteMmaFull);
        tc::tc_fence_after_sync();
        return ok;
      };
      // The score products of step i+1 are issued as soon as their TMEM tile is free again, so they
      // (and the gradient products of step i) run while the compute warps are busy:
      //   P(i) ready -> dV += P.dO (MODE 0) -> T0 is free: S(i+1)
      //   G(i) ready -> acc1 += G.Y0        -> T1 is free: dP(i+1)
      if (alive && wait_stage(0)) {
        issue_scores(0, 0);
        issue_scores(1, 0);
        for (int step = 0; step < steps; ++step) {
          const bool more = step + 1 < steps;
          if (!tc::mbar_wait(&bars->p_ready, step & 1, abort_flag, status, tc::kSiteMmaTmemEmpty)) break;
          tc::tc_fence_after_sync();
          if (MODE == 0) issue_gradient(tmem_acc0, tmem_t0, 1, step);
          // S(i+1) needs the next streamed tiles, acc1 += G.Y0 needs G(i): whichever is ready first is
          // issued first.  With a two-stage ring the next tiles are requested only once this step's
          // gradient product has released its stage, so issuing that product without waiting for the
          // tiles of step i+1 gives their copy a head start.
          bool scores_issued = !more, gradient_issued = false;
          const long long waiting_since = clock64();
          uint32_t spins = 0;
          while (!(scores_issued && gradient_issued)) {
            if (!scores_issued &&
                tc::mbar_try_wait(&bars->y_full[(step + 1) % kStages], ((step + 1) / kStages) & 1)) {
              tc::tc_fence_after_sync();
              issue_scores(0, step + 1);
              scores_issued = true;
            } else if (!gradient_issued && tc::mbar_try_wait(&bars->g_ready, step & 1)) {
              tc::tc_fence_after_sync();
              issue_gradient(tmem_acc1, tmem_t1, 0, step);
              if (issuer) tc::mma_commit(&bars->y_empty[step % kStages]);  // both gradient products of the step have read its tiles
              gradient_issued = true;
            } else if ((++spins & 0x3ffu) == 0) {
              if (*abort_flag) break;
              if (clock64() - waiting_since > tc::kWaitCycles) {
                *abort_flag = 1;
                if (atomicCAS(status, 0, 1) == 0) status[1] = tc::kSiteMmaTmemEmpty;
                __threadfence();
                break;
              }
            }
          }
          if (!(scores_issued && gradient_issued)) break;
          if (more) issue_scores(1, step + 1);
          else if (issuer) tc::mma_commit(&bars->acc_full);
        }
      }
    }
  } else {
    // -------------------------------------------------------------- compute
    const int quadrant = warp & 3;                       // TMEM lanes [32*quadrant, +32) are this warp's
    const int half = (warp - 2) >> 2;                    // columns [64*half, +64) of the step are this thread's
    const int compute_warp = warp - 2;
    const int row_in_tile = quadrant * 32 + lane;
    const int row = row0 + row_in_tile;                  // key (MODE 0) or query (MODE 1) index of this lane
    const uint32_t lane_base = static_cast<uint32_t>(quadrant * 32) << 16;
    const int stationary_extent = MODE == 0 ? shape.seq_k : shape.seq_q;
    float row_lse = 0.0f, row_delta = 0.0f;
    if (MODE == 1 && row < shape.seq_q) {
      const int64_t at = batch * shape.lse_stride[0] + head * shape.lse_stride[1] + row * shape.lse_stride[2];
      const int64_t dat = batch * shape.delta_stride[0] + head * shape.delta_stride[1] + row * shape.delta_stride[2];
      row_lse = lse[at] * kLog2e;
      row_delta = delta[dat];
    }
    bool alive = true;
    // MODE 0: the per-query lse and delta of a step are requested one step ahead (their global loads
    // would otherwise sit in front of every step; nothing touches the loaded values until the next
    // step parks them, scaled, in this warp's shared-memory copy)
    float next_lse[kTile / 64], next_delta[kTile / 64];
    // (head, first row) of the streamed tiles, stepped without divisions: `ahead` is one step in front
    int now_head = MODE == 0 ? head * shape.head_group : head / shape.head_group, now_tile = first;
    int ahead_head = now_head, ahead_tile = first;
    auto advance = [&](int &h, int &t) {
      if (++t == first + per_head) { t = first; ++h; }
    };
    auto request_columns = [&](int step) {
#pragma unroll
      for (int part = 0; part < kTile / 64; ++part) {
        next_lse[part] = INFINITY;
        next_delta[part] = 0.0f;
        if (MODE == 0 && step < steps) {
          const int query = ahead_tile * kTile + half * 64 + part * 32 + lane, hq = ahead_head;
          if (query < shape.seq_q) {
            next_lse[part] = load_now(lse + batch * shape.lse_stride[0] + hq * shape.lse_stride[1] + query * shape.lse_stride[2]);
            next_delta[part] = load_now(delta + batch * shape.delta_stride[0] + hq * shape.delta_stride[1] + query * shape.delta_stride[2]);
          }
        }
      }
    };
    request_columns(0);
    advance(ahead_head, ahead_tile);
    for (int step = 0; alive && step < steps; ++step) {
      const int parity = step & 1;
      const int streamed0 = now_tile * kTile;
      advance(now_head, now_tile);
      if (MODE == 0) {
        // every warp keeps its own copy, so no barrier between warps is needed (the previous step's
        // reads ended at its __syncwarp)
#pragma unroll
        for (int part = 0; part < kTile / 64; ++part) {
          bars->columns[compute_warp][0][part * 32 + lane] = next_lse[part] * kLog2e;   // first use of the loaded value
          bars->columns[compute_warp][1][part * 32 + lane] = next_delta[part];
        }
        __syncwarp();
        request_columns(step + 1);
        advance(ahead_head, ahead_tile);
      }
      // column c of the tile is excluded when its key lies after its query
      //   MODE 0: key = row, query = streamed0 + c  -> excluded when c < row - streamed0
      //   MODE 1: key = streamed0 + c, query = row  -> excluded when c > row - streamed0
      const int diagonal = row - streamed0;
      const bool masked = shape.causal && (MODE == 0 ? streamed0 < row0 + kTile - 1 : streamed0 + kTile - 1 > row0);
      // phase A: P from T0, kept in registers for phase B; its 16-bit copy goes back over T0 (MODE 0)
      float probability[kTile / 2];
      if (!tc::mbar_wait(&bars->t0_full, parity, abort_flag, status, tc::kSiteSoftmax)) { alive = false; break; }
      tc::tc_fence_after_sync();
#pragma unroll
      for (int chunk = 0; chunk < kTile / 64; ++chunk) {
        uint32_t t0[32];
        tc::tmem_load_32x32(tmem_t0 + lane_base + half * 64 + chunk * 32, t0);
        tc::tmem_load_wait();
        uint32_t p16[16];
#pragma unroll
        for (int quad = 0; quad < 8; ++quad) {   // four columns at a time: lse comes as one 128-bit read
          float l[4] = {row_lse, row_lse, row_lse, row_lse};
          if (MODE == 0) {
            const float4 l4 = *reinterpret_cast<const float4 *>(&bars->columns[compute_warp][0][chunk * 32 + quad * 4]);
            l[0] = l4.x; l[1] = l4.y; l[2] = l4.z; l[3] = l4.w;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int mine = chunk * 32 + quad * 4 + e, column = half * 64 + mine;
            float p = ex2_approx_ftz(fmaf(__uint_as_float(t0[quad * 4 + e]), shape.score_scale, -l[e]));
            if (masked && (MODE == 0 ? column < diagonal : column > diagonal)) p = 0.0f;
            probability[mine] = p;
          }
          p16[quad * 2] = pack_pair<T>(probability[chunk * 32 + quad * 4], probability[chunk * 32 + quad * 4 + 1]);
          p16[quad * 2 + 1] = pack_pair<T>(probability[chunk * 32 + quad * 4 + 2], probability[chunk * 32 + quad * 4 + 3]);
        }
        // packed columns [64*half + 16*chunk, +16) lie over f32 columns this thread has already consumed
        if (MODE == 0) tc::tmem_store_32x16(tmem_t0 + lane_base + half * 64 + chunk * 16, p16);
      }
      if (MODE == 0) tc::tmem_store_wait();
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&bars->p_ready);      // T0 has been read (and, MODE 0, holds P)
      // phase B: G = P * (T1 - delta), 16 bits, back over T1
      if (!tc::mbar_wait(&bars->t1_full, parity, abort_flag, status, tc::kSiteSoftmax)) { alive = false; break; }
      tc::tc_fence_after_sync();
#pragma unroll
      for (int chunk = 0; chunk < kTile / 64; ++chunk) {
        uint32_t t1[32];
        tc::tmem_load_32x32(tmem_t1 + lane_base + half * 64 + chunk * 32, t1);
        tc::tmem_load_wait();
        uint32_t g16[16];
#pragma unroll
        for (int quad = 0; quad < 8; ++quad) {
          float d[4] = {row_delta, row_delta, row_delta, row_delta};
          if (MODE == 0) {
            const float4 d4 = *reinterpret_cast<const float4 *>(&bars->columns[compute_warp][1][chunk * 32 + quad * 4]);
            d[0] = d4.x; d[1] = d4.y; d[2] = d4.z; d[3] = d4.w;
          }
          float g[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            g[e] = probability[chunk * 32 + quad * 4 + e] * (__uint_as_float(t1[quad * 4 + e]) - d[e]);
          g16[quad * 2] = pack_pair<T>(g[0], g[1]);
          g16[quad * 2 + 1] = pack_pair<T>(g[2], g[3]);
        }
        tc::tmem_store_32x16(tmem_t1 + lane_base + half * 64 + chunk * 16, g16);
      }
      tc::tmem_store_wait();
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&bars->g_ready);
    }
    // ---- epilogue: out0 = acc1 * scale, out1 = acc0 (MODE 0)
    const bool have = steps > 0 && alive && tc::mbar_wait(&bars->acc_full, 0, abort_flag, status, tc::kSiteEpilogueTmemFull);
    if (steps == 0 || have) {
      if (have) tc::tc_fence_after_sync();
#pragma unroll 1
      for (int which = 0; which < (MODE == 0 ? 2 : 1); ++which) {
        T *out = which ? out1 : out0;
        const int64_t *stride = which ? shape.out1_stride : shape.out0_stride;
        const float factor = which ? 1.0f : shape.scale;
        constexpr int kMine = kHeadDim / 2;                 // output columns per thread
        T *destination = out + batch * stride[0] + head * stride[1] + (int64_t)row * stride[2] + half * kMine;
        const bool vector_ok = ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && stride[0] % 8 == 0 && stride[1] % 8 == 0 &&
                               stride[2] % 8 == 0;
#pragma unroll 1
        for (int chunk = 0; chunk < kMine / 32; ++chunk) {
          uint32_t raw[32];
          if (have) {
            tc::tmem_load_32x32((which ? tmem_acc0 : tmem_acc1) + lane_base + half * kMine + chunk * 32, raw);
            tc::tmem_load_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) raw[i] = 0u;
          }
          if (row < stationary_extent) {
            if (vector_ok) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 v;
                v.x = pack_pair<T>(__uint_as_float(raw[q * 8 + 0]) * factor, __uint_as_float(raw[q * 8 + 1]) * factor);
                v.y = pack_pair<T>(__uint_as_float(raw[q * 8 + 2]) * factor, __uint_as_float(raw[q * 8 + 3]) * factor);
                v.z = pack_pair<T>(__uint_as_float(raw[q * 8 + 4]) * factor, __uint_as_float(raw[q * 8 + 5]) * factor);
                v.w = pack_pair<T>(__uint_as_float(raw[q * 8 + 6]) * factor, __uint_as_float(raw[q * 8 + 7]) * factor);
                *reinterpret_cast<uint4 *>(destination + chunk * 32 + q * 8) = v;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                destination[chunk * 32 + i] = Element<T>::narrow(__uint_as_float(raw[i]) * factor);
            }
          }
        }
      }
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemColumns);
  }
}

// delta[b, h, q] = sum_d f32(O) * f32(dO).  LANES threads share a row, 8 elements (one 128-bit
// access) per thread and pass; LANES = 1 is the scalar form for rows that are not 16-byte aligned.
template <typename T, int LANES>
__global__ void __launch_bounds__(256)
attention_delta_kernel(const T *__restrict__ output, const T *__restrict__ grad_output, float *__restrict__ delta,
                       int64_t rows, int heads, int sequence, int head_dim, int64_t os0, int64_t os1, int64_t os2,
                       int64_t gs0, int64_t gs1, int64_t gs2, int64_t ds0, int64_t ds1, int64_t ds2) {
  const int64_t thread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t threads = (int64_t)gridDim.x * blockDim.x;
  const int lane = (int)(thread % LANES);
  // the loop bound is the same for the 32 threads of a warp, so the shuffles below see whole warps;
  // unrolled so that the loads of four rows are in flight together
#pragma unroll 4
  for (int64_t base = (thread - thread % 32) / LANES; base < rows; base += threads / LANES) {
    const int64_t row = base + (thread % 32) / LANES;
    float sum = 0.0f;
    int64_t b = 0, h = 0, q = 0;
    if (row < rows) {
      b = row / ((int64_t)heads * sequence); h = (row / sequence) % heads; q = row % sequence;
      const T *o = output + b * os0 + h * os1 + q * os2, *g = grad_output + b * gs0 + h * gs1 + q * gs2;
      if (LANES > 1) {
        for (int c = lane * 8; c < head_dim; c += LANES * 8) {
          float ov[8], gv[8];
          load_vector<T>(o + c, ov);
          load_vector<T>(g + c, gv);
#pragma unroll
          for (int i = 0; i < 8; ++i) sum += ov[i] * gv[i];
        }
      } else {
        for (int c = 0; c < head_dim; ++c) sum += Element<T>::widen(o[c]) * Element<T>::widen(g[c]);
      }
    }
#pragma unroll
    for (int offset = LANES / 2; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
    if (lane == 0 && row < rows) delta[b * ds0 + h * ds1 + q * ds2] = sum;
  }
}

// With no query at all the key/value gradients are zero.
template <typename T>
__global__ void zero_view_kernel(T *out, int64_t total, int64_t heads, int64_t sequence, int64_t head_dim, int64_t s0,
                                 int64_t s1, int64_t s2) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t d = i % head_dim, row = i / head_dim;
    const int64_t b = row / (heads * sequence), h = (row / sequence) % heads, q = row % sequence;
    out[b * s0 + h * s1 + q * s2 + d] = Element<T>::narrow(0.0f);
  }
}

int tensor_map_4d(CUtensorMap *map, const void *base, const int64_t *extents, const int64_t *strides) {
  // innermost first: (D, S, H, B); a size-1 dimension may carry any stride, give TMA a legal one
  const uint64_t dims[4] = {(uint64_t)extents[3], (uint64_t)extents[2], (uint64_t)extents[1], (uint64_t)extents[0]};
  auto legal = [&](int64_t stride, int64_t extent, int64_t fallback) {
    return (uint64_t)((extent > 1 ? stride : fallback) * 2);
  };
  const int64_t row = (extents[3] + 7) / 8 * 8;
  const uint64_t byte_strides[3] = {legal(strides[2], extents[2], row), legal(strides[1], extents[1], row * extents[2]),
                                    legal(strides[0], extents[0], row * extents[2] * extents[1])};
  const uint32_t box[4] = {64, 128, 1, 1};
  return encode_tensor_map_16bit(map, base, 4, dims, byte_strides, box, true);
}

struct View4 {
  const void *base;
  int64_t extents[4], strides[4];
};
struct View3 {
  const void *base;
  int64_t extents[3], strides[3];
};

template <typename T, int kHeadDim, int MODE>
int launch_backward(const View4 &q, const View4 &k, const View4 &v, const View4 &grad_output, const View3 &lse,
                    const View3 &delta, const View4 &out0, const View4 *out1, float scale, int head_group, int causal,
                    int *status, cudaStream_t stream) {
  using L = Layout<kHeadDim>;
  if (MODE == 0 && q.extents[2] == 0) {
    const int64_t total = k.extents[0] * k.extents[1] * k.extents[2] * kHeadDim;
    for (const View4 *out : {&out0, out1})
      zero_view_kernel<T><<<sm_count() * 4, 256, 0, stream>>>((T *)out->base, total, k.extents[1], k.extents[2], kHeadDim,
                                                              out->strides[0], out->strides[1], out->strides[2]);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  CUtensorMap map_q, map_k, map_v, map_g;
  int result = tensor_map_4d(&map_q, q.base, q.extents, q.strides);
  if (result == B200_OK) result = tensor_map_4d(&map_k, k.base, k.extents, k.strides);
  if (result == B200_OK) result = tensor_map_4d(&map_v, v.base, v.extents, v.strides);
  if (result == B200_OK) result = tensor_map_4d(&map_g, grad_output.base, grad_output.extents, grad_output.strides);
  if (result != B200_OK) return result;
  constexpr size_t smem = 1024 + (2 + 2 * L::kStages) * L::kTileBytes + sizeof(Barriers);
  auto kernel = attention_backward_kernel<T, kHeadDim, MODE>;
  B200_CUDA_TRY(opt_in_dynamic_smem(kernel, smem));
  Shape shape;
  shape.heads_q = (int)q.extents[1]; shape.heads_k = (int)k.extents[1];
  shape.seq_q = (int)q.extents[2]; shape.seq_k = (int)k.extents[2];
  shape.head_group = head_group; shape.causal = causal;
  shape.score_scale = scale * kLog2e;
  shape.scale = scale;
  for (int i = 0; i < 3; ++i) {
    shape.lse_stride[i] = lse.strides[i];
    shape.delta_stride[i] = delta.strides[i];
    shape.out0_stride[i] = out0.strides[i];
    shape.out1_stride[i] = out1 ? out1->strides[i] : 0;
  }
  const int64_t stationary = MODE == 0 ? k.extents[2] : q.extents[2];
  const int64_t heads = MODE == 0 ? k.extents[1] : q.extents[1];
  const dim3 grid((unsigned)((stationary + kTile - 1) / kTile), (unsigned)heads, (unsigned)q.extents[0]);
  if (MODE == 0)
    kernel<<<grid, kThreads, smem, stream>>>(map_k, map_v, map_q, map_g, (const float *)lse.base, (const float *)delta.base,
                                             (T *)out0.base, (T *)(out1 ? out1->base : nullptr), shape, status);
  else
    kernel<<<grid, kThreads, smem, stream>>>(map_q, map_g, map_k, map_v, (const float *)lse.base, (const float *)delta.base,
                                             (T *)out0.base, (T *)nullptr, shape, status);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

int check_half_view(const char *entry, const char *name, const View4 &view, bool tma) {
  for (int i = 0; i < 4; ++i)
    if (view.extents[i] < 0) return fail(B200_ERR_INVALID_ARGUMENT, "%s: %s has a negative extent", entry, name);
  const bool empty = view.extents[0] == 0 || view.extents[1] == 0 || view.extents[2] == 0 || view.extents[3] == 0;
  if (!view.base && !empty) return fail(B200_ERR_INVALID_ARGUMENT, "%s: %s is null", entry, name);
  if (view.extents[3] > 1 && view.strides[3] != 1)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "%s: %s must have unit innermost stride", entry, name);
  if (tma) {
    if (!aligned16(view.base)) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "%s: TMA needs a 16-byte aligned %s", entry, name);
    for (int axis = 0; axis < 3; ++axis)
      if (view.extents[axis] > 1 && (view.strides[axis] % 8 || view.strides[axis] <= 0))
        return fail(B200_ERR_UNSUPPORTED_LAYOUT, "%s: outer strides of %s must be positive multiples of 8 elements", entry, name);
  }
  return B200_OK;
}

// Shared argument checks and dispatch of the two gradient entries.
int backward_entry(const char *entry, int mode, const View4 &q, const View4 &k, const View4 &v, const View4 &grad_output,
                   const View3 &lse, const View3 &delta, const View4 &out0, const View4 *out1, float scale,
                   void *workspace, int64_t ws_d0, int64_t ws_s0, int32_t dtype, int32_t head_group, int32_t causal,
                   void *stream) {
  const View4 *halves[4] = {&q, &k, &v, &grad_output};
  const char *names[4] = {"q", "k", "v", "grad_output"};
  for (int i = 0; i < 4; ++i) {
    const int result = check_half_view(entry, names[i], *halves[i], true);
    if (result != B200_OK) return result;
  }
  int result = check_half_view(entry, "the first output", out0, false);
  if (result == B200_OK && out1) result = check_half_view(entry, "the second output", *out1, false);
  if (result != B200_OK) return result;
  const int64_t b = q.extents[0], hq = q.extents[1], sq = q.extents[2], d = q.extents[3];
  const int64_t hk = k.extents[1], sk = k.extents[2];
  bool consistent = head_group >= 1 && hq == hk * head_group && k.extents[0] == b && v.extents[0] == b &&
                    grad_output.extents[0] == b && v.extents[1] == hk && v.extents[2] == sk && k.extents[3] == d &&
                    v.extents[3] == d && grad_output.extents[1] == hq && grad_output.extents[2] == sq &&
                    grad_output.extents[3] == d;
  for (const View3 *rows : {&lse, &delta})
    consistent = consistent && rows->extents[0] == b && rows->extents[1] == hq && rows->extents[2] == sq;
  const View4 &like0 = mode == 0 ? k : q;
  for (int i = 0; i < 4; ++i) {
    consistent = consistent && out0.extents[i] == like0.extents[i];
    if (out1) consistent = consistent && out1->extents[i] == v.extents[i];
  }
  if (!consistent)
    return fail(B200_ERR_INVALID_ARGUMENT, "%s: q, grad_output (B,HQ,Q,D), k, v (B,HK,K,D), lse, delta (B,HQ,Q), HQ = HK * head_group", entry);
  if (dtype != B200_F16 && dtype != B200_BF16) return fail(B200_ERR_INVALID_ARGUMENT, "%s: element type %d is not f16/bf16", entry, dtype);
  if (d != 64 && d != 128) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "%s: head dimension must be 64 or 128 (got %lld)", entry, (long long)d);
  if (b * hq * sq == 0 && (mode == 1 || b * hk * sk == 0)) return B200_OK;      // nothing to write
  if (b * hq * sq != 0 && (!lse.base || !delta.base)) return fail(B200_ERR_INVALID_ARGUMENT, "%s: null lse or delta", entry);
  if (!workspace || ws_d0 < B200_WORKSPACE_WORDS || (ws_d0 > 1 && ws_s0 != 1))
    return fail(B200_ERR_INVALID_ARGUMENT, "%s: workspace must hold %d contiguous int32 words", entry, B200_WORKSPACE_WORDS);
  if (sq > INT32_MAX - 256 || sk > INT32_MAX - 256 || hq > 65535 || b > 65535)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "%s: extent exceeds the launch limits", entry);
  const int64_t outputs = mode == 0 ? b * hk * sk : b * hq * sq;
  if (outputs == 0 || d == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int *status = static_cast<int *>(workspace);
#define B200_BACKWARD(T, D, MODE) \
  launch_backward<T, D, MODE>(q, k, v, grad_output, lse, delta, out0, out1, scale, head_group, causal, status, s)
  if (mode == 0) {
    if (dtype == B200_F16) return d == 64 ? B200_BACKWARD(__half, 64, 0) : B200_BACKWARD(__half, 128, 0);
    return d == 64 ? B200_BACKWARD(__nv_bfloat16, 64, 0) : B200_BACKWARD(__nv_bfloat16, 128, 0);
  }
  if (dtype == B200_F16) return d == 64 ? B200_BACKWARD(__half, 64, 1) : B200_BACKWARD(__half, 128, 1);
  return d == 64 ? B200_BACKWARD(__nv_bfloat16, 64, 1) : B200_BACKWARD(__nv_bfloat16, 128, 1);
#undef B200_BACKWARD
}

}  // namespace
}  // namespace b200

using namespace b200;

#define B200_VIEW4(name) \
  const void *name, int64_t name##_d0, int64_t name##_d1, int64_t name##_d2, int64_t name##_d3, int64_t name##_s0, \
      int64_t name##_s1, int64_t name##_s2, int64_t name##_s3
#define B200_OUT4(name) \
  void *name, int64_t name##_d0, int64_t name##_d1, int64_t name##_d2, int64_t name##_d3, int64_t name##_s0, \
      int64_t name##_s1, int64_t name##_s2, int64_t name##_s3
#define B200_VIEW3(name) \
  const void *name, int64_t name##_d0, int64_t name##_d1, int64_t name##_d2, int64_t name##_s0, int64_t name##_s1, \
      int64_t name##_s2
#define B200_MAKE4(name) \
  View4 { name, {name##_d0, name##_d1, name##_d2, name##_d3}, {name##_s0, name##_s1, name##_s2, name##_s3} }
#define B200_MAKE3(name) \
  View3 { name, {name##_d0, name##_d1, name##_d2}, {name##_s0, name##_s1, name##_s2} }

extern "C" int b200_attention_backward_delta(B200_VIEW4(output), B200_VIEW4(grad_output), void *delta,
                                             int64_t delta_d0, int64_t delta_d1, int64_t delta_d2, int64_t delta_s0,
                                             int64_t delta_s1, int64_t delta_s2,
                                             int32_t dtype, void *stream) {
  const View4 o = B200_MAKE4(output), g = B200_MAKE4(grad_output);
  int result = check_half_view("attention_backward_delta", "output", o, false);
  if (result == B200_OK) result = check_half_view("attention_backward_delta", "grad_output", g, false);
  if (result != B200_OK) return result;
  for (int i = 0; i < 4; ++i)
    if (o.extents[i] != g.extents[i])
      return fail(B200_ERR_INVALID_ARGUMENT, "attention_backward_delta: output and grad_output must share one shape");
  if (delta_d0 != o.extents[0] || delta_d1 != o.extents[1] || delta_d2 != o.extents[2])
    return fail(B200_ERR_INVALID_ARGUMENT, "attention_backward_delta: delta must be (B, HQ, Q)");
  if (dtype != B200_F16 && dtype != B200_BF16)
    return fail(B200_ERR_INVALID_ARGUMENT, "attention_backward_delta: element type %d is not f16/bf16", dtype);
  const int64_t rows = o.extents[0] * o.extents[1] * o.extents[2];
  if (rows == 0) return B200_OK;
  if (!delta) return fail(B200_ERR_INVALID_ARGUMENT, "attention_backward_delta: null delta");
  if (o.extents[1] > INT32_MAX || o.extents[2] > INT32_MAX || o.extents[3] > INT32_MAX)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "attention_backward_delta: extent too large");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int d = (int)o.extents[3];
  const bool vectors = d % 8 == 0 && aligned16(output) && aligned16(grad_output) && output_s0 % 8 == 0 && output_s1 % 8 == 0 &&
                       output_s2 % 8 == 0 && grad_output_s0 % 8 == 0 && grad_output_s1 % 8 == 0 && grad_output_s2 % 8 == 0;
  const int lanes = !vectors ? 1 : d >= 128 ? 16 : d >= 64 ? 8 : d >= 32 ? 4 : d >= 16 ? 2 : 1;
  const int64_t wanted = (rows * lanes + 255) / 256, limit = (int64_t)sm_count() * 8;
  const unsigned grid = (unsigned)(wanted < limit ? wanted : limit);
#define B200_DELTA(T, LANES)                                                                                         \
  attention_delta_kernel<T, LANES><<<grid, 256, 0, s>>>((const T *)output, (const T *)grad_output, (float *)delta, rows, \
                                                        (int)o.extents[1], (int)o.extents[2], d, output_s0, output_s1,   \
                                                        output_s2, grad_output_s0, grad_output_s1, grad_output_s2,       \
                                                        delta_s0, delta_s1, delta_s2)
#define B200_DELTA_LANES(T)                              \
  switch (lanes) {                                       \
  case 16: B200_DELTA(T, 16); break;                     \
  case 8: B200_DELTA(T, 8); break;                       \
  case 4: B200_DELTA(T, 4); break;                       \
  case 2: B200_DELTA(T, 2); break;                       \
  default: B200_DELTA(T, 1); break;                      \
  }
  if (dtype == B200_F16) { B200_DELTA_LANES(__half) } else { B200_DELTA_LANES(__nv_bfloat16) }
#undef B200_DELTA_LANES
#undef B200_DELTA
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_attention_backward_dkdv(B200_VIEW4(q), B200_VIEW4(k), B200_VIEW4(v), B200_VIEW4(grad_output),
                                            B200_VIEW3(lse), B200_VIEW3(delta), B200_OUT4(grad_k), B200_OUT4(grad_v),
                                            float scale, void *workspace, int64_t ws_d0, int64_t ws_s0, int32_t dtype,
                                            int32_t head_group, int32_t causal, void *stream) {
  const View4 out1 = B200_MAKE4(grad_v);
  return backward_entry("attention_backward_dkdv", 0, B200_MAKE4(q), B200_MAKE4(k), B200_MAKE4(v), B200_MAKE4(grad_output),
                        B200_MAKE3(lse), B200_MAKE3(delta), B200_MAKE4(grad_k), &out1, scale, workspace, ws_d0, ws_s0,
                        dtype, head_group, causal, stream);
}

extern "C" int b200_attention_backward_dq(B200_VIEW4(q), B200_VIEW4(k), B200_VIEW4(v), B200_VIEW4(grad_output),
                                          B200_VIEW3(lse), B200_VIEW3(delta), B200_OUT4(grad_q), float scale,
                                          void *workspace, int64_t ws_d0, int64_t ws_s0, int32_t dtype, int32_t head_group,
                                          int32_t causal, void *stream) {
  return backward_entry("attention_backward_dq", 1, B200_MAKE4(q), B200_MAKE4(k), B200_MAKE4(v), B200_MAKE4(grad_output),
                        B200_MAKE3(lse), B200_MAKE3(delta), B200_MAKE4(grad_q), nullptr, scale, workspace, ws_d0, ws_s0,
                        dtype, head_group, causal, stream);
}
