// Fused GEMM-SwiGLU for B200 (sm_100a):  Y = silu(X·Wg^T) * (X·Wu^T),  W = [Wg ; Wu] packed along rows.
//
// One warp-specialised kernel serves both schedules the host picks between:
//   MMA    (large M): persistent CTAs walk 128 x block_n output tiles in a banded raster; the fp32
//          accumulators for gate and up (2*block_n tensor-memory columns) are double-buffered so the
//          epilogue of tile i overlaps the MMAs of tile i+1.
//   STREAM (M <= 128): N is cut into at most one slab per SM (block_n up to 256 columns, any multiple
//          of 16), so every SM streams a disjoint slice of the weight exactly once through a deep
//          TMA ring; the run time is the time to read W from HBM.
// Data path of both: TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) -> shared memory ->
// tcgen05.mma (bf16 x bf16 -> fp32 in tensor memory) -> tcgen05.ld -> silu(g)*u in fp32 -> one
// rounding to bf16 -> 16-byte global stores.  The 2N-wide intermediate never exists in HBM.
//
// MMA2 is the MMA schedule on CTA pairs (thread-block clusters of 2, tcgen05 cta_group::2): one 256-row MMA
// spans both CTAs, each CTA loads its own 128 rows of X and only HALF of the weight tile, so every SM
// pulls a third fewer bytes per FLOP through L2 and the ring is deeper.  The leader CTA (cluster rank 0)
// issues the MMAs and owns the "stage full" barriers; both CTAs run their own producer and epilogue.
//
// Warp roles (384 threads): warps 0 and 3 = TMA producers (one lane each: X tiles, W tiles), warp 1 = MMA
// issuer (one lane), warp 2 = tensor-memory allocator, warps 4..11 = epilogue (warp w reads TMEM lanes 32*(w%4)..+31;
// the two warps of a lane quarter take alternate 32-column chunks of the tile).
//
// Every wait on an mbarrier is bounded: after kWaitLimitCycles the waiting role records itself in
// g_watchdog, raises a CTA-wide abort flag and all roles fall through to the common teardown, which
// frees tensor memory.  No wait in this file can spin forever.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/magi_swiglu.h"
#include "ptx_sm100.cuh"

namespace magi {

constexpr int kBM = 128;             // rows of X per tile = tensor-memory lanes
constexpr int kBK = 64;              // K elements per pipeline stage = one 128-byte swizzle row
constexpr int kEpiWarps = 8;          // two warps per tensor-memory lane quarter share a tile's columns
constexpr int kThreads = 128 + 32 * kEpiWarps;
constexpr int kMaxStages = 12;
constexpr int kTmemCols = 512;       // whole tensor memory of the SM (one CTA per SM)
constexpr uint32_t kABytes = kBM * kBK * 2;
constexpr int kSmemLimit = 232448 - 1024;  // dynamic part of the 227 KB opt-in maximum (static barriers take the rest)
constexpr int kSmemFloor = 120 * 1024;  // keeps a second CTA off the SM (it would block in tcgen05.alloc)
constexpr long long kWaitLimitCycles = 6000000000LL;  // three to four seconds of SM cycles

__device__ unsigned int g_watchdog[4];  // {role that gave up, block, stage/buffer, parity}
// {SM cycles, nanoseconds} block 0 of the most recent tile kernel spent between set-up and teardown: the
// SM clock the kernel really ran at (power capping moves it within a millisecond; nvidia-smi cannot see that)
__device__ unsigned long long g_clock_probe[2];

#ifdef MAGI_SWIGLU_TRACE
// Tuning builds only: SM-cycle timestamps of block 0's second tile (MMA issuer and first epilogue warp).
__device__ long long g_trace[16];
#define MAGI_TRACE(slot, cond) do { if (blockIdx.x == 0 && (cond)) g_trace[slot] = clock64(); } while (0)
#define MAGI_TRACE_T0() const long long trace_t0 = clock64()
#define MAGI_TRACE_ADD(slot) do { if (blockIdx.x == 0) g_trace[slot] += clock64() - trace_t0; } while (0)
#else
#define MAGI_TRACE(slot, cond) do { } while (0)
#define MAGI_TRACE_T0() do { } while (0)
#define MAGI_TRACE_ADD(slot) do { } while (0)
#endif

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct KArgs {
  __nv_bfloat16* y;
  long long ldy;
  int M, N;
  int block_n;        // output columns per tile
  int num_m_tiles, num_n_tiles, num_k_blocks;  // num_m_tiles counts 128-row (256-row for CTA pairs) units
  int group_m;        // row-tiles per raster band
  int stages;
  uint32_t stage_bytes;
  int n_mma;          // 1: one MMA of N = 2*block_n covers gate|up;  2: one MMA each
  uint32_t b_second;  // byte offset of the second MMA's weight rows inside a stage's weight tile
  int split;          // CTA pairs, two MMAs: tensor memory holds [gate_lo|up_lo|gate_hi|up_hi]; the low half of
                      // the tile is handed back to the MMA issuer before the high half has been drained
  int acc_bufs;       // tensor-memory accumulator buffers (2 = epilogue overlaps next tile)
  int wide_store;     // y base and row pitch are 32-byte aligned: 256-bit stores (one full sector per thread)
  int x_hint, w_hint, y_hint;  // L2 eviction priority of X tiles, W tiles and Y stores: 0 normal, 1 first, 2 last
  // Split-K (STREAM schedule on narrow weights): k_splits CTAs share one tile, each sums kb_per_split K-steps and
  // parks its fp32 partial sums in `ws`; swiglu_splitk_reduce_kernel adds them in split order and writes Y.
  // k_splits == 1: no scratch is touched.
  int k_splits, kb_per_split;
  float* ws;  // [tile][split][M rows][2*block_n] fp32
};

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned role,
                                             unsigned idx) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort_flag = 1;
        if (atomicCAS(&g_watchdog[0], 0u, role) == 0u) {
          g_watchdog[1] = blockIdx.x;
          g_watchdog[2] = idx;
          g_watchdog[3] = parity;
        }
        return false;
      }
    }
  }
}

// Banded raster: tiles are numbered band by band (group_m row-tiles per band); inside a band the
// row-tile index runs fastest, so the CTAs of one wave share a few X row-panels and W column-panels in L2.
__device__ __forceinline__ void tile_coords(const KArgs& a, int t, int& mt, int& nt) {
  const int per_band = a.group_m * a.num_n_tiles;
  const int band = t / per_band;
  const int first_m = band * a.group_m;
  const int rows = min(a.group_m, a.num_m_tiles - first_m);
  const int r = t - band * per_band;
  mt = first_m + r % rows;
  nt = r / rows;
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  // silu(g) = g / (1 + exp(-g)); ex2.approx + div.approx are far below bf16 resolution
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

__device__ __forceinline__ uint64_t l2_policy(int hint) {
  return hint == 1 ? l2_policy_evict_first() : (hint == 2 ? l2_policy_evict_last() : l2_policy_evict_normal());
}

__device__ __forceinline__ uint4 swiglu_pack8(const uint32_t* g, const uint32_t* u) {
  uint4 v;
  __nv_bfloat162 p;
  p = __floats2bfloat162_rn(silu_mul(__uint_as_float(g[0]), __uint_as_float(u[0])),
                            silu_mul(__uint_as_float(g[1]), __uint_as_float(u[1])));
  v.x = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(silu_mul(__uint_as_float(g[2]), __uint_as_float(u[2])),
                            silu_mul(__uint_as_float(g[3]), __uint_as_float(u[3])));
  v.y = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(silu_mul(__uint_as_float(g[4]), __uint_as_float(u[4])),
                            silu_mul(__uint_as_float(g[5]), __uint_as_float(u[5])));
  v.z = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(silu_mul(__uint_as_float(g[6]), __uint_as_float(u[6])),
                            silu_mul(__uint_as_float(g[7]), __uint_as_float(u[7])));
  v.w = *reinterpret_cast<uint32_t*>(&p);
  return v;
}

// n (8, 16, 24 or 32 ...) consecutive outputs of one row starting at dst; `wide` = dst is 32-byte aligned
template <int kCols>
__device__ __forceinline__ void store_cols(__nv_bfloat16* dst, const uint32_t* g, const uint32_t* u, int cols_valid,
                                           bool wide, uint64_t policy) {
#pragma unroll
  for (int j = 0; j < kCols / 16; ++j) {
    if (16 * j + 16 <= cols_valid) {
      const uint4 lo = swiglu_pack8(g + 16 * j, u + 16 * j);
      const uint4 hi = swiglu_pack8(g + 16 * j + 8, u + 16 * j + 8);
      if (wide) {
        st_global_v8_hint(dst + 16 * j, lo, hi, policy);
      } else {
        st_global_v4_hint(dst + 16 * j, lo, policy);
        st_global_v4_hint(dst + 16 * j + 8, hi, policy);
      }
    } else if (16 * j + 8 <= cols_valid) {
      st_global_v4_hint(dst + 16 * j, swiglu_pack8(g + 16 * j, u + 16 * j), policy);
    }
  }
}

template <int kCtas>
__global__ void __launch_bounds__(kThreads, 1)
swiglu_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const KArgs a) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kMaxStages + 4];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCtas == 2) ? cluster_ctarank() : 0u;  // rank 0 of a pair leads
  const int unit = blockIdx.x / kCtas;                              // index of this CTA (pair) in the grid
  const int units = gridDim.x / kCtas;
  // 128-byte-swizzled tiles must start on 1024-byte boundaries (same offset in both CTAs of a pair)
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bar0 + 8u * (2 * kMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bar0 + 8u * (2 * kMaxStages + 2 + b); };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), kEpiWarps * kCtas);  // lane 0 of each epilogue warp (of both CTAs of a pair)
    }
    fence_barrier_init();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
  }
  if (warp == 2) {
    tmem_alloc<kCtas>(smem_u32(&tmem_slot), kTmemCols);
    tmem_relinquish<kCtas>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kCtas == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  // A kernel launched behind this one with programmatic stream serialisation (the split-K reduce) may be scheduled
  // now; it still waits for this grid to complete before it reads anything (griddepcontrol.wait on its side).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  long long probe_c0 = 0;
  unsigned long long probe_t0 = 0;
  if (blockIdx.x == 0 && threadIdx.x == 64) {  // lane 0 of the allocator warp, idle between set-up and teardown
    probe_c0 = clock64();
    probe_t0 = global_timer_ns();
  }

  const int num_items = a.num_m_tiles * a.num_n_tiles * a.k_splits;  // (tile, K split) work items
  const int acc_cols = 2 * a.block_n;

  if (warp == 0 || warp == 3) {
    // ------------------------------------------------------------ TMA producers (every CTA loads its own tiles)
    // Two issuing threads, because one thread cannot issue tensor copies fast enough for the narrow tiles:
    // warp 0 arms the "stage full" barrier and brings the X tile, warp 3 brings the W tile.
    if (lane == 0) {
      const bool x_role = (warp == 0);
      const uint64_t policy = l2_policy(x_role ? a.x_hint : a.w_hint);
      // CTA pairs: the bytes of both CTAs are counted on the leader's barrier
      const uint32_t full_remote0 = (kCtas == 2) ? map_to_cta(full_bar(0), 0) : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = unit; item < num_items && ok; item += units) {
        const int t = item / a.k_splits;
        const int kb0 = (item - t * a.k_splits) * a.kb_per_split;
        const int kb1 = min(a.num_k_blocks, kb0 + a.kb_per_split);
        int mt, nt;
        tile_coords(a, t, mt, nt);
        const int row0 = (mt * kCtas + (int)cta_rank) * kBM;
        for (int kb = kb0; kb < kb1; ++kb) {
          {
            MAGI_TRACE_T0();
            if (!wait_bounded(empty_bar(stage), phase ^ 1u, &abort_flag, x_role ? 1u : 4u, stage)) {
              ok = false;
              break;
            }
            MAGI_TRACE_ADD(x_role ? 12 : 13);  // producers: cycles spent waiting for a free stage
          }
          if (x_role && (kCtas == 1 || cta_rank == 0)) mbar_arrive_expect_tx(full_bar(stage), kCtas * a.stage_bytes);
          const uint32_t bar = (kCtas == 2) ? full_remote0 + 8u * stage : full_bar(stage);
          const uint32_t st_a = tiles_base + stage * a.stage_bytes;  // X tile of this stage
          const uint32_t st_b = st_a + kABytes;                     // W rows of this stage
          const int k0 = kb * kBK;  // past the end of K the copy is zero-filled
          if constexpr (kCtas == 1) {
            if (x_role)
              tma_load_2d_hint(st_a, &tm_x, bar, k0, row0, policy);
            else
              tma_load_3d_hint(st_b, &tm_w, bar, k0, nt * a.block_n, 0, policy);
          } else {
            if (x_role)
              tma_load_2d_pair_hint(st_a, &tm_x, bar, k0, row0, policy);
            else if (a.n_mma == 1 || a.split)  // rank 0 brings the tile's gate rows, rank 1 its up rows
              tma_load_3d_pair_hint(st_b, &tm_w, bar, k0, nt * a.block_n, (int)cta_rank, policy);
            else  // half of the gate rows and the matching half of the up rows
              tma_load_3d_pair_hint(st_b, &tm_w, bar, k0, nt * a.block_n + (int)cta_rank * (a.block_n / 2), 0, policy);
          }
          if (++stage == a.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta_rank == 0) {
      const uint32_t mma_n = (a.n_mma == 1) ? 2u * a.block_n : (uint32_t)a.block_n;
      const uint32_t idesc = umma_idesc_bf16(kBM * kCtas, mma_n);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int item = unit; item < num_items && ok; item += units, ++it) {
        const int kb0 = (item % a.k_splits) * a.kb_per_split;  // split-K is never combined with CTA pairs
        const int kb1 = min(a.num_k_blocks, kb0 + a.kb_per_split);
        const int buf = (a.acc_bufs == 2) ? (it & 1) : 0;
        const uint32_t acc_phase = (a.acc_bufs == 2) ? ((it >> 1) & 1) : (it & 1);
        MAGI_TRACE(0, it == 2);  // issuer starts waiting for the accumulator of tile 2
        {
          MAGI_TRACE_T0();
          if (!wait_bounded(acc_empty_bar(buf), acc_phase ^ 1u, &abort_flag, 2u, 16 + buf)) break;
          MAGI_TRACE_ADD(15);  // issuer: cycles spent waiting for a free accumulator
        }
        MAGI_TRACE(1, it == 2);  // accumulator free
        tc_fence_after_sync();
        const uint32_t d_gate = tmem_base + (uint32_t)(buf * acc_cols);
        int kb = kb0;
        if (kCtas == 2 && a.split) {
          // The low half [gate_lo|up_lo] is free while the epilogue still drains the high half: run the
          // first MMA of as many K-steps as the ring holds, then wait for the high half and catch up.
          const int ahead = min(a.stages, a.num_k_blocks);
          int s2 = stage;
          uint32_t p2 = phase;
          for (int j = 0; j < ahead && ok; ++j) {
            if (!wait_bounded(full_bar(s2), p2, &abort_flag, 2u, s2)) {
              ok = false;
              break;
            }
            MAGI_TRACE(2, it == 2 && j == 0);
            tc_fence_after_sync();
            const uint32_t sa = tiles_base + s2 * a.stage_bytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_bf16<kCtas>(d_gate, umma_desc_k_sw128(sa + k * 32), umma_desc_k_sw128(sa + kABytes + k * 32), idesc,
                               (uint32_t)((j | k) != 0));
            if (++s2 == a.stages) {
              s2 = 0;
              p2 ^= 1u;
            }
          }
          if (!ok) break;
          if (!wait_bounded(acc_empty_bar(1), acc_phase ^ 1u, &abort_flag, 2u, 17)) break;
          tc_fence_after_sync();
          for (int j = 0; j < ahead; ++j) {
            const uint32_t sa = tiles_base + stage * a.stage_bytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_bf16<kCtas>(d_gate + a.block_n, umma_desc_k_sw128(sa + k * 32),
                               umma_desc_k_sw128(sa + kABytes + a.b_second + k * 32), idesc, (uint32_t)((j | k) != 0));
            umma_commit<kCtas>(empty_bar(stage));
            if (++stage == a.stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          kb = ahead;
        }
        for (; kb < kb1; ++kb) {
          {
            MAGI_TRACE_T0();
            if (!wait_bounded(full_bar(stage), phase, &abort_flag, 2u, stage)) {
              ok = false;
              break;
            }
            MAGI_TRACE_ADD(14);  // issuer: cycles spent waiting for operands
          }
          MAGI_TRACE(2, it == 2 && kb == 0);                   // first stage of tile 2 available
          MAGI_TRACE(3, it == 1 && kb == kb1 - 1);  // last stage of tile 1 available
          tc_fence_after_sync();
          {
            MAGI_TRACE_T0();
            const uint32_t sa = tiles_base + stage * a.stage_bytes;
            const uint32_t sb = sa + kABytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
              const uint32_t acc = ((kb - kb0) | k) != 0;
              const uint64_t ad = umma_desc_k_sw128(sa + k * 32);
              umma_bf16<kCtas>(d_gate, ad, umma_desc_k_sw128(sb + k * 32), idesc, acc);
              if (a.n_mma == 2)
                umma_bf16<kCtas>(d_gate + a.block_n, ad, umma_desc_k_sw128(sb + a.b_second + k * 32), idesc, acc);
            }
            MAGI_TRACE_ADD(10);  // issuer: cycles spent issuing MMAs
          }
          {
            MAGI_TRACE_T0();
            umma_commit<kCtas>(empty_bar(stage));  // frees the stage (in both CTAs) once these MMAs have read it
            MAGI_TRACE_ADD(11);  // issuer: cycles spent in the commit
          }
          if (++stage == a.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit<kCtas>(acc_full_bar(buf));
        MAGI_TRACE(4, it == 1);  // all MMAs of tile 1 issued
        MAGI_TRACE(9, it == 2);  // all MMAs of tile 2 issued
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (every CTA drains its own 128 rows)
    const int q = warp & 3;
    const uint64_t y_policy = l2_policy(a.y_hint);
    const uint32_t acc_empty_remote0 = (kCtas == 2) ? map_to_cta(acc_empty_bar(0), 0) : 0u;
    int it = 0;
    for (int item = unit; item < num_items; item += units, ++it) {
      const int t = item / a.k_splits;
      const int zsplit = item - t * a.k_splits;
      const int buf = (a.acc_bufs == 2) ? (it & 1) : 0;
      const uint32_t acc_phase = (a.acc_bufs == 2) ? ((it >> 1) & 1) : (it & 1);
      int mt, nt;
      tile_coords(a, t, mt, nt);
      bool ok = wait_bounded(acc_full_bar(buf), acc_phase, &abort_flag, 3u, buf);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      MAGI_TRACE(5, it == 1 && warp == 4 && lane == 0);  // epilogue sees tile 1 complete
      tc_fence_after_sync();

      const int row = (mt * kCtas + (int)cta_rank) * kBM + q * 32 + lane;
      const bool row_ok = row < a.M;
      const int col0 = nt * a.block_n;
      const int valid_tile = min(a.block_n, a.N - col0);  // multiple of 8
      const uint32_t t_tile = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * acc_cols);
      __nv_bfloat16* yrow_tile = a.y + (long long)row * a.ldy + col0;
      const bool wide = a.wide_store != 0;  // every 16-column group of every row starts on a 32-byte boundary

      if (kCtas == 1 && a.k_splits > 1) {
        // ---- split-K: park this CTA's fp32 partial sums; swiglu_splitk_reduce_kernel finishes the tile
        const int slot = warp - 4;
        const int ws_ld = 2 * a.block_n;
        const int r_loc = q * 32 + lane;
        float* part = a.ws + ((size_t)(t * a.k_splits + zsplit) * a.M + r_loc) * ws_ld;
        auto chunk_w = [&](int c) { return (c + 32 <= a.block_n) ? 32 : ((c + 16 == a.block_n) ? 16 : 0); };
        uint32_t g[32], u[32];
        bool released = false;
        for (int c = 32 * (slot >> 2), w = chunk_w(c); w; c += 64, w = chunk_w(c)) {
          if (w == 32) {
            tmem_ld_x32(t_tile + c, g);
            tmem_ld_x32(t_tile + a.block_n + c, u);
          } else {
            tmem_ld_x16_into32(t_tile + c, g);
            tmem_ld_x16_into32(t_tile + a.block_n + c, u);
          }
          tmem_ld_wait();
          if (!chunk_w(c + 64)) {  // last read of the accumulator: hand it back before the stores
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(buf));
            released = true;
          }
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (4 * j < w) {
                *reinterpret_cast<uint4*>(part + c + 4 * j) = make_uint4(g[4 * j], g[4 * j + 1], g[4 * j + 2], g[4 * j + 3]);
                *reinterpret_cast<uint4*>(part + a.block_n + c + 4 * j) =
                    make_uint4(u[4 * j], u[4 * j + 1], u[4 * j + 2], u[4 * j + 3]);
              }
            }
          }
        }
        if (!released) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(buf));
        }
        continue;
      }

      // A tile is drained in one segment (gate columns [0,bn), up columns [bn,2bn)) or, in split mode, in two
      // (low half then high half, each [gate|up] of bn/2 columns) that are released separately.
      const int num_seg = (kCtas == 2 && a.split) ? 2 : 1;
      const int seg_cols = a.block_n / num_seg;
      for (int seg = 0; seg < num_seg; ++seg) {
        const uint32_t t_gate = t_tile + (uint32_t)(seg * a.block_n);
        const uint32_t t_up = t_gate + (uint32_t)seg_cols;
        const int valid = max(0, min(seg_cols, valid_tile - seg * seg_cols));
        __nv_bfloat16* yrow = yrow_tile + seg * seg_cols;
        const int release_buf = (num_seg == 2) ? seg : buf;

        // 32-column chunks alternate between the two warps of this lane quarter; a 16-column remainder goes to
        // whichever warp is next in turn.  The accumulator segment is handed back to the MMA issuer as soon as
        // this warp's LAST load from it has landed, so that chunk's arithmetic and stores overlap the next MMAs.
        auto width_at = [&](int c) {
          return (c < valid && c + 32 <= seg_cols) ? 32 : ((c < valid && c + 16 == seg_cols) ? 16 : 0);
        };
        auto load = [&](uint32_t (&g)[32], uint32_t (&u)[32], int c, int w) {
          if (w == 32) {
            tmem_ld_x32(t_gate + c, g);
            tmem_ld_x32(t_up + c, u);
          } else {
            tmem_ld_x16_into32(t_gate + c, g);
            tmem_ld_x16_into32(t_up + c, u);
          }
        };
        auto process = [&](const uint32_t (&g)[32], const uint32_t (&u)[32], int c, int w) {
          if (!row_ok) return;
          if (w == 32)
            store_cols<32>(yrow + c, g, u, valid - c, wide, y_policy);
          else
            store_cols<16>(yrow + c, g, u, valid - c, wide, y_policy);
        };
        auto release = [&]() {
          MAGI_TRACE(6 + seg * 4, it == 1 && warp == 4 && lane == 0);  // warp 4 has read its last column
          MAGI_TRACE(7 + seg * 4, it == 1 && warp == 11 && lane == 0);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kCtas == 1)
              mbar_arrive(acc_empty_bar(release_buf));
            else  // the leader's MMA issuer waits for both CTAs
              mbar_arrive_cluster(acc_empty_remote0 + 8u * release_buf);
          }
        };
        uint32_t g[32], u[32];
        int c = 32 * ((warp - 4) >> 2);
        int w = width_at(c);
        bool released = false;
        while (w) {
          load(g, u, c, w);
          tmem_ld_wait();
          const int c2 = c + 64, w2 = width_at(c2);
          if (!w2) {  // that was this warp's last read of the segment
            release();
            released = true;
          }
          process(g, u, c, w);
          c = c2;
          w = w2;
        }
        if (!released) release();
      }
    }
  }

  // ------------------------------------------------------------ teardown (also the abort path)
  __syncwarp();
  if (*reinterpret_cast<volatile int*>(&abort_flag)) {
    // give copies and MMAs that may still be in flight time to land before tensor memory is freed
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 64) {
    g_clock_probe[0] = (unsigned long long)(clock64() - probe_c0);
    g_clock_probe[1] = global_timer_ns() - probe_t0;
  }
  // a pair leaves together: the leader's MMAs read the peer's shared memory and both barriers sets are shared
  if constexpr (kCtas == 2) cluster_sync_all();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}

// Second step of a split-K launch: Y[row, tile columns] = silu(sum_z g_z) * (sum_z u_z), partial sums added in
// split order (bit-identical from run to run).  One thread per 8 output columns, coalesced along a row.
__global__ void __launch_bounds__(256)
swiglu_splitk_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ y, int M, int N, long long ldy,
                            int block_n, int num_n_tiles, int k_splits) {
  const int groups = block_n / 8;
  const long long total = (long long)num_n_tiles * M * groups;
  const uint64_t policy = l2_policy_evict_first();
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the partial sums of the tile kernel are complete and visible
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int cg = (int)(i % groups);
    const int row = (int)((i / groups) % M);
    const int t = (int)(i / ((long long)groups * M));
    const int col = t * block_n + cg * 8;
    if (col >= N) continue;  // N is a multiple of 8: a group is inside or outside as a whole
    const float* p = ws + (((size_t)t * k_splits) * M + row) * (2 * block_n) + cg * 8;
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0}, u[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int z = 0; z < k_splits; ++z, p += (size_t)M * 2 * block_n) {
      const float4 g0 = __ldcg(reinterpret_cast<const float4*>(p)), g1 = __ldcg(reinterpret_cast<const float4*>(p + 4));
      const float4 u0 = __ldcg(reinterpret_cast<const float4*>(p + block_n));
      const float4 u1 = __ldcg(reinterpret_cast<const float4*>(p + block_n + 4));
      g[0] += g0.x; g[1] += g0.y; g[2] += g0.z; g[3] += g0.w; g[4] += g1.x; g[5] += g1.y; g[6] += g1.z; g[7] += g1.w;
      u[0] += u0.x; u[1] += u0.y; u[2] += u0.z; u[3] += u0.w; u[4] += u1.x; u[5] += u1.y; u[6] += u1.z; u[7] += u1.w;
    }
    uint32_t gb[8], ub[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gb[j] = __float_as_uint(g[j]);
      ub[j] = __float_as_uint(u[j]);
    }
    st_global_v4_hint(y + (long long)row * ldy + col, swiglu_pack8(gb, ub), policy);
  }
}

// Backward of the activation: from the recomputed pre-activations H = [G | U] (bf16, [M, 2N]) and dY ([M, N]):
//   dG = dY * U * s * (1 + G * (1 - s)),   dU = dY * G * s,   s = sigmoid(G)
// written as dH = [dG | dU] (bf16).  Element-wise, HBM-bound (10 bytes per output element); 8 columns per thread
// with 16-byte accesses, fp32 arithmetic, one rounding per result.
__global__ void __launch_bounds__(256)
swiglu_bwd_act_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ dy,
                      __nv_bfloat16* __restrict__ dh, int M, int N, long long ldh, long long lddy, long long lddh) {
  const int groups = N / 8;
  const long long total = (long long)M * groups;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / groups;
    const int col = (int)(i - row * groups) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(h + row * ldh + col);
    const uint4 uv = *reinterpret_cast<const uint4*>(h + row * ldh + N + col);
    const uint4 dv = *reinterpret_cast<const uint4*>(dy + row * lddy + col);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
    uint4 og, ou;
    __nv_bfloat162* og2 = reinterpret_cast<__nv_bfloat162*>(&og);
    __nv_bfloat162* ou2 = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]), d = __bfloat1622float2(d2[j]);
      const float sx = __fdividef(1.0f, 1.0f + __expf(-g.x)), sy = __fdividef(1.0f, 1.0f + __expf(-g.y));
      og2[j] = __floats2bfloat162_rn(d.x * u.x * sx * (1.0f + g.x * (1.0f - sx)),
                                     d.y * u.y * sy * (1.0f + g.y * (1.0f - sy)));
      ou2[j] = __floats2bfloat162_rn(d.x * g.x * sx, d.y * g.y * sy);
    }
    *reinterpret_cast<uint4*>(dh + row * lddh + col) = og;
    *reinterpret_cast<uint4*>(dh + row * lddh + N + col) = ou;
  }
}

// Plain CUDA-core kernel: one thread per output, 16x16 outputs per block, K staged through shared
// memory in slices of 32.  Same arithmetic contract (fp32 accumulate, one rounding).  Validation only.
__global__ void __launch_bounds__(256)
swiglu_simt_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, int M, int N, int K, long long ldx, long long ldw, long long ldy) {
  __shared__ float xs[16][33], gs[16][33], us[16][33];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row0 = blockIdx.y * 16, col0 = blockIdx.x * 16;
  float accg = 0.f, accu = 0.f;
  for (int k0 = 0; k0 < K; k0 += 32) {
    for (int i = threadIdx.x; i < 16 * 32; i += 256) {
      const int r = i >> 5, k = i & 31;
      const bool kin = (k0 + k) < K;
      xs[r][k] = (kin && row0 + r < M) ? __bfloat162float(x[(long long)(row0 + r) * ldx + k0 + k]) : 0.f;
      gs[r][k] = (kin && col0 + r < N) ? __bfloat162float(w[(long long)(col0 + r) * ldw + k0 + k]) : 0.f;
      us[r][k] = (kin && col0 + r < N) ? __bfloat162float(w[(long long)(N + col0 + r) * ldw + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      accg = fmaf(xs[ty][k], gs[tx][k], accg);
      accu = fmaf(xs[ty][k], us[tx][k], accu);
    }
    __syncthreads();
  }
  const int row = row0 + ty, col = col0 + tx;
  if (row < M && col < N) y[(long long)row * ldy + col] = __float2bfloat16_rn(accg / (1.0f + expf(-accg)) * accu);
}

// ================================================================== host side
thread_local char g_err[512] = "";

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
static int fail_cuda(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return e == cudaSuccess ? 1 : (int)e;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) return (EncodeTiledFn) nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  int queried = 0;  // 1 = ok, -1 = unusable
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  int smem_optin_set = 0;
  int pair_clusters = 0;  // co-resident 2-CTA clusters of the pair kernel (0 = not queried yet, -1 = none)
};
static DeviceInfo g_dev[kMaxDevices];
static std::mutex g_dev_mutex;

static const DeviceInfo* device_info(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceInfo& d = g_dev[device];
  if (d.queried == 0) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device >= n) {
      cudaGetLastError();
      d.queried = -1;
    } else {
      cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device);
      cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, device);
      cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, device);
      d.queried = 1;
    }
  }
  return d.queried == 1 ? &d : nullptr;
}

struct Plan {
  int variant, block_n, stages, grid, tiles, smem_bytes, acc_bufs, n_mma;
  int num_m_tiles, num_n_tiles, num_k_blocks, group_m;
  int ctas;  // CTAs per tile: 1, or 2 for the CTA-pair schedule
  int split; // CTA pairs with two MMAs per step and block_n % 32 == 0: two separately released half tiles
  int k_splits, kb_per_split;          // split-K of the STREAM schedule (1 = off)
  int64_t ws_bytes;                    // fp32 partial sums of a split-K plan (0 = none)
  uint32_t stage_bytes, b_second;
};

static inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

constexpr int64_t kWorkspaceCap = 64LL << 20;  // never plan for more scratch than this

// Scratch bytes of a split-K plan: per tile k_splits x M x 2*block_n fp32 partial sums.
static inline int64_t splitk_bytes(int64_t tiles, int64_t z, int64_t M, int64_t bn) { return tiles * z * M * 2 * bn * 4; }

// Estimated time (ns) of the STREAM schedule: every CTA runs kb_per_split K-steps; a K-step costs at least
// ~530 ns of MMA issue (measured) and otherwise its share of HBM bandwidth; split-K adds a reduction.
static inline double stream_cost_ns(int64_t N, int64_t num_kb, int bn, int z, int ctas) {
  const int64_t slabs = (N + bn - 1) / bn;
  const int64_t items = slabs * z;
  const int64_t waves = (items + ctas - 1) / ctas;
  const int64_t active = items < ctas ? items : ctas;
  const int64_t kpz = (num_kb + z - 1) / z;
  const double step_ns = 256.0 * bn * (double)active / 6200.0;  // 2*bn rows x 128 B per K-step over ~6.2 TB/s
  return (double)waves * ((double)kpz * (step_ns > 533.0 ? step_ns : 533.0) + 1500.0 + 6.0 * bn + (z > 1 ? 2500.0 : 0.0));
}

static int make_plan(int64_t M, int64_t N, int64_t K, int variant, int block_n, int stages, int group_m, int max_ctas,
                     int sm_count, int64_t ws_limit, Plan* p) {
  if (M < 0 || N <= 0 || K <= 0 || M > 0x7fffff00LL || N > 0x3fffff00LL || K > 0x7fffff00LL)
    return fail(MAGI_SWIGLU_ERR_SHAPE, "shape out of range: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (N % 8 != 0 || K % 8 != 0)
    return fail(MAGI_SWIGLU_ERR_SHAPE, "N (%lld) and K (%lld) must be multiples of 8", (long long)N, (long long)K);
  if (variant == MAGI_SWIGLU_VARIANT_AUTO) variant = (M <= 128) ? MAGI_SWIGLU_VARIANT_STREAM : MAGI_SWIGLU_VARIANT_MMA2;
  if (variant != MAGI_SWIGLU_VARIANT_MMA && variant != MAGI_SWIGLU_VARIANT_STREAM &&
      variant != MAGI_SWIGLU_VARIANT_SIMT && variant != MAGI_SWIGLU_VARIANT_MMA2)
    return fail(MAGI_SWIGLU_ERR_VARIANT, "unknown variant %d", variant);
  if (sm_count <= 0) return fail(MAGI_SWIGLU_ERR_DEVICE, "sm_count must be positive");
  memset(p, 0, sizeof(*p));
  p->variant = variant;
  if (variant == MAGI_SWIGLU_VARIANT_SIMT) {
    p->block_n = 16;
    p->tiles = (int)(((M + 15) / 16) * ((N + 15) / 16));
    p->grid = p->tiles;
    return 0;
  }
  if (variant == MAGI_SWIGLU_VARIANT_STREAM && M > kBM)
    return fail(MAGI_SWIGLU_ERR_VARIANT, "STREAM variant needs M <= %d (got %lld)", kBM, (long long)M);
  const int pair = (variant == MAGI_SWIGLU_VARIANT_MMA2) ? 2 : 1;
  int stream_auto_width = 0;
  p->ctas = pair;
  int ctas = (max_ctas > 0 && max_ctas < sm_count) ? max_ctas : sm_count;
  if (pair == 2) ctas = ctas / 2 * 2;
  if (ctas < pair) return fail(MAGI_SWIGLU_ERR_VARIANT, "max_ctas=%d leaves no room for a CTA pair", max_ctas);
  if (block_n == 0) {
    if (variant == MAGI_SWIGLU_VARIANT_MMA2) {
      // Wide tiles move the fewest operand bytes per FLOP (256 columns fill tensor memory: gate + up = 512
      // fp32 columns), but the persistent grid runs whole waves of tiles.  Measured on B200, one tile of
      // width bn costs about (bn + 146) units of time (fixed part: epilogue, pipeline refill and the
      // narrower tiles' lower operand reuse), so pick the width with the cheapest total of waves x tile cost.
      if (N < 128) {
        block_n = round_up((int)N, 16);
      } else {
        const int64_t units = ctas / 2;
        const int64_t m_units = (M + 2 * kBM - 1) / (2 * kBM);
        int64_t best_cost = -1;
        for (int bn = 256; bn >= 128; bn -= 32) {  // multiples of 32: both half tiles stay multiples of 16
          const int64_t tiles = m_units * ((N + bn - 1) / bn);
          const int64_t cost = ((tiles + units - 1) / units) * (bn + 146);
          if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            block_n = bn;
          }
        }
      }
    } else if (variant == MAGI_SWIGLU_VARIANT_MMA) {
      block_n = (N >= 128) ? 128 : round_up((int)N, 16);
    } else {
      // one slab per SM if it fits in tensor memory (gate + up <= 512 fp32 columns)
      int64_t per = (N + ctas - 1) / ctas;
      block_n = round_up((int)(per < 16 ? 16 : per), 16);
      if (block_n > 256) block_n = 256;
      stream_auto_width = 1;
    }
  }
  int k_splits = 1;
  if (variant == MAGI_SWIGLU_VARIANT_STREAM && M > 0) {
    // Narrow weights (a column shard of a decode GEMM) leave each SM too little W per K-step to hide the MMA
    // issue time; with scratch available, several CTAs share a slab and split K between them.
    const int64_t num_kb = (K + kBK - 1) / kBK;
    if (ws_limit > kWorkspaceCap) ws_limit = kWorkspaceCap;
    int forced = 0;
    if (const char* env = getenv("MAGI_SWIGLU_K_SPLITS")) forced = atoi(env);  // tuning aid
    double best = stream_cost_ns(N, num_kb, block_n, 1, ctas);
    const int bn_lo = stream_auto_width ? 32 : block_n, bn_hi = stream_auto_width ? 256 : block_n;
    for (int bn = bn_lo; bn <= bn_hi; bn += 16) {
      for (int z = 1; z <= 8; ++z) {
        if (forced > 0 && z != forced) continue;
        if (z > 1 && ((num_kb + z - 1) / z < 4 || (int64_t)((num_kb + z - 1) / z) * (z - 1) >= num_kb)) continue;
        const int64_t slabs = (N + bn - 1) / bn;
        if (z > 1 && splitk_bytes(slabs, z, M, bn) > ws_limit) continue;
        const double c = stream_cost_ns(N, num_kb, bn, z, ctas);
        if (c < best * 0.97 || (forced > 0 && z == forced && k_splits != forced)) {  // 3 %: prefer the simpler plan
          best = c;
          block_n = bn;
          k_splits = z;
        }
      }
    }
  }
  if (block_n < 16 || block_n > 256 || block_n % 16 != 0)
    return fail(MAGI_SWIGLU_ERR_VARIANT, "block_n=%d must be a multiple of 16 in [16,256]", block_n);
  p->block_n = block_n;
  p->n_mma = (2 * block_n <= 256) ? 1 : 2;
  p->acc_bufs = (4 * block_n <= kTmemCols) ? 2 : 1;
  // weight rows per CTA and stage: gate + up rows of the tile, split between the CTAs of a pair
  p->stage_bytes = kABytes + 2u * (uint32_t)block_n * 128u / (uint32_t)pair;
  p->b_second = (uint32_t)block_n * 128u / (uint32_t)pair;
  p->split = (pair == 2 && p->n_mma == 2 && block_n % 32 == 0 && !getenv("MAGI_SWIGLU_NO_SPLIT")) ? 1 : 0;
  const int fit = (kSmemLimit - 1024) / (int)p->stage_bytes;
  int max_stages = fit < kMaxStages ? fit : kMaxStages;
  if (stages == 0) stages = max_stages;
  if (stages < 2 || stages > max_stages)
    return fail(MAGI_SWIGLU_ERR_VARIANT, "stages=%d out of range [2,%d] for block_n=%d", stages, max_stages, block_n);
  p->stages = stages;
  int smem = stages * (int)p->stage_bytes + 1024;
  p->smem_bytes = smem < kSmemFloor ? kSmemFloor : smem;
  p->num_m_tiles = (int)((M + kBM * pair - 1) / (kBM * pair));
  p->num_n_tiles = (int)((N + block_n - 1) / block_n);
  p->num_k_blocks = (int)((K + kBK - 1) / kBK);
  if ((int64_t)p->num_m_tiles * p->num_n_tiles > 0x7fffffffLL) return fail(MAGI_SWIGLU_ERR_SHAPE, "too many tiles");
  p->tiles = p->num_m_tiles * p->num_n_tiles;
  if (group_m <= 0) {
    // band height: keep one band of X rows (group_m units x K) around 32 MB so it stays in L2 while W streams by
    const int64_t unit_bytes = (int64_t)kBM * pair * K * 2;
    int64_t g = (32LL << 20) / (unit_bytes > 0 ? unit_bytes : 1);
    group_m = (int)(g < 4 ? 4 : (g > 64 ? 64 : g));
  }
  p->group_m = group_m;
  p->k_splits = k_splits;
  p->kb_per_split = (p->num_k_blocks + k_splits - 1) / k_splits;
  if (k_splits > 1) p->ws_bytes = splitk_bytes(p->tiles, k_splits, M, block_n);
  const int64_t items = (int64_t)p->tiles * pair * k_splits;
  p->grid = (items < ctas) ? (int)items : ctas;
  return 0;
}

static int encode_maps(const void* x, const void* w, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw,
                       const Plan& p, CUtensorMap* tm_x, CUtensorMap* tm_w) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return fail(MAGI_SWIGLU_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MAGI_SWIGLU_ERR_DRIVER, "tensor map for X rejected by the driver (CUresult %d)", (int)r);
  }
  {
    // W viewed as [2][N][K].  One CTA per tile: one box brings block_n gate rows and the matching block_n up
    // rows.  CTA pair: each CTA brings half of the MMA's weight rows — all gate rows or all up rows when one
    // MMA covers gate|up or the tile is split in halves, else half of each.
    cuuint32_t box_rows = (cuuint32_t)p.block_n, box_halves = 2;
    if (p.ctas == 2) {
      if (p.n_mma == 1 || p.split) box_halves = 1;  // rank 0 loads gate rows, rank 1 up rows
      else box_rows = (cuuint32_t)p.block_n / 2;
    }
    const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)N, 2};
    const cuuint64_t strides[2] = {(cuuint64_t)ldw * 2, (cuuint64_t)N * (cuuint64_t)ldw * 2};
    const cuuint32_t box[3] = {(cuuint32_t)kBK, box_rows, box_halves};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MAGI_SWIGLU_ERR_DRIVER, "tensor map for W rejected by the driver (CUresult %d)", (int)r);
  }
  return 0;
}

struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  cudaError_t set(int device) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    if (prev != device) {
      e = cudaSetDevice(device);
      changed = (e == cudaSuccess);
    }
    return e;
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
};

static int forward_impl(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx,
                        int64_t ldw, int64_t ldy, int device, void* stream_v, int variant, int block_n, int stages,
                        int group_m, int max_ctas, void* workspace, int64_t workspace_bytes) {
  g_err[0] = 0;
  if (M == 0 && N > 0 && K > 0) return 0;
  if (!x || !w || !y) return fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  if (ldx < K || ldw < K || ldy < N)
    return fail(MAGI_SWIGLU_ERR_SHAPE, "row strides too small: ldx=%lld ldw=%lld (K=%lld) ldy=%lld (N=%lld)",
                (long long)ldx, (long long)ldw, (long long)K, (long long)ldy, (long long)N);
  if (ldx % 8 || ldw % 8 || ldy % 8) return fail(MAGI_SWIGLU_ERR_ALIGN, "row strides must be multiples of 8 elements");
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15u)
    return fail(MAGI_SWIGLU_ERR_ALIGN, "x, w_gate_up and y must be 16-byte aligned");
  const DeviceInfo* di = device_info(device);
  if (!di) return fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  if (di->cc_major != 10 || di->cc_minor != 0)
    return fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is sm_%d%d; this library runs on sm_100 (B200) only", device,
                di->cc_major, di->cc_minor);
  Plan p;
  if (workspace && (((uintptr_t)workspace & 255u) || workspace_bytes < 0))
    return fail(MAGI_SWIGLU_ERR_ALIGN, "workspace must be 256-byte aligned");
  int rc = make_plan(M, N, K, variant, block_n, stages, group_m, max_ctas, di->sm_count,
                     workspace ? workspace_bytes : 0, &p);
  if (rc) return rc;

  DeviceGuard guard;
  cudaError_t e = guard.set(device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  if (p.variant == MAGI_SWIGLU_VARIANT_SIMT) {
    dim3 grid((unsigned)((N + 15) / 16), (unsigned)((M + 15) / 16));
    if (grid.y > 65535u) return fail(MAGI_SWIGLU_ERR_VARIANT, "SIMT validation kernel supports M <= 1048560");
    swiglu_simt_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                 static_cast<const __nv_bfloat16*>(w),
                                                 static_cast<__nv_bfloat16*>(y), (int)M, (int)N, (int)K, ldx, ldw, ldy);
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : fail_cuda(e, "launch of swiglu_simt_kernel");
  }

  CUtensorMap tm_x, tm_w;
  rc = encode_maps(x, w, M, N, K, ldx, ldw, p, &tm_x, &tm_w);
  if (rc) return rc;

  int pair_clusters = 0;
  {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[device];
    if (!d.smem_optin_set) {
      e = cudaFuncSetAttribute(swiglu_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(swiglu_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
      if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
      d.smem_optin_set = 1;
    }
    if (p.ctas == 2 && d.pair_clusters == 0) {
      // how many CTA pairs the GPU can hold at once (GPCs with an odd SM count leave one SM out)
      cudaLaunchConfig_t qc = {};
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      qc.gridDim = dim3((unsigned)(d.sm_count / 2 * 2));
      qc.blockDim = dim3(kThreads);
      qc.dynamicSmemBytes = kSmemLimit;
      qc.attrs = qa;
      qc.numAttrs = 1;
      int n = 0;
      e = cudaOccupancyMaxActiveClusters(&n, swiglu_tc_kernel<2>, &qc);
      if (e != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      d.pair_clusters = n > 0 ? n : -1;
    }
    pair_clusters = d.pair_clusters;
  }

  KArgs a;
  a.y = static_cast<__nv_bfloat16*>(y);
  a.ldy = ldy;
  a.M = (int)M;
  a.N = (int)N;
  a.block_n = p.block_n;
  a.num_m_tiles = p.num_m_tiles;
  a.num_n_tiles = p.num_n_tiles;
  a.num_k_blocks = p.num_k_blocks;
  a.group_m = p.group_m;
  a.stages = p.stages;
  a.stage_bytes = p.stage_bytes;
  a.n_mma = p.n_mma;
  a.b_second = p.b_second;
  a.split = p.split;
  a.acc_bufs = p.acc_bufs;
  a.wide_store = (((uintptr_t)y & 31u) == 0 && ldy % 16 == 0) ? 1 : 0;
  a.k_splits = p.k_splits;
  a.kb_per_split = p.kb_per_split;
  a.ws = p.k_splits > 1 ? static_cast<float*>(workspace) : nullptr;
  // Default L2 priorities (ncu, DRAM bytes per launch).  X: a band of X rows is re-read by every column tile ->
  // keep.  Y: written once -> evict first.  W: in the tile schedules a W tile is shared by all row units of the band
  // that run at the same time, and marking it evict-first makes late CTAs miss it (+25..70 % DRAM reads) -> normal;
  // in the STREAM schedule every W byte is read exactly once -> evict first.
  a.x_hint = 2;
  a.w_hint = (p.variant == MAGI_SWIGLU_VARIANT_STREAM) ? 1 : 0;
  a.y_hint = 1;
  if (const char* env = getenv("MAGI_SWIGLU_L2_HINTS")) {  // three digits "xwy", each 0/1/2 (tuning aid)
    if (strlen(env) == 3) {
      a.x_hint = env[0] - '0';
      a.w_hint = env[1] - '0';
      a.y_hint = env[2] - '0';
    }
  }

  if (p.ctas == 1) {
    swiglu_tc_kernel<1><<<p.grid, kThreads, p.smem_bytes, stream>>>(tm_x, tm_w, a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, "launch of swiglu_tc_kernel<1>");
    if (p.k_splits > 1) {
      const long long work = (long long)p.num_n_tiles * M * (p.block_n / 8);
      const int blocks = (int)((work + 255) / 256 < 4LL * di->sm_count ? (work + 255) / 256 : 4LL * di->sm_count);
      // scheduled while the tile kernel drains (programmatic dependent launch); it waits for that grid itself
      cudaLaunchConfig_t rc_cfg = {};
      cudaLaunchAttribute rc_attr[1];
      rc_attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      rc_attr[0].val.programmaticStreamSerializationAllowed = 1;
      rc_cfg.gridDim = dim3((unsigned)blocks);
      rc_cfg.blockDim = dim3(256);
      rc_cfg.stream = stream;
      rc_cfg.attrs = rc_attr;
      rc_cfg.numAttrs = 1;
      e = cudaLaunchKernelEx(&rc_cfg, swiglu_splitk_reduce_kernel, (const float*)a.ws, a.y, a.M, a.N, a.ldy, p.block_n,
                             p.num_n_tiles, p.k_splits);
      if (e != cudaSuccess) return fail_cuda(e, "launch of swiglu_splitk_reduce_kernel");
    }
    return 0;
  }
  if (pair_clusters <= 0) return fail(MAGI_SWIGLU_ERR_VARIANT, "this device cannot co-schedule 2-CTA clusters of the pair kernel");
  int grid = p.grid;
  if (grid > 2 * pair_clusters) grid = 2 * pair_clusters;  // persistent: never more pairs than fit at once
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (size_t)p.smem_bytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, swiglu_tc_kernel<2>, tm_x, tm_w, a);
  return e == cudaSuccess ? 0 : fail_cuda(e, "launch of swiglu_tc_kernel<2>");
}

// ------------------------------------------------------------------ built-in scratch (no allocation anywhere)
// Scratch for magi_swiglu_forward_bf16_static.  It is part of the loaded module: every GPU that loads the
// library carries these bytes until the process exits.  In host code the name below is only a handle for the
// symbol, not a device pointer; the device address is looked up once per device with cudaGetSymbolAddress.
constexpr int64_t kStaticScratchBytes = 8LL << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static void* g_static_scratch_addr[kMaxDevices];  // device address of g_static_scratch, per device (nullptr = not set up)

// Looks the scratch array's device address up on first use for `device` (which must be the current device).
static int static_scratch_address(int device, void** out) {
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_static_scratch_addr[device]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(g_static_scratch)");
    if (!ptr) return fail(MAGI_SWIGLU_ERR_DRIVER, "cudaGetSymbolAddress returned a null address for the built-in scratch");
    g_static_scratch_addr[device] = ptr;
  }
  *out = g_static_scratch_addr[device];
  return 0;
}

}  // namespace magi

// ================================================================== C ABI
extern "C" {

int magi_swiglu_version(void) { return MAGI_SWIGLU_ABI_VERSION; }

int magi_swiglu_supported(int device) {
  const magi::DeviceInfo* di = magi::device_info(device);
  return (di && di->cc_major == 10 && di->cc_minor == 0) ? 1 : 0;
}

int magi_swiglu_forward_bf16(const void* x, const void* w_gate_up, void* y, int64_t M, int64_t N, int64_t K,
                             int64_t ldx, int64_t ldw, int64_t ldy, int device, void* cuda_stream, int variant) {
  return magi::forward_impl(x, w_gate_up, y, M, N, K, ldx, ldw, ldy, device, cuda_stream, variant, 0, 0, 0, 0,
                            nullptr, 0);
}

int magi_swiglu_forward_bf16_ex(const void* x, const void* w_gate_up, void* y, int64_t M, int64_t N, int64_t K,
                                int64_t ldx, int64_t ldw, int64_t ldy, int device, void* cuda_stream, int variant,
                                int block_n, int stages, int group_m, int max_ctas) {
  return magi::forward_impl(x, w_gate_up, y, M, N, K, ldx, ldw, ldy, device, cuda_stream, variant, block_n, stages,
                            group_m, max_ctas, nullptr, 0);
}

int magi_swiglu_forward_bf16_ws(const void* x, const void* w_gate_up, void* y, int64_t M, int64_t N, int64_t K,
                                int64_t ldx, int64_t ldw, int64_t ldy, int device, void* cuda_stream, int variant,
                                int block_n, int stages, int group_m, int max_ctas, void* workspace,
                                int64_t workspace_bytes) {
  return magi::forward_impl(x, w_gate_up, y, M, N, K, ldx, ldw, ldy, device, cuda_stream, variant, block_n, stages,
                            group_m, max_ctas, workspace, workspace_bytes);
}

int magi_swiglu_forward_bf16_static(const void* x, const void* w_gate_up, void* y, int64_t M, int64_t N, int64_t K,
                                    int64_t ldx, int64_t ldw, int64_t ldy, int device, void* cuda_stream) {
  magi::g_err[0] = 0;
  if (M == 0 && N > 0 && K > 0) return 0;
  const magi::DeviceInfo* di = magi::device_info(device);
  if (!di) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  // the schedule the scratch-taking entry point prefers for this problem, and the scratch it wants
  magi::Plan p;
  int rc = magi::make_plan(M, N, K, MAGI_SWIGLU_VARIANT_AUTO, 0, 0, 0, 0, di->sm_count, magi::kWorkspaceCap, &p);
  if (rc) return rc;
  if (p.ws_bytes > magi::kStaticScratchBytes)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE,
                      "M=%lld N=%lld K=%lld needs %lld bytes of scratch; the built-in scratch of "
                      "magi_swiglu_forward_bf16_static holds %lld (use magi_swiglu_forward_bf16_ws with your own)",
                      (long long)M, (long long)N, (long long)K, (long long)p.ws_bytes,
                      (long long)magi::kStaticScratchBytes);
  void* scratch = nullptr;
  {
    magi::DeviceGuard guard;  // the symbol's address is per device: look it up with `device` current
    cudaError_t e = guard.set(device);
    if (e != cudaSuccess) return magi::fail_cuda(e, "cudaSetDevice");
    rc = magi::static_scratch_address(device, &scratch);
    if (rc) return rc;
  }
  return magi::forward_impl(x, w_gate_up, y, M, N, K, ldx, ldw, ldy, device, cuda_stream, MAGI_SWIGLU_VARIANT_AUTO, 0, 0,
                            0, 0, scratch, magi::kStaticScratchBytes);
}

int magi_swiglu_backward_act_bf16(const void* h, const void* dy, void* dh, int64_t M, int64_t N, int64_t ldh,
                                  int64_t lddy, int64_t lddh, int device, void* cuda_stream) {
  magi::g_err[0] = 0;
  if (M == 0 && N > 0) return 0;
  if (!h || !dy || !dh) return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  if (M < 0 || N <= 0 || N % 8 != 0 || M > 0x7fffff00LL || N > 0x3fffff00LL)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "bad shape M=%lld N=%lld (N must be a positive multiple of 8)", (long long)M,
                      (long long)N);
  if (ldh < 2 * N || lddh < 2 * N || lddy < N) return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "row strides too small");
  if (ldh % 8 || lddh % 8 || lddy % 8 || (((uintptr_t)h | (uintptr_t)dy | (uintptr_t)dh) & 15u))
    return magi::fail(MAGI_SWIGLU_ERR_ALIGN, "pointers must be 16-byte aligned and row strides multiples of 8 elements");
  const magi::DeviceInfo* di = magi::device_info(device);
  if (!di) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  if (di->cc_major != 10 || di->cc_minor != 0)
    return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not sm_100 (B200)", device);
  magi::DeviceGuard guard;
  cudaError_t e = guard.set(device);
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaSetDevice");
  const long long work = M * (N / 8);
  const long long want = (work + 255) / 256;
  const int blocks = (int)(want < 16LL * di->sm_count ? want : 16LL * di->sm_count);
  magi::swiglu_bwd_act_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dh),
      (int)M, (int)N, ldh, lddy, lddh);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : magi::fail_cuda(e, "launch of swiglu_bwd_act_kernel");
}

int64_t magi_swiglu_workspace_bytes(int64_t M, int64_t N, int64_t K, int variant, int block_n, int stages, int group_m,
                                    int max_ctas, int device, int sm_count) {
  magi::g_err[0] = 0;
  if (sm_count <= 0) {
    const magi::DeviceInfo* di = magi::device_info(device);
    if (!di) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
    sm_count = di->sm_count;
  }
  if (M == 0) return 0;
  magi::Plan p;
  int rc = magi::make_plan(M, N, K, variant, block_n, stages, group_m, max_ctas, sm_count, magi::kWorkspaceCap, &p);
  return rc ? (int64_t)rc : p.ws_bytes;
}

int magi_swiglu_plan(int64_t M, int64_t N, int64_t K, int variant, int block_n, int stages, int group_m, int max_ctas,
                     int device, int sm_count, int32_t out[12]) {
  magi::g_err[0] = 0;
  if (!out) return magi::fail(MAGI_SWIGLU_ERR_NULL, "out is null");
  if (sm_count <= 0) {
    const magi::DeviceInfo* di = magi::device_info(device);
    if (!di) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
    sm_count = di->sm_count;
  }
  magi::Plan p;
  int rc = magi::make_plan(M, N, K, variant, block_n, stages, group_m, max_ctas, sm_count, magi::kWorkspaceCap, &p);
  if (rc) return rc;
  out[0] = p.variant;
  out[1] = p.block_n;
  out[2] = p.stages;
  out[3] = p.grid;
  out[4] = p.tiles;
  out[5] = p.smem_bytes;
  out[6] = p.acc_bufs;
  out[7] = p.n_mma;
  out[8] = p.ctas;
  out[9] = p.group_m;
  out[10] = p.split;
  out[11] = p.k_splits;
  return 0;
}

int magi_swiglu_device_status(int device, int32_t out[4]) {
  magi::g_err[0] = 0;
  if (!out) return magi::fail(MAGI_SWIGLU_ERR_NULL, "out is null");
  if (!magi::device_info(device)) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  magi::DeviceGuard guard;
  cudaError_t e = guard.set(device);
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaSetDevice");
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaDeviceSynchronize");
  unsigned int host[4] = {0, 0, 0, 0};
  e = cudaMemcpyFromSymbol(host, magi::g_watchdog, sizeof(host));
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaMemcpyFromSymbol(g_watchdog)");
  for (int i = 0; i < 4; ++i) out[i] = (int32_t)host[i];
  if (host[0] != 0) {
    const unsigned int zero[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(magi::g_watchdog, zero, sizeof(zero));
    if (e != cudaSuccess) return magi::fail_cuda(e, "cudaMemcpyToSymbol(g_watchdog)");
  }
  return 0;
}

#ifdef MAGI_SWIGLU_TRACE
int magi_swiglu_trace(long long out[16]) {  // reads the trace and clears its accumulating slots
  cudaDeviceSynchronize();
  int rc = (int)cudaMemcpyFromSymbol(out, magi::g_trace, sizeof(long long) * 16);
  long long zero[16] = {0};
  cudaMemcpyToSymbol(magi::g_trace, zero, sizeof(zero));
  return rc;
}
#endif

int magi_swiglu_kernel_clock(int device, double out[2]) {
  magi::g_err[0] = 0;
  if (!out) return magi::fail(MAGI_SWIGLU_ERR_NULL, "out is null");
  if (!magi::device_info(device)) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  magi::DeviceGuard guard;
  cudaError_t e = guard.set(device);
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaSetDevice");
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaDeviceSynchronize");
  unsigned long long host[2] = {0, 0};
  e = cudaMemcpyFromSymbol(host, magi::g_clock_probe, sizeof(host));
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaMemcpyFromSymbol(g_clock_probe)");
  out[0] = host[1] ? (double)host[0] * 1e3 / (double)host[1] : 0.0;  // cycles per ns -> MHz
  out[1] = (double)host[1] * 1e-3;
  return 0;
}

const char* magi_swiglu_last_error(void) { return magi::g_err; }

}  // extern "C"
