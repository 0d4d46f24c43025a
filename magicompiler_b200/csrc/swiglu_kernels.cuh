// Device code of the fused GEMM-SwiGLU for B200 (sm_100a):  Y = silu(X·Wg^T) * (X·Wu^T),  W = [Wg ; Wu] by rows.
//
// swiglu_tc_kernel<kCtas> is one warp-specialised kernel that the host runs under three schedules:
//   MMA2   (M > 128, kCtas = 2): CTA pairs (clusters of 2, tcgen05 cta_group::2).  One 256-row MMA spans both
//          CTAs; each CTA loads its own 128 rows of X and HALF of the tile's weight rows.  With 256 output columns
//          a K-step issues two independent N = 256 MMAs (gate and up fill all 512 tensor-memory columns), which is
//          what keeps the tensor pipe busy; the tile is drained in two halves that are released separately so the
//          next tile's first MMAs overlap the rest of the epilogue.  Persistent grid, banded raster.
//   MMA    (kCtas = 1): 128-row tiles, one CTA each; double-buffered accumulators when they fit.
//   STREAM (M <= 128, kCtas = 1): N is cut into about one slab per SM, each SM streams its slab of W exactly once
//          through a deep TMA ring; for narrow weights several CTAs share a slab and split K, park fp32 partial
//          sums in scratch memory, and swiglu_splitk_reduce_kernel finishes the tile.
// Data path: TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) -> shared-memory ring -> tcgen05.mma
// (bf16 x bf16 -> fp32 in tensor memory) -> tcgen05.ld -> silu(g)*u in fp32 -> one rounding to bf16 -> 256-bit
// global stores.  The 2N-wide intermediate never exists in HBM.
//
// Warp roles (384 threads): warps 0 and 3 = TMA producers (one lane each: X tiles, W tiles), warp 1 = MMA
// issuer (one lane, leader CTA only), warp 2 = tensor-memory allocator, warps 4..11 = epilogue (warp w reads
// TMEM lanes 32*(w%4)..+31; the two warps of a lane quarter take alternate 32-column chunks).
//
// Every wait on an mbarrier is bounded: after kWaitLimitCycles the waiting role records itself in
// g_watchdog, raises a CTA-wide abort flag and all roles fall through to the common teardown, which
// frees tensor memory.  No wait in this file can spin forever.
//
// Also here: swiglu_bwd_act_kernel (element-wise backward of the activation) and swiglu_simt_kernel (validation).
#pragma once
#include <cuda_runtime.h>

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
constexpr long long kWaitLimitCycles = 6000000000LL;  // default wait limit: three to four seconds of SM cycles
constexpr int kStageOutBytes = 2048;   // one 32-row x 32-column bf16 box of Y on its way to a TMA store
constexpr int kStagingBytes = kEpiWarps * 2 * kStageOutBytes;  // two boxes per epilogue warp

constexpr int kMaxScatterOwners = 8;  // GPUs of one NVLink domain a scattered plain GEMM can write to
// Tensor maps of a scattered plain GEMM's destinations: [set][owner], one per GPU that owns a block of C's rows
// (this GPU included), written once by magi_swiglu_scatter_setup.  Two sets so that consecutive steps can alternate.
__constant__ CUtensorMap g_scatter_maps[2][kMaxScatterOwners];
// The same destinations as boxes of 32 rows x 64 columns (128-byte rows, 128-byte swizzle): half as many, twice as
// large writes on the links.  Used when the tile width allows (scatter_wide).
__constant__ CUtensorMap g_scatter_maps_wide[2][kMaxScatterOwners];

__device__ unsigned int g_watchdog[4];  // {role that gave up, block, stage/buffer, parity}
// {SM cycles, nanoseconds} block 0 of the most recent tile kernel spent between set-up and teardown: the
// SM clock the kernel really ran at (power capping moves it within a millisecond; nvidia-smi cannot see that)
__device__ unsigned long long g_clock_probe[2];

#ifdef MAGI_SWIGLU_TRACE
// Tuning builds only: SM-cycle timestamps of block 0's second tile (MMA issuer and first epilogue warp).
__device__ long long g_trace[32];
#define MAGI_TRACE(slot, cond) do { if (blockIdx.x == 0 && (cond)) g_trace[slot] = clock64(); } while (0)
#define MAGI_TRACE_T0() const long long trace_t0 = clock64()
#define MAGI_TRACE_ADD(slot) do { if (blockIdx.x == 0) g_trace[slot] += clock64() - trace_t0; } while (0)
#define MAGI_TRACE_ADD_IF(slot, cond) do { if (blockIdx.x == 0 && (cond)) g_trace[slot] += clock64() - trace_t0; } while (0)
#else
#define MAGI_TRACE(slot, cond) do { } while (0)
#define MAGI_TRACE_T0() do { } while (0)
#define MAGI_TRACE_ADD(slot) do { } while (0)
#define MAGI_TRACE_ADD_IF(slot, cond) do { } while (0)
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
  const float* row_scale;  // optional [M] fp32: accumulators of row m are multiplied by row_scale[m] before the
                           // epilogue (a fused RMSNorm: 1/rms(x_m), the norm weight being folded into W); null = none
  __nv_bfloat16* h;   // non-null: the forward also writes the pre-activations H = [G | U] (bf16, [M, 2N], row stride ldh)
  long long ldh;
  int wide_h;         // rows of H allow 32-byte stores
  const __nv_bfloat16* dy;  // non-null: backward mode, Y is dH [M, 2N] = [dG | dU] computed from the accumulators and dY
  long long lddy;
  const float* out_scale;  // out_kind 1: Y is fp8 e4m3 (one byte per element), y = sat(silu(g)*u / *out_scale);
                           // out_kind 2: Y is nvfp4 (two e2m1 codes per byte), *out_scale is the tensor-wide scale
  int out_kind;            // 0 bf16, 1 fp8, 2 nvfp4
  uint8_t* sf;             // nvfp4: e4m3 scale factor per (row, 16 columns)
  long long ld_sf;         // linear layout: bytes per row of sf
  int sf_swizzled;         // 1: 128 x 4 tiled layout
  int sf_ktiles;
  int a_mn, b_mn;     // plain GEMM only: 1 = that operand is stored with the reduction index as the ROW index
                      // (A as [K, M], B as [K, N]), so its shared-memory tile is MN-major
  int plain;          // 1: plain GEMM C = A·B^T; B's first N rows fill output columns [0,N), its last N rows [N,2N)
  int x_hint, w_hint, y_hint;  // L2 eviction priority of X tiles, W tiles and Y stores: 0 normal, 1 first, 2 last
  // Split-K (STREAM schedule on narrow weights): k_splits CTAs share one tile, each sums kb_per_split K-steps and
  // parks its fp32 partial sums in `ws`; swiglu_splitk_reduce_kernel adds them in split order and writes Y.
  // k_splits == 1: no scratch is touched.
  int k_splits, kb_per_split;
  float* ws;  // [tile][split][lane quarter < ceil(M/32)][chunk][gate float4s | up float4s][32 lanes] fp32
  // Stream-K (tile schedules, with scratch): tiles [0, sk_first_tile) are whole-tile work items dealt round-robin
  // in full waves; the K-steps of the remaining tiles (one full wave plus the partial one) form one iteration space
  // cut into equal ranges, one per CTA (pair), so the last wave is never mostly empty.  A range that ends inside a
  // tile leaves that tile's head piece with this unit (the owner) and its later piece with the next unit, which
  // parks fp32 partial sums in scratch slot `unit` and raises sk_flags[unit * kCtas + cta_rank] once per epilogue
  // warp; the owner adds them before its epilogue.  sk_first_tile == number of tiles: off.
  int sk_first_tile, sk_iters_per_unit, sk_total_iters, sk_min_kb;
  int* sk_flags;       // [units * kCtas], zeroed by the host before the launch
  float* sk_partials;  // [units * kCtas][8 epilogue warps][chunks per warp][16 float4][32 lanes] fp32
  int y_tma;  // 1: bf16 Y (or the plain GEMM's C) leaves through shared memory and TMA stores (tm_y is valid)
  // Scattered plain GEMM: rows [o * scatter_rows, (o + 1) * scatter_rows) of C go to the buffer of owner o through
  // g_scatter_maps[scatter_set][o] (TMA stores only; y is null).  0: off.
  int scatter_rows, scatter_set;
  int scatter_wide;  // 1: CTA pairs in split mode with half-tiles that are multiples of 64 columns: 64-column boxes
  long long wait_limit;  // SM cycles after which a wait on an mbarrier gives up (kWaitLimitCycles by default)
};

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned role,
                                             unsigned idx, long long limit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
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

// Bounded wait for a counter in global memory that CTAs of the same launch raise (stream-K hand-over).
__device__ __forceinline__ bool wait_flag_bounded(const int* flag, int target, volatile int* abort_flag, unsigned role,
                                                  unsigned idx, long long limit) {
  const long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = 1;
        if (atomicCAS(&g_watchdog[0], 0u, role) == 0u) {
          g_watchdog[1] = blockIdx.x;
          g_watchdog[2] = idx;
          g_watchdog[3] = (unsigned)v;
        }
        return false;
      }
    }
  }
}

// One piece of work of a CTA (pair): a whole tile, one split of a STREAM split-K tile, or a K range of a stream-K tile.
struct WorkItem {
  int t;                 // tile index in raster order
  int kb0, kb1;          // K-steps [kb0, kb1)
  int zsplit;            // STREAM split-K: which split of the tile
  int sk_role;           // stream-K: 0 whole tile, 1 head piece (owns the tile), 2 later piece (parks partial sums)
  int sk_first_peer, sk_peers;  // head piece: units first_peer .. first_peer + peers - 1 hold the tile's other pieces
};

// First iteration of unit v's stream-K range: v equal shares, moved to a tile boundary when the cut would leave a
// piece shorter than sk_min_kb K-steps.  Both neighbours evaluate the same function, so ranges tile the space.
__host__ __device__ __forceinline__ int sk_boundary(const KArgs& a, int v) {
  const long long raw = (long long)v * a.sk_iters_per_unit;
  const int x = raw < a.sk_total_iters ? (int)raw : a.sk_total_iters;
  const int off = x % a.num_k_blocks;
  if (off == 0) return x;
  if (off < a.sk_min_kb) return x - off;
  if (a.num_k_blocks - off < a.sk_min_kb) return x + (a.num_k_blocks - off);
  return x;
}

// The sequence of work items of one unit; every role of the CTA walks the same sequence.
struct WorkIter {
  const KArgs& a;
  int unit, units, item, cur, end;
  bool in_sk;
  __host__ __device__ __forceinline__ WorkIter(const KArgs& args, int unit_, int units_)
      : a(args), unit(unit_), units(units_), item(unit_), cur(0), end(0), in_sk(false) {}
  __host__ __device__ __forceinline__ bool next(WorkItem& w) {
    if (!in_sk) {
      const int dp_items = a.sk_first_tile * a.k_splits;
      if (item < dp_items) {
        w.t = item / a.k_splits;
        w.zsplit = item - w.t * a.k_splits;
        w.kb0 = w.zsplit * a.kb_per_split;
        w.kb1 = w.kb0 + a.kb_per_split < a.num_k_blocks ? w.kb0 + a.kb_per_split : a.num_k_blocks;
        w.sk_role = 0;
        w.sk_first_peer = w.sk_peers = 0;
        item += units;
        return true;
      }
      in_sk = true;
      if (a.sk_total_iters > 0) {
        cur = sk_boundary(a, unit);
        end = sk_boundary(a, unit + 1);
      }
    }
    if (cur >= end) return false;
    const int nk = a.num_k_blocks;
    const int t_rel = cur / nk;
    const int off = cur - t_rel * nk;
    const int tile_end = (t_rel + 1) * nk;
    const int piece_end = end < tile_end ? end : tile_end;
    w.t = a.sk_first_tile + t_rel;
    w.kb0 = off;
    w.kb1 = piece_end - t_rel * nk;
    w.zsplit = 0;
    w.sk_first_peer = w.sk_peers = 0;
    if (off > 0) {
      w.sk_role = 2;
    } else if (piece_end == tile_end) {
      w.sk_role = 0;
    } else {  // the tile continues in the ranges of the next unit(s)
      w.sk_role = 1;
      w.sk_first_peer = unit + 1;
      int v = unit + 1;
      while (v < units && sk_boundary(a, v) < tile_end) ++v;
      w.sk_peers = v - (unit + 1);
    }
    cur = piece_end;
    return true;
  }
};

// Exercises the bounded wait by itself: one mbarrier that nothing ever signals, no copy or MMA in flight.  Thread 0
// waits on it, gives up after `limit` cycles, records {role 7, block 0, index 42, parity 0} in g_watchdog like any
// role of the tile kernels would, and the kernel returns normally.
constexpr unsigned kWatchdogSelftestRole = 7u, kWatchdogSelftestIndex = 42u;
__global__ void watchdog_selftest_kernel(long long limit) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) wait_bounded(smem_u32(&bar), 0u, &abort_flag, kWatchdogSelftestRole, kWatchdogSelftestIndex, limit);
  __syncthreads();
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

// y[i] = silu(g[i]) * u[i] for four neighbouring columns of one row, branch-free.
// The epilogue is bound by the special-function unit (16 results per cycle and SM) and by instruction issue, so
// the four sigmoids share ONE reciprocal: with a_i = 1 + 2^(-g_i*log2(e)), 1/a_i = (product of the other three a)
// / (product of all four) — nine multiplications on the FMA pipe instead of three more rcp, 1.25 special-function
// results per output instead of 2.  The exponent is clamped at 31 so the product stays below 2^125: exact down to
// g = -21.49; below that the result is g*u*2^-31 instead of g*u*e^g (both below 1e-8*|u|), a NaN or infinity in one
// column cannot reach its neighbours (min() drops a NaN exponent, the NaN returns through g*u), and g = -inf gives
// an infinity of the sign of -u where the plain formula gives NaN.  Groups are aligned to four columns of Y whatever
// the schedule, tile width or column shard, so every schedule still produces the same bits.
__device__ __forceinline__ void silu_mul4(const uint32_t* g, const uint32_t* u, float (&y)[4]) {
  constexpr float kNegLog2e = -1.4426950408889634f;
#ifdef MAGI_SWIGLU_PLAIN_SILU  // tuning builds only: one ex2 and one rcp per output, for comparison
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float gi = __uint_as_float(g[i]);
    y[i] = (gi * __uint_as_float(u[i])) * rcp_approx(1.0f + ex2_approx(gi * kNegLog2e));
  }
#else
  float a[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) a[i] = 1.0f + ex2_approx(fminf(__uint_as_float(g[i]) * kNegLog2e, 31.0f));
  const float p01 = a[0] * a[1], p23 = a[2] * a[3];
  const float r = rcp_approx(p01 * p23);
  const float r01 = r * p23, r23 = r * p01;
  y[0] = (__uint_as_float(g[0]) * __uint_as_float(u[0])) * (r01 * a[1]);
  y[1] = (__uint_as_float(g[1]) * __uint_as_float(u[1])) * (r01 * a[0]);
  y[2] = (__uint_as_float(g[2]) * __uint_as_float(u[2])) * (r23 * a[3]);
  y[3] = (__uint_as_float(g[3]) * __uint_as_float(u[3])) * (r23 * a[2]);
#endif
}

__device__ __forceinline__ uint4 swiglu_pack8(const uint32_t* g, const uint32_t* u) {
  float lo[4], hi[4];
  silu_mul4(g, u, lo);
  silu_mul4(g + 4, u + 4, hi);
  uint4 v;
  __nv_bfloat162 p;
  p = __floats2bfloat162_rn(lo[0], lo[1]);
  v.x = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(lo[2], lo[3]);
  v.y = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(hi[0], hi[1]);
  v.z = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(hi[2], hi[3]);
  v.w = *reinterpret_cast<uint32_t*>(&p);
  return v;
}

// Plain-GEMM epilogue: eight fp32 accumulator values rounded to bf16, no activation.
__device__ __forceinline__ uint4 plain_pack8(const uint32_t* v) {
  uint4 o;
  __nv_bfloat162 p;
  p = __floats2bfloat162_rn(__uint_as_float(v[0]), __uint_as_float(v[1]));
  o.x = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(__uint_as_float(v[2]), __uint_as_float(v[3]));
  o.y = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(__uint_as_float(v[4]), __uint_as_float(v[5]));
  o.z = *reinterpret_cast<uint32_t*>(&p);
  p = __floats2bfloat162_rn(__uint_as_float(v[6]), __uint_as_float(v[7]));
  o.w = *reinterpret_cast<uint32_t*>(&p);
  return o;
}

template <int kCols>
__device__ __forceinline__ void store_cols_plain(__nv_bfloat16* dst, const uint32_t* v, int cols_valid, bool wide,
                                                 uint64_t policy) {
#pragma unroll
  for (int j = 0; j < kCols / 16; ++j) {
    if (16 * j + 16 <= cols_valid) {
      const uint4 lo = plain_pack8(v + 16 * j), hi = plain_pack8(v + 16 * j + 8);
      if (wide) {
        st_global_v8_hint(dst + 16 * j, lo, hi, policy);
      } else {
        st_global_v4_hint(dst + 16 * j, lo, policy);
        st_global_v4_hint(dst + 16 * j + 8, hi, policy);
      }
    } else if (16 * j + 8 <= cols_valid) {
      st_global_v4_hint(dst + 16 * j, plain_pack8(v + 16 * j), policy);
    }
  }
}

// Backward of the activation on fp32 accumulators: from G, U (recomputed, never rounded) and dY (bf16, read here)
//   dG = dY * U * s * (1 + G * (1 - s)),   dU = dY * G * s,   s = sigmoid(G)
// kCols consecutive columns of one row; dG goes to dst_g, dU to dst_u (N columns further in the same row of dH).
template <int kCols>
__device__ __forceinline__ void store_cols_bwd(__nv_bfloat16* dst_g, __nv_bfloat16* dst_u, const __nv_bfloat16* dy,
                                               const uint32_t* g, const uint32_t* u, int cols_valid, uint64_t policy) {
#pragma unroll
  for (int j = 0; j < kCols / 8; ++j) {
    if (8 * j + 8 <= cols_valid) {
      const uint4 dv = __ldg(reinterpret_cast<const uint4*>(dy + 8 * j));
      const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
      uint4 og, ou;
      __nv_bfloat162* og2 = reinterpret_cast<__nv_bfloat162*>(&og);
      __nv_bfloat162* ou2 = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 d = __bfloat1622float2(d2[q]);
        const float gx = __uint_as_float(g[8 * j + 2 * q]), gy = __uint_as_float(g[8 * j + 2 * q + 1]);
        const float ux = __uint_as_float(u[8 * j + 2 * q]), uy = __uint_as_float(u[8 * j + 2 * q + 1]);
        const float sx = __fdividef(1.0f, 1.0f + __expf(-gx)), sy = __fdividef(1.0f, 1.0f + __expf(-gy));
        og2[q] = __floats2bfloat162_rn(d.x * ux * sx * (1.0f + gx * (1.0f - sx)),
                                       d.y * uy * sy * (1.0f + gy * (1.0f - sy)));
        ou2[q] = __floats2bfloat162_rn(d.x * gx * sx, d.y * gy * sy);
      }
      st_global_v4_hint(dst_g + 8 * j, og, policy);
      st_global_v4_hint(dst_u + 8 * j, ou, policy);
    }
  }
}

// fp8 (e4m3, saturating) output: kCols consecutive outputs of one row, 16 per 16-byte store; N % 16 == 0.
template <int kCols>
__device__ __forceinline__ void store_cols_fp8(uint8_t* dst, const uint32_t* g, const uint32_t* u, int cols_valid,
                                               float inv_scale, uint64_t policy) {
#pragma unroll
  for (int j = 0; j < kCols / 16; ++j) {
    if (16 * j + 16 <= cols_valid) {
      uint32_t w4[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int i = 16 * j + 4 * q;
        const float v0 = silu_mul(__uint_as_float(g[i]), __uint_as_float(u[i])) * inv_scale;
        const float v1 = silu_mul(__uint_as_float(g[i + 1]), __uint_as_float(u[i + 1])) * inv_scale;
        const float v2 = silu_mul(__uint_as_float(g[i + 2]), __uint_as_float(u[i + 2])) * inv_scale;
        const float v3 = silu_mul(__uint_as_float(g[i + 3]), __uint_as_float(u[i + 3])) * inv_scale;
        uint16_t lo, hi;  // cvt packs its first source into the upper byte
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(v1), "f"(v0));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(v3), "f"(v2));
        w4[q] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      st_global_v4_hint(dst + 16 * j, make_uint4(w4[0], w4[1], w4[2], w4[3]), policy);
    }
  }
}

// Where the scale factor of row m, 16-column block kb lives.  Linear: sf[m * ld + kb].  Swizzled: the 128 x 4 tiling
// of block-scaled GEMM operands (tiles of 128 rows x 4 blocks, 512 bytes each, tile row r at (r % 32) * 16 +
// (r / 32) * 4), `ktiles` = ceil(blocks per row / 4).
__device__ __forceinline__ long long nvfp4_sf_offset(long long m, int kb, int swizzled, long long ld, int ktiles) {
  if (!swizzled) return m * ld + kb;
  const long long tile = (m >> 7) * ktiles + (kb >> 2);
  const int r = (int)(m & 127);
  return tile * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3);
}

// nvfp4 output: blocks of 16 consecutive outputs share one e4m3 scale factor,
//   sf = e4m3(gs * max|y| / 6),   code_i = e2m1(y_i * gs / sf)   (0 when sf == 0),
// two codes per byte (even column in the low nibble); gs is the tensor-wide scale.  N % 16 == 0.
template <int kCols>
__device__ __forceinline__ void store_cols_fp4(uint8_t* dst, uint8_t* sf, long long m, int kb0, int sf_swizzled,
                                               long long ld_sf, int sf_ktiles, const uint32_t* g, const uint32_t* u,
                                               int cols_valid, float gs, float inv_gs, uint64_t policy) {
#pragma unroll
  for (int j = 0; j < kCols / 16; ++j) {
    if (16 * j + 16 <= cols_valid) {
      float v[16];
      float vmax = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        v[i] = silu_mul(__uint_as_float(g[16 * j + i]), __uint_as_float(u[16 * j + i]));
        vmax = fmaxf(vmax, fabsf(v[i]));
      }
      const uint32_t sf8 = f32_to_e4m3(gs * (vmax * (1.0f / 6.0f)));
      const float sff = e4m3_to_f32(sf8);
      const float os = (sff != 0.0f) ? __fdividef(1.0f, sff * inv_gs) : 0.0f;
      uint2 o;
      o.x = pack8_e2m1(v[0] * os, v[1] * os, v[2] * os, v[3] * os, v[4] * os, v[5] * os, v[6] * os, v[7] * os);
      o.y = pack8_e2m1(v[8] * os, v[9] * os, v[10] * os, v[11] * os, v[12] * os, v[13] * os, v[14] * os, v[15] * os);
      st_global_v2_hint(dst + 8 * j, o, policy);
      sf[nvfp4_sf_offset(m, kb0 + j, sf_swizzled, ld_sf, sf_ktiles)] = (uint8_t)sf8;
    }
  }
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
swiglu_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                 const __grid_constant__ CUtensorMap tm_y, const KArgs a) {
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
    if (a.y_tma) prefetch_tensormap(&tm_y);
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
      WorkIter work(a, unit, units);
      WorkItem wk;
      while (ok && work.next(wk)) {
        const int t = wk.t, kb0 = wk.kb0, kb1 = wk.kb1;
        int mt, nt;
        tile_coords(a, t, mt, nt);
        const int row0 = (mt * kCtas + (int)cta_rank) * kBM;
        for (int kb = kb0; kb < kb1; ++kb) {
          {
            MAGI_TRACE_T0();
            if (!wait_bounded(empty_bar(stage), phase ^ 1u, &abort_flag, x_role ? 1u : 4u, stage, a.wait_limit)) {
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
          if (x_role && a.a_mn) {
            // A stored [K, M]: two boxes of 64 rows-of-A x 64 K (8 KB each, one 128-byte line per K index)
#pragma unroll
            for (int i = 0; i < kBM / 64; ++i) {
              if constexpr (kCtas == 1)
                tma_load_2d_hint(st_a + i * 8192, &tm_x, bar, row0 + 64 * i, k0, policy);
              else
                tma_load_2d_pair_hint(st_a + i * 8192, &tm_x, bar, row0 + 64 * i, k0, policy);
            }
          } else if (!x_role && a.b_mn) {
            // B stored [K, 2N]: this CTA's columns of the first half, then of the second half, 64 at a time.
            // One CTA: block_n columns of each half.  Pair: rank r brings all block_n columns of half r (one MMA
            // over both halves, or split mode), else half of the columns of each half.
            const int nb = a.block_n / 64;  // block_n is a multiple of 64 in this mode
            for (int i = 0; i < 2 * nb / kCtas; ++i) {
              int col;
              if constexpr (kCtas == 1) {
                col = (i / nb) * a.N + nt * a.block_n + 64 * (i % nb);
              } else if (a.n_mma == 1 || a.split) {
                col = (int)cta_rank * a.N + nt * a.block_n + 64 * i;
              } else {
                const int hb = nb / 2;
                col = (i / hb) * a.N + nt * a.block_n + (int)cta_rank * (a.block_n / 2) + 64 * (i % hb);
              }
              if constexpr (kCtas == 1)
                tma_load_2d_hint(st_b + i * 8192, &tm_w, bar, col, k0, policy);
              else
                tma_load_2d_pair_hint(st_b + i * 8192, &tm_w, bar, col, k0, policy);
            }
          } else if constexpr (kCtas == 1) {
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
      const uint32_t idesc = umma_idesc_bf16(kBM * kCtas, mma_n, (uint32_t)a.a_mn, (uint32_t)a.b_mn);
      // operand descriptors of the k-th 16-wide K step of a stage (K-major: 32 bytes further along each row;
      // MN-major: 16 rows = 2048 bytes further)
      const bool a_mn = a.a_mn != 0, b_mn = a.b_mn != 0;
      auto desc_a = [&](uint32_t base, int k) {
        return a_mn ? umma_desc_mn_sw128(base + k * 2048) : umma_desc_k_sw128(base + k * 32);
      };
      auto desc_b = [&](uint32_t base, int k) {
        return b_mn ? umma_desc_mn_sw128(base + k * 2048) : umma_desc_k_sw128(base + k * 32);
      };
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      WorkIter work(a, unit, units);
      WorkItem wk;
      for (; ok && work.next(wk); ++it) {
        const int kb0 = wk.kb0, kb1 = wk.kb1;
        const int buf = (a.acc_bufs == 2) ? (it & 1) : 0;
        const uint32_t acc_phase = (a.acc_bufs == 2) ? ((it >> 1) & 1) : (it & 1);
        MAGI_TRACE(0, it == 2);  // issuer starts waiting for the accumulator of tile 2
        {
          MAGI_TRACE_T0();
          if (!wait_bounded(acc_empty_bar(buf), acc_phase ^ 1u, &abort_flag, 2u, 16 + buf, a.wait_limit)) break;
          MAGI_TRACE_ADD(15);  // issuer: cycles spent waiting for a free accumulator
        }
        MAGI_TRACE(1, it == 2);  // accumulator free
        tc_fence_after_sync();
        const uint32_t d_gate = tmem_base + (uint32_t)(buf * acc_cols);
        int kb = kb0;
        if (kCtas == 2 && a.split) {
          // The low half [gate_lo|up_lo] is free while the epilogue still drains the high half: run the
          // first MMA of as many K-steps as the ring holds, then wait for the high half and catch up.
          const int ahead = min(a.stages, kb1 - kb0);
          int s2 = stage;
          uint32_t p2 = phase;
          for (int j = 0; j < ahead && ok; ++j) {
            if (!wait_bounded(full_bar(s2), p2, &abort_flag, 2u, s2, a.wait_limit)) {
              ok = false;
              break;
            }
            MAGI_TRACE(2, it == 2 && j == 0);
            tc_fence_after_sync();
            const uint32_t sa = tiles_base + s2 * a.stage_bytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_bf16<kCtas>(d_gate, desc_a(sa, k), desc_b(sa + kABytes, k), idesc, (uint32_t)((j | k) != 0));
            if (++s2 == a.stages) {
              s2 = 0;
              p2 ^= 1u;
            }
          }
          if (!ok) break;
          if (!wait_bounded(acc_empty_bar(1), acc_phase ^ 1u, &abort_flag, 2u, 17, a.wait_limit)) break;
          tc_fence_after_sync();
          for (int j = 0; j < ahead; ++j) {
            const uint32_t sa = tiles_base + stage * a.stage_bytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_bf16<kCtas>(d_gate + a.block_n, desc_a(sa, k), desc_b(sa + kABytes + a.b_second, k), idesc,
                               (uint32_t)((j | k) != 0));
            umma_commit<kCtas>(empty_bar(stage));
            if (++stage == a.stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          kb = kb0 + ahead;
        }
        // Split mode ends a tile the way it begins one, mirrored: the low-half MMAs of the last K-steps (as many as
        // the ring holds) go first and the low half is handed to the epilogue while the high-half MMAs of those
        // steps still run, so the drain of the low half overlaps tensor work at both ends of the tile.
        const int kb_tail = (kCtas == 2 && a.split) ? max(kb, kb1 - a.stages) : kb1;
        bool low_done = false;
        for (; kb < kb_tail; ++kb) {
          {
            MAGI_TRACE_T0();
            if (!wait_bounded(full_bar(stage), phase, &abort_flag, 2u, stage, a.wait_limit)) {
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
              const uint64_t ad = desc_a(sa, k);
              umma_bf16<kCtas>(d_gate, ad, desc_b(sb, k), idesc, acc);
              if (a.n_mma == 2) umma_bf16<kCtas>(d_gate + a.block_n, ad, desc_b(sb + a.b_second, k), idesc, acc);
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
        if (ok && kb < kb1) {  // split mode: the tile's last K-steps, low half first
          const int n_tail = kb1 - kb;
          int s2 = stage;
          uint32_t p2 = phase;
          for (int j = 0; j < n_tail && ok; ++j) {
            if (!wait_bounded(full_bar(s2), p2, &abort_flag, 2u, s2, a.wait_limit)) {
              ok = false;
              break;
            }
            MAGI_TRACE(3, it == 1 && j == n_tail - 1);  // last stage of tile 1 available
            tc_fence_after_sync();
            const uint32_t sa = tiles_base + s2 * a.stage_bytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_bf16<kCtas>(d_gate, desc_a(sa, k), desc_b(sa + kABytes, k), idesc, 1u);
            if (++s2 == a.stages) {
              s2 = 0;
              p2 ^= 1u;
            }
          }
          if (!ok) break;
          umma_commit<kCtas>(acc_full_bar(0));  // the low half is complete
          low_done = true;
          MAGI_TRACE(22, it == 1);  // low half of tile 1 committed
          for (int j = 0; j < n_tail; ++j) {
            const uint32_t sa = tiles_base + stage * a.stage_bytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_bf16<kCtas>(d_gate + a.block_n, desc_a(sa, k), desc_b(sa + kABytes + a.b_second, k), idesc, 1u);
            umma_commit<kCtas>(empty_bar(stage));
            if (++stage == a.stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
        if (ok) {
          if (kCtas == 2 && a.split) {  // one "complete" barrier per half
            if (!low_done) umma_commit<kCtas>(acc_full_bar(0));
            umma_commit<kCtas>(acc_full_bar(1));
          } else {
            umma_commit<kCtas>(acc_full_bar(buf));
          }
        }
        MAGI_TRACE(4, it == 1);  // all MMAs of tile 1 issued
        MAGI_TRACE(9, it == 2);  // all MMAs of tile 2 issued
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue (every CTA drains its own 128 rows)
    const int q = warp & 3;
    const uint64_t y_policy = l2_policy(a.y_hint);
    const uint32_t acc_empty_remote0 = (kCtas == 2) ? map_to_cta(acc_empty_bar(0), 0) : 0u;
    // Y through shared memory: this warp's two 32-row x 32-column boxes (64-byte rows, 64-byte swizzle) behind the ring
    const uint32_t stg_base = tiles_base + (uint32_t)a.stages * a.stage_bytes + (uint32_t)(warp - 4) * (2u * kStageOutBytes);
    uint32_t stg_par = 0;
    int it = 0;
    WorkIter work(a, unit, units);
    WorkItem wk;
    for (; work.next(wk); ++it) {
      const int t = wk.t, zsplit = wk.zsplit;
      const int buf = (a.acc_bufs == 2) ? (it & 1) : 0;
      const uint32_t acc_phase = (a.acc_bufs == 2) ? ((it >> 1) & 1) : (it & 1);
      int mt, nt;
      tile_coords(a, t, mt, nt);
      // split mode: acc_full_bar(0) = low half complete, acc_full_bar(1) = high half complete (waited for below)
      bool ok = wait_bounded(acc_full_bar(buf), acc_phase, &abort_flag, 3u, buf, a.wait_limit);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      MAGI_TRACE(5, it == 1 && warp == 4 && lane == 0);  // epilogue sees tile 1 complete
      tc_fence_after_sync();
      if (wk.sk_role == 1) {
        // Stream-K head piece: the tile's later pieces were the FIRST items of the next units' ranges and were parked
        // long ago; every epilogue warp of the parking CTA raises the flag once.
        bool peers_ok = true;
        if (lane == 0) {
          for (int pz = 0; pz < wk.sk_peers && peers_ok; ++pz)
            peers_ok = wait_flag_bounded(a.sk_flags + (wk.sk_first_peer + pz) * kCtas + (int)cta_rank, kEpiWarps,
                                         &abort_flag, 5u, (unsigned)(wk.sk_first_peer + pz), a.wait_limit);
        }
        peers_ok = __all_sync(0xffffffffu, peers_ok);
        if (!peers_ok) break;
      }
      // Stream-K scratch of one CTA: [epilogue warp][chunk of the warp][16 float4 = 8 of gate, 8 of up][lane].  The
      // parking warp and the owning warp walk the same chunks with the same lanes, so lane l's k-th float4 of a
      // chunk sits next to lane l+1's: every store and load of a warp is one contiguous 512-byte piece.
      const int sk_chunks = (kCtas == 2 && a.split ? 2 : 1) * ((a.block_n / (kCtas == 2 && a.split ? 2 : 1) + 63) / 64);
      const size_t sk_cta_f4 = (size_t)kEpiWarps * sk_chunks * 16 * 32;
      auto sk_slab = [&](int of_unit) {
        return reinterpret_cast<uint4*>(a.sk_partials) + ((size_t)(of_unit * kCtas + (int)cta_rank)) * sk_cta_f4 +
               (size_t)(warp - 4) * sk_chunks * 16 * 32 + lane;
      };
      int sk_ck = 0;  // chunks of this tile this warp has dealt with
      const int row = (mt * kCtas + (int)cta_rank) * kBM + q * 32 + lane;
      const bool row_ok = row < a.M;
      const int col0 = nt * a.block_n;
      const int valid_tile = min(a.block_n, a.N - col0);  // multiple of 8
      const uint32_t t_tile = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * acc_cols);
      __nv_bfloat16* yrow_tile = a.y + (long long)row * a.ldy + col0;
      const bool wide = a.wide_store != 0;  // every 16-column group of every row starts on a 32-byte boundary
      const float row_scale_m = (a.row_scale != nullptr && row_ok) ? __ldg(a.row_scale + row) : 1.0f;
      const float out_gs = (a.out_kind != 0) ? __ldg(a.out_scale) : 1.0f;
      const float out_inv_scale = 1.0f / out_gs;

      if (kCtas == 2 && a.scatter_wide) {
        // ---- scattered plain GEMM, wide boxes.  Tensor memory holds [lo: first | second][hi: first | second] halves
        // of B's two row blocks, each seg_cols wide; the two warps of a lane quarter take one block each and drain it
        // in groups of 64 columns: two tensor-memory loads, one 32-row x 64-column box (128-byte rows, 128-byte
        // swizzle) in this warp's 4 KiB of staging memory, one TMA store through the map of the GPU that owns the rows.
        const int blk = (warp - 4) >> 2;  // 0: rows [0, N) of B (output columns n), 1: rows [N, 2N) (columns N + n)
        const int seg_cols = a.block_n / 2;
        const uint32_t stage_buf = stg_base;
        const int box_row0 = (mt * kCtas + (int)cta_rank) * kBM + q * 32;
        const int owner = box_row0 / a.scatter_rows;
        const CUtensorMap* dst_map = &g_scatter_maps_wide[a.scatter_set][owner];
        bool seg_ok = true;
        for (int seg = 0; seg < 2; ++seg) {
          if (seg == 1) {
            seg_ok = wait_bounded(acc_full_bar(1), acc_phase, &abort_flag, 3u, 1, a.wait_limit);
            seg_ok = __all_sync(0xffffffffu, seg_ok);
            if (!seg_ok) break;
            tc_fence_after_sync();
          }
          const uint32_t t_src0 = t_tile + (uint32_t)(seg * a.block_n + blk * seg_cols);
          const int valid = max(0, min(seg_cols, valid_tile - seg * seg_cols));
          for (int c = 0; c < seg_cols; c += 64) {
            uint32_t v0[32], v1[32];
            tmem_ld_x32(t_src0 + c, v0);
            tmem_ld_x32(t_src0 + c + 32, v1);
            tmem_ld_wait();
            tmem_regs_ready(v0);
            tmem_regs_ready(v1);
            if (c + 64 >= seg_cols) {  // last read of this half: hand it back before the stores
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster_relaxed(acc_empty_remote0 + 8u * seg);
            }
            if (c >= valid) continue;  // columns past N (whole boxes: N is a multiple of 64 here)
            if (lane == 0) bulk_wait_group_read<0>();  // the previous box has left the staging memory
            __syncwarp();
            const uint32_t rowaddr = stage_buf + (uint32_t)lane * 128u;
            const uint32_t sw = (uint32_t)lane & 7u;
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              const uint4 lo = plain_pack8(v0 + 8 * j), hi = plain_pack8(v1 + 8 * j);
              st_shared_v4(rowaddr + ((j ^ sw) << 4), lo.x, lo.y, lo.z, lo.w);
              st_shared_v4(rowaddr + (((j + 4) ^ sw) << 4), hi.x, hi.y, hi.z, hi.w);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && box_row0 < a.M) {
              tma_store_3d(stage_buf, dst_map, col0 + seg * seg_cols + c, blk, box_row0 - owner * a.scatter_rows);
              bulk_commit_group();
            }
          }
        }
        if (!seg_ok) break;
        continue;
      }
      if (kCtas == 1 && a.k_splits > 1) {
        // ---- split-K: park this CTA's fp32 partial sums; swiglu_splitk_reduce_kernel finishes the tile.
        // Scratch of one (tile, split): [lane quarter < ceil(M/32)][chunk][gate float4s, then up float4s][32 lanes]:
        // lane l's k-th float4 of a chunk sits next to lane l+1's, so each store of a warp is one 512-byte piece.
        const int slot = warp - 4;
        const int quarters = (a.M + 31) >> 5;
        auto chunk_w = [&](int c) { return (c + 32 <= a.block_n) ? 32 : ((c + 16 == a.block_n) ? 16 : 0); };
        uint4* part = reinterpret_cast<uint4*>(a.ws) +
                      ((size_t)(t * a.k_splits + zsplit) * quarters + q) * (size_t)(a.block_n / 2) * 32 + lane;
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
          tmem_regs_ready(g);
          tmem_regs_ready(u);
          if (!chunk_w(c + 64)) {  // last read of the accumulator: hand it back before the stores
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_relaxed(acc_empty_bar(buf));
            released = true;
          }
          if (row_ok) {
            uint4* dst = part + (size_t)(c / 32) * 16 * 32;  // every chunk before this one is 32 columns wide
            const int nv = w / 4;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (j < nv) {
                __stcg(dst + j * 32, make_uint4(g[4 * j], g[4 * j + 1], g[4 * j + 2], g[4 * j + 3]));
                __stcg(dst + (nv + j) * 32, make_uint4(u[4 * j], u[4 * j + 1], u[4 * j + 2], u[4 * j + 3]));
              }
            }
          }
        }
        if (!released) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_relaxed(acc_empty_bar(buf));
        }
        continue;
      }

      // A tile is drained in one segment (gate columns [0,bn), up columns [bn,2bn)) or, in split mode, in two
      // (low half then high half, each [gate|up] of bn/2 columns) that are released separately.
      const int num_seg = (kCtas == 2 && a.split) ? 2 : 1;
      const int seg_cols = a.block_n / num_seg;
      bool seg_ok = true;
      for (int seg = 0; seg < num_seg; ++seg) {
        if (seg == 1) {  // the high half has its own "complete" barrier
          seg_ok = wait_bounded(acc_full_bar(1), acc_phase, &abort_flag, 3u, 1, a.wait_limit);
          seg_ok = __all_sync(0xffffffffu, seg_ok);
          if (!seg_ok) break;
          tc_fence_after_sync();
        }
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
        // One box of Y on its way out: the warp writes its 32 rows x 32 columns (16 packed words per lane) into the
        // free one of its two staging buffers and lane 0 hands the buffer to a TMA store.  Row r of the box is
        // 64 bytes; its 16-byte piece j sits at piece j ^ ((r >> 1) & 3) (the 64-byte swizzle of the tensor map),
        // which spreads the lanes' 16-byte writes over all banks.  Rows and columns outside Y are clipped by the copy.
        auto stage_out = [&](const uint32_t (&pk)[16], int col, int half) {
          MAGI_TRACE_T0();
          const uint32_t buf = stg_base + stg_par * kStageOutBytes;
          if (lane == 0) bulk_wait_group_read<1>();  // the store that last read this buffer has finished reading it
          __syncwarp();
          const uint32_t rowaddr = buf + (uint32_t)lane * 64u;
          const uint32_t sw = ((uint32_t)lane >> 1) & 3u;
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j)
            st_shared_v4(rowaddr + ((j ^ sw) << 4), pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          const int box_row0 = (mt * kCtas + (int)cta_rank) * kBM + q * 32;
          if (lane == 0 && box_row0 < a.M) {
            if (a.scatter_rows) {  // this box belongs to one owner (scatter_rows is a multiple of 32)
              const int owner = box_row0 / a.scatter_rows;
              tma_store_3d(buf, &g_scatter_maps[a.scatter_set][owner], col, half, box_row0 - owner * a.scatter_rows);
            } else {
              tma_store_3d_hint(buf, &tm_y, col, half, box_row0, y_policy);
            }
            bulk_commit_group();
          }
          stg_par ^= 1u;
          MAGI_TRACE_ADD_IF(27, warp == 4 && lane == 0);  // staging + TMA store issue of one box
        };
        auto process = [&](uint32_t (&g)[32], uint32_t (&u)[32], int c, int w) {
          if (wk.sk_role == 2) {  // stream-K later piece: park the raw fp32 sums of this chunk (all 128 rows)
            uint4* dst = sk_slab(unit) + (size_t)sk_ck * 16 * 32;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (4 * j < w) {
                __stcg(dst + j * 32, make_uint4(g[4 * j], g[4 * j + 1], g[4 * j + 2], g[4 * j + 3]));
                __stcg(dst + (8 + j) * 32, make_uint4(u[4 * j], u[4 * j + 1], u[4 * j + 2], u[4 * j + 3]));
              }
            }
            return;
          }
          if (a.row_scale != nullptr) {  // 1 for rows past M
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              g[j] = __float_as_uint(__uint_as_float(g[j]) * row_scale_m);
              u[j] = __float_as_uint(__uint_as_float(u[j]) * row_scale_m);
            }
          }
          if (a.y_tma && w == 32 && a.h == nullptr) {  // bf16 Y (or plain C) through shared memory, all lanes take part
            const int col = col0 + seg * seg_cols + c;
            uint32_t pk[16];
            if (a.plain) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 v = plain_pack8(g + 8 * j);
                pk[4 * j] = v.x, pk[4 * j + 1] = v.y, pk[4 * j + 2] = v.z, pk[4 * j + 3] = v.w;
              }
              stage_out(pk, col, 0);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 v = plain_pack8(u + 8 * j);
                pk[4 * j] = v.x, pk[4 * j + 1] = v.y, pk[4 * j + 2] = v.z, pk[4 * j + 3] = v.w;
              }
              stage_out(pk, col, 1);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 v = swiglu_pack8(g + 8 * j, u + 8 * j);
                pk[4 * j] = v.x, pk[4 * j + 1] = v.y, pk[4 * j + 2] = v.z, pk[4 * j + 3] = v.w;
              }
              stage_out(pk, col, 0);
            }
            return;
          }
          if (!row_ok || a.scatter_rows) return;  // a scattered GEMM has no direct-store path (the host only plans whole boxes)
          if (a.h != nullptr) {  // training forward: keep the pre-activations for the backward
            __nv_bfloat16* hrow = a.h + (long long)row * a.ldh + col0 + seg * seg_cols + c;
            if (w == 32) {
              store_cols_plain<32>(hrow, g, valid - c, a.wide_h != 0, y_policy);
              store_cols_plain<32>(hrow + a.N, u, valid - c, a.wide_h != 0, y_policy);
            } else {
              store_cols_plain<16>(hrow, g, valid - c, a.wide_h != 0, y_policy);
              store_cols_plain<16>(hrow + a.N, u, valid - c, a.wide_h != 0, y_policy);
            }
          }
          if (a.dy != nullptr) {  // backward: dH = [dG | dU] from the recomputed pre-activations and dY
            const __nv_bfloat16* dyp = a.dy + (long long)row * a.lddy + col0 + seg * seg_cols + c;
            if (w == 32)
              store_cols_bwd<32>(yrow + c, yrow + a.N + c, dyp, g, u, valid - c, y_policy);
            else
              store_cols_bwd<16>(yrow + c, yrow + a.N + c, dyp, g, u, valid - c, y_policy);
          } else if (a.out_kind == 2) {  // nvfp4 output: half a byte per element + one scale byte per 16
            const int colg = col0 + seg * seg_cols + c;
            uint8_t* y4 = reinterpret_cast<uint8_t*>(a.y) + (long long)row * a.ldy + (colg >> 1);
            if (w == 32)
              store_cols_fp4<32>(y4, a.sf, row, colg >> 4, a.sf_swizzled, a.ld_sf, a.sf_ktiles, g, u, valid - c,
                                 out_gs, out_inv_scale, y_policy);
            else
              store_cols_fp4<16>(y4, a.sf, row, colg >> 4, a.sf_swizzled, a.ld_sf, a.sf_ktiles, g, u, valid - c,
                                 out_gs, out_inv_scale, y_policy);
          } else if (a.out_kind == 1) {  // fp8 output: one byte per element
            uint8_t* y8 = reinterpret_cast<uint8_t*>(a.y) + (long long)row * a.ldy + col0 + seg * seg_cols + c;
            if (w == 32)
              store_cols_fp8<32>(y8, g, u, valid - c, out_inv_scale, y_policy);
            else
              store_cols_fp8<16>(y8, g, u, valid - c, out_inv_scale, y_policy);
          } else if (a.plain) {  // plain GEMM: the "gate" accumulator is output column n, the "up" accumulator column N + n
            if (w == 32) {
              store_cols_plain<32>(yrow + c, g, valid - c, wide, y_policy);
              store_cols_plain<32>(yrow + a.N + c, u, valid - c, wide, y_policy);
            } else {
              store_cols_plain<16>(yrow + c, g, valid - c, wide, y_policy);
              store_cols_plain<16>(yrow + a.N + c, u, valid - c, wide, y_policy);
            }
          } else if (w == 32) {
            store_cols<32>(yrow + c, g, u, valid - c, wide, y_policy);
          } else {
            store_cols<16>(yrow + c, g, u, valid - c, wide, y_policy);
          }
        };
        auto release = [&]() {
          MAGI_TRACE(6 + seg * 14, it == 1 && warp == 4 && lane == 0);  // warp 4 has read its last column (20: high half)
          MAGI_TRACE(7 + seg * 14, it == 1 && warp == 11 && lane == 0);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            // Relaxed arrivals: the tensor-memory reads being signalled are complete (tcgen05.wait::ld) and nothing else
            // is published through this barrier, so the arrival must not wait for this warp's earlier global stores
            // to become visible, which a releasing arrival does (about a thousand cycles on the tile's critical path).
            if constexpr (kCtas == 1)
              mbar_arrive_relaxed(acc_empty_bar(release_buf));
            else  // the leader's MMA issuer waits for both CTAs
              mbar_arrive_cluster_relaxed(acc_empty_remote0 + 8u * release_buf);
          }
        };
        uint32_t g[32], u[32];
        int c = 32 * ((warp - 4) >> 2);
        int w = width_at(c);
        bool released = false;
        while (w) {
          {
            MAGI_TRACE_T0();
            load(g, u, c, w);
            tmem_ld_wait();
            tmem_regs_ready(g);
            tmem_regs_ready(u);
            if (wk.sk_role == 1) {  // add the parked sums of the tile's later pieces, in unit order
              for (int pz = 0; pz < wk.sk_peers; ++pz) {
                const uint4* src = sk_slab(wk.sk_first_peer + pz) + (size_t)sk_ck * 16 * 32;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (4 * j < w) {
                    const uint4 pg = __ldcg(src + j * 32);
                    const uint4 pu = __ldcg(src + (8 + j) * 32);
                    g[4 * j] = __float_as_uint(__uint_as_float(g[4 * j]) + __uint_as_float(pg.x));
                    g[4 * j + 1] = __float_as_uint(__uint_as_float(g[4 * j + 1]) + __uint_as_float(pg.y));
                    g[4 * j + 2] = __float_as_uint(__uint_as_float(g[4 * j + 2]) + __uint_as_float(pg.z));
                    g[4 * j + 3] = __float_as_uint(__uint_as_float(g[4 * j + 3]) + __uint_as_float(pg.w));
                    u[4 * j] = __float_as_uint(__uint_as_float(u[4 * j]) + __uint_as_float(pu.x));
                    u[4 * j + 1] = __float_as_uint(__uint_as_float(u[4 * j + 1]) + __uint_as_float(pu.y));
                    u[4 * j + 2] = __float_as_uint(__uint_as_float(u[4 * j + 2]) + __uint_as_float(pu.z));
                    u[4 * j + 3] = __float_as_uint(__uint_as_float(u[4 * j + 3]) + __uint_as_float(pu.w));
                  }
                }
              }
            }
            MAGI_TRACE_ADD_IF(24, warp == 4 && lane == 0);  // epilogue warp 4: tensor-memory loads and their wait
          }
          const int c2 = c + 64, w2 = width_at(c2);
          if (!w2) {  // that was this warp's last read of the segment
            MAGI_TRACE_T0();
            release();
            released = true;
            MAGI_TRACE_ADD_IF(25, warp == 4 && lane == 0);  // hand-back of the accumulator
          }
          {
            MAGI_TRACE_T0();
            process(g, u, c, w);
            MAGI_TRACE_ADD_IF(26, warp == 4 && lane == 0);  // arithmetic + stores of one chunk
          }
          ++sk_ck;
          c = c2;
          w = w2;
        }
        if (!released) release();
      }
      if (!seg_ok) break;
      if (wk.sk_role == 2) {  // this warp's share of the parked sums is written: publish it
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          atomicAdd(a.sk_flags + unit * kCtas + (int)cta_rank, 1);
        }
      }
    }
    if (a.y_tma && lane == 0) {
      if (a.scatter_rows)
        bulk_wait_group<0>();  // stores into other GPUs' memory: complete, not just read, before this CTA retires
      else
        bulk_wait_group_read<0>();  // shared memory stays valid until the last store has read it
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
// split order (bit-identical from run to run).  One thread per row and 8 output columns; consecutive threads take
// consecutive rows of a lane quarter, which are consecutive float4s of the scratch (see the parking code).
__global__ void __launch_bounds__(256)
swiglu_splitk_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ y, int M, int N, long long ldy,
                            int block_n, int num_n_tiles, int k_splits, const float* __restrict__ row_scale) {
  const int groups = block_n / 8;
  const int quarters = (M + 31) >> 5;
  const long long total = (long long)num_n_tiles * quarters * groups * 32;
  const size_t quarter_f4 = (size_t)(block_n / 2) * 32;      // float4s of one (tile, split, quarter)
  const size_t z_stride = (size_t)quarters * quarter_f4;      // ... of one (tile, split)
  const uint64_t policy = l2_policy_evict_first();
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the partial sums of the tile kernel are complete and visible
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int lane = (int)(i & 31);
    const int cg = (int)((i >> 5) % groups);
    const int q = (int)((i / (32LL * groups)) % quarters);
    const int t = (int)(i / (32LL * groups * quarters));
    const int row = q * 32 + lane;
    const int col = t * block_n + cg * 8;
    if (row >= M || col >= N) continue;  // N is a multiple of 8: a group is inside or outside as a whole
    const int ci = cg >> 2, jp = cg & 3;                       // 32-column chunk and pair of float4s inside it
    const int nv = (block_n - 32 * ci >= 32) ? 8 : 4;          // float4s of gate (and of up) in this chunk
    const float4* p = reinterpret_cast<const float4*>(ws) + ((size_t)t * k_splits * quarters + q) * quarter_f4 +
                      (size_t)ci * 16 * 32 + (size_t)(2 * jp) * 32 + lane;
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0}, u[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int z0 = 0; z0 < k_splits; z0 += 4, p += 4 * z_stride) {
      // four splits' loads are issued before the first add so their latencies overlap; the adds keep split order
      float4 v[4][4];
#pragma unroll
      for (int zz = 0; zz < 4; ++zz) {
        if (z0 + zz < k_splits) {
          const float4* r = p + zz * z_stride;
          v[zz][0] = __ldcg(r);
          v[zz][1] = __ldcg(r + 32);
          v[zz][2] = __ldcg(r + nv * 32);
          v[zz][3] = __ldcg(r + nv * 32 + 32);
        }
      }
#pragma unroll
      for (int zz = 0; zz < 4; ++zz) {
        if (z0 + zz < k_splits) {
          g[0] += v[zz][0].x; g[1] += v[zz][0].y; g[2] += v[zz][0].z; g[3] += v[zz][0].w;
          g[4] += v[zz][1].x; g[5] += v[zz][1].y; g[6] += v[zz][1].z; g[7] += v[zz][1].w;
          u[0] += v[zz][2].x; u[1] += v[zz][2].y; u[2] += v[zz][2].z; u[3] += v[zz][2].w;
          u[4] += v[zz][3].x; u[5] += v[zz][3].y; u[6] += v[zz][3].z; u[7] += v[zz][3].w;
        }
      }
    }
    const float rs = row_scale != nullptr ? __ldg(row_scale + row) : 1.0f;
    uint32_t gb[8], ub[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gb[j] = __float_as_uint(g[j] * rs);
      ub[j] = __float_as_uint(u[j] * rs);
    }
    st_global_v4_hint(y + (long long)row * ldy + col, swiglu_pack8(gb, ub), policy);
  }
}

// out[i] = sum over slots of src[slot * slot_stride + i], added in slot order in fp32 and rounded once to bf16: the
// last step of a scattered row-parallel GEMM, where slot r holds what GPU r's epilogue wrote for this GPU's rows.
// The sums are stored to every destination in dst (one local buffer for a reduce-scatter; this GPU's block of the
// result in every GPU's memory, peers included, for an all-reduce: plain coalesced 16-byte stores over NVLink).
// Element-wise, HBM-bound; 8 elements per thread with 16-byte accesses (n % 8 == 0).
struct SumDst {  // where the sums go: one buffer, or the same place in the memory of every GPU of the group
  __nv_bfloat16* p[kMaxScatterOwners];
  int n;
};
__global__ void __launch_bounds__(256)
swiglu_sum_slots_kernel(const __nv_bfloat16* __restrict__ src, const SumDst dst, int slots, long long slot_stride,
                        long long n) {
  const long long groups = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < groups; i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int sl = 0; sl < slots; ++sl) {
      const uint4 v = __ldcs(reinterpret_cast<const uint4*>(src + sl * slot_stride + 8 * i));
      const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    for (int d = 0; d < dst.n; ++d) *reinterpret_cast<uint4*>(dst.p[d] + 8 * i) = o;
  }
}

// Row scales of a fused RMSNorm: out[m] = rsqrt(mean_k x[m,k]^2 + eps), one warp per row, fp32 sums, 16-byte loads.
__global__ void __launch_bounds__(256)
swiglu_row_rms_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int M, int K, long long ldx,
                      float eps) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < M; row += warps) {
    const __nv_bfloat16* xr = x + (long long)row * ldx;
    float acc = 0.f;
    for (int k = lane * 8; k < K; k += 256) {  // K % 8 == 0
      const uint4 v = *reinterpret_cast<const uint4*>(xr + k);
      const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v2[j]);
        acc = fmaf(f.x, f.x, acc);
        acc = fmaf(f.y, f.y, acc);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[row] = rsqrtf(acc / (float)K + eps);
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

}  // namespace magi
