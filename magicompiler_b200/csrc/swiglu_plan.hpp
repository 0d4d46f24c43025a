// Host-side schedule selection for the SwiGLU kernels: which variant, tile width, ring depth, raster band, CTA
// count and (for narrow small-M problems) how many CTAs split K, plus the error-text helpers of the C ABI.
// Pure host arithmetic: nothing here touches a GPU.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/magi_swiglu.h"
#include "swiglu_kernels.cuh"

namespace magi {

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
  cudaGetLastError();  // the error has been reported here: do not leave it for the next, unrelated launch check
  return e == cudaSuccess ? 1 : (int)e;
}

// Tuning aids.  Their initial values are read from the environment ONCE (first use), never on the launch path; tests
// and sweeps change them afterwards through magi_swiglu_tuning():
//   MAGI_SWIGLU_L2_HINTS=xwy  L2 priority of X tiles, W tiles, Y stores (each 0 normal, 1 evict-first, 2 evict-last)
//   MAGI_SWIGLU_K_SPLITS=z    force z-way split-K in the STREAM schedule
//   MAGI_SWIGLU_NO_SPLIT=1    drain pair tiles in one piece instead of two separately released halves
//   MAGI_SWIGLU_Y_TMA=0|1     force Y through direct stores (0) or shared memory + TMA stores (1) in the tile schedules
//   MAGI_SWIGLU_STREAM_K=0|1  never / whenever possible: balance the last waves of the tile schedules by K ranges
struct Tuning {
  int hints[3] = {-1, -1, -1};
  int k_splits = 0;
  int no_split = 0;
  int y_tma = -1;
  int stream_k = -1;  // -1 choose, 0 never, 1 whenever it is possible
  int scatter_wide = 1;  // scattered GEMM: 64-column store boxes where the tile allows (0: always 32-column boxes)
};
static Tuning& tuning() {
  static Tuning t = [] {
    Tuning v;
    if (const char* env = getenv("MAGI_SWIGLU_L2_HINTS")) {
      if (strlen(env) == 3)
        for (int i = 0; i < 3; ++i) v.hints[i] = (env[i] >= '0' && env[i] <= '2') ? env[i] - '0' : -1;
    }
    if (const char* env = getenv("MAGI_SWIGLU_K_SPLITS")) v.k_splits = atoi(env);
    if (getenv("MAGI_SWIGLU_NO_SPLIT")) v.no_split = 1;
    if (const char* env = getenv("MAGI_SWIGLU_Y_TMA")) v.y_tma = atoi(env) != 0;
    if (const char* env = getenv("MAGI_SWIGLU_STREAM_K")) v.stream_k = atoi(env) != 0;
    return v;
  }();
  return t;
}

struct Plan {
  int variant, block_n, stages, grid, tiles, smem_bytes, acc_bufs, n_mma;
  int num_m_tiles, num_n_tiles, num_k_blocks, group_m;
  int ctas;  // CTAs per tile: 1, or 2 for the CTA-pair schedule
  int split; // CTA pairs with two MMAs per step and block_n % 32 == 0: two separately released half tiles
  int k_splits, kb_per_split;          // split-K of the STREAM schedule (1 = off)
  int64_t ws_bytes;                    // fp32 partial sums of a split-K plan (0 = none)
  uint32_t stage_bytes, b_second;
  int y_tma;  // tile schedules: Y leaves through per-warp staging boxes in shared memory and TMA stores
  // stream-K (tile schedules with scratch): tiles from sk_first_tile on are cut into equal K ranges, one per worker
  int sk_first_tile, sk_iters_per_unit, sk_total_iters, sk_min_kb;
  int64_t sk_flag_bytes;
};

static inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

constexpr int64_t kWorkspaceCap = 64LL << 20;  // never plan for more scratch than this

// Scratch bytes of a split-K plan: per tile k_splits x (M rounded up to whole warps of 32 rows) x 2*block_n fp32
// partial sums.
static inline int64_t splitk_bytes(int64_t tiles, int64_t z, int64_t M, int64_t bn) {
  return tiles * z * ((M + 31) / 32 * 32) * 2 * bn * 4;
}

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

constexpr int kSkMinKb = 8;  // shortest piece of a split tile in K-steps: a shorter one costs more to hand over than it balances

// Scratch of a stream-K plan for `units` workers of `ctas` CTAs each: one flag and one slab of fp32 partial sums per CTA.
static inline int64_t sk_flag_bytes(int units, int ctas) { return ((int64_t)units * ctas * 4 + 255) / 256 * 256; }
static inline int64_t sk_bytes(int units, int ctas, int bn) {
  // per CTA: 8 epilogue warps x chunks per warp x (16 float4 x 32 lanes); a warp takes every other 32-column chunk
  // of a tile half (pairs with two separately released halves) or of the whole tile
  const bool halves = ctas == 2 && 2 * bn > 256 && bn % 32 == 0;
  const int chunks = (halves ? 2 : 1) * ((bn / (halves ? 2 : 1) + 63) / 64);
  return sk_flag_bytes(units, ctas) + (int64_t)units * ctas * kEpiWarps * chunks * 16 * 32 * 16;
}

// Whether `tiles` tiles of num_kb K-steps on `units` workers should end in a stream-K phase (scratch permitting).
// In that phase neighbouring workers sit at K offsets one remainder-fraction of a tile apart, so tiles that share an
// operand panel stop reading it at the same time once the fraction grows: measured on B200 the phase pays up to a
// quarter of a wave of remainder (a last wave at most a quarter full) and costs more than it saves beyond that.
static inline bool sk_wanted(int64_t tiles, int num_kb, int units, int ctas, int bn, int64_t ws_limit) {
  if (tuning().stream_k == 0 || units < 2 || tiles < 1) return false;
  const int64_t waves = tiles / units, rem = tiles - waves * units;
  if (rem == 0) return false;
  if (tuning().stream_k != 1 && rem * 4 > (int64_t)units) return false;
  const int64_t sk_tiles = waves >= 1 ? units + rem : tiles;
  const int64_t total = sk_tiles * num_kb, q = (total + units - 1) / units;
  if (q < 2 * kSkMinKb || 4 * q < num_kb || total > 0x3fffffffLL) return false;  // pieces too short / too many per tile
  return sk_bytes(units, ctas, bn) <= ws_limit;
}

// Fills the plan's stream-K fields for `units` workers; returns the scratch bytes (0 = plain whole-tile schedule).
static int64_t sk_setup(Plan* p, int units, int64_t ws_limit) {
  p->sk_first_tile = p->tiles;
  p->sk_iters_per_unit = p->sk_total_iters = 0;
  p->sk_min_kb = kSkMinKb;
  p->sk_flag_bytes = 0;
  if (p->variant != MAGI_SWIGLU_VARIANT_MMA && p->variant != MAGI_SWIGLU_VARIANT_MMA2) return 0;
  if (p->k_splits != 1 || !sk_wanted(p->tiles, p->num_k_blocks, units, p->ctas, p->block_n, ws_limit)) return 0;
  const int waves = p->tiles / units, rem = p->tiles - waves * units;
  const int sk_tiles = waves >= 1 ? units + rem : p->tiles;
  p->sk_first_tile = p->tiles - sk_tiles;
  p->sk_total_iters = sk_tiles * p->num_k_blocks;
  p->sk_iters_per_unit = (p->sk_total_iters + units - 1) / units;
  p->sk_flag_bytes = sk_flag_bytes(units, p->ctas);
  return sk_bytes(units, p->ctas, p->block_n);
}

// Cheapest tile width for a persistent grid of `units` workers on tiles of `rows` x bn.  One tile of width bn costs
// (bn + 146) x `unit_cost` (fixed part: epilogue, pipeline refill, lower operand reuse of narrow tiles; measured on
// B200).  Without scratch the grid runs whole waves of tiles; with enough of it (ws_limit) and a last wave that
// would be mostly empty, the last waves are balanced by K ranges and only the total work counts, plus a hand-over.
// Widths are multiples of 32 down to 128.
static double tile_wave_cost(int64_t M, int64_t N, int64_t K, int rows, int64_t units, int bn_max, double unit_cost,
                             int64_t ws_limit, int* bn_out) {
  double best = -1.0;
  if (units < 1) units = 1;
  const int num_kb = (int)((K + kBK - 1) / kBK);
  for (int bn = bn_max; bn >= 128; bn -= 32) {
    const int64_t tiles = ((M + rows - 1) / rows) * ((N + bn - 1) / bn);
    double cost;
    if (sk_wanted(tiles, num_kb, (int)units, rows / kBM, bn, ws_limit))  // only the total work counts, plus a hand-over
      cost = ((double)tiles / (double)units * (bn + 146) + 60.0) * unit_cost;
    else
      cost = (double)((tiles + units - 1) / units) * (bn + 146) * unit_cost;
    if (best < 0 || cost < best) {
      best = cost;
      *bn_out = bn;
    }
  }
  return best;
}

// allow_y_tma: the output is plain bf16 rows (Y of the fused op, C of the plain GEMM) that a TMA store can write.
static int make_plan(int64_t M, int64_t N, int64_t K, int variant, int block_n, int stages, int group_m, int max_ctas,
                     int sm_count, int64_t ws_limit, Plan* p, int allow_y_tma = 1) {
  if (M < 0 || N <= 0 || K <= 0 || M > 0x7fffff00LL || N > 0x3fffff00LL || K > 0x7fffff00LL)
    return fail(MAGI_SWIGLU_ERR_SHAPE, "shape out of range: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (N % 8 != 0 || K % 8 != 0)
    return fail(MAGI_SWIGLU_ERR_SHAPE, "N (%lld) and K (%lld) must be multiples of 8", (long long)N, (long long)K);
  if (variant == MAGI_SWIGLU_VARIANT_AUTO) {
    variant = (M <= 128) ? MAGI_SWIGLU_VARIANT_STREAM : MAGI_SWIGLU_VARIANT_MMA2;
    // A CTA pair works on 256 rows at a time; when the last 256-row unit is at most half full and there are few
    // units (M = 320 or 384, say), 128-row tiles on single CTAs waste less.  Measured on B200, a single-CTA tile of
    // width bn takes about 1.12 x the time of a pair tile of the same width (each CTA loads all of W's tile rows
    // instead of half), and bn <= 224 keeps three pipeline stages in shared memory.
    if (M > kBM && N >= 128 && block_n == 0 && sm_count >= 2 && (max_ctas <= 0 || max_ctas >= 2)) {
      const int avail = (max_ctas > 0 && max_ctas < sm_count) ? max_ctas : sm_count;
      int bn_pair = 0, bn_single = 0;
      const double cost_pair = tile_wave_cost(M, N, K, 2 * kBM, avail / 2, 256, 1.0, ws_limit, &bn_pair);
      const double cost_single = tile_wave_cost(M, N, K, kBM, avail, 224, 1.12, ws_limit, &bn_single);
      if (cost_single < 0.95 * cost_pair) {  // 5 %: the pair schedule is the better-measured default
        variant = MAGI_SWIGLU_VARIANT_MMA;
        block_n = bn_single;
      }
    }
  }
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
        // multiples of 32: both half tiles stay multiples of 16
        tile_wave_cost(M, N, K, 2 * kBM, ctas / 2, 256, 1.0, ws_limit, &block_n);
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
    const int forced = tuning().k_splits;
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
  p->split = (pair == 2 && p->n_mma == 2 && block_n % 32 == 0 && !tuning().no_split) ? 1 : 0;
  const int fit = (kSmemLimit - 1024) / (int)p->stage_bytes;
  int max_stages = fit < kMaxStages ? fit : kMaxStages;
  // Y through shared memory (tile schedules): the staging boxes take room behind the ring.  Taken when the ring keeps
  // its depth or at least four stages (measured: the scattered per-row stores cost more than a fifth stage gains).
  if (allow_y_tma && variant != MAGI_SWIGLU_VARIANT_STREAM && tuning().y_tma != 0) {
    const int fit_tma = (kSmemLimit - 1024 - kStagingBytes) / (int)p->stage_bytes;
    const int max_tma = fit_tma < kMaxStages ? fit_tma : kMaxStages;
    const int want = stages > 0 ? stages : max_stages;
    if (want <= max_tma || (stages == 0 && max_tma >= 4) || (tuning().y_tma == 1 && max_tma >= 2)) {
      p->y_tma = 1;
      max_stages = max_tma;
    }
  }
  if (stages == 0) stages = max_stages;
  if (stages < 2 || stages > max_stages)
    return fail(MAGI_SWIGLU_ERR_VARIANT, "stages=%d out of range [2,%d] for block_n=%d", stages, max_stages, block_n);
  p->stages = stages;
  int smem = stages * (int)p->stage_bytes + 1024 + (p->y_tma ? kStagingBytes : 0);
  p->smem_bytes = smem < kSmemFloor ? kSmemFloor : smem;
  p->num_m_tiles = (int)((M + kBM * pair - 1) / (kBM * pair));
  p->num_n_tiles = (int)((N + block_n - 1) / block_n);
  p->num_k_blocks = (int)((K + kBK - 1) / kBK);
  if ((int64_t)p->num_m_tiles * p->num_n_tiles > 0x7fffffffLL) return fail(MAGI_SWIGLU_ERR_SHAPE, "too many tiles");
  p->tiles = p->num_m_tiles * p->num_n_tiles;
  if (group_m <= 0) {
    // band height: keep one band of X rows (group_m units x K) around 32 MB so it stays in L2 while W streams by.
    // With a long K no band fits anyway and what is shared is the K block the CTAs of a wave are working on at the
    // same time, which wants the wave (74 pair tiles) close to square: at least 12 row units (measured: 4 -> 16 row
    // units at K = 28672 is +6 % through a higher clock under the power cap; the cycle count does not change).
    const int64_t unit_bytes = (int64_t)kBM * pair * K * 2;
    int64_t g = (32LL << 20) / (unit_bytes > 0 ? unit_bytes : 1);
    group_m = (int)(g < 12 ? 12 : (g > 64 ? 64 : g));
  }
  p->group_m = group_m;
  p->k_splits = k_splits;
  p->kb_per_split = (p->num_k_blocks + k_splits - 1) / k_splits;
  if (k_splits > 1) p->ws_bytes = splitk_bytes(p->tiles, k_splits, M, block_n);
  const int64_t items = (int64_t)p->tiles * pair * k_splits;
  p->grid = (items < ctas) ? (int)items : ctas;
  if (k_splits == 1) p->ws_bytes = sk_setup(p, p->grid / pair, ws_limit);
  else sk_setup(p, 0, 0);
  return 0;
}
}  // namespace magi
