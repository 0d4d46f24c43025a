// C ABI of the B200 fused GEMM-SwiGLU library (include/magi_swiglu.h): argument checks, tensor-map encoding,
// kernel launches.  Device code lives in swiglu_kernels.cuh, schedule selection in swiglu_plan.hpp.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/magi_swiglu.h"
#include "swiglu_kernels.cuh"
#include "swiglu_plan.hpp"

namespace magi {

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
struct ScatterSet {  // what magi_swiglu_scatter_setup last wrote into g_scatter_maps[set] of a device
  int world = 0;
  int64_t rows = 0, n = 0;
};
static ScatterSet g_scatter[kMaxDevices][2];
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
// A 2-D map over a matrix stored with the reduction index as the row index ([K, cols], row stride ld elements):
// boxes of 64 columns x 64 K rows, i.e. one 128-byte swizzled line per K index (the MN-major operand tile).
static int encode_mn_major_map(EncodeTiledFn enc, const void* ptr, int64_t cols, int64_t K, int64_t ld, CUtensorMap* tm,
                               const char* what) {
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)K};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)kBK};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MAGI_SWIGLU_ERR_DRIVER, "tensor map for %s rejected by the driver (CUresult %d)", what, (int)r);
  return 0;
}

static int encode_maps(const void* x, const void* w, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw,
                       const Plan& p, CUtensorMap* tm_x, CUtensorMap* tm_w, int a_mn = 0, int b_mn = 0) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return fail(MAGI_SWIGLU_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  if (a_mn) {
    if (int rc = encode_mn_major_map(enc, x, M, K, ldx, tm_x, "A ([K, M])")) return rc;
  } else {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MAGI_SWIGLU_ERR_DRIVER, "tensor map for X rejected by the driver (CUresult %d)", (int)r);
  }
  if (b_mn) {
    if (int rc = encode_mn_major_map(enc, w, 2 * N, K, ldw, tm_w, "B ([K, N])")) return rc;
  } else {
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

// Y (or the plain GEMM's C) as a 3-D tensor [rows][halves][cols] for the epilogue's TMA stores: boxes of 32 rows x 32
// columns (64-byte rows, 64-byte swizzle).  `halves` is 1 for the fused op and 2 for the plain GEMM, whose two
// accumulator halves land `cols` columns apart; a box never spills from one half into the other.
static int encode_y_map(const void* y, int64_t rows, int64_t cols, int64_t halves, int64_t ldy, CUtensorMap* tm,
                        int box_cols = 32) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return fail(MAGI_SWIGLU_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)halves, (cuuint64_t)rows};
  // a dimension of extent 1 is never stepped along: give it the row pitch so the strides stay multiples of each other
  const cuuint64_t strides[2] = {(cuuint64_t)(halves > 1 ? cols : ldy) * 2, (cuuint64_t)ldy * 2};
  const cuuint32_t box[3] = {(cuuint32_t)box_cols, 1, 32};  // 64- or 128-byte rows, swizzled over the same width
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(y), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MAGI_SWIGLU_ERR_DRIVER, "tensor map for Y rejected by the driver (CUresult %d)", (int)r);
  return 0;
}

struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  cudaError_t set(int device) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    // Always set the device, even when it already is the current one: on a thread that has made no CUDA call yet
    // (an autograd worker, say) this is what binds the device's primary context, which the driver-level
    // tensor-map encoder needs.
    e = cudaSetDevice(device);
    changed = (e == cudaSuccess && prev != device);
    return e;
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
};

static int forward_impl(const void* x, const void* w, void* y, int64_t M, int64_t N, int64_t K, int64_t ldx,
                        int64_t ldw, int64_t ldy, int device, void* stream_v, int variant, int block_n, int stages,
                        int group_m, int max_ctas, void* workspace, int64_t workspace_bytes, int plain = 0,
                        const float* row_scale = nullptr, const float* out_scale = nullptr, const void* dy = nullptr,
                        int64_t lddy = 0, void* h = nullptr, int64_t ldh = 0, void* sf = nullptr, int64_t ld_sf = 0,
                        int sf_swizzled = 0, int a_mn = 0, int b_mn = 0, int64_t scatter_rows = 0, int scatter_set = 0) {
  g_err[0] = 0;
  if (M == 0 && N > 0 && K > 0) return 0;
  if (!x || !w || (!y && !scatter_rows)) return fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  // an operand stored [K, cols] has rows of `cols` elements; an nvfp4 output row is N/2 bytes
  if (ldx < (a_mn ? M : K) || ldw < (b_mn ? 2 * N : K) || ldy < (plain ? 2 * N : (sf ? N / 2 : N)))
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
  // bf16 rows a TMA store can write: Y of the fused op or C of the plain GEMM (not the quantised, pre-activation or
  // backward outputs, whose epilogues store directly)
  const int allow_y_tma = (!out_scale && !dy && !h) ? 1 : 0;
  int rc = make_plan(M, N, K, variant, block_n, stages, group_m, max_ctas, di->sm_count,
                     workspace ? workspace_bytes : 0, &p, allow_y_tma);
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

  CUtensorMap tm_x, tm_w, tm_y;
  memset(&tm_y, 0, sizeof(tm_y));
  if ((a_mn || b_mn) && (p.variant != MAGI_SWIGLU_VARIANT_MMA && p.variant != MAGI_SWIGLU_VARIANT_MMA2))
    return fail(MAGI_SWIGLU_ERR_VARIANT, "transposed operands need a tile schedule");
  // an MN-major B tile is made of blocks of 64 columns: every MMA must start on a block and cover whole blocks per CTA
  if (b_mn && (p.block_n % 64 != 0 || (p.n_mma == 2 && p.block_n % 128 != 0)))
    return fail(MAGI_SWIGLU_ERR_VARIANT, "a B operand stored [K, N] needs a tile width of 64, 128 or 256 (got %d)", p.block_n);
  rc = encode_maps(x, w, M, N, K, ldx, ldw, p, &tm_x, &tm_w, a_mn, b_mn);
  if (rc) return rc;
  // a Y layout the tensor-map encoder refuses simply keeps the direct stores (the staging boxes stay unused)
  int y_tma = 0;
  if (scatter_rows) {  // the destinations' maps are in constant memory already; only whole 32 x 32 boxes can leave
    if (!p.y_tma || p.ctas != 2 || p.block_n % 64 != 0 || N % 32 != 0)
      return fail(MAGI_SWIGLU_ERR_VARIANT, "this shape cannot be scattered (pair tiles with staged stores and whole 32-column boxes are needed; tile width %d)", p.block_n);
    y_tma = 1;
  } else {
    y_tma = (p.y_tma && encode_y_map(y, M, N, plain ? 2 : 1, ldy, &tm_y) == 0) ? 1 : 0;
  }
  g_err[0] = 0;

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
  a.wide_store = (((uintptr_t)y & 31u) == 0 && ldy % 16 == 0 && (!plain || N % 16 == 0)) ? 1 : 0;
  a.plain = plain;
  a.a_mn = a_mn;
  a.b_mn = b_mn;
  a.row_scale = row_scale;
  a.out_scale = out_scale;
  a.out_kind = out_scale ? (sf ? 2 : 1) : 0;
  a.sf = static_cast<uint8_t*>(sf);
  a.ld_sf = ld_sf;
  a.sf_swizzled = sf_swizzled;
  a.sf_ktiles = (int)((N / 16 + 3) / 4);
  a.dy = static_cast<const __nv_bfloat16*>(dy);
  a.lddy = lddy;
  a.h = static_cast<__nv_bfloat16*>(h);
  a.ldh = ldh;
  a.wide_h = (((uintptr_t)h & 31u) == 0 && ldh % 16 == 0 && N % 16 == 0) ? 1 : 0;
  a.k_splits = p.k_splits;
  a.kb_per_split = p.kb_per_split;
  a.ws = p.k_splits > 1 ? static_cast<float*>(workspace) : nullptr;
  a.y_tma = y_tma;
  a.scatter_rows = (int)scatter_rows;
  a.scatter_set = scatter_set;
  // 64-column boxes when both half-tiles are whole numbers of them and no box can straddle the end of a row block
  a.scatter_wide = (scatter_rows && p.split && p.block_n % 128 == 0 && N % 64 == 0 && tuning().scatter_wide != 0) ? 1 : 0;
  a.wait_limit = kWaitLimitCycles;
  auto fill_stream_k = [&]() {
    a.sk_first_tile = p.sk_first_tile;
    a.sk_iters_per_unit = p.sk_iters_per_unit;
    a.sk_total_iters = p.sk_total_iters;
    a.sk_min_kb = p.sk_min_kb;
    a.sk_flags = p.sk_total_iters > 0 ? static_cast<int*>(workspace) : nullptr;
    a.sk_partials = p.sk_total_iters > 0 ? reinterpret_cast<float*>(static_cast<char*>(workspace) + p.sk_flag_bytes) : nullptr;
  };
  fill_stream_k();
  // the hand-over flags of a stream-K launch start at zero (a memset node: nothing is allocated, nothing synchronises)
  auto clear_flags = [&]() -> cudaError_t {
    return p.sk_total_iters > 0 ? cudaMemsetAsync(workspace, 0, (size_t)p.sk_flag_bytes, stream) : cudaSuccess;
  };
  // Default L2 priorities (ncu, DRAM bytes per launch).  X: a band of X rows is re-read by every column tile ->
  // keep.  Y: written once -> evict first.  W: in the tile schedules a W tile is shared by all row units of the band
  // that run at the same time, and marking it evict-first makes late CTAs miss it (+25..70 % DRAM reads) -> normal;
  // in the STREAM schedule every W byte is read exactly once -> evict first.
  a.x_hint = 2;
  a.w_hint = (p.variant == MAGI_SWIGLU_VARIANT_STREAM) ? 1 : 0;
  a.y_hint = 1;
  const Tuning& tune = tuning();  // overrides for sweeps (environment at load, magi_swiglu_tuning afterwards)
  if (tune.hints[0] >= 0) a.x_hint = tune.hints[0];
  if (tune.hints[1] >= 0) a.w_hint = tune.hints[1];
  if (tune.hints[2] >= 0) a.y_hint = tune.hints[2];

  if (p.ctas == 1) {
    e = clear_flags();
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(stream-K flags)");
    swiglu_tc_kernel<1><<<p.grid, kThreads, p.smem_bytes, stream>>>(tm_x, tm_w, tm_y, a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, "launch of swiglu_tc_kernel<1>");
    if (p.k_splits > 1) {
      const long long work = (long long)p.num_n_tiles * ((M + 31) / 32) * 32 * (p.block_n / 8);
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
                             p.num_n_tiles, p.k_splits, row_scale);
      if (e != cudaSuccess) return fail_cuda(e, "launch of swiglu_splitk_reduce_kernel");
    }
    return 0;
  }
  if (pair_clusters <= 0) return fail(MAGI_SWIGLU_ERR_VARIANT, "this device cannot co-schedule 2-CTA clusters of the pair kernel");
  int grid = p.grid;
  if (grid > 2 * pair_clusters) {  // persistent: never more pairs than fit at once
    grid = 2 * pair_clusters;
    sk_setup(&p, grid / 2, workspace ? workspace_bytes : 0);  // the K ranges are cut for the workers that really run
    fill_stream_k();
  }
  e = clear_flags();
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(stream-K flags)");
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
  e = cudaLaunchKernelEx(&cfg, swiglu_tc_kernel<2>, tm_x, tm_w, tm_y, a);
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
  if (di->cc_major != 10 || di->cc_minor != 0)  // before the symbol look-up, which has no image on other GPUs
    return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is sm_%d%d; this library runs on sm_100 (B200) only", device,
                      di->cc_major, di->cc_minor);
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

int magi_swiglu_row_rms_f32(const void* x, float* out, int64_t M, int64_t K, int64_t ldx, float eps, int device,
                            void* cuda_stream) {
  magi::g_err[0] = 0;
  if (M == 0 && K > 0) return 0;
  if (!x || !out) return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  if (M < 0 || K <= 0 || K % 8 != 0 || M > 0x7fffff00LL || K > 0x7fffff00LL || ldx < K || ldx % 8 != 0)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "bad shape M=%lld K=%lld ldx=%lld (K and ldx multiples of 8)", (long long)M,
                      (long long)K, (long long)ldx);
  if (((uintptr_t)x & 15u) || ((uintptr_t)out & 3u)) return magi::fail(MAGI_SWIGLU_ERR_ALIGN, "x must be 16-byte aligned");
  const magi::DeviceInfo* di = magi::device_info(device);
  if (!di) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  magi::DeviceGuard guard;
  cudaError_t e = guard.set(device);
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaSetDevice");
  const long long want = (M + 7) / 8;  // eight rows (warps) per block
  const int blocks = (int)(want < 32LL * di->sm_count ? want : 32LL * di->sm_count);
  magi::swiglu_row_rms_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(x), out, (int)M, (int)K, ldx, eps);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : magi::fail_cuda(e, "launch of swiglu_row_rms_kernel");
}

int magi_swiglu_forward_bf16_scaled(const void* x, const void* w_gate_up, void* y, const float* row_scale, int64_t M,
                                    int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int device,
                                    void* cuda_stream, void* workspace, int64_t workspace_bytes) {
  if (M > 0 && !row_scale) {
    magi::g_err[0] = 0;
    return magi::fail(MAGI_SWIGLU_ERR_NULL, "row_scale is null");
  }
  return magi::forward_impl(x, w_gate_up, y, M, N, K, ldx, ldw, ldy, device, cuda_stream, MAGI_SWIGLU_VARIANT_AUTO, 0, 0,
                            0, 0, workspace, workspace_bytes, 0, row_scale);
}

int magi_swiglu_forward_fp8_e4m3(const void* x, const void* w_gate_up, void* y_fp8, const float* scale, int64_t M,
                                 int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int device,
                                 void* cuda_stream) {
  magi::g_err[0] = 0;
  if (M > 0 && !scale) return magi::fail(MAGI_SWIGLU_ERR_NULL, "scale is null");
  if (N % 16 != 0 || ldy % 16 != 0)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "fp8 output needs N (%lld) and ldy (%lld) to be multiples of 16", (long long)N,
                      (long long)ldy);
  // the one-byte output row is addressed in the kernel; the bf16 checks of the common path see ldy in elements.
  // No scratch: the split-K reduce kernel writes bf16 only, so narrow problems run unsplit here.
  const int variant = MAGI_SWIGLU_VARIANT_AUTO;
  return magi::forward_impl(x, w_gate_up, y_fp8, M, N, K, ldx, ldw, ldy, device, cuda_stream, variant, 0, 0, 0, 0, nullptr,
                            0, 0, nullptr, scale);
}

int magi_swiglu_forward_nvfp4(const void* x, const void* w_gate_up, void* y_fp4, void* y_scale, const float* global_scale,
                              int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int64_t ld_scale,
                              int scale_layout, int device, void* cuda_stream) {
  magi::g_err[0] = 0;
  if (M > 0 && (!global_scale || !y_scale)) return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  if (N % 16 != 0 || ldy % 8 != 0 || ldy < N / 2)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE,
                      "nvfp4 output needs N (%lld) to be a multiple of 16 and ldy (%lld bytes) a multiple of 8 >= N/2",
                      (long long)N, (long long)ldy);
  if (scale_layout != MAGI_SWIGLU_SCALES_LINEAR && scale_layout != MAGI_SWIGLU_SCALES_SWIZZLED_128X4)
    return magi::fail(MAGI_SWIGLU_ERR_VARIANT, "unknown scale layout %d", scale_layout);
  if (scale_layout == MAGI_SWIGLU_SCALES_LINEAR && ld_scale < N / 16)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "ld_scale=%lld is smaller than N/16=%lld", (long long)ld_scale,
                      (long long)(N / 16));
  // No scratch: narrow problems run unsplit (the split-K reduce kernel writes bf16 only).
  return magi::forward_impl(x, w_gate_up, y_fp4, M, N, K, ldx, ldw, ldy, device, cuda_stream, MAGI_SWIGLU_VARIANT_AUTO, 0,
                            0, 0, 0, nullptr, 0, 0, nullptr, global_scale, nullptr, 0, nullptr, 0, y_scale, ld_scale,
                            scale_layout == MAGI_SWIGLU_SCALES_SWIZZLED_128X4);
}

int magi_swiglu_forward_bf16_preact(const void* x, const void* w_gate_up, void* y, void* h, int64_t M, int64_t N, int64_t K,
                                    int64_t ldx, int64_t ldw, int64_t ldy, int64_t ldh, int device, void* cuda_stream) {
  magi::g_err[0] = 0;
  if (M > 0 && !h) return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  if (ldh < 2 * N)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "row stride too small: ldh=%lld (2N=%lld)", (long long)ldh, (long long)(2 * N));
  if (ldh % 8 || ((uintptr_t)h & 15u))
    return magi::fail(MAGI_SWIGLU_ERR_ALIGN, "h must be 16-byte aligned with a row stride that is a multiple of 8");
  // no scratch: the split-K reduce kernel does not write H, so narrow problems run unsplit here
  return magi::forward_impl(x, w_gate_up, y, M, N, K, ldx, ldw, ldy, device, cuda_stream, MAGI_SWIGLU_VARIANT_AUTO, 0, 0, 0,
                            0, nullptr, 0, 0, nullptr, nullptr, nullptr, 0, h, ldh);
}

int magi_swiglu_backward_dh_bf16(const void* x, const void* w_gate_up, const void* dy, void* dh, int64_t M, int64_t N,
                                 int64_t K, int64_t ldx, int64_t ldw, int64_t lddy, int64_t lddh, int device,
                                 void* cuda_stream) {
  magi::g_err[0] = 0;
  if (M > 0 && !dy) return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  if (lddy < N || lddh < 2 * N)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "row strides too small: lddy=%lld (N=%lld) lddh=%lld (2N=%lld)",
                      (long long)lddy, (long long)N, (long long)lddh, (long long)(2 * N));
  if (lddy % 8 || ((uintptr_t)dy & 15u))
    return magi::fail(MAGI_SWIGLU_ERR_ALIGN, "dy must be 16-byte aligned with a row stride that is a multiple of 8");
  // `plain` makes the common checks see dH's width (2N); the backward epilogue takes precedence in the kernel.
  // No scratch is passed, so narrow problems run unsplit (the split-K reduce kernel has no backward epilogue).
  return magi::forward_impl(x, w_gate_up, dh, M, N, K, ldx, ldw, lddh, device, cuda_stream, MAGI_SWIGLU_VARIANT_AUTO, 0,
                            0, 0, 0, nullptr, 0, 1, nullptr, nullptr, dy, lddy);
}

int magi_swiglu_gemm_nt_bf16(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                      int64_t ldc, int device, void* cuda_stream) {
  magi::g_err[0] = 0;
  if (N <= 0 || N % 16 != 0)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "magi_swiglu_gemm_nt_bf16 needs N (%lld) to be a positive multiple of 16", (long long)N);
  // The tile kernels see B as a packed pair: rows [0, N/2) and rows [N/2, N) land in the two accumulator halves
  // and the plain epilogue writes them to output columns n and N/2 + n.  M <= 128 runs the one-CTA tile schedule
  // (the streaming schedule's split-K reduce applies the activation).
  const int variant = (M <= 128) ? MAGI_SWIGLU_VARIANT_MMA : MAGI_SWIGLU_VARIANT_MMA2;
  return magi::forward_impl(a, b, c, M, N / 2, K, lda, ldb, ldc, device, cuda_stream, variant, 0, 0, 0, 0, nullptr, 0, 1);
}

int magi_swiglu_scatter_setup(int device, int set, void* const* dst, int world, int64_t rows_per_owner, int64_t N,
                              int64_t ldc) {
  magi::g_err[0] = 0;
  if (set < 0 || set > 1) return magi::fail(MAGI_SWIGLU_ERR_VARIANT, "destination set must be 0 or 1 (got %d)", set);
  if (world < 1 || world > magi::kMaxScatterOwners)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "a scattered GEMM writes to 1..%d owners (got %d)", magi::kMaxScatterOwners, world);
  if (!dst) return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  if (rows_per_owner <= 0 || rows_per_owner % 32 != 0 || rows_per_owner > 0x7fffff00LL / world)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "rows per owner (%lld) must be a positive multiple of 32", (long long)rows_per_owner);
  if (N <= 0 || N % 64 != 0 || ldc < N || ldc % 8 != 0)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "a scattered GEMM needs N (%lld) to be a multiple of 64 and ldc (%lld) >= N, a multiple of 8",
                      (long long)N, (long long)ldc);
  const magi::DeviceInfo* di = magi::device_info(device);
  if (!di) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  if (di->cc_major != 10 || di->cc_minor != 0)
    return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not sm_100 (B200)", device);
  magi::DeviceGuard guard;
  cudaError_t e = guard.set(device);
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaSetDevice");
  CUtensorMap maps[magi::kMaxScatterOwners], wide[magi::kMaxScatterOwners];
  memset(maps, 0, sizeof(maps));
  memset(wide, 0, sizeof(wide));
  for (int o = 0; o < world; ++o) {
    if (!dst[o] || ((uintptr_t)dst[o] & 15u))
      return magi::fail(MAGI_SWIGLU_ERR_ALIGN, "destination %d must be a 16-byte aligned device pointer", o);
    int rc = magi::encode_y_map(dst[o], rows_per_owner, N / 2, 2, ldc, &maps[o]);
    if (rc == 0) rc = magi::encode_y_map(dst[o], rows_per_owner, N / 2, 2, ldc, &wide[o], 64);
    if (rc) return rc;
  }
  // plain synchronous copies into the module's constant memory: set-up time, not the data path
  e = cudaMemcpyToSymbol(magi::g_scatter_maps, maps, sizeof(maps), (size_t)set * sizeof(maps), cudaMemcpyHostToDevice);
  if (e == cudaSuccess)
    e = cudaMemcpyToSymbol(magi::g_scatter_maps_wide, wide, sizeof(wide), (size_t)set * sizeof(wide), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaMemcpyToSymbol(scatter maps)");
  std::lock_guard<std::mutex> lock(magi::g_dev_mutex);
  magi::ScatterSet& ss = magi::g_scatter[device][set];
  ss.world = world;
  ss.rows = rows_per_owner;
  ss.n = N;
  return 0;
}

int magi_swiglu_gemm_nt_bf16_scatter(const void* a, const void* b, int set, int64_t M, int64_t N, int64_t K, int64_t lda,
                                     int64_t ldb, int device, void* cuda_stream, void* workspace,
                                     int64_t workspace_bytes) {
  magi::g_err[0] = 0;
  if (set < 0 || set > 1) return magi::fail(MAGI_SWIGLU_ERR_VARIANT, "destination set must be 0 or 1 (got %d)", set);
  if (device < 0 || device >= magi::kMaxDevices) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  magi::ScatterSet ss;
  {
    std::lock_guard<std::mutex> lock(magi::g_dev_mutex);
    ss = magi::g_scatter[device][set];
  }
  if (ss.world == 0) return magi::fail(MAGI_SWIGLU_ERR_VARIANT, "destination set %d of device %d has not been set up", set, device);
  if (N != ss.n || M != ss.rows * ss.world)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "destination set %d was set up for C[%lld, %lld], not [%lld, %lld]", set,
                      (long long)(ss.rows * ss.world), (long long)ss.n, (long long)M, (long long)N);
  if (M <= 128) return magi::fail(MAGI_SWIGLU_ERR_VARIANT, "a scattered GEMM needs more than 128 rows (pair tiles)");
  const int block_n = (N / 2) % 256 == 0 ? 256 : ((N / 2) % 128 == 0 ? 128 : 64);
  return magi::forward_impl(a, b, nullptr, M, N / 2, K, lda, ldb, N, device, cuda_stream, MAGI_SWIGLU_VARIANT_MMA2, block_n,
                            0, 0, 0, workspace, workspace_bytes, 1, nullptr, nullptr, nullptr, 0, nullptr, 0, nullptr, 0, 0,
                            0, 0, ss.rows, set);
}

static int sum_slots_impl(const void* src, void* const* dst, int n_dst, int slots, int64_t slot_stride, int64_t n, int device,
                          void* cuda_stream) {
  magi::g_err[0] = 0;
  if (n_dst < 1 || n_dst > magi::kMaxScatterOwners)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "1..%d destinations (got %d)", magi::kMaxScatterOwners, n_dst);
  if (!src || !dst) return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  magi::SumDst sd;
  memset(&sd, 0, sizeof(sd));
  sd.n = n_dst;
  uintptr_t bits = (uintptr_t)src;
  for (int d = 0; d < n_dst; ++d) {
    if (!dst[d]) return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
    sd.p[d] = static_cast<__nv_bfloat16*>(dst[d]);
    bits |= (uintptr_t)dst[d];
  }
  if (n == 0) return 0;
  if (slots < 1 || slots > 64 || n < 0 || n % 8 != 0 || slot_stride < n || slot_stride % 8 != 0)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "bad slots=%d n=%lld slot_stride=%lld (n and the stride must be multiples of 8)", slots,
                      (long long)n, (long long)slot_stride);
  if (bits & 15u) return magi::fail(MAGI_SWIGLU_ERR_ALIGN, "pointers must be 16-byte aligned");
  const magi::DeviceInfo* di = magi::device_info(device);
  if (!di) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  magi::DeviceGuard guard;
  cudaError_t e = guard.set(device);
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaSetDevice");
  const long long want = (n / 8 + 255) / 256;
  const int blocks = (int)(want < 16LL * di->sm_count ? want : 16LL * di->sm_count);
  magi::swiglu_sum_slots_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const __nv_bfloat16*>(src), sd, slots, (long long)slot_stride, (long long)n);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : magi::fail_cuda(e, "launch of swiglu_sum_slots_kernel");
}

int magi_swiglu_sum_slots_bf16(const void* src, void* out, int slots, int64_t slot_stride, int64_t n, int device,
                               void* cuda_stream) {
  void* const one[1] = {out};
  if (!out) {
    magi::g_err[0] = 0;
    return magi::fail(MAGI_SWIGLU_ERR_NULL, "null pointer argument");
  }
  return sum_slots_impl(src, one, 1, slots, slot_stride, n, device, cuda_stream);
}

int magi_swiglu_sum_slots_bf16_bcast(const void* src, void* const* dst, int n_dst, int slots, int64_t slot_stride, int64_t n,
                                     int device, void* cuda_stream) {
  return sum_slots_impl(src, dst, n_dst, slots, slot_stride, n, device, cuda_stream);
}

// tile width an MN-major B tile allows (256 with two MMAs per step for pairs, 128, 64); 0 = let the planner choose
static int gemm_bf16_block_n(int64_t M, int64_t N, int b_layout, int variant, int device) {
  if (b_layout != 1) return 0;
  const int64_t half = N / 2;
  if (half < 128) return 64;
  if (variant == MAGI_SWIGLU_VARIANT_MMA) return 128;
  const magi::DeviceInfo* di = magi::device_info(device);
  const int64_t units = di ? di->sm_count / 2 : 74;
  const int64_t m_units = (M + 2 * magi::kBM - 1) / (2 * magi::kBM);
  const int64_t c256 = ((m_units * ((half + 255) / 256) + units - 1) / units) * (256 + 146);
  const int64_t c128 = ((m_units * ((half + 127) / 128) + units - 1) / units) * (128 + 146);
  return (c256 <= c128) ? 256 : 128;
}

int64_t magi_swiglu_gemm_bf16_workspace_bytes(int64_t M, int64_t N, int64_t K, int b_layout, int device) {
  magi::g_err[0] = 0;
  if (N <= 0 || N % 16 != 0) return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "N (%lld) must be a positive multiple of 16", (long long)N);
  const int variant = (M <= 128) ? MAGI_SWIGLU_VARIANT_MMA : MAGI_SWIGLU_VARIANT_MMA2;
  return magi_swiglu_workspace_bytes(M, N / 2, K, variant, gemm_bf16_block_n(M, N, b_layout, variant, device), 0, 0, 0, device, 0);
}

int magi_swiglu_gemm_bf16_ws(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                             int64_t ldc, int a_layout, int b_layout, int device, void* cuda_stream, void* workspace,
                             int64_t workspace_bytes) {
  magi::g_err[0] = 0;
  if (N <= 0 || N % 16 != 0)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "magi_swiglu_gemm_bf16 needs N (%lld) to be a positive multiple of 16", (long long)N);
  if ((a_layout != 0 && a_layout != 1) || (b_layout != 0 && b_layout != 1))
    return magi::fail(MAGI_SWIGLU_ERR_VARIANT, "operand layouts must be 0 (reduction index contiguous) or 1 (stored [K, rows])");
  if (a_layout == 1 && M % 8 != 0)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "an A operand stored [K, M] needs M (%lld) to be a multiple of 8", (long long)M);
  const int variant = (M <= 128) ? MAGI_SWIGLU_VARIANT_MMA : MAGI_SWIGLU_VARIANT_MMA2;
  return magi::forward_impl(a, b, c, M, N / 2, K, lda, ldb, ldc, device, cuda_stream, variant,
                            gemm_bf16_block_n(M, N, b_layout, variant, device), 0, 0, 0, workspace, workspace_bytes, 1, nullptr,
                            nullptr, nullptr, 0, nullptr, 0, nullptr, 0, 0, a_layout, b_layout);
}

int magi_swiglu_gemm_bf16(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                          int64_t ldc, int a_layout, int b_layout, int device, void* cuda_stream) {
  return magi_swiglu_gemm_bf16_ws(a, b, c, M, N, K, lda, ldb, ldc, a_layout, b_layout, device, cuda_stream, nullptr, 0);
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
                     int device, int sm_count, int32_t out[16]) {
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
  out[12] = p.y_tma;
  out[13] = p.tiles - p.sk_first_tile;
  out[14] = out[15] = 0;
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

int magi_swiglu_schedule(int64_t M, int64_t N, int64_t K, int variant, int block_n, int stages, int group_m, int max_ctas,
                         int sm_count, int64_t workspace_bytes, int unit, int32_t* out, int max_items) {
  magi::g_err[0] = 0;
  if (!out || max_items < 0) return magi::fail(MAGI_SWIGLU_ERR_NULL, "out is null");
  if (sm_count <= 0) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "sm_count must be positive");
  magi::Plan p;
  int rc = magi::make_plan(M, N, K, variant, block_n, stages, group_m, max_ctas, sm_count, workspace_bytes, &p);
  if (rc) return rc;
  if (p.variant == MAGI_SWIGLU_VARIANT_SIMT) return 0;
  magi::KArgs a;
  memset(&a, 0, sizeof(a));
  a.num_k_blocks = p.num_k_blocks;
  a.k_splits = p.k_splits;
  a.kb_per_split = p.kb_per_split;
  a.sk_first_tile = p.sk_first_tile;
  a.sk_iters_per_unit = p.sk_iters_per_unit;
  a.sk_total_iters = p.sk_total_iters;
  a.sk_min_kb = p.sk_min_kb;
  const int units = p.grid / p.ctas;
  if (unit < 0 || unit >= units) return 0;
  magi::WorkIter it(a, unit, units);
  magi::WorkItem w;
  int n = 0;
  while (it.next(w)) {
    if (n < max_items) {
      int32_t* o = out + 6 * n;
      o[0] = w.t, o[1] = w.kb0, o[2] = w.kb1, o[3] = w.sk_role, o[4] = w.sk_first_peer, o[5] = w.sk_peers;
    }
    ++n;
  }
  return n;
}

int magi_swiglu_tuning(int knob, int value) {
  magi::g_err[0] = 0;
  magi::Tuning& t = magi::tuning();
  int prev = 0;
  switch (knob) {
    case MAGI_SWIGLU_TUNE_K_SPLITS:
      prev = t.k_splits;
      t.k_splits = value > 0 ? value : 0;
      return prev;
    case MAGI_SWIGLU_TUNE_NO_SPLIT:
      prev = t.no_split;
      t.no_split = value != 0;
      return prev;
    case MAGI_SWIGLU_TUNE_Y_TMA:
      prev = t.y_tma;
      t.y_tma = value < 0 ? -1 : (value != 0);
      return prev;
    case MAGI_SWIGLU_TUNE_SCATTER_WIDE:
      prev = t.scatter_wide;
      t.scatter_wide = value != 0;
      return prev;
    case MAGI_SWIGLU_TUNE_STREAM_K:
      prev = t.stream_k;
      t.stream_k = value < 0 ? -1 : (value != 0);
      return prev;
    case MAGI_SWIGLU_TUNE_L2_HINTS: {
      prev = t.hints[0] < 0 ? -1 : t.hints[0] * 100 + t.hints[1] * 10 + t.hints[2];
      const int h[3] = {value / 100, (value / 10) % 10, value % 10};
      const bool ok = value >= 0 && h[0] <= 2 && h[1] <= 2 && h[2] <= 2;
      for (int i = 0; i < 3; ++i) t.hints[i] = ok ? h[i] : -1;
      return prev;
    }
    default:
      return magi::fail(MAGI_SWIGLU_ERR_VARIANT, "unknown tuning knob %d", knob);
  }
}

int magi_swiglu_watchdog_selftest(int device, void* cuda_stream, int64_t limit_cycles) {
  magi::g_err[0] = 0;
  if (limit_cycles < 1000 || limit_cycles > 2000000000LL)
    return magi::fail(MAGI_SWIGLU_ERR_SHAPE, "limit_cycles=%lld out of range [1000, 2e9]", (long long)limit_cycles);
  if (!magi::device_info(device)) return magi::fail(MAGI_SWIGLU_ERR_DEVICE, "device %d is not available", device);
  magi::DeviceGuard guard;
  cudaError_t e = guard.set(device);
  if (e != cudaSuccess) return magi::fail_cuda(e, "cudaSetDevice");
  magi::watchdog_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>((long long)limit_cycles);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : magi::fail_cuda(e, "launch of watchdog_selftest_kernel");
}

#ifdef MAGI_SWIGLU_TRACE
int magi_swiglu_trace(long long out[32]) {  // reads the trace and clears its accumulating slots
  cudaDeviceSynchronize();
  int rc = (int)cudaMemcpyFromSymbol(out, magi::g_trace, sizeof(long long) * 32);
  long long zero[32] = {0};
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
