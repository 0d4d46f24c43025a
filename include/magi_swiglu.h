/*
 * magi_swiglu.h — C ABI of the B200 (sm_100a) fused GEMM-SwiGLU library.
 *
 *     Y[M,N] = silu(X[M,K] · Wg[N,K]^T) * (X[M,K] · Wu[N,K]^T)
 *
 * with one packed weight W[2N,K] = [Wg ; Wu] (gate rows first), bf16 inputs and
 * output, fp32 accumulation, fp32 epilogue and a single rounding to bf16.
 *
 * Reference interface replaced by this ABI (paths inside MagiCompiler):
 *   - the body of a custom op registered through
 *     magi_compiler/_magi_register_custom_op.py:168-204 (the decorated Python
 *     function is what the dispatcher finally calls; here that body is one call
 *     of magi_swiglu_forward_bf16);
 *   - the arithmetic of TransformerMLP.forward's gate/up part,
 *     tests/model_definition.py:336-339, and FeedForward.forward,
 *     example/training/llama3.py:172-173;
 *   - the calling style follows magi_compiler/cuda/cudart.py:24-62 (a ctypes
 *     call into a shared library with plain pointers and sizes).
 *
 * All pointers are raw device pointers owned by the caller.  No entry point
 * allocates device memory, synchronises the device or reads device memory on
 * the host, except where stated (magi_swiglu_device_status).
 *
 * Return convention: 0 = ok; negative = argument rejected on the host, nothing
 * was launched; positive = a CUDA runtime/driver error code.  The text of the
 * last error of the calling thread is available from magi_swiglu_last_error().
 */
#ifndef MAGI_SWIGLU_H_
#define MAGI_SWIGLU_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MAGI_SWIGLU_ABI_VERSION 8

/* variant selector of magi_swiglu_forward_bf16 */
#define MAGI_SWIGLU_VARIANT_AUTO   0  /* M <= 128 -> STREAM, else MMA2           */
#define MAGI_SWIGLU_VARIANT_MMA    1  /* persistent tcgen05 tile kernel, 1 CTA per tile */
#define MAGI_SWIGLU_VARIANT_STREAM 2  /* weight-streaming schedule for small M   */
#define MAGI_SWIGLU_VARIANT_SIMT   3  /* plain CUDA-core kernel, validation only */
#define MAGI_SWIGLU_VARIANT_MMA2   4  /* MMA schedule on CTA pairs (tcgen05 cta_group::2, clusters of 2) */

/* host-side argument errors (negative return values) */
#define MAGI_SWIGLU_ERR_NULL       -1  /* null pointer                                */
#define MAGI_SWIGLU_ERR_SHAPE      -2  /* M/N/K/ld out of range or inconsistent       */
#define MAGI_SWIGLU_ERR_ALIGN      -3  /* pointer or stride not 16-byte aligned       */
#define MAGI_SWIGLU_ERR_VARIANT    -4  /* unknown variant, or variant cannot run shape */
#define MAGI_SWIGLU_ERR_DEVICE     -5  /* device is not compute capability 10.0       */
#define MAGI_SWIGLU_ERR_DRIVER     -6  /* tensor-map encoder unavailable / failed     */

/* ABI version of the loaded library (== MAGI_SWIGLU_ABI_VERSION).
 * Replaces: nothing in the reference; lets the Python host refuse a stale build. */
int magi_swiglu_version(void);

/* 1 iff `device` exists and is compute capability 10.0 (B200, sm_100a), else 0.
 * Replaces: the implicit "is CUDA available" assumption of the reference's
 * custom-op bodies (tests/api_tests/test_register_custom_op.py run on any device). */
int magi_swiglu_supported(int device);

/* The fused op.  x is [M,K] with row stride ldx, w_gate_up is [2N,K] with row
 * stride ldw (rows 0..N-1 = gate, N..2N-1 = up), y is [M,N] with row stride ldy;
 * strides are in elements.  Requirements: K % 8 == 0, N % 8 == 0,
 * ldx/ldw/ldy % 8 == 0, all three base pointers 16-byte aligned, M >= 0.
 * M == 0 is a successful no-op.  The kernel is enqueued on `cuda_stream`
 * (a cudaStream_t; NULL = legacy default stream) of `device` and the call
 * returns without waiting for it.
 * Replaces: gate = F.silu(gate_proj(x)); up = up_proj(x); gate * up
 * (tests/model_definition.py:337-339) on the packed weight. */
int magi_swiglu_forward_bf16(const void* x, const void* w_gate_up, void* y,
                             int64_t M, int64_t N, int64_t K,
                             int64_t ldx, int64_t ldw, int64_t ldy,
                             int device, void* cuda_stream, int variant);

/* Same as magi_swiglu_forward_bf16 with explicit schedule knobs, for tuning
 * sweeps and tests: block_n = output columns per tile (multiple of 16, 16..256;
 * 0 = heuristic), stages = shared-memory pipeline depth (0 = as many as fit),
 * group_m = row-tiles per rasterisation band (0 = heuristic), max_ctas = cap on
 * the persistent grid (0 = one per SM).
 * Replaces: nothing in the reference (the reference has no kernel to tune). */
int magi_swiglu_forward_bf16_ex(const void* x, const void* w_gate_up, void* y,
                                int64_t M, int64_t N, int64_t K,
                                int64_t ldx, int64_t ldw, int64_t ldy,
                                int device, void* cuda_stream, int variant,
                                int block_n, int stages, int group_m, int max_ctas);

/* Same as magi_swiglu_forward_bf16_ex, with caller-owned scratch memory.  Narrow weights with M <= 128 (a
 * column shard of a decode GEMM) run faster when several CTAs share a slab of W and split K between them; their
 * fp32 partial sums live in `workspace` (device memory, 256-byte aligned, `workspace_bytes` long) and a second,
 * small kernel on the same stream adds them in a fixed order and writes Y.  magi_swiglu_workspace_bytes() tells
 * how much the best schedule wants; with less (or NULL) a schedule that fits is used.  The workspace needs no
 * initialisation and holds nothing between calls.  Two launches that may overlap on the GPU must not share a
 * workspace.  The library itself allocates nothing.
 * Replaces: nothing in the reference. */
int magi_swiglu_forward_bf16_ws(const void* x, const void* w_gate_up, void* y,
                                int64_t M, int64_t N, int64_t K,
                                int64_t ldx, int64_t ldw, int64_t ldy,
                                int device, void* cuda_stream, int variant,
                                int block_n, int stages, int group_m, int max_ctas,
                                void* workspace, int64_t workspace_bytes);

/* magi_swiglu_forward_bf16_ws without a workspace argument: the split-K partial sums go into an 8 MiB array that
 * is built into the library (a file-scope __device__ array; every GPU that loads the library holds it until the
 * process exits).  This entry point has no counterpart in the reference.
 * It is for callers that have no way to get device memory at the point of the call: a ctypes/C caller with no
 * allocator of its own, a serving process whose memory pool already owns the whole GPU, code running where a
 * cudaMalloc would be refused or would stall the device.  It calls no cudaMalloc/cudaFree and no allocating library
 * routine; the caller still passes x, w_gate_up and y.
 *  - The FIRST call on each device looks the array's device address up (cudaGetSymbolAddress); make that first call
 *    outside any stream capture.
 *  - A problem whose preferred schedule wants more than 8 MiB of scratch (magi_swiglu_workspace_bytes tells) is
 *    rejected with MAGI_SWIGLU_ERR_SHAPE and nothing is launched.  Problems that need no scratch run as usual.
 *  - All calls on a device share the one array.  It keeps the previous call's contents, which is harmless: every
 *    partial sum is written before it is read, nothing has to start at zero.  Calls that may overlap on the GPU
 *    (different streams) race on it: serialise them, or use magi_swiglu_forward_bf16_ws with separate workspaces. */
int magi_swiglu_forward_bf16_static(const void* x, const void* w_gate_up, void* y,
                                    int64_t M, int64_t N, int64_t K,
                                    int64_t ldx, int64_t ldw, int64_t ldy,
                                    int device, void* cuda_stream);

/* Row scales of an RMSNorm: out[m] = rsqrt(mean_k x[m,k]^2 + eps) in fp32 (x bf16 [M,K], K % 8 == 0).
 * Replaces: the variance/rsqrt part of RMSNorm.forward, tests/model_definition.py:53-54. */
int magi_swiglu_row_rms_f32(const void* x, float* out, int64_t M, int64_t K, int64_t ldx, float eps,
                            int device, void* cuda_stream);

/* The fused op with a per-row scale applied to both accumulators before the activation:
 *   y[m, n] = silu(s_m · x_m·Wg[n]) * (s_m · x_m·Wu[n]),   s = row_scale [M] fp32.
 * With s from magi_swiglu_row_rms_f32 and the norm weight folded into W's columns this is RMSNorm followed by the
 * SwiGLU projection without the normalised activations ever being written.  Same requirements and workspace rules as
 * magi_swiglu_forward_bf16_ws (workspace may be NULL).
 * Replaces: x = self.post_attention_layernorm(x) feeding self.mlp(x), tests/model_definition.py:360-361, gate/up part. */
int magi_swiglu_forward_bf16_scaled(const void* x, const void* w_gate_up, void* y, const float* row_scale,
                                    int64_t M, int64_t N, int64_t K,
                                    int64_t ldx, int64_t ldw, int64_t ldy,
                                    int device, void* cuda_stream, void* workspace, int64_t workspace_bytes);

/* The fused op with a statically scaled fp8 (e4m3, saturating) output: y[m,n] = fp8(silu(g)*u / *scale), one byte per
 * element, row stride ldy in bytes.  `scale` points to ONE fp32 value in device memory (it is read by the kernel, not
 * by the host).  N % 16 == 0, ldy % 16 == 0; other requirements as magi_swiglu_forward_bf16.
 * Replaces: the merged gate/up linear followed by vLLM's silu_and_mul_quant(result, input, scale), the quantising
 * activation op the reference's de-functionalisation pass handles (passes/piecewise_graph/fix_functionalization.py:110-112). */
int magi_swiglu_forward_fp8_e4m3(const void* x, const void* w_gate_up, void* y_fp8, const float* scale,
                                 int64_t M, int64_t N, int64_t K,
                                 int64_t ldx, int64_t ldw, int64_t ldy,
                                 int device, void* cuda_stream);

/* Layouts of the nvfp4 scale factors. */
#define MAGI_SWIGLU_SCALES_LINEAR 0          /* scale of (row m, 16-column block b) at y_scale[m * ld_scale + b] */
#define MAGI_SWIGLU_SCALES_SWIZZLED_128X4 1  /* tiles of 128 rows x 4 blocks (512 bytes), tile (m/128, b/4) at
                                              * ((m/128) * ceil(N/64) + b/4) * 512, inside it row r = m % 128 at
                                              * (r % 32) * 16 + (r / 32) * 4 + b % 4: the layout block-scaled GEMMs
                                              * read; buffer of round_up(M,128) * round_up(N/16,4) bytes, padding
                                              * entries are not written */

/* The fused op with an nvfp4 output: blocks of 16 consecutive outputs share one e4m3 scale factor
 *   sf = e4m3(gs * max|y| / 6),   code = e2m1(y * gs / sf)   (all codes 0 when sf == 0),
 * gs = *global_scale (one fp32 value in device memory, read by the kernel; usually 448 * 6 / max|y| of a calibration
 * run), y = silu(g)*u taken from the fp32 accumulators.  y_fp4 is [M, N/2] bytes, two codes per byte with the even
 * column in the low nibble, row stride ldy BYTES (a multiple of 8); y_scale holds one byte per block in the chosen
 * layout.  N % 16 == 0; other requirements as magi_swiglu_forward_bf16.
 * Replaces: the merged gate/up linear followed by vLLM's silu_and_mul_nvfp4_quant(result, result_block_scale, input,
 * input_global_scale), which the reference's de-functionalisation pass handles
 * (passes/piecewise_graph/fix_functionalization.py:113-120). */
int magi_swiglu_forward_nvfp4(const void* x, const void* w_gate_up, void* y_fp4, void* y_scale,
                              const float* global_scale,
                              int64_t M, int64_t N, int64_t K,
                              int64_t ldx, int64_t ldw, int64_t ldy, int64_t ld_scale, int scale_layout,
                              int device, void* cuda_stream);

/* Plain bf16 GEMM on the same tile kernels: C[M,N] = A[M,K] · B[N,K]^T (both operands row-major with the reduction
 * dimension contiguous, i.e. y = F.linear(a, b)), fp32 accumulation, one rounding.  N % 16 == 0, K % 8 == 0, strides
 * multiples of 8, 16-byte aligned pointers.  Used for the row-parallel down projection of the MLP block.
 * Replaces: self.down_proj(...) of TransformerMLP.forward (tests/model_definition.py:339) and w2 of FeedForward
 * (example/training/llama3.py:169,173), which the reference runs through a library GEMM. */
int magi_swiglu_gemm_nt_bf16(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, int device, void* cuda_stream);

/* The row-parallel down projection with the reduction's first half fused into its epilogue: the plain GEMM above,
 * but block o of C's rows ([o * rows_per_owner, (o + 1) * rows_per_owner)) is written by the epilogue's TMA stores
 * straight into dst[o], a [rows_per_owner, N] bf16 matrix (row stride ldc) that may live in ANOTHER GPU's memory
 * mapped into this process (peer access, e.g. a symmetric-memory allocation).  With every GPU of a tensor-parallel
 * group pointing dst[o] at "its own slot in owner o's receive buffer", each owner ends up with one partial product
 * per GPU for its rows and finishes with magi_swiglu_sum_slots_bf16 - a reduce-scatter whose data movement is the
 * GEMM's own output stores, overlapped with the tensor work tile by tile, with no copy of C in between.
 *
 * magi_swiglu_scatter_setup encodes the destinations' tensor maps into one of two sets kept in the library's constant
 * memory for `device` (set-up time: it copies synchronously; do not call it while a scattered GEMM of that set may be
 * running).  world <= 8, rows_per_owner % 32 == 0, N % 64 == 0.  magi_swiglu_gemm_nt_bf16_scatter then runs
 * C = A[M,K] · B[N,K]^T with M == world * rows_per_owner and N as set up, M > 128.  The call orders nothing between
 * GPUs: the caller makes sure the destinations are free before the launch and that all writers have finished (a
 * barrier across the GPUs on the streams involved) before anyone reads them.  Scratch as in
 * magi_swiglu_forward_bf16_ws (optional).
 * Replaces: the all-reduce after fairscale's RowParallelLinear w2 (example/training/llama3.py:169,173); the reference
 * has no fused form of it. */
int magi_swiglu_scatter_setup(int device, int set, void* const* dst, int world, int64_t rows_per_owner, int64_t N,
                              int64_t ldc);
int magi_swiglu_gemm_nt_bf16_scatter(const void* a, const void* b, int set, int64_t M, int64_t N, int64_t K,
                                     int64_t lda, int64_t ldb, int device, void* cuda_stream, void* workspace,
                                     int64_t workspace_bytes);

/* out[i] = sum over s < slots of src[s * slot_stride + i], i < n: bf16 in, fp32 sums in slot order, one rounding to
 * bf16.  n % 8 == 0, slot_stride % 8 == 0, 16-byte aligned pointers.  The last step of the scattered down projection
 * (slot s = what GPU s wrote for this GPU's rows); HBM-bound, element-wise.  It has no counterpart in the reference
 * (NCCL's reduction kernel does this inside the all-reduce). */
int magi_swiglu_sum_slots_bf16(const void* src, void* out, int slots, int64_t slot_stride, int64_t n, int device,
                               void* cuda_stream);

/* The same sum stored to n_dst (<= 8) destinations at once: dst[d] is where this GPU's block of the result lives in
 * GPU d's copy of the full result (this GPU's own copy included; peers' memory mapped into this process).  With it the
 * scattered down projection ends as an ALL-reduce: every GPU sums its own rows and writes them into every GPU's
 * result with plain coalesced 16-byte stores over NVLink; a second barrier across the GPUs then makes the whole
 * result readable everywhere.  It has no counterpart in the reference (NCCL's all-gather phase does this). */
int magi_swiglu_sum_slots_bf16_bcast(const void* src, void* const* dst, int n_dst, int slots, int64_t slot_stride,
                                     int64_t n, int device, void* cuda_stream);

/* The same plain GEMM with either operand stored the other way round, C[M,N] = op(A) · op(B)^T in bf16:
 *   a_layout 0: A is [M, K] (row stride lda);  1: A is stored [K, M] (its transpose, row stride lda, M % 8 == 0);
 *   b_layout 0: B is [N, K] (row stride ldb);  1: B is stored [K, N] (row stride ldb).
 * With layout 1 the operand tile is MN-major in shared memory (tensor-map boxes of 64 columns x 64 reduction rows,
 * operand descriptors and the MMA's major bits say so); nothing is transposed in memory.  N % 16 == 0, K % 8 == 0
 * when K is a contiguous index, strides multiples of 8, 16-byte aligned pointers.
 * Used for the two gradient GEMMs of the backward: dX = dH · W (b_layout 1) and dW = dH^T · X (both 1).
 * Replaces: the matmuls PyTorch's autograd runs for the two projections of tests/model_definition.py:337-339. */
int magi_swiglu_gemm_bf16(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                          int64_t lda, int64_t ldb, int64_t ldc, int a_layout, int b_layout,
                          int device, void* cuda_stream);

/* The same GEMM with optional scratch (size from magi_swiglu_gemm_bf16_workspace_bytes; 0 = none wanted; caller-owned,
 * 256-byte aligned, no initialisation needed): with it the last waves of the tile schedule are balanced stream-K
 * fashion as in magi_swiglu_forward_bf16_ws where the last wave would be at most a quarter full (dW = dH^T · X of the
 * Llama shape: 896 tiles on 74 CTA pairs).  Results differ from the scratch-less call by fp32 summation order in the
 * tiles that were cut.
 * Replaces: the same library GEMMs as magi_swiglu_gemm_bf16. */
int magi_swiglu_gemm_bf16_ws(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K,
                             int64_t lda, int64_t ldb, int64_t ldc, int a_layout, int b_layout, int device,
                             void* cuda_stream, void* workspace, int64_t workspace_bytes);
int64_t magi_swiglu_gemm_bf16_workspace_bytes(int64_t M, int64_t N, int64_t K, int b_layout, int device);

/* Backward of the activation.  h is [M, 2N] = [G | U], the pre-activations X·Wg^T and X·Wu^T (bf16, row stride ldh),
 * dy is [M, N]; writes dh = [dG | dU] ([M, 2N], row stride lddh) with dG = dY*U*s*(1 + G*(1-s)), dU = dY*G*s,
 * s = sigmoid(G); fp32 arithmetic, one rounding.  The GEMMs around it (recomputing h, dX = dH·W, dW = dH^T·X) are
 * plain library GEMMs on the host side.  N % 8 == 0, strides % 8 == 0, 16-byte aligned pointers.
 * Replaces: the autograd of F.silu(gate_proj(x)) * up_proj(x) (tests/model_definition.py:337-339) that the
 * reference gets from PyTorch; wired up through the setup_context_fn/backward_fn arguments of
 * magi_compiler/_magi_register_custom_op.py:198-200. */
int magi_swiglu_backward_act_bf16(const void* h, const void* dy, void* dh,
                                  int64_t M, int64_t N, int64_t ldh, int64_t lddy, int64_t lddh,
                                  int device, void* cuda_stream);

/* The forward for training: as magi_swiglu_forward_bf16, and the same kernel also writes the pre-activations
 * h = [G | U] ([M, 2N] bf16, row stride ldh, each value rounded once from its fp32 accumulator), so that the backward
 * (magi_swiglu_backward_act_bf16 on h and dY) needs no recomputation.  Costs one extra write of M x 2N bf16.
 * Replaces: the tensors PyTorch's autograd saves for F.silu(gate_proj(x)) * up_proj(x)
 * (tests/model_definition.py:337-339): the outputs of the two projections. */
int magi_swiglu_forward_bf16_preact(const void* x, const void* w_gate_up, void* y, void* h,
                                    int64_t M, int64_t N, int64_t K,
                                    int64_t ldx, int64_t ldw, int64_t ldy, int64_t ldh,
                                    int device, void* cuda_stream);

/* The first half of the backward in ONE kernel: recomputes G = X·Wg^T and U = X·Wu^T on the tile kernels and, in the
 * epilogue, turns the fp32 accumulators and dY straight into dH = [dG | dU] (formulas as above) — the 2N-wide
 * pre-activations are never written to memory.  x [M,K], w_gate_up [2N,K], dy [M,N] (row stride lddy), dh [M,2N] (row
 * stride lddh); requirements as magi_swiglu_forward_bf16, plus lddy % 8 == 0 and a 16-byte aligned dy.
 * Replaces: the same autograd as magi_swiglu_backward_act_bf16, together with the recomputation in front of it. */
int magi_swiglu_backward_dh_bf16(const void* x, const void* w_gate_up, const void* dy, void* dh,
                                 int64_t M, int64_t N, int64_t K,
                                 int64_t ldx, int64_t ldw, int64_t lddy, int64_t lddh,
                                 int device, void* cuda_stream);

/* Scratch bytes the preferred schedule of magi_swiglu_forward_bf16_ws wants for this problem (0 = none needed;
 * negative = argument error).  Needs no GPU when sm_count > 0.
 * Replaces: nothing in the reference. */
int64_t magi_swiglu_workspace_bytes(int64_t M, int64_t N, int64_t K, int variant,
                                    int block_n, int stages, int group_m, int max_ctas,
                                    int device, int sm_count);

/* Describes the schedule magi_swiglu_forward_bf16_ws would use when given all the scratch it asks for, without
 * launching: out[0]=variant, out[1]=block_n, out[2]=stages, out[3]=grid CTAs,
 * out[4]=tiles, out[5]=dynamic shared memory bytes, out[6]=accumulator buffers,
 * out[7]=MMAs per K=16 step, out[8]=CTAs per tile (1 or 2), out[9]=row units per raster band,
 * out[10]=1 if the tile is released to the MMA issuer in two halves, out[11]=CTAs that split K for one tile,
 * out[12]=1 if Y leaves through shared memory and TMA stores (0 = direct stores), out[13]=number of trailing tiles
 * whose K-steps are dealt to the workers as equal ranges (stream-K; 0 = whole tiles only), out[14..15]=0 (reserved).
 * `sm_count` <= 0 means "query `device`".  Needs no GPU when sm_count > 0.
 * Replaces: nothing in the reference. */
int magi_swiglu_plan(int64_t M, int64_t N, int64_t K, int variant,
                     int block_n, int stages, int group_m, int max_ctas,
                     int device, int sm_count, int32_t out[16]);

/* Reads (and clears) the device-side watchdog word of `device`.  Every wait in
 * the kernels is bounded; a wait that expires records
 * out[0]=code (0 = none; 1 = X producer, 2 = mma issuer, 3 = epilogue, 4 = W producer, 7 = self-test),
 * out[1]=block index, out[2]=pipeline stage or accumulator buffer, out[3]=phase.
 * A kernel whose wait expired returns normally (tensor memory freed, context usable) but its output is
 * incomplete, and the host learns of it ONLY here: callers poll this at a point where they synchronise anyway.
 * This call SYNCHRONISES the device; it is for tests and debugging.
 * Replaces: nothing in the reference. */
int magi_swiglu_device_status(int device, int32_t out[4]);

/* The work items worker `unit` (a CTA, or a CTA pair) of the planned schedule walks through, in order, without
 * launching anything: up to max_items records of six ints {tile, first K-step, end K-step, role, first peer, peers}
 * are written to `out`, and the number of items the worker has is returned (negative = error).  role 0 = the whole
 * K range given, nothing to exchange; 1 = head piece of a stream-K tile: the worker owns the tile and adds the sums
 * that workers first_peer .. first_peer+peers-1 park in scratch; 2 = a later piece: the worker parks its sums.
 * `workspace_bytes` is the scratch the caller would pass (0 = none: whole tiles only).  Pure host arithmetic.
 * Replaces: nothing in the reference. */
int magi_swiglu_schedule(int64_t M, int64_t N, int64_t K, int variant, int block_n, int stages, int group_m, int max_ctas,
                         int sm_count, int64_t workspace_bytes, int unit, int32_t* out, int max_items);

/* Tuning aids for sweeps and tests (process-wide; not meant for production callers).  Sets knob `knob` to `value`
 * and returns the previous value (for K_SPLITS/NO_SPLIT/Y_TMA >= -1, for L2_HINTS -1 or xwy), or
 * MAGI_SWIGLU_ERR_VARIANT for an unknown knob.  Initial values come from the environment, read once when the first
 * plan is made: MAGI_SWIGLU_K_SPLITS, MAGI_SWIGLU_NO_SPLIT, MAGI_SWIGLU_Y_TMA, MAGI_SWIGLU_L2_HINTS, MAGI_SWIGLU_STREAM_K.
 *   K_SPLITS  z > 0: force z-way split-K in the STREAM schedule (0 = choose)
 *   NO_SPLIT  1: drain CTA-pair tiles in one piece instead of two separately released halves
 *   Y_TMA     0 / 1: force direct stores / shared memory + TMA stores for Y in the tile schedules (-1 = choose)
 *   STREAM_K  0 / 1: never / whenever possible, balance the last waves of the tile schedules by K ranges (-1 = choose)
 *   L2_HINTS  three decimal digits xwy, each 0 normal / 1 evict-first / 2 evict-last, for X tiles, W tiles and Y
 *             stores (-1 = defaults)
 *   SCATTER_WIDE 0 / 1: the scattered GEMM stores 32-column boxes always / 64-column boxes where the tile allows
 * Replaces: nothing in the reference. */
#define MAGI_SWIGLU_TUNE_K_SPLITS 0
#define MAGI_SWIGLU_TUNE_NO_SPLIT 1
#define MAGI_SWIGLU_TUNE_Y_TMA    2
#define MAGI_SWIGLU_TUNE_L2_HINTS 3
#define MAGI_SWIGLU_TUNE_STREAM_K 4
#define MAGI_SWIGLU_TUNE_SCATTER_WIDE 5
int magi_swiglu_tuning(int knob, int value);

/* Runs the kernels' bounded wait by itself: a one-block kernel whose thread 0 waits on an mbarrier that nothing
 * signals (no copy, no MMA in flight), gives up after `limit_cycles` SM cycles (1e3..2e9) and records
 * {code 7, block 0, index 42, phase 0} for magi_swiglu_device_status.  The kernel returns normally; nothing
 * faults.  For tests of the give-up / report / clear path.
 * Replaces: nothing in the reference. */
int magi_swiglu_watchdog_selftest(int device, void* cuda_stream, int64_t limit_cycles);

/* SM clock the most recent MMA/MMA2/STREAM kernel on `device` really ran at: out[0] = average MHz
 * (SM cycles / wall nanoseconds, both read inside the kernel by block 0), out[1] = that span in
 * microseconds.  Power capping moves the clock within a millisecond, which a sampling tool cannot see.
 * This call SYNCHRONISES the device; it is a measurement aid for the benchmark.
 * Replaces: nothing in the reference. */
int magi_swiglu_kernel_clock(int device, double out[2]);

/* Text of the last error returned to the calling thread ("" if none).
 * Replaces: the Python exception text a reference custom-op body would raise. */
const char* magi_swiglu_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* MAGI_SWIGLU_H_ */
