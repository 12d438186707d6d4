/*
 * nova_b200.h — C ABI of libnova_b200, the B200 (sm_100a) execution backend for
 * the Nova compiler's matmul hot path.
 *
 * The Nova reference lowers nova.matmul / nova.linear / linalg.matmul /
 * linalg.batch_matmul (+ fused bias / ReLU / GELU consumers) to device code it
 * generates itself.  This library replaces everything below the point where
 * those ops reach code generation: a lowering pass rewrites each contraction
 * (and the row-wise ops next to it) into ONE call through this header.  The
 * reference already calls C runtimes from compiled IR in exactly this style —
 * plain `llvm.call`s to externs declared by getOrDeclareFunc
 * (lib/Transforms/FixGpuLaunch.cpp:17-33), with device pointers taken from
 * memref-descriptor field 1 (:245-246) and a stream handle (:99-104).
 *
 * Conventions
 *  - every function returns a nova_b200_status (0 == OK); nothing throws,
 *    aborts or exits;  nova_b200_last_error_string() describes the last failure
 *    on the calling thread.
 *  - pointers named *_dev are device pointers on the current CUDA device; the
 *    library never allocates user-visible outputs.
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream); calls
 *    only enqueue work, they do not synchronise (the *_host helpers do).
 *  - there is no CPU fallback: without a usable sm_100 device every compute
 *    entry point fails with NOVA_B200_ERR_NO_DEVICE.
 */
#ifndef NOVA_B200_H_
#define NOVA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* the library is built with -fvisibility=hidden; everything declared here is exported */
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define NOVA_B200_ABI_VERSION 1

typedef enum nova_b200_status {
  NOVA_B200_OK = 0,
  NOVA_B200_ERR_INVALID_ARG = 1,    /* null pointer, negative extent, bad enum                      */
  NOVA_B200_ERR_LAYOUT = 2,         /* stride / pitch combination the kernels cannot express        */
  NOVA_B200_ERR_UNSUPPORTED = 3,    /* valid request with no kernel (e.g. f64)                      */
  NOVA_B200_ERR_CUDA = 4,           /* a CUDA runtime / driver call failed                          */
  NOVA_B200_ERR_NO_DEVICE = 5,      /* no CUDA device, or not compute capability 10.x               */
  NOVA_B200_ERR_DEVICE_TIMEOUT = 6, /* a bounded in-kernel wait gave up (see nova_b200_device_status) */
  NOVA_B200_ERR_TOO_LARGE = 7       /* extent exceeds a documented limit                            */
} nova_b200_status;

typedef enum nova_b200_dtype {
  NOVA_B200_F32 = 0,
  NOVA_B200_F16 = 1,
  NOVA_B200_BF16 = 2,
  NOVA_B200_I16 = 3, /* index types for gather; i16 is zero-extended like the reference */
  NOVA_B200_I32 = 4,
  NOVA_B200_I64 = 5,
  NOVA_B200_I1 = 6   /* one byte per element, 0 or 1: results of nova.compare in the textual front-end only */
} nova_b200_dtype;

/* Fused consumers of the contraction, as classified by the reference's isEpilogue
 * (lib/Transforms/LLVMGPU/Config/NovaKernelConfig.cpp:1876-1895). */
typedef enum nova_b200_act {
  NOVA_B200_ACT_NONE = 0,
  NOVA_B200_ACT_RELU = 1,      /* nova.relu -> arith.maximumf(x, 0)  (NovaToLinalg.cpp:1053-1084)           */
  NOVA_B200_ACT_GELU_TANH = 2, /* nova.gelu, tanh form (NovaToLinalgGeneric.cpp:1277-1337)                 */
  NOVA_B200_ACT_GELU_TANH_GRAD = 3 /* contraction followed by nova.gelu_backward (NovaToLinalgGeneric.cpp:1339-1420):
                                    * C = (init + A.B) * gelu_tanh'(Z).  Z, the forward pre-activation, is read through
                                    * `residual` / `ldr` / `batch_stride_r` and is NOT added; init must then be ZERO,
                                    * BIAS_ROW or FROM_C.  Only nova_b200_gemm* accept it. */
} nova_b200_act;

/* What the accumulator starts from.  FuseMatmulBias (lib/Transforms/FuseMatmulBias.cpp:95-193)
 * turns `fill(0) + matmul + add` into a matmul whose outs IS the (broadcast) bias or a full
 * residual tensor; a matmul whose outs is a live tensor reads C itself
 * (readingExistingAccBuffer, NovaKernelConfig.cpp:386-397). */
typedef enum nova_b200_acc_init {
  NOVA_B200_INIT_ZERO = 0,
  NOVA_B200_INIT_BIAS_ROW = 1,      /* bias[N], broadcast along rows                         */
  NOVA_B200_INIT_RESIDUAL_FULL = 2, /* residual[batch, M, N] (own pitch and batch stride)     */
  NOVA_B200_INIT_FROM_C = 3,        /* C holds the initial accumulator and is overwritten     */
  NOVA_B200_INIT_BIAS_AND_RESIDUAL = 4, /* bias[N] + residual[batch, M, N]: the "out + x + b_down" generic after
                                        * the FFN-down contraction (docs/SelectLoweringStrategy_Report.md rows 15, 25) */
  NOVA_B200_INIT_LN_FOLD = 5           /* the contraction consumes a layer-normalised A without it ever being written:
                                        * C = act( rstd_i * (A.W' - mean_i * c_j) + d_j ), see nova_b200_ln_fold_prepare.
                                        * `bias` then points at fp32 {c[N], d[N]} and `residual` at fp32 {mean, rstd}[M]
                                        * (both from the library's own routines); batch must be 1 */
} nova_b200_acc_init;

typedef enum nova_b200_f32_mode {
  NOVA_B200_TF32X3 = 0, /* hi/lo split, three tensor-core products: rel. error ~1e-6 (default)            */
  NOVA_B200_TF32X1 = 1  /* single TF32 product, what the reference's own GPU path computes
                           (NVIDIATargetUtils.cpp:58-65)                                                  */
} nova_b200_f32_mode;

/* One (batched) contraction  C[b] = act( init[b] + op(A[b]) * op(B[b]) ).
 *
 * Replaces, per call: linalg.matmul / linalg.batch_matmul as emitted by NovaMatmulOpLowering
 * (include/Compiler/Translation/NovaToLinalg/NovaToLinalg.cpp:874-1050), the rank-2/3 forms of
 * NovaLinearOpLowering (NovaToLinalgGeneric.cpp:1623-1823) including its batch-shared weight
 * (batch_stride_b == 0, :1726-1753), linalg.matmul_transpose_a (NovaToLinalg.cpp:824-872, trans_a),
 * the bias-as-accumulator form of FuseMatmulBias and the trailing GELU / ReLU generic.
 *
 * Layout: all tensors row-major with unit inner stride; ld* are row pitches in ELEMENTS,
 * batch strides are in elements (0 = the same matrix for every batch).  With trans_a the buffer
 * holds A as [K, M] (lda >= M); with trans_b it holds B as [N, K] (ldb >= K).  Accumulation is
 * always fp32.  Ragged M/N/K need no padding of extents.
 *
 * Scratch: two kinds of call pass their operands through library-owned device scratch first (scratch_bytes > 0 in
 * nova_b200_gemm_plan): f32 operands in TF32X3 mode (hi/lo split), and 16-bit / TF32X1 operands whose base or row
 * pitch is not a multiple of 16 bytes, which no tensor map can describe: by default they are copied once per call
 * to an aligned pitch ("re-pitch", loader_a/b == 2; nova_b200_operand_prepare does that copy once for a constant
 * operand), or, with option "repitch" = 0, read in place by loader warps at a fraction of the rate (loader == 1, no
 * scratch).  Scratch is kept per (device, stream), so calls on different streams never share it; it grows on
 * demand with cudaMalloc (never synchronising, never freeing a buffer that enqueued work may still read), which is
 * refused while the stream is being captured: make one call of the same size, or nova_b200_reserve_scratch, before
 * capturing.  A captured graph stays valid until nova_b200_shutdown. */
typedef struct nova_b200_gemm_args {
  uint32_t struct_size; /* = sizeof(nova_b200_gemm_args), for ABI evolution */
  int32_t dtype_ab;     /* NOVA_B200_F32 / F16 / BF16: element type of A and B */
  int32_t dtype_c;      /* element type of C, bias and residual */
  int32_t trans_a;
  int32_t trans_b;
  int32_t act;          /* nova_b200_act */
  int32_t init;         /* nova_b200_acc_init */
  int32_t f32_mode;     /* nova_b200_f32_mode, used when dtype_ab == F32 */
  int64_t batch, M, N, K;
  const void* A;
  const void* B;
  void* C;
  const void* bias;     /* [N], dtype_c; used when init == BIAS_ROW */
  const void* residual; /* used when init == RESIDUAL_FULL */
  int64_t lda, ldb, ldc, ldr;
  int64_t batch_stride_a, batch_stride_b, batch_stride_c, batch_stride_r;
} nova_b200_gemm_args;

/* How a call will be executed; filled by nova_b200_gemm_plan without launching anything.  The plan is the one a
 * 148-SM B200 executes (no device is needed to ask for it). */
typedef struct nova_b200_gemm_plan_info {
  int32_t loader_a;     /* 0 = TMA; unaligned base or pitch: 2 = re-pitched into aligned scratch first, then TMA
                           (the default), 1 = predicated ld.global loader warps (NOVA_B200_REPITCH=0) */
  int32_t loader_b;
  int32_t store_c;      /* 0 = TMA stores of swizzled 32x128-byte boxes, 1 = element stores (unaligned C, or rows that end inside a 16-byte chunk) */
  int32_t block_m, block_n, block_k;
  int32_t stages;
  int32_t grid;         /* persistent CTAs launched */
  int64_t tiles;        /* output tiles over all batches */
  int64_t scratch_bytes;/* device scratch the call uses (hi/lo split of f32 operands, re-pitched copies), else 0 */
} nova_b200_gemm_plan_info;

/* Binds the calling thread's current device (or `device` >= 0) : checks compute capability 10.x,
 * resolves the tensor-map encoder, allocates the 4-byte device status word.  Idempotent.
 * Counterpart in the reference: none explicit — mgpuModuleLoad does this implicitly
 * (lib/Transforms/LLVMGPU/Passes.cpp:482-483). */
int32_t nova_b200_init(int32_t device);
/* Frees per-device state (scratch pool, status words).  Safe to call without init. */
int32_t nova_b200_shutdown(void);
const char* nova_b200_last_error_string(void);
int32_t nova_b200_abi_version(void);

/* Tuning switches, process-wide.  Each is seeded once from the environment variable NOVA_B200_<NAME> and can be
 * changed at run time (later calls see the new value; cached plans are dropped):
 *   "repitch" (1)  unaligned operands: 1 = copy to an aligned pitch in scratch and stream with TMA, 0 = loader warps
 *   "pair" (-1)    CTA-pair (cta_group::2) kernel: -1 = cost model, 0 = never, 1 = whenever legal
 *   "block_n" (0)  tile width: 0 = cost model, else 64 / 128 / 256
 *   "short_k" (1)  eight epilogue warps for K <= 256
 *   "group_m" (16) raster group height in row blocks
 *   "prefetch" (-1) L2 prefetch distance of the pair kernel in ring stages: -1 = planner, 0 = off
 *   "pdl" (1)      launch contractions with programmatic stream serialization (prologue overlaps the previous kernel's tail)
 *   "ring_rows" (1) the row kernels (layer_norm forward / backward, softmax, row statistics) in packed fp32 arithmetic,
 *                  rows of a few KB streamed through shared memory by bulk copies; 0 = their scalar-arithmetic
 *                  predecessors (register kernels only; for A/B runs and cross-checks); 2 = also the shared-memory-ring
 *                  form of the layer_norm backward kernel (slower than the default where measured)
 *   "ring_stages" / "ring_ctas" (0) ring depth and CTAs per SM of those kernels, 0 = built-in choice (tuning;
 *                  "ring_ctas" = 1 also selects the four-rows-per-trip form of the layer_norm backward kernel)
 *   "host_tiles" (0) nova_b200_gemm_host on one large product: 0 = tiles of about 2048 x 2048 released in a growing
 *                  square, -1 = row blocks only, rows * 100 + cols = that many row blocks and column slabs, + 10000 = slab
 *                  by slab instead of the growing square (tuning)
 *   "split_k" (-1) K split into ranges that run as one launch and are summed by a second kernel, for products whose
 *                  output tiles fill at most half of the SMs (or leave the last wave mostly empty while K is very
 *                  long) and for f32 products with K > 1024: -1 = planner, 0 = never, n >= 2 = n ranges.  A split product differs from
 *                  the unsplit one in the last bits (fp32 additions associate differently)
 *   "plan_cache" (1) reuse plans and tensor maps of repeated calls;  "debug" (0)
 * No counterpart in the reference (its schedule is fixed at compile time by lowering_config attributes,
 * lib/Transforms/LLVMGPU/Config/NovaKernelConfig.cpp:1487-1577). */
int32_t nova_b200_set_option(const char* name, int64_t value);
int32_t nova_b200_get_option(const char* name, int64_t* value_out);

/* An f32 matrix that several contractions read (a gradient that feeds both the input-gradient and the weight-gradient
 * product): splits it ONCE into the hi / lo halves of the 3xTF32 scheme, stream-ordered on `stream`, and remembers them.
 * Until the release, every nova_b200_gemm on this device whose A or B is exactly this matrix (same pointer, stored
 * rows, columns and pitch; not batched) uses the halves and skips its own split pass.  The caller promises that the
 * matrix does not change in between and that those contractions run on `stream` or after it.  No counterpart in the
 * reference (its f32 contractions are single-pass TF32, NVIDIATargetUtils.cpp:58-65). */
int32_t nova_b200_f32_presplit(const void* x_dev, int64_t rows, int64_t cols, int64_t ld, void* stream, void** handle_out);
/* Forgets the matrix and frees the halves in stream order (after the contractions enqueued so far on `stream`). */
int32_t nova_b200_f32_presplit_release(void* handle, void* stream);

/* Makes sure `stream` of the current device owns at least `bytes` of library scratch (see nova_b200_gemm_args), so
 * that later calls on it, e.g. under stream capture, need not allocate.  Counterpart in the reference: the
 * cudaMallocAsync calls its generated host code makes per launch (lib/Transforms/FixGpuLaunch.cpp:49-50). */
int32_t nova_b200_reserve_scratch(int64_t bytes, void* stream);

/* A constant operand (a weight) whose base or row pitch is not a multiple of 16 bytes, copied ONCE into
 * library-owned memory with an aligned pitch: pass the returned view to nova_b200_gemm as A or B and the call
 * streams it with TMA at the full rate without the per-call re-pitch copy.  `src_dev` is [batch, rows, cols]
 * with row pitch `ld` and batch stride `batch_stride` (elements; 0 = one matrix); rows/cols are those of the
 * STORED matrix (for B [K, N]: rows = K, cols = N).  The copy is enqueued on `stream`.  This is the compile-time
 * counterpart of the reference's per-tile PadOperands copy (lib/Transforms/LLVMGPU/Tiling/NovaGPUPadOperands.cpp:34-65):
 * done once for the operand instead of inside every workgroup tile, and only the pitch is padded, not the extents. */
typedef struct nova_b200_operand nova_b200_operand;
int32_t nova_b200_operand_prepare(const void* src_dev, int32_t dtype, int64_t batch, int64_t rows, int64_t cols, int64_t ld,
                                  int64_t batch_stride, void* stream, nova_b200_operand** out);
int32_t nova_b200_operand_view(const nova_b200_operand* op, const void** data_dev, int64_t* ld, int64_t* batch_stride);
void nova_b200_operand_free(nova_b200_operand* op);

/* The contraction; device pointers; enqueues on `stream`.  In a process that sees several devices, operands that
 * live on another device than the current one are refused (NOVA_B200_ERR_INVALID_ARG) before anything is launched. */
int32_t nova_b200_gemm(const nova_b200_gemm_args* args, void* stream);
/* Validation + kernel selection only (no launch); usable without a GPU. */
int32_t nova_b200_gemm_plan(const nova_b200_gemm_args* args, nova_b200_gemm_plan_info* out);
/* nova_b200_gemm with every field passed as a scalar: the form compiled IR calls.  The lowering pass
 * (mlir/ConvertNovaContractionsToB200Calls.cpp) emits `func.call @nova_b200_gemm_flat(...)` with the operands'
 * aligned pointers as i64 (memref.extract_aligned_pointer_as_index, the pointer FixGpuLaunch takes from descriptor
 * field 1: lib/Transforms/FixGpuLaunch.cpp:245-246) and the extents, pitches and enums as i64 / i32 constants; no
 * struct has to be laid out in IR and the element type does not appear in the callee's signature.  `stream` is the
 * cudaStream_t as an integer (0 = default stream).  Returns a nova_b200_status. */
int32_t nova_b200_gemm_flat(int64_t A, int64_t B, int64_t C, int64_t bias, int64_t residual, int64_t batch, int64_t M,
                            int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr,
                            int64_t batch_stride_a, int64_t batch_stride_b, int64_t batch_stride_c, int64_t batch_stride_r,
                            int32_t dtype_ab, int32_t dtype_c, int32_t trans_a, int32_t trans_b, int32_t act, int32_t init,
                            int32_t f32_mode, int64_t stream);
/* Same contraction with HOST pointers for A, B, C, bias, residual: stages them through
 * library-owned device buffers (H2D, kernel, D2H) and synchronises before returning.  This is the
 * form the reference's host harnesses use (driver.cpp:22-40: host descriptors in, result out). */
int32_t nova_b200_gemm_host(const nova_b200_gemm_args* args);

/* The f32 (NOVA_B200_TF32X3) contraction for callers that cannot allocate device memory.
 * No counterpart in the reference: its generated host code calls cudaMallocAsync freely
 * (lib/Transforms/FixGpuLaunch.cpp:49-50).
 *
 * nova_b200_gemm splits f32 operands into hi/lo halves in a scratch buffer it obtains with cudaMalloc,
 * and its per-device status word is allocated too.  Some callers must not allocate: a compiled graph
 * running inside a memory-planned region that already owns the whole device, a plug-in under a host
 * framework that forbids allocation on its streams, a latency-critical loop that may not take the
 * allocator's locks.  This entry point computes the same result (same kernels, same arguments, device
 * pointers for A, B, C, bias, residual) but keeps the scratch and the status word in ONE fixed array
 * inside the library image and calls no cudaMalloc / cudaFree / allocating routine.
 *
 *  - Limit: the split needs 8 bytes per element of A and of B (rows padded to a multiple of 4
 *    elements); the array holds 16 MiB of it (e.g. 1024x1024x1024, or batch 4 of 512^3).  Larger
 *    requests return NOVA_B200_ERR_TOO_LARGE; non-f32 or TF32X1 requests return
 *    NOVA_B200_ERR_UNSUPPORTED (with 16-byte-aligned operands they use no scratch in nova_b200_gemm).
 *  - Every GPU on which the library is loaded holds the 16 MiB + 256 B until the process exits.
 *  - The first call on each device resolves the array's device address and the tensor-map encoder
 *    (no allocation, but driver calls): make that first call outside any stream capture.
 *  - All calls on a device share the array, and it keeps the previous call's contents.  Each call
 *    clears the status word and rewrites every scratch byte it reads, so consecutive calls on one
 *    stream are safe; calls that overlap on the GPU (different streams, or this and another process
 *    thread) race on the scratch and give wrong results.
 *  - wait_code_out == NULL: the call only enqueues; a wait that gave up is then reported by the next
 *    nova_b200_device_status.  Otherwise the call clears the status word, synchronises `stream`, stores the
 *    device-side wait code (0 = every bounded wait completed) and returns
 *    NOVA_B200_ERR_DEVICE_TIMEOUT when it is non-zero. */
int32_t nova_b200_gemm_f32_static(const nova_b200_gemm_args* args, void* stream, uint32_t* wait_code_out);

/* Layer norm folded into the contraction that consumes it (the reference fuses LN-apply into the FFN-up
 * contraction's scf.forall as a prologue: isPrologue, lib/Transforms/LLVMGPU/Config/NovaKernelConfig.cpp:1898-1917;
 * docs/TileAndDistribute_Report.md:50-60).  With y = (x - mean) * rstd * gamma + beta (NovaLayerNormPattern,
 * NovaToLinalgGeneric.cpp:2103-2116):
 *     (y . W + b)_ij = rstd_i * ( (x . W')_ij - mean_i * c_j ) + d_j,
 *     W' = diag(gamma) . W (rounded to the operand dtype),  c_j = sum_k W'_kj,  d_j = sum_k beta_k W_kj + b_j,
 * so the tensor cores read x itself, y is never written to or read from HBM, and the normalisation costs two
 * fused multiply-adds per output element in the epilogue.
 *   nova_b200_ln_fold_prepare: once per (weight, gamma, beta, bias): writes W' [K, N] (pitch N, dtype) to wprime_dev and
 *     fp32 {c[N], d[N]} to cd_dev (2 * N floats).  bias_dev may be NULL.
 *   nova_b200_row_stats: per call, one read of x [rows, D]: fp32 {mean_i, rstd_i} (eps 1e-5, as the reference) to
 *     stats_dev (2 * rows floats).
 *   then nova_b200_gemm with A = x, B = W', init = NOVA_B200_INIT_LN_FOLD, bias = cd_dev, residual = stats_dev.
 * Rounding: the unfused order rounds y to the operand dtype before the contraction, this one rounds gamma * W
 * instead; the two results differ from each other by about sqrt(2) operand roundings (f16 ~3e-4, bf16 ~2.5e-3
 * relative Frobenius) while each is equally close to the exact value.  The identity loses digits when |mean| is
 * much larger than the row's standard deviation (the two terms cancel), as any E[x^2]-E[x]^2 style formula does. */
int32_t nova_b200_ln_fold_prepare(const void* w_dev, const void* gamma_dev, const void* beta_dev, const void* bias_dev,
                                  void* wprime_dev, float* cd_dev, int64_t K, int64_t N, int64_t ldw, int32_t dtype,
                                  void* stream);
int32_t nova_b200_row_stats(const void* x_dev, float* stats_dev, int64_t rows, int64_t D, int32_t dtype, void* stream);

/* y = act(x), n elements, standalone nova.gelu / nova.relu (NovaToLinalgGeneric.cpp:1277-1337,
 * NovaToLinalg.cpp:1053-1084) for graphs where the activation is not adjacent to a contraction. */
int32_t nova_b200_activation(const void* x_dev, void* y_dev, int64_t n, int32_t dtype, int32_t act, void* stream);

/* nova.layer_norm_backward over [rows, D] (NovaLayerNormBackwardPattern, NovaToLinalgGeneric.cpp:2128-2376;
 * operand order of NovaOps.td:1038-1049): grad_y, x [rows, D]; gamma [D]; mean_sum, rstd [rows] as the forward
 * (nova_b200_layer_norm) returned them -- mean_sum is the RAW row sum.  Writes dx [rows, D], dgamma [D], dbeta [D].
 * gy and x are read once and dx written once; the column sums use the library's per-device scratch.  Rows of more
 * than 2048 sixteen-byte vectors (2048 elements when a pointer or D is not 16-byte aligned) are refused. */
int32_t nova_b200_layer_norm_backward(const void* grad_y_dev, const void* x_dev, const void* gamma_dev,
                                      const void* mean_sum_dev, const void* rstd_dev, void* dx_dev, void* dgamma_dev,
                                      void* dbeta_dev, int64_t rows, int64_t D, int32_t dtype, void* stream);

/* y = grad_out * gelu_tanh'(x), n elements: standalone nova.gelu_backward (NovaToLinalgGeneric.cpp:1339-1420;
 * ltest/_gelu.mlir, ltest/test.mlir:41). */
int32_t nova_b200_gelu_backward(const void* grad_out_dev, const void* x_dev, void* y_dev, int64_t n, int32_t dtype,
                                void* stream);

/* out[r, c] = a[r, c] + b[c]  (b_is_full == 0)  or  a[r, c] + b[r, c]: nova.add with a row-broadcast
 * operand (NovaToLinalg.cpp:115-194; the `[1,10]` bias of ltest/test_cpu.mlir). */
int32_t nova_b200_add_rowbcast(const void* a_dev, const void* b_dev, void* out_dev, int64_t rows, int64_t cols,
                               int32_t b_is_full, int32_t dtype, void* stream);

/* out = a (op) b, elementwise with numpy-style, right-aligned broadcasting: nova.add / nova.sub / nova.mul
 * (NovaToLinalgElementwiseConverter, NovaToLinalg.cpp:115-194; operand broadcast :154-168; result shape
 * lib/Dialect/nova/Broadcast.cpp:9-52).  `shape` is the OUTPUT shape (rank <= 6, contiguous row-major);
 * a_strides / b_strides are element strides per output dim, 0 where the operand has extent 1 and stretches.
 * Same-dtype float operands only (the reference's f16+bf16 -> f32 promotion is out of scope). */
typedef enum nova_b200_binary_op { NOVA_B200_BIN_ADD = 0, NOVA_B200_BIN_SUB = 1, NOVA_B200_BIN_MUL = 2 } nova_b200_binary_op;
int32_t nova_b200_binary(const void* a_dev, const void* b_dev, void* out_dev, int32_t rank, const int64_t* shape,
                         const int64_t* a_strides, const int64_t* b_strides, int32_t op, int32_t dtype, void* stream);

/* out[c] = sum over rows of x[r, c], fp32 accumulation: the bias gradient of nova.linear_backward, a column sum
 * over the flattened batch*M rows (NovaLinearBackwardPattern, NovaToLinalgGeneric.cpp:1970-1985).  x is
 * contiguous [rows, cols]; out holds cols elements of `dtype`.  Uses the per-device scratch for partial sums
 * (calls on different streams of one device must not overlap). */
int32_t nova_b200_column_sum(const void* x_dev, void* out_dev, int64_t rows, int64_t cols, int32_t dtype, void* stream);

/* nova.layer_norm over the last dim of x[rows, D] (NovaLayerNormPattern,
 * NovaToLinalgGeneric.cpp:1997-2126): y = (x - mean) * rsqrt(var + 1e-5) * gamma + beta with
 * var = E[x^2] - mean^2; also returns the RAW row sum (not the mean) and rstd, as the reference does
 * (:2121-2123).  Statistics are computed in fp32; mean_sum / rstd have dtype `dtype`. Either may be NULL. */
int32_t nova_b200_layer_norm(const void* x_dev, const void* gamma_dev, const void* beta_dev, void* y_dev,
                             void* mean_sum_dev, void* rstd_dev, int64_t rows, int64_t D, int32_t dtype,
                             void* stream);

/* nova.softmax along the last dim of x[rows, D] (NovaSoftmaxForwardPattern,
 * NovaToLinalgGeneric.cpp:1427-1534): e = exp(x - max), out = e * (1 / max(sum e, 1e-7)). */
int32_t nova_b200_softmax(const void* x_dev, void* y_dev, int64_t rows, int64_t D, int32_t dtype, void* stream);

/* nova.sce over the last dim of logits[rows, C] with one target class per row (NovaSceForwardLowering,
 * NovaToLinalgGeneric.cpp:801-1010): softmax_out = exp(x - max) / max(sum, 1e-7) and
 * loss_out[0] = mean over rows of log(max(sum, 1e-7)) - (x[target] - max).  Targets narrower than 32 bits are
 * zero-extended; a target outside [0, C) contributes x[target] = 0 and is counted in *bad_count_dev (int64, may be
 * NULL).  The row statistics pass through the library's per-device scratch. */
int32_t nova_b200_sce(const void* logits_dev, const void* targets_dev, void* softmax_out_dev, void* loss_out_dev,
                      int64_t rows, int64_t C, int32_t dtype, int32_t idx_dtype, int64_t* bad_count_dev, void* stream);

/* nova.sce_backward, class dim last (NovaSceBackwardLowering, NovaToLinalgGeneric.cpp:1012-1137):
 * grad[r, c] = (softmax[r, c] - (c == target[r])) * (1 / rows). */
int32_t nova_b200_sce_backward(const void* softmax_dev, const void* targets_dev, void* grad_dev, int64_t rows, int64_t C,
                               int32_t dtype, int32_t idx_dtype, void* stream);
/* The same followed by a multiplication with one scalar (the incoming gradient of the loss: `nova.mul %grad, %cst` after
 * nova.sce_backward in the reference's training graphs, ltest/test.mlir:43-45), in the same pass over the logits-sized
 * tensor: grad = (softmax - onehot) * ((1 / rows) * scale). */
int32_t nova_b200_sce_backward_scaled(const void* softmax_dev, const void* targets_dev, void* grad_dev, int64_t rows,
                                      int64_t C, int32_t dtype, int32_t idx_dtype, float scale, void* stream);

/* nova.scatter_add (NovaScatterAddOpLowering, NovaToLinalg.cpp:1086-1294) IN PLACE on the canonical view
 * inout[pre, axis_len, post], idx[n_idx], src[pre, n_idx, post]: inout[p, idx[i], q] += src[p, i, q] with atomic
 * adds (repeated indices accumulate in an unspecified order, as in the reference); indices outside [0, axis_len)
 * are skipped and counted in *bad_count_dev (int64, may be NULL).  The caller copies `input` first when the op's
 * input must survive. */
int32_t nova_b200_scatter_add(void* inout_dev, const void* idx_dev, const void* src_dev, int64_t pre, int64_t axis_len,
                              int64_t post, int64_t n_idx, int32_t idx_dtype, int32_t dtype, int64_t* bad_count_dev,
                              void* stream);

/* nova.gather (NovaGatherOpLowering, NovaToLinalgGeneric.cpp:2372-2472) on the canonical view
 * in[pre, axis_len, post], idx[n_idx] (or idx[pre, n_idx] when batched_idx != 0) -> out[pre, n_idx, post].
 * Bit-exact row copies.  Indices < 32 bits wide are zero-extended (:2446-2449).  Out-of-range
 * indices produce zero rows and are counted in *bad_count_dev (int64, may be NULL). */
int32_t nova_b200_gather(const void* in_dev, const void* idx_dev, void* out_dev, int64_t pre, int64_t axis_len,
                         int64_t post, int64_t n_idx, int32_t idx_dtype, int32_t batched_idx, int32_t elem_bytes,
                         int64_t* bad_count_dev, void* stream);

/* Multi-GPU, single large GEMM split by N-column slabs: after the ranks' output slabs have been all-gathered into
 * staging_dev = [world, rows, slab_pitch] (slab r in staging[r], its first width(r) columns valid), writes the
 * row-major [rows, cols] matrix to out_dev.  The slabs are the partition used throughout: whole `align`-column
 * units dealt out contiguously over the ranks, the first (units mod world) ranks one unit more, the ragged
 * remainder in the last non-empty slab.  16-byte copies when every boundary allows, element copies otherwise.
 * No counterpart in the reference, which has no multi-device code (its #nova.device attribute only separates
 * host from GPU: lib/Transforms/RemDevAttr.cpp:33-41). */
int32_t nova_b200_interleave_slabs(const void* staging_dev, void* out_dev, int64_t rows, int64_t cols, int32_t world,
                                   int64_t slab_pitch, int64_t align, int32_t elem_bytes, void* stream);

/* Multi-GPU, one process per GPU: the contraction whose epilogue ALSO stores every finished output box into the
 * matrices of up to 7 peer GPUs (plain 16-byte stores to peer-mapped addresses over NVLink; no TMA, no multicast, no
 * peer loads), so that a GEMM split by N-column slabs leaves the whole C on every GPU without a separate all-gather:
 * rank r passes C = its own full matrix + its slab's column offset and peer_c[i] = the same position in peer i's
 * matrix (same pitch and batch stride).  The transfer overlaps the contraction tile by tile; the peers may read
 * their matrices once every rank's kernel has completed and the ranks have met (a barrier or any collective enqueued
 * after the call on each rank's stream).  Needs C 16-byte aligned (base, pitch, batch stride) and N * element size a
 * multiple of 16.  No counterpart in the reference (single device).
 *
 * Peer-mapped addresses across processes: nova_b200_peer_buffer_alloc allocates device memory and fills a 64-byte
 * handle that another process of the same machine turns into an address in ITS address space with
 * nova_b200_peer_buffer_open (CUDA IPC; peer access is enabled on first use).  Close before the owner frees. */
int32_t nova_b200_gemm_push(const nova_b200_gemm_args* args, void* const* peer_c, int32_t n_peers, void* stream);
int32_t nova_b200_peer_buffer_alloc(int64_t bytes, void** ptr_out, unsigned char handle_out[64]);
int32_t nova_b200_peer_buffer_open(const unsigned char handle[64], void** ptr_out);
int32_t nova_b200_peer_buffer_close(void* opened_ptr);
int32_t nova_b200_peer_buffer_free(void* owned_ptr);

/* Reads (and clears) the device-side status words of the current device (the allocated one and, once
 * nova_b200_gemm_f32_static has run there, the one inside its static array): 0 when every bounded wait inside the
 * kernels completed; otherwise a code naming the wait that gave up.  Synchronises the device. */
int32_t nova_b200_device_status(uint32_t* code_out);

/* ---- memref-descriptor entry points ------------------------------------------------------------
 * The outer boundary of the reference is `_mlir_ciface_<fn>(MemRef* result, MemRef* in0, ...)` with
 * descriptors {allocated, aligned, offset, sizes[R], strides[R]} (driver.cpp:9-15,
 * robust_driver.cpp:9-23; expanded 7-scalar form in test/wrapper.c:15-24).  The lowering pass emits
 * `func.call`s with llvm.emit_c_interface to the functions below, so they take that struct as-is.
 * `aligned + offset` is the first element; strides are in elements; the inner stride must be 1
 * (or the two inner dims swapped, which selects trans_a / trans_b).  Buffers may be device or
 * host memory (detected per pointer); host buffers are staged like nova_b200_gemm_host. */
typedef struct nova_b200_memref2d {
  void* allocated;
  void* aligned;
  int64_t offset;
  int64_t sizes[2];
  int64_t strides[2];
} nova_b200_memref2d;

typedef struct nova_b200_memref3d {
  void* allocated;
  void* aligned;
  int64_t offset;
  int64_t sizes[3];
  int64_t strides[3];
} nova_b200_memref3d;

typedef struct nova_b200_memref4d {
  void* allocated;
  void* aligned;
  int64_t offset;
  int64_t sizes[4];
  int64_t strides[4];
} nova_b200_memref4d;

typedef struct nova_b200_memref1d {
  void* allocated;
  void* aligned;
  int64_t offset;
  int64_t sizes[1];
  int64_t strides[1];
} nova_b200_memref1d;

/* C = A * B (linalg.matmul, NovaToLinalg.cpp:1028-1048).  dtype is the element type of all three
 * (f32 / f16 / bf16 with fp32 accumulation).  Returns a status as well as writing C. */
int32_t _mlir_ciface_nova_b200_matmul(nova_b200_memref2d* C, nova_b200_memref2d* A, nova_b200_memref2d* B,
                                      int32_t dtype);
/* C[b] = A[b] * B[b] (linalg.batch_matmul, NovaToLinalg.cpp:1039-1043); ab_dtype inputs, c_dtype output. */
int32_t _mlir_ciface_nova_b200_batch_matmul(nova_b200_memref3d* C, nova_b200_memref3d* A, nova_b200_memref3d* B,
                                            int32_t ab_dtype, int32_t c_dtype);
/* Rank-4 batch_matmul: nova.matmul on rank > 3 operands collapses the batch dims to one, runs batch_matmul and
 * expands the result (NovaToLinalg.cpp:904-989); the collapse is metadata when the two batch dims of an operand
 * are contiguous with each other (else the outer dim is walked, one batched call per slice).  A batch dim of
 * size 1 in B broadcasts. */
int32_t _mlir_ciface_nova_b200_batch_matmul_4d(nova_b200_memref4d* C, nova_b200_memref4d* A, nova_b200_memref4d* B,
                                               int32_t ab_dtype, int32_t c_dtype);
/* Y = act(X * W + bias) (nova.linear rank 2, NovaToLinalgGeneric.cpp:1623-1823, + optional activation). */
int32_t _mlir_ciface_nova_b200_linear(nova_b200_memref2d* Y, nova_b200_memref2d* X, nova_b200_memref2d* W,
                                      nova_b200_memref1d* bias, int32_t dtype, int32_t act);

/* ---- textual front-end ---------------------------------------------------------------------------
 * Runs a function written in the restricted textual subset of the nova / linalg dialects that reaches
 * the contraction path: nova.matmul / linear / gelu / relu / add / softmax / layer_norm / gather / reshape /
 * transpose / cast / to_device, linalg.matmul / batch_matmul with linalg.fill + tensor.empty +
 * arith.constant, bufferization.to_tensor / materialize_in_destination (the forms of the reference's
 * ltest/ and test/pipeline-tests/ fixtures; tensor encodings such as #nova.device<"1"> are ignored, as
 * lib/Transforms/RemDevAttr.cpp:33-41 strips them).  It is the stand-in for the lowering pass, which needs
 * MLIR to build: shapes are inferred as the dialect does, `matmul + add + relu/gelu` chains are fused the
 * way FuseMatmulBias and the epilogue classification would fuse them, a transpose feeding a contraction
 * becomes trans_a / trans_b, and every step is one call of the entry points above.
 * Replaces, for such graphs, nova-opt --nova-gpu-optimized-pipeline + a driver (tools/nova-opt/nova-opt.cpp:75-144,
 * driver.cpp:17-40). */
typedef struct nova_b200_module nova_b200_module;

/* A contiguous row-major device buffer. */
typedef struct nova_b200_tensor {
  void* data;
  int32_t dtype; /* nova_b200_dtype */
  int32_t rank;  /* <= 6 */
  int64_t shape[6];
} nova_b200_tensor;

/* Parses, infers shapes, checks that every op is in the subset.  Needs no GPU. */
int32_t nova_b200_module_parse(const char* text, nova_b200_module** out);
void nova_b200_module_free(nova_b200_module* m);
/* Type of argument / result `index` of @func (data = NULL); *count receives how many there are.  `out` may be NULL. */
int32_t nova_b200_module_signature(const nova_b200_module* m, const char* func, int32_t index, int32_t is_result,
                                   nova_b200_tensor* out, int32_t* count);
/* Human-readable list of the calls a run will make, after fusion.  Needs no GPU. */
int32_t nova_b200_module_plan(const nova_b200_module* m, const char* func, char* buf, int64_t buflen);
/* Runs @func: `args` in signature order, `results` caller-provided buffers in return order.  Intermediates
 * are allocated with cudaMallocAsync on `stream` and freed when the call returns (stream-ordered).  The first run on a
 * device raises the release threshold of that device's default memory pool from 0 (if the application left it there)
 * so that the freed blocks are reused by the next run instead of going back to the driver at every synchronisation. */
int32_t nova_b200_module_run(const nova_b200_module* m, const char* func, const nova_b200_tensor* args, int32_t n_args,
                             nova_b200_tensor* results, int32_t n_results, void* stream);

/* The dynamic-argument form of the outer entry point: the reference renames a multi-argument `main` to
 * `_mlir_ciface_main_impl` and emits `_mlir_ciface_main(result*, void** args)` that unpacks the pointer array
 * (lib/Transforms/GenerateDynamicWrapper.cpp:34-95).  Here: `args[i]` points at the memref descriptor
 * {allocated, aligned, offset, sizes[R], strides[R]} of argument i of @func and `result` at the descriptor of its
 * result (several results: their descriptors one after the other, as MLIR packs a struct of memrefs); ranks and
 * element types come from the function's signature.  Descriptors must be row-major contiguous.  Buffers may be
 * host or device memory (detected per pointer; host buffers are staged).  Result buffers are caller-provided
 * (result->aligned != NULL): the library never allocates user-visible outputs.  Synchronises before returning. */
int32_t nova_b200_module_call_ciface(const nova_b200_module* m, const char* func, void* result, void** args);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* NOVA_B200_H_ */
