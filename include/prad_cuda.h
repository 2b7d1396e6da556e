/*
 * libprad_cuda -- C ABI of the B200 (sm_100a) backward-pass engine for
 * ParallelReverseAutoDiff (RMAD double / PRADLite float).
 *
 * The reference has no native ABI of its own: its seam is the managed
 * IOperation / IBatchOperation contract (src/RMAD/IOperation.cs:17-25,
 * src/RMAD/IBatchOperation.cs:11-19) plus the CudaBlas singleton lifecycle
 * (src/RMAD/CudaBlas.cs:104-160).  Every entry point below names the managed
 * member it stands in for; a C# operation class binds it with [DllImport].
 *
 * Conventions
 *  - every call returns a prad_status (0 = PRAD_OK); nothing throws or aborts;
 *    prad_last_error() returns the calling thread's last message;
 *  - matrices are dense row-major (the device form of the reference's jagged
 *    T[rows][cols]); a DeepMatrix is `depth` consecutive matrices;
 *  - device buffers are plain device pointers obtained from prad_alloc (or any
 *    other CUDA allocation of the same device); host spans say so in their name;
 *  - work is enqueued on the context's stream; prad_sync waits for it; calls on
 *    one context must not overlap, different contexts may be used concurrently
 *    from different threads (the visitor calls Backward from thread-pool threads,
 *    src/RMAD/OperationNeuralNetworkVisitor.cs:303-306);
 *  - dtype selects the arithmetic and storage type: PRAD_F64 for RMAD/PRAD,
 *    PRAD_F32 for PRADLite.
 *  - there is no CPU fallback: without a usable CUDA device every call fails.
 */
#ifndef PRAD_CUDA_H_
#define PRAD_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t prad_status;
enum {
  PRAD_OK = 0,
  PRAD_ERR_INVALID = 1,          /* null pointer / bad enum / negative size            */
  PRAD_ERR_SHAPE = 2,            /* InvalidOperationException("... do not match ...")  */
  PRAD_ERR_NOT_INITIALIZED = 3,  /* CudaNotInitializedException                        */
  PRAD_ERR_CUDA = 4,             /* InvalidOperationException("CUBLAS failure.") class */
  PRAD_ERR_OOM = 5,
  PRAD_ERR_UNSUPPORTED = 6,
  PRAD_ERR_COMM = 7,             /* NCCL error                                          */
  PRAD_ERR_TIMEOUT = 8           /* a bounded wait ran out (visitor TimeoutInMinutes)   */
};

typedef enum { PRAD_F32 = 0, PRAD_F64 = 1 } prad_dtype;

/* activation selector for the fused and stand-alone kernels */
typedef enum {
  PRAD_ACT_NONE = 0,
  PRAD_ACT_LEAKY_RELU = 1, /* LeakyReLUOperation: backward reads the INPUT x           */
  PRAD_ACT_SIGMOID = 2,    /* SigmoidOperation:   backward reads the OUTPUT y          */
  PRAD_ACT_TANH = 3,       /* TanhOperation:      backward reads the OUTPUT y          */
  PRAD_ACT_GELU = 4,       /* GELUOperation:      backward reads the INPUT x           */
  PRAD_ACT_RELU = 5,       /* ReLUOperation (src/RMAD/ReLUOperation.cs:38-78): reads the INPUT x */
  PRAD_ACT_AMPLIFIED_SIGMOID = 6 /* AmplifiedSigmoidOperation.cs:45-83: reads the INPUT x      */
} prad_act;

typedef enum { PRAD_ADAM_RMAD = 0, PRAD_ADAM_PRAD = 1 } prad_adam_form;

typedef struct prad_ctx prad_ctx;

/* ---------------------------------------------------------------- lifecycle
 * prad_init / prad_shutdown replace CudaBlas.Instance.Initialize() / Dispose()
 * with DeviceId (src/RMAD/CudaBlas.cs:104,120-160). */
prad_status prad_init(int device, prad_ctx** out_ctx);
prad_status prad_shutdown(prad_ctx* ctx);
/* thread-local text of the last failure on this thread ("" if none) */
const char* prad_last_error(void);
/* library version string and the sm architecture it was built for */
const char* prad_version(void);
/* options:
 *  "gemm_f32" = "auto" | "simt" | "simt_fma" | "fp16x3" | "tf32b16" | "tf32x3" | "bf16x3";
 *  "gemm_f64" = "auto" | "simt" | "simt_fma" | "dmma"
 *    simt     : multiply and add rounded separately, k ascending -- bit-identical to the managed
 *               code's sequential `Output[i][j] += a*b` loop (the default for small products);
 *    simt_fma : same order with fused multiply-add (twice the rate, one rounding per step);
 *    fp16x3   : tcgen05 kernel; every block of 128 or 256 consecutive k of an operand row is scaled by
 *               its own power of two and split into two FP16 pieces (22 significant bits); three FP16
 *               products per term (h1*h0' + h0*h1' + h0*h0'); what "auto" uses for large products.
 *               Error of an output element: 2^-22 * sum_k |a_ik b_kj| like the TF32 pair, plus at most
 *               sqrt(K) * 2^-39 * (largest |a| times largest |b| of a block): an element more than ~8
 *               decades below the largest of its block keeps fewer than 22 bits.  Block scales are
 *               limited to 2^-126 .. 2^90: blocks whose largest magnitude is below 2^-112 lose bits and
 *               values above 2^106 (8e31) overflow.  Irrelevant for activations and gradients; a caller
 *               whose products pair a huge factor with a tiny one inside one block should use "tf32b16";
 *    tf32b16  : tcgen05 kernel, one TF32 product + two BF16 correction products;
 *    tf32x3   : tcgen05 kernel, three TF32 products per term (a_hi*b_hi + a_lo*b_hi + a_hi*b_lo);
 *    bf16x3   : tcgen05 kernel, six BF16 products of three-piece operands;
 *    dmma     : FP64 mma.sync kernel; all tensor-core kernels stay within the documented tolerance;
 *    auto     : tensor-core kernel for large products (>= 2^27 multiply-adds), "simt" otherwise;
 *  "tc_auto" = "fp16x3" | "tf32b16" | "tf32x3" | "bf16x3": the scheme "auto" uses for large products;
 *  "tc_chunk_k" = "128" | "256" | "512" | "1024": k summed inside the tensor core before the partial
 *    sum is added in FP32 with round-to-nearest (the tensor core truncates; default 256: rms error
 *    9e-7 of the result for any K; 512 is 4 % faster at 1.8e-6); for fp16x3 the block length of the
 *    scales is the chunk: 128 unless this option is set to 256 or more (then 256);
 *  "tc_split_k" = "on" | "off"; "tc_persistent" = "on" | "off" (tf32b16 on the one-tile-per-CTA kernel);
 *  "tc_reserve_sms" = n: SMs the persistent GEMM leaves idle (default 0);
 *  "tc_prefetch" = n (0..64, default 0): the product of packed operands asks L2 for the row operand's tile n k-blocks
 *    of 32 ahead of its load (measured: no gain on B200, the loads are not what the tensor pipe waits for);
 *  "tc_pair" = "1" (default) | "2" | "0": products of packed operands on pairs of CTAs (tcgen05 cta_group::2: two
 *    neighbouring SMs share a 256 x 256 tile, each holding half of the column operand) when k or N is at least 1024 ("1"),
 *    whatever k is ("2"), or always on one CTA per 128 x 256 tile ("0");
 *  "gemm_small" = "1" (default) | "0": strided batches of at least one product per SM whose outputs are at most
 *    64 x 64 (per-window attention products) run on one CTA per product sized to the output, instead of 64 x 64 tiles;
 *    the values are the same bit for bit;
 *  "tc_panel_n" = n: column tiles per panel of the persistent GEMM's tile walk (0 = automatic: two
 *    panels when the column operand exceeds 40 MB, so that a panel of it stays in L2);
 *  "tc_pipeline" = "16x4" | "32x2" | "8x8" (k-block floats x stages of the tf32x3 kernel) */
prad_status prad_set_option(prad_ctx* ctx, const char* key, const char* value);
/* wait for everything enqueued on the context (what the managed code gets for free
 * because GetAsArray2D blocks, src/RMAD/GpuMatrixMultiplyOperation.cs:199-201) */
prad_status prad_sync(prad_ctx* ctx);
/* number of kernels this context has launched since prad_init (introspection) */
prad_status prad_launch_count(prad_ctx* ctx, int64_t* out_count);
/* cudaStream_t of the context (so that a caller can order its own work against it) */
prad_status prad_stream(prad_ctx* ctx, void** out_stream);
/* makes the context enqueue on a caller-provided cudaStream_t (NULL restores its own) */
prad_status prad_use_stream(prad_ctx* ctx, void* stream);

/* Device and library facts for the managed side (the reference exposes none; CudaBlas only has
 * DeviceId, src/RMAD/CudaBlas.cs:104). */
typedef struct {
  int32_t device;                /* CUDA ordinal of the context                          */
  int32_t sm_count;
  int32_t cc_major, cc_minor;    /* compute capability (10.0 on B200)                    */
  int32_t l2_bytes;
  int32_t smem_per_block_optin;  /* largest dynamic shared memory a kernel may ask for   */
  int32_t sm_clock_khz, mem_clock_khz; /* nominal maxima as the runtime reports them     */
  uint64_t total_bytes, free_bytes;    /* device memory now                              */
  uint64_t scratch_bytes;        /* library scratch currently held by this context       */
  char name[64];
} prad_device_info_t;
prad_status prad_device_info(prad_ctx* ctx, prad_device_info_t* out);
/* Arithmetic rate of one pipe of this device, measured now with a register-resident kernel (eight
 * independent chains per thread, every SM full, best of three): pipe 0 = FP64 fused multiply-add,
 * 1 = FP64 tensor-core MMA (mma.sync m8n8k4), 2 = FP32 fused multiply-add; in TFLOP/s.  It is the
 * denominator for the SIMT and DMMA GEMM kernels (takes a few milliseconds). */
prad_status prad_measure_pipe_rate(prad_ctx* ctx, int pipe, double* out_tflops);
/* Self-test of the give-up path of the tensor-core kernels.  Every wait inside those kernels is bounded;
 * when one runs out the kernel raises a flag, frees what it holds and returns, later tensor-core
 * products and optimiser steps on the context become no-ops (weights, moments and gradients are left
 * untouched), and the next prad_sync / prad_download* / prad_get_timings returns PRAD_ERR_TIMEOUT and
 * clears the flag -- the counterpart of the visitor's wait with TimeoutInMinutes whose failure surfaces
 * as a queued exception (src/RMAD/OperationNeuralNetworkVisitor.cs:27,79-90,264-270).  This call
 * enqueues a one-CTA kernel that waits `polls` polls on a barrier nobody arrives on, i.e. it makes that
 * path run without any fault or hang; results computed between it and the next prad_sync are invalid,
 * as after a real give-up. */
prad_status prad_selftest_bounded_wait(prad_ctx* ctx, int polls);
/* CUDA-event timing of caller-chosen regions of the context's stream (the reference has no timers;
 * its only trace is Debug.WriteLine inside AdamOptimizer, src/RMAD/AdamOptimizer.cs:215-217).
 * prad_timing_begin(label) ... prad_timing_end() bracket whatever is enqueued in between; brackets do
 * not nest and cost two event records.  prad_get_timings waits for the stream, writes up to `capacity`
 * finished brackets in the order they were opened, stores their total number in *out_count, and forgets
 * them if they all fitted. */
typedef struct {
  char label[48];
  double milliseconds;  /* device time between the two events */
  int64_t launches;     /* kernels this library launched inside the bracket */
} prad_timing_t;
prad_status prad_timing_begin(prad_ctx* ctx, const char* label);
prad_status prad_timing_end(prad_ctx* ctx);
prad_status prad_get_timings(prad_ctx* ctx, prad_timing_t* out, int capacity, int* out_count);

/* ---------------------------------------------------------------- memory
 * Stand in for accelerator.Allocate2DDenseX / CopyFromCPU / GetAsArray2D
 * (src/RMAD/GpuMatrixMultiplyOperation.cs:190-201) and for the jagged<->flat
 * conversion (:210-271), but buffers persist across operations. */
prad_status prad_alloc(prad_ctx* ctx, size_t bytes, void** out_dptr);
prad_status prad_free(prad_ctx* ctx, void* dptr);
prad_status prad_zero(prad_ctx* ctx, void* dptr, size_t bytes);
prad_status prad_copy(prad_ctx* ctx, void* dst, const void* src, size_t bytes);
/* Strided device-to-device copy of `rows` rows of `width_bytes` (pitches in bytes).  It is what
 * MatrixConcatenateOperation / MatrixHorizontalConcatenateOperation do element by element
 * (src/RMAD/MatrixConcatenateOperation.cs:41-96): Forward copies each input into its column range
 * of the output, Backward copies each column range of dOutput back out. */
prad_status prad_copy_2d(prad_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                         size_t width_bytes, size_t rows);
prad_status prad_upload(prad_ctx* ctx, void* dst, const void* src_host, size_t bytes);
prad_status prad_download(prad_ctx* ctx, void* dst_host, const void* src, size_t bytes);
/* Overlapped upload: enqueues the copy on the context's separate copy stream, so it runs while
 * kernels enqueued earlier (or later) on the compute stream execute; prad_upload_join makes
 * the compute stream wait for every prefetch issued so far.  src_host must be page-locked
 * (prad_alloc_host) and stay untouched until the join; dst must not be in use by work that is
 * still running on the compute stream (use a second buffer). */
prad_status prad_upload_prefetch(prad_ctx* ctx, void* dst, const void* src_host, size_t bytes);
prad_status prad_upload_join(prad_ctx* ctx);
/* jagged form: `rows` host row pointers of row_bytes each <-> one dense device matrix */
prad_status prad_upload_rows(prad_ctx* ctx, void* dst, const void* const* src_rows, int rows,
                             size_t row_bytes);
prad_status prad_download_rows(prad_ctx* ctx, void* const* dst_rows, const void* src, int rows,
                               size_t row_bytes);
/* Many device tensors <-> ONE packed host block, in list order, with a single wait: what
 * ModelLayer.SaveWeightsAndMoments / LoadWeightsAndMoments need (src/RMAD/ModelLayer.cs:219-320; the
 * file holds all weights, then all first moments, then all second moments, each in element order, so the
 * caller lists the pointers in that order).  *_host arguments are host arrays of `count` entries. */
prad_status prad_download_many(prad_ctx* ctx, void* dst_host, const void* const* srcs_host, const size_t* bytes_host,
                               int count);
prad_status prad_upload_many(prad_ctx* ctx, void* const* dsts_host, const void* src_host, const size_t* bytes_host,
                             int count);
/* Intermediate slots: the device form of IOperationBase.Store(Guid) / Restore(Guid)
 * (src/RMAD/IOperationBase.cs:183-194, OperationBase.cs:251-258; e.g. MatrixMultiplyOperation.cs:31-42
 * keeps { input1, input2 } per id in IntermediateMatrixArrays; ComputationGraph.StoreOperationIntermediates
 * / RestoreOperationIntermediates, src/RMAD/ComputationGraph.cs:161-181, call it on every operation so
 * that several forward passes can be replayed backwards later).  A slot is a list of device buffers
 * under a 16-byte id:
 *   copy == 0  the slot keeps the POINTERS, as the managed code keeps references: the caller must not
 *              overwrite those buffers before the restore (it allocates fresh outputs per forward);
 *   copy != 0  the slot keeps device COPIES made on the context's stream (for callers that reuse their
 *              activation buffers from one forward pass to the next); restore returns the copies.
 * Storing under an id that exists replaces it (AddOrUpdate); restoring an unknown id is
 * PRAD_ERR_INVALID (the dictionary's KeyNotFoundException); prad_slot_drop frees a slot's copies. */
prad_status prad_slot_store(prad_ctx* ctx, const void* guid_16_bytes, const void* const* ptrs_host,
                            const size_t* bytes_host, int count, int copy);
prad_status prad_slot_restore(prad_ctx* ctx, const void* guid_16_bytes, void** out_ptrs_host, int count);
prad_status prad_slot_drop(prad_ctx* ctx, const void* guid_16_bytes);
prad_status prad_slot_count(prad_ctx* ctx, int* out_count);
/* pinned host staging memory for the two calls above and for *_host entry points */
prad_status prad_alloc_host(prad_ctx* ctx, size_t bytes, void** out_hptr);
prad_status prad_free_host(prad_ctx* ctx, void* hptr);

/* ---------------------------------------------------------------- GEMM
 * General row-major product C = alpha*op(A)*op(B) + beta*C over `batch` slices
 * (stride 0 = operand shared by all slices).  op(A) is MxK, op(B) is KxN.
 * Replaces the ILGPU tiled kernel (src/RMAD/GpuMatrixMultiplyOperation.cs:39-91)
 * and the cuBLAS Gemm call (src/RMAD/CudaBlas.cs:245,293). */
prad_status prad_gemm(prad_ctx* ctx, prad_dtype dt, int transA, int transB, int M, int N, int K,
                      double alpha, const void* A, int lda, const void* B, int ldb, double beta,
                      void* C, int ldc, int batch, int64_t strideA, int64_t strideB,
                      int64_t strideC);

/* ---------------------------------------------------------------- packed operands (float32, tensor cores)
 * The tensor-core path of the float GEMM multiplies operands that were first PACKED: cut into blocks of
 * 128 or 256 consecutive k, every block scaled by its own power of two and every value written as two
 * FP16 pieces (22 significant bits; see the option "fp16x3").  prad_gemm / prad_matmul_* pack their
 * operands into scratch on every call.  A caller that keeps a matrix for several products -- the
 * activation A_l of MatrixMultiplyOperation.Forward that its Backward multiplies again
 * (src/RMAD/MatrixMultiplyOperation.cs:50-126), the gradient dZ_l that feeds both dA and dW -- packs it
 * once into a prad_packed object, and can have an elementwise operation write the packed form directly:
 * LeakyReLU / Sigmoid / Tanh / GELU ... .Forward followed by the next MatrixMultiplyOperation, or an
 * activation's Backward (dx = dy (.) act'(saved), e.g. GELUOperation.cs:66-84) followed by the
 * MatrixMultiplyOperation.Backward below it, without the FP32 tensor in between ever being stored.
 * An object belongs to one R x C matrix shape and holds either or both orientations:
 *   PRAD_PACK_ROWS  the matrix as an operand with R rows and k = C  (A in A*B; dZ in dZ*W^T; W in dZ*W^T)
 *   PRAD_PACK_COLS  its transpose: C rows and k = R                 (A and dZ in A^T*dZ; W in A*W)
 * block_* = 0 picks the block length: 128, unless the "tc_chunk_k" option was set to 256 or more (then
 * 256).  With 128 one pass writes both forms out of a 128 x 128 tile; a 256 x 256 tile does not fit in
 * shared memory, so an object with two 256-long forms is packed in two passes.  Two operands of a
 * product need equal k and equal block length.
 * prad_gemm_packed: C (M x N, pitch ldc) = alpha * opA * opB^T + beta * C (+ bias row), opA M x k, opB N x k.
 * Accuracy is that of "fp16x3" with the range condition applying per block instead of per row. */
typedef struct prad_packed prad_packed;
enum { PRAD_PACK_ROWS = 1, PRAD_PACK_COLS = 2 };
prad_status prad_packed_create(prad_ctx* ctx, int rows, int cols, int forms, int block_rows_form, int block_cols_form,
                               prad_packed** out);
prad_status prad_packed_destroy(prad_packed* p);
/* rows, cols, forms and the block lengths of an object (any output may be NULL) */
prad_status prad_packed_shape(const prad_packed* p, int* rows, int* cols, int* forms, int* block_rows_form,
                              int* block_cols_form);
/* packs the dense float matrix x (pitch ld floats) */
prad_status prad_pack(prad_packed* p, const void* x, int64_t ld);
/* y = act(x) packed; y (dense FP32 copy of the result) may be NULL */
prad_status prad_act_forward_pack(prad_packed* p, prad_act act, const void* x, void* y, double act_alpha);
/* dx = dy (.) act'(saved) packed; dx (dense FP32 copy) may be NULL; PRAD_ACT_NONE packs dy itself */
prad_status prad_act_backward_pack(prad_packed* p, prad_act act, const void* saved, const void* dy, void* dx,
                                   double act_alpha);
/* The last layer's step: dx = [2 / (rows_total * cols) * (output - target)] (.) act'(saved) packed -- the
 * MeanSquaredErrorLossOperation.Backward (Loss/MeanSquaredErrorLossOperation.cs:65-84) and the output
 * activation's Backward in one pass, the loss gradient never stored. */
prad_status prad_mse_act_backward_pack(prad_packed* p, prad_act act, const void* saved, const void* output, const void* target,
                                       int64_t rows_total, void* dx, double act_alpha);
prad_status prad_gemm_packed(prad_ctx* ctx, const prad_packed* A, int form_a, const prad_packed* B, int form_b,
                             double alpha, double beta, void* C, int64_t ldc, const void* bias);

/* MatrixMultiplyOperation.Forward (src/RMAD/MatrixMultiplyOperation.cs:50-80) with the
 * optional fused tail  Z = A*B (+ bias row), Y = act(Z):  bias, Z_out and the activation
 * may each be absent (NULL / PRAD_ACT_NONE).  A is MxK, B is KxN. */
prad_status prad_matmul_forward(prad_ctx* ctx, prad_dtype dt, const void* A, const void* B,
                                void* Y, int M, int K, int N, const void* bias, void* Z_out,
                                prad_act act, double act_alpha);

/* MatrixMultiplyOperation.Backward (src/RMAD/MatrixMultiplyOperation.cs:83-126):
 *   dA = dC * B^T (MxK),  dB = A^T * dC (KxN).  Either output may be NULL.
 * accumulate_dB != 0 adds into dB (OperationBase.AccumulateGradient,
 * src/RMAD/OperationBase.cs:295-303) instead of overwriting it; dB_scale multiplies the
 * product first (1/count for the batch mean of OperationNeuralNetworkVisitor.cs:449-478).
 * If act_below != PRAD_ACT_NONE the dA result is multiplied in the epilogue by the
 * derivative of the activation that produced A (saved_below = that op's saved tensor),
 * i.e. the call also performs the next node's elementwise Backward. */
prad_status prad_matmul_backward(prad_ctx* ctx, prad_dtype dt, const void* A, const void* B,
                                 const void* dC, void* dA, void* dB, int M, int K, int N,
                                 int accumulate_dB, double dB_scale, prad_act act_below,
                                 const void* saved_below, double act_alpha);

/* The node of benchmark config 1: MatMul -> activation.  dPre = dOut (.) act'(saved),
 * dA = dPre*B^T, dB = A^T*dPre, all three returned (dPre must be non-NULL). */
prad_status prad_matmul_act_backward(prad_ctx* ctx, prad_dtype dt, const void* A, const void* B,
                                     const void* dOut, prad_act act, const void* saved,
                                     double act_alpha, void* dPre, void* dA, void* dB, int M,
                                     int K, int N);

/* Same node with HOST buffers (what a managed caller holding jagged Matrix data pays):
 * uploads A, B, dOut, saved; runs prad_matmul_act_backward; downloads dPre, dA, dB and
 * returns after the copies completed.  Host spans are dense row-major. */
prad_status prad_matmul_act_backward_host(prad_ctx* ctx, prad_dtype dt, const void* A_host,
                                          const void* B_host, const void* dOut_host,
                                          prad_act act, const void* saved_host, double act_alpha,
                                          void* dPre_host, void* dA_host, void* dB_host, int M,
                                          int K, int N);

/* BatchMatrixMultiplyOperation.Forward/Backward (src/RMAD/BatchMatrixMultiplyOperation.cs:
 * 51-94) over `depth` slices; b_shared != 0 is the (DeepMatrix, Matrix) overload.  With
 * b_shared the per-slice dB results are returned slice by slice (depth x K x N) exactly as
 * the reference does when dB_mean == NULL; if dB_mean != NULL the library instead writes the
 * visitor's combined result sum_d(dB_d)*(1/depth) (OperationNeuralNetworkVisitor.cs:
 * 449-478) there with one long-K product and dB may be NULL. */
prad_status prad_batch_matmul_forward(prad_ctx* ctx, prad_dtype dt, const void* A, const void* B,
                                      void* C, int depth, int M, int K, int N, int b_shared);
prad_status prad_batch_matmul_backward(prad_ctx* ctx, prad_dtype dt, const void* A,
                                       const void* B, const void* dC, void* dA, void* dB,
                                       void* dB_mean, int depth, int M, int K, int N,
                                       int b_shared);

/* (Gpu)MatrixMultiplyAndSumOperation (src/RMAD/GpuMatrixMultiplyAndSumOperation.cs:114-154,
 * src/RMAD/MatrixMultiplyAndSumOperation.cs:50-89): out[q] = sum_ij (A*B_q)_ij ; backward
 * dB_q = A^T*dOut[q], dA = sum_q B_q^T*dOut[q] (scalar products, not GEMMs).
 * A is RxC, B is P slices of CxN, out/dOut is 1xP, dA is NxC, dB is P slices of CxR. */
prad_status prad_matmul_and_sum_forward(prad_ctx* ctx, prad_dtype dt, const void* A,
                                        const void* B, void* out, int R, int C, int N, int P);
prad_status prad_matmul_and_sum_backward(prad_ctx* ctx, prad_dtype dt, const void* A,
                                         const void* B, const void* dOut, void* dA, void* dB,
                                         int R, int C, int N, int P);

/* ---------------------------------------------------------------- elementwise
 * LeakyReLUOperation.cs:54-93, SigmoidOperation.cs:46-84, TanhOperation.cs:42-78,
 * GELUOperation.cs:44-101 (and the lite float twins).  `saved` is the tensor the managed
 * op keeps for Backward: the input x for LeakyReLU/GELU, the output y for Sigmoid/Tanh. */
prad_status prad_act_forward(prad_ctx* ctx, prad_dtype dt, prad_act act, const void* x, void* y,
                             int64_t n, double act_alpha);
prad_status prad_act_backward(prad_ctx* ctx, prad_dtype dt, prad_act act, const void* saved,
                              const void* dy, void* dx, int64_t n, double act_alpha);
/* SwishOperation.cs:41-107: y = x * sigmoid(beta x); beta and dbeta are device scalars (the op's
 * [1 x 1] matrices); computed in double for either storage type, as the managed code does.
 * Backward as written there: dx = dy * s * ((1 + beta x)(1 - s)), dbeta = sum dy * (x s (1 - s) -
 * x^2 s^2); accumulate != 0 adds into dbeta. */
prad_status prad_swish_forward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* beta, void* y,
                               int64_t n);
prad_status prad_swish_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* beta,
                                const void* dy, void* dx, void* dbeta, int64_t n, int accumulate);
/* SwigLUOperation.cs:59-145: y = swish(x w_j + b_j) * (x v_j + c_j); w, v, b, c hold one value per
 * COLUMN (the op's [cols x 1] matrices, `cols` contiguous values each), beta is the constructor's
 * scalar (NeuralNetworkParameters.SwigLUBeta).  Backward as written there (der = swish + beta *
 * sigmoid * (1 - swish)); dw, dv, db, dc are `cols` long. */
prad_status prad_swiglu_forward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* w, const void* v,
                                const void* b, const void* c, double beta, void* y, int64_t rows, int cols);
prad_status prad_swiglu_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* w, const void* v,
                                 const void* b, const void* c, double beta, const void* dy, void* dx,
                                 void* dw, void* dv, void* db, void* dc, int64_t rows, int cols);
/* HadamardProductOperation.cs:50-118 */
prad_status prad_hadamard_forward(prad_ctx* ctx, prad_dtype dt, const void* a, const void* b,
                                  void* y, int64_t n);
prad_status prad_hadamard_backward(prad_ctx* ctx, prad_dtype dt, const void* a, const void* b,
                                   const void* dy, void* da, void* db, int64_t n);
/* The Backward of one LSTM cell (one time step) as ONE kernel: the step's loss gradient
 * (MeanSquaredErrorLossOperation.Backward, loss_scale = 2 / (rows_total * cols), target may be NULL), the
 * fan-in sum at h_t in list order (GradientUtils.AccumulateGradients, src/RMAD/GradientUtils.cs:22-42; the
 * loss gradient first, then the n_contrib <= 8 further gradients w.r.t. h_t), HadamardProductOperation
 * .Backward for h = o (.) tanh(c), TanhOperation.Backward, the fan-in sum at c_t (+ dc_next, may be NULL),
 * HadamardProductOperation.Backward for i (.) g and f (.) c_prev, and the four gate derivatives (Sigmoid for
 * i, f, o; Tanh for g; both read their outputs).  Host arrays: gates_ifgo_host = { i, f, g, o } outputs,
 * dpre_ifgo_host = the four gradients w.r.t. the gate pre-activations.  c_prev == NULL (first time step:
 * c_{-1} = 0) gives dpre_f = 0 and needs dc_prev == NULL; otherwise dc_prev receives dc_t (.) f_t, the next
 * call's dc_next.  Every element follows the rounding sequence of the separate operations, so the
 * results are bit-identical to calling them one by one; n = elements per tensor. */
prad_status prad_lstm_cell_backward(prad_ctx* ctx, prad_dtype dt, int64_t n, const void* h, const void* target,
                                    double loss_scale, const void* const* dh_contrib_host, int n_contrib,
                                    const void* dc_next, const void* const* gates_ifgo_host, const void* tanh_c,
                                    const void* c_prev, void* const* dpre_ifgo_host, void* dc_prev);
/* MatrixAddOperation.cs:29-68 / MatrixAddThreeOperation.cs:30-67 (c may be NULL).  Their
 * Backward returns copies of dOut; prad_copy (or simply aliasing dOut) provides that. */
prad_status prad_add_forward(prad_ctx* ctx, prad_dtype dt, const void* a, const void* b,
                             const void* c, void* y, int64_t n);
/* MatrixAddBroadcastingOperation.cs:32-69: y = x + bias row; backward: dBias[j] = sum_i
 * dOut[i][j] (the input gradient is dOut itself).  accumulate != 0 adds into dbias. */
prad_status prad_add_broadcast_forward(prad_ctx* ctx, prad_dtype dt, const void* x,
                                       const void* bias, void* y, int rows, int cols);
prad_status prad_add_broadcast_backward(prad_ctx* ctx, prad_dtype dt, const void* dy,
                                        void* dbias, int rows, int cols, int accumulate);
/* Allocation-free form of prad_add_broadcast_backward.  It has no counterpart in the
 * reference.  It exists for callers that must not allocate device memory at the moment they
 * need the bias gradient: a plug-in running inside a host application that has handed out
 * all device memory up front, a component whose rules of engagement ban allocator calls
 * after start-up, or a latency-critical loop where the device-wide synchronisation a
 * cudaMalloc implies is unacceptable.  It takes a cudaStream_t instead of a context, needs
 * no prad_init, and calls no allocator of any kind: its partial sums go to a fixed 4 MiB
 * array inside the library image (so every GPU that loads the library carries those 4 MiB
 * until the process ends).
 *  - limit: cols <= PRAD_STATIC_COLSUM_MAX_COLS (more is refused with PRAD_ERR_UNSUPPORTED);
 *    rows >= 1;
 *  - the device it works on is the calling thread's current device (cudaSetDevice);
 *  - the first call on each device looks up the array's device address; make that first
 *    call before starting any stream capture on that device;
 *  - all calls share the one array and leave their partial sums in it; each call overwrites
 *    every entry it later reads, so nothing has to be cleared, but two calls whose kernels
 *    may run at the same time on one GPU (different streams, different threads) race on
 *    it: serialise them. */
#define PRAD_STATIC_COLSUM_MAX_COLS 32768
prad_status prad_add_broadcast_backward_static(void* stream, prad_dtype dt, const void* dy,
                                               void* dbias, int rows, int cols, int accumulate);
/* MatrixMultiplyScalarOperation.cs:48-88 (forward and backward are the same scaling) */
prad_status prad_scale(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, int64_t n,
                       double s);
/* MatrixTransposeOperation.cs:28-64 over `depth` slices: y (cols x rows) = x^T */
prad_status prad_transpose(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, int rows,
                           int cols, int depth);

/* ---------------------------------------------------------------- row operations
 * SoftmaxOperation.cs:45-109 (rows = all rows of all slices) */
prad_status prad_softmax_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y,
                                 int64_t rows, int cols);
prad_status prad_softmax_backward(prad_ctx* ctx, prad_dtype dt, const void* y, const void* dy,
                                  void* dx, int64_t rows, int cols);
/* SineSoftmaxOperation.cs:47-77,155-176 (the attention weights of the GraphAttentionPaths networks):
 * y_j = e_j / (M + e_j) with e = exp(sin x) and M the row's sum of e; Backward as written there,
 * dx_j = dy_j * (M * e_j * cos x_j) / (M + e_j)^2, reads the INPUT x. */
prad_status prad_sine_softmax_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, int64_t rows, int cols);
prad_status prad_sine_softmax_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* dy, void* dx, int64_t rows,
                                       int cols);
/* LayerNormalizationOperation.cs:56-112: population sigma, eps (1e-9) added to sigma; the
 * backward is the reference's diagonal-only form.  mean/stdv are rows long (the op's state). */
prad_status prad_layernorm_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y,
                                   void* mean, void* stdv, int64_t rows, int cols);
prad_status prad_layernorm_backward(prad_ctx* ctx, prad_dtype dt, const void* x,
                                    const void* mean, const void* stdv, const void* dy, void* dx,
                                    int64_t rows, int cols);
/* MatrixSumOperation.cs:38-68 and MatrixAverageOperation.cs:38-67 (average != 0): y[i] = LINQ Sum /
 * Average of row i (`rows` values); backward: dx[i][j] = dy[i] (or dy[i] / cols). */
prad_status prad_row_sum_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, int64_t rows, int cols,
                                 int average);
prad_status prad_row_sum_backward(prad_ctx* ctx, prad_dtype dt, const void* dy, void* dx, int64_t rows, int cols,
                                  int average);
/* MatrixBroadcastOperation.cs:48-88: y[i][j] = x[i % in_rows][j % in_cols]; backward: every input
 * element collects its copies, rows outer, columns inner, added in the storage type. */
prad_status prad_broadcast_forward(prad_ctx* ctx, prad_dtype dt, const void* x, int in_rows, int in_cols, void* y,
                                   int out_rows, int out_cols);
prad_status prad_broadcast_backward(prad_ctx* ctx, prad_dtype dt, const void* dy, int out_rows, int out_cols,
                                    void* dx, int in_rows, int in_cols);
/* BatchNormalizationOperation.cs:52-158, as written: the whole matrix is one population, computed
 * in double.  Its Forward normalises with the SUM of the elements and the sum of squared deviations
 * from that sum (the local variables at that point, EPSILON 1e-6); its Backward reads the fields
 * mean = sum / n and var = that second sum / n.  `stats` is the op's state on the device:
 * 4 doubles { mean, var, sum, second sum }, written by forward, read by backward. */
prad_status prad_batchnorm_forward(prad_ctx* ctx, prad_dtype dt, const void* x, void* y, void* stats, int64_t rows,
                                   int cols);
prad_status prad_batchnorm_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* stats, const void* dy,
                                    void* dx, int64_t rows, int cols);
/* ScaleAndShiftOperation.cs:55-106: y[i][j] = x[i][j] * beta[i] + gamma[i] with one beta and
 * one gamma per ROW (the op's [rows x 1] matrices, passed as `rows` contiguous values).
 * Backward: dx = dy * beta[i]; dbeta[i] = sum_j dy*x; dgamma[i] = sum_j dy. */
prad_status prad_scale_shift_forward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* beta,
                                     const void* gamma, void* y, int64_t rows, int cols);
prad_status prad_scale_shift_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* beta,
                                      const void* dy, void* dx, void* dbeta, void* dgamma,
                                      int64_t rows, int cols);
/* RMSNormOperation.cs:47-118: rms = sqrt(sum_j x^2 / cols) per row, y = (x / rms) * g with g
 * [rows x cols]; the backward is the diagonal form written there,
 * dx = dy * (g/rms - x*g*x / (cols * rms^3)), dg = dy * x / rms. */
prad_status prad_rmsnorm_forward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* g, void* y,
                                 int64_t rows, int cols);
prad_status prad_rmsnorm_backward(prad_ctx* ctx, prad_dtype dt, const void* x, const void* g,
                                  const void* dy, void* dx, void* dg, int64_t rows, int cols);

/* ---------------------------------------------------------------- losses
 * Loss/MeanSquaredErrorLossOperation.cs:37-84 and
 * Loss/CategoricalCrossEntropyLossOperation.cs:37-87.  loss_out is one device scalar.
 * rows_total is the row count used in the normaliser: == rows for one matrix; the global row
 * count when the batch is sharded over several GPUs; 1 when every row is a separate sample
 * with its own loss operation (the Batch* graph spelling). */
prad_status prad_mse_forward(prad_ctx* ctx, prad_dtype dt, const void* out, const void* target,
                             void* loss_out, int64_t rows, int cols);
prad_status prad_mse_backward(prad_ctx* ctx, prad_dtype dt, const void* out, const void* target,
                              void* grad, int64_t rows, int cols, int64_t rows_total);
prad_status prad_cce_forward(prad_ctx* ctx, prad_dtype dt, const void* out, const void* target,
                             void* loss_out, int64_t rows, int cols);
prad_status prad_cce_backward(prad_ctx* ctx, prad_dtype dt, const void* out, const void* target,
                              void* grad, int64_t rows, int cols, int64_t rows_total);

/* ---------------------------------------------------------------- embedding
 * EmbeddingOperation.cs:49-86.  index_col holds the row indices as values of the matrix
 * type (column 0 of the input matrix, cast with (int)).  The backward adds duplicate
 * indices in input-row order, so the result is bit-identical to the sequential loop. */
prad_status prad_embedding_forward(prad_ctx* ctx, prad_dtype dt, const void* index_col,
                                   const void* W, void* out, int n, int vocab, int dim);
prad_status prad_embedding_backward(prad_ctx* ctx, prad_dtype dt, const void* index_col,
                                    const void* dOut, void* dW, int n, int vocab, int dim);

/* ---------------------------------------------------------------- gradient accumulation
 * prad_segmented_sum: GradientUtils.AccumulateGradients (src/RMAD/GradientUtils.cs:22-42),
 * out[i] = sum over the `count` sources in list order (deterministic; replaces the
 * visitor's lock + semaphore hand-off, OperationNeuralNetworkVisitor.cs:231-273).
 * srcs_host is a HOST array of `count` device pointers.
 * prad_accumulate: dest += src (OperationBase.cs:295-303).
 * prad_batch_mean: left-fold sum times 1/count (OperationNeuralNetworkVisitor.cs:449-478). */
prad_status prad_segmented_sum(prad_ctx* ctx, prad_dtype dt, const void* const* srcs_host,
                               int count, void* out, int64_t n);
prad_status prad_accumulate(prad_ctx* ctx, prad_dtype dt, void* dest, const void* src,
                            int64_t n);
prad_status prad_batch_mean(prad_ctx* ctx, prad_dtype dt, const void* const* srcs_host,
                            int count, void* out, int64_t n);

/* ---------------------------------------------------------------- clip + Adam
 * Multi-tensor calls: *_host arguments are HOST arrays of `count` device pointers / sizes
 * (one entry per model element, as GradientClipper.Clip / AdamOptimizer.Optimize walk the
 * layers' identifiers, src/RMAD/GradientClipper.cs:31-71, AdamOptimizer.cs:32-90).
 * prad_clip_reference: per-tensor z-score clamp + minimum threshold, in place
 *   (GradientClipper.cs:118-157,212-253).
 * prad_clip_global_norm: NOT in the reference; scale all tensors by max_norm/max(norm,
 *   max_norm); norm_out (host double, may be NULL) receives the norm before clipping.
 * prad_adam: form RMAD = AdamOptimizer.cs:195-239 (reciprocal bias correction),
 *   form PRAD = src/PRAD/AdamOptimizer.cs:79-103; `iteration` is NeuralNetworkParameters.
 *   AdamIteration (set by the caller); zero_grad != 0 also clears the gradients
 *   (GradientClearer.Clear, src/RMAD/GradientClearer.cs:21-86).
 * prad_clip_adam: the two steps in one pass over the gradients (clip_mode 0 = none,
 *   1 = reference, 2 = global norm). */
prad_status prad_clip_reference(prad_ctx* ctx, prad_dtype dt, void* const* grads_host,
                                const int64_t* sizes_host, int count, double clip_value,
                                double min_value);
prad_status prad_clip_global_norm(prad_ctx* ctx, prad_dtype dt, void* const* grads_host,
                                  const int64_t* sizes_host, int count, double max_norm,
                                  double* norm_out);
prad_status prad_adam(prad_ctx* ctx, prad_dtype dt, void* const* w_host, void* const* g_host,
                      void* const* m_host, void* const* v_host, const int64_t* sizes_host,
                      int count, double lr, double beta1, double beta2, double eps,
                      double iteration, prad_adam_form form, int zero_grad);
prad_status prad_clip_adam(prad_ctx* ctx, prad_dtype dt, void* const* w_host,
                           void* const* g_host, void* const* m_host, void* const* v_host,
                           const int64_t* sizes_host, int count, int clip_mode,
                           double clip_value, double min_value, double lr, double beta1,
                           double beta2, double eps, double iteration, prad_adam_form form,
                           int zero_grad);

/* ---------------------------------------------------------------- graph mode
 * Static-schedule replacement of OperationNeuralNetworkVisitor.Traverse
 * (src/RMAD/OperationNeuralNetworkVisitor.cs:143-337) and of the consumer counting of
 * OperationGraphVisitor (src/RMAD/OperationGraphVisitor.cs:124-162).  The managed side keeps
 * building the graph from JSON (ComputationGraph.ConstructFromArchitecture) and hands the
 * resulting DAG over: values (matrices) and nodes (operations on values, added in forward
 * order).  prad_graph_backward walks the nodes once in reverse order on the context's
 * stream -- no tasks, locks or semaphores:
 *   - the gradient of a value with several consumers is the sum of the consumers'
 *     contributions in the order the consumers were added (GradientUtils.AccumulateGradients,
 *     src/RMAD/GradientUtils.cs:22-42), one deterministic prad_segmented_sum;
 *   - a value with a gradient destination (a weight) gets `destination += gradient`
 *     (OperationBase.AccumulateGradient, src/RMAD/OperationBase.cs:273-304), so a weight
 *     shared by several nodes or time steps accumulates all of them;
 *   - every Backward runs once per node (the visitor re-runs it once per incoming edge).
 * Buffers of intermediate values and gradients are allocated on first use and reused. */
typedef struct prad_graph prad_graph;
typedef enum {
  PRAD_OP_MATMUL = 0,        /* MatrixMultiplyOperation(a, b)                     */
  PRAD_OP_ADD = 1,           /* MatrixAddOperation(a, b)                          */
  PRAD_OP_ADD3 = 2,          /* MatrixAddThreeOperation(a, b, c)                  */
  PRAD_OP_ADD_BROADCAST = 3, /* MatrixAddBroadcastingOperation(x, bias[1 x cols]) */
  PRAD_OP_HADAMARD = 4,      /* HadamardProductOperation(a, b)                    */
  PRAD_OP_LEAKY_RELU = 5,    /* scalar = alpha                                    */
  PRAD_OP_SIGMOID = 6,
  PRAD_OP_TANH = 7,
  PRAD_OP_GELU = 8,
  PRAD_OP_SOFTMAX = 9,
  PRAD_OP_LAYERNORM = 10,
  PRAD_OP_SCALE = 11,        /* MatrixMultiplyScalarOperation, scalar = factor    */
  PRAD_OP_TRANSPOSE = 12,
  PRAD_OP_RELU = 13,
  PRAD_OP_AMPLIFIED_SIGMOID = 14,
  PRAD_OP_SINE_SOFTMAX = 15
} prad_op;

prad_status prad_graph_create(prad_ctx* ctx, prad_dtype dt, prad_graph** out_graph);
prad_status prad_graph_destroy(prad_graph* g);
/* A value is a rows x cols matrix.  data != NULL: caller-owned device matrix (input, weight,
 * constant); data == NULL: produced by a node, owned by the graph. */
prad_status prad_graph_add_value(prad_graph* g, int rows, int cols, void* data, int* out_value);
/* A DeepMatrix value: `depth` consecutive rows x cols slices (the operand type of the Batch* operations,
 * src/RMAD/BatchOperation.cs:11-58, one slice per sample).  A node whose output is deep runs the operation
 * on every slice; an input is deep as well, or ONE Matrix shared by all slices where the managed Batch*
 * class has such an overload -- the second operand of BatchMatrixAddOperation, the third of
 * BatchMatrixAddThreeOperation, the bias of BatchMatrixAddBroadcastingOperation, either operand of
 * Batch(Gpu)MatrixMultiplyOperation.  A shared Matrix must be a leaf; the gradient it receives is the
 * visitor's combined result, the mean over the slices (CombineResults, src/RMAD/
 * OperationNeuralNetworkVisitor.cs:449-478). */
prad_status prad_graph_add_deep_value(prad_graph* g, int depth, int rows, int cols, void* data, int* out_value);
/* Weight-style value: its gradient is ADDED into this caller-owned matrix on every backward. */
prad_status prad_graph_set_gradient_destination(prad_graph* g, int value, void* grad_matrix);
/* Nodes must be added in forward (topological) order; `out_value` must be graph-owned. */
prad_status prad_graph_add_node(prad_graph* g, prad_op op, const int* in_values, int n_in,
                                int out_value, double scalar, int* out_node);
prad_status prad_graph_forward(prad_graph* g);
/* Backward from `start_value` with upstream gradient d_start (device matrix of that shape). */
prad_status prad_graph_backward(prad_graph* g, int start_value, const void* d_start);
/* Backward from several start values at once (host arrays of `count` entries): one reverse walk in which
 * every listed value receives its upstream gradient -- the losses of all time steps of an unrolled
 * recurrent graph in one pass, where the managed code starts one visitor per time step
 * (OperationNeuralNetworkVisitor with a startOperationIndex, src/RMAD/OperationNeuralNetworkVisitor.cs:
 * 60-78) and every visitor walks the whole graph below its start again.  The result is the sum of the
 * single-start backwards (the walk is linear in the upstream gradients); a start value that also has
 * consumers inside the walk adds its upstream gradient first, then the consumers' in their order. */
prad_status prad_graph_backward_multi(prad_graph* g, const int* start_values, const void* const* d_starts, int count);
/* Device pointers valid until the next forward/backward (NULL gradient = not reached). */
prad_status prad_graph_value_data(prad_graph* g, int value, void** out_data);
prad_status prad_graph_value_gradient(prad_graph* g, int value, void** out_grad);
/* How many consumers each value had in the last backward (BackwardDependencyCounts). */
prad_status prad_graph_consumer_count(prad_graph* g, int value, int* out_count);

/* ---------------------------------------------------------------- Tensor elementwise operations
 * The reference's second public API (PRAD `Tensor` / `TensorReverse`, src/PRAD/Tensor.Common.cs and
 * src/PRAD/TensorReverse.Common.cs) evaluates these with MKL VML calls over flat arrays; the entry
 * points follow the same sequence of roundings in the storage type.  Reverse formulas are the ones
 * written there: LogReverse (base-10 forward) multiplies by 1/x like LnReverse;
 * ElementwiseSquareRootReverse is 0.5 * dy / maxmag(sqrt x, 1e-10); ReciprocalReverse reads the
 * forward RESULT (pass it as `saved`); every other reverse reads the input x.
 * Binary reverse: add -> (dy, dy); sub -> (dy, -dy); mul -> (dy*b, dy*a); div -> (dy/b,
 * -((dy*a)/(b*b))); da or db may be NULL. */
typedef enum {
  PRAD_TENSOR_EXP = 0,        /* Tensor.Exp / ExpReverse                                   */
  PRAD_TENSOR_LN = 1,         /* Tensor.Ln / LnReverse                                     */
  PRAD_TENSOR_LOG10 = 2,      /* Tensor.Log (Vml.Log10) / LogReverse                       */
  PRAD_TENSOR_ABS = 3,        /* Tensor.Abs / AbsReverse                                   */
  PRAD_TENSOR_SQUARE = 4,     /* ElementwiseSquare / ElementwiseSquareReverse              */
  PRAD_TENSOR_SQRT = 5,       /* ElementwiseSquareRoot / ElementwiseSquareRootReverse      */
  PRAD_TENSOR_SIN = 6,        /* ElementwiseSin / ElementwiseSinReverse                    */
  PRAD_TENSOR_COS = 7,        /* ElementwiseCos / ElementwiseCosReverse                    */
  PRAD_TENSOR_RECIPROCAL = 8, /* Reciprocal / ReciprocalReverse                            */
  PRAD_TENSOR_NEGATE = 9,     /* ElementwiseNegate                                         */
  PRAD_TENSOR_ADD = 16,       /* ElementwiseAdd / ElementwiseAddReverse                    */
  PRAD_TENSOR_SUB = 17,       /* ElementwiseSub / ElementwiseSubReverse                    */
  PRAD_TENSOR_MUL = 18,       /* ElementwiseMultiply / ElementwiseMultiplyReverse          */
  PRAD_TENSOR_DIV = 19        /* ElementwiseDivide / ElementwiseDivideReverse              */
} prad_tensor_op;
prad_status prad_tensor_unary(prad_ctx* ctx, prad_dtype dt, prad_tensor_op op, const void* x, void* y, int64_t n);
prad_status prad_tensor_unary_reverse(prad_ctx* ctx, prad_dtype dt, prad_tensor_op op, const void* saved,
                                      const void* dy, void* dx, int64_t n);
prad_status prad_tensor_binary(prad_ctx* ctx, prad_dtype dt, prad_tensor_op op, const void* a, const void* b, void* y,
                               int64_t n);
prad_status prad_tensor_binary_reverse(prad_ctx* ctx, prad_dtype dt, prad_tensor_op op, const void* a, const void* b,
                                       const void* dy, void* da, void* db, int64_t n);

/* Tensor.MatrixMultiply (src/PRAD/Tensor.cs:572-613, MKL dgemm / sgemm, row-major NN): C = alpha*A*B +
 * beta*C for 2-D tensors.  The shape rule of :582-585 is kept: a_cols != b_rows returns PRAD_ERR_SHAPE
 * with the managed message "Incompatible shapes for matrix multiplication.".
 * TensorReverse.MatrixMultiplyReverse (src/PRAD/TensorReverse.cs:94-160): dA = dC * B^T (gemm NoTrans,
 * Trans), dB = A^T * dC (gemm Trans, NoTrans); either result may be NULL.  Both run on the same GEMM
 * kernels as prad_gemm (MKL's own summation order is not reproduced: tolerance-level parity). */
prad_status prad_tensor_matmul(prad_ctx* ctx, prad_dtype dt, const void* A, int a_rows, int a_cols, const void* B,
                               int b_rows, int b_cols, double alpha, double beta, void* C);
prad_status prad_tensor_matmul_reverse(prad_ctx* ctx, prad_dtype dt, const void* A, int a_rows, int a_cols,
                                       const void* B, int b_rows, int b_cols, const void* dC, void* dA, void* dB);
/* Tensor.Gather (src/PRAD/Tensor.Common.cs:959-1090) along one axis: the tensor is passed as
 * x[outer][axis_len][inner] (outer / inner = product of the dimensions before / after the axis), the
 * `count` indices are values of the storage type (negative ones count from the end, :974), the result
 * is y[outer][count][inner]; an index outside the axis returns PRAD_ERR_INVALID (ArgumentException).
 * TensorReverse.GatherReverse (src/PRAD/TensorReverse.Common.cs:2358-2426): dx[o][indices[c]][i] +=
 * upstream[o][c][i].  The managed loop is a Parallel.For with a lock, so duplicates are added in a
 * thread-dependent order there; here they are added in ascending c (the order of a sequential loop),
 * bit-identical for unique indices and deterministic for repeated ones. */
prad_status prad_tensor_gather(prad_ctx* ctx, prad_dtype dt, const void* x, int64_t outer, int axis_len, int64_t inner,
                               const void* indices, int count, void* y);
prad_status prad_tensor_gather_reverse(prad_ctx* ctx, prad_dtype dt, const void* upstream, int64_t outer, int axis_len,
                                       int64_t inner, const void* indices, int count, void* dx);
/* Tensor.Tile (src/PRAD/Tensor.Common.cs:1096-1230) for 2-D tensors: y[r][c] = x[r % rows][c % cols], y is
 * (rows*mult_rows) x (cols*mult_cols).  TensorReverse.TileReverse (src/PRAD/TensorReverse.Common.cs:
 * 2713-2785): every input element collects its copies in the order of the upstream gradient's flat
 * index.  As written there, multiples {m, 1} take a specialised routine (:3326-3370) that reads rows
 * i*m .. i*m+m-1 of the upstream gradient for input row i; that is reproduced. */
prad_status prad_tensor_tile(prad_ctx* ctx, prad_dtype dt, const void* x, int rows, int cols, int mult_rows, int mult_cols,
                             void* y);
prad_status prad_tensor_tile_reverse(prad_ctx* ctx, prad_dtype dt, const void* upstream, int rows, int cols, int mult_rows,
                                     int mult_cols, void* dx);
/* The remaining 2-D Tensor operations map onto existing entry points: Tensor.SumRows (src/PRAD/Tensor.cs:
 * 769-786) = prad_row_sum_forward, TensorReverse.SumRowsReverse (TensorReverse.Common.cs:2936-2958) =
 * prad_row_sum_backward; Tensor.Transpose {1,0} and {0,2,1} and TensorReverse.TransposeReverse
 * (TensorReverse.Common.cs:2967-3040) = prad_transpose (the reverse of a transposition is the
 * transposition of the upstream gradient with rows and cols exchanged); Tensor.Embedding /
 * EmbeddingReverse = prad_embedding_forward / prad_embedding_backward. */

/* ---------------------------------------------------------------- recorded launch sequences
 * No counterpart in the reference, whose executor walks the operation list and calls each
 * Backward from managed code every step (src/RMAD/ComputationGraph.cs, NeuralNetwork
 * AutomaticBackwardPropagate).  For the small configurations that walk is the cost: hundreds
 * of launches of a few microseconds each.  Between prad_capture_begin and prad_capture_end
 * every entry point that only enqueues device work (GEMMs, elementwise and row operations,
 * losses, accumulation, clip/Adam without a host result, prad_zero, prad_copy, graph-mode
 * forward/backward) records into a launch sequence instead of running; nothing executes.
 * prad_sequence_launch then replays the whole sequence with one submission, on the same
 * buffers with whatever they hold at that moment.
 * Entry points that wait for the device, move host data, check embedding indices or grow
 * library scratch return PRAD_ERR_INVALID while a recording is open: run the step once
 * unrecorded first, so that scratch has its final size.  Scratch that a live sequence may
 * address is kept until the last sequence of the context is destroyed.  The buffers a
 * sequence addresses must stay allocated while it is in use. */
typedef struct prad_sequence prad_sequence;
prad_status prad_capture_begin(prad_ctx* ctx);
prad_status prad_capture_end(prad_ctx* ctx, prad_sequence** out_sequence);
prad_status prad_sequence_launch(prad_ctx* ctx, prad_sequence* sequence);
/* How many kernel launches one replay stands for (added to prad_launch_count per replay). */
prad_status prad_sequence_launch_count(prad_sequence* sequence, int64_t* out_count);
prad_status prad_sequence_destroy(prad_ctx* ctx, prad_sequence* sequence);

/* ---------------------------------------------------------------- data parallel
 * Not in the reference (it has no multi-device code; its closest relative is the offline
 * averaging of GradientStore.AverageGradients, src/RMAD/GradientStore.cs:24-104).
 * One process per GPU.  Rank 0 calls prad_dp_unique_id and ships the 128 bytes to the
 * other ranks by any host channel; every rank then calls prad_dp_init.
 * prad_dp_allreduce enqueues a SUM all-reduce on the context's communication stream after
 * everything enqueued so far on the compute stream, so it overlaps with later compute;
 * prad_dp_wait makes the compute stream wait for all outstanding all-reduces. */
prad_status prad_dp_unique_id(void* out_id_128_bytes);
prad_status prad_dp_init(prad_ctx* ctx, const void* id_128_bytes, int rank, int world_size);
prad_status prad_dp_allreduce(prad_ctx* ctx, prad_dtype dt, void* buf, int64_t n);
prad_status prad_dp_wait(prad_ctx* ctx);
/* Sharded optimiser: prad_dp_reduce leaves the SUM over all ranks in `buf` of rank `root` only (the
 * other ranks' buffers keep their partial sums); prad_dp_broadcast copies `buf` of rank `root` into `buf`
 * of every rank.  Both are enqueued on the communication stream after everything enqueued so far on the
 * compute stream, like prad_dp_allreduce; prad_dp_wait joins.  The owner of a tensor clips and updates
 * it alone (the reference's clip needs only that tensor's own statistics, src/RMAD/GradientClipper.cs:
 * 118-157) and broadcasts the new weights. */
prad_status prad_dp_reduce(prad_ctx* ctx, prad_dtype dt, void* buf, int64_t n, int root);
prad_status prad_dp_broadcast(prad_ctx* ctx, prad_dtype dt, void* buf, int64_t n, int root);
/* Finer joins than prad_dp_wait: prad_dp_mark remembers, under `slot` (0 .. PRAD_DP_MARKS - 1), the position the
 * communication stream has reached -- everything enqueued on it so far; prad_dp_wait_mark makes the compute stream
 * wait for that position only.  With one mark per broadcast, the first layer of the next pass starts as soon
 * as ITS weights have arrived while the other tensors are still on their way. */
#define PRAD_DP_MARKS 256
prad_status prad_dp_mark(prad_ctx* ctx, int slot);
prad_status prad_dp_wait_mark(prad_ctx* ctx, int slot);
/* Host-side join with a deadline, the counterpart of the visitor's bounded wait on a sibling task
 * (TimeoutInMinutes, src/RMAD/OperationNeuralNetworkVisitor.cs:27,264-270): blocks the calling thread
 * until the outstanding collectives have completed (then the compute stream is joined as by
 * prad_dp_wait), NCCL reports an asynchronous error (PRAD_ERR_COMM), or timeout_ms have passed
 * (PRAD_ERR_TIMEOUT: a rank never arrived).  In both failure cases the communicator is aborted, so the
 * kernels of the collective leave the GPU; every later prad_dp_* call fails with PRAD_ERR_COMM until
 * prad_dp_shutdown + prad_dp_init build a new communicator. */
prad_status prad_dp_wait_host(prad_ctx* ctx, double timeout_ms);
prad_status prad_dp_shutdown(prad_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* PRAD_CUDA_H_ */
