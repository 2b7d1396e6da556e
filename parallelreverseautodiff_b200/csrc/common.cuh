// Shared plumbing of libprad_cuda: context, error reporting, launch helpers.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/prad_cuda.h"

namespace prad {

void set_error(const char* fmt, ...);

enum class GemmF32 { Auto, Simt, SimtFma, Tf32x3, Tf32B16, Bf16x3, Fp16x3 };
enum class GemmF64 { Auto, Simt, SimtFma, Dmma };

struct DpState;  // data-parallel state (dp.cu)

}  // namespace prad

struct prad_ctx {
  int device = 0;
  cudaStream_t own_stream = nullptr;  // created by prad_init
  cudaStream_t stream = nullptr;      // the stream work is enqueued on
  int sm_count = 0;
  cudaStream_t copy_stream = nullptr;  // prad_upload_prefetch
  cudaEvent_t copy_done = nullptr;
  bool copy_pending = false;
  int64_t launches = 0;
  prad::GemmF32 gemm_f32 = prad::GemmF32::Auto;
  prad::GemmF64 gemm_f64 = prad::GemmF64::Auto;
  // scratch (grown on demand, never shrunk): device workspace, pointer tables, pinned host
  void* ws = nullptr;
  size_t ws_bytes = 0;
  void* host_ws = nullptr;
  size_t host_ws_bytes = 0;
  // host-buffer entry points keep their device staging here
  void* stage = nullptr;
  size_t stage_bytes = 0;
  prad::DpState* dp = nullptr;
  // give-up flag of the tensor-core GEMMs (device int, sticky until the host reads it)
  int* tc_err = nullptr;
  bool tc_pending_check = false;
  int tc_variant = 0;  // pipeline shape of the tensor-core GEMM (option "tc_pipeline")
  bool tc_split_k = true;  // option "tc_split_k": cut k across CTAs when the tile count wastes SMs
  int tc_prefetch = 0;     // option "tc_prefetch": k-blocks of 32 by which the packed FP16 product prefetches its row operand into L2
  int gemm_small = 1;      // option "gemm_small": batches of products of at most 64 x 64 outputs on one CTA per product
  int tc_pair = 1;         // option "tc_pair": packed FP16 products on CTA pairs (tcgen05 cta_group::2, 256-row tiles): 0 never, 1 for k or N >= 1024, 2 always
  int tc_panel_n = 0;      // option "tc_panel_n": column tiles per panel of the persistent GEMM's tile walk (0 = automatic)
  int tc_chunk_k = 256;    // option "tc_chunk_k": k per accumulation chunk of the persistent GEMM
  bool tc_chunk_k_set = false;   // the option was given (packed FP16 operands default to 128-long blocks otherwise)
  int tc_reserve_sms = 0;  // option "tc_reserve_sms": SMs the persistent GEMM leaves free (for a collective's kernels)
  bool tc_persistent = true;  // option "tc_persistent": TF32+BF16 products run on the persistent kernel
  int tc_auto_mode = 3;  // split scheme "auto" picks: 0 = 3xTF32, 1 = TF32 + BF16 corrections, 2 = BF16 x 6, 3 = FP16 x 3
  // recorded launch sequences (prad_capture_begin ... prad_sequence_launch)
  bool capturing = false;
  int64_t capture_launches0 = 0;
  int live_sequences = 0;
  std::vector<void*> retired;  // scratch blocks a live sequence may still address; freed with the last sequence
  uint32_t magic = 0x50524144u;  // "PRAD"
};

struct prad_sequence {
  cudaGraphExec_t exec = nullptr;
  int64_t launches = 0;
  prad_ctx* owner = nullptr;
  uint32_t magic = 0x50534551u;  // "PSEQ"
};

namespace prad {

inline bool ctx_ok(const prad_ctx* c) { return c != nullptr && c->magic == 0x50524144u; }

#define PRAD_CHECK_CTX(ctx)                                                              \
  do {                                                                                   \
    if (!prad::ctx_ok(ctx)) {                                                            \
      prad::set_error("context is null or was shut down (call prad_init first)");        \
      return PRAD_ERR_NOT_INITIALIZED;                                                   \
    }                                                                                    \
    cudaError_t e_ = cudaSetDevice((ctx)->device);                                       \
    if (e_ != cudaSuccess) {                                                             \
      prad::set_error("cudaSetDevice(%d): %s", (ctx)->device, cudaGetErrorString(e_));   \
      return PRAD_ERR_CUDA;                                                              \
    }                                                                                    \
  } while (0)

#define PRAD_CUDA(call)                                                                  \
  do {                                                                                   \
    cudaError_t e_ = (call);                                                             \
    if (e_ != cudaSuccess) {                                                             \
      prad::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__,  \
                      __LINE__);                                                         \
      return e_ == cudaErrorMemoryAllocation ? PRAD_ERR_OOM : PRAD_ERR_CUDA;             \
    }                                                                                    \
  } while (0)

// entry points that must wait for the device (or move host data) cannot be recorded
#define PRAD_NOT_CAPTURING(ctx, what)                                                    \
  do {                                                                                   \
    if ((ctx)->capturing) {                                                              \
      prad::set_error("%s cannot be recorded into a launch sequence (it waits for the "  \
                      "device, moves host data or grows scratch); call it outside "      \
                      "prad_capture_begin/prad_capture_end", what);                      \
      return PRAD_ERR_INVALID;                                                           \
    }                                                                                    \
  } while (0)

#define PRAD_REQUIRE(cond, code, ...)                                                    \
  do {                                                                                   \
    if (!(cond)) {                                                                       \
      prad::set_error(__VA_ARGS__);                                                      \
      return code;                                                                       \
    }                                                                                    \
  } while (0)

// after a kernel launch: count it and surface launch-configuration errors
#define PRAD_LAUNCHED(ctx)                                                               \
  do {                                                                                   \
    (ctx)->launches++;                                                                   \
    cudaError_t e_ = cudaPeekAtLastError();                                              \
    if (e_ != cudaSuccess) {                                                             \
      (void)cudaGetLastError();                                                          \
      prad::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e_),        \
                      __FILE__, __LINE__);                                               \
      return PRAD_ERR_CUDA;                                                              \
    }                                                                                    \
  } while (0)

inline bool dtype_ok(prad_dtype dt) { return dt == PRAD_F32 || dt == PRAD_F64; }
inline size_t dtype_size(prad_dtype dt) { return dt == PRAD_F64 ? 8 : 4; }

// grows ctx->ws to at least `bytes` (256-byte aligned) ; previous contents are lost
prad_status ensure_workspace(prad_ctx* ctx, size_t bytes);
// grows the pinned host scratch
prad_status ensure_host_workspace(prad_ctx* ctx, size_t bytes);
prad_status ensure_stage(prad_ctx* ctx, size_t bytes);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// grid size for a grid-stride streaming kernel: a multiple of the SM count
inline int stream_grid(const prad_ctx* ctx, int64_t work_items, int per_block, int ctas_per_sm) {
  int64_t need = ceil_div(work_items, per_block);
  int64_t cap = (int64_t)ctx->sm_count * ctas_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

// ---- internal entry points shared between translation units -------------------------------
struct GemmEpilogue {
  // C = alpha*acc + beta*C ; then  + bias[n] ; store Z_out ; then act / act' multiply
  const void* bias = nullptr;      // row vector of N (forward)
  void* z_out = nullptr;           // pre-activation copy (forward)
  prad_act act = PRAD_ACT_NONE;    // forward activation applied to the value
  prad_act dact = PRAD_ACT_NONE;   // backward: multiply by act'(saved[m][n])
  const void* saved = nullptr;     // M x N tensor (ld = ldc) read by dact
  double act_alpha = 0.0;
};

// reads (and clears) the tensor-core GEMM give-up flag; PRAD_ERR_TIMEOUT if it was raised
prad_status gemm_tf32x3_check(prad_ctx* ctx);

prad_status gemm_dispatch(prad_ctx* ctx, prad_dtype dt, bool transA, bool transB, int M, int N,
                          int K, double alpha, const void* A, int lda, const void* B, int ldb,
                          double beta, void* C, int ldc, int batch, int64_t sA, int64_t sB,
                          int64_t sC, const GemmEpilogue& epi);

// dW[idx[i]][:] += dOut[i][:] for i ascending (bit-identical to the sequential loop); loss_embedding.cu
prad_status embedding_scatter_ordered(prad_ctx* ctx, prad_dtype dt, const void* index_col, const void* dOut,
                                      void* dW, int n, int vocab, int dim, int* bad);

}  // namespace prad
