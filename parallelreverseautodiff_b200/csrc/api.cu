// Lifecycle, error reporting and memory entry points of libprad_cuda.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace prad {

static thread_local char g_err[1024] = {0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static prad_status grow(prad_ctx* ctx, void** p, size_t* have, size_t need, bool host, const char* what) {
  if (*have >= need) return PRAD_OK;
  PRAD_NOT_CAPTURING(ctx, what);
  // earlier kernels may still read the old block
  cudaError_t e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) { set_error("sync before %s: %s", what, cudaGetErrorString(e)); return PRAD_ERR_CUDA; }
  size_t want = need + need / 4;
  want = (want + 255) & ~(size_t)255;
  if (*p) {
    if (host) cudaFreeHost(*p);
    else if (ctx->live_sequences > 0) ctx->retired.push_back(*p);   // a recorded sequence may address it
    else cudaFree(*p);
    *p = nullptr;
    *have = 0;
  }
  e = host ? cudaMallocHost(p, want) : cudaMalloc(p, want);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error("scratch allocation of %zu bytes failed: %s", want, cudaGetErrorString(e));
    return PRAD_ERR_OOM;
  }
  *have = want;
  return PRAD_OK;
}

prad_status ensure_workspace(prad_ctx* ctx, size_t bytes) {
  return grow(ctx, &ctx->ws, &ctx->ws_bytes, bytes, false, "growth of the device scratch");
}
prad_status ensure_host_workspace(prad_ctx* ctx, size_t bytes) {
  return grow(ctx, &ctx->host_ws, &ctx->host_ws_bytes, bytes, true, "growth of the pinned host scratch");
}
prad_status ensure_stage(prad_ctx* ctx, size_t bytes) {
  return grow(ctx, &ctx->stage, &ctx->stage_bytes, bytes, false, "growth of the staging scratch");
}

prad_status dp_destroy(prad_ctx* ctx);  // dp.cu
void runtime_destroy(prad_ctx* ctx);    // runtime.cu

}  // namespace prad

using namespace prad;

extern "C" {

const char* prad_last_error(void) { return g_err; }

const char* prad_version(void) { return "libprad_cuda 0.1 (sm_100a)"; }

prad_status prad_init(int device, prad_ctx** out_ctx) {
  PRAD_REQUIRE(out_ctx != nullptr, PRAD_ERR_INVALID, "prad_init: out_ctx is null");
  *out_ctx = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    set_error("prad_init: no usable CUDA device (%s); this library has no CPU fallback",
              e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    return PRAD_ERR_NOT_INITIALIZED;
  }
  PRAD_REQUIRE(device >= 0 && device < count, PRAD_ERR_INVALID,
               "prad_init: device %d out of range (0..%d)", device, count - 1);
  PRAD_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  PRAD_CUDA(cudaGetDeviceProperties(&prop, device));
  PRAD_REQUIRE(prop.major == 10, PRAD_ERR_UNSUPPORTED,
               "prad_init: device %d is sm_%d%d; this library is built for sm_100a only", device,
               prop.major, prop.minor);
  prad_ctx* c = new prad_ctx();
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  e = cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    set_error("prad_init: cudaStreamCreate: %s", cudaGetErrorString(e));
    delete c;
    return PRAD_ERR_CUDA;
  }
  c->stream = c->own_stream;
  e = cudaMalloc((void**)&c->tc_err, 256);
  if (e == cudaSuccess) e = cudaMemset(c->tc_err, 0, 256);
  if (e != cudaSuccess) {
    set_error("prad_init: flag allocation: %s", cudaGetErrorString(e));
    cudaStreamDestroy(c->own_stream);
    delete c;
    return PRAD_ERR_CUDA;
  }
  *out_ctx = c;
  g_err[0] = 0;
  return PRAD_OK;
}

prad_status prad_shutdown(prad_ctx* ctx) {
  PRAD_CHECK_CTX(ctx);
  cudaStreamSynchronize(ctx->stream);
  dp_destroy(ctx);
  runtime_destroy(ctx);
  if (ctx->ws) cudaFree(ctx->ws);
  if (ctx->tc_err) cudaFree(ctx->tc_err);
  for (void* r : ctx->retired) cudaFree(r);
  if (ctx->stage) cudaFree(ctx->stage);
  if (ctx->host_ws) cudaFreeHost(ctx->host_ws);
  if (ctx->copy_stream) { cudaStreamSynchronize(ctx->copy_stream); cudaStreamDestroy(ctx->copy_stream); }
  if (ctx->copy_done) cudaEventDestroy(ctx->copy_done);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  ctx->magic = 0;
  delete ctx;
  return PRAD_OK;
}

prad_status prad_set_option(prad_ctx* ctx, const char* key, const char* value) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(key && value, PRAD_ERR_INVALID, "prad_set_option: null key or value");
  if (!strcmp(key, "gemm_f32")) {
    if (!strcmp(value, "auto")) ctx->gemm_f32 = GemmF32::Auto;
    else if (!strcmp(value, "simt")) ctx->gemm_f32 = GemmF32::Simt;
    else if (!strcmp(value, "simt_fma")) ctx->gemm_f32 = GemmF32::SimtFma;
    else if (!strcmp(value, "tf32x3")) ctx->gemm_f32 = GemmF32::Tf32x3;
    else if (!strcmp(value, "tf32b16")) ctx->gemm_f32 = GemmF32::Tf32B16;
    else if (!strcmp(value, "bf16x3")) ctx->gemm_f32 = GemmF32::Bf16x3;
    else if (!strcmp(value, "fp16x3")) ctx->gemm_f32 = GemmF32::Fp16x3;
    else { set_error("prad_set_option: gemm_f32 must be auto|simt|simt_fma|tf32x3|tf32b16|bf16x3|fp16x3, got '%s'", value); return PRAD_ERR_INVALID; }
    return PRAD_OK;
  }
  if (!strcmp(key, "gemm_f64")) {
    if (!strcmp(value, "auto")) ctx->gemm_f64 = GemmF64::Auto;
    else if (!strcmp(value, "simt")) ctx->gemm_f64 = GemmF64::Simt;
    else if (!strcmp(value, "simt_fma")) ctx->gemm_f64 = GemmF64::SimtFma;
    else if (!strcmp(value, "dmma")) ctx->gemm_f64 = GemmF64::Dmma;
    else { set_error("prad_set_option: gemm_f64 must be auto|simt|simt_fma|dmma, got '%s'", value); return PRAD_ERR_INVALID; }
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_auto")) {   // which split scheme gemm_f32=auto uses for large products
    if (!strcmp(value, "tf32x3")) ctx->tc_auto_mode = 0;
    else if (!strcmp(value, "tf32b16")) ctx->tc_auto_mode = 1;
    else if (!strcmp(value, "bf16x3")) ctx->tc_auto_mode = 2;
    else if (!strcmp(value, "fp16x3")) ctx->tc_auto_mode = 3;
    else { set_error("prad_set_option: tc_auto must be tf32x3|tf32b16|bf16x3|fp16x3, got '%s'", value); return PRAD_ERR_INVALID; }
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_prefetch")) {
    const int n = atoi(value);
    PRAD_REQUIRE(n >= 0 && n <= 64, PRAD_ERR_INVALID, "prad_set_option: tc_prefetch must be 0..64, got '%s'", value);
    ctx->tc_prefetch = n;
    return PRAD_OK;
  }
  if (!strcmp(key, "gemm_small")) {
    PRAD_REQUIRE(!strcmp(value, "0") || !strcmp(value, "1"), PRAD_ERR_INVALID, "prad_set_option: gemm_small must be 0 or 1, got '%s'", value);
    ctx->gemm_small = atoi(value);
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_pair")) {
    PRAD_REQUIRE(!strcmp(value, "0") || !strcmp(value, "1") || !strcmp(value, "2"), PRAD_ERR_INVALID, "prad_set_option: tc_pair must be 0, 1 or 2, got '%s'", value);
    ctx->tc_pair = atoi(value);
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_panel_n")) {
    const int n = atoi(value);
    PRAD_REQUIRE(n >= 0, PRAD_ERR_INVALID, "prad_set_option: tc_panel_n must be >= 0, got '%s'", value);
    ctx->tc_panel_n = n;
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_chunk_k")) {
    const int n = atoi(value);
    PRAD_REQUIRE(n == 128 || n == 256 || n == 512 || n == 1024, PRAD_ERR_INVALID,
                 "prad_set_option: tc_chunk_k must be 128, 256, 512 or 1024, got '%s'", value);
    ctx->tc_chunk_k = n;
    ctx->tc_chunk_k_set = true;
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_reserve_sms")) {
    const int n = atoi(value);
    PRAD_REQUIRE(n >= 0 && n < ctx->sm_count, PRAD_ERR_INVALID, "prad_set_option: tc_reserve_sms must be in [0, %d), got '%s'",
                 ctx->sm_count, value);
    ctx->tc_reserve_sms = n;
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_persistent")) {
    ctx->tc_persistent = strcmp(value, "off") != 0 && strcmp(value, "0") != 0;
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_split_k")) {
    ctx->tc_split_k = strcmp(value, "off") != 0 && strcmp(value, "0") != 0;
    return PRAD_OK;
  }
  if (!strcmp(key, "tc_pipeline")) {  // tensor-core GEMM pipeline: k-block floats x stages
    if (!strcmp(value, "16x4")) ctx->tc_variant = 0;
    else if (!strcmp(value, "32x2")) ctx->tc_variant = 1;
    else if (!strcmp(value, "8x8")) ctx->tc_variant = 2;
    else { set_error("prad_set_option: tc_pipeline must be 32x2|16x4|8x8, got '%s'", value); return PRAD_ERR_INVALID; }
    return PRAD_OK;
  }
  set_error("prad_set_option: unknown key '%s'", key);
  return PRAD_ERR_INVALID;
}

prad_status prad_sync(prad_ctx* ctx) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_sync");
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  return gemm_tf32x3_check(ctx);
}

prad_status prad_launch_count(prad_ctx* ctx, int64_t* out_count) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(out_count, PRAD_ERR_INVALID, "prad_launch_count: null output");
  *out_count = ctx->launches;
  return PRAD_OK;
}

prad_status prad_stream(prad_ctx* ctx, void** out_stream) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(out_stream, PRAD_ERR_INVALID, "prad_stream: null output");
  *out_stream = (void*)ctx->stream;
  return PRAD_OK;
}

prad_status prad_use_stream(prad_ctx* ctx, void* stream) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_use_stream");
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  ctx->stream = stream ? (cudaStream_t)stream : ctx->own_stream;
  return PRAD_OK;
}

prad_status prad_alloc(prad_ctx* ctx, size_t bytes, void** out_dptr) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(out_dptr, PRAD_ERR_INVALID, "prad_alloc: null output");
  *out_dptr = nullptr;
  if (bytes == 0) bytes = 16;
  cudaError_t e = cudaMalloc(out_dptr, bytes);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error("prad_alloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
    return e == cudaErrorMemoryAllocation ? PRAD_ERR_OOM : PRAD_ERR_CUDA;
  }
  return PRAD_OK;
}

prad_status prad_free(prad_ctx* ctx, void* dptr) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_free");
  if (!dptr) return PRAD_OK;
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  PRAD_CUDA(cudaFree(dptr));
  return PRAD_OK;
}

prad_status prad_alloc_host(prad_ctx* ctx, size_t bytes, void** out_hptr) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(out_hptr, PRAD_ERR_INVALID, "prad_alloc_host: null output");
  *out_hptr = nullptr;
  if (bytes == 0) bytes = 16;
  cudaError_t e = cudaMallocHost(out_hptr, bytes);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error("prad_alloc_host(%zu bytes): %s", bytes, cudaGetErrorString(e));
    return PRAD_ERR_OOM;
  }
  return PRAD_OK;
}

prad_status prad_free_host(prad_ctx* ctx, void* hptr) {
  PRAD_CHECK_CTX(ctx);
  if (!hptr) return PRAD_OK;
  PRAD_CUDA(cudaFreeHost(hptr));
  return PRAD_OK;
}

prad_status prad_zero(prad_ctx* ctx, void* dptr, size_t bytes) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(dptr || bytes == 0, PRAD_ERR_INVALID, "prad_zero: null pointer");
  if (bytes) PRAD_CUDA(cudaMemsetAsync(dptr, 0, bytes, ctx->stream));
  return PRAD_OK;
}

prad_status prad_copy(prad_ctx* ctx, void* dst, const void* src, size_t bytes) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE((dst && src) || bytes == 0, PRAD_ERR_INVALID, "prad_copy: null pointer");
  if (bytes) PRAD_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return PRAD_OK;
}

prad_status prad_copy_2d(prad_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                         size_t width_bytes, size_t rows) {
  PRAD_CHECK_CTX(ctx);
  if (width_bytes == 0 || rows == 0) return PRAD_OK;
  PRAD_REQUIRE(dst && src && dst_pitch >= width_bytes && src_pitch >= width_bytes, PRAD_ERR_INVALID,
               "prad_copy_2d: null pointer or a pitch smaller than the row width");
  PRAD_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDeviceToDevice, ctx->stream));
  return PRAD_OK;
}

prad_status prad_upload(prad_ctx* ctx, void* dst, const void* src_host, size_t bytes) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_upload");
  PRAD_REQUIRE((dst && src_host) || bytes == 0, PRAD_ERR_INVALID, "prad_upload: null pointer");
  if (bytes) PRAD_CUDA(cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return PRAD_OK;
}

prad_status prad_download(prad_ctx* ctx, void* dst_host, const void* src, size_t bytes) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_download");
  PRAD_REQUIRE((dst_host && src) || bytes == 0, PRAD_ERR_INVALID, "prad_download: null pointer");
  if (bytes) {
    PRAD_CUDA(cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  return gemm_tf32x3_check(ctx);
}

prad_status prad_upload_prefetch(prad_ctx* ctx, void* dst, const void* src_host, size_t bytes) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_upload_prefetch");
  PRAD_REQUIRE((dst && src_host) || bytes == 0, PRAD_ERR_INVALID, "prad_upload_prefetch: null pointer");
  if (bytes == 0) return PRAD_OK;
  if (!ctx->copy_stream) {
    PRAD_CUDA(cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    PRAD_CUDA(cudaEventCreateWithFlags(&ctx->copy_done, cudaEventDisableTiming));
  }
  PRAD_CUDA(cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
  ctx->copy_pending = true;
  return PRAD_OK;
}

prad_status prad_upload_join(prad_ctx* ctx) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_upload_join");
  if (!ctx->copy_pending) return PRAD_OK;
  PRAD_CUDA(cudaEventRecord(ctx->copy_done, ctx->copy_stream));
  PRAD_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->copy_done, 0));
  ctx->copy_pending = false;
  return PRAD_OK;
}

// Jagged rows are gathered into one pinned block first, so the device sees ONE copy.
prad_status prad_upload_rows(prad_ctx* ctx, void* dst, const void* const* src_rows, int rows,
                             size_t row_bytes) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_upload_rows");
  PRAD_REQUIRE(rows >= 0, PRAD_ERR_INVALID, "prad_upload_rows: negative row count");
  if (rows == 0 || row_bytes == 0) return PRAD_OK;
  PRAD_REQUIRE(dst && src_rows, PRAD_ERR_INVALID, "prad_upload_rows: null pointer");
  size_t total = (size_t)rows * row_bytes;
  prad_status s = ensure_host_workspace(ctx, total);
  if (s) return s;
  // the pinned block may still feed an earlier asynchronous copy
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  for (int i = 0; i < rows; ++i) {
    PRAD_REQUIRE(src_rows[i], PRAD_ERR_INVALID, "prad_upload_rows: row %d is null", i);
    memcpy((char*)ctx->host_ws + (size_t)i * row_bytes, src_rows[i], row_bytes);
  }
  PRAD_CUDA(cudaMemcpyAsync(dst, ctx->host_ws, total, cudaMemcpyHostToDevice, ctx->stream));
  return PRAD_OK;
}

prad_status prad_download_rows(prad_ctx* ctx, void* const* dst_rows, const void* src, int rows,
                               size_t row_bytes) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_download_rows");
  PRAD_REQUIRE(rows >= 0, PRAD_ERR_INVALID, "prad_download_rows: negative row count");
  if (rows == 0 || row_bytes == 0) return PRAD_OK;
  PRAD_REQUIRE(dst_rows && src, PRAD_ERR_INVALID, "prad_download_rows: null pointer");
  size_t total = (size_t)rows * row_bytes;
  prad_status s = ensure_host_workspace(ctx, total);
  if (s) return s;
  PRAD_CUDA(cudaMemcpyAsync(ctx->host_ws, src, total, cudaMemcpyDeviceToHost, ctx->stream));
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  for (int i = 0; i < rows; ++i) {
    PRAD_REQUIRE(dst_rows[i], PRAD_ERR_INVALID, "prad_download_rows: row %d is null", i);
    memcpy(dst_rows[i], (const char*)ctx->host_ws + (size_t)i * row_bytes, row_bytes);
  }
  return PRAD_OK;
}

// ---- recorded launch sequences ---------------------------------------------------------
prad_status prad_capture_begin(prad_ctx* ctx) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(!ctx->capturing, PRAD_ERR_INVALID, "prad_capture_begin: a recording is already open");
  PRAD_REQUIRE(!ctx->copy_pending, PRAD_ERR_INVALID, "prad_capture_begin: join the pending prefetch first");
  PRAD_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  ctx->capturing = true;
  ctx->capture_launches0 = ctx->launches;
  return PRAD_OK;
}

prad_status prad_capture_end(prad_ctx* ctx, prad_sequence** out_sequence) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(ctx->capturing, PRAD_ERR_INVALID, "prad_capture_end: no recording is open");
  ctx->capturing = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
  if (e != cudaSuccess || graph == nullptr) {
    (void)cudaGetLastError();
    set_error("prad_capture_end: the recording was invalidated (%s); an entry point that cannot be recorded "
              "was probably called in between", cudaGetErrorString(e));
    return PRAD_ERR_CUDA;
  }
  PRAD_REQUIRE(out_sequence, PRAD_ERR_INVALID, "prad_capture_end: null output");
  prad_sequence* seq = new prad_sequence();
  e = cudaGraphInstantiate(&seq->exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    delete seq;
    set_error("prad_capture_end: cudaGraphInstantiate: %s", cudaGetErrorString(e));
    return PRAD_ERR_CUDA;
  }
  seq->launches = ctx->launches - ctx->capture_launches0;
  ctx->launches = ctx->capture_launches0;   // nothing ran while recording
  seq->owner = ctx;
  ctx->live_sequences++;
  *out_sequence = seq;
  return PRAD_OK;
}

prad_status prad_sequence_launch(prad_ctx* ctx, prad_sequence* seq) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(seq && seq->magic == 0x50534551u && seq->owner == ctx, PRAD_ERR_INVALID,
               "prad_sequence_launch: not a sequence of this context");
  PRAD_NOT_CAPTURING(ctx, "prad_sequence_launch");
  PRAD_CUDA(cudaGraphLaunch(seq->exec, ctx->stream));
  ctx->launches += seq->launches;
  ctx->tc_pending_check = true;
  return PRAD_OK;
}

prad_status prad_sequence_launch_count(prad_sequence* seq, int64_t* out_count) {
  PRAD_REQUIRE(seq && seq->magic == 0x50534551u && out_count, PRAD_ERR_INVALID, "prad_sequence_launch_count: bad argument");
  *out_count = seq->launches;
  return PRAD_OK;
}

prad_status prad_sequence_destroy(prad_ctx* ctx, prad_sequence* seq) {
  PRAD_CHECK_CTX(ctx);
  if (!seq) return PRAD_OK;
  PRAD_REQUIRE(seq->magic == 0x50534551u && seq->owner == ctx, PRAD_ERR_INVALID,
               "prad_sequence_destroy: not a sequence of this context");
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  cudaGraphExecDestroy(seq->exec);
  seq->magic = 0;
  delete seq;
  if (--ctx->live_sequences == 0) {
    for (void* r : ctx->retired) cudaFree(r);
    ctx->retired.clear();
  }
  return PRAD_OK;
}

}  // extern "C"
