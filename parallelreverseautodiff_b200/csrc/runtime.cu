// Runtime services around the kernels: intermediate slots keyed by Guid (the device form of the
// managed Store/Restore pair), packed download / upload of many tensors (what SaveWeightsAndMoments
// needs), device introspection and CUDA-event timing brackets.
#include <array>
#include <cstring>
#include <map>
#include <mutex>

#include "common.cuh"

namespace prad {

using Guid = std::array<uint8_t, 16>;

struct Slot {
  std::vector<void*> ptrs;      // what Restore hands back
  std::vector<size_t> bytes;
  bool owns = false;            // copies made by the store (freed when the slot is dropped)
};

struct TimingBracket {
  char label[48];
  cudaEvent_t begin = nullptr, end = nullptr;
  int64_t launches0 = 0, launches1 = 0;
  bool closed = false;
};

// per-context runtime state; lives in a side table so that the context struct stays plain
struct RuntimeState {
  std::map<Guid, Slot> slots;
  std::vector<TimingBracket> brackets;
  int open_bracket = -1;
};

static std::mutex g_rt_mu;
static std::map<prad_ctx*, RuntimeState*> g_rt;

static RuntimeState* rt_of(prad_ctx* ctx) {
  std::lock_guard<std::mutex> lock(g_rt_mu);
  auto it = g_rt.find(ctx);
  if (it != g_rt.end()) return it->second;
  RuntimeState* r = new RuntimeState();
  g_rt[ctx] = r;
  return r;
}

static void free_slot(Slot& s) {
  if (s.owns)
    for (void* p : s.ptrs)
      if (p) cudaFree(p);
  s.ptrs.clear();
  s.bytes.clear();
}

static void free_brackets(RuntimeState* r) {
  for (TimingBracket& b : r->brackets) {
    if (b.begin) cudaEventDestroy(b.begin);
    if (b.end) cudaEventDestroy(b.end);
  }
  r->brackets.clear();
  r->open_bracket = -1;
}

// called by prad_shutdown
void runtime_destroy(prad_ctx* ctx) {
  RuntimeState* r = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_rt_mu);
    auto it = g_rt.find(ctx);
    if (it == g_rt.end()) return;
    r = it->second;
    g_rt.erase(it);
  }
  for (auto& kv : r->slots) free_slot(kv.second);
  free_brackets(r);
  delete r;
}

static Guid guid_of(const void* p) {
  Guid g;
  memcpy(g.data(), p, 16);
  return g;
}

}  // namespace prad

using namespace prad;

extern "C" {

// ---------------------------------------------------------------- intermediate slots
prad_status prad_slot_store(prad_ctx* ctx, const void* guid_16_bytes, const void* const* ptrs_host,
                            const size_t* bytes_host, int count, int copy) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(guid_16_bytes && count >= 0 && (count == 0 || (ptrs_host && bytes_host)), PRAD_ERR_INVALID,
               "prad_slot_store: null guid or pointer list");
  if (copy) PRAD_NOT_CAPTURING(ctx, "prad_slot_store with copies");
  RuntimeState* r = rt_of(ctx);
  Slot fresh;
  fresh.owns = copy != 0;
  for (int i = 0; i < count; ++i) {
    void* p = const_cast<void*>(ptrs_host[i]);
    if (copy && p && bytes_host[i]) {
      void* q = nullptr;
      cudaError_t e = cudaMalloc(&q, bytes_host[i]);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        free_slot(fresh);
        set_error("prad_slot_store: copy of %zu bytes could not be allocated: %s", bytes_host[i], cudaGetErrorString(e));
        return PRAD_ERR_OOM;
      }
      fresh.ptrs.push_back(q);
      fresh.bytes.push_back(bytes_host[i]);
      e = cudaMemcpyAsync(q, p, bytes_host[i], cudaMemcpyDeviceToDevice, ctx->stream);
      if (e != cudaSuccess) {
        free_slot(fresh);
        set_error("prad_slot_store: device copy failed: %s", cudaGetErrorString(e));
        return PRAD_ERR_CUDA;
      }
    } else {
      fresh.ptrs.push_back(copy ? nullptr : p);
      fresh.bytes.push_back(bytes_host[i]);
    }
  }
  // AddOrUpdate: a second store under the same id replaces the first
  auto it = r->slots.find(guid_of(guid_16_bytes));
  if (it != r->slots.end()) {
    if (it->second.owns) PRAD_CUDA(cudaStreamSynchronize(ctx->stream));   // a kernel may still read the old copies
    free_slot(it->second);
    it->second = std::move(fresh);
  } else {
    r->slots.emplace(guid_of(guid_16_bytes), std::move(fresh));
  }
  return PRAD_OK;
}

prad_status prad_slot_restore(prad_ctx* ctx, const void* guid_16_bytes, void** out_ptrs_host, int count) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(guid_16_bytes && count >= 0 && (count == 0 || out_ptrs_host), PRAD_ERR_INVALID,
               "prad_slot_restore: null guid or output list");
  RuntimeState* r = rt_of(ctx);
  auto it = r->slots.find(guid_of(guid_16_bytes));
  PRAD_REQUIRE(it != r->slots.end(), PRAD_ERR_INVALID,
               "prad_slot_restore: nothing was stored under this id (KeyNotFoundException)");
  PRAD_REQUIRE((int)it->second.ptrs.size() == count, PRAD_ERR_SHAPE,
               "prad_slot_restore: the slot holds %d buffers, %d were asked for", (int)it->second.ptrs.size(), count);
  for (int i = 0; i < count; ++i) out_ptrs_host[i] = it->second.ptrs[i];
  return PRAD_OK;
}

prad_status prad_slot_drop(prad_ctx* ctx, const void* guid_16_bytes) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_slot_drop");
  PRAD_REQUIRE(guid_16_bytes, PRAD_ERR_INVALID, "prad_slot_drop: null guid");
  RuntimeState* r = rt_of(ctx);
  auto it = r->slots.find(guid_of(guid_16_bytes));
  if (it == r->slots.end()) return PRAD_OK;
  if (it->second.owns) PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  free_slot(it->second);
  r->slots.erase(it);
  return PRAD_OK;
}

prad_status prad_slot_count(prad_ctx* ctx, int* out_count) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(out_count, PRAD_ERR_INVALID, "prad_slot_count: null output");
  *out_count = (int)rt_of(ctx)->slots.size();
  return PRAD_OK;
}

// ---------------------------------------------------------------- packed transfers
prad_status prad_download_many(prad_ctx* ctx, void* dst_host, const void* const* srcs_host, const size_t* bytes_host,
                               int count) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_download_many");
  PRAD_REQUIRE(count >= 0 && (count == 0 || (dst_host && srcs_host && bytes_host)), PRAD_ERR_INVALID,
               "prad_download_many: null pointer");
  char* out = (char*)dst_host;
  for (int i = 0; i < count; ++i) {
    PRAD_REQUIRE(srcs_host[i] || bytes_host[i] == 0, PRAD_ERR_INVALID, "prad_download_many: tensor %d is null", i);
    if (bytes_host[i]) PRAD_CUDA(cudaMemcpyAsync(out, srcs_host[i], bytes_host[i], cudaMemcpyDeviceToHost, ctx->stream));
    out += bytes_host[i];
  }
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  return gemm_tf32x3_check(ctx);
}

prad_status prad_upload_many(prad_ctx* ctx, void* const* dsts_host, const void* src_host, const size_t* bytes_host,
                             int count) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_upload_many");
  PRAD_REQUIRE(count >= 0 && (count == 0 || (dsts_host && src_host && bytes_host)), PRAD_ERR_INVALID,
               "prad_upload_many: null pointer");
  const char* in = (const char*)src_host;
  for (int i = 0; i < count; ++i) {
    PRAD_REQUIRE(dsts_host[i] || bytes_host[i] == 0, PRAD_ERR_INVALID, "prad_upload_many: tensor %d is null", i);
    if (bytes_host[i]) PRAD_CUDA(cudaMemcpyAsync(dsts_host[i], in, bytes_host[i], cudaMemcpyHostToDevice, ctx->stream));
    in += bytes_host[i];
  }
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));   // the host block may be reused when the call returns
  return PRAD_OK;
}

// ---------------------------------------------------------------- introspection
prad_status prad_device_info(prad_ctx* ctx, prad_device_info_t* out) {
  PRAD_CHECK_CTX(ctx);
  PRAD_REQUIRE(out, PRAD_ERR_INVALID, "prad_device_info: null output");
  memset(out, 0, sizeof(*out));
  cudaDeviceProp p;
  PRAD_CUDA(cudaGetDeviceProperties(&p, ctx->device));
  size_t free_b = 0, total_b = 0;
  PRAD_CUDA(cudaMemGetInfo(&free_b, &total_b));
  out->device = ctx->device;
  out->sm_count = p.multiProcessorCount;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->l2_bytes = p.l2CacheSize;
  out->smem_per_block_optin = (int)p.sharedMemPerBlockOptin;
  int khz = 0;
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device) == cudaSuccess) out->sm_clock_khz = khz;
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrMemoryClockRate, ctx->device) == cudaSuccess) out->mem_clock_khz = khz;
  (void)cudaGetLastError();
  out->total_bytes = (uint64_t)total_b;
  out->free_bytes = (uint64_t)free_b;
  out->scratch_bytes = (uint64_t)(ctx->ws_bytes + ctx->stage_bytes);
  strncpy(out->name, p.name, sizeof(out->name) - 1);
  return PRAD_OK;
}

prad_status prad_timing_begin(prad_ctx* ctx, const char* label) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_timing_begin");
  RuntimeState* r = rt_of(ctx);
  PRAD_REQUIRE(r->open_bracket < 0, PRAD_ERR_INVALID, "prad_timing_begin: the previous bracket is still open");
  PRAD_REQUIRE(r->brackets.size() < 65536, PRAD_ERR_UNSUPPORTED,
               "prad_timing_begin: 65536 brackets are pending; read them with prad_get_timings");
  TimingBracket b;
  memset(b.label, 0, sizeof(b.label));
  if (label) strncpy(b.label, label, sizeof(b.label) - 1);
  PRAD_CUDA(cudaEventCreate(&b.begin));
  cudaError_t e = cudaEventCreate(&b.end);
  if (e != cudaSuccess) { cudaEventDestroy(b.begin); set_error("prad_timing_begin: %s", cudaGetErrorString(e)); return PRAD_ERR_CUDA; }
  b.launches0 = ctx->launches;
  e = cudaEventRecord(b.begin, ctx->stream);
  if (e != cudaSuccess) {
    cudaEventDestroy(b.begin); cudaEventDestroy(b.end);
    set_error("prad_timing_begin: %s", cudaGetErrorString(e));
    return PRAD_ERR_CUDA;
  }
  r->brackets.push_back(b);
  r->open_bracket = (int)r->brackets.size() - 1;
  return PRAD_OK;
}

prad_status prad_timing_end(prad_ctx* ctx) {
  PRAD_CHECK_CTX(ctx);
  RuntimeState* r = rt_of(ctx);
  PRAD_REQUIRE(r->open_bracket >= 0, PRAD_ERR_INVALID, "prad_timing_end: no bracket is open");
  TimingBracket& b = r->brackets[r->open_bracket];
  PRAD_CUDA(cudaEventRecord(b.end, ctx->stream));
  b.launches1 = ctx->launches;
  b.closed = true;
  r->open_bracket = -1;
  return PRAD_OK;
}

prad_status prad_get_timings(prad_ctx* ctx, prad_timing_t* out, int capacity, int* out_count) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_get_timings");
  PRAD_REQUIRE(out_count && capacity >= 0 && (capacity == 0 || out), PRAD_ERR_INVALID, "prad_get_timings: bad argument");
  RuntimeState* r = rt_of(ctx);
  PRAD_REQUIRE(r->open_bracket < 0, PRAD_ERR_INVALID, "prad_get_timings: a bracket is still open");
  PRAD_CUDA(cudaStreamSynchronize(ctx->stream));
  const int n = (int)r->brackets.size();
  *out_count = n;
  for (int i = 0; i < n && i < capacity; ++i) {
    TimingBracket& b = r->brackets[i];
    float ms = 0.f;
    PRAD_CUDA(cudaEventElapsedTime(&ms, b.begin, b.end));
    memset(&out[i], 0, sizeof(out[i]));
    memcpy(out[i].label, b.label, sizeof(out[i].label));
    out[i].milliseconds = (double)ms;
    out[i].launches = b.launches1 - b.launches0;
  }
  if (capacity >= n) free_brackets(r);   // everything was handed over
  return gemm_tf32x3_check(ctx);
}

}  // extern "C"
