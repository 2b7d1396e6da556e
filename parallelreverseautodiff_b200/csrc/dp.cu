// Batch-sharded data parallelism: weight-gradient all-reduce over NCCL (NVLink 5 / NVSwitch),
// one process per GPU.  The reference has nothing like it (no multi-device code at all); the
// semantics follow from its single-device maths: a [batch x in] product sums weight gradients
// over rows, so shards are combined with SUM.
//
// The all-reduce runs on a second, high-priority stream.  prad_dp_allreduce records an event
// on the compute stream and makes the communication stream wait for it, so the collective of
// layer l overlaps with the backward kernels of layers l-1..0 that are enqueued afterwards;
// prad_dp_wait joins the two streams again before the optimiser reads the gradients.
//
// Sharded optimiser: prad_dp_reduce sends the sum of a gradient to ONE rank (its owner) instead of
// to all; the owner alone clips and updates that tensor (the reference's z-score clip needs only the
// tensor's own mean and sigma) and prad_dp_broadcast returns the new weights to everybody, on the
// communication stream, while the next step's first kernels already run.  Same bytes on the wire as an
// all-reduce, 1/N of the optimiser work and of the moment memory per rank.
//
// prad_dp_wait_host is the failure path: a host-side wait with a deadline (dp_deadline.h); when a peer
// never arrives the communicator is aborted and the call returns PRAD_ERR_TIMEOUT instead of hanging.
//
// NCCL is bound at run time with dlopen: the process may already hold the copy that ships
// with PyTorch, and the library must still load on a machine without NCCL (every prad_dp_*
// call then fails with PRAD_ERR_COMM; nothing else is affected).
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "common.cuh"
#include "dp_deadline.h"

namespace prad {

// Minimal NCCL surface (stable since NCCL 2.0).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;  // 0 = ncclSuccess
enum { ncclFloat32 = 7, ncclFloat64 = 8, ncclSum = 0 };

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Reduce)(const void*, void*, size_t, int, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
  std::string why;
};

static NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) {
      api.why = std::string("libnccl.so.2 could not be loaded: ") + (dlerror() ? dlerror() : "?");
      return;
    }
#define LOAD(field, sym)                                                        \
  api.field = (decltype(api.field))dlsym(api.handle, sym);                      \
  if (!api.field) { api.why = std::string("NCCL symbol missing: ") + sym; return; }
    LOAD(GetUniqueId, "ncclGetUniqueId")
    LOAD(CommInitRank, "ncclCommInitRank")
    LOAD(CommDestroy, "ncclCommDestroy")
    LOAD(CommAbort, "ncclCommAbort")
    LOAD(AllReduce, "ncclAllReduce")
    LOAD(Reduce, "ncclReduce")
    LOAD(Broadcast, "ncclBroadcast")
    LOAD(CommGetAsyncError, "ncclCommGetAsyncError")
    LOAD(GetErrorString, "ncclGetErrorString")
#undef LOAD
    api.ok = true;
  });
  return api;
}

struct DpState {
  ncclComm_t comm = nullptr;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ready = nullptr;  // compute -> comm
  cudaEvent_t done = nullptr;   // comm -> compute
  int rank = 0, world = 1;
  bool pending = false;
  bool aborted = false;         // the communicator was aborted after a deadline or an asynchronous error
  cudaEvent_t marks[PRAD_DP_MARKS] = {};   // prad_dp_mark: positions on the communication stream, created on first use
};

#define PRAD_NCCL(call)                                                                \
  do {                                                                                 \
    ncclResult_t r_ = (call);                                                          \
    if (r_ != 0) {                                                                     \
      set_error("%s failed: %s", #call, nccl().GetErrorString(r_));                    \
      return PRAD_ERR_COMM;                                                            \
    }                                                                                  \
  } while (0)

prad_status dp_destroy(prad_ctx* ctx) {
  DpState* d = ctx->dp;
  if (!d) return PRAD_OK;
  if (d->comm_stream && !d->aborted) cudaStreamSynchronize(d->comm_stream);
  if (d->comm && nccl().ok && !d->aborted) nccl().CommDestroy(d->comm);
  if (d->ready) cudaEventDestroy(d->ready);
  if (d->done) cudaEventDestroy(d->done);
  for (cudaEvent_t& m : d->marks)
    if (m) { cudaEventDestroy(m); m = nullptr; }
  if (d->comm_stream) cudaStreamDestroy(d->comm_stream);
  delete d;
  ctx->dp = nullptr;
  return PRAD_OK;
}

}  // namespace prad

using namespace prad;

extern "C" {

prad_status prad_dp_unique_id(void* out_id_128_bytes) {
  PRAD_REQUIRE(out_id_128_bytes, PRAD_ERR_INVALID, "prad_dp_unique_id: null output");
  PRAD_REQUIRE(nccl().ok, PRAD_ERR_COMM, "prad_dp_unique_id: %s", nccl().why.c_str());
  ncclUniqueId id;
  PRAD_NCCL(nccl().GetUniqueId(&id));
  memcpy(out_id_128_bytes, &id, sizeof(id));
  return PRAD_OK;
}

prad_status prad_dp_init(prad_ctx* ctx, const void* id_128_bytes, int rank, int world_size) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_init");
  PRAD_REQUIRE(id_128_bytes && world_size >= 1 && rank >= 0 && rank < world_size, PRAD_ERR_INVALID,
               "prad_dp_init: bad rank/world size or null id");
  PRAD_REQUIRE(nccl().ok, PRAD_ERR_COMM, "prad_dp_init: %s", nccl().why.c_str());
  PRAD_REQUIRE(ctx->dp == nullptr, PRAD_ERR_INVALID, "prad_dp_init: already initialised");
  DpState* d = new DpState();
  d->rank = rank;
  d->world = world_size;
  ctx->dp = d;
  // any failure below leaves the context as it was before the call, so that prad_dp_init can be retried
  auto body = [&]() -> prad_status {
    int lo = 0, hi = 0;
    PRAD_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    PRAD_CUDA(cudaStreamCreateWithPriority(&d->comm_stream, cudaStreamNonBlocking, hi));
    PRAD_CUDA(cudaEventCreateWithFlags(&d->ready, cudaEventDisableTiming));
    PRAD_CUDA(cudaEventCreateWithFlags(&d->done, cudaEventDisableTiming));
    ncclUniqueId id;
    memcpy(&id, id_128_bytes, sizeof(id));
    PRAD_NCCL(nccl().CommInitRank(&d->comm, world_size, id, rank));
    return PRAD_OK;
  };
  const prad_status st = body();
  if (st != PRAD_OK) dp_destroy(ctx);
  return st;
}

namespace prad {
// the communication stream picks up after everything enqueued so far on the compute stream
static prad_status comm_after_compute(prad_ctx* ctx) {
  DpState* d = ctx->dp;
  PRAD_CUDA(cudaEventRecord(d->ready, ctx->stream));
  PRAD_CUDA(cudaStreamWaitEvent(d->comm_stream, d->ready, 0));
  return PRAD_OK;
}
#define PRAD_DP_READY(ctx, who)                                                                              \
  PRAD_REQUIRE((ctx)->dp && (ctx)->dp->comm, PRAD_ERR_NOT_INITIALIZED, who ": call prad_dp_init first");     \
  PRAD_REQUIRE(!(ctx)->dp->aborted, PRAD_ERR_COMM, who ": the communicator was aborted after a failure; "    \
               "call prad_dp_shutdown and prad_dp_init again")
}  // namespace prad

prad_status prad_dp_reduce(prad_ctx* ctx, prad_dtype dt, void* buf, int64_t n, int root) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_reduce");
  PRAD_DP_READY(ctx, "prad_dp_reduce");
  DpState* d = ctx->dp;
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (buf || n == 0) && root >= 0 && root < d->world, PRAD_ERR_INVALID,
               "prad_dp_reduce: bad argument (root %d of %d ranks)", root, d->world);
  if (n == 0) return PRAD_OK;
  prad_status s = comm_after_compute(ctx);
  if (s) return s;
  PRAD_NCCL(nccl().Reduce(buf, buf, (size_t)n, dt == PRAD_F32 ? ncclFloat32 : ncclFloat64, ncclSum, root, d->comm,
                          d->comm_stream));
  d->pending = true;
  return PRAD_OK;
}

prad_status prad_dp_broadcast(prad_ctx* ctx, prad_dtype dt, void* buf, int64_t n, int root) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_broadcast");
  PRAD_DP_READY(ctx, "prad_dp_broadcast");
  DpState* d = ctx->dp;
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (buf || n == 0) && root >= 0 && root < d->world, PRAD_ERR_INVALID,
               "prad_dp_broadcast: bad argument (root %d of %d ranks)", root, d->world);
  if (n == 0) return PRAD_OK;
  prad_status s = comm_after_compute(ctx);
  if (s) return s;
  PRAD_NCCL(nccl().Broadcast(buf, buf, (size_t)n, dt == PRAD_F32 ? ncclFloat32 : ncclFloat64, root, d->comm,
                             d->comm_stream));
  d->pending = true;
  return PRAD_OK;
}

prad_status prad_dp_wait_host(prad_ctx* ctx, double timeout_ms) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_wait_host");
  PRAD_DP_READY(ctx, "prad_dp_wait_host");
  PRAD_REQUIRE(timeout_ms > 0, PRAD_ERR_INVALID, "prad_dp_wait_host: the deadline must be positive");
  DpState* d = ctx->dp;
  PRAD_CUDA(cudaEventRecord(d->done, d->comm_stream));
  cudaError_t query_failure = cudaSuccess;
  ncclResult_t async = 0;
  const WaitOutcome out = wait_with_deadline(
      [&] {
        const cudaError_t q = cudaEventQuery(d->done);
        if (q == cudaSuccess) return true;
        if (q != cudaErrorNotReady) { query_failure = q; (void)cudaGetLastError(); }
        return false;
      },
      [&] {
        if (query_failure != cudaSuccess) return true;
        ncclResult_t r = 0;
        if (nccl().CommGetAsyncError(d->comm, &r) != 0) return true;
        async = r;
        return r != 0;
      },
      [&] {
        nccl().CommAbort(d->comm);   // returns the ranks that did arrive from the collective
        d->aborted = true;
        d->pending = false;
      },
      timeout_ms);
  if (out == WaitOutcome::Done) {
    PRAD_CUDA(cudaStreamWaitEvent(ctx->stream, d->done, 0));
    d->pending = false;
    return PRAD_OK;
  }
  if (out == WaitOutcome::TimedOut) {
    set_error("prad_dp_wait_host: the collectives did not complete within %.0f ms (a rank never arrived?); "
              "the communicator was aborted", timeout_ms);
    return PRAD_ERR_TIMEOUT;
  }
  set_error("prad_dp_wait_host: %s; the communicator was aborted",
            query_failure != cudaSuccess ? cudaGetErrorString(query_failure)
                                         : (async ? nccl().GetErrorString(async) : "NCCL could not report its state"));
  return PRAD_ERR_COMM;
}

prad_status prad_dp_allreduce(prad_ctx* ctx, prad_dtype dt, void* buf, int64_t n) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_allreduce");
  PRAD_DP_READY(ctx, "prad_dp_allreduce");
  PRAD_REQUIRE(dtype_ok(dt) && n >= 0 && (buf || n == 0), PRAD_ERR_INVALID, "prad_dp_allreduce: bad argument");
  if (n == 0) return PRAD_OK;
  DpState* d = ctx->dp;
  PRAD_CUDA(cudaEventRecord(d->ready, ctx->stream));
  PRAD_CUDA(cudaStreamWaitEvent(d->comm_stream, d->ready, 0));
  PRAD_NCCL(nccl().AllReduce(buf, buf, (size_t)n, dt == PRAD_F32 ? ncclFloat32 : ncclFloat64, ncclSum,
                             d->comm, d->comm_stream));
  d->pending = true;
  return PRAD_OK;
}

prad_status prad_dp_wait(prad_ctx* ctx) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_wait");
  PRAD_DP_READY(ctx, "prad_dp_wait");
  DpState* d = ctx->dp;
  if (!d->pending) return PRAD_OK;
  PRAD_CUDA(cudaEventRecord(d->done, d->comm_stream));
  PRAD_CUDA(cudaStreamWaitEvent(ctx->stream, d->done, 0));
  d->pending = false;
  ncclResult_t async = 0;
  PRAD_NCCL(nccl().CommGetAsyncError(d->comm, &async));
  if (async != 0) {
    set_error("prad_dp_wait: NCCL reported an asynchronous error: %s", nccl().GetErrorString(async));
    return PRAD_ERR_COMM;
  }
  return PRAD_OK;
}

prad_status prad_dp_mark(prad_ctx* ctx, int slot) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_mark");
  PRAD_DP_READY(ctx, "prad_dp_mark");
  PRAD_REQUIRE(slot >= 0 && slot < PRAD_DP_MARKS, PRAD_ERR_INVALID, "prad_dp_mark: slot %d outside 0..%d", slot, PRAD_DP_MARKS - 1);
  DpState* d = ctx->dp;
  if (!d->marks[slot]) PRAD_CUDA(cudaEventCreateWithFlags(&d->marks[slot], cudaEventDisableTiming));
  PRAD_CUDA(cudaEventRecord(d->marks[slot], d->comm_stream));
  return PRAD_OK;
}

prad_status prad_dp_wait_mark(prad_ctx* ctx, int slot) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_wait_mark");
  PRAD_DP_READY(ctx, "prad_dp_wait_mark");
  PRAD_REQUIRE(slot >= 0 && slot < PRAD_DP_MARKS, PRAD_ERR_INVALID, "prad_dp_wait_mark: slot %d outside 0..%d", slot, PRAD_DP_MARKS - 1);
  DpState* d = ctx->dp;
  PRAD_REQUIRE(d->marks[slot], PRAD_ERR_INVALID, "prad_dp_wait_mark: slot %d was never marked", slot);
  PRAD_CUDA(cudaStreamWaitEvent(ctx->stream, d->marks[slot], 0));
  return PRAD_OK;
}

prad_status prad_dp_shutdown(prad_ctx* ctx) {
  PRAD_CHECK_CTX(ctx);
  PRAD_NOT_CAPTURING(ctx, "prad_dp_shutdown");
  return dp_destroy(ctx);
}

}  // extern "C"
