// Data-parallel gradient reduction over NCCL (NVLink 5 / NVSwitch). The reference is single-device
// (no collective anywhere); this is the one exchange step data parallelism adds: an f32 sum of the
// gradient arena across ranks, issued per bucket on a side stream so it overlaps the rest of backward.
// NCCL is resolved at run time (dlopen) so single-GPU users never need it.
#include <dlfcn.h>
#include <string.h>
#include <time.h>

#include "common.cuh"

namespace {
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
struct Nccl {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
};
Nccl g_nccl;
std::string g_nccl_err;

bool load_nccl() {
  if (g_nccl.lib) return true;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) { h = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (h) break; }
  if (!h) { g_nccl_err = std::string("cannot load libnccl.so.2: ") + dlerror(); return false; }
#define SYM(field, name) *(void**)(&g_nccl.field) = dlsym(h, name); if (!g_nccl.field) { g_nccl_err = "libnccl lacks " name; return false; }
  SYM(GetUniqueId, "ncclGetUniqueId") SYM(CommInitRank, "ncclCommInitRank") SYM(AllReduce, "ncclAllReduce") SYM(AllGather, "ncclAllGather")
  SYM(CommDestroy, "ncclCommDestroy") SYM(CommAbort, "ncclCommAbort") SYM(GetErrorString, "ncclGetErrorString")
  SYM(CommGetAsyncError, "ncclCommGetAsyncError")
#undef SYM
  g_nccl.lib = h;
  return true;
}
}  // namespace

struct GtDp {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t stream = nullptr;
  cudaEvent_t ready = nullptr, done = nullptr;
  bool pending = false;
};

void gt_dp_teardown(gt_ctx* ctx) {
  if (!ctx->dp) return;
  GtDp* d = ctx->dp;
  if (d->stream) cudaStreamSynchronize(d->stream);
  if (d->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(d->comm);
  if (d->ready) cudaEventDestroy(d->ready);
  if (d->done) cudaEventDestroy(d->done);
  if (d->stream) cudaStreamDestroy(d->stream);
  delete d;
  ctx->dp = nullptr;
}

gt_status gt_dp_rank(gt_ctx* ctx, int* rank, int* world) {
  if (!ctx->dp) return gt_fail(ctx, GT_ERR_STATE, "no communicator: gt_dp_init has not run");
  *rank = ctx->dp->rank;
  *world = ctx->dp->world;
  return GT_OK;
}

gt_status gt_dp_allgather(gt_ctx* ctx, float* buf, size_t count) {
  GtDp* d = ctx->dp;
  if (!d || !d->comm) return gt_fail(ctx, GT_ERR_STATE, "gt_dp_allgather: no communicator");
  ncclResult_t r = g_nccl.AllGather(buf + (size_t)d->rank * count, buf, count, /*ncclFloat32*/ 7, d->comm, ctx->stream);
  if (r != 0) return gt_fail(ctx, GT_ERR_NCCL, "ncclAllGather: %s", g_nccl.GetErrorString(r));
  return GT_OK;
}

extern "C" {

gt_status gt_dp_unique_id(uint8_t* out128) {
  if (!out128) return gt_fail(nullptr, GT_ERR_ARG, "gt_dp_unique_id: null output");
  if (!load_nccl()) return gt_fail(nullptr, GT_ERR_NCCL, "%s", g_nccl_err.c_str());
  ncclUniqueId id;
  ncclResult_t r = g_nccl.GetUniqueId(&id);
  if (r != 0) return gt_fail(nullptr, GT_ERR_NCCL, "ncclGetUniqueId: %s", g_nccl.GetErrorString(r));
  memcpy(out128, &id, 128);
  return GT_OK;
}

gt_status gt_dp_init(gt_ctx* ctx, int32_t rank, int32_t world, const uint8_t* id128) {
  GT_REQUIRE(ctx, world >= 1 && rank >= 0 && rank < world && id128, "gt_dp_init: rank %d of %d", rank, world);
  if (ctx->dp) return gt_fail(ctx, GT_ERR_STATE, "gt_dp_init: already initialised");
  if (!load_nccl()) return gt_fail(ctx, GT_ERR_NCCL, "%s", g_nccl_err.c_str());
  GtDp* d = new GtDp();
  d->rank = rank; d->world = world;
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  GT_CUDA(ctx, cudaSetDevice(ctx->device));
  ncclResult_t r = g_nccl.CommInitRank(&d->comm, world, id, rank);
  if (r != 0) { delete d; return gt_fail(ctx, GT_ERR_NCCL, "ncclCommInitRank(rank %d of %d): %s", rank, world, g_nccl.GetErrorString(r)); }
  GT_CUDA(ctx, cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  GT_CUDA(ctx, cudaEventCreateWithFlags(&d->ready, cudaEventDisableTiming));
  GT_CUDA(ctx, cudaEventCreateWithFlags(&d->done, cudaEventDisableTiming));
  ctx->dp = d;
  return GT_OK;
}

gt_status gt_dp_allreduce_start(gt_ctx* ctx, gt_buf buf, uint64_t count) {
  GtDp* d = ctx->dp;
  if (!d) return gt_fail(ctx, GT_ERR_STATE, "gt_dp_allreduce_start: gt_dp_init has not run");
  if (!d->comm) return gt_fail(ctx, GT_ERR_NCCL, "gt_dp_allreduce_start: the communicator was aborted; gt_dp_destroy and gt_dp_init again");
  if (count == 0) return GT_OK;
  GT_REQUIRE(ctx, buf, "gt_dp_allreduce_start: null buffer");
  GT_CUDA(ctx, cudaEventRecord(d->ready, ctx->stream));
  GT_CUDA(ctx, cudaStreamWaitEvent(d->stream, d->ready, 0));
  ncclResult_t r = g_nccl.AllReduce(gt_ptr<void>(buf), gt_ptr<void>(buf), count, /*ncclFloat32*/ 7, /*ncclSum*/ 0, d->comm, d->stream);
  if (r != 0) return gt_fail(ctx, GT_ERR_NCCL, "ncclAllReduce: %s", g_nccl.GetErrorString(r));
  d->pending = true;
  return GT_OK;
}

gt_status gt_dp_wait(gt_ctx* ctx) {
  GtDp* d = ctx->dp;
  if (!d) return gt_fail(ctx, GT_ERR_STATE, "gt_dp_wait: gt_dp_init has not run");
  if (!d->pending) return GT_OK;
  GT_CUDA(ctx, cudaEventRecord(d->done, d->stream));
  GT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, d->done, 0));
  d->pending = false;
  ncclResult_t async = 0;
  if (d->comm && g_nccl.CommGetAsyncError(d->comm, &async) == 0 && async != 0 && async != 7 /* ncclInProgress */)
    return gt_fail(ctx, GT_ERR_NCCL, "NCCL asynchronous error: %s", g_nccl.GetErrorString(async));
  return GT_OK;
}

// Host-side form of the wait, for callers that want to know that the exchange completed (or did not) before they
// launch anything else: polls the last reduction's completion and the communicator's asynchronous error state for at
// most timeout_ms. On expiry or on an NCCL error the communicator is aborted (ncclCommAbort ends its kernels, which
// otherwise wait for the missing rank for ever) and the status is GT_ERR_NCCL; the context itself stays usable for
// single-GPU work and gt_dp_init may be called again after gt_dp_destroy.
gt_status gt_dp_wait_host(gt_ctx* ctx, int32_t timeout_ms) {
  GtDp* d = ctx->dp;
  if (!d) return gt_fail(ctx, GT_ERR_STATE, "gt_dp_wait_host: gt_dp_init has not run");
  GT_REQUIRE(ctx, timeout_ms > 0, "gt_dp_wait_host: timeout %d ms", timeout_ms);
  if (!d->comm) return gt_fail(ctx, GT_ERR_NCCL, "gt_dp_wait_host: the communicator was aborted");
  if (d->pending) {
    gt_status s = gt_dp_wait(ctx);
    if (s) return s;
  }
  cudaEvent_t ev = d->done;
  GT_CUDA(ctx, cudaEventRecord(ev, d->stream));
  timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  for (;;) {
    cudaError_t q = cudaEventQuery(ev);
    if (q == cudaSuccess) return GT_OK;
    if (q != cudaErrorNotReady) return gt_check_cuda(ctx, q, "gt_dp_wait_host");
    ncclResult_t async = 0;
    const bool bad = g_nccl.CommGetAsyncError(d->comm, &async) == 0 && async != 0 && async != 7 /* ncclInProgress */;
    timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const double ms = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) / 1e6;
    if (bad || ms > timeout_ms) {
      g_nccl.CommAbort(d->comm);
      d->comm = nullptr;
      if (bad) return gt_fail(ctx, GT_ERR_NCCL, "NCCL asynchronous error: %s; communicator aborted", g_nccl.GetErrorString(async));
      return gt_fail(ctx, GT_ERR_NCCL, "gradient exchange did not complete within %d ms (a rank is missing or stuck); communicator aborted", timeout_ms);
    }
    timespec nap = {0, 200000};
    nanosleep(&nap, nullptr);
  }
}

// While a reduction runs beside compute, its kernel holds a few SMs. A persistent kernel that still launches one CTA
// per SM of the whole device then has CTAs that only start when others finish: its last wave doubles. Reserving those
// SMs makes the persistent matrix-product kernels size their grids (and choose their tiles) for what is left.
gt_status gt_dp_reserve_sms(gt_ctx* ctx, int32_t n) {
  GT_REQUIRE(ctx, n >= 0 && n < ctx->sm_count, "gt_dp_reserve_sms: %d of %d SMs", n, ctx->sm_count);
  ctx->sm_reserved = n;
  return GT_OK;
}

gt_status gt_dp_destroy(gt_ctx* ctx) {
  gt_dp_teardown(ctx);
  return GT_OK;
}

}  // extern "C"
