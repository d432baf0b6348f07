// Context, pooled device memory, copies, sync, graphs and events.
// Stands in for the device/queue/pool half of WebGPUBackend (src/backend/webgpu.ts:214-262, 406-576,
// 764-777, 1465-1503).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

static std::string g_init_error;

gt_status gt_fail(gt_ctx* ctx, gt_status code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf; else g_init_error = buf;
  return code;
}

gt_status gt_check_cuda(gt_ctx* ctx, cudaError_t e, const char* what) {
  if (e == cudaSuccess) return GT_OK;
  gt_status code = (e == cudaErrorMemoryAllocation) ? GT_ERR_OOM : GT_ERR_CUDA;
  return gt_fail(ctx, code, "CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
}

gt_status gt_scratch(gt_ctx* ctx, uint64_t bytes, float** out) {
  if (bytes > ctx->scratch_bytes) {
    if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "scratch growth to %llu bytes inside a graph capture; run the step once eagerly first", (unsigned long long)bytes);
    // the old block may still be read by queued kernels: drain first
    GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) cudaFree(ctx->scratch);
    ctx->scratch = nullptr;
    uint64_t want = bytes < (8u << 20) ? (8u << 20) : bytes;
    GT_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
  }
  *out = ctx->scratch;
  return GT_OK;
}

extern "C" {

gt_status gt_init(int32_t device, gt_ctx** out) {
  if (!out) return gt_fail(nullptr, GT_ERR_ARG, "gt_init: out is null");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return gt_fail(nullptr, GT_ERR_CUDA, "no GPU adapter found (%s)", e == cudaSuccess ? "0 devices" : cudaGetErrorString(e));
  if (device < 0 || device >= n) return gt_fail(nullptr, GT_ERR_ARG, "gt_init: device %d of %d", device, n);
  e = cudaSetDevice(device);
  if (e != cudaSuccess) return gt_fail(nullptr, GT_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  gt_ctx* ctx = new gt_ctx();
  ctx->device = device;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) ctx->sm_count = prop.multiProcessorCount;
  e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete ctx;
    return gt_fail(nullptr, GT_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e));
  }
  *out = ctx;
  return GT_OK;
}

gt_status gt_destroy(gt_ctx* ctx) {
  if (!ctx) return GT_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  gt_dp_teardown(ctx);
  gt_optim_destroy(ctx);
  for (auto g : ctx->graphs) if (g) cudaGraphExecDestroy(g);
  for (auto& kv : ctx->free_lists) for (void* p : kv.second) cudaFree(p);
  for (auto& kv : ctx->live) cudaFree(kv.first);
  for (auto& kv : ctx->state) cudaFree(kv.first);
  for (auto& kv : ctx->rope_tables) cudaFree(kv.second);
  for (auto ev : ctx->events) if (ev) cudaEventDestroy(ev);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return GT_OK;
}

const char* gt_last_error(gt_ctx* ctx) { return ctx ? ctx->err.c_str() : g_init_error.c_str(); }

gt_status gt_device_name(gt_ctx* ctx, char* out, int32_t cap) {
  cudaDeviceProp prop;
  GT_CUDA(ctx, cudaGetDeviceProperties(&prop, ctx->device));
  snprintf(out, cap, "%s (sm_%d%d, %d SMs)", prop.name, prop.major, prop.minor, prop.multiProcessorCount);
  return GT_OK;
}

gt_status gt_set_precision(gt_ctx* ctx, int32_t mode) {
  GT_REQUIRE(ctx, mode >= GT_PREC_FP32 && mode <= GT_PREC_BF16, "gt_set_precision: unknown mode %d", mode);
  ctx->precision = mode;
  return GT_OK;
}

gt_status gt_set_batch(gt_ctx* ctx, int32_t batch, int32_t seq_len) {
  GT_REQUIRE(ctx, batch >= 0 && (batch == 0 || seq_len > 0), "gt_set_batch: batch %d seq_len %d", batch, seq_len);
  ctx->batch = batch;
  ctx->seq_len = batch ? seq_len : 0;
  return GT_OK;
}

static uint64_t bucket(uint64_t bytes) { return bytes < 256 ? 256 : (bytes + 255) / 256 * 256; }

gt_status gt_alloc(gt_ctx* ctx, uint64_t bytes, gt_buf* out) {
  uint64_t size = bucket(bytes);
  auto it = ctx->free_lists.find(size);
  void* p = nullptr;
  if (it != ctx->free_lists.end() && !it->second.empty()) {
    p = it->second.back();
    it->second.pop_back();
  } else {
    if (ctx->capturing)
      return gt_fail(ctx, GT_ERR_STATE, "gt_alloc of %llu bytes missed the pool inside a graph capture; run the same step once eagerly first", (unsigned long long)size);
    cudaError_t e = cudaMalloc(&p, size);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return gt_fail(ctx, GT_ERR_OOM, "device allocation of %llu bytes failed (%s); %llu bytes already pooled. Lower the batch or sequence length, or use recompute.",
                     (unsigned long long)size, cudaGetErrorString(e), (unsigned long long)ctx->pool_bytes);
    }
    ctx->pool_bytes += size;
  }
  ctx->live[p] = size;
  *out = (gt_buf)(uintptr_t)p;
  return GT_OK;
}

gt_status gt_alloc_state(gt_ctx* ctx, uint64_t bytes, gt_buf* out) {
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_alloc_state inside a graph capture");
  uint64_t size = bucket(bytes);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, size);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return gt_fail(ctx, GT_ERR_OOM, "state allocation of %llu bytes failed (%s)", (unsigned long long)size, cudaGetErrorString(e));
  }
  GT_CUDA(ctx, cudaMemsetAsync(p, 0, size, ctx->stream));
  ctx->state[p] = size;
  ctx->state_bytes += size;
  *out = (gt_buf)(uintptr_t)p;
  return GT_OK;
}

gt_status gt_free(gt_ctx* ctx, gt_buf buf) {
  void* p = gt_ptr<void>(buf);
  auto it = ctx->live.find(p);
  if (it == ctx->live.end()) {
    auto st = ctx->state.find(p);
    if (st == ctx->state.end()) return gt_fail(ctx, GT_ERR_ARG, "gt_free: %p is not a live allocation of this context", p);
    // state buffers are not pooled; stream order makes the free safe
    GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(p);
    ctx->state_bytes -= st->second;
    ctx->state.erase(st);
    return GT_OK;
  }
  // Work that still reads the block is already queued on the one stream every later user
  // is queued on too, so handing it out again needs no fence (the ordering argument at
  // webgpu.ts:507-563).
  ctx->free_lists[it->second].push_back(p);
  ctx->live.erase(it);
  return GT_OK;
}

static gt_status ensure_pinned(gt_ctx* ctx, uint64_t bytes) {
  if (bytes <= ctx->pinned_bytes) return GT_OK;
  GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  ctx->pinned = nullptr;
  ctx->pinned_bytes = 0;
  uint64_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
  GT_CUDA(ctx, cudaMallocHost(&ctx->pinned, want));
  ctx->pinned_bytes = want;
  return GT_OK;
}

gt_status gt_write(gt_ctx* ctx, gt_buf dst, const void* host, uint64_t bytes) {
  if (bytes == 0) return GT_OK;
  GT_REQUIRE(ctx, dst && host, "gt_write: null argument");
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_write inside a graph capture: write the inputs before gt_graph_launch instead");
  // The host array is only borrowed for this call: small writes go through pinned staging and
  // stay asynchronous; large ones (weight uploads) copy synchronously from pageable memory.
  if (bytes <= (4u << 20)) {
    // the staging block may still be the source of an earlier queued copy
    gt_status s = ensure_pinned(ctx, 8u << 20);
    if (s) return s;
    uint64_t& cursor = ctx->pinned_cursor;
    if (cursor + bytes > ctx->pinned_bytes) {
      GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      cursor = 0;
    }
    char* stage = (char*)ctx->pinned + cursor;
    memcpy(stage, host, bytes);
    cursor += (bytes + 255) / 256 * 256;
    GT_CUDA(ctx, cudaMemcpyAsync(gt_ptr<void>(dst), stage, bytes, cudaMemcpyHostToDevice, ctx->stream));
  } else {
    GT_CUDA(ctx, cudaMemcpyAsync(gt_ptr<void>(dst), host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  return GT_OK;
}

gt_status gt_read(gt_ctx* ctx, gt_buf src, void* host, uint64_t bytes) {
  if (bytes == 0) return GT_OK;
  GT_REQUIRE(ctx, src && host, "gt_read: null argument");
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_read inside a graph capture");
  GT_CUDA(ctx, cudaMemcpyAsync(host, gt_ptr<void>(src), bytes, cudaMemcpyDeviceToHost, ctx->stream));
  GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->readback_bytes += bytes;
  return GT_OK;
}

gt_status gt_zero(gt_ctx* ctx, gt_buf buf, uint64_t bytes) {
  if (bytes == 0) return GT_OK;
  GT_CUDA(ctx, cudaMemsetAsync(gt_ptr<void>(buf), 0, bytes, ctx->stream));
  return GT_OK;
}

gt_status gt_copy(gt_ctx* ctx, gt_buf dst, gt_buf src, uint64_t bytes) {
  if (bytes == 0) return GT_OK;
  GT_CUDA(ctx, cudaMemcpyAsync(gt_ptr<void>(dst), gt_ptr<void>(src), bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return GT_OK;
}

gt_status gt_sync(gt_ctx* ctx) {
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_sync inside a graph capture");
  GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return gt_check_cuda(ctx, e, "gt_sync (latched)");
  ctx->readback_bytes = 0;
  gt_status ts = gt_gemm_tc_check(ctx);
  if (ts) return ts;
  return GT_OK;
}

gt_status gt_stats(gt_ctx* ctx, uint64_t* out4) {
  out4[0] = ctx->pool_bytes;
  out4[1] = ctx->state_bytes;
  out4[2] = ctx->readback_bytes;
  out4[3] = ctx->launches;
  return GT_OK;
}

// ---- graphs ----
gt_status gt_graph_begin(gt_ctx* ctx) {
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_graph_begin: already capturing");
  GT_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  ctx->capturing = true;
  return GT_OK;
}

gt_status gt_graph_end(gt_ctx* ctx, uint64_t* out_graph) {
  if (!ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_graph_end: not capturing");
  ctx->capturing = false;
  cudaGraph_t g = nullptr;
  GT_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &g));
  cudaGraphExec_t ex = nullptr;
  cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return gt_check_cuda(ctx, e, "cudaGraphInstantiate");
  ctx->graphs.push_back(ex);
  *out_graph = ctx->graphs.size();  // 1-based handle
  return GT_OK;
}

gt_status gt_graph_launch(gt_ctx* ctx, uint64_t graph) {
  GT_REQUIRE(ctx, graph >= 1 && graph <= ctx->graphs.size() && ctx->graphs[graph - 1], "gt_graph_launch: bad handle %llu", (unsigned long long)graph);
  GT_CUDA(ctx, cudaGraphLaunch(ctx->graphs[graph - 1], ctx->stream));
  return GT_OK;
}

gt_status gt_graph_destroy(gt_ctx* ctx, uint64_t graph) {
  GT_REQUIRE(ctx, graph >= 1 && graph <= ctx->graphs.size() && ctx->graphs[graph - 1], "gt_graph_destroy: bad handle %llu", (unsigned long long)graph);
  GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  cudaGraphExecDestroy(ctx->graphs[graph - 1]);
  ctx->graphs[graph - 1] = nullptr;
  return GT_OK;
}

// ---- events ----
gt_status gt_event_record(gt_ctx* ctx, int32_t slot) {
  GT_REQUIRE(ctx, slot >= 0 && slot < 64, "gt_event_record: slot %d", slot);
  if (!ctx->events[slot]) GT_CUDA(ctx, cudaEventCreate(&ctx->events[slot]));
  GT_CUDA(ctx, cudaEventRecord(ctx->events[slot], ctx->stream));
  return GT_OK;
}

gt_status gt_event_elapsed_ms(gt_ctx* ctx, int32_t a, int32_t b, float* ms) {
  GT_REQUIRE(ctx, a >= 0 && a < 64 && b >= 0 && b < 64 && ctx->events[a] && ctx->events[b], "gt_event_elapsed_ms: slots %d,%d not recorded", a, b);
  GT_CUDA(ctx, cudaEventSynchronize(ctx->events[b]));
  GT_CUDA(ctx, cudaEventElapsedTime(ms, ctx->events[a], ctx->events[b]));
  return GT_OK;
}

}  // extern "C"
