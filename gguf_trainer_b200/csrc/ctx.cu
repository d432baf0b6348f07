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
    // The old block may still be read by queued kernels, and every graph captured so far has its address recorded
    // in its kernel nodes: it is retired, not freed, and goes away with the context.
    if (ctx->scratch) ctx->retired_scratch.push_back(ctx->scratch);
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    uint64_t want = bytes < (8u << 20) ? (8u << 20) : bytes;
    GT_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
  }
  *out = ctx->scratch;
  return GT_OK;
}

int* gt_flags(gt_ctx* ctx) {
  if (!ctx->flags) {
    if (ctx->capturing) return nullptr;
    if (cudaMalloc(&ctx->flags, 256 * sizeof(int)) != cudaSuccess) { cudaGetLastError(); ctx->flags = nullptr; return nullptr; }
    cudaMemsetAsync(ctx->flags, 0, 256 * sizeof(int), ctx->stream);
  }
  return ctx->flags;
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
  for (auto& kv : ctx->attn_orders) cudaFree(kv.second);
  for (auto ev : ctx->events) if (ev) cudaEventDestroy(ev);
  if (ctx->scratch) cudaFree(ctx->scratch);
  for (float* p : ctx->retired_scratch) cudaFree(p);
  if (ctx->pinned) cudaFreeHost(ctx->pinned);
  if (ctx->flags) cudaFree(ctx->flags);
  if (ctx->copy_stream) cudaStreamSynchronize(ctx->copy_stream);
  for (auto& kv : ctx->async_reads) { cudaFreeHost(kv.second.pinned); cudaEventDestroy(kv.second.done); }
  for (auto& kv : ctx->pinned_free) cudaFreeHost(kv.second);
  if (ctx->copy_fork) cudaEventDestroy(ctx->copy_fork);
  if (ctx->copy_done) cudaEventDestroy(ctx->copy_done);
  if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
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
  if (mode == GT_PREC_BF16)
    return gt_fail(ctx, GT_ERR_UNSUPPORTED, "gt_set_precision: there are no BF16 kernels in this library (a single BF16 product is 1.6e-3 off in "
                   "relative L2, which leaves no room under the 2e-3 bound of a whole step); use GT_PREC_TF32 or GT_PREC_FP32");
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
  if (ctx->flags) {
    int h = 0;
    GT_CUDA(ctx, cudaMemcpyAsync(&h, ctx->flags + GT_FLAG_WINDOW, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (h != 0) {
      cudaMemsetAsync(ctx->flags + GT_FLAG_WINDOW, 0, sizeof(int), ctx->stream);
      return gt_fail(ctx, GT_ERR_ARG, "gt_gather_windows: a window start past corpus length - T - 1 was given; its rows were ignored");
    }
  }
  return GT_OK;
}

// ---- asynchronous reads: weights and optimizer state on their way to a checkpoint while the next step runs
//      (readStateBuffer, src/backend/webgpu.ts:1492-1503, is the blocking form) ----
static gt_status copy_stream_ready(gt_ctx* ctx) {
  if (ctx->copy_stream) return GT_OK;
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_read_async inside a graph capture");
  GT_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
  GT_CUDA(ctx, cudaEventCreateWithFlags(&ctx->copy_fork, cudaEventDisableTiming));
  GT_CUDA(ctx, cudaEventCreateWithFlags(&ctx->copy_done, cudaEventDisableTiming));
  return GT_OK;
}

gt_status gt_read_async(gt_ctx* ctx, gt_buf src, uint64_t bytes, uint64_t* out_ticket) {
  GT_REQUIRE(ctx, src && bytes > 0 && out_ticket, "gt_read_async: null argument");
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_read_async inside a graph capture");
  gt_status s = copy_stream_ready(ctx);
  if (s) return s;
  // a pinned block of at least this size, recycled from finished reads when one fits
  void* pinned = nullptr;
  uint64_t cap = (bytes + 4095) / 4096 * 4096;
  auto it = ctx->pinned_free.lower_bound(cap);
  if (it != ctx->pinned_free.end() && it->first <= 2 * cap) {
    pinned = it->second;
    cap = it->first;
    ctx->pinned_free.erase(it);
  } else {
    GT_CUDA(ctx, cudaMallocHost(&pinned, cap));
  }
  gt_ctx::AsyncRead r{pinned, cap, nullptr};
  GT_CUDA(ctx, cudaEventCreateWithFlags(&r.done, cudaEventDisableTiming));
  // the copy starts once everything enqueued so far on the compute stream has run, and runs beside what follows
  GT_CUDA(ctx, cudaEventRecord(ctx->copy_fork, ctx->stream));
  GT_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->copy_fork, 0));
  GT_CUDA(ctx, cudaMemcpyAsync(pinned, gt_ptr<void>(src), bytes, cudaMemcpyDeviceToHost, ctx->copy_stream));
  GT_CUDA(ctx, cudaEventRecord(r.done, ctx->copy_stream));
  ctx->copy_pending = true;
  const uint64_t ticket = ctx->next_ticket++;
  ctx->async_reads[ticket] = r;
  *out_ticket = ticket;
  return GT_OK;
}

gt_status gt_read_fence(gt_ctx* ctx) {
  if (!ctx->copy_pending) return GT_OK;
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_read_fence inside a graph capture");
  GT_CUDA(ctx, cudaEventRecord(ctx->copy_done, ctx->copy_stream));
  GT_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->copy_done, 0));
  ctx->copy_pending = false;
  return GT_OK;
}

gt_status gt_read_finish(gt_ctx* ctx, uint64_t ticket, void* host, uint64_t bytes) {
  auto it = ctx->async_reads.find(ticket);
  if (it == ctx->async_reads.end()) return gt_fail(ctx, GT_ERR_ARG, "gt_read_finish: unknown ticket %llu", (unsigned long long)ticket);
  GT_REQUIRE(ctx, host && bytes <= it->second.bytes, "gt_read_finish: %llu bytes asked of a %llu-byte read", (unsigned long long)bytes,
             (unsigned long long)it->second.bytes);
  GT_CUDA(ctx, cudaEventSynchronize(it->second.done));
  memcpy(host, it->second.pinned, bytes);
  ctx->readback_bytes += bytes;
  cudaEventDestroy(it->second.done);
  ctx->pinned_free.emplace(it->second.bytes, it->second.pinned);
  ctx->async_reads.erase(it);
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
