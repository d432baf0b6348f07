// Shared declarations for libgguftrain_cuda.so (internal; the public ABI is include/gguftrain.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/gguftrain.h"

struct GtAdamW;
struct GtMuon;
struct GtDp;

struct gt_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  std::string err;
  int precision = GT_PREC_FP32;
  int batch = 0, seq_len = 0;  // gt_set_batch
  int sm_count = 148;
  int sm_reserved = 0;   // SMs left to a collective in flight (gt_dp_reserve_sms): persistent kernels size their grids without them
  // pool (BufferPool, webgpu.ts:214-262): exact-size free lists, 256-byte buckets
  std::map<uint64_t, std::vector<void*>> free_lists;
  std::unordered_map<void*, uint64_t> live;   // allocation -> bucket size (pooled)
  std::unordered_map<void*, uint64_t> state;  // allocation -> bytes (state buffers)
  uint64_t pool_bytes = 0, state_bytes = 0, readback_bytes = 0, launches = 0;
  // rope tables keyed by (T, hd, base, posOffset)
  struct RopeKey {
    int T, hd, off;
    double base;
    bool operator<(const RopeKey& o) const {
      if (T != o.T) return T < o.T;
      if (hd != o.hd) return hd < o.hd;
      if (off != o.off) return off < o.off;
      return base < o.base;
    }
  };
  std::map<RopeKey, float*> rope_tables;  // [T, hd/2, 2] (cos, sin)
  // launch orders of the attention dK/dV kernel, keyed by (key blocks, (kv head, sequence) pairs, query blocks per key block
  // step, window): see attn_dkv_order
  std::map<std::vector<int>, int*> attn_orders;
  // small scratch for reductions (never pooled)
  float* scratch = nullptr;
  uint64_t scratch_bytes = 0;
  std::vector<float*> retired_scratch;   // outgrown scratch blocks: captured graphs may still name them, freed with the context
  int* flags = nullptr;   // 256 zero-initialised device words: latched conditions and self-resetting counters (gt_flags)
  // staging
  void* pinned = nullptr;
  uint64_t pinned_bytes = 0, pinned_cursor = 0;
  bool capturing = false;
  std::vector<GtAdamW*> adamws;
  std::vector<GtMuon*> muons;
  std::vector<cudaGraphExec_t> graphs;
  cudaEvent_t events[64] = {};
  GtDp* dp = nullptr;
  // asynchronous reads (gt_read_async): a copy stream, and pinned blocks recycled by size
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t copy_fork = nullptr, copy_done = nullptr;
  bool copy_pending = false;
  struct AsyncRead { void* pinned; uint64_t bytes; cudaEvent_t done; };
  std::unordered_map<uint64_t, AsyncRead> async_reads;
  std::multimap<uint64_t, void*> pinned_free;
  uint64_t next_ticket = 1;
};

gt_status gt_fail(gt_ctx* ctx, gt_status code, const char* fmt, ...);
gt_status gt_check_cuda(gt_ctx* ctx, cudaError_t e, const char* what);
// scratch of at least `bytes` (grows outside graph capture only)
gt_status gt_scratch(gt_ctx* ctx, uint64_t bytes, float** out);
// 256 device words that start at zero (allocated on first use, never inside a graph capture: null then).
// GT_FLAG_WINDOW is raised by the window gather when a window leaves the corpus and is read and cleared by gt_sync;
// the counters are left at zero by the kernels that use them.
int* gt_flags(gt_ctx* ctx);
enum { GT_FLAG_WINDOW = 0, GT_FLAG_TOKEN_MAX = 1, GT_FLAG_NORM_COUNTER = 8 };

#define GT_CUDA(ctx, call)                                              \
  do {                                                                  \
    cudaError_t _e = (call);                                            \
    if (_e != cudaSuccess) return gt_check_cuda(ctx, _e, #call);        \
  } while (0)
#define GT_LAUNCHED(ctx, name)                                          \
  do {                                                                  \
    (ctx)->launches++;                                                  \
    cudaError_t _e = cudaPeekAtLastError();                             \
    if (_e != cudaSuccess) return gt_check_cuda(ctx, _e, name);         \
  } while (0)
#define GT_REQUIRE(ctx, cond, ...)                                      \
  do {                                                                  \
    if (!(cond)) return gt_fail(ctx, GT_ERR_ARG, __VA_ARGS__);          \
  } while (0)

template <typename T>
static inline T* gt_ptr(gt_buf b) { return reinterpret_cast<T*>(static_cast<uintptr_t>(b)); }
static inline int gt_cdiv(long a, long b) { return (int)((a + b - 1) / b); }

// internal cross-file entry points
gt_status gt_gemm_simt(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, float alpha);
gt_status gt_gemm_tc(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, float alpha,
                     bool* handled);
gt_status gt_gemm_tc_batched(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c,
                             int batch, bool* handled);
// batch of same-shape products through whichever path gt_gemm would take for one of them
gt_status gt_gemm_batched(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, int batch);
gt_status gt_gemm_tc_multi(gt_ctx* ctx, int kind, int accum, int M, int N, int nparts, const int* Ks, const float* const* as,
                           const float* const* bs, float* c, bool* handled);
// ropes (may be null): groups whose output is rotated as it is written (NT, heads 64 wide), with the table and period
// gt_rope_table gives
gt_status gt_gemm_tc_grouped(gt_ctx* ctx, int kind, int ngroups, const int* Ms, const int* Ns, int K, const float* const* as,
                             const float* const* bs, float* const* cs, const int* accums, const int* ropes, const float2* rope_tab,
                             int rope_period, float alpha, bool* handled);
gt_status gt_rope_table(gt_ctx* ctx, int rows, int hd, double base, int pos_offset, const float2** tab, int* period);
gt_status gt_rope_apply(gt_ctx* ctx, bool bwd, int rows, int H, int hd, double base, int pos_offset, const float* in, float* out, int accum);
gt_status gt_glu_linear_tc(gt_ctx* ctx, int op, int rows, int ffn, int in, const float* x, const float* wg, const float* wu, float* gate,
                           float* up, float* out, bool* handled);
gt_status gt_gemm_tc_check(gt_ctx* ctx);
void gt_optim_destroy(gt_ctx* ctx);
void gt_dp_teardown(gt_ctx* ctx);
// rank and world of the context's communicator (an error when gt_dp_init has not run)
gt_status gt_dp_rank(gt_ctx* ctx, int* rank, int* world);
// in place on the compute stream: rank r's `count` floats at buf + r*count reach every rank
gt_status gt_dp_allgather(gt_ctx* ctx, float* buf, size_t count);
