// Attention backward for callers that must not allocate device memory.
//
// Some hosts hand every byte of HBM to their own arena at start-up and treat any later driver allocation
// as an error; others run steps under a latency budget in which cudaMalloc's device-wide synchronisation
// is not acceptable. The regular gt_attention_bwd keeps its per-(head,row) dot products D = sum_d dO*O in
// the context's scratch block, which grows with cudaMalloc the first time a larger shape arrives. This
// entry point runs the same f32 kernels with D in a fixed array that is part of the library image, so it
// never calls cudaMalloc, cudaFree or any allocating routine, whatever the shape history.
//
// The array lives in every GPU context that loads the library (4 MiB per device until the process exits).
// It is shared by all calls: two calls whose kernels overlap on the GPU (different streams, different
// contexts on one device) race on it, so issue them on one stream or serialise them yourself. Nothing in
// it has to start at zero: each call writes every element it later reads.
#include "common.cuh"

gt_status gt_attention_bwd_simt_scratch(gt_ctx* ctx, float* D, int rows, int T, int Hq, int Hkv, int hd, int window,
                                        const float* q, const float* k, const float* v, const float* out, const float* lse,
                                        const float* go, float* gq, int accum_q, float* gk, int accum_k, float* gv,
                                        int accum_v);

// rows * Hq may not exceed this many elements (e.g. 16384 rows x 64 query heads).
#define GT_STATIC_SCRATCH_FLOATS (1u << 20)

static __device__ __align__(256) float g_attn_bwd_d[GT_STATIC_SCRATCH_FLOATS];

// In host code the array's name is only a handle for the runtime, not an address a kernel can use: the
// device address is looked up once per device, with that device current, and cached here.
static float* g_attn_bwd_d_addr[64] = {};

extern "C" gt_status gt_attention_bwd_static(gt_ctx* ctx, int32_t rows, int32_t Hq, int32_t Hkv, int32_t hd, int32_t window,
                                             gt_buf q, gt_buf k, gt_buf v, gt_buf out, gt_buf lse, gt_buf gout, gt_buf gq,
                                             int32_t accum_q, gt_buf gk, int32_t accum_k, gt_buf gv, int32_t accum_v) {
  if (!ctx) return gt_fail(nullptr, GT_ERR_ARG, "gt_attention_bwd_static: null context");
  GT_REQUIRE(ctx, rows > 0 && Hq > 0 && Hkv > 0 && hd > 0 && hd <= 256 && window >= 0,
             "gt_attention_bwd_static: rows %d Hq %d Hkv %d hd %d window %d (hd must be in 1..256)", rows, Hq, Hkv, hd, window);
  GT_REQUIRE(ctx, Hq % Hkv == 0, "gt_attention_bwd_static: %d KV heads do not divide %d query heads", Hkv, Hq);
  GT_REQUIRE(ctx, (uint64_t)rows * (uint64_t)Hq <= GT_STATIC_SCRATCH_FLOATS,
             "gt_attention_bwd_static: rows*Hq = %llu exceeds the built-in scratch of %u elements; use gt_attention_bwd, which sizes its scratch to the shape",
             (unsigned long long)rows * (unsigned long long)Hq, GT_STATIC_SCRATCH_FLOATS);
  GT_REQUIRE(ctx, q && k && v && out && lse && gout, "gt_attention_bwd_static: null operand");
  int T = ctx->batch ? ctx->seq_len : rows;
  if (ctx->batch) GT_REQUIRE(ctx, rows == ctx->batch * ctx->seq_len, "gt_attention_bwd_static: %d rows but the batch is %d x %d", rows, ctx->batch, ctx->seq_len);
  if (!gq && !gk && !gv) return GT_OK;
  GT_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "gt_attention_bwd_static: device index %d out of range", ctx->device);
  float* D = g_attn_bwd_d_addr[ctx->device];
  if (!D) {
    // First call on this device: resolve the array's device address. This is the only set-up the entry
    // point ever does, so make this first call before any stream capture begins.
    GT_CUDA(ctx, cudaSetDevice(ctx->device));
    GT_CUDA(ctx, cudaGetSymbolAddress((void**)&D, g_attn_bwd_d));
    if (!D) return gt_fail(ctx, GT_ERR_CUDA, "gt_attention_bwd_static: the scratch symbol resolved to a null address");
    g_attn_bwd_d_addr[ctx->device] = D;
  }
  return gt_attention_bwd_simt_scratch(ctx, D, rows, T, Hq, Hkv, hd, window, gt_ptr<const float>(q), gt_ptr<const float>(k),
                                       gt_ptr<const float>(v), gt_ptr<const float>(out), gt_ptr<const float>(lse),
                                       gt_ptr<const float>(gout), gt_ptr<float>(gq), accum_q, gt_ptr<float>(gk), accum_k,
                                       gt_ptr<float>(gv), accum_v);
}
