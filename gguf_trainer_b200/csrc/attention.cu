// Attention entry points: validation and the choice between the tensor-core kernels and the
// any-head-dimension f32 kernels (WebGPUBackend.attention picks between its materialised and flash
// kernels the same way, src/backend/webgpu.ts:1125-1192).
#include "common.cuh"

gt_status gt_attention_fwd_simt(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q,
                                const float* k, const float* v, float* out, float* lse);
gt_status gt_attention_bwd_simt(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q,
                                const float* k, const float* v, const float* out, const float* lse, const float* go,
                                float* gq, int accum_q, float* gk, int accum_k, float* gv, int accum_v);
gt_status gt_attention_fwd_tc(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q,
                              const float* k, const float* v, float* out, float* lse, bool* handled);
gt_status gt_attention_bwd_tc(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q,
                              const float* k, const float* v, const float* out, const float* lse, const float* go,
                              float* gq, int accum_q, float* gk, int accum_k, float* gv, int accum_v, bool* handled);

static gt_status check_shape(gt_ctx* ctx, int rows, int Hq, int Hkv, int hd, int window, int* T) {
  GT_REQUIRE(ctx, rows > 0 && Hq > 0 && Hkv > 0 && hd > 0 && hd <= 256 && window >= 0, "gt_attention: rows %d Hq %d Hkv %d hd %d window %d (hd must be in 1..256)", rows, Hq, Hkv, hd, window);
  GT_REQUIRE(ctx, Hq % Hkv == 0, "gt_attention: %d KV heads do not divide %d query heads", Hkv, Hq);
  *T = ctx->batch ? ctx->seq_len : rows;
  if (ctx->batch) GT_REQUIRE(ctx, rows == ctx->batch * ctx->seq_len, "gt_attention: %d rows but the batch is %d x %d", rows, ctx->batch, ctx->seq_len);
  return GT_OK;
}

extern "C" {

gt_status gt_attention_fwd(gt_ctx* ctx, int32_t rows, int32_t Hq, int32_t Hkv, int32_t hd, int32_t window, gt_buf q, gt_buf k,
                           gt_buf v, gt_buf out, gt_buf lse) {
  int T;
  gt_status s = check_shape(ctx, rows, Hq, Hkv, hd, window, &T);
  if (s) return s;
  GT_REQUIRE(ctx, q && k && v && out && lse, "gt_attention_fwd: null operand");
  if (ctx->precision != GT_PREC_FP32) {
    bool handled = false;
    s = gt_attention_fwd_tc(ctx, rows, T, Hq, Hkv, hd, window, gt_ptr<const float>(q), gt_ptr<const float>(k), gt_ptr<const float>(v),
                            gt_ptr<float>(out), gt_ptr<float>(lse), &handled);
    if (s || handled) return s;
  }
  return gt_attention_fwd_simt(ctx, rows, T, Hq, Hkv, hd, window, gt_ptr<const float>(q), gt_ptr<const float>(k), gt_ptr<const float>(v),
                               gt_ptr<float>(out), gt_ptr<float>(lse));
}

gt_status gt_attention_bwd(gt_ctx* ctx, int32_t rows, int32_t Hq, int32_t Hkv, int32_t hd, int32_t window, gt_buf q, gt_buf k,
                           gt_buf v, gt_buf out, gt_buf lse, gt_buf gout, gt_buf gq, int32_t accum_q, gt_buf gk, int32_t accum_k,
                           gt_buf gv, int32_t accum_v) {
  int T;
  gt_status s = check_shape(ctx, rows, Hq, Hkv, hd, window, &T);
  if (s) return s;
  GT_REQUIRE(ctx, q && k && v && out && lse && gout, "gt_attention_bwd: null operand");
  if (!gq && !gk && !gv) return GT_OK;
  if (ctx->precision != GT_PREC_FP32) {
    bool handled = false;
    s = gt_attention_bwd_tc(ctx, rows, T, Hq, Hkv, hd, window, gt_ptr<const float>(q), gt_ptr<const float>(k), gt_ptr<const float>(v),
                            gt_ptr<const float>(out), gt_ptr<const float>(lse), gt_ptr<const float>(gout), gt_ptr<float>(gq), accum_q,
                            gt_ptr<float>(gk), accum_k, gt_ptr<float>(gv), accum_v, &handled);
    if (s || handled) return s;
  }
  return gt_attention_bwd_simt(ctx, rows, T, Hq, Hkv, hd, window, gt_ptr<const float>(q), gt_ptr<const float>(k), gt_ptr<const float>(v),
                               gt_ptr<const float>(out), gt_ptr<const float>(lse), gt_ptr<const float>(gout), gt_ptr<float>(gq), accum_q,
                               gt_ptr<float>(gk), accum_k, gt_ptr<float>(gv), accum_v);
}

}  // extern "C"
