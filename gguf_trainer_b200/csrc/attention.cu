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
                              float* gq, int accum_q, float* gk, int accum_k, float* gv, int accum_v, const float2* rope,
                              bool* handled);

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
  int T = 0;
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
  int T = 0;
  gt_status s = check_shape(ctx, rows, Hq, Hkv, hd, window, &T);
  if (s) return s;
  GT_REQUIRE(ctx, q && k && v && out && lse && gout, "gt_attention_bwd: null operand");
  if (!gq && !gk && !gv) return GT_OK;
  if (ctx->precision != GT_PREC_FP32) {
    bool handled = false;
    s = gt_attention_bwd_tc(ctx, rows, T, Hq, Hkv, hd, window, gt_ptr<const float>(q), gt_ptr<const float>(k), gt_ptr<const float>(v),
                            gt_ptr<const float>(out), gt_ptr<const float>(lse), gt_ptr<const float>(gout), gt_ptr<float>(gq), accum_q,
                            gt_ptr<float>(gk), accum_k, gt_ptr<float>(gv), accum_v, nullptr, &handled);
    if (s || handled) return s;
  }
  return gt_attention_bwd_simt(ctx, rows, T, Hq, Hkv, hd, window, gt_ptr<const float>(q), gt_ptr<const float>(k), gt_ptr<const float>(v),
                               gt_ptr<const float>(out), gt_ptr<const float>(lse), gt_ptr<const float>(gout), gt_ptr<float>(gq), accum_q,
                               gt_ptr<float>(gk), accum_k, gt_ptr<float>(gv), accum_v);
}

// Attention backward whose q and k came out of a rotary embedding: gq and gk receive the gradients with respect to the
// rotation's INPUTS. On the tensor-core path the transposed rotation is applied to the dQ and dK accumulators as they
// are written; elsewhere the plain backward writes into scratch and the rotation's backward follows as its own pass.
gt_status gt_attention_bwd_rope(gt_ctx* ctx, int32_t rows, int32_t Hq, int32_t Hkv, int32_t hd, int32_t window, gt_buf q, gt_buf k,
                                gt_buf v, gt_buf out, gt_buf lse, gt_buf gout, gt_buf gq, int32_t accum_q, gt_buf gk, int32_t accum_k,
                                gt_buf gv, int32_t accum_v, double base, int32_t pos_offset) {
  int T = 0;
  gt_status s = check_shape(ctx, rows, Hq, Hkv, hd, window, &T);
  if (s) return s;
  GT_REQUIRE(ctx, q && k && v && out && lse && gout, "gt_attention_bwd_rope: null operand");
  GT_REQUIRE(ctx, hd % 2 == 0, "gt_attention_bwd_rope: head size %d (must be even)", hd);
  if (!gq && !gk && !gv) return GT_OK;
  const float2* tab = nullptr;
  int period = 0;
  s = gt_rope_table(ctx, rows, hd, base, pos_offset, &tab, &period);
  if (s) return s;
  if (ctx->precision != GT_PREC_FP32) {
    bool handled = false;
    s = gt_attention_bwd_tc(ctx, rows, T, Hq, Hkv, hd, window, gt_ptr<const float>(q), gt_ptr<const float>(k), gt_ptr<const float>(v),
                            gt_ptr<const float>(out), gt_ptr<const float>(lse), gt_ptr<const float>(gout), gt_ptr<float>(gq), accum_q,
                            gt_ptr<float>(gk), accum_k, gt_ptr<float>(gv), accum_v, tab, &handled);
    if (s || handled) return s;
  }
  // scratch: the row dots the plain backward asks for (it gets the head of the same block), then dQ and dK before the rotation
  const size_t nd = ((size_t)rows * Hq + 63) / 64 * 64, nq = (size_t)rows * Hq * hd, nk = (size_t)rows * Hkv * hd;
  float* blk = nullptr;
  s = gt_scratch(ctx, sizeof(float) * (nd + nq + nk), &blk);
  if (s) return s;
  float* tq = gq ? blk + nd : nullptr;
  float* tk = gk ? blk + nd + nq : nullptr;
  s = gt_attention_bwd(ctx, rows, Hq, Hkv, hd, window, q, k, v, out, lse, gout, (gt_buf)(uintptr_t)tq, 0, (gt_buf)(uintptr_t)tk, 0, gv, accum_v);
  if (s) return s;
  if (gq) s = gt_rope_apply(ctx, true, rows, Hq, hd, base, pos_offset, tq, gt_ptr<float>(gq), accum_q);
  if (s) return s;
  if (gk) s = gt_rope_apply(ctx, true, rows, Hkv, hd, base, pos_offset, tk, gt_ptr<float>(gk), accum_k);
  return s;
}

}  // extern "C"
