// Elementwise ops and their backward: add, mul, silu, gelu(tanh), scale
// (src/model/autograd.ts:382-469; src/backend/webgpu.ts:905-1078). HBM-bound: 128-bit loads and
// stores on the aligned body, a grid of a few CTAs per SM striding over the array.
#include "common.cuh"

namespace {

constexpr float GELU_K = 0.7978845608028654f;  // sqrt(2/pi), autograd.ts:433
constexpr float GELU_A = 0.044715f;            // autograd.ts:434

template <int OP>
__device__ __forceinline__ float ew_f(float a, float b, float c) {
  if (OP == GT_EW_ADD) return a + b;
  if (OP == GT_EW_MUL) return a * b;
  if (OP == GT_EW_SILU) return a / (1.f + __expf(-a));
  if (OP == GT_EW_GELU) {
    float u = GELU_K * (a + GELU_A * a * a * a);
    return 0.5f * a * (1.f + tanhf(u));
  }
  return a * c;
}

// d(out)/d(a) factor (times upstream g); for add/mul the b-side factor comes from swapping operands.
template <int OP>
__device__ __forceinline__ float ew_da(float a, float b, float c) {
  if (OP == GT_EW_ADD) return 1.f;
  if (OP == GT_EW_MUL) return b;
  if (OP == GT_EW_SILU) {
    float s = 1.f / (1.f + __expf(-a));
    return s + a * s * (1.f - s);
  }
  if (OP == GT_EW_GELU) {
    float a2 = a * a;
    float u = GELU_K * (a + GELU_A * a * a2);
    float th = tanhf(u);
    float dudx = GELU_K * (1.f + 3.f * GELU_A * a2);
    return 0.5f * (1.f + th) + 0.5f * a * (1.f - th * th) * dudx;
  }
  return c;
}

template <int OP>
__global__ void ew_fwd_kernel(size_t n, const float* __restrict__ a, const float* __restrict__ b, float c,
                              float* __restrict__ out) {
  constexpr bool BIN = (OP == GT_EW_ADD || OP == GT_EW_MUL);
  size_t n4 = n / 4;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 va = ((const float4*)a)[i];
    float4 vb = BIN ? ((const float4*)b)[i] : make_float4(0, 0, 0, 0);
    float4 r;
    r.x = ew_f<OP>(va.x, vb.x, c); r.y = ew_f<OP>(va.y, vb.y, c);
    r.z = ew_f<OP>(va.z, vb.z, c); r.w = ew_f<OP>(va.w, vb.w, c);
    ((float4*)out)[i] = r;
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = ew_f<OP>(a[i], BIN ? b[i] : 0.f, c);
}

// ga (+)= g * d/da ; gb (+)= g * d/db. ga/gb may alias each other (add(t,t), mul(t,t)): then both
// contributions are summed into one write so the aliased buffer sees a+b exactly once.
template <int OP>
__global__ void ew_bwd_kernel(size_t n, const float* __restrict__ a, const float* __restrict__ b, float c,
                              const float* __restrict__ g, float* ga, int acc_a, float* gb, int acc_b) {
  constexpr bool BIN = (OP == GT_EW_ADD || OP == GT_EW_MUL);
  const bool alias = BIN && ga && ga == gb;
  size_t n4 = n / 4;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 vg = ((const float4*)g)[i];
    float4 va = (OP == GT_EW_ADD || OP == GT_EW_SCALE) ? make_float4(0, 0, 0, 0) : ((const float4*)a)[i];
    float4 vb = (OP == GT_EW_MUL) ? ((const float4*)b)[i] : make_float4(0, 0, 0, 0);
    float4 da, db;
    da.x = vg.x * ew_da<OP>(va.x, vb.x, c); da.y = vg.y * ew_da<OP>(va.y, vb.y, c);
    da.z = vg.z * ew_da<OP>(va.z, vb.z, c); da.w = vg.w * ew_da<OP>(va.w, vb.w, c);
    if (BIN) {
      db.x = vg.x * ew_da<OP>(vb.x, va.x, c); db.y = vg.y * ew_da<OP>(vb.y, va.y, c);
      db.z = vg.z * ew_da<OP>(vb.z, va.z, c); db.w = vg.w * ew_da<OP>(vb.w, va.w, c);
    }
    if (alias) {
      float4 o = acc_a ? ((float4*)ga)[i] : make_float4(0, 0, 0, 0);
      o.x += da.x + db.x; o.y += da.y + db.y; o.z += da.z + db.z; o.w += da.w + db.w;
      ((float4*)ga)[i] = o;
      continue;
    }
    if (ga) {
      float4 o = acc_a ? ((float4*)ga)[i] : make_float4(0, 0, 0, 0);
      o.x += da.x; o.y += da.y; o.z += da.z; o.w += da.w;
      ((float4*)ga)[i] = o;
    }
    if (BIN && gb) {
      float4 o = acc_b ? ((float4*)gb)[i] : make_float4(0, 0, 0, 0);
      o.x += db.x; o.y += db.y; o.z += db.z; o.w += db.w;
      ((float4*)gb)[i] = o;
    }
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float va = (OP == GT_EW_ADD || OP == GT_EW_SCALE) ? 0.f : a[i];
    float vb = (OP == GT_EW_MUL) ? b[i] : 0.f;
    float da = g[i] * ew_da<OP>(va, vb, c);
    float db = BIN ? g[i] * ew_da<OP>(vb, va, c) : 0.f;
    if (alias) { ga[i] = (acc_a ? ga[i] : 0.f) + da + db; continue; }
    if (ga) ga[i] = (acc_a ? ga[i] : 0.f) + da;
    if (BIN && gb) gb[i] = (acc_b ? gb[i] : 0.f) + db;
  }
}

// Gated unit in one pass: out = act(x) * u with act = silu (SwiGLU) or tanh-gelu (GeGLU). The reference issues the
// activation and the product as two ops (src/arch/llama.ts:209-211, gemma3.ts:208-210); fused, the activated gate never
// touches HBM: forward 12 B/element instead of 20, backward 20 instead of 32.
template <int OP>
__global__ void glu_fwd_kernel(size_t n, const float* __restrict__ x, const float* __restrict__ u, float* __restrict__ out) {
  size_t n4 = n / 4, stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 a = ((const float4*)x)[i], b = ((const float4*)u)[i], r;
    r.x = ew_f<OP>(a.x, 0.f, 0.f) * b.x; r.y = ew_f<OP>(a.y, 0.f, 0.f) * b.y;
    r.z = ew_f<OP>(a.z, 0.f, 0.f) * b.z; r.w = ew_f<OP>(a.w, 0.f, 0.f) * b.w;
    ((float4*)out)[i] = r;
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = ew_f<OP>(x[i], 0.f, 0.f) * u[i];
}

// gx (+)= g * u * act'(x) ; gu (+)= g * act(x)
template <int OP>
__global__ void glu_bwd_kernel(size_t n, const float* __restrict__ x, const float* __restrict__ u, const float* __restrict__ g,
                               float* gx, int acc_x, float* gu, int acc_u) {
  size_t n4 = n / 4, stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 a = ((const float4*)x)[i], b = ((const float4*)u)[i], go = ((const float4*)g)[i];
    if (gx) {
      float4 o = acc_x ? ((float4*)gx)[i] : make_float4(0, 0, 0, 0);
      o.x += go.x * b.x * ew_da<OP>(a.x, 0.f, 0.f); o.y += go.y * b.y * ew_da<OP>(a.y, 0.f, 0.f);
      o.z += go.z * b.z * ew_da<OP>(a.z, 0.f, 0.f); o.w += go.w * b.w * ew_da<OP>(a.w, 0.f, 0.f);
      ((float4*)gx)[i] = o;
    }
    if (gu) {
      float4 o = acc_u ? ((float4*)gu)[i] : make_float4(0, 0, 0, 0);
      o.x += go.x * ew_f<OP>(a.x, 0.f, 0.f); o.y += go.y * ew_f<OP>(a.y, 0.f, 0.f);
      o.z += go.z * ew_f<OP>(a.z, 0.f, 0.f); o.w += go.w * ew_f<OP>(a.w, 0.f, 0.f);
      ((float4*)gu)[i] = o;
    }
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (gx) gx[i] = (acc_x ? gx[i] : 0.f) + g[i] * u[i] * ew_da<OP>(x[i], 0.f, 0.f);
    if (gu) gu[i] = (acc_u ? gu[i] : 0.f) + g[i] * ew_f<OP>(x[i], 0.f, 0.f);
  }
}

inline int ew_grid(gt_ctx* ctx, size_t n) {
  size_t want = (n / 4 + 255) / 256;
  size_t cap = (size_t)ctx->sm_count * 8;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

extern "C" {

gt_status gt_ew_fwd(gt_ctx* ctx, int32_t op, uint64_t n, gt_buf a, gt_buf b, float c, gt_buf out) {
  if (n == 0) return GT_OK;
  const float* pa = gt_ptr<const float>(a);
  const float* pb = gt_ptr<const float>(b);
  float* po = gt_ptr<float>(out);
  GT_REQUIRE(ctx, pa && po && aligned16(pa) && aligned16(po) && aligned16(pb), "gt_ew_fwd: operands must be non-null and 16-byte aligned");
  int grid = ew_grid(ctx, n);
  switch (op) {
    case GT_EW_ADD: GT_REQUIRE(ctx, pb, "gt_ew_fwd: add needs b"); ew_fwd_kernel<GT_EW_ADD><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, po); break;
    case GT_EW_MUL: GT_REQUIRE(ctx, pb, "gt_ew_fwd: mul needs b"); ew_fwd_kernel<GT_EW_MUL><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, po); break;
    case GT_EW_SILU: ew_fwd_kernel<GT_EW_SILU><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, po); break;
    case GT_EW_GELU: ew_fwd_kernel<GT_EW_GELU><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, po); break;
    case GT_EW_SCALE: ew_fwd_kernel<GT_EW_SCALE><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, po); break;
    default: return gt_fail(ctx, GT_ERR_ARG, "gt_ew_fwd: unknown op %d", op);
  }
  GT_LAUNCHED(ctx, "ew_fwd_kernel");
  return GT_OK;
}

gt_status gt_ew_bwd(gt_ctx* ctx, int32_t op, uint64_t n, gt_buf a, gt_buf b, float c, gt_buf gout, gt_buf ga,
                    int32_t accum_a, gt_buf gb, int32_t accum_b) {
  if (n == 0 || (!ga && !gb)) return GT_OK;
  const float* pa = gt_ptr<const float>(a);
  const float* pb = gt_ptr<const float>(b);
  const float* pg = gt_ptr<const float>(gout);
  float* pga = gt_ptr<float>(ga);
  float* pgb = gt_ptr<float>(gb);
  GT_REQUIRE(ctx, pg && aligned16(pa) && aligned16(pb) && aligned16(pg) && aligned16(pga) && aligned16(pgb), "gt_ew_bwd: operands must be 16-byte aligned");
  int grid = ew_grid(ctx, n);
  switch (op) {
    case GT_EW_ADD: ew_bwd_kernel<GT_EW_ADD><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, pg, pga, accum_a, pgb, accum_b); break;
    case GT_EW_MUL: GT_REQUIRE(ctx, pa && pb, "gt_ew_bwd: mul needs a and b"); ew_bwd_kernel<GT_EW_MUL><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, pg, pga, accum_a, pgb, accum_b); break;
    case GT_EW_SILU: GT_REQUIRE(ctx, pa, "gt_ew_bwd: silu needs a"); ew_bwd_kernel<GT_EW_SILU><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, pg, pga, accum_a, pgb, accum_b); break;
    case GT_EW_GELU: GT_REQUIRE(ctx, pa, "gt_ew_bwd: gelu needs a"); ew_bwd_kernel<GT_EW_GELU><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, pg, pga, accum_a, pgb, accum_b); break;
    case GT_EW_SCALE: ew_bwd_kernel<GT_EW_SCALE><<<grid, 256, 0, ctx->stream>>>(n, pa, pb, c, pg, pga, accum_a, pgb, accum_b); break;
    default: return gt_fail(ctx, GT_ERR_ARG, "gt_ew_bwd: unknown op %d", op);
  }
  GT_LAUNCHED(ctx, "ew_bwd_kernel");
  return GT_OK;
}

gt_status gt_glu_fwd(gt_ctx* ctx, int32_t op, uint64_t n, gt_buf x, gt_buf u, gt_buf out) {
  if (n == 0) return GT_OK;
  const float* px = gt_ptr<const float>(x); const float* pu = gt_ptr<const float>(u); float* po = gt_ptr<float>(out);
  GT_REQUIRE(ctx, px && pu && po && aligned16(px) && aligned16(pu) && aligned16(po), "gt_glu_fwd: operands must be non-null and 16-byte aligned");
  GT_REQUIRE(ctx, op == GT_EW_SILU || op == GT_EW_GELU, "gt_glu_fwd: the gate activation must be silu or gelu, got op %d", op);
  int grid = ew_grid(ctx, n);
  if (op == GT_EW_SILU) glu_fwd_kernel<GT_EW_SILU><<<grid, 256, 0, ctx->stream>>>(n, px, pu, po);
  else glu_fwd_kernel<GT_EW_GELU><<<grid, 256, 0, ctx->stream>>>(n, px, pu, po);
  GT_LAUNCHED(ctx, "glu_fwd_kernel");
  return GT_OK;
}

// gate = x.Wg^T, up = x.Wu^T, out = act(gate) * up: the two projections of a gated FFN and the gated unit. One launch on
// the tensor-core path (the unit is applied where the projections' tiles are written), three otherwise.
gt_status gt_glu_linear_fwd(gt_ctx* ctx, int32_t op, int32_t rows, int32_t ffn, int32_t in, gt_buf x, gt_buf wg, gt_buf wu, gt_buf gate,
                            gt_buf up, gt_buf out) {
  GT_REQUIRE(ctx, rows > 0 && ffn > 0 && in > 0 && x && wg && wu && gate && up && out, "gt_glu_linear_fwd: bad argument");
  GT_REQUIRE(ctx, op == GT_EW_SILU || op == GT_EW_GELU, "gt_glu_linear_fwd: the gate activation must be silu or gelu, got op %d", op);
  if (ctx->precision != GT_PREC_FP32) {
    bool handled = false;
    gt_status s = gt_glu_linear_tc(ctx, op, rows, ffn, in, gt_ptr<const float>(x), gt_ptr<const float>(wg), gt_ptr<const float>(wu),
                                   gt_ptr<float>(gate), gt_ptr<float>(up), gt_ptr<float>(out), &handled);
    if (s != GT_OK || handled) return s;
  }
  gt_status s = gt_gemm(ctx, GT_GEMM_NT, 0, rows, ffn, in, x, wg, gate);
  if (!s) s = gt_gemm(ctx, GT_GEMM_NT, 0, rows, ffn, in, x, wu, up);
  if (!s) s = gt_glu_fwd(ctx, op, (uint64_t)rows * ffn, gate, up, out);
  return s;
}

gt_status gt_glu_bwd(gt_ctx* ctx, int32_t op, uint64_t n, gt_buf x, gt_buf u, gt_buf gout, gt_buf gx, int32_t accum_x, gt_buf gu,
                     int32_t accum_u) {
  if (n == 0 || (!gx && !gu)) return GT_OK;
  const float* px = gt_ptr<const float>(x); const float* pu = gt_ptr<const float>(u); const float* pg = gt_ptr<const float>(gout);
  float* pgx = gt_ptr<float>(gx); float* pgu = gt_ptr<float>(gu);
  GT_REQUIRE(ctx, px && pu && pg && aligned16(px) && aligned16(pu) && aligned16(pg) && aligned16(pgx) && aligned16(pgu),
             "gt_glu_bwd: operands must be non-null and 16-byte aligned");
  GT_REQUIRE(ctx, op == GT_EW_SILU || op == GT_EW_GELU, "gt_glu_bwd: the gate activation must be silu or gelu, got op %d", op);
  GT_REQUIRE(ctx, !pgx || pgx != pgu, "gt_glu_bwd: the two gradient outputs alias");
  int grid = ew_grid(ctx, n);
  if (op == GT_EW_SILU) glu_bwd_kernel<GT_EW_SILU><<<grid, 256, 0, ctx->stream>>>(n, px, pu, pg, pgx, accum_x, pgu, accum_u);
  else glu_bwd_kernel<GT_EW_GELU><<<grid, 256, 0, ctx->stream>>>(n, px, pu, pg, pgx, accum_x, pgu, accum_u);
  GT_LAUNCHED(ctx, "glu_bwd_kernel");
  return GT_OK;
}

}  // extern "C"
