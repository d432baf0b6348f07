// Strict-f32 matrix product: f32 loads, FFMA, f32 accumulate. This is the precision mode whose results
// must stay within 1e-5 relative L2 of the reference's f64-accumulating loops (src/model/autograd.ts:348-377);
// the tensor-core path lives in gemm_tc.cu. Covers the three operand layouts of WebGPUBackend.gemm
// (src/backend/webgpu.ts:1654-1671) with ragged edges in every dimension.
#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8, PAD = 4;

// Element (m,k) of A is a[m*sam + k*sak]; element (n,k) of B is b[n*sbn + k*sbk].
template <bool A_KCONTIG, bool B_KCONTIG>
__global__ void __launch_bounds__(256) gemm_f32_kernel(int M, int N, int K, const float* __restrict__ a, long sam, long sak,
                                                       const float* __restrict__ b, long sbn, long sbk,
                                                       float* __restrict__ c, int accum, int ksplit, float alpha,
                                                       float* __restrict__ part) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Bs[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;
  // split-K: slice z covers k in [kb, ke)
  const int kper = ((K + ksplit - 1) / ksplit + BK - 1) / BK * BK;
  const int kb = blockIdx.z * kper;
  const int ke = min(K, kb + kper);

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

  for (int k0 = kb; k0 < ke; k0 += BK) {
#pragma unroll
    for (int i = 0; i < (BM * BK) / 256; i++) {
      int idx = tid + i * 256;
      int mm, kk;
      if (A_KCONTIG) { kk = idx % BK; mm = idx / BK; } else { mm = idx % BM; kk = idx / BM; }
      int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < ke) ? a[(long)gm * sam + (long)gk * sak] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < (BN * BK) / 256; i++) {
      int idx = tid + i * 256;
      int nn, kk;
      if (B_KCONTIG) { kk = idx % BK; nn = idx / BK; } else { nn = idx % BN; kk = idx / BN; }
      int gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < N && gk < ke) ? b[(long)gn * sbn + (long)gk * sbk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float av[TM], bv[TN];
      // two float4 per operand: rows ty*4..+3 and 64+ty*4..+3 (same for columns)
      *(float4*)&av[0] = *(const float4*)&As[kk][ty * 4];
      *(float4*)&av[4] = *(const float4*)&As[kk][64 + ty * 4];
      *(float4*)&bv[0] = *(const float4*)&Bs[kk][tx * 4];
      *(float4*)&bv[4] = *(const float4*)&Bs[kk][64 + tx * 4];
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; i++) {
    int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; j++) {
      int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (gn >= N) continue;
      float* dst = c + (long)gm * N + gn;
      const float v = acc[i][j] * alpha;
      if (ksplit > 1) part[((size_t)blockIdx.z * M + gm) * N + gn] = v;   // summed in slice order by splitk_sum_kernel
      else *dst = accum ? *dst + v : v;
    }
  }
}

// c (+)= part[0] + part[1] + ... in slice order: split-K without atomics, the same bits on every run
__global__ void splitk_sum_kernel(long n, int ksplit, const float* __restrict__ part, float* __restrict__ c, int accum) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float acc = accum ? c[i] : 0.f;
    for (int z = 0; z < ksplit; z++) acc += part[(size_t)z * n + i];
    c[i] = acc;
  }
}

}  // namespace

gt_status gt_gemm_simt(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, float alpha) {
  dim3 grid(gt_cdiv(N, BN), gt_cdiv(M, BM), 1);
  // Few output tiles and a deep K (the dW product, K = rows): split K across CTAs; the slices' partial products go
  // to scratch and are added in slice order by a second kernel, so the result does not depend on scheduling.
  int ksplit = 1;
  long tiles = (long)grid.x * grid.y;
  if (tiles < ctx->sm_count && K >= 1024) {
    ksplit = (int)min((long)(2 * ctx->sm_count / tiles), (long)(K / 256));
    if (ksplit < 1) ksplit = 1;
  }
  float* part = nullptr;
  if (ksplit > 1) {
    gt_status s = gt_scratch(ctx, sizeof(float) * (size_t)ksplit * M * N, &part);
    if (s) return s;
  }
  grid.z = ksplit;
  switch (kind) {
    case GT_GEMM_NT:
      gemm_f32_kernel<true, true><<<grid, 256, 0, ctx->stream>>>(M, N, K, a, K, 1, b, K, 1, c, accum, ksplit, alpha, part);
      break;
    case GT_GEMM_NN:
      gemm_f32_kernel<true, false><<<grid, 256, 0, ctx->stream>>>(M, N, K, a, K, 1, b, 1, N, c, accum, ksplit, alpha, part);
      break;
    case GT_GEMM_TN:
      gemm_f32_kernel<false, false><<<grid, 256, 0, ctx->stream>>>(M, N, K, a, 1, M, b, 1, N, c, accum, ksplit, alpha, part);
      break;
    default:
      return gt_fail(ctx, GT_ERR_ARG, "gt_gemm: unknown kind %d", kind);
  }
  GT_LAUNCHED(ctx, "gemm_f32_kernel");
  if (ksplit > 1) {
    const long n = (long)M * N;
    splitk_sum_kernel<<<(int)min((long)ctx->sm_count * 8, (n + 255) / 256), 256, 0, ctx->stream>>>(n, ksplit, part, c, accum);
    GT_LAUNCHED(ctx, "splitk_sum_kernel");
  }
  return GT_OK;
}

gt_status gt_gemm_batched(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, int batch) {
  if (ctx->precision != GT_PREC_FP32) {
    bool handled = false;
    gt_status s = gt_gemm_tc_batched(ctx, kind, accum, M, N, K, a, b, c, batch, &handled);
    if (s != GT_OK || handled) return s;
  }
  for (int i = 0; i < batch; i++) {
    gt_status s = gt_gemm_simt(ctx, kind, accum, M, N, K, a + (size_t)i * M * K, b + (size_t)i * N * K, c + (size_t)i * M * N, 1.f);
    if (s) return s;
  }
  return GT_OK;
}

// c (+)= alpha * op(a).op(b): the factor is applied to the f32 accumulator when it is written out
extern "C" gt_status gt_gemm_scaled(gt_ctx* ctx, int32_t kind, int32_t accum, int32_t M, int32_t N, int32_t K, gt_buf a, gt_buf b, gt_buf c,
                                    float alpha) {
  GT_REQUIRE(ctx, M > 0 && N > 0 && K > 0, "gt_gemm: empty product %dx%dx%d", M, N, K);
  GT_REQUIRE(ctx, a && b && c, "gt_gemm: null operand");
  if (ctx->precision != GT_PREC_FP32) {
    bool handled = false;
    gt_status s = gt_gemm_tc(ctx, kind, accum, M, N, K, gt_ptr<const float>(a), gt_ptr<const float>(b), gt_ptr<float>(c), alpha, &handled);
    if (s != GT_OK || handled) return s;
  }
  return gt_gemm_simt(ctx, kind, accum, M, N, K, gt_ptr<const float>(a), gt_ptr<const float>(b), gt_ptr<float>(c), alpha);
}

extern "C" gt_status gt_gemm(gt_ctx* ctx, int32_t kind, int32_t accum, int32_t M, int32_t N, int32_t K, gt_buf a, gt_buf b, gt_buf c) {
  return gt_gemm_scaled(ctx, kind, accum, M, N, K, a, b, c, 1.f);
}

// c (+)= sum_p op(a_p).op(b_p): one launch on the tensor-core path (each product's K blocks follow the previous one's in
// the main loop), accumulating products otherwise.
extern "C" gt_status gt_gemm_multi(gt_ctx* ctx, int32_t kind, int32_t accum, int32_t M, int32_t N, int32_t nparts, const int32_t* Ks,
                                   const gt_buf* as, const gt_buf* bs, gt_buf c) {
  GT_REQUIRE(ctx, M > 0 && N > 0 && nparts >= 1 && nparts <= 8 && Ks && as && bs && c, "gt_gemm_multi: %dx%d, %d products (1..8)", M, N, nparts);
  const float* pa[8];
  const float* pb[8];
  int k[8];
  for (int p = 0; p < nparts; p++) {
    GT_REQUIRE(ctx, Ks[p] > 0 && as[p] && bs[p], "gt_gemm_multi: product %d is empty or has a null operand", p);
    pa[p] = gt_ptr<const float>(as[p]); pb[p] = gt_ptr<const float>(bs[p]); k[p] = Ks[p];
  }
  if (ctx->precision != GT_PREC_FP32) {
    bool handled = false;
    gt_status s = gt_gemm_tc_multi(ctx, kind, accum, M, N, nparts, k, pa, pb, gt_ptr<float>(c), &handled);
    if (s != GT_OK || handled) return s;
  }
  for (int p = 0; p < nparts; p++) {
    gt_status s = gt_gemm(ctx, kind, p ? 1 : accum, M, N, k[p], as[p], bs[p], c);
    if (s) return s;
  }
  return GT_OK;
}

// ngroups products of one layout and one depth K, each with its own operands, extents and accumulate flag: one launch
// on the tensor-core path, one product after the other otherwise. alpha multiplies every product.
extern "C" gt_status gt_gemm_grouped_scaled(gt_ctx* ctx, int32_t kind, int32_t ngroups, const int32_t* Ms, const int32_t* Ns, int32_t K,
                                            const gt_buf* as, const gt_buf* bs, const gt_buf* cs, const int32_t* accums, float alpha) {
  GT_REQUIRE(ctx, ngroups >= 1 && ngroups <= 8 && K > 0 && Ms && Ns && as && bs && cs && accums, "gt_gemm_grouped: %d products (1..8), K %d", ngroups, K);
  const float* pa[8];
  const float* pb[8];
  float* pc[8];
  int m[8], n[8], acc[8];
  for (int g = 0; g < ngroups; g++) {
    GT_REQUIRE(ctx, Ms[g] > 0 && Ns[g] > 0 && as[g] && bs[g] && cs[g], "gt_gemm_grouped: product %d is empty or has a null operand", g);
    pa[g] = gt_ptr<const float>(as[g]); pb[g] = gt_ptr<const float>(bs[g]); pc[g] = gt_ptr<float>(cs[g]);
    m[g] = Ms[g]; n[g] = Ns[g]; acc[g] = accums[g];
  }
  if (ctx->precision != GT_PREC_FP32 && ngroups > 1) {
    bool handled = false;
    gt_status s = gt_gemm_tc_grouped(ctx, kind, ngroups, m, n, K, pa, pb, pc, acc, nullptr, nullptr, 0, alpha, &handled);
    if (s != GT_OK || handled) return s;
  }
  for (int g = 0; g < ngroups; g++) {
    gt_status s = gt_gemm_scaled(ctx, kind, acc[g], m[g], n[g], K, as[g], bs[g], cs[g], alpha);
    if (s) return s;
  }
  return GT_OK;
}

extern "C" gt_status gt_gemm_grouped(gt_ctx* ctx, int32_t kind, int32_t ngroups, const int32_t* Ms, const int32_t* Ns, int32_t K,
                                     const gt_buf* as, const gt_buf* bs, const gt_buf* cs, const int32_t* accums) {
  return gt_gemm_grouped_scaled(ctx, kind, ngroups, Ms, Ns, K, as, bs, cs, accums, 1.f);
}

// Projections y_g = x.W_g^T of one input launched together, the rotary embedding applied to the outputs that take one
// (heads[g] > 0) as their tiles are written; elsewhere each product followed by the rotation as a pass over its output.
extern "C" gt_status gt_linear_rope_grouped(gt_ctx* ctx, int32_t ngroups, int32_t rows, int32_t K, gt_buf x, const int32_t* Ns,
                                            const gt_buf* ws, const gt_buf* ys, const int32_t* heads, int32_t hd, double base,
                                            int32_t pos_offset) {
  GT_REQUIRE(ctx, ngroups >= 1 && ngroups <= 8 && rows > 0 && K > 0 && x && Ns && ws && ys && heads, "gt_linear_rope_grouped: %d projections (1..8), rows %d, K %d",
             ngroups, rows, K);
  GT_REQUIRE(ctx, hd > 0 && hd % 2 == 0, "gt_linear_rope_grouped: head size %d (must be even)", hd);
  const float* pa[8];
  const float* pb[8];
  float* pc[8];
  int m[8], n[8], acc[8], rp[8];
  bool any = false;
  for (int g = 0; g < ngroups; g++) {
    GT_REQUIRE(ctx, Ns[g] > 0 && ws[g] && ys[g], "gt_linear_rope_grouped: projection %d is empty or has a null operand", g);
    GT_REQUIRE(ctx, heads[g] == 0 || heads[g] * hd == Ns[g], "gt_linear_rope_grouped: projection %d is %d wide, not %d heads of %d", g, Ns[g], heads[g], hd);
    pa[g] = gt_ptr<const float>(x); pb[g] = gt_ptr<const float>(ws[g]); pc[g] = gt_ptr<float>(ys[g]);
    m[g] = rows; n[g] = Ns[g]; acc[g] = 0; rp[g] = heads[g] > 0;
    any = any || rp[g];
  }
  const float2* tab = nullptr;
  int period = 0;
  if (any) {
    gt_status s = gt_rope_table(ctx, rows, hd, base, pos_offset, &tab, &period);
    if (s) return s;
  }
  if (ctx->precision != GT_PREC_FP32 && ngroups > 1 && (!any || hd == 64)) {
    bool handled = false;
    gt_status s = gt_gemm_tc_grouped(ctx, GT_GEMM_NT, ngroups, m, n, K, pa, pb, pc, acc, rp, tab, period, 1.f, &handled);
    if (s != GT_OK || handled) return s;
  }
  for (int g = 0; g < ngroups; g++) {
    gt_status s = gt_gemm(ctx, GT_GEMM_NT, 0, rows, n[g], K, x, ws[g], ys[g]);
    if (s) return s;
    if (rp[g]) s = gt_rope_apply(ctx, false, rows, heads[g], hd, base, pos_offset, pc[g], pc[g], 0);
    if (s) return s;
  }
  return GT_OK;
}

extern "C" gt_status gt_gemm2(gt_ctx* ctx, int32_t kind, int32_t accum, int32_t M, int32_t N, int32_t K, gt_buf a, gt_buf b, int32_t K2,
                              gt_buf a2, gt_buf b2, gt_buf c) {
  GT_REQUIRE(ctx, M > 0 && N > 0 && K > 0 && K2 > 0, "gt_gemm2: empty product %dx%dx(%d+%d)", M, N, K, K2);
  GT_REQUIRE(ctx, a && b && a2 && b2 && c, "gt_gemm2: null operand");
  const int32_t Ks[2] = {K, K2};
  const gt_buf as[2] = {a, a2}, bs[2] = {b, b2};
  return gt_gemm_multi(ctx, kind, accum, M, N, 2, Ks, as, bs, c);
}
