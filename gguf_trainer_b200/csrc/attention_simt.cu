// Causal grouped-query attention with optional sliding window, forward and backward, for any head
// dimension (src/model/autograd.ts:640-729; srcAttnFwd/BwdD/BwdDq/BwdDkv src/backend/wgsl.ts:657-918).
// f32 FMA throughout. This is the strict-precision path and the one that covers head dimensions the
// tensor-core kernels do not (the reference's tests use hd 4, 6, 12, 24).
// Same formulation as the reference's flash kernels: scores in the exp2 domain
// (SCALE2 = log2(e)/sqrt(hd)), running max with sentinel -3e38, LSE[h,row] = m + log2(l) as the only
// side buffer, backward recomputing p = exp2(q.k*SCALE2 - LSE). No atomics: one warp owns one output row
// (dQ) or one key row (dK, dV, reducing its GQA group in-thread), so results are deterministic.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAXND = 8;  // hd <= 256
constexpr float NEG = -3.0e38f;

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float dotrow(const float* __restrict__ a_smem, const float* __restrict__ b, int hd, bool vec) {
  float acc = 0.f;
  if (vec) {
    for (int d = 0; d < hd; d += 4) {
      float4 x = *(const float4*)(a_smem + d);
      float4 y = __ldg((const float4*)(b + d));
      acc = fmaf(x.x, y.x, acc); acc = fmaf(x.y, y.y, acc); acc = fmaf(x.z, y.z, acc); acc = fmaf(x.w, y.w, acc);
    }
  } else {
    for (int d = 0; d < hd; d++) acc = fmaf(a_smem[d], __ldg(b + d), acc);
  }
  return acc;
}

// warp per (row, h). rows = nseq*T.
__global__ void __launch_bounds__(WARPS * 32) attn_fwd_kernel(int rows, int T, int Hq, int Hkv, int hd, int window,
                                                               float scale2, const float* __restrict__ q,
                                                               const float* __restrict__ k, const float* __restrict__ v,
                                                               float* __restrict__ out, float* __restrict__ lse) {
  extern __shared__ __align__(16) float sm[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long w = (long)blockIdx.x * WARPS + wib;
  if (w >= (long)rows * Hq) return;
  const int h = (int)(w % Hq);
  const int row = (int)(w / Hq);
  const int t = row % T, base = row - t;
  const int kv = h / (Hq / Hkv);
  const bool vec = (hd & 3) == 0;
  float* qs = sm + wib * hd;
  const size_t qS = (size_t)Hq * hd, kS = (size_t)Hkv * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = q[(size_t)row * qS + (size_t)h * hd + d];
  __syncwarp();
  const int s0 = (window > 0 && t + 1 > window) ? t + 1 - window : 0;
  float m = NEG, l = 0.f, acc[MAXND];
#pragma unroll
  for (int i = 0; i < MAXND; i++) acc[i] = 0.f;
  for (int sb = s0; sb <= t; sb += 32) {
    int s = sb + lane;
    float sc = NEG;
    if (s <= t) sc = dotrow(qs, k + (size_t)(base + s) * kS + (size_t)kv * hd, hd, vec) * scale2;
    float mn = fmaxf(m, wmax(sc));
    float alpha = exp2f(m - mn);
    float p = (s <= t) ? exp2f(sc - mn) : 0.f;
    l = l * alpha + wsum(p);
    m = mn;
    int cnt = min(32, t - sb + 1);
#pragma unroll
    for (int i = 0; i < MAXND; i++) acc[i] *= alpha;
    for (int j = 0; j < cnt; j++) {
      float pj = __shfl_sync(0xffffffffu, p, j);
      const float* vr = v + (size_t)(base + sb + j) * kS + (size_t)kv * hd;
#pragma unroll
      for (int i = 0; i < MAXND; i++) { int d = lane + 32 * i; if (d < hd) acc[i] = fmaf(pj, __ldg(vr + d), acc[i]); }
    }
  }
  float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < MAXND; i++) { int d = lane + 32 * i; if (d < hd) out[(size_t)row * qS + (size_t)h * hd + d] = acc[i] * inv; }
  if (lane == 0) lse[(size_t)h * rows + row] = m + log2f(l);
}

// D[h,row] = sum_d dO*O   (srcAttnBwdD)
__global__ void attn_bwd_d_kernel(int rows, int Hq, int hd, const float* __restrict__ go, const float* __restrict__ o,
                                  float* __restrict__ D) {
  const int lane = threadIdx.x & 31;
  const long w = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (w >= (long)rows * Hq) return;
  const int h = (int)(w % Hq);
  const long row = w / Hq;
  const size_t b = (size_t)row * Hq * hd + (size_t)h * hd;
  float acc = 0.f;
  for (int d = lane; d < hd; d += 32) acc = fmaf(go[b + d], o[b + d], acc);
  acc = wsum(acc);
  if (lane == 0) D[(size_t)h * rows + row] = acc;
}

// warp per (row, h): dQ   (srcAttnBwdDq)
__global__ void __launch_bounds__(WARPS * 32) attn_bwd_dq_kernel(int rows, int T, int Hq, int Hkv, int hd, int window,
                                                                  float scale2, float scale, const float* __restrict__ q,
                                                                  const float* __restrict__ k, const float* __restrict__ v,
                                                                  const float* __restrict__ go, const float* __restrict__ lse,
                                                                  const float* __restrict__ D, float* gq, int accum) {
  extern __shared__ __align__(16) float sm[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long w = (long)blockIdx.x * WARPS + wib;
  if (w >= (long)rows * Hq) return;
  const int h = (int)(w % Hq);
  const int row = (int)(w / Hq);
  const int t = row % T, base = row - t;
  const int kv = h / (Hq / Hkv);
  const bool vec = (hd & 3) == 0;
  float* qs = sm + (wib * 2) * hd;
  float* gs = qs + hd;
  const size_t qS = (size_t)Hq * hd, kS = (size_t)Hkv * hd;
  const size_t qb = (size_t)row * qS + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) { qs[d] = q[qb + d]; gs[d] = go[qb + d]; }
  __syncwarp();
  const float L = lse[(size_t)h * rows + row], Dr = D[(size_t)h * rows + row];
  const int s0 = (window > 0 && t + 1 > window) ? t + 1 - window : 0;
  float acc[MAXND];
#pragma unroll
  for (int i = 0; i < MAXND; i++) acc[i] = 0.f;
  for (int sb = s0; sb <= t; sb += 32) {
    int s = sb + lane;
    float ds = 0.f;
    if (s <= t) {
      const float* kr = k + (size_t)(base + s) * kS + (size_t)kv * hd;
      const float* vr = v + (size_t)(base + s) * kS + (size_t)kv * hd;
      float p = exp2f(dotrow(qs, kr, hd, vec) * scale2 - L);
      float dp = dotrow(gs, vr, hd, vec);
      ds = p * (dp - Dr) * scale;
    }
    int cnt = min(32, t - sb + 1);
    for (int j = 0; j < cnt; j++) {
      float dj = __shfl_sync(0xffffffffu, ds, j);
      const float* kr = k + (size_t)(base + sb + j) * kS + (size_t)kv * hd;
#pragma unroll
      for (int i = 0; i < MAXND; i++) { int d = lane + 32 * i; if (d < hd) acc[i] = fmaf(dj, __ldg(kr + d), acc[i]); }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXND; i++) {
    int d = lane + 32 * i;
    if (d < hd) gq[qb + d] = accum ? gq[qb + d] + acc[i] : acc[i];
  }
}

// warp per (key row, kv head): dK and dV, summing the GQA group in-thread   (srcAttnBwdDkv)
__global__ void __launch_bounds__(WARPS * 32) attn_bwd_dkv_kernel(int rows, int T, int Hq, int Hkv, int hd, int window,
                                                                   float scale2, float scale, const float* __restrict__ q,
                                                                   const float* __restrict__ k, const float* __restrict__ v,
                                                                   const float* __restrict__ go, const float* __restrict__ lse,
                                                                   const float* __restrict__ D, float* gk, int accum_k,
                                                                   float* gv, int accum_v) {
  extern __shared__ __align__(16) float sm[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long w = (long)blockIdx.x * WARPS + wib;
  if (w >= (long)rows * Hkv) return;
  const int kvh = (int)(w % Hkv);
  const int row = (int)(w / Hkv);
  const int s = row % T, base = row - s;
  const int group = Hq / Hkv;
  const bool vec = (hd & 3) == 0;
  float* ks = sm + (wib * 2) * hd;
  float* vs = ks + hd;
  const size_t qS = (size_t)Hq * hd, kS = (size_t)Hkv * hd;
  const size_t kb = (size_t)row * kS + (size_t)kvh * hd;
  for (int d = lane; d < hd; d += 32) { ks[d] = k[kb + d]; vs[d] = v[kb + d]; }
  __syncwarp();
  const int tmax = (window > 0) ? min(T - 1, s + window - 1) : T - 1;
  float dk[MAXND], dv[MAXND];
#pragma unroll
  for (int i = 0; i < MAXND; i++) { dk[i] = 0.f; dv[i] = 0.f; }
  for (int h = kvh * group; h < (kvh + 1) * group; h++) {
    for (int tb = s; tb <= tmax; tb += 32) {
      int t = tb + lane;
      float p = 0.f, ds = 0.f;
      if (t <= tmax) {
        const size_t qb = (size_t)(base + t) * qS + (size_t)h * hd;
        p = exp2f(dotrow(ks, q + qb, hd, vec) * scale2 - lse[(size_t)h * rows + base + t]);
        float dp = dotrow(vs, go + qb, hd, vec);
        ds = p * (dp - D[(size_t)h * rows + base + t]) * scale;
      }
      int cnt = min(32, tmax - tb + 1);
      for (int j = 0; j < cnt; j++) {
        float pj = __shfl_sync(0xffffffffu, p, j);
        float dj = __shfl_sync(0xffffffffu, ds, j);
        const size_t qb = (size_t)(base + tb + j) * qS + (size_t)h * hd;
#pragma unroll
        for (int i = 0; i < MAXND; i++) {
          int d = lane + 32 * i;
          if (d < hd) { dk[i] = fmaf(dj, __ldg(q + qb + d), dk[i]); dv[i] = fmaf(pj, __ldg(go + qb + d), dv[i]); }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXND; i++) {
    int d = lane + 32 * i;
    if (d < hd) {
      if (gk) gk[kb + d] = accum_k ? gk[kb + d] + dk[i] : dk[i];
      if (gv) gv[kb + d] = accum_v ? gv[kb + d] + dv[i] : dv[i];
    }
  }
}

}  // namespace

gt_status gt_attention_fwd_simt(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q,
                                const float* k, const float* v, float* out, float* lse) {
  const float scale2 = 1.4426950408889634f / sqrtf((float)hd);
  long warps = (long)rows * Hq;
  attn_fwd_kernel<<<gt_cdiv(warps, WARPS), WARPS * 32, sizeof(float) * WARPS * hd, ctx->stream>>>(rows, T, Hq, Hkv, hd, window, scale2, q, k, v, out, lse);
  GT_LAUNCHED(ctx, "attn_fwd_kernel");
  return GT_OK;
}

gt_status gt_attention_bwd_simt_scratch(gt_ctx* ctx, float* D, int rows, int T, int Hq, int Hkv, int hd, int window,
                                        const float* q, const float* k, const float* v, const float* out, const float* lse,
                                        const float* go, float* gq, int accum_q, float* gk, int accum_k, float* gv,
                                        int accum_v);

gt_status gt_attention_bwd_simt(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q,
                                const float* k, const float* v, const float* out, const float* lse, const float* go,
                                float* gq, int accum_q, float* gk, int accum_k, float* gv, int accum_v) {
  float* D = nullptr;
  gt_status s = gt_scratch(ctx, sizeof(float) * (size_t)rows * Hq, &D);
  if (s) return s;
  return gt_attention_bwd_simt_scratch(ctx, D, rows, T, Hq, Hkv, hd, window, q, k, v, out, lse, go, gq, accum_q, gk, accum_k, gv,
                                       accum_v);
}

// The backward launches with the row-dot scratch D supplied by the caller: the context's growable scratch block
// (gt_attention_bwd_simt above) or the fixed array of the entry point that must not allocate.
gt_status gt_attention_bwd_simt_scratch(gt_ctx* ctx, float* D, int rows, int T, int Hq, int Hkv, int hd, int window,
                                        const float* q, const float* k, const float* v, const float* out, const float* lse,
                                        const float* go, float* gq, int accum_q, float* gk, int accum_k, float* gv,
                                        int accum_v) {
  const float scale = 1.f / sqrtf((float)hd);
  const float scale2 = 1.4426950408889634f * scale;
  long warps = (long)rows * Hq;
  attn_bwd_d_kernel<<<gt_cdiv(warps * 32, 256), 256, 0, ctx->stream>>>(rows, Hq, hd, go, out, D);
  GT_LAUNCHED(ctx, "attn_bwd_d_kernel");
  if (gq) {
    attn_bwd_dq_kernel<<<gt_cdiv(warps, WARPS), WARPS * 32, sizeof(float) * WARPS * 2 * hd, ctx->stream>>>(
        rows, T, Hq, Hkv, hd, window, scale2, scale, q, k, v, go, lse, D, gq, accum_q);
    GT_LAUNCHED(ctx, "attn_bwd_dq_kernel");
  }
  if (gk || gv) {
    long kw = (long)rows * Hkv;
    attn_bwd_dkv_kernel<<<gt_cdiv(kw, WARPS), WARPS * 32, sizeof(float) * WARPS * 2 * hd, ctx->stream>>>(
        rows, T, Hq, Hkv, hd, window, scale2, scale, q, k, v, go, lse, D, gk, accum_k, gv, accum_v);
    GT_LAUNCHED(ctx, "attn_bwd_dkv_kernel");
  }
  return GT_OK;
}
