// RMSNorm over the last dimension of a [rows, d] view, forward and backward
// (src/model/autograd.ts:472-545; srcRmsNormFwd/BwdX/BwdW src/backend/wgsl.ts:217-303).
// The per-head variant (rmsNormHeads) is the same kernels on the [T*H, hd] view with a shared w[hd].
// HBM-bound. One warp owns a row: the row lives in registers between the reduction and the
// write, so x is read once. Backward produces dx and the column sums for dw in the same pass
// (the reference re-reads x and g once per column in srcRmsNormBwdW).
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Column sums for dw, two ways. Atomic: warps add into the CTA's shared array and CTAs into gw with f32 atomics, in
// whatever order they arrive (the tensor-core modes, whose split-K products are order-dependent anyway). Ordered
// (`part` given; strict-f32 mode): warps add one after the other, each CTA stores its sums to part[cta][d], and the
// CTA that arrives last (a counter it leaves at zero again) adds the CTAs' rows in index order on top of gw or of
// zero: the same bits on every run, which is what lets a recompute step equal a plain one bit for bit.
template <typename AddOwn>
__device__ __forceinline__ void dw_finish(float* sdw, int d, float* gw, int accum_w, float* part, int* counter, AddOwn add_own) {
  if (part == nullptr) {
    add_own(true);
    __syncthreads();
    for (int j = threadIdx.x; j < d; j += blockDim.x) atomicAdd(&gw[j], sdw[j]);
    return;
  }
  const int wcta = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int wi = 0; wi < nw; wi++) {
    if (wcta == wi) add_own(false);
    __syncthreads();
  }
  for (int j = threadIdx.x; j < d; j += blockDim.x) part[(size_t)blockIdx.x * d + j] = sdw[j];
  __threadfence();
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(counter, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float acc = accum_w ? gw[j] : 0.f;
    for (unsigned b = 0; b < gridDim.x; b++) acc += __ldcg(&part[(size_t)b * d + j]);
    gw[j] = acc;
  }
  if (threadIdx.x == 0) *counter = 0;
}

// NPL = elements per lane (d <= 32*NPL)
// With `xb` the row normalised is x + xb, and that sum is also written to `sum` (the residual add that precedes the
// norm in every block, src/arch/llama.ts:203-208, done in the same pass over the row).
// With `rope` (per-head norms of 64, 128 or 256 columns, d == 32 * NPL; a row is one head of one token, row = token * H +
// head) the normalised head is rotated before it is written (the `rope` that follows the q and k norms in
// src/arch/qwen3.ts:169-172): lane l holds columns l + 32 i, so both members of pair (j, j + d/2) sit in one lane.
template <int NPL>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(int rows, int d, const float* __restrict__ x,
                                                          const float* __restrict__ xb, float* __restrict__ sum,
                                                          const float* __restrict__ w, float eps,
                                                          float* __restrict__ y, float* __restrict__ rinv,
                                                          const float2* __restrict__ rope, int H, int period) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  float wv[NPL];
#pragma unroll
  for (int i = 0; i < NPL; i++) { int j = lane + 32 * i; wv[i] = j < d ? w[j] : 0.f; }
  for (int row = warp; row < rows; row += nwarps) {
    const float* xr = x + (size_t)row * d;
    float v[NPL];
    float ss = 0.f;
    float2 cs[NPL / 2];
    if (rope) {   // requested with the row itself, so that the two reads are in flight together
      const float2* tr = rope + (size_t)((row / H) % period) * (d >> 1);
#pragma unroll
      for (int i = 0; i < NPL / 2; i++) cs[i] = __ldg(tr + lane + 32 * i);
    }
    if (xb) {
      const float* br = xb + (size_t)row * d;
      float* sr = sum + (size_t)row * d;
#pragma unroll
      for (int i = 0; i < NPL; i++) {
        int j = lane + 32 * i;
        v[i] = j < d ? xr[j] + br[j] : 0.f;
        if (j < d) sr[j] = v[i];
        ss = fmaf(v[i], v[i], ss);
      }
    } else {
#pragma unroll
      for (int i = 0; i < NPL; i++) { int j = lane + 32 * i; v[i] = j < d ? xr[j] : 0.f; ss = fmaf(v[i], v[i], ss); }
    }
    ss = warp_sum(ss);
    float r = 1.f / sqrtf(ss / (float)d + eps);
    if (lane == 0) rinv[row] = r;
    float* yr = y + (size_t)row * d;
#pragma unroll
    for (int i = 0; i < NPL; i++) v[i] = v[i] * r * wv[i];
    if (rope) {
#pragma unroll
      for (int i = 0; i < NPL / 2; i++) {
        const float a0 = v[i], a1 = v[i + NPL / 2];
        v[i] = a0 * cs[i].x - a1 * cs[i].y;
        v[i + NPL / 2] = a0 * cs[i].y + a1 * cs[i].x;
      }
    }
#pragma unroll
    for (int i = 0; i < NPL; i++) { int j = lane + 32 * i; if (j < d) yr[j] = v[i]; }
  }
}

// The same forward pass with 16-byte accesses (d a multiple of 4, 16-byte aligned operands, d <= 128 * V4): lane l
// holds the float4s l, l + 32, ... of its row. Every load of the row (and of the row added to it) is issued before
// anything is stored. With `rope`, pair (c, c + d/2) is rotated after the norm: for d = 256 both members sit in one
// lane (float4 i and i + 1), for d = 128 and 64 in lanes 16 and 8 apart, fetched by shuffle.
template <int V4>
__global__ void __launch_bounds__(256) rmsnorm_fwd_vec_kernel(int rows, int d, const float* __restrict__ x,
                                                              const float* __restrict__ xb, float* __restrict__ sum,
                                                              const float* __restrict__ w, float eps,
                                                              float* __restrict__ y, float* __restrict__ rinv,
                                                              const float2* __restrict__ rope, int H, int period) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int d4 = d >> 2, h4 = d4 >> 1;   // float4s per row, per half row
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 wv[V4];
#pragma unroll
  for (int i = 0; i < V4; i++) { const int j = lane + 32 * i; wv[i] = j < d4 ? __ldg(reinterpret_cast<const float4*>(w) + j) : zero; }
  for (int row = warp; row < rows; row += nwarps) {
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * d);
    float4 v[V4];
#pragma unroll
    for (int i = 0; i < V4; i++) { const int j = lane + 32 * i; v[i] = j < d4 ? __ldg(xr + j) : zero; }
    float4 cs0 = zero, cs1 = zero;   // (cos, sin) of this lane's four pairs (d <= 256: one float4 per half row and lane)
    if (rope) {
      const int jl = lane & (h4 - 1);   // float4 index within the half row (h4 is 8, 16 or 32)
      const float4* tr = reinterpret_cast<const float4*>(rope + (size_t)((row / H) % period) * (d >> 1)) + 2 * jl;
      cs0 = __ldg(tr);
      cs1 = __ldg(tr + 1);
    }
    if (xb) {
      const float4* br = reinterpret_cast<const float4*>(xb + (size_t)row * d);
      float4 b[V4];
#pragma unroll
      for (int i = 0; i < V4; i++) { const int j = lane + 32 * i; b[i] = j < d4 ? __ldg(br + j) : zero; }
      float4* sr = reinterpret_cast<float4*>(sum + (size_t)row * d);
#pragma unroll
      for (int i = 0; i < V4; i++) {
        const int j = lane + 32 * i;
        v[i] = make_float4(v[i].x + b[i].x, v[i].y + b[i].y, v[i].z + b[i].z, v[i].w + b[i].w);
        if (j < d4) sr[j] = v[i];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < V4; i++) ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)d + eps);
    if (lane == 0) rinv[row] = r;
#pragma unroll
    for (int i = 0; i < V4; i++) v[i] = make_float4(v[i].x * r * wv[i].x, v[i].y * r * wv[i].y, v[i].z * r * wv[i].z, v[i].w * r * wv[i].w);
    if (rope) {
      if (V4 == 2 && h4 == 32) {          // d = 256: float4 0 is the first half, float4 1 the second
        const float4 a0 = v[0], a1 = v[V4 - 1];
        v[0] = make_float4(a0.x * cs0.x - a1.x * cs0.y, a0.y * cs0.z - a1.y * cs0.w, a0.z * cs1.x - a1.z * cs1.y, a0.w * cs1.z - a1.w * cs1.w);
        v[V4 - 1] = make_float4(a0.x * cs0.y + a1.x * cs0.x, a0.y * cs0.w + a1.y * cs0.z, a0.z * cs1.y + a1.z * cs1.x, a0.w * cs1.w + a1.w * cs1.z);
      } else {                            // d = 128 or 64: the other member is in lane ^ h4
        const float4 own = v[0];
        float4 oth;
        oth.x = __shfl_xor_sync(0xffffffffu, own.x, h4); oth.y = __shfl_xor_sync(0xffffffffu, own.y, h4);
        oth.z = __shfl_xor_sync(0xffffffffu, own.z, h4); oth.w = __shfl_xor_sync(0xffffffffu, own.w, h4);
        if ((lane & h4) == 0)   // first half: a0 = own, a1 = other
          v[0] = make_float4(own.x * cs0.x - oth.x * cs0.y, own.y * cs0.z - oth.y * cs0.w, own.z * cs1.x - oth.z * cs1.y, own.w * cs1.z - oth.w * cs1.w);
        else                    // second half: a0 = other, a1 = own
          v[0] = make_float4(oth.x * cs0.y + own.x * cs0.x, oth.y * cs0.w + own.y * cs0.z, oth.z * cs1.y + own.z * cs1.x, oth.w * cs1.w + own.w * cs1.z);
      }
    }
    float4* yr = reinterpret_cast<float4*>(y + (size_t)row * d);
#pragma unroll
    for (int i = 0; i < V4; i++) { const int j = lane + 32 * i; if (j < d4) yr[j] = v[i]; }
  }
}

template <int NPL>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(int rows, int d, const float* __restrict__ x,
                                                          const float* __restrict__ w, const float* __restrict__ rinv,
                                                          const float* __restrict__ g, const float* gadd, float* gx, int accum_x,
                                                          float* gw, int accum_w, float* part, int* counter) {
  extern __shared__ float sdw[];  // [d] block-level column partials
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  if (gw) {
    for (int j = threadIdx.x; j < d; j += blockDim.x) sdw[j] = 0.f;
    __syncthreads();
  }
  float wv[NPL], dwv[NPL];
#pragma unroll
  for (int i = 0; i < NPL; i++) { int j = lane + 32 * i; wv[i] = j < d ? w[j] : 0.f; dwv[i] = 0.f; }
  const float invd = 1.f / (float)d;
  for (int row = warp; row < rows; row += nwarps) {
    const float* xr = x + (size_t)row * d;
    const float* gr = g + (size_t)row * d;
    float xv[NPL], gv[NPL];
    float S = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; i++) {
      int j = lane + 32 * i;
      xv[i] = j < d ? xr[j] : 0.f;
      gv[i] = j < d ? gr[j] : 0.f;
      S = fmaf(gv[i] * wv[i], xv[i], S);
    }
    S = warp_sum(S);
    const float r = rinv[row];
    const float k = r * r * r * S * invd;
    if (gx) {
      float* o = gx + (size_t)row * d;
      const float* prev = gadd ? gadd + (size_t)row * d : o;   // what the term is added to: another buffer, or gx itself
#pragma unroll
      for (int i = 0; i < NPL; i++) {
        int j = lane + 32 * i;
        if (j < d) {
          float v = wv[i] * r * gv[i] - xv[i] * k;
          o[j] = accum_x ? prev[j] + v : v;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NPL; i++) dwv[i] = fmaf(gv[i] * xv[i], r, dwv[i]);
  }
  if (gw) {
    dw_finish(sdw, d, gw, accum_w, part, counter, [&](bool atomic) {
#pragma unroll
      for (int i = 0; i < NPL; i++) {
        int j = lane + 32 * i;
        if (j < d) { if (atomic) atomicAdd(&sdw[j], dwv[i]); else sdw[j] += dwv[i]; }
      }
    });
  }
}

// 128-bit variant for d % 4 == 0: lane owns float4 columns lane, lane+32, ... (V4 of them). One CTA per SM with 16
// warps striding over the rows keeps the number of CTAs that finish with global atomics on dw at the SM count.
template <int V4, int TH>
__global__ void __launch_bounds__(TH) rmsnorm_bwd_vec_kernel(int rows, int d, const float* __restrict__ x, const float* __restrict__ w,
                                                              const float* __restrict__ rinv, const float* __restrict__ g,
                                                              const float* gadd, float* gx, int accum_x, float* gw, int accum_w,
                                                              float* part, int* counter) {
  extern __shared__ float sdw[];
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int d4 = d >> 2;
  if (gw) {
    for (int j = threadIdx.x; j < d; j += blockDim.x) sdw[j] = 0.f;
    __syncthreads();
  }
  float4 wv[V4], dwv[V4];
#pragma unroll
  for (int i = 0; i < V4; i++) {
    const int j = lane + 32 * i;
    wv[i] = j < d4 ? reinterpret_cast<const float4*>(w)[j] : make_float4(0, 0, 0, 0);
    dwv[i] = make_float4(0, 0, 0, 0);
  }
  const float invd = 1.f / (float)d;
  for (int row = warp; row < rows; row += nwarps) {
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * d);
    const float4* gr = reinterpret_cast<const float4*>(g + (size_t)row * d);
    float4 xv[V4], gv[V4], pv[V4];
    float S = 0.f;
    if (gx && accum_x) {   // the old dx values are fetched with the row, not after the reduction (one round trip, not two)
      const float4* orow = reinterpret_cast<const float4*>((gadd ? gadd : gx) + (size_t)row * d);
#pragma unroll
      for (int i = 0; i < V4; i++) {
        const int j = lane + 32 * i;
        pv[i] = j < d4 ? orow[j] : make_float4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int i = 0; i < V4; i++) {
      const int j = lane + 32 * i;
      xv[i] = j < d4 ? xr[j] : make_float4(0, 0, 0, 0);
      gv[i] = j < d4 ? gr[j] : make_float4(0, 0, 0, 0);
      S = fmaf(gv[i].x * wv[i].x, xv[i].x, S); S = fmaf(gv[i].y * wv[i].y, xv[i].y, S);
      S = fmaf(gv[i].z * wv[i].z, xv[i].z, S); S = fmaf(gv[i].w * wv[i].w, xv[i].w, S);
    }
    S = warp_sum(S);
    const float r = rinv[row];
    const float k = r * r * r * S * invd;
    if (gx) {
      float4* o = reinterpret_cast<float4*>(gx + (size_t)row * d);
#pragma unroll
      for (int i = 0; i < V4; i++) {
        const int j = lane + 32 * i;
        if (j < d4) {
          float4 v;
          v.x = wv[i].x * r * gv[i].x - xv[i].x * k; v.y = wv[i].y * r * gv[i].y - xv[i].y * k;
          v.z = wv[i].z * r * gv[i].z - xv[i].z * k; v.w = wv[i].w * r * gv[i].w - xv[i].w * k;
          if (accum_x) { v.x += pv[i].x; v.y += pv[i].y; v.z += pv[i].z; v.w += pv[i].w; }
          o[j] = v;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < V4; i++) {
      dwv[i].x = fmaf(gv[i].x * xv[i].x, r, dwv[i].x); dwv[i].y = fmaf(gv[i].y * xv[i].y, r, dwv[i].y);
      dwv[i].z = fmaf(gv[i].z * xv[i].z, r, dwv[i].z); dwv[i].w = fmaf(gv[i].w * xv[i].w, r, dwv[i].w);
    }
  }
  if (gw) {
    dw_finish(sdw, d, gw, accum_w, part, counter, [&](bool atomic) {
#pragma unroll
      for (int i = 0; i < V4; i++) {
        const int j = lane + 32 * i;
        if (j < d4) {
          if (atomic) {
            atomicAdd(&sdw[4 * j + 0], dwv[i].x); atomicAdd(&sdw[4 * j + 1], dwv[i].y);
            atomicAdd(&sdw[4 * j + 2], dwv[i].z); atomicAdd(&sdw[4 * j + 3], dwv[i].w);
          } else {
            sdw[4 * j + 0] += dwv[i].x; sdw[4 * j + 1] += dwv[i].y; sdw[4 * j + 2] += dwv[i].z; sdw[4 * j + 3] += dwv[i].w;
          }
        }
      }
    });
  }
}

// Prepares dw's accumulation: ordered mode gets the per-CTA partial rows (context scratch) and the arrival counter;
// atomic mode clears gw first unless it accumulates.
gt_status dw_mode(gt_ctx* ctx, int blocks, int d, float* gw, int accum_w, bool ordered, float** part, int** counter) {
  if (ordered) {
    int* flags = gt_flags(ctx);
    if (!flags) return gt_fail(ctx, GT_ERR_STATE, "gt_rmsnorm_bwd: first use inside a graph capture; run the step once eagerly first");
    gt_status s = gt_scratch(ctx, sizeof(float) * (size_t)blocks * d, part);
    if (s) return s;
    *counter = flags + GT_FLAG_NORM_COUNTER;
    return GT_OK;
  }
  if (!accum_w) GT_CUDA(ctx, cudaMemsetAsync(gw, 0, sizeof(float) * d, ctx->stream));
  return GT_OK;
}

template <int V4, int TH = (V4 >= 8 ? 256 : 512)>
gt_status launch_bwd_vec(gt_ctx* ctx, int rows, int d, const float* x, const float* w, const float* rinv, const float* g,
                         const float* gadd, float* gx, int accum_x, float* gw, int accum_w, bool ordered) {
  // Narrow rows (the per-head norms, d = 128 or 256) keep few bytes in flight per warp: more resident CTAs make up for it.
  // (Only with many rows: every CTA ends with d atomics on dw, which a short launch would feel.)
  const int per_sm = (V4 <= 2 && rows >= 65536) ? (V4 == 1 ? 4 : 3) : 512 / TH;
  int blocks = min(gt_cdiv(rows, TH / 32), ctx->sm_count * per_sm);
  float* part = nullptr;
  int* counter = nullptr;
  if (gw) {
    gt_status s = dw_mode(ctx, blocks, d, gw, accum_w, ordered, &part, &counter);
    if (s) return s;
  }
  rmsnorm_bwd_vec_kernel<V4, TH><<<blocks, TH, sizeof(float) * d, ctx->stream>>>(rows, d, x, w, rinv, g, gadd, gx, accum_x, gw, accum_w, part, counter);
  GT_LAUNCHED(ctx, "rmsnorm_bwd_vec_kernel");
  return GT_OK;
}

template <int NPL>
gt_status launch_fwd(gt_ctx* ctx, int rows, int d, const float* x, const float* xb, float* sum, const float* w, float eps, float* y,
                     float* rinv, const float2* rope = nullptr, int H = 1, int period = 1) {
  int blocks = min(gt_cdiv(rows, 8), ctx->sm_count * 8);
  rmsnorm_fwd_kernel<NPL><<<blocks, 256, 0, ctx->stream>>>(rows, d, x, xb, sum, w, eps, y, rinv, rope, H, period);
  GT_LAUNCHED(ctx, "rmsnorm_fwd_kernel");
  return GT_OK;
}
template <int V4>
gt_status launch_fwd_vec(gt_ctx* ctx, int rows, int d, const float* x, const float* xb, float* sum, const float* w, float eps, float* y,
                         float* rinv, const float2* rope, int H, int period) {
  int blocks = min(gt_cdiv(rows, 8), ctx->sm_count * 8);
  rmsnorm_fwd_vec_kernel<V4><<<blocks, 256, 0, ctx->stream>>>(rows, d, x, xb, sum, w, eps, y, rinv, rope, H, period);
  GT_LAUNCHED(ctx, "rmsnorm_fwd_vec_kernel");
  return GT_OK;
}
template <int NPL>
gt_status launch_bwd(gt_ctx* ctx, int rows, int d, const float* x, const float* w, const float* rinv, const float* g,
                     const float* gadd, float* gx, int accum_x, float* gw, int accum_w, bool ordered) {
  // fewer, fatter blocks when dw is wanted: each block ends with d global atomics
  int blocks = min(gt_cdiv(rows, 8), ctx->sm_count * (gw ? 4 : 8));
  float* part = nullptr;
  int* counter = nullptr;
  if (gw) {
    gt_status s = dw_mode(ctx, blocks, d, gw, accum_w, ordered, &part, &counter);
    if (s) return s;
  }
  rmsnorm_bwd_kernel<NPL><<<blocks, 256, sizeof(float) * d, ctx->stream>>>(rows, d, x, w, rinv, g, gadd, gx, accum_x, gw, accum_w, part, counter);
  GT_LAUNCHED(ctx, "rmsnorm_bwd_kernel");
  return GT_OK;
}

}  // namespace

extern "C" {

static gt_status rmsnorm_fwd_any(gt_ctx* ctx, int rows, int d, const float* px, const float* pb, float* ps, const float* pw, float eps,
                                 float* py, float* pr, const float2* rope = nullptr, int H = 1, int period = 1) {
  const bool aligned = ((((uintptr_t)px) | ((uintptr_t)pb) | ((uintptr_t)ps) | ((uintptr_t)pw) | ((uintptr_t)py)) & 15) == 0;
  if ((d & 3) == 0 && d >= 64 && d <= 1024 && aligned && (!rope || d == 64 || d == 128 || d == 256)) {
    if (d <= 128) return launch_fwd_vec<1>(ctx, rows, d, px, pb, ps, pw, eps, py, pr, rope, H, period);
    if (d <= 256) return launch_fwd_vec<2>(ctx, rows, d, px, pb, ps, pw, eps, py, pr, rope, H, period);
    if (d <= 640) return launch_fwd_vec<5>(ctx, rows, d, px, pb, ps, pw, eps, py, pr, rope, H, period);
    return launch_fwd_vec<8>(ctx, rows, d, px, pb, ps, pw, eps, py, pr, rope, H, period);
  }
  if (rope) {   // (unaligned operands) the scalar kernels, which hold both members of a pair in one lane
    if (d == 64) return launch_fwd<2>(ctx, rows, d, px, pb, ps, pw, eps, py, pr, rope, H, period);
    if (d == 128) return launch_fwd<4>(ctx, rows, d, px, pb, ps, pw, eps, py, pr, rope, H, period);
    return launch_fwd<8>(ctx, rows, d, px, pb, ps, pw, eps, py, pr, rope, H, period);
  }
  if (d <= 64) return launch_fwd<2>(ctx, rows, d, px, pb, ps, pw, eps, py, pr);
  if (d <= 128) return launch_fwd<4>(ctx, rows, d, px, pb, ps, pw, eps, py, pr);
  if (d <= 256) return launch_fwd<8>(ctx, rows, d, px, pb, ps, pw, eps, py, pr);
  if (d <= 640) return launch_fwd<20>(ctx, rows, d, px, pb, ps, pw, eps, py, pr);
  if (d <= 1024) return launch_fwd<32>(ctx, rows, d, px, pb, ps, pw, eps, py, pr);
  return launch_fwd<64>(ctx, rows, d, px, pb, ps, pw, eps, py, pr);
}

gt_status gt_rmsnorm_fwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf x, gt_buf w, float eps, gt_buf y, gt_buf rinv) {
  GT_REQUIRE(ctx, rows > 0 && d > 0 && d <= 2048, "gt_rmsnorm_fwd: rows %d d %d (d must be in 1..2048)", rows, d);
  GT_REQUIRE(ctx, x && w && y && rinv, "gt_rmsnorm_fwd: null operand");
  return rmsnorm_fwd_any(ctx, rows, d, gt_ptr<const float>(x), nullptr, nullptr, gt_ptr<const float>(w), eps, gt_ptr<float>(y),
                         gt_ptr<float>(rinv));
}

gt_status gt_add_rmsnorm_fwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf a, gt_buf b, gt_buf w, float eps, gt_buf sum, gt_buf y,
                             gt_buf rinv) {
  GT_REQUIRE(ctx, rows > 0 && d > 0 && d <= 2048, "gt_add_rmsnorm_fwd: rows %d d %d (d must be in 1..2048)", rows, d);
  GT_REQUIRE(ctx, a && b && w && sum && y && rinv, "gt_add_rmsnorm_fwd: null operand");
  return rmsnorm_fwd_any(ctx, rows, d, gt_ptr<const float>(a), gt_ptr<const float>(b), gt_ptr<float>(sum), gt_ptr<const float>(w), eps,
                         gt_ptr<float>(y), gt_ptr<float>(rinv));
}

// rmsNormHeads followed by rope (src/arch/qwen3.ts:169-172, src/arch/gemma3.ts:194-197) as one pass over the heads.
gt_status gt_rmsnorm_heads_rope_fwd(gt_ctx* ctx, int32_t rows, int32_t H, int32_t hd, gt_buf x, gt_buf w, float eps, gt_buf y, gt_buf rinv,
                                    double base, int32_t pos_offset) {
  GT_REQUIRE(ctx, rows > 0 && H > 0 && hd > 0 && hd <= 2048 && hd % 2 == 0, "gt_rmsnorm_heads_rope_fwd: rows %d H %d hd %d", rows, H, hd);
  GT_REQUIRE(ctx, x && w && y && rinv, "gt_rmsnorm_heads_rope_fwd: null operand");
  const float* px = gt_ptr<const float>(x); const float* pw = gt_ptr<const float>(w);
  float* py = gt_ptr<float>(y); float* pr = gt_ptr<float>(rinv);
  const float2* tab = nullptr;
  int period = 0;
  gt_status s = gt_rope_table(ctx, rows, hd, base, pos_offset, &tab, &period);
  if (s) return s;
  const int n = rows * H;
  if (hd == 64 || hd == 128 || hd == 256) return rmsnorm_fwd_any(ctx, n, hd, px, nullptr, nullptr, pw, eps, py, pr, tab, H, period);
  s = rmsnorm_fwd_any(ctx, n, hd, px, nullptr, nullptr, pw, eps, py, pr);     // other head sizes: two passes
  if (s) return s;
  return gt_rope_apply(ctx, false, rows, H, hd, base, pos_offset, py, py, 0);
}

static gt_status rmsnorm_bwd_any(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf x, gt_buf w, gt_buf rinv, gt_buf gy, gt_buf gadd, gt_buf gx,
                                 int32_t accum_x, gt_buf gw, int32_t accum_w) {
  GT_REQUIRE(ctx, rows > 0 && d > 0 && d <= 2048, "gt_rmsnorm_bwd: rows %d d %d (d must be in 1..2048)", rows, d);
  GT_REQUIRE(ctx, x && w && rinv && gy, "gt_rmsnorm_bwd: null operand");
  if (!gx && !gw) return GT_OK;
  const float* pa = gt_ptr<const float>(gadd);
  const float* px = gt_ptr<const float>(x); const float* pw = gt_ptr<const float>(w);
  const float* pr = gt_ptr<const float>(rinv); const float* pg = gt_ptr<const float>(gy);
  float* pgx = gt_ptr<float>(gx); float* pgw = gt_ptr<float>(gw);
  const bool ordered = ctx->precision == GT_PREC_FP32;   // strict-f32 mode: dw bit-identical from run to run
  if ((d & 3) == 0 && d >= 128 && d <= 1024 && ((((uintptr_t)px) | ((uintptr_t)pw) | ((uintptr_t)pg) | ((uintptr_t)pgx) | ((uintptr_t)pa)) & 15) == 0) {
    if (d <= 128) return launch_bwd_vec<1>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
    if (d <= 256) return launch_bwd_vec<2>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
    if (d <= 640) return launch_bwd_vec<5>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
    return launch_bwd_vec<8>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
  }
  if (d <= 64) return launch_bwd<2>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
  if (d <= 128) return launch_bwd<4>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
  if (d <= 256) return launch_bwd<8>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
  if (d <= 640) return launch_bwd<20>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
  if (d <= 1024) return launch_bwd<32>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
  return launch_bwd<64>(ctx, rows, d, px, pw, pr, pg, pa, pgx, accum_x, pgw, accum_w, ordered);
}

gt_status gt_rmsnorm_bwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf x, gt_buf w, gt_buf rinv, gt_buf gy, gt_buf gx,
                         int32_t accum_x, gt_buf gw, int32_t accum_w) {
  return rmsnorm_bwd_any(ctx, rows, d, x, w, rinv, gy, 0, gx, accum_x, gw, accum_w);
}

gt_status gt_rmsnorm_bwd_add(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf x, gt_buf w, gt_buf rinv, gt_buf gy, gt_buf gadd, gt_buf gx,
                             gt_buf gw, int32_t accum_w) {
  GT_REQUIRE(ctx, gadd && gx, "gt_rmsnorm_bwd_add: null operand");
  return rmsnorm_bwd_any(ctx, rows, d, x, w, rinv, gy, gadd, gx, 1, gw, accum_w);
}

}  // extern "C"
