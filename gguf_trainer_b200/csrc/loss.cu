// Cross entropy over [rows, V] logits, the chunked readout+CE pieces, and the sparse-teacher soft CE
// (src/model/autograd.ts:897-1138; srcCeFwd/Reduce/Bwd, srcCeChunkStats/LossFromStats/ChunkGrad,
// srcSoftCeFwd/BwdP/BwdQ in src/backend/wgsl.ts:936-1247). HBM-bound: one CTA per row, one pass of
// online max/sum in forward (4 B/element), backward recomputes exp(z-m)/sum from the logits instead of
// keeping a second [rows, V] buffer of probabilities (8 B/element, 12 when accumulating).
// Losses are per sequence: each sequence's mean over its kept rows, then the mean over sequences
// (the reference calls the loss once per sequence and averages, src/backend/train-gpu.ts:200-219).
#include "common.cuh"

namespace {

constexpr float NEG = -3.0e38f;
constexpr uint32_t IGNORE = 0xffffffffu;
constexpr int ROWT = 256;

struct MS { float m, s; };
__device__ __forceinline__ MS ms_merge(MS a, MS b) {
  float m = fmaxf(a.m, b.m);
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ MS block_ms(MS v, MS* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MS t{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = ms_merge(v, t);
  }
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) sh[w] = v;
  __syncthreads();
  MS r = sh[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); i++) r = ms_merge(r, sh[i]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ MS row_ms(const float* __restrict__ z, int V) {
  MS v{NEG, 0.f};
  if ((V & 3) == 0 && (((uintptr_t)z) & 15) == 0) {
    for (int i = threadIdx.x; i < V / 4; i += blockDim.x) {
      float4 x = ((const float4*)z)[i];
      float m = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
      float mn = fmaxf(v.m, m);
      v.s = v.s * __expf(v.m - mn) + __expf(x.x - mn) + __expf(x.y - mn) + __expf(x.z - mn) + __expf(x.w - mn);
      v.m = mn;
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float x = z[i];
      float mn = fmaxf(v.m, x);
      v.s = v.s * __expf(v.m - mn) + __expf(x - mn);
      v.m = mn;
    }
  }
  return v;
}

// stats[row] = (max, 1/sum, row loss, unused)
__global__ void __launch_bounds__(ROWT) ce_fwd_kernel(int V, const float* __restrict__ logits,
                                                      const uint32_t* __restrict__ targets, float4* __restrict__ stats) {
  __shared__ MS sh[ROWT / 32];
  const int row = blockIdx.x;
  const float* z = logits + (size_t)row * V;
  MS r = block_ms(row_ms(z, V), sh);
  if (threadIdx.x == 0) {
    uint32_t t = targets[row];
    float rl = (t != IGNORE) ? (logf(r.s) + r.m - z[t]) : 0.f;
    stats[row] = make_float4(r.m, 1.f / r.s, rl, 0.f);
  }
}

// One CTA, fixed summation order. rowloss_of(row) comes from stats[row].z (dense, soft) or run[row] (chunked).
// kept rows: targets[row*tstride] != IGNORE.
template <int MODE>  // 0: stats float4 .z ; 1: run float3 -> log(sum)+max-tl
__global__ void __launch_bounds__(1024) loss_reduce_kernel(int rows, int T, int nseq, const float* __restrict__ src,
                                                           const uint32_t* __restrict__ targets, int tstride,
                                                           float* __restrict__ loss, float* __restrict__ inv_kept) {
  __shared__ float ssum[32];
  __shared__ int scnt[32];
  __shared__ float total;
  if (threadIdx.x == 0) total = 0.f;
  for (int s = 0; s < nseq; s++) {
    float acc = 0.f;
    int cnt = 0;
    for (int i = threadIdx.x; i < T; i += blockDim.x) {
      int row = s * T + i;
      if (targets[(size_t)row * tstride] != IGNORE) {
        cnt++;
        if (MODE == 0) acc += src[(size_t)row * 4 + 2];
        else acc += logf(src[(size_t)row * 3 + 1]) + src[(size_t)row * 3 + 0] - src[(size_t)row * 3 + 2];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { acc += __shfl_xor_sync(0xffffffffu, acc, o); cnt += __shfl_xor_sync(0xffffffffu, cnt, o); }
    if ((threadIdx.x & 31) == 0) { ssum[threadIdx.x >> 5] = acc; scnt[threadIdx.x >> 5] = cnt; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.f; int c = 0;
      for (int i = 0; i < (int)(blockDim.x >> 5); i++) { a += ssum[i]; c += scnt[i]; }
      float denom = c > 0 ? (float)c : 1.f;
      float ls = a / denom;
      loss[1 + s] = ls;
      inv_kept[s] = 1.f / denom;
      total += ls;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) loss[0] = total / (float)nseq;
}

__global__ void __launch_bounds__(ROWT) ce_bwd_kernel(int V, int T, int nseq, const float* __restrict__ logits,
                                                      const uint32_t* __restrict__ targets, const float4* __restrict__ stats,
                                                      const float* __restrict__ inv_kept, const float* __restrict__ gloss,
                                                      float* glogits, int accum) {
  const int row = blockIdx.x;
  const uint32_t tg = targets[row];
  float* g = glogits + (size_t)row * V;
  if (tg == IGNORE) {
    if (!accum) for (int i = threadIdx.x; i < V; i += blockDim.x) g[i] = 0.f;
    return;
  }
  const float* z = logits + (size_t)row * V;
  const float4 st = stats[row];
  const float sc = gloss[0] * inv_kept[row / T] / (float)nseq;
  const float m = st.x, inv = st.y;
  if ((V & 3) == 0 && ((((uintptr_t)z) | ((uintptr_t)g)) & 15) == 0) {
    for (int i = threadIdx.x; i < V / 4; i += blockDim.x) {
      float4 x = ((const float4*)z)[i];
      float4 o = accum ? ((float4*)g)[i] : make_float4(0, 0, 0, 0);
      int v0 = i * 4;
      o.x += sc * (__expf(x.x - m) * inv - ((uint32_t)(v0 + 0) == tg ? 1.f : 0.f));
      o.y += sc * (__expf(x.y - m) * inv - ((uint32_t)(v0 + 1) == tg ? 1.f : 0.f));
      o.z += sc * (__expf(x.z - m) * inv - ((uint32_t)(v0 + 2) == tg ? 1.f : 0.f));
      o.w += sc * (__expf(x.w - m) * inv - ((uint32_t)(v0 + 3) == tg ? 1.f : 0.f));
      ((float4*)g)[i] = o;
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float v = sc * (__expf(z[i] - m) * inv - ((uint32_t)i == tg ? 1.f : 0.f));
      g[i] = accum ? g[i] + v : v;
    }
  }
}

// run[row] = (max, sum, target logit), updated with chunk columns [v0, v0+n)
__global__ void __launch_bounds__(ROWT) ce_chunk_stats_kernel(int n, int v0, int first, const float* __restrict__ chunk,
                                                              const uint32_t* __restrict__ targets, float* __restrict__ run) {
  __shared__ MS sh[ROWT / 32];
  const int row = blockIdx.x;
  const float* z = chunk + (size_t)row * n;
  MS r = block_ms(row_ms(z, n), sh);
  if (threadIdx.x == 0) {
    float* rr = run + (size_t)row * 3;
    MS prev = first ? MS{NEG, 0.f} : MS{rr[0], rr[1]};
    MS nw = ms_merge(prev, r);
    rr[0] = nw.m;
    rr[1] = nw.s;
    uint32_t t = targets[row];
    if (first) rr[2] = 0.f;
    if (t != IGNORE && t >= (uint32_t)v0 && t < (uint32_t)(v0 + n)) rr[2] = z[t - v0];
  }
}

// in place: chunk = scale_row * (exp(chunk - max)/sum - [v == target]); ignored rows zeroed
__global__ void __launch_bounds__(ROWT) ce_chunk_grad_kernel(int n, int v0, int T, int nseq, float* chunk,
                                                             const uint32_t* __restrict__ targets, const float* __restrict__ run,
                                                             const float* __restrict__ inv_kept, const float* __restrict__ gloss) {
  const int row = blockIdx.x;
  float* z = chunk + (size_t)row * n;
  const uint32_t tg = targets[row];
  if (tg == IGNORE) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) z[i] = 0.f;
    return;
  }
  const float m = run[(size_t)row * 3], inv = 1.f / run[(size_t)row * 3 + 1];
  const float sc = gloss[0] * inv_kept[row / T] / (float)nseq;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    z[i] = sc * (__expf(z[i] - m) * inv - ((uint32_t)(v0 + i) == tg ? 1.f : 0.f));
}

// soft CE forward: stats[row] = (max, 1/sum, row loss, row mass)
__global__ void __launch_bounds__(ROWT) soft_ce_fwd_kernel(int V, int k, const float* __restrict__ logits,
                                                           const uint32_t* __restrict__ tids, const float* __restrict__ tprobs,
                                                           float4* __restrict__ stats) {
  __shared__ MS sh[ROWT / 32];
  const int row = blockIdx.x;
  const float* z = logits + (size_t)row * V;
  MS r = block_ms(row_ms(z, V), sh);
  if (threadIdx.x == 0) {
    float rl = 0.f, mass = 0.f;
    if (tids[(size_t)row * k] != IGNORE) {
      float lz = logf(r.s) + r.m;
      for (int j = 0; j < k; j++) {
        float qq = tprobs[(size_t)row * k + j];
        if (qq == 0.f) continue;
        rl += qq * (lz - z[tids[(size_t)row * k + j]]);
        mass += qq;
      }
    }
    stats[row] = make_float4(r.m, 1.f / r.s, rl, mass);
  }
}

__global__ void __launch_bounds__(ROWT) soft_ce_bwd_kernel(int V, int k, int T, int nseq, const float* __restrict__ logits,
                                                           const uint32_t* __restrict__ tids, const float* __restrict__ tprobs,
                                                           const float4* __restrict__ stats, const float* __restrict__ inv_kept,
                                                           const float* __restrict__ gloss, float* glogits, int accum) {
  const int row = blockIdx.x;
  float* g = glogits + (size_t)row * V;
  if (tids[(size_t)row * k] == IGNORE) {
    if (!accum) for (int i = threadIdx.x; i < V; i += blockDim.x) g[i] = 0.f;
    return;
  }
  const float* z = logits + (size_t)row * V;
  const float4 st = stats[row];
  const float sc = gloss[0] * inv_kept[row / T] / (float)nseq;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = sc * st.w * __expf(z[i] - st.x) * st.y;
    g[i] = accum ? g[i] + v : v;
  }
  __syncthreads();
  // the k teacher slots of a row are subtracted by one thread, in order (duplicates allowed)
  if (threadIdx.x == 0)
    for (int j = 0; j < k; j++) g[tids[(size_t)row * k + j]] -= sc * tprobs[(size_t)row * k + j];
}

inline void seq_shape(gt_ctx* ctx, int rows, int* T, int* nseq) {
  if (ctx->batch) { *T = ctx->seq_len; *nseq = ctx->batch; } else { *T = rows; *nseq = 1; }
}

}  // namespace

extern "C" {

gt_status gt_ce_fwd(gt_ctx* ctx, int32_t rows, int32_t V, gt_buf logits, gt_buf targets, gt_buf stats, gt_buf loss, gt_buf inv_kept) {
  GT_REQUIRE(ctx, rows > 0 && V > 0 && logits && targets && stats && loss && inv_kept, "gt_ce_fwd: bad argument");
  int T, nseq; seq_shape(ctx, rows, &T, &nseq);
  GT_REQUIRE(ctx, rows == T * nseq, "gt_ce_fwd: %d rows but the batch is %d x %d", rows, nseq, T);
  ce_fwd_kernel<<<rows, ROWT, 0, ctx->stream>>>(V, gt_ptr<const float>(logits), gt_ptr<const uint32_t>(targets), gt_ptr<float4>(stats));
  GT_LAUNCHED(ctx, "ce_fwd_kernel");
  loss_reduce_kernel<0><<<1, 1024, 0, ctx->stream>>>(rows, T, nseq, gt_ptr<const float>(stats), gt_ptr<const uint32_t>(targets), 1, gt_ptr<float>(loss), gt_ptr<float>(inv_kept));
  GT_LAUNCHED(ctx, "loss_reduce_kernel");
  return GT_OK;
}

gt_status gt_ce_bwd(gt_ctx* ctx, int32_t rows, int32_t V, gt_buf logits, gt_buf targets, gt_buf stats, gt_buf inv_kept, gt_buf gloss, gt_buf glogits, int32_t accum) {
  if (!glogits) return GT_OK;
  GT_REQUIRE(ctx, rows > 0 && V > 0 && logits && targets && stats && inv_kept && gloss, "gt_ce_bwd: bad argument");
  int T, nseq; seq_shape(ctx, rows, &T, &nseq);
  ce_bwd_kernel<<<rows, ROWT, 0, ctx->stream>>>(V, T, nseq, gt_ptr<const float>(logits), gt_ptr<const uint32_t>(targets), gt_ptr<const float4>(stats),
                                                gt_ptr<const float>(inv_kept), gt_ptr<const float>(gloss), gt_ptr<float>(glogits), accum);
  GT_LAUNCHED(ctx, "ce_bwd_kernel");
  return GT_OK;
}

gt_status gt_ce_chunk_stats(gt_ctx* ctx, int32_t rows, int32_t n, int32_t v0, int32_t first, gt_buf chunk, gt_buf targets, gt_buf run) {
  GT_REQUIRE(ctx, rows > 0 && n > 0 && v0 >= 0 && chunk && targets && run, "gt_ce_chunk_stats: bad argument");
  ce_chunk_stats_kernel<<<rows, ROWT, 0, ctx->stream>>>(n, v0, first, gt_ptr<const float>(chunk), gt_ptr<const uint32_t>(targets), gt_ptr<float>(run));
  GT_LAUNCHED(ctx, "ce_chunk_stats_kernel");
  return GT_OK;
}

gt_status gt_ce_loss_from_stats(gt_ctx* ctx, int32_t rows, gt_buf run, gt_buf targets, gt_buf loss, gt_buf inv_kept) {
  GT_REQUIRE(ctx, rows > 0 && run && targets && loss && inv_kept, "gt_ce_loss_from_stats: bad argument");
  int T, nseq; seq_shape(ctx, rows, &T, &nseq);
  GT_REQUIRE(ctx, rows == T * nseq, "gt_ce_loss_from_stats: %d rows but the batch is %d x %d", rows, nseq, T);
  loss_reduce_kernel<1><<<1, 1024, 0, ctx->stream>>>(rows, T, nseq, gt_ptr<const float>(run), gt_ptr<const uint32_t>(targets), 1, gt_ptr<float>(loss), gt_ptr<float>(inv_kept));
  GT_LAUNCHED(ctx, "loss_reduce_kernel");
  return GT_OK;
}

gt_status gt_ce_chunk_grad(gt_ctx* ctx, int32_t rows, int32_t n, int32_t v0, gt_buf chunk, gt_buf targets, gt_buf run, gt_buf inv_kept, gt_buf gloss) {
  GT_REQUIRE(ctx, rows > 0 && n > 0 && chunk && targets && run && inv_kept && gloss, "gt_ce_chunk_grad: bad argument");
  int T, nseq; seq_shape(ctx, rows, &T, &nseq);
  ce_chunk_grad_kernel<<<rows, ROWT, 0, ctx->stream>>>(n, v0, T, nseq, gt_ptr<float>(chunk), gt_ptr<const uint32_t>(targets), gt_ptr<const float>(run),
                                                       gt_ptr<const float>(inv_kept), gt_ptr<const float>(gloss));
  GT_LAUNCHED(ctx, "ce_chunk_grad_kernel");
  return GT_OK;
}

gt_status gt_soft_ce_fwd(gt_ctx* ctx, int32_t rows, int32_t V, int32_t k, gt_buf logits, gt_buf tids, gt_buf tprobs, gt_buf stats, gt_buf loss, gt_buf inv_kept) {
  GT_REQUIRE(ctx, rows > 0 && V > 0 && k > 0 && logits && tids && tprobs && stats && loss && inv_kept, "gt_soft_ce_fwd: bad argument");
  int T, nseq; seq_shape(ctx, rows, &T, &nseq);
  GT_REQUIRE(ctx, rows == T * nseq, "gt_soft_ce_fwd: %d rows but the batch is %d x %d", rows, nseq, T);
  soft_ce_fwd_kernel<<<rows, ROWT, 0, ctx->stream>>>(V, k, gt_ptr<const float>(logits), gt_ptr<const uint32_t>(tids), gt_ptr<const float>(tprobs), gt_ptr<float4>(stats));
  GT_LAUNCHED(ctx, "soft_ce_fwd_kernel");
  loss_reduce_kernel<0><<<1, 1024, 0, ctx->stream>>>(rows, T, nseq, gt_ptr<const float>(stats), gt_ptr<const uint32_t>(tids), k, gt_ptr<float>(loss), gt_ptr<float>(inv_kept));
  GT_LAUNCHED(ctx, "loss_reduce_kernel");
  return GT_OK;
}

gt_status gt_soft_ce_bwd(gt_ctx* ctx, int32_t rows, int32_t V, int32_t k, gt_buf logits, gt_buf tids, gt_buf tprobs, gt_buf stats, gt_buf inv_kept, gt_buf gloss, gt_buf glogits, int32_t accum) {
  if (!glogits) return GT_OK;
  GT_REQUIRE(ctx, rows > 0 && V > 0 && k > 0 && logits && tids && tprobs && stats && inv_kept && gloss, "gt_soft_ce_bwd: bad argument");
  int T, nseq; seq_shape(ctx, rows, &T, &nseq);
  soft_ce_bwd_kernel<<<rows, ROWT, 0, ctx->stream>>>(V, k, T, nseq, gt_ptr<const float>(logits), gt_ptr<const uint32_t>(tids), gt_ptr<const float>(tprobs),
                                                     gt_ptr<const float4>(stats), gt_ptr<const float>(inv_kept), gt_ptr<const float>(gloss), gt_ptr<float>(glogits), accum);
  GT_LAUNCHED(ctx, "soft_ce_bwd_kernel");
  return GT_OK;
}

}  // extern "C"
