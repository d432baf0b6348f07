// NeoX RoPE (src/model/autograd.ts:579-632; srcRope src/backend/wgsl.ts:346-384) and the embedding
// gather / scatter-add (autograd.ts:548-573; wgsl.ts:305-344). HBM-bound.
// RoPE: the reference evaluates pow/cos/sin in f64 per (position, pair) and stores them as f32. Here the
// same f64 evaluation runs once per (seq_len, hd, base, offset) into a cached device table, so the
// per-step kernels are pure loads and FMAs.
#include "common.cuh"

namespace {

__global__ void rope_table_kernel(int T, int half, int hd, double base, int pos_offset, float2* __restrict__ tab) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  int t = i / half, j = i % half;
  double freq = pow(base, (-2.0 * j) / hd);
  double ang = (double)(t + pos_offset) * freq;
  tab[i] = make_float2((float)cos(ang), (float)sin(ang));
}

// one thread per (row, head, pair); pairs are the fastest index so loads coalesce
template <bool BWD>
__global__ void rope_kernel(long npairs, int H, int hd, int period, const float2* __restrict__ tab,
                            const float* __restrict__ in, float* out, int accum) {
  const int half = hd >> 1;
  long stride = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < npairs; i += stride) {
    int j = (int)(i % half);
    long rh = i / half;  // row*H + h
    long row = rh / H;
    int t = (int)(row % period);
    float2 cs = tab[(long)t * half + j];
    long b = rh * hd;
    float a0 = in[b + j], a1 = in[b + j + half];
    float o0, o1;
    if (!BWD) { o0 = a0 * cs.x - a1 * cs.y; o1 = a0 * cs.y + a1 * cs.x; }
    else { o0 = cs.x * a0 + cs.y * a1; o1 = -cs.y * a0 + cs.x * a1; }
    if (accum) { out[b + j] += o0; out[b + j + half] += o1; }
    else { out[b + j] = o0; out[b + j + half] = o1; }
  }
}

__global__ void embedding_fwd_kernel(long n, int d, const float* __restrict__ w, const uint32_t* __restrict__ ids,
                                     float* __restrict__ out) {
  long stride = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    long t = i / d;
    int j = (int)(i % d);
    out[i] = w[(long)ids[t] * d + j];
  }
}

// scatter-add with f32 reductions in L2 (red.global.add): O(rows*d) work where the reference scans all
// rows for every element of the table. Summation order across duplicate ids is not fixed.
__global__ void embedding_bwd_kernel(long n, int d, const float* __restrict__ g, const uint32_t* __restrict__ ids,
                                     float* gw) {
  long stride = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    long t = i / d;
    int j = (int)(i % d);
    atomicAdd(&gw[(long)ids[t] * d + j], g[i]);
  }
}

gt_status rope_table(gt_ctx* ctx, int T, int hd, double base, int pos_offset, const float2** out) {
  gt_ctx::RopeKey key{T, hd, pos_offset, base};
  auto it = ctx->rope_tables.find(key);
  if (it == ctx->rope_tables.end()) {
    if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "rope table for (T=%d, hd=%d) is built on first use; run the step once eagerly before capturing", T, hd);
    float* p = nullptr;
    int half = hd / 2;
    GT_CUDA(ctx, cudaMalloc(&p, sizeof(float2) * (size_t)T * half));
    rope_table_kernel<<<gt_cdiv((long)T * half, 256), 256, 0, ctx->stream>>>(T, half, hd, base, pos_offset, (float2*)p);
    GT_LAUNCHED(ctx, "rope_table_kernel");
    ctx->state_bytes += sizeof(float2) * (size_t)T * half;
    it = ctx->rope_tables.emplace(key, p).first;
  }
  *out = (const float2*)it->second;
  return GT_OK;
}

template <bool BWD>
gt_status rope_run(gt_ctx* ctx, int rows, int H, int hd, double base, int pos_offset, const float* in, float* out, int accum) {
  GT_REQUIRE(ctx, rows > 0 && H > 0 && hd > 0 && hd % 2 == 0, "gt_rope: rows %d H %d hd %d (hd must be even)", rows, H, hd);
  GT_REQUIRE(ctx, in && out, "gt_rope: null operand");
  int period = ctx->batch ? ctx->seq_len : rows;
  if (ctx->batch) GT_REQUIRE(ctx, rows == ctx->batch * ctx->seq_len, "gt_rope: %d rows but the batch is %d x %d", rows, ctx->batch, ctx->seq_len);
  const float2* tab = nullptr;
  gt_status s = rope_table(ctx, period, hd, base, pos_offset, &tab);
  if (s) return s;
  long npairs = (long)rows * H * (hd / 2);
  int grid = (int)min((long)ctx->sm_count * 16, (npairs + 255) / 256);
  rope_kernel<BWD><<<grid, 256, 0, ctx->stream>>>(npairs, H, hd, period, tab, in, out, accum);
  GT_LAUNCHED(ctx, "rope_kernel");
  return GT_OK;
}

}  // namespace

extern "C" {

gt_status gt_rope_fwd(gt_ctx* ctx, int32_t rows, int32_t H, int32_t hd, double base, int32_t pos_offset, gt_buf x, gt_buf y) {
  return rope_run<false>(ctx, rows, H, hd, base, pos_offset, gt_ptr<const float>(x), gt_ptr<float>(y), 0);
}

gt_status gt_rope_bwd(gt_ctx* ctx, int32_t rows, int32_t H, int32_t hd, double base, int32_t pos_offset, gt_buf gy, gt_buf gx, int32_t accum) {
  if (!gx) return GT_OK;
  return rope_run<true>(ctx, rows, H, hd, base, pos_offset, gt_ptr<const float>(gy), gt_ptr<float>(gx), accum);
}

gt_status gt_embedding_fwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf w, gt_buf ids, gt_buf out) {
  GT_REQUIRE(ctx, rows > 0 && d > 0 && w && ids && out, "gt_embedding_fwd: bad argument");
  long n = (long)rows * d;
  int grid = (int)min((long)ctx->sm_count * 16, (n + 255) / 256);
  embedding_fwd_kernel<<<grid, 256, 0, ctx->stream>>>(n, d, gt_ptr<const float>(w), gt_ptr<const uint32_t>(ids), gt_ptr<float>(out));
  GT_LAUNCHED(ctx, "embedding_fwd_kernel");
  return GT_OK;
}

gt_status gt_embedding_bwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf gy, gt_buf ids, gt_buf gw) {
  if (!gw) return GT_OK;
  GT_REQUIRE(ctx, rows > 0 && d > 0 && gy && ids, "gt_embedding_bwd: bad argument");
  long n = (long)rows * d;
  int grid = (int)min((long)ctx->sm_count * 16, (n + 255) / 256);
  embedding_bwd_kernel<<<grid, 256, 0, ctx->stream>>>(n, d, gt_ptr<const float>(gy), gt_ptr<const uint32_t>(ids), gt_ptr<float>(gw));
  GT_LAUNCHED(ctx, "embedding_bwd_kernel");
  return GT_OK;
}

}  // extern "C"
