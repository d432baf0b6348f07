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
                            const float* in, float* out, int accum) {   // in == out is allowed: a thread reads its pair before it writes it
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

// Four pairs per thread (hd a multiple of 8, 16-byte aligned operands, fewer than 2^31 pairs): two 16-byte loads of
// the row, two of the table, two 16-byte stores, 32-bit index arithmetic.
template <bool BWD>
__global__ void rope_vec_kernel(unsigned nvec, int H, int hd, int period, const float2* __restrict__ tab,
                                const float* in, float* out, int accum) {   // in == out is allowed, as above
  const unsigned half = hd >> 1, hv = half >> 2;
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const unsigned j = (i % hv) * 4, rh = i / hv;   // first pair of the four, row*H + h
    const unsigned t = (rh / (unsigned)H) % (unsigned)period;
    const float4* tp = reinterpret_cast<const float4*>(tab + (size_t)t * half + j);
    const float4 c01 = __ldg(tp), c23 = __ldg(tp + 1);   // (cos, sin) of pairs j..j+3
    const size_t b = (size_t)rh * hd + j;
    const float4 a0 = *reinterpret_cast<const float4*>(in + b), a1 = *reinterpret_cast<const float4*>(in + b + half);
    float4 o0, o1;
    if (!BWD) {
      o0 = make_float4(a0.x * c01.x - a1.x * c01.y, a0.y * c01.z - a1.y * c01.w, a0.z * c23.x - a1.z * c23.y, a0.w * c23.z - a1.w * c23.w);
      o1 = make_float4(a0.x * c01.y + a1.x * c01.x, a0.y * c01.w + a1.y * c01.z, a0.z * c23.y + a1.z * c23.x, a0.w * c23.w + a1.w * c23.z);
    } else {
      o0 = make_float4(c01.x * a0.x + c01.y * a1.x, c01.z * a0.y + c01.w * a1.y, c23.x * a0.z + c23.y * a1.z, c23.z * a0.w + c23.w * a1.w);
      o1 = make_float4(-c01.y * a0.x + c01.x * a1.x, -c01.w * a0.y + c01.z * a1.y, -c23.y * a0.z + c23.x * a1.z, -c23.w * a0.w + c23.z * a1.w);
    }
    float4* p0 = reinterpret_cast<float4*>(out + b);
    float4* p1 = reinterpret_cast<float4*>(out + b + half);
    if (accum) {
      const float4 q0 = *p0, q1 = *p1;
      o0 = make_float4(q0.x + o0.x, q0.y + o0.y, q0.z + o0.z, q0.w + o0.w);
      o1 = make_float4(q1.x + o1.x, q1.y + o1.y, q1.z + o1.z, q1.w + o1.w);
    }
    *p0 = o0;
    *p1 = o1;
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

// The same scatter-add with one owner per table row and a fixed order of additions (strict-f32 mode): the CTA of
// position t does nothing unless t is the first occurrence of its id; otherwise it marks every later occurrence in a
// shared-memory bitmap and each thread adds its columns over the marked rows in ascending position. This is the
// reference's rule (one owner per gradient element, src/backend/webgpu.ts:21-26) without its O(V) scan.
__global__ void __launch_bounds__(128) embedding_bwd_ordered_kernel(int rows, int d, const float* __restrict__ g,
                                                                    const uint32_t* __restrict__ ids, float* gw) {
  extern __shared__ uint32_t bits[];   // one bit per position
  const int t = blockIdx.x;
  const uint32_t id = ids[t];
  int earlier = 0;
  for (int u = threadIdx.x; u < t; u += blockDim.x) earlier |= (ids[u] == id);
  if (__syncthreads_or(earlier)) return;
  const int words = (rows + 31) >> 5;
  for (int wd = threadIdx.x; wd < words; wd += blockDim.x) bits[wd] = 0u;
  __syncthreads();
  for (int u = t + (int)threadIdx.x; u < rows; u += blockDim.x)
    if (ids[u] == id) atomicOr(&bits[u >> 5], 1u << (u & 31));
  __syncthreads();
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float acc = gw[(size_t)id * d + j];
    for (int wd = t >> 5; wd < words; wd++) {
      uint32_t m = bits[wd];
      while (m) {
        const int u = (wd << 5) + __ffs(m) - 1;
        m &= m - 1;
        acc += g[(size_t)u * d + j];
      }
    }
    gw[(size_t)id * d + j] = acc;
  }
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
  if (hd % 8 == 0 && npairs < (1l << 31) && ((((uintptr_t)in) | ((uintptr_t)out)) & 15) == 0) {
    const long nvec = npairs / 4;
    int grid = (int)min((long)ctx->sm_count * 8, (nvec + 255) / 256);
    rope_vec_kernel<BWD><<<grid, 256, 0, ctx->stream>>>((unsigned)nvec, H, hd, period, tab, in, out, accum);
    GT_LAUNCHED(ctx, "rope_vec_kernel");
    return GT_OK;
  }
  int grid = (int)min((long)ctx->sm_count * 16, (npairs + 255) / 256);
  rope_kernel<BWD><<<grid, 256, 0, ctx->stream>>>(npairs, H, hd, period, tab, in, out, accum);
  GT_LAUNCHED(ctx, "rope_kernel");
  return GT_OK;
}

}  // namespace

// For the kernels that apply the rotation themselves: the table of this shape (built on first use) and the number of
// positions it holds (the sequence length when a batch is set, else the row count).
gt_status gt_rope_table(gt_ctx* ctx, int rows, int hd, double base, int pos_offset, const float2** tab, int* period) {
  *period = ctx->batch ? ctx->seq_len : rows;
  if (ctx->batch) GT_REQUIRE(ctx, rows == ctx->batch * ctx->seq_len, "gt_rope: %d rows but the batch is %d x %d", rows, ctx->batch, ctx->seq_len);
  return rope_table(ctx, *period, hd, base, pos_offset, tab);
}

// The rotation (or its transpose) as a pass of its own; `in` may be `out` when accum is 0.
gt_status gt_rope_apply(gt_ctx* ctx, bool bwd, int rows, int H, int hd, double base, int pos_offset, const float* in, float* out, int accum) {
  return bwd ? rope_run<true>(ctx, rows, H, hd, base, pos_offset, in, out, accum) : rope_run<false>(ctx, rows, H, hd, base, pos_offset, in, out, accum);
}

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
  if (ctx->precision == GT_PREC_FP32 && rows <= 8 * 40960) {   // (the bitmap fits the default shared-memory limit)
    embedding_bwd_ordered_kernel<<<rows, 128, sizeof(uint32_t) * ((rows + 31) / 32), ctx->stream>>>(rows, d, gt_ptr<const float>(gy),
                                                                                                  gt_ptr<const uint32_t>(ids), gt_ptr<float>(gw));
    GT_LAUNCHED(ctx, "embedding_bwd_ordered_kernel");
    return GT_OK;
  }
  long n = (long)rows * d;
  int grid = (int)min((long)ctx->sm_count * 16, (n + 255) / 256);
  embedding_bwd_kernel<<<grid, 256, 0, ctx->stream>>>(n, d, gt_ptr<const float>(gy), gt_ptr<const uint32_t>(ids), gt_ptr<float>(gw));
  GT_LAUNCHED(ctx, "embedding_bwd_kernel");
  return GT_OK;
}

}  // extern "C"
