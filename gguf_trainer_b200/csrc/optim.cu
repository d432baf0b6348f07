// Device-resident optimizers: AdamW with global-norm clipping and Muon with quintic Newton-Schulz
// (src/train/adam.ts:46-82, src/train/muon.ts:69-158; GPU forms src/backend/adamw-gpu.ts:32-129 and
// src/backend/muon-gpu.ts:51-252). AdamW is HBM-bound at 28 B/parameter (read g, m, v, w; write m, v, w):
// one multi-tensor launch covers the whole group through a chunk table, 128-bit accesses. The
// Newton-Schulz products go through the same matrix-product path as the model's linears.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int CHUNK = 32768;  // elements per CTA
constexpr int OT = 256;

struct Chunk { int tensor; uint32_t start; uint32_t count; };

__device__ __forceinline__ float block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  if (threadIdx.x < 32) {
    r = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  return r;  // valid in thread 0
}

__global__ void __launch_bounds__(OT) sumsq_partial_kernel(const Chunk* __restrict__ chunks, float* const* __restrict__ grads,
                                                           float* __restrict__ partials) {
  __shared__ float sh[OT / 32];
  const Chunk c = chunks[blockIdx.x];
  const float* g = grads[c.tensor] + c.start;
  float s = 0.f;
  const uint32_t n4 = ((((uintptr_t)g) & 15) == 0) ? c.count / 4 : 0;
  for (uint32_t i = threadIdx.x; i < n4; i += OT) {
    float4 x = ((const float4*)g)[i];
    s = fmaf(x.x, x.x, s); s = fmaf(x.y, x.y, s); s = fmaf(x.z, x.z, s); s = fmaf(x.w, x.w, s);
  }
  for (uint32_t i = n4 * 4 + threadIdx.x; i < c.count; i += OT) s = fmaf(g[i], g[i], s);
  s = block_sum(s, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

// same reduction over one plain array; CTA b covers elements [b*CHUNK, (b+1)*CHUNK)
__global__ void __launch_bounds__(OT) sumsq_direct_kernel(const float* __restrict__ g, size_t n, float* __restrict__ partials) {
  __shared__ float sh[OT / 32];
  size_t start = (size_t)blockIdx.x * CHUNK;
  size_t end = start + CHUNK < n ? start + CHUNK : n;
  float s = 0.f;
  for (size_t i = start + threadIdx.x; i < end; i += OT) s = fmaf(g[i], g[i], s);
  s = block_sum(s, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

// mode 0: out[0] = clip scale (norm > clip ? clip/(norm+1e-12) : 1)   (adam.ts:51-62)
// mode 1: out[0] = 1/(sqrt(sum)+1e-7)                                  (muon.ts:140-141)
__global__ void __launch_bounds__(1024) sumsq_final_kernel(int n, const float* __restrict__ partials, int mode, float clip,
                                                           float* __restrict__ out) {
  __shared__ double sh[32];
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += (double)partials[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += sh[i];
    double norm = sqrt(t);
    if (mode == 0) out[0] = norm > (double)clip ? (float)((double)clip / (norm + 1e-12)) : 1.f;
    else out[0] = (float)(1.0 / (norm + 1e-7));
  }
}

__global__ void __launch_bounds__(OT) adamw_kernel(const Chunk* __restrict__ chunks, float* const* __restrict__ datas,
                                                   float* const* __restrict__ grads, float* const* __restrict__ ms,
                                                   float* const* __restrict__ vs, const float* __restrict__ scale_p, float lr,
                                                   float bc1, float bc2, float b1, float b2, float eps, float wd) {
  const Chunk c = chunks[blockIdx.x];
  float* w = datas[c.tensor] + c.start;
  const float* g = grads[c.tensor] + c.start;
  float* m = ms[c.tensor] + c.start;
  float* v = vs[c.tensor] + c.start;
  const float scale = scale_p ? scale_p[0] : 1.f;
  const float ib1 = 1.f / bc1, ib2 = 1.f / bc2;
  auto upd = [&](float gi, float& mi, float& vi, float& wi) {
    float gg = gi * scale;
    mi = b1 * mi + (1.f - b1) * gg;
    vi = b2 * vi + (1.f - b2) * gg * gg;
    float u = (mi * ib1) / (sqrtf(vi * ib2) + eps);
    if (wd > 0.f) u += wd * wi;
    wi -= lr * u;
  };
  const bool al = (((uintptr_t)w | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0;
  const uint32_t n4 = al ? c.count / 4 : 0;
  for (uint32_t i = threadIdx.x; i < n4; i += OT) {
    float4 G = ((const float4*)g)[i], M = ((float4*)m)[i], V = ((float4*)v)[i], W = ((float4*)w)[i];
    upd(G.x, M.x, V.x, W.x); upd(G.y, M.y, V.y, W.y); upd(G.z, M.z, V.z, W.z); upd(G.w, M.w, V.w, W.w);
    ((float4*)m)[i] = M; ((float4*)v)[i] = V; ((float4*)w)[i] = W;
  }
  for (uint32_t i = n4 * 4 + threadIdx.x; i < c.count; i += OT) {
    float M = m[i], V = v[i], W = w[i];
    upd(g[i], M, V, W);
    m[i] = M; v[i] = V; w[i] = W;
  }
}

// ---- Muon elementwise pieces ----
// X[r,c] = (flip ? U^T : U) * inv[0], U is [m,n]   (srcNormalize muon-gpu.ts:100-135)
__global__ void muon_normalize_kernel(int m, int n, int flip, const float* __restrict__ U, const float* __restrict__ inv,
                                      float* __restrict__ X) {
  size_t total = (size_t)m * n, stride = (size_t)gridDim.x * blockDim.x;
  const float s = inv[0];
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    if (!flip) { X[i] = U[i] * s; }
    else { size_t a = i / m, b = i % m; X[i] = U[b * n + a] * s; }  // X is [n, m]: X[a][b] = U[b][a]
  }
}
// out = ca*a + cb*b
__global__ void axpby_kernel(size_t n, float ca, const float* __restrict__ a, float cb, const float* __restrict__ b, float* out) {
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = ca * a[i] + cb * b[i];
}
// W[m,n] -= lr*scale * (flip ? X^T : X)    (srcApply muon-gpu.ts:173-190)
__global__ void muon_apply_kernel(int m, int n, int flip, float f, const float* __restrict__ X, float* __restrict__ W) {
  size_t total = (size_t)m * n, stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    float o;
    if (!flip) o = X[i];
    else { size_t a = i / n, b = i % n; o = X[b * m + a]; }  // W[a][b] uses X[b][a], X is [n, m]
    W[i] -= f * o;
  }
}

// ---- the same pieces over a group of same-shape matrices: blockIdx.y = matrix, workspaces are [nb, rows, cols] ----
__global__ void muon_momentum_batched_kernel(size_t el, float* const* __restrict__ grads, float* const* __restrict__ bufs,
                                             float* __restrict__ U, float mu, int nesterov) {
  const int b = blockIdx.y;
  const float* g = grads[b];
  float* buf = bufs[b];
  float* u = U + (size_t)b * el;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < el; i += stride) {
    float v = mu * buf[i] + g[i];
    buf[i] = v;
    u[i] = nesterov ? g[i] + mu * v : v;
  }
}
// 16-byte forms of the batched pieces (el % 4 == 0, 16-byte aligned matrices), without the transposition: the
// Newton-Schulz products are issued in the layout the matrix is stored in (see gt_muon_step).
__global__ void muon_momentum_batched_v4_kernel(size_t el4, float* const* __restrict__ grads, float* const* __restrict__ bufs,
                                                float* __restrict__ U, float mu, int nesterov) {
  const int b = blockIdx.y;
  const float4* g = reinterpret_cast<const float4*>(grads[b]);
  float4* buf = reinterpret_cast<float4*>(bufs[b]);
  float4* u = reinterpret_cast<float4*>(U) + (size_t)b * el4;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < el4; i += stride) {
    const float4 gv = g[i];
    float4 v = buf[i];
    v.x = mu * v.x + gv.x; v.y = mu * v.y + gv.y; v.z = mu * v.z + gv.z; v.w = mu * v.w + gv.w;
    buf[i] = v;
    u[i] = nesterov ? make_float4(gv.x + mu * v.x, gv.y + mu * v.y, gv.z + mu * v.z, gv.w + mu * v.w) : v;
  }
}
// X = U * inv[matrix]
__global__ void muon_scale_batched_v4_kernel(size_t el4, const float* __restrict__ U, const float* __restrict__ inv, float* __restrict__ X) {
  const int b = blockIdx.y;
  const float s = inv[b];
  const float4* u = reinterpret_cast<const float4*>(U) + (size_t)b * el4;
  float4* x = reinterpret_cast<float4*>(X) + (size_t)b * el4;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < el4; i += stride) {
    const float4 v = u[i];
    x[i] = make_float4(v.x * s, v.y * s, v.z * s, v.w * s);
  }
}
// W -= f * X
__global__ void muon_apply_batched_v4_kernel(size_t el4, float f, const float* __restrict__ X, float* const* __restrict__ datas) {
  const int b = blockIdx.y;
  const float4* x = reinterpret_cast<const float4*>(X) + (size_t)b * el4;
  float4* w = reinterpret_cast<float4*>(datas[b]);
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < el4; i += stride) {
    const float4 o = x[i];
    float4 v = w[i];
    v.x -= f * o.x; v.y -= f * o.y; v.z -= f * o.z; v.w -= f * o.w;
    w[i] = v;
  }
}
// B' = ca*I + cb*A + cc*AA over nb matrices of r x r, written over AA: then a*X + (b*A + c*A.A).X is the one product B'.X
__global__ void ns_poly_batched_kernel(size_t n, int r, float ca, float cb, const float* __restrict__ A, float cc, float* AA) {
  size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t rr = (size_t)r * r;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const size_t e = i % rr;
    AA[i] = cb * A[i] + cc * AA[i] + ((e / r == e % r) ? ca : 0.f);
  }
}
__global__ void __launch_bounds__(OT) sumsq_batched_kernel(const float* __restrict__ U, size_t el, int nch, float* __restrict__ partials) {
  __shared__ float sh[OT / 32];
  const int b = blockIdx.y;
  const float* g = U + (size_t)b * el;
  size_t start = (size_t)blockIdx.x * CHUNK;
  size_t end = start + CHUNK < el ? start + CHUNK : el;
  float s = 0.f;
  for (size_t i = start + threadIdx.x; i < end; i += OT) s = fmaf(g[i], g[i], s);
  s = block_sum(s, sh);
  if (threadIdx.x == 0) partials[(size_t)b * nch + blockIdx.x] = s;
}
__global__ void frob_inv_batched_kernel(int nch, const float* __restrict__ partials, float* __restrict__ inv) {
  // one small CTA per matrix, fixed order
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < nch; i++) t += (double)partials[(size_t)b * nch + i];
    inv[b] = (float)(1.0 / (sqrt(t) + 1e-7));
  }
}
__global__ void muon_normalize_batched_kernel(int m, int n, int flip, const float* __restrict__ U, const float* __restrict__ inv,
                                              float* __restrict__ X) {
  const int b = blockIdx.y;
  size_t total = (size_t)m * n, stride = (size_t)gridDim.x * blockDim.x;
  const float s = inv[b];
  const float* u = U + (size_t)b * total;
  float* x = X + (size_t)b * total;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    if (!flip) x[i] = u[i] * s;
    else { size_t a = i / m, c = i % m; x[i] = u[c * n + a] * s; }
  }
}
__global__ void muon_apply_batched_kernel(int m, int n, int flip, float f, const float* __restrict__ X, float* const* __restrict__ datas) {
  const int b = blockIdx.y;
  size_t total = (size_t)m * n, stride = (size_t)gridDim.x * blockDim.x;
  const float* x = X + (size_t)b * total;
  float* w = datas[b];
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    float o;
    if (!flip) o = x[i];
    else { size_t a = i / n, c = i % n; o = x[c * m + a]; }
    w[i] -= f * o;
  }
}

inline int egrid(gt_ctx* ctx, size_t n) {
  size_t want = (n + 255) / 256, cap = (size_t)ctx->sm_count * 8;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

struct GtAdamW {
  int n = 0;
  std::vector<float*> data, grad, m, v;
  std::vector<uint64_t> sizes;
  float lr, b1, b2, eps, wd, clip;
  int t = 0;
  int nchunks = 0;
  Chunk* d_chunks = nullptr;
  float** d_ptrs = nullptr;  // [4][n]: data, grad, m, v
  float* d_partials = nullptr;
  float* d_scale = nullptr;
};

// Matrices of one shape are orthogonalised together: one launch of each elementwise piece and one batched matrix
// product per Newton-Schulz step for the whole group (the reference records a separate dispatch chain per matrix,
// src/backend/muon-gpu.ts:385-411).
struct MuonGroup {
  int rows = 0, cols = 0, nb = 0;
  std::vector<int> idx;
  float *U = nullptr, *X = nullptr, *BX = nullptr, *A = nullptr, *AA = nullptr, *partials = nullptr, *inv = nullptr;
  float** d_ptrs = nullptr;   // [3][nb]: grad, momentum, data
  bool v4 = false;            // every matrix of the group 16-byte aligned and a multiple of 4 elements
};

struct GtMuon {
  std::vector<MuonGroup> groups;
  int n = 0;
  std::vector<float*> data, grad, buf;
  std::vector<int> rows, cols;
  float lr, mu;
  int nesterov, ns;
  bool sharded = false;   // Newton-Schulz work split over the data-parallel ranks (gt_muon_set_sharded)
  // workspaces sized for the largest matrix
  float *U = nullptr, *X = nullptr, *BX = nullptr, *A = nullptr, *AA = nullptr, *partials = nullptr, *inv = nullptr;
  size_t maxel = 0;
  int maxr = 0;
};

static gt_status dev_alloc(gt_ctx* ctx, void** p, size_t bytes, bool zero) {
  GT_CUDA(ctx, cudaMalloc(p, bytes < 256 ? 256 : bytes));
  if (zero) GT_CUDA(ctx, cudaMemsetAsync(*p, 0, bytes, ctx->stream));
  ctx->state_bytes += bytes;
  return GT_OK;
}

// Newton-Schulz on X [r,c] in place using A, AA [r,r] and BX [r,c]  (muon.ts:143-155, muon-gpu.ts:224-252)
static gt_status ns_iterations(gt_ctx* ctx, int r, int c, int steps, float* X, float* A, float* AA, float* BX) {
  for (int s = 0; s < steps; s++) {
    gt_status st = gt_gemm(ctx, GT_GEMM_NT, 0, r, r, c, (gt_buf)(uintptr_t)X, (gt_buf)(uintptr_t)X, (gt_buf)(uintptr_t)A);
    if (st) return st;
    st = gt_gemm(ctx, GT_GEMM_NN, 0, r, r, r, (gt_buf)(uintptr_t)A, (gt_buf)(uintptr_t)A, (gt_buf)(uintptr_t)AA);
    if (st) return st;
    axpby_kernel<<<egrid(ctx, (size_t)r * r), 256, 0, ctx->stream>>>((size_t)r * r, -4.7750f, A, 2.0315f, AA, AA);
    GT_LAUNCHED(ctx, "axpby_kernel");
    st = gt_gemm(ctx, GT_GEMM_NN, 0, r, c, r, (gt_buf)(uintptr_t)AA, (gt_buf)(uintptr_t)X, (gt_buf)(uintptr_t)BX);
    if (st) return st;
    axpby_kernel<<<egrid(ctx, (size_t)r * c), 256, 0, ctx->stream>>>((size_t)r * c, 3.4445f, X, 1.f, BX, X);
    GT_LAUNCHED(ctx, "axpby_kernel");
  }
  return GT_OK;
}

// inv[0] = 1/(||U||_F + 1e-7) for one array of n elements, using `partials` (>= ceil(n/CHUNK) floats)
static gt_status frob_inv(gt_ctx* ctx, const float* U, size_t n, float* partials, float* inv) {
  int nch = gt_cdiv((long)n, CHUNK);
  sumsq_direct_kernel<<<nch, OT, 0, ctx->stream>>>(U, n, partials);
  GT_LAUNCHED(ctx, "sumsq_direct_kernel");
  sumsq_final_kernel<<<1, 1024, 0, ctx->stream>>>(nch, partials, 1, 0.f, inv);
  GT_LAUNCHED(ctx, "sumsq_final_kernel");
  return GT_OK;
}

void gt_optim_destroy(gt_ctx* ctx) {
  for (GtAdamW* a : ctx->adamws) {
    if (!a) continue;
    for (float* p : a->m) cudaFree(p);
    for (float* p : a->v) cudaFree(p);
    cudaFree(a->d_chunks); cudaFree(a->d_ptrs); cudaFree(a->d_partials); cudaFree(a->d_scale);
    delete a;
  }
  ctx->adamws.clear();
  for (GtMuon* m : ctx->muons) {
    if (!m) continue;
    for (float* p : m->buf) cudaFree(p);
    for (auto& g : m->groups) { cudaFree(g.U); cudaFree(g.X); cudaFree(g.BX); cudaFree(g.A); cudaFree(g.AA); cudaFree(g.partials); cudaFree(g.inv); cudaFree(g.d_ptrs); }
    cudaFree(m->U); cudaFree(m->X); cudaFree(m->BX); cudaFree(m->A); cudaFree(m->AA); cudaFree(m->partials); cudaFree(m->inv);
    delete m;
  }
  ctx->muons.clear();
}

extern "C" {

gt_status gt_adamw_create(gt_ctx* ctx, int32_t n, const gt_buf* data, const gt_buf* grad, const uint64_t* sizes, float lr,
                          float beta1, float beta2, float eps, float weight_decay, float clip, uint64_t* out_handle) {
  GT_REQUIRE(ctx, n >= 0 && out_handle, "gt_adamw_create: bad argument");
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_adamw_create inside a graph capture");
  GtAdamW* a = new GtAdamW();
  a->n = n; a->lr = lr; a->b1 = beta1; a->b2 = beta2; a->eps = eps; a->wd = weight_decay; a->clip = clip;
  std::vector<Chunk> chunks;
  for (int i = 0; i < n; i++) {
    if (!data[i] || !grad[i] || sizes[i] == 0 || sizes[i] > 0xffffffffull) {
      delete a;
      return gt_fail(ctx, GT_ERR_ARG, "gt_adamw_create: tensor %d has a null buffer or an unsupported size", i);
    }
    a->data.push_back(gt_ptr<float>(data[i]));
    a->grad.push_back(gt_ptr<float>(grad[i]));
    a->sizes.push_back(sizes[i]);
    float *m = nullptr, *v = nullptr;
    gt_status s = dev_alloc(ctx, (void**)&m, sizeof(float) * sizes[i], true);
    if (!s) s = dev_alloc(ctx, (void**)&v, sizeof(float) * sizes[i], true);
    if (s) { delete a; return s; }
    a->m.push_back(m); a->v.push_back(v);
    for (uint64_t st = 0; st < sizes[i]; st += CHUNK)
      chunks.push_back(Chunk{i, (uint32_t)st, (uint32_t)(st + CHUNK <= sizes[i] ? CHUNK : sizes[i] - st)});
  }
  a->nchunks = (int)chunks.size();
  if (n > 0) {
    gt_status s = dev_alloc(ctx, (void**)&a->d_chunks, sizeof(Chunk) * chunks.size(), false);
    if (!s) s = dev_alloc(ctx, (void**)&a->d_ptrs, sizeof(float*) * 4 * n, false);
    if (!s) s = dev_alloc(ctx, (void**)&a->d_partials, sizeof(float) * chunks.size(), false);
    if (!s) s = dev_alloc(ctx, (void**)&a->d_scale, 256, true);
    if (s) { delete a; return s; }
    std::vector<float*> ptrs;
    ptrs.insert(ptrs.end(), a->data.begin(), a->data.end());
    ptrs.insert(ptrs.end(), a->grad.begin(), a->grad.end());
    ptrs.insert(ptrs.end(), a->m.begin(), a->m.end());
    ptrs.insert(ptrs.end(), a->v.begin(), a->v.end());
    GT_CUDA(ctx, cudaMemcpyAsync(a->d_chunks, chunks.data(), sizeof(Chunk) * chunks.size(), cudaMemcpyHostToDevice, ctx->stream));
    GT_CUDA(ctx, cudaMemcpyAsync(a->d_ptrs, ptrs.data(), sizeof(float*) * ptrs.size(), cudaMemcpyHostToDevice, ctx->stream));
    GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  ctx->adamws.push_back(a);
  *out_handle = ctx->adamws.size();
  return GT_OK;
}

static GtAdamW* adamw_of(gt_ctx* ctx, uint64_t h) {
  if (h < 1 || h > ctx->adamws.size()) return nullptr;
  return ctx->adamws[h - 1];
}

gt_status gt_adamw_set_lr(gt_ctx* ctx, uint64_t h, float lr) {
  GtAdamW* a = adamw_of(ctx, h);
  GT_REQUIRE(ctx, a, "gt_adamw_set_lr: bad handle");
  a->lr = lr;
  return GT_OK;
}

gt_status gt_adamw_step(gt_ctx* ctx, uint64_t h) {
  GtAdamW* a = adamw_of(ctx, h);
  GT_REQUIRE(ctx, a, "gt_adamw_step: bad handle");
  a->t += 1;
  if (a->n == 0) return GT_OK;
  float** P = a->d_ptrs;
  const float* scale = nullptr;
  if (a->clip > 0.f) {
    sumsq_partial_kernel<<<a->nchunks, OT, 0, ctx->stream>>>(a->d_chunks, P + a->n, a->d_partials);
    GT_LAUNCHED(ctx, "sumsq_partial_kernel");
    sumsq_final_kernel<<<1, 1024, 0, ctx->stream>>>(a->nchunks, a->d_partials, 0, a->clip, a->d_scale);
    GT_LAUNCHED(ctx, "sumsq_final_kernel");
    scale = a->d_scale;
  }
  float bc1 = (float)(1.0 - pow((double)a->b1, (double)a->t));
  float bc2 = (float)(1.0 - pow((double)a->b2, (double)a->t));
  adamw_kernel<<<a->nchunks, OT, 0, ctx->stream>>>(a->d_chunks, P, P + a->n, P + 2 * a->n, P + 3 * a->n, scale, a->lr, bc1, bc2,
                                                   a->b1, a->b2, a->eps, a->wd);
  GT_LAUNCHED(ctx, "adamw_kernel");
  return GT_OK;
}

gt_status gt_adamw_state(gt_ctx* ctx, uint64_t h, int32_t i, gt_buf* m, gt_buf* v) {
  GtAdamW* a = adamw_of(ctx, h);
  GT_REQUIRE(ctx, a && i >= 0 && i < a->n, "gt_adamw_state: bad handle or index");
  *m = (gt_buf)(uintptr_t)a->m[i];
  *v = (gt_buf)(uintptr_t)a->v[i];
  return GT_OK;
}
gt_status gt_adamw_get_t(gt_ctx* ctx, uint64_t h, int32_t* t) {
  GtAdamW* a = adamw_of(ctx, h);
  GT_REQUIRE(ctx, a, "gt_adamw_get_t: bad handle");
  *t = a->t;
  return GT_OK;
}
gt_status gt_adamw_set_t(gt_ctx* ctx, uint64_t h, int32_t t) {
  GtAdamW* a = adamw_of(ctx, h);
  GT_REQUIRE(ctx, a && t >= 0, "gt_adamw_set_t: bad handle or step");
  a->t = t;
  return GT_OK;
}

gt_status gt_muon_create(gt_ctx* ctx, int32_t n, const gt_buf* data, const gt_buf* grad, const int32_t* rows, const int32_t* cols,
                         float lr, float momentum, int32_t nesterov, int32_t ns_steps, uint64_t* out_handle) {
  GT_REQUIRE(ctx, n >= 0 && out_handle && ns_steps >= 0, "gt_muon_create: bad argument");
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_muon_create inside a graph capture");
  GtMuon* m = new GtMuon();
  m->n = n; m->lr = lr; m->mu = momentum; m->nesterov = nesterov; m->ns = ns_steps;
  for (int i = 0; i < n; i++) {
    if (!data[i] || !grad[i] || rows[i] <= 0 || cols[i] <= 0) { delete m; return gt_fail(ctx, GT_ERR_ARG, "gt_muon_create: matrix %d is malformed", i); }
    m->data.push_back(gt_ptr<float>(data[i]));
    m->grad.push_back(gt_ptr<float>(grad[i]));
    m->rows.push_back(rows[i]); m->cols.push_back(cols[i]);
    size_t el = (size_t)rows[i] * cols[i];
    float* b = nullptr;
    gt_status s = dev_alloc(ctx, (void**)&b, sizeof(float) * el, true);
    if (s) { delete m; return s; }
    m->buf.push_back(b);
    if (el > m->maxel) m->maxel = el;
    int r = rows[i] < cols[i] ? rows[i] : cols[i];
    if (r > m->maxr) m->maxr = r;
  }
  // group by shape, in first-seen order
  for (int i = 0; i < n; i++) {
    MuonGroup* g = nullptr;
    for (auto& gg : m->groups) if (gg.rows == m->rows[i] && gg.cols == m->cols[i]) { g = &gg; break; }
    if (!g) { m->groups.emplace_back(); g = &m->groups.back(); g->rows = m->rows[i]; g->cols = m->cols[i]; }
    g->idx.push_back(i);
  }
  for (auto& g : m->groups) {
    g.nb = (int)g.idx.size();
    const size_t el = (size_t)g.rows * g.cols;
    const int r = g.rows < g.cols ? g.rows : g.cols;
    const int nch = gt_cdiv((long)el, CHUNK);
    gt_status s = dev_alloc(ctx, (void**)&g.U, sizeof(float) * el * g.nb, false);
    if (!s) s = dev_alloc(ctx, (void**)&g.X, sizeof(float) * el * g.nb, false);
    if (!s) s = dev_alloc(ctx, (void**)&g.BX, sizeof(float) * el * g.nb, false);
    if (!s) s = dev_alloc(ctx, (void**)&g.A, sizeof(float) * (size_t)r * r * g.nb, false);
    if (!s) s = dev_alloc(ctx, (void**)&g.AA, sizeof(float) * (size_t)r * r * g.nb, false);
    if (!s) s = dev_alloc(ctx, (void**)&g.partials, sizeof(float) * (size_t)nch * g.nb, false);
    if (!s) s = dev_alloc(ctx, (void**)&g.inv, sizeof(float) * g.nb, true);
    if (!s) s = dev_alloc(ctx, (void**)&g.d_ptrs, sizeof(float*) * 3 * g.nb, false);
    if (s) { delete m; return s; }
    std::vector<float*> ptrs;
    for (int i : g.idx) ptrs.push_back(m->grad[i]);
    for (int i : g.idx) ptrs.push_back(m->buf[i]);
    for (int i : g.idx) ptrs.push_back(m->data[i]);
    g.v4 = (el % 4) == 0;
    for (float* q : ptrs) g.v4 = g.v4 && (((uintptr_t)q) & 15) == 0;
    GT_CUDA(ctx, cudaMemcpyAsync(g.d_ptrs, ptrs.data(), sizeof(float*) * ptrs.size(), cudaMemcpyHostToDevice, ctx->stream));
    GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  ctx->muons.push_back(m);
  *out_handle = ctx->muons.size();
  return GT_OK;
}

static GtMuon* muon_of(gt_ctx* ctx, uint64_t h) {
  if (h < 1 || h > ctx->muons.size()) return nullptr;
  return ctx->muons[h - 1];
}

gt_status gt_muon_set_lr(gt_ctx* ctx, uint64_t h, float lr) {
  GtMuon* m = muon_of(ctx, h);
  GT_REQUIRE(ctx, m, "gt_muon_set_lr: bad handle");
  m->lr = lr;
  return GT_OK;
}

// Every rank of a data-parallel job holds the same gradients after the exchange and would run the same Newton-Schulz
// iterations on all matrices. Sharded, rank r orthogonalises matrices [r*slice, (r+1)*slice) of each same-shape group
// (slice = ceil(nb / world)) and the ranks exchange the results with one all-gather per group, so the iteration's
// products cost 1/world per rank; momentum and the apply pass stay replicated (they are what keeps state and weights
// identical everywhere). The group's two iteration buffers are re-made with room for world*slice matrices.
gt_status gt_muon_set_sharded(gt_ctx* ctx, uint64_t h, int32_t on) {
  GtMuon* m = muon_of(ctx, h);
  GT_REQUIRE(ctx, m, "gt_muon_set_sharded: bad handle");
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_muon_set_sharded inside a graph capture");
  if (!on) { m->sharded = false; return GT_OK; }
  int rank = 0, world = 1;
  gt_status s = gt_dp_rank(ctx, &rank, &world);
  if (s) return s;
  GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (auto& g : m->groups) {
    if (!g.v4) continue;
    const size_t el = (size_t)g.rows * g.cols;
    const int slice = gt_cdiv(g.nb, world);
    const size_t want = sizeof(float) * el * (size_t)slice * world;
    if (want > sizeof(float) * el * g.nb) {
      cudaFree(g.X); cudaFree(g.BX);
      g.X = g.BX = nullptr;
      s = dev_alloc(ctx, (void**)&g.X, want, true);
      if (!s) s = dev_alloc(ctx, (void**)&g.BX, want, true);
      if (s) return s;
    }
  }
  m->sharded = true;
  return GT_OK;
}

gt_status gt_muon_step(gt_ctx* ctx, uint64_t h) {
  GtMuon* m = muon_of(ctx, h);
  GT_REQUIRE(ctx, m, "gt_muon_step: bad handle");
  int dp_rank = 0, dp_world = 1;
  if (m->sharded) {
    gt_status s = gt_dp_rank(ctx, &dp_rank, &dp_world);
    if (s) return s;
  }
  for (auto& g : m->groups) {
    const int rows = g.rows, cols = g.cols, nb = g.nb;
    const size_t el = (size_t)rows * cols;
    const int flip = rows > cols;
    const int r = flip ? cols : rows, c = flip ? rows : cols;
    const int nch = gt_cdiv((long)el, CHUNK);
    const dim3 eg((unsigned)max(1, min(egrid(ctx, el), (ctx->sm_count * 8 + nb - 1) / nb)), (unsigned)nb);
    float** P = g.d_ptrs;
    const float f = m->lr * sqrtf(fmaxf(1.f, (float)rows / (float)cols));
    if (g.v4) {
      // The iteration runs on the matrix as it is stored. The reference transposes a tall matrix first so that
      // A = X.X^T is the small Gram matrix (muon.ts:120-131); here the same Gram matrix is X^T.X (a TN product) and the
      // update X.B'^T (an NT product), so no transposed copy is made. And a*X + (b*A + c*A.A).X is formed as ONE
      // product B'.X with B' = a*I + b*A + c*A.A, into the other of two buffers, instead of a product and a pass.
      const size_t el4 = el / 4;
      muon_momentum_batched_v4_kernel<<<eg, 256, 0, ctx->stream>>>(el4, P, P + nb, g.U, m->mu, m->nesterov);
      GT_LAUNCHED(ctx, "muon_momentum_batched_v4_kernel");
      sumsq_batched_kernel<<<dim3(nch, nb), OT, 0, ctx->stream>>>(g.U, el, nch, g.partials);
      GT_LAUNCHED(ctx, "sumsq_batched_kernel");
      frob_inv_batched_kernel<<<nb, 32, 0, ctx->stream>>>(nch, g.partials, g.inv);
      GT_LAUNCHED(ctx, "frob_inv_batched_kernel");
      float *X = g.X, *Y = g.BX;
      muon_scale_batched_v4_kernel<<<eg, 256, 0, ctx->stream>>>(el4, g.U, g.inv, X);
      GT_LAUNCHED(ctx, "muon_scale_batched_v4_kernel");
      // this rank's share of the group's matrices: all of them, or its slice when the work is sharded
      const int slice = gt_cdiv(nb, dp_world);
      const int lo = m->sharded ? min(nb, dp_rank * slice) : 0, hi = m->sharded ? min(nb, lo + slice) : nb;
      const int mine = hi - lo;
      for (int it = 0; it < m->ns; it++) {
        float *Xs = X + (size_t)lo * el, *Ys = Y + (size_t)lo * el;
        if (mine > 0) {
          gt_status st = flip ? gt_gemm_batched(ctx, GT_GEMM_TN, 0, r, r, c, Xs, Xs, g.A, mine)   // X is [c, r]: A = X^T.X
                              : gt_gemm_batched(ctx, GT_GEMM_NT, 0, r, r, c, Xs, Xs, g.A, mine);  // X is [r, c]: A = X.X^T
          if (st) return st;
          st = gt_gemm_batched(ctx, GT_GEMM_NN, 0, r, r, r, g.A, g.A, g.AA, mine);
          if (st) return st;
          const size_t rr = (size_t)r * r * mine;
          ns_poly_batched_kernel<<<egrid(ctx, rr), 256, 0, ctx->stream>>>(rr, r, 3.4445f, -4.7750f, g.A, 2.0315f, g.AA);
          GT_LAUNCHED(ctx, "ns_poly_batched_kernel");
          st = flip ? gt_gemm_batched(ctx, GT_GEMM_NT, 0, c, r, r, Xs, g.AA, Ys, mine)             // [c, r] = X.B'^T
                    : gt_gemm_batched(ctx, GT_GEMM_NN, 0, r, c, r, g.AA, Xs, Ys, mine);            // [r, c] = B'.X
          if (st) return st;
        }
        float* t = X; X = Y; Y = t;
      }
      if (m->sharded && dp_world > 1) {   // every rank's slice of the orthogonalised matrices, to every rank
        gt_status st = gt_dp_allgather(ctx, X, (size_t)slice * el);
        if (st) return st;
      }
      muon_apply_batched_v4_kernel<<<eg, 256, 0, ctx->stream>>>(el4, f, X, P + 2 * nb);
      GT_LAUNCHED(ctx, "muon_apply_batched_v4_kernel");
      continue;
    }
    muon_momentum_batched_kernel<<<eg, 256, 0, ctx->stream>>>(el, P, P + nb, g.U, m->mu, m->nesterov);
    GT_LAUNCHED(ctx, "muon_momentum_batched_kernel");
    sumsq_batched_kernel<<<dim3(nch, nb), OT, 0, ctx->stream>>>(g.U, el, nch, g.partials);
    GT_LAUNCHED(ctx, "sumsq_batched_kernel");
    frob_inv_batched_kernel<<<nb, 32, 0, ctx->stream>>>(nch, g.partials, g.inv);
    GT_LAUNCHED(ctx, "frob_inv_batched_kernel");
    muon_normalize_batched_kernel<<<eg, 256, 0, ctx->stream>>>(rows, cols, flip, g.U, g.inv, g.X);
    GT_LAUNCHED(ctx, "muon_normalize_batched_kernel");
    for (int it = 0; it < m->ns; it++) {   // A = X.X^T ; AA = A.A ; B = b*A + c*AA ; X = a*X + B.X   (muon.ts:143-155)
      gt_status st = gt_gemm_batched(ctx, GT_GEMM_NT, 0, r, r, c, g.X, g.X, g.A, nb);
      if (st) return st;
      st = gt_gemm_batched(ctx, GT_GEMM_NN, 0, r, r, r, g.A, g.A, g.AA, nb);
      if (st) return st;
      const size_t rr = (size_t)r * r * nb;
      axpby_kernel<<<egrid(ctx, rr), 256, 0, ctx->stream>>>(rr, -4.7750f, g.A, 2.0315f, g.AA, g.AA);
      GT_LAUNCHED(ctx, "axpby_kernel");
      st = gt_gemm_batched(ctx, GT_GEMM_NN, 0, r, c, r, g.AA, g.X, g.BX, nb);
      if (st) return st;
      axpby_kernel<<<egrid(ctx, el * nb), 256, 0, ctx->stream>>>(el * nb, 3.4445f, g.X, 1.f, g.BX, g.X);
      GT_LAUNCHED(ctx, "axpby_kernel");
    }
    muon_apply_batched_kernel<<<eg, 256, 0, ctx->stream>>>(rows, cols, flip, f, g.X, P + 2 * nb);
    GT_LAUNCHED(ctx, "muon_apply_batched_kernel");
  }
  return GT_OK;
}

gt_status gt_muon_state(gt_ctx* ctx, uint64_t h, int32_t i, gt_buf* momentum) {
  GtMuon* m = muon_of(ctx, h);
  GT_REQUIRE(ctx, m && i >= 0 && i < m->n, "gt_muon_state: bad handle or index");
  *momentum = (gt_buf)(uintptr_t)m->buf[i];
  return GT_OK;
}

gt_status gt_newton_schulz(gt_ctx* ctx, int32_t mm, int32_t nn, int32_t steps, gt_buf g, gt_buf out) {
  GT_REQUIRE(ctx, mm > 0 && nn > 0 && steps >= 0 && g && out, "gt_newton_schulz: bad argument");
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_newton_schulz inside a graph capture");
  const size_t el = (size_t)mm * nn;
  const int flip = mm > nn;
  const int r = flip ? nn : mm, c = flip ? mm : nn;
  float *X, *BX, *A, *AA, *partials, *inv;
  GT_CUDA(ctx, cudaMalloc(&X, sizeof(float) * el)); GT_CUDA(ctx, cudaMalloc(&BX, sizeof(float) * el));
  GT_CUDA(ctx, cudaMalloc(&A, sizeof(float) * r * r)); GT_CUDA(ctx, cudaMalloc(&AA, sizeof(float) * r * r));
  GT_CUDA(ctx, cudaMalloc(&partials, sizeof(float) * (el / CHUNK + 2))); GT_CUDA(ctx, cudaMalloc(&inv, 256));
  gt_status s = frob_inv(ctx, gt_ptr<const float>(g), el, partials, inv);
  if (!s) {
    muon_normalize_kernel<<<egrid(ctx, el), 256, 0, ctx->stream>>>(mm, nn, flip, gt_ptr<const float>(g), inv, X);
    ctx->launches++;
    s = ns_iterations(ctx, r, c, steps, X, A, AA, BX);
  }
  if (!s) {
    // out = 0 - (-1) * (flip ? X^T : X): the apply kernel with factor -1 into a zeroed tensor (muon-gpu.ts:270-279)
    cudaMemsetAsync(gt_ptr<float>(out), 0, sizeof(float) * el, ctx->stream);
    muon_apply_kernel<<<egrid(ctx, el), 256, 0, ctx->stream>>>(mm, nn, flip, -1.f, X, gt_ptr<float>(out));
    ctx->launches++;
  }
  cudaStreamSynchronize(ctx->stream);
  cudaFree(X); cudaFree(BX); cudaFree(A); cudaFree(AA); cudaFree(partials); cudaFree(inv);
  if (s) return s;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? GT_OK : gt_check_cuda(ctx, e, "gt_newton_schulz");
}

}  // extern "C"
