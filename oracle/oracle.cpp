// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// CPU restatement of gguf-trainer's own reference implementation of the training
// hot path (its TypeScript "reference" ops, optimizers and architectures), used
// as the parity oracle for the CUDA library and as the timed CPU baseline.
// Nothing in the shipped library or its host package may call into this file.
//
// Numeric rule (JavaScript semantics): arrays are f32 (`Float32Array`), every
// arithmetic expression is evaluated in f64 and rounded once on store; a
// `grad[i] += e` rounds after each addition. libm doubles stand in for `Math.*`.
//
// Pinned against the reference's own known-answer tests (closed-form cross
// entropy at logit gaps 1..90, mean*kept == summed NLL, fused == dense CE,
// checkpoint on == off bit-exact, WSD golden values, MuonClip landing on tau,
// finite-difference gradchecks): see tests/test_oracle_golden.py.
//
// Each function cites the reference file:line it follows (paths inside the
// gguf-trainer project).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_set>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace orc {

// ---------------------------------------------------------------------------
// PRNG: src/model/autograd.ts:61-78 (randn, mulberry32)
// ---------------------------------------------------------------------------
struct Rng {
  uint32_t a;
  explicit Rng(uint32_t seed) : a(seed) {}
  double next() {
    a += 0x6d2b79f5u;
    uint32_t t = (a ^ (a >> 15)) * (1u | a);
    t = (t + ((t ^ (t >> 7)) * (61u | t))) ^ t;
    return (double)(t ^ (t >> 14)) / 4294967296.0;
  }
};

static double randn(Rng& r) {
  double u = 0, v = 0;
  while (u == 0) u = r.next();
  while (v == 0) v = r.next();
  return std::sqrt(-2 * std::log(u)) * std::cos(2 * M_PI * v);
}

// ---------------------------------------------------------------------------
// Tensor + tape: src/model/autograd.ts:20-51, 81-93
// ---------------------------------------------------------------------------
struct Tensor;
using TP = std::shared_ptr<Tensor>;
static long g_created = 0;

struct Tensor {
  std::vector<float> data, grad;
  std::vector<int> shape;
  bool requiresGrad;
  std::function<void()> backward_fn;
  std::vector<TP> prev;
  long seq;
  Tensor(std::vector<int> sh, bool rg) : shape(std::move(sh)), requiresGrad(rg), seq(g_created++) {
    size_t n = 1;
    for (int s : shape) n *= (size_t)s;
    data.assign(n, 0.f);
    grad.assign(n, 0.f);
  }
  size_t size() const { return data.size(); }
  void zeroGrad() { std::fill(grad.begin(), grad.end(), 0.f); }
};

static TP zeros(std::vector<int> shape, bool rg = false) { return std::make_shared<Tensor>(std::move(shape), rg); }

// src/model/autograd.ts:54-58
static TP param(std::vector<int> shape, double std_, Rng& rng) {
  TP t = zeros(std::move(shape), true);
  for (size_t i = 0; i < t->size(); i++) t->data[i] = (float)(randn(rng) * std_);
  return t;
}
// src/arch/common.ts `ones`
static TP ones(std::vector<int> shape) {
  TP t = zeros(std::move(shape), true);
  std::fill(t->data.begin(), t->data.end(), 1.f);
  return t;
}

static void build_topo(const TP& t, std::unordered_set<Tensor*>& seen, std::vector<TP>& topo) {
  // iterative DFS with the same visiting order as the recursive reference
  struct Frame { TP t; size_t i; };
  if (seen.count(t.get())) return;
  std::vector<Frame> st;
  seen.insert(t.get());
  st.push_back({t, 0});
  while (!st.empty()) {
    Frame& f = st.back();
    if (f.i < f.t->prev.size()) {
      TP p = f.t->prev[f.i++];
      if (!seen.count(p.get())) {
        seen.insert(p.get());
        st.push_back({p, 0});
      }
    } else {
      topo.push_back(f.t);
      st.pop_back();
    }
  }
}

// src/model/autograd.ts:81-93
static void backward(const TP& loss, double seed) {
  std::vector<TP> topo;
  std::unordered_set<Tensor*> seen;
  build_topo(loss, seen, topo);
  loss->grad[0] = (float)seed;
  for (size_t i = topo.size(); i-- > 0;)
    if (topo[i]->backward_fn) topo[i]->backward_fn();
}

// ---------------------------------------------------------------------------
// checkpoint: src/model/autograd.ts:171-273
// ---------------------------------------------------------------------------
static bool g_checkpointing = false;

static TP checkpoint(std::vector<TP> inputs, std::function<TP()> fn) {
  if (!g_checkpointing) return fn();
  TP out = fn();
  out->prev = inputs;
  Tensor* o = out.get();
  out->backward_fn = [o, inputs, fn]() {
    TP replay = fn();
    replay->grad = o->grad;
    std::vector<TP> topo;
    std::unordered_set<Tensor*> seen;
    for (auto& in : inputs) seen.insert(in.get());
    build_topo(replay, seen, topo);
    for (size_t i = topo.size(); i-- > 0;)
      if (topo[i]->backward_fn) topo[i]->backward_fn();
  };
  return out;
}

// ---------------------------------------------------------------------------
// LoRA routing: src/model/autograd.ts:286-319
// ---------------------------------------------------------------------------
struct LoraAdapter { TP a, b; double scale; };
static std::map<Tensor*, LoraAdapter> g_lora;

// ---------------------------------------------------------------------------
// Raw op kernels on plain arrays (shared by the tape ops and the per-op C API).
// All backward kernels ACCUMULATE into their gradient outputs.
// ---------------------------------------------------------------------------
#define F64(x) ((double)(x))
#define ACC(dst, e) (dst) = (float)(F64(dst) + (e))

// src/model/autograd.ts:348-357
static void linear_fwd(const float* x, const float* w, int T, int in, int out, float* y) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++)
    for (int o = 0; o < out; o++) {
      double acc = 0;
      const float* xb = x + (size_t)t * in;
      const float* wb = w + (size_t)o * in;
      for (int i = 0; i < in; i++) acc += F64(xb[i]) * F64(wb[i]);
      y[(size_t)t * out + o] = (float)acc;
    }
}
// src/model/autograd.ts:360-377 (loop nest t,o,i; zero upstream entries skipped).
// The OpenMP variant splits dX by row and dW by output row; each element still
// receives its additions in the reference's order (o ascending for dX, t
// ascending for dW), so results are bit-identical to the serial nest.
static void linear_bwd(const float* x, const float* w, const float* gy, int T, int in, int out, float* gx,
                       float* gw) {
#pragma omp parallel
  {
#pragma omp for schedule(static) nowait
    for (int t = 0; t < T; t++)
      for (int o = 0; o < out; o++) {
        float g = gy[(size_t)t * out + o];
        if (g == 0) continue;
        float* gxb = gx + (size_t)t * in;
        const float* wb = w + (size_t)o * in;
        for (int i = 0; i < in; i++) ACC(gxb[i], F64(g) * F64(wb[i]));
      }
    if (gw) {
#pragma omp for schedule(static)
      for (int o = 0; o < out; o++)
        for (int t = 0; t < T; t++) {
          float g = gy[(size_t)t * out + o];
          if (g == 0) continue;
          const float* xb = x + (size_t)t * in;
          float* gwb = gw + (size_t)o * in;
          for (int i = 0; i < in; i++) ACC(gwb[i], F64(g) * F64(xb[i]));
        }
    }
  }
}

static const double GELU_K = 0.7978845608028654;  // src/model/autograd.ts:433-434
static const double GELU_A = 0.044715;

// src/model/autograd.ts:472-501 (rows=T,d) and :505-544 (rows=T*H,d=hd): the
// per-head variant is the same arithmetic on the [T*H, hd] view.
static void rmsnorm_fwd(const float* x, const float* w, int rows, int d, double eps, float* y, float* rinv) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < rows; t++) {
    double ms = 0;
    const float* xb = x + (size_t)t * d;
    for (int j = 0; j < d; j++) ms += F64(xb[j]) * F64(xb[j]);
    ms /= d;
    double r = 1 / std::sqrt(ms + eps);
    rinv[t] = (float)r;
    for (int j = 0; j < d; j++) y[(size_t)t * d + j] = (float)(F64(xb[j]) * r * F64(w[j]));
  }
}
static void rmsnorm_bwd(const float* x, const float* w, const float* rinv, const float* gy, int rows, int d,
                        float* gx, float* gw) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < rows; t++) {
    const float* xb = x + (size_t)t * d;
    const float* gb = gy + (size_t)t * d;
    double r = rinv[t];
    double S = 0;
    for (int j = 0; j < d; j++) S += F64(gb[j]) * F64(w[j]) * F64(xb[j]);
    for (int j = 0; j < d; j++) {
      double g = gb[j];
      ACC(gx[(size_t)t * d + j], F64(w[j]) * r * g - (F64(xb[j]) / d) * r * r * r * S);
    }
  }
  if (gw)
    for (int t = 0; t < rows; t++) {
      const float* xb = x + (size_t)t * d;
      const float* gb = gy + (size_t)t * d;
      double r = rinv[t];
      for (int j = 0; j < d; j++) ACC(gw[j], F64(gb[j]) * F64(xb[j]) * r);
    }
}

// src/model/autograd.ts:588-631
static void rope_tables(int T, int hd, double base, int posOffset, std::vector<float>& cs, std::vector<float>& sn) {
  int half = hd / 2;
  cs.resize((size_t)T * half);
  sn.resize((size_t)T * half);
  for (int t = 0; t < T; t++) {
    double pos = t + posOffset;
    for (int j = 0; j < half; j++) {
      double freq = std::pow(base, (-2.0 * j) / hd);
      double ang = pos * freq;
      cs[(size_t)t * half + j] = (float)std::cos(ang);
      sn[(size_t)t * half + j] = (float)std::sin(ang);
    }
  }
}
static void rope_fwd(const float* x, int T, int H, int hd, const float* cs, const float* sn, float* y) {
  int half = hd / 2;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++)
    for (int h = 0; h < H; h++) {
      size_t b = (size_t)t * H * hd + (size_t)h * hd;
      for (int j = 0; j < half; j++) {
        double c = cs[(size_t)t * half + j], s = sn[(size_t)t * half + j];
        double x0 = x[b + j], x1 = x[b + j + half];
        y[b + j] = (float)(x0 * c - x1 * s);
        y[b + j + half] = (float)(x0 * s + x1 * c);
      }
    }
}
static void rope_bwd(const float* gy, int T, int H, int hd, const float* cs, const float* sn, float* gx) {
  int half = hd / 2;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++)
    for (int h = 0; h < H; h++) {
      size_t b = (size_t)t * H * hd + (size_t)h * hd;
      for (int j = 0; j < half; j++) {
        double c = cs[(size_t)t * half + j], s = sn[(size_t)t * half + j];
        double g0 = gy[b + j], g1 = gy[b + j + half];
        ACC(gx[b + j], c * g0 + s * g1);
        ACC(gx[b + j + half], -s * g0 + c * g1);
      }
    }
}

// src/model/autograd.ts:640-729. probs is [Hq][T][T] dense (entries outside the
// causal window stay 0), which stores the same values as the reference's ragged rows.
static void attention_fwd(const float* q, const float* k, const float* v, int T, int Hq, int Hkv, int hd, int window,
                          float* out, float* probs) {
  int group = Hq / Hkv;
  double scale = 1 / std::sqrt((double)hd);
  size_t qS = (size_t)Hq * hd, kvS = (size_t)Hkv * hd;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
  for (int h = 0; h < Hq; h++)
    for (int t = 0; t < T; t++) {
      int kv = h / group;
      int s0 = (window > 0 && t + 1 > window) ? t + 1 - window : 0;
      float* sc = probs + ((size_t)h * T + t) * T;
      double maxS = -INFINITY;
      size_t qb = (size_t)t * qS + (size_t)h * hd;
      for (int s = s0; s <= t; s++) {
        size_t kb = (size_t)s * kvS + (size_t)kv * hd;
        double dot = 0;
        for (int d = 0; d < hd; d++) dot += F64(q[qb + d]) * F64(k[kb + d]);
        dot *= scale;
        sc[s] = (float)dot;
        if (dot > maxS) maxS = dot;
      }
      double sum = 0;
      for (int s = s0; s <= t; s++) {
        double e = std::exp(F64(sc[s]) - maxS);
        sc[s] = (float)e;
        sum += e;
      }
      for (int s = s0; s <= t; s++) sc[s] = (float)(F64(sc[s]) / sum);
      size_t ob = (size_t)t * qS + (size_t)h * hd;
      for (int s = s0; s <= t; s++) {
        double p = sc[s];
        size_t vb = (size_t)s * kvS + (size_t)kv * hd;
        for (int d = 0; d < hd; d++) ACC(out[ob + d], p * F64(v[vb + d]));
      }
    }
}
// The reference walks h outer, t inner, and every dK/dV element receives its
// additions in that order. The parallel variant gives each KV head to one thread
// and keeps (h ascending within the group, t ascending) inside it, so every
// element sees the same sequence of additions.
static void attention_bwd(const float* q, const float* k, const float* v, const float* probs, const float* gout, int T,
                          int Hq, int Hkv, int hd, int window, float* gq, float* gk, float* gv) {
  int group = Hq / Hkv;
  double scale = 1 / std::sqrt((double)hd);
  size_t qS = (size_t)Hq * hd, kvS = (size_t)Hkv * hd;
#pragma omp parallel for schedule(dynamic, 1)
  for (int kvh = 0; kvh < Hkv; kvh++) {
    std::vector<float> dP(T);
    for (int h = kvh * group; h < (kvh + 1) * group; h++) {
      int kv = kvh;
      for (int t = 0; t < T; t++) {
        int s0 = (window > 0 && t + 1 > window) ? t + 1 - window : 0;
        const float* p = probs + ((size_t)h * T + t) * T;
        size_t ob = (size_t)t * qS + (size_t)h * hd, qb = ob;
        for (int s = s0; s <= t; s++) {
          size_t vb = (size_t)s * kvS + (size_t)kv * hd;
          double acc = 0;
          for (int d = 0; d < hd; d++) {
            acc += F64(gout[ob + d]) * F64(v[vb + d]);
            ACC(gv[vb + d], F64(p[s]) * F64(gout[ob + d]));
          }
          dP[s] = (float)acc;
        }
        double dot = 0;
        for (int s = s0; s <= t; s++) dot += F64(p[s]) * F64(dP[s]);
        for (int s = s0; s <= t; s++) {
          double dscore = F64(p[s]) * (F64(dP[s]) - dot) * scale;
          size_t kb = (size_t)s * kvS + (size_t)kv * hd;
          for (int d = 0; d < hd; d++) {
            ACC(gq[qb + d], dscore * F64(k[kb + d]));
            ACC(gk[kb + d], dscore * F64(q[qb + d]));
          }
        }
      }
    }
  }
}

// src/model/autograd.ts:897-952. probs [T,V] scratch; returns loss.
static float ce_fwd(const float* logits, const int* targets, int T, int V, int kept, float* probs) {
  std::vector<double> rowLoss(T, 0.0);
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++) {
    size_t b = (size_t)t * V;
    double maxL = -INFINITY;
    for (int v = 0; v < V; v++)
      if (logits[b + v] > maxL) maxL = logits[b + v];
    double sum = 0;
    for (int v = 0; v < V; v++) {
      double e = std::exp(F64(logits[b + v]) - maxL);
      probs[b + v] = (float)e;
      sum += e;
    }
    for (int v = 0; v < V; v++) probs[b + v] = (float)(F64(probs[b + v]) / sum);
    if (targets[t] >= 0) rowLoss[t] = std::log(sum) + maxL - F64(logits[b + targets[t]]);
  }
  double total = 0;
  for (int t = 0; t < T; t++)
    if (targets[t] >= 0) total += rowLoss[t];
  int denom = kept > 0 ? kept : 1;
  return (float)(total / denom);
}
static void ce_bwd(const float* probs, const int* targets, int T, int V, int kept, float lossGrad, float* glogits) {
  int denom = kept > 0 ? kept : 1;
  double scale = F64(lossGrad) / denom;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; t++) {
    if (targets[t] < 0) continue;
    size_t b = (size_t)t * V;
    for (int v = 0; v < V; v++) ACC(glogits[b + v], scale * (F64(probs[b + v]) - (v == targets[t] ? 1 : 0)));
  }
}

// ---------------------------------------------------------------------------
// Tape ops
// ---------------------------------------------------------------------------
static TP add(const TP& a, const TP& b);
static TP scale_op(const TP& x, double c);

// src/model/autograd.ts:321-379
static TP linearRaw(const TP& x, const TP& w) {
  int T = x->shape[0], in = x->shape[1], out = w->shape[0];
  if (in != w->shape[1]) throw std::runtime_error("linear dim mismatch");
  TP y = zeros({T, out});
  linear_fwd(x->data.data(), w->data.data(), T, in, out, y->data.data());
  y->prev = {x, w};
  bool wantsDW = w->requiresGrad;
  Tensor* o = y.get();
  y->backward_fn = [o, x, w, T, in, out, wantsDW]() {
    linear_bwd(x->data.data(), w->data.data(), o->grad.data(), T, in, out, x->grad.data(),
               wantsDW ? w->grad.data() : nullptr);
  };
  return y;
}
// src/model/autograd.ts:311-319
static TP linear(const TP& x, const TP& w) {
  if (!g_lora.empty()) {
    auto it = g_lora.find(w.get());
    if (it != g_lora.end()) {
      const LoraAdapter& ad = it->second;
      return add(linearRaw(x, w), scale_op(linearRaw(linearRaw(x, ad.a), ad.b), ad.scale));
    }
  }
  return linearRaw(x, w);
}

// src/model/autograd.ts:382-394
static TP add(const TP& a, const TP& b) {
  TP out = zeros(a->shape);
  size_t n = a->size();
  for (size_t i = 0; i < n; i++) out->data[i] = (float)(F64(a->data[i]) + F64(b->data[i]));
  out->prev = {a, b};
  Tensor* o = out.get();
  out->backward_fn = [o, a, b, n]() {
    for (size_t i = 0; i < n; i++) {
      ACC(a->grad[i], F64(o->grad[i]));
      ACC(b->grad[i], F64(o->grad[i]));
    }
  };
  return out;
}
// src/model/autograd.ts:397-409
static TP mul(const TP& a, const TP& b) {
  TP out = zeros(a->shape);
  size_t n = a->size();
  for (size_t i = 0; i < n; i++) out->data[i] = (float)(F64(a->data[i]) * F64(b->data[i]));
  out->prev = {a, b};
  Tensor* o = out.get();
  out->backward_fn = [o, a, b, n]() {
    for (size_t i = 0; i < n; i++) {
      ACC(a->grad[i], F64(o->grad[i]) * F64(b->data[i]));
      ACC(b->grad[i], F64(o->grad[i]) * F64(a->data[i]));
    }
  };
  return out;
}
// src/model/autograd.ts:412-429
static TP silu(const TP& x) {
  TP out = zeros(x->shape);
  size_t n = x->size();
  auto sig = std::make_shared<std::vector<float>>(n);
  for (size_t i = 0; i < n; i++) {
    double s = 1 / (1 + std::exp(-F64(x->data[i])));
    (*sig)[i] = (float)s;
    out->data[i] = (float)(F64(x->data[i]) * s);
  }
  out->prev = {x};
  Tensor* o = out.get();
  out->backward_fn = [o, x, sig, n]() {
    for (size_t i = 0; i < n; i++) {
      double s = (*sig)[i];
      ACC(x->grad[i], F64(o->grad[i]) * (s + F64(x->data[i]) * s * (1 - s)));
    }
  };
  return out;
}
// src/model/autograd.ts:437-457
static TP gelu(const TP& x) {
  TP out = zeros(x->shape);
  size_t n = x->size();
  for (size_t i = 0; i < n; i++) {
    double v = x->data[i];
    out->data[i] = (float)(0.5 * v * (1 + std::tanh(GELU_K * (v + GELU_A * v * v * v))));
  }
  out->prev = {x};
  Tensor* o = out.get();
  out->backward_fn = [o, x, n]() {
    for (size_t i = 0; i < n; i++) {
      double v = x->data[i];
      double v2 = v * v;
      double u = GELU_K * (v + GELU_A * v * v2);
      double th = std::tanh(u);
      double dudx = GELU_K * (1 + 3 * GELU_A * v2);
      double g = 0.5 * (1 + th) + 0.5 * v * (1 - th * th) * dudx;
      ACC(x->grad[i], F64(o->grad[i]) * g);
    }
  };
  return out;
}
// src/model/autograd.ts:460-469
static TP scale_op(const TP& x, double c) {
  TP out = zeros(x->shape);
  size_t n = x->size();
  for (size_t i = 0; i < n; i++) out->data[i] = (float)(F64(x->data[i]) * c);
  out->prev = {x};
  Tensor* o = out.get();
  out->backward_fn = [o, x, c, n]() {
    for (size_t i = 0; i < n; i++) ACC(x->grad[i], F64(o->grad[i]) * c);
  };
  return out;
}
// src/model/autograd.ts:472-502
static TP rmsNorm(const TP& x, const TP& w, double eps) {
  int T = x->shape[0], d = x->shape[1];
  TP out = zeros({T, d});
  auto rinv = std::make_shared<std::vector<float>>(T);
  rmsnorm_fwd(x->data.data(), w->data.data(), T, d, eps, out->data.data(), rinv->data());
  out->prev = {x, w};
  bool wantsDW = w->requiresGrad;
  Tensor* o = out.get();
  out->backward_fn = [o, x, w, rinv, T, d, wantsDW]() {
    rmsnorm_bwd(x->data.data(), w->data.data(), rinv->data(), o->grad.data(), T, d, x->grad.data(),
                wantsDW ? w->grad.data() : nullptr);
  };
  return out;
}
// src/model/autograd.ts:505-545
static TP rmsNormHeads(const TP& x, const TP& w, int T, int H, int hd, double eps) {
  TP out = zeros({T, H * hd});
  auto rinv = std::make_shared<std::vector<float>>((size_t)T * H);
  rmsnorm_fwd(x->data.data(), w->data.data(), T * H, hd, eps, out->data.data(), rinv->data());
  out->prev = {x, w};
  bool wantsDW = w->requiresGrad;
  Tensor* o = out.get();
  out->backward_fn = [o, x, w, rinv, T, H, hd, wantsDW]() {
    rmsnorm_bwd(x->data.data(), w->data.data(), rinv->data(), o->grad.data(), T * H, hd, x->grad.data(),
                wantsDW ? w->grad.data() : nullptr);
  };
  return out;
}
// src/model/autograd.ts:548-573
static TP embedding(const TP& weight, const std::vector<int>& ids) {
  int V = weight->shape[0], d = weight->shape[1];
  int T = (int)ids.size();
  for (int t = 0; t < T; t++)
    if (ids[t] < 0 || ids[t] >= V) throw std::runtime_error("embedding: id out of range");
  TP out = zeros({T, d});
  for (int t = 0; t < T; t++)
    std::memcpy(&out->data[(size_t)t * d], &weight->data[(size_t)ids[t] * d], sizeof(float) * d);
  out->prev = {weight};
  bool wantsDW = weight->requiresGrad;
  Tensor* o = out.get();
  out->backward_fn = [o, weight, ids, T, d, wantsDW]() {
    if (!wantsDW) return;
    for (int t = 0; t < T; t++) {
      size_t src = (size_t)ids[t] * d, dst = (size_t)t * d;
      for (int j = 0; j < d; j++) ACC(weight->grad[src + j], F64(o->grad[dst + j]));
    }
  };
  return out;
}
// src/model/autograd.ts:579-632
static TP rope(const TP& x, int T, int H, int hd, double base, int posOffset = 0) {
  TP out = zeros({T, H * hd});
  auto cs = std::make_shared<std::vector<float>>();
  auto sn = std::make_shared<std::vector<float>>();
  rope_tables(T, hd, base, posOffset, *cs, *sn);
  rope_fwd(x->data.data(), T, H, hd, cs->data(), sn->data(), out->data.data());
  out->prev = {x};
  Tensor* o = out.get();
  out->backward_fn = [o, x, cs, sn, T, H, hd]() {
    rope_bwd(o->grad.data(), T, H, hd, cs->data(), sn->data(), x->grad.data());
  };
  return out;
}
// src/model/autograd.ts:640-729
static TP attention(const TP& q, const TP& k, const TP& v, int T, int Hq, int Hkv, int hd, int window) {
  TP out = zeros({T, Hq * hd});
  auto probs = std::make_shared<std::vector<float>>((size_t)Hq * T * T, 0.f);
  attention_fwd(q->data.data(), k->data.data(), v->data.data(), T, Hq, Hkv, hd, window, out->data.data(),
                probs->data());
  out->prev = {q, k, v};
  Tensor* o = out.get();
  out->backward_fn = [o, q, k, v, probs, T, Hq, Hkv, hd, window]() {
    attention_bwd(q->data.data(), k->data.data(), v->data.data(), probs->data(), o->grad.data(), T, Hq, Hkv, hd,
                  window, q->grad.data(), k->grad.data(), v->grad.data());
  };
  return out;
}

// src/model/autograd.ts:875-894
static int keptRowsInVocab(const std::vector<int>& targets, int T, int V) {
  if ((int)targets.size() != T) throw std::runtime_error("targets length != T");
  int kept = 0;
  for (int t = 0; t < T; t++) {
    int g = targets[t];
    if (g < -1 || g >= V) throw std::runtime_error("target out of range");
    if (g >= 0) kept++;
  }
  return kept;
}

// src/model/autograd.ts:897-952
static TP crossEntropy(const TP& logits, const std::vector<int>& targets) {
  int T = logits->shape[0], V = logits->shape[1];
  int kept = keptRowsInVocab(targets, T, V);
  TP loss = zeros({1});
  auto probs = std::make_shared<std::vector<float>>((size_t)T * V);
  loss->data[0] = ce_fwd(logits->data.data(), targets.data(), T, V, kept, probs->data());
  loss->prev = {logits};
  Tensor* o = loss.get();
  loss->backward_fn = [o, logits, probs, targets, T, V, kept]() {
    ce_bwd(probs->data(), targets.data(), T, V, kept, o->grad[0], logits->grad.data());
  };
  return loss;
}

// src/model/autograd.ts:968-1055
static TP fusedCrossEntropy(const TP& hidden, const TP& w, const std::vector<int>& targets, int chunk) {
  int T = hidden->shape[0], H = hidden->shape[1], V = w->shape[0];
  if (H != w->shape[1]) throw std::runtime_error("fusedCrossEntropy dim mismatch");
  if (chunk <= 0) throw std::runtime_error("fusedCrossEntropy chunk must be positive");
  if (g_lora.count(w.get())) throw std::runtime_error("fusedCrossEntropy: readout carries a LoRA adapter");
  int kept = keptRowsInVocab(targets, T, V);
  TP loss = zeros({1});
  auto rowMax = std::make_shared<std::vector<float>>(T, -INFINITY);
  auto rowSum = std::make_shared<std::vector<float>>(T, 0.f);
  std::vector<float> tgtLogit(T, 0.f);
  const float* hd = hidden->data.data();
  const float* wd = w->data.data();
  auto dot = [hd, wd, H](int t, int v) {
    double acc = 0;
    for (int i = 0; i < H; i++) acc += F64(hd[(size_t)t * H + i]) * F64(wd[(size_t)v * H + i]);
    return acc;
  };
  for (int v0 = 0; v0 < V; v0 += chunk) {
    int v1 = std::min(v0 + chunk, V);
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
      double chunkMax = -INFINITY;
      for (int v = v0; v < v1; v++) {
        double z = dot(t, v);
        if (z > chunkMax) chunkMax = z;
      }
      double mNew = std::max(F64((*rowMax)[t]), chunkMax);
      double sum = 0;
      for (int v = v0; v < v1; v++) sum += std::exp(dot(t, v) - mNew);
      (*rowSum)[t] = (float)(F64((*rowSum)[t]) * std::exp(F64((*rowMax)[t]) - mNew) + sum);
      (*rowMax)[t] = (float)mNew;
      int g = targets[t];
      if (g >= v0 && g < v1) tgtLogit[t] = (float)dot(t, g);
    }
  }
  double total = 0;
  for (int t = 0; t < T; t++) {
    if (targets[t] < 0) continue;
    total += std::log(F64((*rowSum)[t])) + F64((*rowMax)[t]) - F64(tgtLogit[t]);
  }
  int denom = kept > 0 ? kept : 1;
  loss->data[0] = (float)(total / denom);
  loss->prev = {hidden, w};
  Tensor* o = loss.get();
  loss->backward_fn = [o, hidden, w, rowMax, rowSum, targets, T, H, V, chunk, denom, dot]() {
    double scale = F64(o->grad[0]) / denom;
    bool wantsDW = w->requiresGrad;
    for (int v0 = 0; v0 < V; v0 += chunk) {
      int v1 = std::min(v0 + chunk, V);
      for (int t = 0; t < T; t++) {
        if (targets[t] < 0) continue;
        for (int v = v0; v < v1; v++) {
          double p = std::exp(dot(t, v) - F64((*rowMax)[t])) / F64((*rowSum)[t]);
          double d = scale * (p - (v == targets[t] ? 1 : 0));
          for (int i = 0; i < H; i++) {
            ACC(hidden->grad[(size_t)t * H + i], d * F64(w->data[(size_t)v * H + i]));
            if (wantsDW) ACC(w->grad[(size_t)v * H + i], d * F64(hidden->data[(size_t)t * H + i]));
          }
        }
      }
    }
  };
  return loss;
}

// src/model/autograd.ts:760-791, 1076-1138
static TP softCrossEntropy(const TP& logits, const std::vector<int>& ids, const std::vector<float>& q, int k) {
  int T = logits->shape[0], V = logits->shape[1];
  if (k < 1) throw std::runtime_error("softCrossEntropy: k must be >= 1");
  if ((int)ids.size() != T * k || (int)q.size() != T * k) throw std::runtime_error("softCrossEntropy: teacher arrays");
  int kept = 0;
  for (int t = 0; t < T; t++) {
    if (ids[(size_t)t * k] == -1) continue;
    for (int j = 0; j < k; j++) {
      int id = ids[(size_t)t * k + j];
      if (id < 0 || id >= V) throw std::runtime_error("softCrossEntropy: teacher id out of range");
    }
    kept++;
  }
  TP loss = zeros({1});
  auto probs = std::make_shared<std::vector<float>>((size_t)T * V);
  auto rowMass = std::make_shared<std::vector<float>>(T, 0.f);
  double total = 0;
  for (int t = 0; t < T; t++) {
    size_t b = (size_t)t * V;
    double maxL = -INFINITY;
    for (int v = 0; v < V; v++)
      if (logits->data[b + v] > maxL) maxL = logits->data[b + v];
    double sum = 0;
    for (int v = 0; v < V; v++) {
      double e = std::exp(F64(logits->data[b + v]) - maxL);
      (*probs)[b + v] = (float)e;
      sum += e;
    }
    for (int v = 0; v < V; v++) (*probs)[b + v] = (float)(F64((*probs)[b + v]) / sum);
    if (ids[(size_t)t * k] < 0) continue;
    for (int j = 0; j < k; j++) {
      int id = ids[(size_t)t * k + j];
      double qq = q[(size_t)t * k + j];
      if (qq == 0) continue;
      total += qq * (std::log(sum) + maxL - F64(logits->data[b + id]));
      ACC((*rowMass)[t], qq);
    }
  }
  int denom = kept > 0 ? kept : 1;
  loss->data[0] = (float)(total / denom);
  loss->prev = {logits};
  Tensor* o = loss.get();
  loss->backward_fn = [o, logits, probs, rowMass, ids, q, T, V, k, denom]() {
    double scale = F64(o->grad[0]) / denom;
    for (int t = 0; t < T; t++) {
      if (ids[(size_t)t * k] < 0) continue;
      size_t b = (size_t)t * V;
      for (int v = 0; v < V; v++) ACC(logits->grad[b + v], scale * F64((*rowMass)[t]) * F64((*probs)[b + v]));
      for (int j = 0; j < k; j++) {
        float& g = logits->grad[b + ids[(size_t)t * k + j]];
        g = (float)(F64(g) - scale * F64(q[(size_t)t * k + j]));
      }
    }
  };
  return loss;
}

// ---------------------------------------------------------------------------
// Architectures: src/arch/llama.ts:138-222, qwen3.ts:87-195, gemma3.ts:102-223
// ---------------------------------------------------------------------------
struct Config {
  int arch;  // 0 llama, 1 qwen3, 2 gemma3
  int vocab, hidden, nLayers, nHeads, nKV, headDim, ffn;
  double ropeBase, ropeBaseLocal, rmsEps;
  int slidingWindow, swaPattern;
  int tie;
  int initMode;  // 0: reference init (emb 0.02, matrices 1/sqrt(fan_in)); 1: every matrix N(0, 0.02)
};

struct Layer {
  TP attnNorm, qProj, kProj, vProj, oProj, qNorm, kNorm, postAttnNorm, ffnNorm, gate, up, down, postFfnNorm;
};

struct Model {
  Config c;
  TP tokenEmbd, outputNorm, output;
  std::vector<Layer> layers;
  std::vector<TP> layerOut;  // last forward's per-layer outputs (test hook)
  TP lastHidden;

  Model(const Config& cfg, Rng& rng) : c(cfg) {
    int h = c.hidden, qDim = c.nHeads * c.headDim, kvDim = c.nKV * c.headDim;
    auto sd = [&](int fanIn) { return c.initMode == 1 ? 0.02 : 1 / std::sqrt((double)fanIn); };
    tokenEmbd = param({c.vocab, h}, 0.02, rng);
    outputNorm = ones({h});
    if (!c.tie) output = param({c.vocab, h}, 0.02, rng);
    for (int l = 0; l < c.nLayers; l++) {
      Layer L;
      L.attnNorm = ones({h});
      L.qProj = param({qDim, h}, sd(h), rng);
      L.kProj = param({kvDim, h}, sd(h), rng);
      L.vProj = param({kvDim, h}, sd(h), rng);
      L.oProj = param({h, qDim}, sd(qDim), rng);
      if (c.arch != 0) {
        L.qNorm = ones({c.headDim});
        L.kNorm = ones({c.headDim});
      }
      if (c.arch == 2) L.postAttnNorm = ones({h});
      L.ffnNorm = ones({h});
      L.gate = param({c.ffn, h}, sd(h), rng);
      L.up = param({c.ffn, h}, sd(h), rng);
      L.down = param({h, c.ffn}, sd(c.ffn), rng);
      if (c.arch == 2) L.postFfnNorm = ones({h});
      layers.push_back(L);
    }
  }

  // params(): llama.ts:173-180, qwen3.ts:110-129, gemma3.ts:133-154
  std::vector<TP> params() const {
    std::vector<TP> ps{tokenEmbd, outputNorm};
    if (output) ps.push_back(output);
    for (const Layer& L : layers) {
      if (c.arch == 0) {
        for (TP t : {L.attnNorm, L.qProj, L.kProj, L.vProj, L.oProj, L.ffnNorm, L.gate, L.up, L.down}) ps.push_back(t);
      } else if (c.arch == 1) {
        for (TP t : {L.attnNorm, L.qProj, L.kProj, L.vProj, L.oProj, L.qNorm, L.kNorm, L.ffnNorm, L.gate, L.up, L.down})
          ps.push_back(t);
      } else {
        for (TP t : {L.attnNorm, L.qProj, L.kProj, L.vProj, L.oProj, L.qNorm, L.kNorm, L.postAttnNorm, L.ffnNorm,
                     L.gate, L.up, L.down, L.postFfnNorm})
          ps.push_back(t);
      }
    }
    return ps;
  }
  // paramGroups(): llama.ts:182-191, qwen3.ts:131-140, gemma3.ts:156-165
  void groups(std::vector<TP>& muon, std::vector<TP>& aux) const {
    aux = {tokenEmbd, outputNorm};
    if (output) aux.push_back(output);
    for (const Layer& L : layers) {
      for (TP t : {L.qProj, L.kProj, L.vProj, L.oProj, L.gate, L.up, L.down}) muon.push_back(t);
      if (c.arch == 0) {
        for (TP t : {L.attnNorm, L.ffnNorm}) aux.push_back(t);
      } else if (c.arch == 1) {
        for (TP t : {L.attnNorm, L.qNorm, L.kNorm, L.ffnNorm}) aux.push_back(t);
      } else {
        for (TP t : {L.attnNorm, L.qNorm, L.kNorm, L.postAttnNorm, L.ffnNorm, L.postFfnNorm}) aux.push_back(t);
      }
    }
  }

  TP block(const TP& hIn, int il, int T) {
    const Layer& L = layers[il];
    TP h = hIn;
    bool global = c.arch != 2 || (c.swaPattern > 0 && il % c.swaPattern == c.swaPattern - 1);
    int window = global ? 0 : c.slidingWindow;
    double ropeB = (c.arch == 2 && !global) ? c.ropeBaseLocal : c.ropeBase;
    TP n1 = rmsNorm(h, L.attnNorm, c.rmsEps);
    TP q = linear(n1, L.qProj);
    TP k = linear(n1, L.kProj);
    TP v = linear(n1, L.vProj);
    if (c.arch != 0) {
      q = rmsNormHeads(q, L.qNorm, T, c.nHeads, c.headDim, c.rmsEps);
      k = rmsNormHeads(k, L.kNorm, T, c.nKV, c.headDim, c.rmsEps);
    }
    q = rope(q, T, c.nHeads, c.headDim, ropeB);
    k = rope(k, T, c.nKV, c.headDim, ropeB);
    TP a = attention(q, k, v, T, c.nHeads, c.nKV, c.headDim, window);
    TP attnOut = linear(a, L.oProj);
    if (c.arch == 2) attnOut = rmsNorm(attnOut, L.postAttnNorm, c.rmsEps);
    h = add(h, attnOut);
    TP n2 = rmsNorm(h, L.ffnNorm, c.rmsEps);
    TP g = c.arch == 2 ? gelu(linear(n2, L.gate)) : silu(linear(n2, L.gate));
    TP u = linear(n2, L.up);
    TP down = linear(mul(g, u), L.down);
    if (c.arch == 2) down = rmsNorm(down, L.postFfnNorm, c.rmsEps);
    h = add(h, down);
    return h;
  }

  TP forwardToReadout(const std::vector<int>& ids, TP& readout) {
    int T = (int)ids.size();
    TP h = embedding(tokenEmbd, ids);
    if (c.arch == 2) h = scale_op(h, std::sqrt((double)c.hidden));
    layerOut.clear();
    for (int il = 0; il < c.nLayers; il++) {
      TP hIn = h;
      h = checkpoint({hIn}, [this, hIn, il, T]() { return block(hIn, il, T); });
      layerOut.push_back(h);
    }
    readout = output ? output : tokenEmbd;
    lastHidden = rmsNorm(h, outputNorm, c.rmsEps);
    return lastHidden;
  }
  TP forward(const std::vector<int>& ids) {
    TP readout;
    TP hidden = forwardToReadout(ids, readout);
    return linear(hidden, readout);
  }
};

// src/train/loss.ts:104-115
static TP sequenceLoss(Model& m, const std::vector<int>& ids, const std::vector<int>& targets, int lossChunk) {
  if (lossChunk > 0) {
    TP readout;
    TP hidden = m.forwardToReadout(ids, readout);
    return fusedCrossEntropy(hidden, readout, targets, lossChunk);
  }
  return crossEntropy(m.forward(ids), targets);
}

// ---------------------------------------------------------------------------
// AdamW: src/train/adam.ts:14-83
// ---------------------------------------------------------------------------
struct AdamW {
  std::vector<TP> params;
  std::vector<std::vector<float>> m, v;
  int t = 0;
  double lr, beta1, beta2, eps, weightDecay, clip, baseLr;
  AdamW(std::vector<TP> ps, double lr_, double b1, double b2, double eps_, double wd, double clip_)
      : params(std::move(ps)), lr(lr_), beta1(b1), beta2(b2), eps(eps_), weightDecay(wd), clip(clip_), baseLr(lr_) {
    for (auto& p : params) {
      m.emplace_back(p->size(), 0.f);
      v.emplace_back(p->size(), 0.f);
    }
  }
  void zeroGrad() { for (auto& p : params) p->zeroGrad(); }
  void setLrScale(double s) { lr = baseLr * s; }
  void step() {
    t += 1;
    if (clip > 0) {
      double sq = 0;
      for (auto& p : params)
        for (size_t i = 0; i < p->size(); i++) sq += F64(p->grad[i]) * F64(p->grad[i]);
      double norm = std::sqrt(sq);
      if (norm > clip) {
        double scale = clip / (norm + 1e-12);
        for (auto& p : params)
          for (size_t i = 0; i < p->size(); i++) p->grad[i] = (float)(F64(p->grad[i]) * scale);
      }
    }
    double bc1 = 1 - std::pow(beta1, t);
    double bc2 = 1 - std::pow(beta2, t);
    for (size_t pi = 0; pi < params.size(); pi++) {
      Tensor& p = *params[pi];
      float* mm = m[pi].data();
      float* vv = v[pi].data();
      for (size_t i = 0; i < p.size(); i++) {
        double g = p.grad[i];
        mm[i] = (float)(beta1 * F64(mm[i]) + (1 - beta1) * g);
        vv[i] = (float)(beta2 * F64(vv[i]) + (1 - beta2) * g * g);
        double mHat = F64(mm[i]) / bc1;
        double vHat = F64(vv[i]) / bc2;
        double update = mHat / (std::sqrt(vHat) + eps);
        if (weightDecay > 0) update += weightDecay * F64(p.data[i]);
        p.data[i] = (float)(F64(p.data[i]) - lr * update);
      }
    }
  }
};

// ---------------------------------------------------------------------------
// Muon + Newton-Schulz: src/train/muon.ts:26-158
// ---------------------------------------------------------------------------
static const double NS_A = 3.4445, NS_B = -4.7750, NS_C = 2.0315;

static std::vector<float> transposeM(const std::vector<float>& A, int r, int c) {
  std::vector<float> out((size_t)r * c);
  for (int i = 0; i < r; i++)
    for (int j = 0; j < c; j++) out[(size_t)j * r + i] = A[(size_t)i * c + j];
  return out;
}
// src/train/muon.ts:100-120 (C[i][j] += a*B[k][j], f32 round per addition, zero a skipped)
static std::vector<float> matmulM(const std::vector<float>& A, int ra, int ca, const std::vector<float>& B, int cb) {
  std::vector<float> C((size_t)ra * cb, 0.f);
#pragma omp parallel for schedule(static)
  for (int i = 0; i < ra; i++)
    for (int k = 0; k < ca; k++) {
      float a = A[(size_t)i * ca + k];
      if (a == 0) continue;
      const float* bRow = &B[(size_t)k * cb];
      float* cRow = &C[(size_t)i * cb];
      for (int j = 0; j < cb; j++) ACC(cRow[j], F64(a) * F64(bRow[j]));
    }
  return C;
}
// src/train/muon.ts:133-158
static std::vector<float> newtonSchulz(const std::vector<float>& G, int m, int n, int steps) {
  bool flip = m > n;
  std::vector<float> X = flip ? transposeM(G, m, n) : G;
  int r = flip ? n : m, c = flip ? m : n;
  double s = 0;
  for (float x : X) s += F64(x) * F64(x);
  double norm = std::sqrt(s) + 1e-7;
  for (float& x : X) x = (float)(F64(x) / norm);
  for (int it = 0; it < steps; it++) {
    std::vector<float> Xt = transposeM(X, r, c);
    std::vector<float> A = matmulM(X, r, c, Xt, r);
    std::vector<float> AA = matmulM(A, r, r, A, r);
    std::vector<float> B((size_t)r * r);
    for (size_t i = 0; i < B.size(); i++) B[i] = (float)(NS_B * F64(A[i]) + NS_C * F64(AA[i]));
    std::vector<float> BX = matmulM(B, r, r, X, c);
    for (size_t i = 0; i < X.size(); i++) X[i] = (float)(NS_A * F64(X[i]) + F64(BX[i]));
  }
  return flip ? transposeM(X, r, c) : X;
}

struct Muon {
  std::vector<TP> muonParams;
  std::vector<std::vector<float>> bufs;
  AdamW aux;
  double lr, momentum, baseLr;
  bool nesterov;
  int nsSteps;
  Muon(std::vector<TP> mp, std::vector<TP> ap, double lr_, double mom, bool nest, int ns, AdamW auxOpt)
      : muonParams(std::move(mp)), aux(std::move(auxOpt)), lr(lr_), momentum(mom), baseLr(lr_), nesterov(nest), nsSteps(ns) {
    (void)ap;
    for (auto& p : muonParams) bufs.emplace_back(p->size(), 0.f);
  }
  void zeroGrad() {
    for (auto& p : muonParams) p->zeroGrad();
    aux.zeroGrad();
  }
  void setLrScale(double s) {
    lr = baseLr * s;
    aux.setLrScale(s);
  }
  void step() {
    for (size_t i = 0; i < muonParams.size(); i++) {
      Tensor& p = *muonParams[i];
      int rows = p.shape[0], cols = p.shape[1];
      std::vector<float>& buf = bufs[i];
      std::vector<float> update;
      for (size_t k = 0; k < buf.size(); k++) buf[k] = (float)(momentum * F64(buf[k]) + F64(p.grad[k]));
      if (nesterov) {
        update.resize(buf.size());
        for (size_t k = 0; k < buf.size(); k++) update[k] = (float)(F64(p.grad[k]) + momentum * F64(buf[k]));
      } else {
        update = buf;
      }
      std::vector<float> ortho = newtonSchulz(update, rows, cols, nsSteps);
      double scale = std::sqrt(std::max(1.0, (double)rows / cols));
      for (size_t k = 0; k < p.size(); k++) p.data[k] = (float)(F64(p.data[k]) - lr * F64(ortho[k]) * scale);
    }
    aux.step();
  }
};

// src/train/schedule.ts:20-36
static double wsd(int warmupSteps, int stableSteps, int cooldownSteps, double minScale, int step) {
  int warmup = std::max(0, warmupSteps), stable = std::max(0, stableSteps), cooldown = std::max(0, cooldownSteps);
  int cooldownStart = warmup + stable, total = cooldownStart + cooldown;
  if (warmup > 0 && step < warmup) return (double)(step + 1) / warmup;
  if (step < cooldownStart) return 1;
  if (cooldown > 0 && step < total) {
    double frac = (double)(step - cooldownStart + 1) / cooldown;
    return 1 - (1 - minScale) * frac;
  }
  return step < total ? 1 : minScale;
}

// src/train/qk-clip.ts:35-64
static double qkLogitScale(const float* qn, const float* kn, int hd) {
  double s = 0;
  for (int d = 0; d < hd; d++) {
    double p = F64(qn[d]) * F64(kn[d]);
    s += p * p;
  }
  return std::sqrt(s) / std::sqrt((double)hd);
}
static int applyQKClip(Model& m, double tau) {
  if (m.c.arch == 0) return 0;
  int hd = m.c.headDim, clipped = 0;
  for (Layer& L : m.layers) {
    double s = qkLogitScale(L.qNorm->data.data(), L.kNorm->data.data(), hd);
    if (s > tau) {
      double f = std::sqrt(tau / s);
      for (int d = 0; d < hd; d++) {
        L.qNorm->data[d] = (float)(F64(L.qNorm->data[d]) * f);
        L.kNorm->data[d] = (float)(F64(L.kNorm->data[d]) * f);
      }
      clipped++;
    }
  }
  return clipped;
}

// src/train/lora.ts:46-108
struct Lora {
  std::vector<TP> aux;
  std::vector<std::pair<TP, LoraAdapter>> adapters;
  int rank;
  double scale;
  void fold(double sign) {
    for (auto& kv : adapters) {
      Tensor& w = *kv.first;
      const LoraAdapter& ad = kv.second;
      int outDim = w.shape[0], inDim = w.shape[1];
      for (int o = 0; o < outDim; o++)
        for (int i = 0; i < inDim; i++) {
          double acc = 0;
          for (int r = 0; r < rank; r++) acc += F64(ad.b->data[(size_t)o * rank + r]) * F64(ad.a->data[(size_t)r * inDim + i]);
          w.data[(size_t)o * inDim + i] = (float)(F64(w.data[(size_t)o * inDim + i]) + sign * scale * acc);
        }
    }
  }
};
static Lora* applyLora(Model& m, int rank, double alpha, Rng& rng) {
  Lora* L = new Lora();
  L->rank = rank;
  L->scale = alpha / rank;
  std::vector<TP> muon, aux;
  m.groups(muon, aux);
  for (auto& t : m.params()) t->requiresGrad = false;
  g_lora.clear();
  for (auto& w : muon) {
    int outDim = w->shape[0], inDim = w->shape[1];
    TP a = param({rank, inDim}, 1 / std::sqrt((double)inDim), rng);
    TP b = zeros({outDim, rank}, true);
    LoraAdapter ad{a, b, L->scale};
    g_lora[w.get()] = ad;
    L->adapters.push_back({w, ad});
    L->aux.push_back(a);
    L->aux.push_back(b);
  }
  return L;
}

}  // namespace orc

// ===========================================================================
// C interface (ctypes). Pointers are plain arrays owned by the caller unless
// stated; handles are opaque.
// ===========================================================================
using namespace orc;
extern "C" {

double orc_rng_next(uint32_t* state) {
  Rng r(*state);
  double v = r.next();
  *state = r.a;
  return v;
}
// randn(rng) * scale stored as f32 (param(), tests' randTensor)
void orc_randn_fill(uint32_t* state, float* out, long n, double scale) {
  Rng r(*state);
  for (long i = 0; i < n; i++) out[i] = (float)(randn(r) * scale);
  *state = r.a;
}
// rng()*2-1 (tests/gpu-parity.ts:103-105 upstream gradient)
void orc_uniform_pm1_fill(uint32_t* state, float* out, long n) {
  Rng r(*state);
  for (long i = 0; i < n; i++) out[i] = (float)(r.next() * 2 - 1);
  *state = r.a;
}

void orc_set_checkpointing(int on) { g_checkpointing = on != 0; }
// Worker threads for the OpenMP loops (1 = the reference's single-threaded behaviour).
void orc_set_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n > 0 ? n : 1);
#else
  (void)n;
#endif
}
int orc_max_threads() {
#ifdef _OPENMP
  return omp_get_num_procs();
#else
  return 1;
#endif
}

// ---- per-op functional entry points (backward ACCUMULATES) ----
void orc_linear_fwd(const float* x, const float* w, int T, int in, int out, float* y) { linear_fwd(x, w, T, in, out, y); }
void orc_linear_bwd(const float* x, const float* w, const float* gy, int T, int in, int out, float* gx, float* gw) {
  linear_bwd(x, w, gy, T, in, out, gx, gw);
}
void orc_rmsnorm_fwd(const float* x, const float* w, int rows, int d, double eps, float* y, float* rinv) {
  rmsnorm_fwd(x, w, rows, d, eps, y, rinv);
}
void orc_rmsnorm_bwd(const float* x, const float* w, const float* rinv, const float* gy, int rows, int d, float* gx,
                     float* gw) {
  rmsnorm_bwd(x, w, rinv, gy, rows, d, gx, gw);
}
void orc_rope_fwd(const float* x, int T, int H, int hd, double base, int posOffset, float* y) {
  std::vector<float> cs, sn;
  rope_tables(T, hd, base, posOffset, cs, sn);
  rope_fwd(x, T, H, hd, cs.data(), sn.data(), y);
}
void orc_rope_bwd(const float* gy, int T, int H, int hd, double base, int posOffset, float* gx) {
  std::vector<float> cs, sn;
  rope_tables(T, hd, base, posOffset, cs, sn);
  rope_bwd(gy, T, H, hd, cs.data(), sn.data(), gx);
}
void orc_attention_fwd(const float* q, const float* k, const float* v, int T, int Hq, int Hkv, int hd, int window,
                       float* out, float* probs) {
  attention_fwd(q, k, v, T, Hq, Hkv, hd, window, out, probs);
}
void orc_attention_bwd(const float* q, const float* k, const float* v, const float* probs, const float* gout, int T,
                       int Hq, int Hkv, int hd, int window, float* gq, float* gk, float* gv) {
  attention_bwd(q, k, v, probs, gout, T, Hq, Hkv, hd, window, gq, gk, gv);
}
float orc_ce_fwd(const float* logits, const int* targets, int T, int V, int kept, float* probs) {
  return ce_fwd(logits, targets, T, V, kept, probs);
}
void orc_ce_bwd(const float* probs, const int* targets, int T, int V, int kept, float lossGrad, float* glogits) {
  ce_bwd(probs, targets, T, V, kept, lossGrad, glogits);
}

// Generic "tape" op runner for the elementwise / loss ops: builds leaves from the
// given arrays, runs op, seeds out.grad with gy (or 1 for a scalar loss when gy is
// null), runs that op's backward closure, returns outputs and input grads.
// op: 0 add, 1 mul, 2 silu, 3 gelu, 4 scale(c)
void orc_elementwise(int op, const float* a, const float* b, long n, double c, const float* gy, float* out, float* ga,
                     float* gb) {
  TP A = zeros({(int)n}, true), B = zeros({(int)n}, true);
  std::memcpy(A->data.data(), a, sizeof(float) * n);
  if (b) std::memcpy(B->data.data(), b, sizeof(float) * n);
  TP o;
  switch (op) {
    case 0: o = add(A, B); break;
    case 1: o = mul(A, B); break;
    case 2: o = silu(A); break;
    case 3: o = gelu(A); break;
    default: o = scale_op(A, c); break;
  }
  std::memcpy(out, o->data.data(), sizeof(float) * n);
  if (gy) {
    std::memcpy(o->grad.data(), gy, sizeof(float) * n);
    o->backward_fn();
    if (ga) std::memcpy(ga, A->grad.data(), sizeof(float) * n);
    if (gb && b) std::memcpy(gb, B->grad.data(), sizeof(float) * n);
  }
}

// embedding forward + backward on arrays (gw accumulates)
void orc_embedding_fwd(const float* w, const int* ids, int T, int d, float* out) {
  for (int t = 0; t < T; t++) std::memcpy(out + (size_t)t * d, w + (size_t)ids[t] * d, sizeof(float) * d);
}
void orc_embedding_bwd(const float* gy, const int* ids, int T, int d, float* gw) {
  for (int t = 0; t < T; t++)
    for (int j = 0; j < d; j++) ACC(gw[(size_t)ids[t] * d + j], F64(gy[(size_t)t * d + j]));
}

// fused CE: returns loss; if lossGrad != 0 also runs backward into gh/gw (accumulating; gw nullable)
float orc_fused_ce(const float* hidden, const float* w, const int* targets, int T, int H, int V, int chunk,
                   float lossGrad, float* gh, float* gw) {
  TP h = zeros({T, H}, true), W = zeros({V, H}, gw != nullptr);
  std::memcpy(h->data.data(), hidden, sizeof(float) * (size_t)T * H);
  std::memcpy(W->data.data(), w, sizeof(float) * (size_t)V * H);
  std::vector<int> tg(targets, targets + T);
  TP loss = fusedCrossEntropy(h, W, tg, chunk);
  if (lossGrad != 0) {
    if (gh) std::memcpy(h->grad.data(), gh, sizeof(float) * (size_t)T * H);
    if (gw) std::memcpy(W->grad.data(), gw, sizeof(float) * (size_t)V * H);
    loss->grad[0] = lossGrad;
    loss->backward_fn();
    if (gh) std::memcpy(gh, h->grad.data(), sizeof(float) * (size_t)T * H);
    if (gw) std::memcpy(gw, W->grad.data(), sizeof(float) * (size_t)V * H);
  }
  return loss->data[0];
}
// soft CE: returns loss; backward into glogits (accumulating) when lossGrad != 0
float orc_soft_ce(const float* logits, const int* ids, const float* q, int T, int V, int k, float lossGrad,
                  float* glogits) {
  TP L = zeros({T, V}, true);
  std::memcpy(L->data.data(), logits, sizeof(float) * (size_t)T * V);
  std::vector<int> id(ids, ids + (size_t)T * k);
  std::vector<float> qq(q, q + (size_t)T * k);
  TP loss = softCrossEntropy(L, id, qq, k);
  if (lossGrad != 0 && glogits) {
    std::memcpy(L->grad.data(), glogits, sizeof(float) * (size_t)T * V);
    loss->grad[0] = lossGrad;
    loss->backward_fn();
    std::memcpy(glogits, L->grad.data(), sizeof(float) * (size_t)T * V);
  }
  return loss->data[0];
}

void orc_newton_schulz(const float* G, int m, int n, int steps, float* out) {
  std::vector<float> g(G, G + (size_t)m * n);
  std::vector<float> o = newtonSchulz(g, m, n, steps);
  std::memcpy(out, o.data(), sizeof(float) * o.size());
}
double orc_wsd(int warmup, int stable, int cooldown, double minScale, int step) {
  return wsd(warmup, stable, cooldown, minScale, step);
}
double orc_qk_logit_scale(const float* qn, const float* kn, int hd) { return qkLogitScale(qn, kn, hd); }

// ---- model handle ----
struct ModelH {
  Model* m;
  std::vector<TP> params;
  std::vector<int> group;  // 0 muon, 1 aux  (for the live trainable set)
  Lora* lora = nullptr;
  AdamW* adam = nullptr;
  Muon* muon = nullptr;
  TP lastLoss;
};

// icfg: arch, vocab, hidden, nLayers, nHeads, nKV, headDim, ffn, slidingWindow, swaPattern, tie, initMode
// fcfg: ropeBase, ropeBaseLocal, rmsEps
void* orc_model_new(const int* icfg, const double* fcfg, uint32_t seed) {
  Config c;
  c.arch = icfg[0]; c.vocab = icfg[1]; c.hidden = icfg[2]; c.nLayers = icfg[3]; c.nHeads = icfg[4]; c.nKV = icfg[5];
  c.headDim = icfg[6]; c.ffn = icfg[7]; c.slidingWindow = icfg[8]; c.swaPattern = icfg[9]; c.tie = icfg[10];
  c.initMode = icfg[11];
  c.ropeBase = fcfg[0]; c.ropeBaseLocal = fcfg[1]; c.rmsEps = fcfg[2];
  Rng rng(seed);
  ModelH* h = new ModelH();
  h->m = new Model(c, rng);
  h->params = h->m->params();
  std::vector<TP> mu, au;
  h->m->groups(mu, au);
  std::unordered_set<Tensor*> ms;
  for (auto& t : mu) ms.insert(t.get());
  for (auto& t : h->params) h->group.push_back(ms.count(t.get()) ? 0 : 1);
  return h;
}
void orc_model_free(void* hp) {
  ModelH* h = (ModelH*)hp;
  g_lora.clear();
  delete h->adam; delete h->muon; delete h->lora; delete h->m; delete h;
}
int orc_model_nparams(void* hp) { return (int)((ModelH*)hp)->params.size(); }
// info: [size, rank, dim0, dim1, group, requiresGrad]
void orc_model_param_info(void* hp, int i, long* info) {
  ModelH* h = (ModelH*)hp;
  Tensor& t = *h->params[i];
  info[0] = (long)t.size(); info[1] = (long)t.shape.size(); info[2] = t.shape[0];
  info[3] = t.shape.size() > 1 ? t.shape[1] : 1; info[4] = h->group[i]; info[5] = t.requiresGrad;
}
float* orc_model_param_data(void* hp, int i) { return ((ModelH*)hp)->params[i]->data.data(); }
float* orc_model_param_grad(void* hp, int i) { return ((ModelH*)hp)->params[i]->grad.data(); }
void orc_model_zero_grad(void* hp) { for (auto& p : ((ModelH*)hp)->params) p->zeroGrad(); }

// applyLora: appends adapters (a0,b0,a1,b1,...) to the handle's param list as aux
int orc_model_apply_lora(void* hp, int rank, double alpha, uint32_t seed) {
  ModelH* h = (ModelH*)hp;
  Rng rng(seed);
  h->lora = applyLora(*h->m, rank, alpha, rng);
  for (auto& t : h->lora->aux) { h->params.push_back(t); h->group.push_back(1); }
  return (int)h->lora->aux.size();
}
void orc_model_lora_fold(void* hp, double sign) { ((ModelH*)hp)->lora->fold(sign); }

// one sequence: loss = sequenceLoss(...); backward(loss, seed) when seed != 0. Returns loss.
float orc_model_loss_backward(void* hp, const int* ids, const int* targets, int T, int lossChunk, double seed) {
  ModelH* h = (ModelH*)hp;
  std::vector<int> id(ids, ids + T), tg(targets, targets + T);
  TP loss = sequenceLoss(*h->m, id, tg, lossChunk);
  if (seed != 0) backward(loss, seed);
  h->lastLoss = loss;
  return loss->data[0];
}
// forward only to logits [T,V]
void orc_model_forward(void* hp, const int* ids, int T, float* logits) {
  ModelH* h = (ModelH*)hp;
  std::vector<int> id(ids, ids + T);
  TP l = h->m->forward(id);
  std::memcpy(logits, l->data.data(), sizeof(float) * l->size());
}
// per-layer outputs of the last forward ([T,hidden] each) and the final normed hidden (layer == nLayers)
void orc_model_layer_out(void* hp, int layer, float* out) {
  ModelH* h = (ModelH*)hp;
  TP t = layer < (int)h->m->layerOut.size() ? h->m->layerOut[layer] : h->m->lastHidden;
  std::memcpy(out, t->data.data(), sizeof(float) * t->size());
}

// optimizers over the handle's trainable params. which: 0 = AdamW on everything trainable,
// 1 = Muon on group 0 + AdamW on group 1.
void orc_opt_new(void* hp, int which, double lr, double auxLr, double beta1, double beta2, double eps, double wd,
                 double clip, double momentum, int nesterov, int nsSteps) {
  ModelH* h = (ModelH*)hp;
  std::vector<TP> mu, au;
  for (size_t i = 0; i < h->params.size(); i++) {
    if (!h->params[i]->requiresGrad) continue;
    if (which == 1 && h->group[i] == 0) mu.push_back(h->params[i]); else au.push_back(h->params[i]);
  }
  delete h->adam; delete h->muon; h->adam = nullptr; h->muon = nullptr;
  if (which == 0) h->adam = new AdamW(au, lr, beta1, beta2, eps, wd, clip);
  else h->muon = new Muon(mu, au, lr, momentum, nesterov != 0, nsSteps, AdamW(au, auxLr, beta1, beta2, eps, wd, clip));
}
void orc_opt_set_lr_scale(void* hp, double s) {
  ModelH* h = (ModelH*)hp;
  if (h->adam) h->adam->setLrScale(s);
  if (h->muon) h->muon->setLrScale(s);
}
void orc_opt_zero_grad(void* hp) {
  ModelH* h = (ModelH*)hp;
  if (h->adam) h->adam->zeroGrad();
  if (h->muon) h->muon->zeroGrad();
}
void orc_opt_step(void* hp) {
  ModelH* h = (ModelH*)hp;
  if (h->adam) h->adam->step();
  if (h->muon) h->muon->step();
}
int orc_model_qk_clip(void* hp, double tau) { return applyQKClip(*((ModelH*)hp)->m, tau); }

// Standalone AdamW / Muon on raw arrays (per-optimizer parity tests): params given as
// n arrays with sizes; state arrays m, v (or momentum) are caller-owned and updated in place.
void orc_adamw_step_arrays(int n, float** data, float** grad, float** m, float** v, const long* sizes, int t, double lr,
                           double beta1, double beta2, double eps, double wd, double clip) {
  std::vector<TP> ps;
  for (int i = 0; i < n; i++) {
    TP p = zeros({(int)sizes[i]}, true);
    std::memcpy(p->data.data(), data[i], sizeof(float) * sizes[i]);
    std::memcpy(p->grad.data(), grad[i], sizeof(float) * sizes[i]);
    ps.push_back(p);
  }
  AdamW opt(ps, lr, beta1, beta2, eps, wd, clip);
  opt.t = t - 1;
  for (int i = 0; i < n; i++) {
    std::memcpy(opt.m[i].data(), m[i], sizeof(float) * sizes[i]);
    std::memcpy(opt.v[i].data(), v[i], sizeof(float) * sizes[i]);
  }
  opt.step();
  for (int i = 0; i < n; i++) {
    std::memcpy(data[i], ps[i]->data.data(), sizeof(float) * sizes[i]);
    std::memcpy(grad[i], ps[i]->grad.data(), sizeof(float) * sizes[i]);
    std::memcpy(m[i], opt.m[i].data(), sizeof(float) * sizes[i]);
    std::memcpy(v[i], opt.v[i].data(), sizeof(float) * sizes[i]);
  }
}
void orc_muon_step_array(float* data, const float* grad, float* buf, int rows, int cols, double lr, double momentum,
                         int nesterov, int nsSteps) {
  TP p = zeros({rows, cols}, true);
  size_t n = (size_t)rows * cols;
  std::memcpy(p->data.data(), data, sizeof(float) * n);
  std::memcpy(p->grad.data(), grad, sizeof(float) * n);
  Muon opt({p}, {}, lr, momentum, nesterov != 0, nsSteps, AdamW({}, 0, 0.9, 0.999, 1e-8, 0, 0));
  std::memcpy(opt.bufs[0].data(), buf, sizeof(float) * n);
  opt.step();
  std::memcpy(data, p->data.data(), sizeof(float) * n);
  std::memcpy(buf, opt.bufs[0].data(), sizeof(float) * n);
}

}  // extern "C"
