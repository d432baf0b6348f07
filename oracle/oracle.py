"""ctypes binding of the CPU oracle (``liboracle.so``, built from ``oracle.cpp``).

TEST INFRASTRUCTURE, NOT PRODUCT CODE: only the test-suite, the smoke check and
the benchmark's CPU-baseline leg import this module. It restates gguf-trainer's
reference (CPU) ops, optimizers and architectures; see ``oracle.cpp`` for the
file:line citations.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

F32P = C.POINTER(C.c_float)
I32P = C.POINTER(C.c_int)


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` next to its source when missing or stale."""
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        L.orc_rng_next.restype = C.c_double
        L.orc_wsd.restype = C.c_double
        L.orc_qk_logit_scale.restype = C.c_double
        L.orc_ce_fwd.restype = C.c_float
        L.orc_fused_ce.restype = C.c_float
        L.orc_soft_ce.restype = C.c_float
        L.orc_model_new.restype = C.c_void_p
        L.orc_model_param_data.restype = F32P
        L.orc_model_param_grad.restype = F32P
        L.orc_model_loss_backward.restype = C.c_float
        _lib = L
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(F32P)


def _i(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(I32P)


def _fp(a):
    """Pointer to an existing contiguous f32 array (in-place use) or NULL."""
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(F32P)


def set_threads(n: int):
    lib().orc_set_threads(int(n))


def max_threads() -> int:
    return int(lib().orc_max_threads())


def set_checkpointing(on: bool):
    lib().orc_set_checkpointing(1 if on else 0)


class Mulberry32:
    """`mulberry32(seed)` of src/model/autograd.ts:69-78, state kept across calls."""

    def __init__(self, seed: int):
        self.state = C.c_uint32(seed & 0xFFFFFFFF)

    def __call__(self) -> float:
        return float(lib().orc_rng_next(C.byref(self.state)))

    def randn(self, shape, scale=1.0) -> np.ndarray:
        """`randn(rng) * scale` per element, f32 (param(), the tests' randTensor)."""
        out = np.empty(shape, dtype=np.float32)
        lib().orc_randn_fill(C.byref(self.state), _fp(out), C.c_long(out.size), C.c_double(scale))
        return out

    def uniform_pm1(self, shape) -> np.ndarray:
        """`rng()*2-1` per element (tests/gpu-parity.ts:103-105)."""
        out = np.empty(shape, dtype=np.float32)
        lib().orc_uniform_pm1_fill(C.byref(self.state), _fp(out), C.c_long(out.size))
        return out

    def randint(self, n: int, hi: int) -> np.ndarray:
        """`Math.floor(rng() * hi)` n times."""
        return np.array([int(self() * hi) for _ in range(n)], dtype=np.int32)


# ---------------------------------------------------------------------------
# per-op functional API (backward accumulates into the arrays passed in)
# ---------------------------------------------------------------------------
def linear_fwd(x, w):
    x, xp = _f(x); w, wp = _f(w)
    T, i = x.shape; o = w.shape[0]
    y = np.empty((T, o), np.float32)
    lib().orc_linear_fwd(xp, wp, T, i, o, _fp(y))
    return y


def linear_bwd(x, w, gy, gx=None, gw=None, want_dw=True):
    x, xp = _f(x); w, wp = _f(w); gy, gp = _f(gy)
    T, i = x.shape; o = w.shape[0]
    gx = np.zeros_like(x) if gx is None else gx
    if want_dw and gw is None:
        gw = np.zeros_like(w)
    lib().orc_linear_bwd(xp, wp, gp, T, i, o, _fp(gx), _fp(gw) if want_dw else None)
    return gx, gw


def elementwise(op, a, b=None, c=0.0, gy=None):
    """op in add/mul/silu/gelu/scale -> (out, ga, gb)."""
    code = {"add": 0, "mul": 1, "silu": 2, "gelu": 3, "scale": 4}[op]
    a, ap = _f(a)
    bp = None
    if b is not None:
        b, bp = _f(b)
    out = np.empty_like(a); ga = np.zeros_like(a); gb = np.zeros_like(a)
    gp = None
    if gy is not None:
        gy, gp = _f(gy)
    lib().orc_elementwise(code, ap, bp, C.c_long(a.size), C.c_double(c), gp, _fp(out), _fp(ga), _fp(gb))
    return out, ga, (gb if b is not None else None)


def rmsnorm_fwd(x, w, eps):
    x, xp = _f(x); w, wp = _f(w)
    d = w.shape[0]; rows = x.size // d
    y = np.empty_like(x); rinv = np.empty(rows, np.float32)
    lib().orc_rmsnorm_fwd(xp, wp, rows, d, C.c_double(eps), _fp(y), _fp(rinv))
    return y, rinv


def rmsnorm_bwd(x, w, rinv, gy, want_dw=True):
    x, xp = _f(x); w, wp = _f(w); rinv, rp = _f(rinv); gy, gp = _f(gy)
    d = w.shape[0]; rows = x.size // d
    gx = np.zeros_like(x); gw = np.zeros_like(w) if want_dw else None
    lib().orc_rmsnorm_bwd(xp, wp, rp, gp, rows, d, _fp(gx), _fp(gw))
    return gx, gw


def rope_fwd(x, T, H, hd, base, pos_offset=0):
    x, xp = _f(x)
    y = np.empty_like(x)
    lib().orc_rope_fwd(xp, T, H, hd, C.c_double(base), pos_offset, _fp(y))
    return y


def rope_bwd(gy, T, H, hd, base, pos_offset=0):
    gy, gp = _f(gy)
    gx = np.zeros_like(gy)
    lib().orc_rope_bwd(gp, T, H, hd, C.c_double(base), pos_offset, _fp(gx))
    return gx


def attention_fwd(q, k, v, T, Hq, Hkv, hd, window=0):
    q, qp = _f(q); k, kp = _f(k); v, vp = _f(v)
    out = np.zeros((T, Hq * hd), np.float32)
    probs = np.zeros((Hq, T, T), np.float32)
    lib().orc_attention_fwd(qp, kp, vp, T, Hq, Hkv, hd, window, _fp(out), _fp(probs))
    return out, probs


def attention_bwd(q, k, v, probs, gout, T, Hq, Hkv, hd, window=0):
    q, qp = _f(q); k, kp = _f(k); v, vp = _f(v); probs, pp = _f(probs); gout, gp = _f(gout)
    gq = np.zeros_like(q); gk = np.zeros_like(k); gv = np.zeros_like(v)
    lib().orc_attention_bwd(qp, kp, vp, pp, gp, T, Hq, Hkv, hd, window, _fp(gq), _fp(gk), _fp(gv))
    return gq, gk, gv


def embedding_fwd(w, ids):
    w, wp = _f(w); ids, ip = _i(ids)
    out = np.empty((ids.size, w.shape[1]), np.float32)
    lib().orc_embedding_fwd(wp, ip, ids.size, w.shape[1], _fp(out))
    return out


def embedding_bwd(gy, ids, V):
    gy, gp = _f(gy); ids, ip = _i(ids)
    gw = np.zeros((V, gy.shape[1]), np.float32)
    lib().orc_embedding_bwd(gp, ip, ids.size, gy.shape[1], _fp(gw))
    return gw


def kept_rows(targets):
    return int((np.asarray(targets) >= 0).sum())


def ce_fwd(logits, targets):
    logits, lp = _f(logits); targets, tp = _i(targets)
    T, V = logits.shape
    probs = np.empty_like(logits)
    loss = lib().orc_ce_fwd(lp, tp, T, V, kept_rows(targets), _fp(probs))
    return np.float32(loss), probs


def ce_bwd(probs, targets, loss_grad=1.0):
    probs, pp = _f(probs); targets, tp = _i(targets)
    T, V = probs.shape
    g = np.zeros_like(probs)
    lib().orc_ce_bwd(pp, tp, T, V, kept_rows(targets), C.c_float(loss_grad), _fp(g))
    return g


def fused_ce(hidden, w, targets, chunk, loss_grad=0.0, want_dw=True):
    hidden, hp = _f(hidden); w, wp = _f(w); targets, tp = _i(targets)
    T, H = hidden.shape; V = w.shape[0]
    gh = np.zeros_like(hidden); gw = np.zeros_like(w) if want_dw else None
    loss = lib().orc_fused_ce(hp, wp, tp, T, H, V, chunk, C.c_float(loss_grad), _fp(gh), _fp(gw))
    return np.float32(loss), gh, gw


def soft_ce(logits, ids, q, k, loss_grad=0.0):
    logits, lp = _f(logits); ids, ip = _i(ids); q, qp = _f(q)
    T, V = logits.shape
    g = np.zeros_like(logits)
    loss = lib().orc_soft_ce(lp, ip, qp, T, V, k, C.c_float(loss_grad), _fp(g))
    return np.float32(loss), g


def newton_schulz(G, steps=5):
    G, gp = _f(G)
    m, n = G.shape
    out = np.empty_like(G)
    lib().orc_newton_schulz(gp, m, n, steps, _fp(out))
    return out


def wsd(warmup, stable, cooldown, min_scale, step) -> float:
    return float(lib().orc_wsd(warmup, stable, cooldown, C.c_double(min_scale), step))


def qk_logit_scale(qn, kn, hd) -> float:
    qn, qp = _f(qn); kn, kp = _f(kn)
    return float(lib().orc_qk_logit_scale(qp, kp, hd))


def adamw_step_arrays(data, grad, m, v, t, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, clip=1.0):
    """One AdamW.step() over a parameter group held as lists of f32 arrays (updated in place)."""
    n = len(data)
    arr = lambda xs: (F32P * n)(*[_fp(x) for x in xs])
    sizes = (C.c_long * n)(*[x.size for x in data])
    lib().orc_adamw_step_arrays(n, arr(data), arr(grad), arr(m), arr(v), sizes, int(t), C.c_double(lr),
                                C.c_double(beta1), C.c_double(beta2), C.c_double(eps), C.c_double(wd),
                                C.c_double(clip))


def muon_step_array(data, grad, buf, lr, momentum=0.95, nesterov=True, ns_steps=5):
    rows, cols = data.shape
    lib().orc_muon_step_array(_fp(data), _fp(grad), _fp(buf), rows, cols, C.c_double(lr), C.c_double(momentum),
                              1 if nesterov else 0, ns_steps)


# ---------------------------------------------------------------------------
# whole model
# ---------------------------------------------------------------------------
ARCH = {"llama": 0, "qwen3": 1, "gemma3": 2}


class Model:
    """A reference-CPU model (llama / qwen3 / gemma3) with its params, grads and optimizers."""

    def __init__(self, cfg: dict, seed: int):
        self.cfg = dict(cfg)
        icfg = (C.c_int * 12)(
            ARCH[cfg["arch"]], cfg["vocab"], cfg["hidden"], cfg["layers"], cfg["heads"], cfg["kv_heads"],
            cfg["head_dim"], cfg["ffn"], cfg.get("window", 0), cfg.get("swa_pattern", 0),
            1 if cfg.get("tie", True) else 0, 1 if cfg.get("init", "reference") == "n002" else 0)
        fcfg = (C.c_double * 3)(cfg["rope_base"], cfg.get("rope_base_local", cfg["rope_base"]), cfg["eps"])
        self.h = C.c_void_p(lib().orc_model_new(icfg, fcfg, C.c_uint32(seed)))

    def close(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def nparams(self) -> int:
        return int(lib().orc_model_nparams(self.h))

    def info(self, i):
        info = (C.c_long * 6)()
        lib().orc_model_param_info(self.h, i, info)
        size, rank, d0, d1, group, rg = [int(x) for x in info]
        shape = (d0, d1) if rank == 2 else (d0,)
        return {"size": size, "shape": shape, "group": "muon" if group == 0 else "aux", "requires_grad": bool(rg)}

    def data(self, i) -> np.ndarray:
        inf = self.info(i)
        p = lib().orc_model_param_data(self.h, i)
        return np.ctypeslib.as_array(p, shape=(inf["size"],)).reshape(inf["shape"])

    def grad(self, i) -> np.ndarray:
        inf = self.info(i)
        p = lib().orc_model_param_grad(self.h, i)
        return np.ctypeslib.as_array(p, shape=(inf["size"],)).reshape(inf["shape"])

    def zero_grad(self):
        lib().orc_model_zero_grad(self.h)

    def apply_lora(self, rank, alpha, seed) -> int:
        return int(lib().orc_model_apply_lora(self.h, rank, C.c_double(alpha), C.c_uint32(seed)))

    def lora_fold(self, sign):
        lib().orc_model_lora_fold(self.h, C.c_double(sign))

    def loss_backward(self, ids, targets, loss_chunk=0, seed=1.0) -> np.float32:
        ids, ip = _i(ids); targets, tp = _i(targets)
        return np.float32(lib().orc_model_loss_backward(self.h, ip, tp, ids.size, loss_chunk, C.c_double(seed)))

    def forward(self, ids) -> np.ndarray:
        ids, ip = _i(ids)
        out = np.empty((ids.size, self.cfg["vocab"]), np.float32)
        lib().orc_model_forward(self.h, ip, ids.size, _fp(out))
        return out

    def layer_out(self, layer, T) -> np.ndarray:
        out = np.empty((T, self.cfg["hidden"]), np.float32)
        lib().orc_model_layer_out(self.h, layer, _fp(out))
        return out

    def make_optimizer(self, kind, lr, aux_lr=None, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, clip=1.0,
                       momentum=0.95, nesterov=True, ns_steps=5):
        lib().orc_opt_new(self.h, 0 if kind == "adamw" else 1, C.c_double(lr),
                          C.c_double(lr if aux_lr is None else aux_lr), C.c_double(beta1), C.c_double(beta2),
                          C.c_double(eps), C.c_double(wd), C.c_double(clip), C.c_double(momentum),
                          1 if nesterov else 0, ns_steps)

    def opt_set_lr_scale(self, s):
        lib().orc_opt_set_lr_scale(self.h, C.c_double(s))

    def opt_zero_grad(self):
        lib().orc_opt_zero_grad(self.h)

    def opt_step(self):
        lib().orc_opt_step(self.h)

    def qk_clip(self, tau) -> int:
        return int(lib().orc_model_qk_clip(self.h, C.c_double(tau)))
