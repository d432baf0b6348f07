"""A stand-in for `libgguftrain_cuda.so` written in numpy, for tests of the HOST side on machines without a GPU.

Test infrastructure only (nothing outside `tests/` imports it). It implements the entry points of
`include/gguftrain.h` that `gguf_trainer_b200/backend.py` calls for an eager (unrecorded) forward and backward, with
the meaning the header gives them: device memory is a dictionary of byte arrays behind made-up addresses, every "kernel"
is a few numpy lines computed in f64 and stored as f32 (the reference's CPU numerics, src/model/autograd.ts), and every
call is written to a log. With it the `-m "not gpu"` suite can drive `CudaBackend` itself: which launches it merges,
which buffers it asks to be accumulated into, what it leaves unwritten, and that gradients come out the same whichever
way the launches were grouped.

It is not a CPU fallback of the product: `CudaBackend` only ever sees it when a test swaps `_lib.load`.
"""
from __future__ import annotations

import bisect
import ctypes as C
import math

import numpy as np

NT, NN, TN = 0, 1, 2
IGNORE = 0xFFFFFFFF


def _ints(arr, n):
    return [int(arr[i]) for i in range(n)]


class FakeLib:
    """One instance = one library + one context."""

    def __init__(self):
        self._bases = []            # sorted base addresses
        self._bufs = {}             # base -> np.uint8 array
        self._next = 0x10000000
        self.log = []               # (entry point name, dict of the arguments a test may want to look at)
        self.launches = 0
        self.batch = (0, 0)
        self.precision = 0
        self._tickets = {}
        self._nextTicket = 1
        self._recording = None      # the list a recording in progress appends to
        self.state_bytes = 0
        self.pool_bytes = 0

    # ------------------------------------------------------------------ recording and replay (gt_graph_*)
    # While a recording is open, device work is not run: the call and its arguments are appended to the recording, and
    # gt_graph_launch runs them in order, as a CUDA graph would. Host-side calls (allocation, statistics) run at once;
    # host transfers are refused, as the library refuses them.
    _HOST_SIDE = {"gt_init", "gt_destroy", "gt_last_error", "gt_device_name", "gt_set_precision", "gt_set_batch", "gt_alloc",
                  "gt_alloc_state", "gt_free", "gt_stats", "gt_graph_begin", "gt_graph_end", "gt_graph_launch", "gt_graph_destroy",
                  "gt_adamw_create", "gt_adamw_set_lr", "gt_adamw_state", "gt_adamw_get_t", "gt_adamw_set_t", "gt_dp_unique_id",
                  "gt_dp_init", "gt_dp_reserve_sms", "gt_dp_destroy", "gt_muon_create", "gt_muon_set_lr", "gt_muon_state",
                  "gt_muon_set_sharded"}
    # (the exchange is issued by the host between recorded segments, never into one)
    _REFUSED_WHILE_RECORDING = {"gt_write", "gt_read", "gt_read_async", "gt_read_fence", "gt_sync", "gt_dp_allreduce_start",
                                "gt_dp_wait", "gt_dp_wait_host"}

    def __getattribute__(self, name):
        attr = object.__getattribute__(self, name)
        if not name.startswith("gt_"):
            return attr
        rec = object.__getattribute__(self, "__dict__").get("_recording")
        if rec is None or name in FakeLib._HOST_SIDE:
            return attr
        if name in FakeLib._REFUSED_WHILE_RECORDING:
            return lambda *a, **k: 4
        batch = self.batch

        def record(*args):
            rec.append((name, args, batch))
            self.launches += 1
            return 0
        return record

    def gt_graph_begin(self, ctx):
        if self.__dict__.get("_recording") is not None:
            return 4
        self._recording = []
        return 0

    def gt_graph_end(self, ctx, ref):
        if not hasattr(self, "_graphs"):
            self._graphs = {}
        h = len(self._graphs) + 1
        self._graphs[h] = self._recording
        self._recording = None
        ref._obj.value = h
        return 0

    def gt_graph_launch(self, ctx, h):
        saved = self.batch
        for name, args, batch in self._graphs[int(h)]:
            self.batch = batch                       # the shapes a recorded kernel was launched with are part of the recording
            st = getattr(FakeLib, name)(self, *args)
            if st:
                return st
        self.batch = saved
        return 0

    def gt_graph_destroy(self, ctx, h):
        self._graphs.pop(int(h), None)
        return 0

    # ------------------------------------------------------------------ memory model
    def _new(self, nbytes, zero):
        size = max(256, (int(nbytes) + 255) // 256 * 256)
        base = self._next
        self._next += size + 256            # a gap, so that running off the end of a buffer is caught by _view
        buf = np.zeros(size, np.uint8) if zero else np.full(size, 0xFF, np.uint8)   # fresh pool memory reads as NaN: using it unwritten shows
        self._bases.append(base)
        self._bufs[base] = buf
        return base

    def _view(self, addr, count, dtype=np.float32):
        addr = int(addr)
        i = bisect.bisect_right(self._bases, addr) - 1
        assert i >= 0, f"address {addr:#x} is below every allocation"
        base = self._bases[i]
        buf = self._bufs[base]
        off = addr - base
        nbytes = int(count) * np.dtype(dtype).itemsize
        assert off + nbytes <= buf.size, f"access of {nbytes} bytes at {addr:#x} runs off its {buf.size}-byte buffer"
        return buf[off:off + nbytes].view(dtype)

    def f32(self, addr, *shape):
        n = int(np.prod(shape))
        return self._view(addr, n).reshape(shape)

    def _store(self, addr, value, accum=0):
        """value (f64 array) into the f32 buffer at addr, added to what is there when accum is set."""
        out = self._view(addr, value.size).reshape(value.shape)
        if accum:
            out[...] = (out.astype(np.float64) + value).astype(np.float32)
        else:
            out[...] = value.astype(np.float32)

    def _called(self, name, **kw):
        self.log.append((name, kw))
        self.launches += 1
        return 0

    def calls(self, name):
        return [kw for n, kw in self.log if n == name]

    def count(self, name):
        return sum(1 for n, _ in self.log if n == name)

    # ------------------------------------------------------------------ context
    def gt_init(self, device, ref):
        ref._obj.value = 1
        return 0

    def gt_destroy(self, ctx):
        return 0

    def gt_last_error(self, ctx):
        return b"fake device"

    def gt_device_name(self, ctx, buf, n):
        buf.value = b"numpy stand-in"
        return 0

    def gt_set_precision(self, ctx, p):
        if p not in (0, 1):
            return 6
        self.precision = p
        return 0

    def gt_set_batch(self, ctx, b, t):
        self.batch = (int(b), int(t) if b else 0)
        return 0

    def _seq(self, rows):
        b, t = self.batch
        if b:
            assert rows == b * t, f"{rows} rows but the batch is {b} x {t}"
            return t, b
        return rows, 1

    def gt_alloc(self, ctx, nbytes, ref):
        ref._obj.value = self._new(nbytes, zero=False)
        self.pool_bytes += int(nbytes)
        return 0

    def gt_alloc_state(self, ctx, nbytes, ref):
        ref._obj.value = self._new(nbytes, zero=True)
        self.state_bytes += int(nbytes)
        return 0

    def gt_free(self, ctx, addr):
        return 0                               # (nothing is reused: stale addresses stay readable, which is harmless here)

    def gt_write(self, ctx, dst, host, nbytes):
        src = np.frombuffer((C.c_ubyte * int(nbytes)).from_address(int(host)), np.uint8)
        self._view(dst, nbytes, np.uint8)[...] = src
        return 0

    def gt_read(self, ctx, src, host, nbytes):
        out = np.frombuffer((C.c_ubyte * int(nbytes)).from_address(int(host)), np.uint8)
        out[...] = self._view(src, nbytes, np.uint8)
        return 0

    def gt_read_async(self, ctx, src, nbytes, ref):
        t = self._nextTicket
        self._nextTicket += 1
        self._tickets[t] = self._view(src, nbytes, np.uint8).copy()
        ref._obj.value = t
        return 0

    def gt_read_fence(self, ctx):
        return 0

    def gt_read_finish(self, ctx, ticket, host, nbytes):
        data = self._tickets.pop(int(ticket))
        out = np.frombuffer((C.c_ubyte * int(nbytes)).from_address(int(host)), np.uint8)
        out[...] = data[:int(nbytes)]
        return 0

    def gt_zero(self, ctx, addr, nbytes):
        self._view(addr, nbytes, np.uint8)[...] = 0
        self.log.append(("gt_zero", dict(addr=int(addr), bytes=int(nbytes))))
        return 0

    def gt_copy(self, ctx, dst, src, nbytes):
        self._view(dst, nbytes, np.uint8)[...] = self._view(src, nbytes, np.uint8)
        self.log.append(("gt_copy", dict(dst=int(dst), src=int(src), bytes=int(nbytes))))
        return 0

    def gt_sync(self, ctx):
        return 0

    def gt_stats(self, ctx, out):
        out[0], out[1], out[2], out[3] = self.pool_bytes, self.state_bytes, 0, self.launches
        return 0

    def gt_event_record(self, ctx, slot):
        return 0

    def gt_event_elapsed_ms(self, ctx, a, b, ref):
        ref._obj.value = 0.0
        return 0

    # ------------------------------------------------------------------ matrix products
    def _operands(self, kind, M, N, K, a, b):
        if kind == NT:
            return self.f32(a, M, K).astype(np.float64), self.f32(b, N, K).astype(np.float64).T
        if kind == NN:
            return self.f32(a, M, K).astype(np.float64), self.f32(b, K, N).astype(np.float64)
        assert kind == TN
        return self.f32(a, K, M).astype(np.float64).T, self.f32(b, K, N).astype(np.float64)

    def _product(self, kind, M, N, K, a, b):
        A, B = self._operands(kind, M, N, K, a, b)
        return A @ B

    def gt_gemm(self, ctx, kind, accum, M, N, K, a, b, c):
        return self.gt_gemm_scaled(ctx, kind, accum, M, N, K, a, b, c, 1.0, _name="gt_gemm")

    def gt_gemm_scaled(self, ctx, kind, accum, M, N, K, a, b, c, alpha, _name="gt_gemm_scaled"):
        self._store(c, float(alpha) * self._product(kind, M, N, K, a, b), accum)
        return self._called(_name, kind=kind, accum=accum, M=M, N=N, K=K, a=int(a), b=int(b), c=int(c))

    def gt_gemm2(self, ctx, kind, accum, M, N, K, a, b, K2, a2, b2, c):
        self._store(c, self._product(kind, M, N, K, a, b) + self._product(kind, M, N, K2, a2, b2), accum)
        return self._called("gt_gemm2", kind=kind, accum=accum, M=M, N=N, K=K, K2=K2, c=int(c))

    def gt_gemm_multi(self, ctx, kind, accum, M, N, nparts, Ks, As, Bs, c):
        total = 0.0
        for p in range(nparts):
            total = total + self._product(kind, M, N, int(Ks[p]), int(As[p]), int(Bs[p]))
        self._store(c, total, accum)
        return self._called("gt_gemm_multi", kind=kind, accum=accum, M=M, N=N, Ks=_ints(Ks, nparts), c=int(c))

    def gt_gemm_grouped(self, ctx, kind, n, Ms, Ns, K, As, Bs, Cs, accums):
        return self.gt_gemm_grouped_scaled(ctx, kind, n, Ms, Ns, K, As, Bs, Cs, accums, 1.0, _name="gt_gemm_grouped")

    def gt_gemm_grouped_scaled(self, ctx, kind, n, Ms, Ns, K, As, Bs, Cs, accums, alpha, _name="gt_gemm_grouped_scaled"):
        for g in range(n):
            self._store(int(Cs[g]), float(alpha) * self._product(kind, int(Ms[g]), int(Ns[g]), K, int(As[g]), int(Bs[g])), int(accums[g]))
        return self._called(_name, kind=kind, n=n, Ms=_ints(Ms, n), Ns=_ints(Ns, n), K=K, accums=_ints(accums, n), cs=_ints(Cs, n))

    # ------------------------------------------------------------------ rotary embedding
    def _angles(self, rows, hd, base, pos_offset):
        T, _nseq = self._seq(rows)
        half = hd // 2
        pos = (np.arange(rows) % T + pos_offset).astype(np.float64)
        freq = np.power(float(base), -2.0 * np.arange(half) / hd)
        ang = pos[:, None] * freq[None, :]
        # the table holds f32 values of f64 cosines and sines
        return np.cos(ang).astype(np.float32).astype(np.float64), np.sin(ang).astype(np.float32).astype(np.float64)

    def _rotate(self, x, rows, H, hd, base, pos_offset, transposed):
        cos, sin = self._angles(rows, hd, base, pos_offset)
        half = hd // 2
        x = x.reshape(rows, H, hd)
        a0, a1 = x[:, :, :half], x[:, :, half:]
        c, s = cos[:, None, :], sin[:, None, :]
        if transposed:
            o0, o1 = c * a0 + s * a1, -s * a0 + c * a1
        else:
            o0, o1 = a0 * c - a1 * s, a0 * s + a1 * c
        return np.concatenate([o0, o1], axis=2).reshape(rows, H * hd)

    def gt_rope_fwd(self, ctx, rows, H, hd, base, pos_offset, x, y):
        self._store(y, self._rotate(self.f32(x, rows, H * hd).astype(np.float64), rows, H, hd, base, pos_offset, False))
        return self._called("gt_rope_fwd", rows=rows, H=H, hd=hd)

    def gt_rope_bwd(self, ctx, rows, H, hd, base, pos_offset, gy, gx, accum):
        if not gx:
            return 0
        self._store(gx, self._rotate(self.f32(gy, rows, H * hd).astype(np.float64), rows, H, hd, base, pos_offset, True), accum)
        return self._called("gt_rope_bwd", rows=rows, H=H, hd=hd, accum=accum)

    def gt_linear_rope_grouped(self, ctx, n, rows, K, x, Ns, Ws, Ys, heads, hd, base, pos_offset):
        for g in range(n):
            N = int(Ns[g])
            y = self._product(NT, rows, N, K, x, int(Ws[g]))
            if int(heads[g]) > 0:
                assert int(heads[g]) * hd == N
                y = self._rotate(y.astype(np.float32).astype(np.float64), rows, int(heads[g]), hd, base, pos_offset, False)
            self._store(int(Ys[g]), y)
        return self._called("gt_linear_rope_grouped", n=n, rows=rows, K=K, Ns=_ints(Ns, n), heads=_ints(heads, n), hd=hd)

    # ------------------------------------------------------------------ elementwise (add 0, mul 1, silu 2, gelu 3, scale 4)
    @staticmethod
    def _act(op, x):
        """value and derivative of silu (2) or tanh-form gelu (3)"""
        if op == 2:
            sig = 1.0 / (1.0 + np.exp(-x))
            return x * sig, sig * (1.0 + x * (1.0 - sig))
        assert op == 3
        k, a = 0.7978845608028654, 0.044715
        th = np.tanh(k * (x + a * x ** 3))
        return 0.5 * x * (1.0 + th), 0.5 * (1.0 + th) + 0.5 * x * (1.0 - th ** 2) * k * (1.0 + 3.0 * a * x * x)

    def gt_ew_fwd(self, ctx, op, n, a, b, c, out):
        A = self.f32(a, n).astype(np.float64)
        if op == 0:
            r = A + self.f32(b, n)
        elif op == 1:
            r = A * self.f32(b, n)
        elif op in (2, 3):
            r = self._act(op, A)[0]
        else:
            r = A * float(c)
        self._store(out, r)
        return self._called("gt_ew_fwd", op=op, n=n, out=int(out))

    def gt_ew_bwd(self, ctx, op, n, a, b, c, gout, ga, acc_a, gb, acc_b):
        g = self.f32(gout, n).astype(np.float64)
        A = self.f32(a, n).astype(np.float64) if a else None
        B = self.f32(b, n).astype(np.float64) if b else None
        if op == 0:
            da, db = g, g
        elif op == 1:
            da, db = g * B, g * A
        elif op in (2, 3):
            da, db = g * self._act(op, A)[1], None
        else:
            da, db = g * float(c), None
        if ga and gb and int(ga) == int(gb):          # add(t, t) / mul(t, t): one buffer takes both terms in one write
            self._store(ga, da + db, acc_a)
        else:
            if ga:
                self._store(ga, da, acc_a)
            if gb and db is not None:
                self._store(gb, db, acc_b)
        return self._called("gt_ew_bwd", op=op, n=n, ga=int(ga), acc_a=acc_a, gb=int(gb), acc_b=acc_b)

    def gt_glu_fwd(self, ctx, op, n, x, u, out):
        self._store(out, self._act(op, self.f32(x, n).astype(np.float64))[0] * self.f32(u, n))
        return self._called("gt_glu_fwd", op=op, n=n)

    def gt_glu_bwd(self, ctx, op, n, x, u, gout, gx, acc_x, gu, acc_u):
        X, U, g = (self.f32(p, n).astype(np.float64) for p in (x, u, gout))
        act, dact = self._act(op, X)
        if gx:
            self._store(gx, g * U * dact, acc_x)
        if gu:
            self._store(gu, g * act, acc_u)
        return self._called("gt_glu_bwd", op=op, n=n, gx=int(gx), acc_x=acc_x, gu=int(gu), acc_u=acc_u)

    def gt_glu_linear_fwd(self, ctx, op, rows, ffn, inDim, x, wg, wu, gate, up, out):
        G = self._product(NT, rows, ffn, inDim, x, wg).astype(np.float32).astype(np.float64)
        U = self._product(NT, rows, ffn, inDim, x, wu).astype(np.float32).astype(np.float64)
        self._store(gate, G)
        self._store(up, U)
        self._store(out, self._act(op, G)[0] * U)
        return self._called("gt_glu_linear_fwd", op=op, rows=rows, ffn=ffn, inDim=inDim)

    # ------------------------------------------------------------------ RMSNorm
    def _norm(self, X, W, eps):
        r = 1.0 / np.sqrt((X * X).mean(axis=1) + float(eps))
        r = r.astype(np.float32).astype(np.float64)           # the statistic is stored as f32 and read back by backward
        return X * r[:, None] * W[None, :], r

    def gt_rmsnorm_fwd(self, ctx, rows, d, x, w, eps, y, rinv):
        Y, r = self._norm(self.f32(x, rows, d).astype(np.float64), self.f32(w, d).astype(np.float64), eps)
        self._store(y, Y)
        self._store(rinv, r)
        return self._called("gt_rmsnorm_fwd", rows=rows, d=d, y=int(y))

    def gt_add_rmsnorm_fwd(self, ctx, rows, d, a, b, w, eps, s, y, rinv):
        S = (self.f32(a, rows, d).astype(np.float64) + self.f32(b, rows, d)).astype(np.float32)
        self.f32(s, rows, d)[...] = S
        Y, r = self._norm(S.astype(np.float64), self.f32(w, d).astype(np.float64), eps)
        self._store(y, Y)
        self._store(rinv, r)
        return self._called("gt_add_rmsnorm_fwd", rows=rows, d=d)

    def gt_rmsnorm_heads_rope_fwd(self, ctx, rows, H, hd, x, w, eps, y, rinv, base, pos_offset):
        Y, r = self._norm(self.f32(x, rows * H, hd).astype(np.float64), self.f32(w, hd).astype(np.float64), eps)
        Y = Y.astype(np.float32).astype(np.float64).reshape(rows, H * hd)
        self._store(y, self._rotate(Y, rows, H, hd, base, pos_offset, False))
        self._store(rinv, r)
        return self._called("gt_rmsnorm_heads_rope_fwd", rows=rows, H=H, hd=hd)

    def _norm_bwd(self, rows, d, x, w, rinv, gy, gadd, gx, accum_x, gw, accum_w):
        X, G = self.f32(x, rows, d).astype(np.float64), self.f32(gy, rows, d).astype(np.float64)
        W, r = self.f32(w, d).astype(np.float64), self.f32(rinv, rows).astype(np.float64)
        if gx:
            S = (G * W[None, :] * X).sum(axis=1)
            dx = W[None, :] * r[:, None] * G - X * (r ** 3 * S / d)[:, None]
            if gadd:
                self._store(gx, self.f32(gadd, rows, d).astype(np.float64) + dx)
            else:
                self._store(gx, dx, accum_x)
        if gw:
            self._store(gw, (G * X * r[:, None]).sum(axis=0), accum_w)

    def gt_rmsnorm_bwd(self, ctx, rows, d, x, w, rinv, gy, gx, accum_x, gw, accum_w):
        self._norm_bwd(rows, d, x, w, rinv, gy, 0, gx, accum_x, gw, accum_w)
        return self._called("gt_rmsnorm_bwd", rows=rows, d=d, gx=int(gx), accum_x=accum_x, gw=int(gw), accum_w=accum_w)

    def gt_rmsnorm_bwd_add(self, ctx, rows, d, x, w, rinv, gy, gadd, gx, gw, accum_w):
        assert gadd and gx
        self._norm_bwd(rows, d, x, w, rinv, gy, gadd, gx, 1, gw, accum_w)
        return self._called("gt_rmsnorm_bwd_add", rows=rows, d=d, gadd=int(gadd), gx=int(gx), gw=int(gw), accum_w=accum_w)

    # ------------------------------------------------------------------ embedding
    def gt_embedding_fwd(self, ctx, rows, d, w, ids, out):
        idx = self._view(ids, rows, np.uint32).astype(np.int64)
        V = int(idx.max()) + 1
        self.f32(out, rows, d)[...] = self.f32(w, V, d)[idx]
        return self._called("gt_embedding_fwd", rows=rows, d=d)

    def gt_embedding_bwd(self, ctx, rows, d, gy, ids, gw):
        idx = self._view(ids, rows, np.uint32).astype(np.int64)
        V = int(idx.max()) + 1
        acc = self.f32(gw, V, d).astype(np.float64)
        np.add.at(acc, idx, self.f32(gy, rows, d).astype(np.float64))      # gw always accumulates
        self.f32(gw, V, d)[...] = acc.astype(np.float32)
        return self._called("gt_embedding_bwd", rows=rows, d=d)

    # ------------------------------------------------------------------ attention (causal, grouped queries, window)
    def _probs(self, Q, K, T, window):
        """Q:[T, hd], K:[T, hd] of one (sequence, head) -> [T, T] softmax over the allowed keys"""
        S = (Q @ K.T) / math.sqrt(Q.shape[1])
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        keep = (j <= i) & ((window == 0) | (j >= i - window + 1))
        S = np.where(keep, S, -np.inf)
        m = S.max(axis=1, keepdims=True)
        E = np.exp(S - m)
        l = E.sum(axis=1, keepdims=True)
        return E / l, m[:, 0] + np.log(l[:, 0])

    def gt_attention_fwd(self, ctx, rows, Hq, Hkv, hd, window, q, k, v, out, lse):
        T, nseq = self._seq(rows)
        Q = self.f32(q, nseq, T, Hq, hd).astype(np.float64)
        K = self.f32(k, nseq, T, Hkv, hd).astype(np.float64)
        V = self.f32(v, nseq, T, Hkv, hd).astype(np.float64)
        O = np.zeros_like(Q)
        L = np.zeros((Hq, rows))
        for s in range(nseq):
            for h in range(Hq):
                P, ls = self._probs(Q[s, :, h], K[s, :, h // (Hq // Hkv)], T, window)
                O[s, :, h] = P @ V[s, :, h // (Hq // Hkv)]
                L[h, s * T:(s + 1) * T] = ls / math.log(2.0)        # the row statistic is kept in log2 units
        self._store(out, O.reshape(rows, Hq * hd))
        self._store(lse, L)
        return self._called("gt_attention_fwd", rows=rows, Hq=Hq, Hkv=Hkv, hd=hd, window=window)

    def _attention_grads(self, rows, Hq, Hkv, hd, window, q, k, v, gout):
        T, nseq = self._seq(rows)
        Q = self.f32(q, nseq, T, Hq, hd).astype(np.float64)
        K = self.f32(k, nseq, T, Hkv, hd).astype(np.float64)
        V = self.f32(v, nseq, T, Hkv, hd).astype(np.float64)
        dO = self.f32(gout, nseq, T, Hq, hd).astype(np.float64)
        dQ, dK, dV = np.zeros_like(Q), np.zeros_like(K), np.zeros_like(V)
        scale = 1.0 / math.sqrt(hd)
        for s in range(nseq):
            for h in range(Hq):
                kh = h // (Hq // Hkv)
                P, _ = self._probs(Q[s, :, h], K[s, :, kh], T, window)
                dV[s, :, kh] += P.T @ dO[s, :, h]
                dP = dO[s, :, h] @ V[s, :, kh].T
                dS = P * (dP - (dP * P).sum(axis=1, keepdims=True)) * scale
                dQ[s, :, h] = dS @ K[s, :, kh]
                dK[s, :, kh] += dS.T @ Q[s, :, h]
        return dQ.reshape(rows, Hq * hd), dK.reshape(rows, Hkv * hd), dV.reshape(rows, Hkv * hd)

    def gt_attention_bwd(self, ctx, rows, Hq, Hkv, hd, window, q, k, v, out, lse, gout, gq, aq, gk, ak, gv, av):
        dQ, dK, dV = self._attention_grads(rows, Hq, Hkv, hd, window, q, k, v, gout)
        for addr, val, acc in ((gq, dQ, aq), (gk, dK, ak), (gv, dV, av)):
            if addr:
                self._store(addr, val, acc)
        return self._called("gt_attention_bwd", rows=rows, gq=int(gq), aq=aq, gk=int(gk), ak=ak, gv=int(gv), av=av)

    def gt_attention_bwd_rope(self, ctx, rows, Hq, Hkv, hd, window, q, k, v, out, lse, gout, gq, aq, gk, ak, gv, av, base, pos_offset):
        dQ, dK, dV = self._attention_grads(rows, Hq, Hkv, hd, window, q, k, v, gout)
        if gq:
            self._store(gq, self._rotate(dQ, rows, Hq, hd, base, pos_offset, True), aq)
        if gk:
            self._store(gk, self._rotate(dK, rows, Hkv, hd, base, pos_offset, True), ak)
        if gv:
            self._store(gv, dV, av)
        return self._called("gt_attention_bwd_rope", rows=rows, gq=int(gq), aq=aq, gk=int(gk), ak=ak, gv=int(gv), av=av)

    # ------------------------------------------------------------------ cross entropy over [rows, V] logits
    def gt_ce_fwd(self, ctx, rows, V, logits, targets, stats, loss, inv_kept):
        T, nseq = self._seq(rows)
        Z = self.f32(logits, rows, V).astype(np.float64)
        tg = self._view(targets, rows, np.uint32)
        m = Z.max(axis=1)
        ssum = np.exp(Z - m[:, None]).sum(axis=1)
        kept = tg != IGNORE
        safe = np.where(kept, tg, 0).astype(np.int64)
        rl = np.where(kept, np.log(ssum) + m - Z[np.arange(rows), safe], 0.0)
        st = self.f32(stats, rows, 4)
        st[:, 0], st[:, 1], st[:, 2], st[:, 3] = m, 1.0 / ssum, rl, 0.0
        L, ik = self.f32(loss, 1 + nseq), self.f32(inv_kept, nseq)
        total = 0.0
        for s in range(nseq):
            rows_s = slice(s * T, (s + 1) * T)
            c = int(kept[rows_s].sum())
            denom = float(c) if c > 0 else 1.0
            L[1 + s] = rl[rows_s][kept[rows_s]].sum() / denom
            ik[s] = 1.0 / denom
            total += float(L[1 + s])
        L[0] = total / nseq
        return self._called("gt_ce_fwd", rows=rows, V=V)

    def gt_ce_bwd(self, ctx, rows, V, logits, targets, stats, inv_kept, gloss, glogits, accum):
        if not glogits:
            return 0
        T, nseq = self._seq(rows)
        Z = self.f32(logits, rows, V).astype(np.float64)
        tg = self._view(targets, rows, np.uint32)
        st = self.f32(stats, rows, 4).astype(np.float64)
        sc = float(self.f32(gloss, 1)[0]) * self.f32(inv_kept, nseq).astype(np.float64)[np.arange(rows) // T] / nseq
        P = np.exp(Z - st[:, 0:1]) * st[:, 1:2]
        kept = tg != IGNORE
        P[np.arange(rows)[kept], tg[kept].astype(np.int64)] -= 1.0
        G = np.where(kept[:, None], sc[:, None] * P, 0.0)
        self._store(glogits, G, accum)
        return self._called("gt_ce_bwd", rows=rows, V=V, accum=accum)

    # ------------------------------------------------------------------ the same loss over vocabulary spans (chunked readout)
    def gt_ce_chunk_stats(self, ctx, rows, n, v0, first, chunk, targets, run):
        Z = self.f32(chunk, rows, n).astype(np.float64)
        tg = self._view(targets, rows, np.uint32).astype(np.int64)
        R = self.f32(run, rows, 3)
        m_c = Z.max(axis=1)
        if first:
            m_prev, s_prev = np.full(rows, -np.inf), np.zeros(rows)
        else:
            m_prev, s_prev = R[:, 0].astype(np.float64), R[:, 1].astype(np.float64)
        m_new = np.maximum(m_prev, m_c)
        s_new = s_prev * np.exp(m_prev - m_new) + np.exp(Z - m_new[:, None]).sum(axis=1)
        inside = (tg >= v0) & (tg < v0 + n)
        R[:, 0], R[:, 1] = m_new, s_new
        R[inside, 2] = Z[np.arange(rows)[inside], tg[inside] - v0]
        return self._called("gt_ce_chunk_stats", rows=rows, n=n, v0=v0, first=first)

    def gt_ce_loss_from_stats(self, ctx, rows, run, targets, loss, inv_kept):
        T, nseq = self._seq(rows)
        R = self.f32(run, rows, 3).astype(np.float64)
        kept = self._view(targets, rows, np.uint32) != IGNORE
        rl = np.where(kept, np.log(R[:, 1]) + R[:, 0] - np.where(kept, R[:, 2], 0.0), 0.0)
        L, ik = self.f32(loss, 1 + nseq), self.f32(inv_kept, nseq)
        total = 0.0
        for s in range(nseq):
            rows_s = slice(s * T, (s + 1) * T)
            c = int(kept[rows_s].sum())
            denom = float(c) if c > 0 else 1.0
            L[1 + s] = rl[rows_s][kept[rows_s]].sum() / denom
            ik[s] = 1.0 / denom
            total += float(L[1 + s])
        L[0] = total / nseq
        return self._called("gt_ce_loss_from_stats", rows=rows)

    def gt_ce_chunk_grad(self, ctx, rows, n, v0, chunk, targets, run, inv_kept, gloss):
        T, nseq = self._seq(rows)
        Zv = self.f32(chunk, rows, n)
        Z = Zv.astype(np.float64)
        tg = self._view(targets, rows, np.uint32)
        R = self.f32(run, rows, 3).astype(np.float64)
        sc = float(self.f32(gloss, 1)[0]) * self.f32(inv_kept, nseq).astype(np.float64)[np.arange(rows) // T] / nseq
        P = np.exp(Z - R[:, 0:1]) / R[:, 1:2]
        kept = tg != IGNORE
        inside = kept & (tg >= v0) & (tg.astype(np.int64) < v0 + n)
        P[np.arange(rows)[inside], tg[inside].astype(np.int64) - v0] -= 1.0
        Zv[...] = np.where(kept[:, None], sc[:, None] * P, 0.0).astype(np.float32)      # in place, as the library does
        return self._called("gt_ce_chunk_grad", rows=rows, n=n, v0=v0)

    # ------------------------------------------------------------------ AdamW over a group of tensors, global-norm clip
    def gt_adamw_create(self, ctx, n, data, grad, sizes, lr, b1, b2, eps, wd, clip, ref):
        if not hasattr(self, "_adamw"):
            self._adamw = {}
        h = len(self._adamw) + 1
        sz = _ints(sizes, n)
        self._adamw[h] = dict(data=_ints(data, n), grad=_ints(grad, n), sizes=sz, lr=float(lr), b1=float(b1), b2=float(b2),
                              eps=float(eps), wd=float(wd), clip=float(clip), t=0,
                              m=[self._new(4 * k, zero=True) for k in sz], v=[self._new(4 * k, zero=True) for k in sz])
        ref._obj.value = h
        return 0

    def gt_adamw_set_lr(self, ctx, h, lr):
        self._adamw[int(h)]["lr"] = float(lr)
        return 0

    def gt_adamw_state(self, ctx, h, i, mref, vref):
        a = self._adamw[int(h)]
        mref._obj.value, vref._obj.value = a["m"][i], a["v"][i]
        return 0

    def gt_adamw_get_t(self, ctx, h, ref):
        ref._obj.value = self._adamw[int(h)]["t"]
        return 0

    def gt_adamw_set_t(self, ctx, h, t):
        self._adamw[int(h)]["t"] = int(t)
        return 0

    def gt_adamw_step(self, ctx, h):
        a = self._adamw[int(h)]
        a["t"] += 1
        scale = 1.0
        if a["clip"] > 0:
            norm = math.sqrt(sum(float((self.f32(g, k).astype(np.float64) ** 2).sum()) for g, k in zip(a["grad"], a["sizes"])))
            if norm > a["clip"]:
                scale = a["clip"] / (norm + 1e-12)
        bc1, bc2 = 1.0 - a["b1"] ** a["t"], 1.0 - a["b2"] ** a["t"]
        for w, g, m, v, k in zip(a["data"], a["grad"], a["m"], a["v"], a["sizes"]):
            G = self.f32(g, k).astype(np.float64) * scale
            M = a["b1"] * self.f32(m, k).astype(np.float64) + (1.0 - a["b1"]) * G
            V = a["b2"] * self.f32(v, k).astype(np.float64) + (1.0 - a["b2"]) * G * G
            W = self.f32(w, k).astype(np.float64)
            u = (M / bc1) / (np.sqrt(V / bc2) + a["eps"])
            if a["wd"] > 0:
                u = u + a["wd"] * W
            self._store(m, M)
            self._store(v, V)
            self._store(w, W - a["lr"] * u)
        return self._called("gt_adamw_step", h=int(h), t=a["t"])

    # ------------------------------------------------------------------ Muon: momentum, five quintic Newton-Schulz steps, apply
    @staticmethod
    def _newton_schulz(G, steps):
        X = G / (np.sqrt((G * G).sum()) + 1e-7)
        flip = X.shape[0] > X.shape[1]
        if flip:
            X = X.T
        for _ in range(steps):
            A = X @ X.T
            X = 3.4445 * X + (-4.7750 * A + 2.0315 * (A @ A)) @ X
        return X.T if flip else X

    def gt_newton_schulz(self, ctx, m, n, steps, g, out):
        self._store(out, self._newton_schulz(self.f32(g, m, n).astype(np.float64), steps))
        return self._called("gt_newton_schulz", m=m, n=n, steps=steps)

    def gt_muon_create(self, ctx, n, data, grad, rows, cols, lr, momentum, nesterov, ns_steps, ref):
        if not hasattr(self, "_muon"):
            self._muon = {}
        h = len(self._muon) + 1
        r, c = _ints(rows, n), _ints(cols, n)
        self._muon[h] = dict(data=_ints(data, n), grad=_ints(grad, n), rows=r, cols=c, lr=float(lr), mu=float(momentum),
                             nesterov=int(nesterov), ns=int(ns_steps), buf=[self._new(4 * a * b, zero=True) for a, b in zip(r, c)])
        ref._obj.value = h
        return 0

    def gt_muon_set_lr(self, ctx, h, lr):
        self._muon[int(h)]["lr"] = float(lr)
        return 0

    def gt_muon_state(self, ctx, h, i, ref):
        ref._obj.value = self._muon[int(h)]["buf"][i]
        return 0

    def gt_muon_set_sharded(self, ctx, h, on):
        return 0

    def gt_muon_step(self, ctx, h):
        m = self._muon[int(h)]
        for w, g, b, r, c in zip(m["data"], m["grad"], m["buf"], m["rows"], m["cols"]):
            G = self.f32(g, r, c).astype(np.float64)
            B = m["mu"] * self.f32(b, r, c).astype(np.float64) + G
            self._store(b, B)
            B = self.f32(b, r, c).astype(np.float64)
            U = G + m["mu"] * B if m["nesterov"] else B
            X = self._newton_schulz(U.astype(np.float32).astype(np.float64), m["ns"])
            self._store(w, self.f32(w, r, c).astype(np.float64) - m["lr"] * math.sqrt(max(1.0, r / c)) * X)
        return self._called("gt_muon_step", h=int(h))

    # ------------------------------------------------------------------ token windows gathered from a resident corpus
    def gt_tokens_max(self, ctx, tokens, bpt, count, ref):
        dt = np.uint16 if int(bpt) == 2 else np.uint32
        ref._obj.value = int(self._view(tokens, count, dt).max()) if count else 0
        return self._called("gt_tokens_max", count=int(count))

    def gt_gather_windows(self, ctx, tokens, mask, bpt, count, starts, B, T, ids, targets):
        dt = np.uint16 if int(bpt) == 2 else np.uint32
        tok = self._view(tokens, count, dt).astype(np.uint32)
        msk = self._view(mask, count, dt) if mask else None
        st = self._view(starts, B, np.uint64).astype(np.int64)
        I, G = self._view(ids, B * T, np.uint32).reshape(B, T), self._view(targets, B * T, np.uint32).reshape(B, T)
        for b in range(B):
            s = int(st[b])
            assert 0 <= s and s + T + 1 <= int(count), "window start past corpus length"
            I[b] = tok[s:s + T]
            G[b] = tok[s + 1:s + 1 + T]
            if msk is not None:
                G[b][msk[s + 1:s + 1 + T] == 0] = IGNORE
        return self._called("gt_gather_windows", B=int(B), T=int(T))

    # ------------------------------------------------------------------ gradient exchange, as seen by ONE rank
    # A single process cannot hold the other ranks; the stand-in plays a world whose ranks all hold the same numbers:
    # the sum over `world` ranks is then `world` times this rank's buffer (exact in f32 for a power of two).
    def gt_dp_unique_id(self, buf):
        for i in range(128):
            buf[i] = i
        return 0

    def gt_dp_init(self, ctx, rank, world, buf):
        self.dp_world = int(world)
        return 0

    def gt_dp_allreduce_start(self, ctx, addr, n):
        v = self.f32(addr, int(n))
        v[...] = (v.astype(np.float64) * self.dp_world).astype(np.float32)
        self.log.append(("gt_dp_allreduce_start", dict(addr=int(addr), n=int(n))))
        return 0

    def gt_dp_wait(self, ctx):
        self.log.append(("gt_dp_wait", {}))
        return 0

    def gt_dp_wait_host(self, ctx, timeout_ms):
        return 0

    def gt_dp_reserve_sms(self, ctx, n):
        return 0

    def gt_dp_destroy(self, ctx):
        return 0


def install(monkeypatch):
    """Make `CudaBackend()` come up on a fresh FakeLib; returns it."""
    from gguf_trainer_b200 import _lib
    fake = FakeLib()
    monkeypatch.setattr(_lib, "load", lambda: fake)
    return fake
