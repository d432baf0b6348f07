"""`CudaBackend`: the device backend behind the op interface, standing in for `WebGPUBackend`
(src/backend/webgpu.ts). Same public surface: `install/uninstall`, the 14 ops of `OpsBackend`, the
`RegionBackend` trio, `uploadParams`, `sync`, `reclaimStepTransients`, `residentBytes`, the raw-buffer
calls the optimizers and checkpoints use, and the introspection fields its tests read. Every method
is a thin enqueue through the C ABI of libgguftrain_cuda.so; nothing here computes.

Differences that are deliberate:
 * Gradient buffers are not cleared and then `+=`-ed into. Each entry tracks whether its gradient
   has been written in the current graph; the first writer overwrites, later ones accumulate. The
   values are the ones a cleared buffer plus `+=` would hold, without the clear's memory traffic.
   `gradClearsIssued` counts only the clears that still happen (a gradient that is read before
   anything was written to it, the scatter-add target of the embedding).
 * Work can be captured once into a CUDA graph and replayed (`beginCapture/endCapture`), which is
   what removes the per-op host cost the reference is bound by.
 * `setBatch(B, T)` lets one call carry B sequences as [B*T] rows.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _lib
from . import autograd as ag
from .autograd import Tensor

_EW = {"add": 0, "mul": 1, "silu": 2, "gelu": 3, "scale": 4}
_KIND = {"NT": 0, "NN": 1, "TN": 2}
PRECISION = {"fp32": 0, "tf32": 1}   # (the C ABI reserves 2 for BF16 and refuses it: there are no BF16 kernels)


class _Entry:
    __slots__ = ("data", "grad", "bytes", "external", "gradLive", "size", "pendingDx", "copyFrom", "pendingDw", "pendingFwd",
                 "lazy", "ropeOf", "ropeFused")

    def __init__(self, data: int, grad: int, nbytes: int, external: bool, size: int):
        self.data = data
        self.grad = grad          # 0 for a frozen external (webgpu.ts frozenGradStub)
        self.bytes = nbytes
        self.external = external
        self.gradLive = False     # has anything been written to grad in the current graph?
        self.size = size
        self.pendingDx = None     # (rows, cols, [(dY address, W address, K)]): input-gradient products not launched yet
        self.copyFrom = 0         # address whose contents are this gradient's value so far (a copy not made yet)
        self.pendingDw = False    # a weight-gradient product into this gradient is noted in _pendingDw, not launched yet
        self.pendingFwd = False   # the projection that produces this tensor is noted in _pendingFwd, not launched yet
        self.lazy = None          # a launch that fills `data`: set on a projection (or per-head norm) whose only reader took it
                                  # rotated, so that it was never written; run if someone else asks for it (_materializeLazy)
        self.ropeOf = None        # for a rotary embedding's output: (input tensor, its entry, H, hd, base, posOffset)
        self.ropeFused = False    # its gradient went straight to the rotation's input (attention backward applied it)


class CapturedGraph:
    """One recorded stretch of device work, replayable with new integer inputs."""

    def __init__(self, gpu: "CudaBackend", handle: int, inputs, owned, outputs, earlier=()):
        self.gpu = gpu
        self.handle = handle
        self.handles = list(earlier) + [handle]   # segments in order when the recording was cut (cutCapture)
        self.inputs = inputs      # [(addr, count, role, bound)] in upload order
        self.owned = owned        # [(addr, size)] transients pinned to this graph
        self.outputs = outputs    # {name: (addr, count)}

    def writeInputs(self, inputs: Sequence[np.ndarray]):
        """Validate and upload the integer inputs of the next replay. The recorded kernels index the embedding table
        and the logits with these values and have no bound of their own, so the checks the eager ops run above the
        dispatch (assertIdsInTable, keptRowsInVocab: src/model/autograd.ts:813-823, 875-894) run here too."""
        if len(inputs) != len(self.inputs):
            raise ValueError(f"graph takes {len(self.inputs)} integer inputs, got {len(inputs)}")
        g = self.gpu
        staged = []
        for (addr, count, role, bound), arr in zip(self.inputs, inputs):
            if np.asarray(arr).size != count:
                raise ValueError(f"graph input has {np.asarray(arr).size} elements, recorded {count}")
            _checkIntegerInput(arr, role, bound)
            staged.append((addr, _as_u32(arr)))
        for addr, a in staged:
            g._check(g.lib.gt_write(g.ctx, addr, a.ctypes.data, a.nbytes))

    def launch(self, inputs: Sequence[np.ndarray]):
        self.writeInputs(inputs)
        self.replay()

    def replay(self, between=None):
        """Launch the recorded segments in order with the inputs already in place. `between[i]` (if given) is called
        after segment i has been enqueued: host-issued work that cannot be recorded, e.g. a collective."""
        g = self.gpu
        for i, h in enumerate(self.handles):
            g._check(g.lib.gt_graph_launch(g.ctx, h))
            if between is not None and i < len(between) and between[i] is not None:
                between[i]()

    def destroy(self):
        g = self.gpu
        for h in self.handles:
            g._check(g.lib.gt_graph_destroy(g.ctx, h))
        for addr, _size in self.owned:
            g._check(g.lib.gt_free(g.ctx, addr))
        self.owned = []


def _checkIntegerInput(values, role: str, bound: int):
    """The range check of one replayed integer input: `ids` index a table of `bound` rows; `targets` are -1 or a
    vocabulary row; `teacher` ids are vocabulary rows except for a -1 in a row's first slot (checked per element here
    as -1 or a row, the eager op checks the slot rule)."""
    if role is None:
        return
    a = np.asarray(values)
    if a.dtype == np.uint32:
        a = a.astype(np.int64)
        a[a == 0xFFFFFFFF] = -1
    if role == "ids":
        ag.assertIdsInTable(a, bound, "embedding (replay)")
    else:
        bad = np.nonzero((a < -1) | (a >= bound))[0]
        if bad.size:
            t = int(bad[0])
            raise ValueError(f"{role} (replay): value {int(a[t])} at position {t} is not -1 (ignore) or an integer in [0,{bound})")


def _as_u32(values) -> np.ndarray:
    """-1 uploads as 0xffffffff, the marker the kernels test for (webgpu.ts:1636-1646)."""
    a = np.asarray(values)
    if a.dtype != np.uint32:
        a = a.astype(np.int64).astype(np.uint32) if a.dtype.kind != "u" else a.astype(np.uint32)
    return np.ascontiguousarray(a)


class _ProfilingLib:
    """Stand-in for the library handle while a profile is open: every enqueueing call is bracketed by two
    events on the library's stream and attributed to its entry point (and, for products, its layout and
    shape), the per-label GPU time the reference collects with timestamp queries (webgpu.ts:817-880)."""

    _SKIP = ("gt_event_", "gt_read", "gt_write", "gt_sync", "gt_alloc", "gt_free", "gt_stats", "gt_last_error",
             "gt_graph_", "gt_set_", "gt_device_name", "gt_adamw_state", "gt_muon_state", "gt_adamw_get_t",
             "gt_adamw_set_", "gt_muon_set_", "gt_adamw_create", "gt_muon_create", "gt_dp_")

    def __init__(self, lib, ctx, totals):
        self._lib, self._ctx, self._totals = lib, ctx, totals

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if name.startswith(self._SKIP):
            return fn
        lib, ctx, totals = self._lib, self._ctx, self._totals

        def timed(*args):
            lib.gt_event_record(ctx, 62)
            st = fn(*args)
            lib.gt_event_record(ctx, 63)
            ms = C.c_float()
            lib.gt_event_elapsed_ms(ctx, 62, 63, C.byref(ms))
            label = name
            if name == "gt_gemm":
                label = f"gt_gemm {('NT', 'NN', 'TN')[args[1]]} {args[3]}x{args[4]}x{args[5]}"
            t = totals.setdefault(label, [0.0, 0])
            t[0] += float(ms.value)
            t[1] += 1
            return st

        return timed


class CudaBackend:
    def __init__(self, device: int = 0, precision: str = "fp32"):
        self.lib = _lib.load()
        ctx = C.c_void_p()
        st = self.lib.gt_init(device, C.byref(ctx))
        if st != 0:
            raise _lib.GtError(st, self.lib.gt_last_error(None).decode())
        self.ctx = ctx
        self.device = device
        name = C.create_string_buffer(256)
        self._check(self.lib.gt_device_name(self.ctx, name, 256))
        self.adapterName = name.value.decode()
        self.timestampSupported = True
        self.lastSyncReadbackBytes = 0
        self.gradClearsIssued = 0
        self.precision = precision
        self._check(self.lib.gt_set_precision(self.ctx, PRECISION[precision]))
        self._entries: "weakref.WeakKeyDictionary[Tensor, _Entry]" = weakref.WeakKeyDictionary()
        self._touched: Dict[int, Tensor] = {}
        self._keptOnDevice: "weakref.WeakSet[Tensor]" = weakref.WeakSet()
        self._transients: List[tuple] = []     # (addr, size)
        self._regionFree: List[tuple] = []
        self._regionsOpened = 0
        # Attention outputs kept across a recompute region (see regionToken / replayOf)
        self.keepAttentionAcrossRecompute = True
        self._regionDepth = 0
        self._curRec: Optional[dict] = None
        self._regionRecs: Dict[int, dict] = {}
        self._nextRegionId = 1
        self._backwardBegun = False
        self._graphSynced = False              # a sync() ran after the current graph was built
        self._graphOpen = False                # forward ops were recorded since the last sync()
        self._capturing = False
        self._captureInputs: List[tuple] = []
        self._captureSegments: List[int] = []
        self._captureMark = 0
        self._batch = (0, 0)
        self._stateBufs: Dict[int, int] = {}
        self._readback = 0
        self._seedBuf = 0
        self._pendingAct = {}   # id(tensor) -> (tensor, op code, input tensor): activations not launched yet
        self._pendingDx: Dict[int, _Entry] = {}   # entries whose gradient still lacks deferred dY.W products
        self.mergeInputGradients = True
        self._pendingFwd: List[dict] = []   # projections of one input not launched yet (see _deferLinear)
        self.groupForward = True
        self._pendingDw: List[tuple] = []   # weight-gradient products not launched yet (see _deferDw)
        self._pendingDwRows = 0
        self.groupWeightGradients = True
        self._pendingAdd = {}   # id(tensor) -> (tensor, a, b): residual adds not launched yet (see add)
        self._pendingCopy: Dict[int, _Entry] = {}  # entries whose gradient is still a view of another buffer (see add)
        self.fuseResidualNorm = True
        self.fuseGatedUnits = True
        self.fuseRope = True               # rotary embeddings applied by the launches before and after them (see rope, attention)
        self.fuseLora = True               # adapter-carrying projections as one op (loraLinear) instead of four
        self._finalizer = weakref.finalize(self, _destroy_ctx, self.lib, self.ctx)

    # ------------------------------------------------------------------ plumbing
    def _check(self, status: int):
        if status != 0:
            raise _lib.GtError(status, self.lib.gt_last_error(self.ctx).decode())

    def describeDevice(self) -> str:
        return self.adapterName

    def startProfile(self):
        """webgpu.ts:817-845. Per-label GPU time until stopProfile(); each call is synchronised, so use it to
        see where time goes, not to measure throughput."""
        if getattr(self, "_profTotals", None) is not None:
            return
        self._profTotals = {}
        self._realLib = self.lib
        self.lib = _ProfilingLib(self._realLib, self.ctx, self._profTotals)

    def stopProfile(self):
        """Returns {label: {"ms": total, "count": n}} and closes the profile (webgpu.ts:847-880)."""
        totals = getattr(self, "_profTotals", None)
        if totals is None:
            return {}
        self.lib = self._realLib
        self._profTotals = None
        return {k: {"ms": v[0], "count": v[1]} for k, v in totals.items()}

    def install(self):
        ag.setOpsBackend(self)

    def uninstall(self):
        ag.setOpsBackend(None)

    def destroy(self):
        """webgpu.ts:764-767."""
        if ag.opsBackend() is self:
            self.uninstall()
        if self._finalizer.alive:
            self._finalizer()
        self.ctx = None

    def setPrecision(self, precision: str):
        self._check(self.lib.gt_set_precision(self.ctx, PRECISION[precision]))
        self.precision = precision

    def setBatch(self, batch: int, seq_len: int = 0):
        """Rows passed to the ops are `batch` sequences of `seq_len` rows; 0 restores one sequence per call."""
        self._check(self.lib.gt_set_batch(self.ctx, batch, seq_len))
        self._batch = (batch, seq_len if batch else 0)

    def stats(self):
        out = (C.c_uint64 * 4)()
        self._check(self.lib.gt_stats(self.ctx, out))
        return {"pool": int(out[0]), "state": int(out[1]), "readback": int(out[2]), "launches": int(out[3])}

    def residentBytes(self):
        """webgpu.ts:774-777."""
        s = self.stats()
        return {"pool": s["pool"], "state": s["state"], "total": s["pool"] + s["state"]}

    def kernelLaunches(self) -> int:
        return self.stats()["launches"]

    # ------------------------------------------------------------------ memory
    def _alloc(self, nbytes: int) -> tuple:
        out = C.c_uint64()
        self._check(self.lib.gt_alloc(self.ctx, max(nbytes, 4), C.byref(out)))
        size = max(256, (max(nbytes, 4) + 255) // 256 * 256)
        return int(out.value), size

    def _acquirePersistent(self, nbytes: int) -> int:
        return self._alloc(nbytes)[0]

    def _acquireTransient(self, nbytes: int) -> int:
        addr, size = self._alloc(nbytes)
        self._transients.append((addr, size))
        return addr

    def _acquireRecycled(self, nbytes: int) -> int:
        """Best fit from the region free-list, else a fresh transient (webgpu.ts acquireRecycled)."""
        want = max(256, (max(nbytes, 4) + 255) // 256 * 256)
        best = -1
        for i, (_a, size) in enumerate(self._regionFree):
            if size >= want and (best < 0 or size < self._regionFree[best][1]):
                best = i
        if best < 0:
            return self._acquireTransient(nbytes)
        tr = self._regionFree.pop(best)
        self._transients.append(tr)
        return tr[0]

    def _write(self, addr: int, arr: np.ndarray):
        arr = np.ascontiguousarray(arr)
        self._check(self.lib.gt_write(self.ctx, addr, arr.ctypes.data, arr.nbytes))

    def _read(self, addr: int, out: np.ndarray):
        assert out.flags["C_CONTIGUOUS"]
        if not self._capturing:
            self._flushAllDx("keep")    # whatever is read must not be missing a launch that was put off
        self._check(self.lib.gt_read(self.ctx, addr, out.ctypes.data, out.nbytes))
        self._readback += out.nbytes

    def _uploadU32(self, values, role: Optional[str] = None, bound: int = 0) -> int:
        if hasattr(values, "addr") and hasattr(values, "bound"):
            return int(values.addr)          # already on the device (ingest.DeviceInts): nothing to upload or replay-patch
        a = _as_u32(values)
        if self._capturing:
            # a replayed graph reads its integer inputs from fixed buffers the launcher rewrites; `role` and `bound`
            # are what the launcher checks new values against
            addr = self._acquirePersistent(a.nbytes)
            self._captureInputs.append((addr, a.size, role, bound))
            return addr
        addr = self._acquireTransient(a.nbytes)
        self._write(addr, a)
        return addr

    def _uploadF32(self, values) -> int:
        a = np.ascontiguousarray(np.asarray(values, dtype=np.float32))
        if self._capturing:
            raise _lib.GtError(4, "float uploads are not replayable; this op cannot be captured")
        addr = self._acquireTransient(a.nbytes)
        self._write(addr, a)
        return addr

    def _entryFor(self, t: Tensor) -> _Entry:
        """webgpu.ts:1539-1573: externals (params, test inputs) get persistent buffers on first use."""
        e = self._entries.get(t)
        if e is None and id(t) in self._pendingAct:
            e = self._materializeAct(t)
        if e is None and id(t) in self._pendingAdd:
            e = self._materializeAdd(t)
        if e is None:
            nbytes = t.size * 4
            if self._capturing:
                raise _lib.GtError(4, "a tensor first reached the device inside a graph capture; upload it first")
            e = _Entry(self._acquirePersistent(nbytes), self._acquirePersistent(nbytes) if t.requiresGrad else 0,
                       nbytes, True, t.size)
            self._entries[t] = e
            self._write(e.data, t.data)
        if e.pendingFwd:
            self._flushFwd()
        if e.lazy is not None:
            self._materializeLazy(e)
        if e.external and id(t) not in self._touched:
            self._touched[id(t)] = t
        return e

    def _entryOf(self, t: Tensor):
        """The device entry of a tensor some op produced (launching it first if it is a deferred activation), or None."""
        e = self._entries.get(t)
        if e is None and id(t) in self._pendingAct:
            e = self._materializeAct(t)
        if e is None and id(t) in self._pendingAdd:
            e = self._materializeAdd(t)
        if e is not None and e.pendingFwd:
            self._flushFwd()
        if e is not None and e.lazy is not None:
            self._materializeLazy(e)
        return e

    def _makeOut(self, shape, prev) -> tuple:
        t = Tensor.zeros(shape)
        t._prev = list(prev)
        nbytes = t.size * 4
        e = _Entry(self._acquireRecycled(nbytes), self._acquireRecycled(nbytes), nbytes, False, t.size)
        self._entries[t] = e
        return t, e

    # The input gradient of `linear` is dX (+)= dY.W. An activation that feeds several projections (the normed input
    # of q, k and v; of gate and up) collects one such product per consumer, and the reference issues them one by one,
    # each re-reading and re-writing the [T, in] buffer (src/backend/webgpu.ts:884-903). Here a closure only notes its
    # (dY, W, K); the products are launched together, as one matrix product whose contraction runs over all the K
    # ranges (gt_gemm_multi), when the gradient is first needed: by the producer's own backward, by another writer, or
    # at a sync, a region's end or a graph cut. Same terms, added in the same order.
    def _deferDx(self, e: _Entry, rows: int, cols: int, dy: int, w: int, K: int):
        if e.pendingDx is None:
            e.pendingDx = (rows, cols, [])
            self._pendingDx[id(e)] = e
        e.pendingDx[2].append((dy, w, K))
        if len(e.pendingDx[2]) == 8 or not self.mergeInputGradients:
            self._flushDx(e)

    # `add` backward hands the upstream gradient to both inputs (src/model/autograd.ts:382-397): two copies of a
    # [T, hidden] buffer per residual connection. Here an input whose gradient has not been written yet only notes the
    # upstream address (`copyFrom`). Readers of that gradient read the upstream buffer in place, and the one writer
    # that follows in a transformer block, the norm's backward, adds its term on top of it while writing the real
    # buffer (gt_rmsnorm_bwd_add). Any other writer makes the copy, and so does every point where the upstream buffer
    # may be recycled while the entry lives on (a region's end, a reclaim). The gradient of an op's OUTPUT (the
    # projection on the other side of the residual connection) is only ever read by that op's backward, in place: where
    # gradients are handed to someone outside the ops (an optimizer, an exchange, a sync) only parameters matter, so the
    # copy into a transient's gradient is not made there (60 copies of [T, hidden] per step of a 30-layer model).
    def _materializeCopy(self, e: _Entry):
        self._check(self.lib.gt_copy(self.ctx, e.grad, e.copyFrom, e.bytes))
        e.copyFrom = 0
        e.gradLive = True
        self._pendingCopy.pop(id(e), None)

    def _flushAllCopies(self, transients: str = "copy"):
        """`transients`: what to do with notes on gradients of op outputs: "copy" (make them), "keep" (leave them
        noted: nothing is being recycled) or "drop" (their entries are about to be recycled with the upstream buffers)."""
        for e in list(self._pendingCopy.values()):
            if e.external or transients == "copy":
                self._materializeCopy(e)
            elif transients == "drop":
                e.copyFrom = 0
                self._pendingCopy.pop(id(e), None)

    def _flushDx(self, e: _Entry):
        if e.copyFrom:
            self._materializeCopy(e)
        rows, cols, parts = e.pendingDx
        e.pendingDx = None
        self._pendingDx.pop(id(e), None)
        acc = 1 if e.gradLive else 0
        e.gradLive = True
        n = len(parts)
        if n == 1:
            self._gemm("NN", acc, rows, cols, parts[0][2], parts[0][0], parts[0][1], e.grad)
            return
        Ks = (C.c_int32 * n)(*[p[2] for p in parts])
        As = (C.c_uint64 * n)(*[p[0] for p in parts])
        Bs = (C.c_uint64 * n)(*[p[1] for p in parts])
        self._check(self.lib.gt_gemm_multi(self.ctx, _KIND["NN"], acc, rows, cols, n, Ks, As, Bs, e.grad))

    # Projections of the same activation (q, k and v of the normed input; gate and up) are noted when recorded and
    # launched together when the first of their outputs is needed: q/k/v as one grouped product (gt_gemm_grouped), gate and
    # up, when a gated unit consumes both, as one launch that also applies the unit (gt_glu_linear_fwd, see _gatedUnit).
    def _deferLinear(self, ex: _Entry, ew: _Entry, eo: _Entry, T: int, inDim: int, outDim: int):
        first = self._pendingFwd[0] if self._pendingFwd else None
        if first is not None and ("norm" in first or "lora" in first or first["ex"] is not ex or len(self._pendingFwd) == 8):
            self._flushFwd()
        self._pendingFwd.append(dict(ex=ex, ew=ew, eo=eo, T=T, inDim=inDim, outDim=outDim))
        eo.pendingFwd = True

    # A per-head norm (q and k of the Qwen3 and Gemma 3 blocks) waits the same way for the rotary embedding that follows
    # it: if that is its first reader, one pass normalises and rotates (gt_rmsnorm_heads_rope_fwd).
    def _deferHeadNorm(self, ex: _Entry, ew: _Entry, eo: _Entry, rinv: int, T: int, H: int, hd: int, eps: float):
        first = self._pendingFwd[0] if self._pendingFwd else None
        if first is not None and ("norm" not in first or len(self._pendingFwd) == 8):
            self._flushFwd()
        self._pendingFwd.append(dict(norm=True, ex=ex, ew=ew, eo=eo, rinv=rinv, T=T, H=H, hd=hd, eps=eps, outDim=H * hd))
        eo.pendingFwd = True

    def _flushFwd(self):
        parts = self._pendingFwd
        if not parts:
            return
        self._pendingFwd = []
        for p in parts:
            p["eo"].pendingFwd = False
        if "lora" in parts[0]:
            n = len(parts)
            p0 = parts[0]
            T, inDim, r, s = p0["T"], p0["inDim"], p0["r"], p0["s"]
            if n == 1:
                self._check(self.lib.gt_gemm_scaled(self.ctx, _KIND["NT"], 0, T, r, inDim, p0["ex"].data, p0["ea"].data, p0["ts"], s))
            else:
                Ms, Ns = (C.c_int32 * n)(*([T] * n)), (C.c_int32 * n)(*([r] * n))
                As = (C.c_uint64 * n)(*([p0["ex"].data] * n))
                Bs = (C.c_uint64 * n)(*[p["ea"].data for p in parts])
                Cs = (C.c_uint64 * n)(*[p["ts"] for p in parts])
                acc = (C.c_int32 * n)(*([0] * n))
                self._check(self.lib.gt_gemm_grouped_scaled(self.ctx, _KIND["NT"], n, Ms, Ns, inDim, As, Bs, Cs, acc, s))
            for p in parts:
                self._gemm2("NT", 0, T, p["outDim"], inDim, p["ex"].data, p["ew"].data, r, p["ts"], p["eb"].data, p["eo"].data)
            return
        if "norm" in parts[0]:
            for p in parts:
                T, H, hd = p["T"], p["H"], p["hd"]
                plain = (lambda p=p: self._check(self.lib.gt_rmsnorm_fwd(self.ctx, p["T"] * p["H"], p["hd"], p["ex"].data, p["ew"].data,
                                                                          p["eps"], p["eo"].data, p["rinv"])))
                if "rope" in p:
                    er, _H, _hd, base, posOffset = p["rope"]
                    er.pendingFwd = False
                    self._check(self.lib.gt_rmsnorm_heads_rope_fwd(self.ctx, T, H, hd, p["ex"].data, p["ew"].data, p["eps"], er.data,
                                                                   p["rinv"], float(base), posOffset))
                    p["eo"].lazy = plain        # (the same row statistics are written again if it ever runs)
                else:
                    plain()
            return
        n = len(parts)
        T, inDim = parts[0]["T"], parts[0]["inDim"]
        roped = [p for p in parts if "rope" in p]
        if roped:
            # projections whose one reader so far is a rotary embedding: the launch writes the rotated values into the
            # embedding's output; the projection's own buffer stays unwritten unless someone else asks for it
            _er, _H, hd, base, posOffset = roped[0]["rope"]
            for p in roped:
                p["rope"][0].pendingFwd = False
                p["eo"].lazy = (lambda p=p: self._gemm("NT", 0, p["T"], p["outDim"], p["inDim"], p["ex"].data, p["ew"].data, p["eo"].data))
            Ns = (C.c_int32 * n)(*[p["outDim"] for p in parts])
            Ws = (C.c_uint64 * n)(*[p["ew"].data for p in parts])
            Ys = (C.c_uint64 * n)(*[(p["rope"][0].data if "rope" in p else p["eo"].data) for p in parts])
            Hs = (C.c_int32 * n)(*[(p["rope"][1] if "rope" in p else 0) for p in parts])
            self._check(self.lib.gt_linear_rope_grouped(self.ctx, n, T, inDim, parts[0]["ex"].data, Ns, Ws, Ys, Hs, hd, float(base), posOffset))
            return
        if n == 1:
            self._gemm("NT", 0, T, parts[0]["outDim"], inDim, parts[0]["ex"].data, parts[0]["ew"].data, parts[0]["eo"].data)
            return
        Ms = (C.c_int32 * n)(*([T] * n))
        Ns = (C.c_int32 * n)(*[p["outDim"] for p in parts])
        As = (C.c_uint64 * n)(*[p["ex"].data for p in parts])
        Bs = (C.c_uint64 * n)(*[p["ew"].data for p in parts])
        Cs = (C.c_uint64 * n)(*[p["eo"].data for p in parts])
        acc = (C.c_int32 * n)(*([0] * n))
        self._check(self.lib.gt_gemm_grouped(self.ctx, _KIND["NT"], n, Ms, Ns, inDim, As, Bs, Cs, acc))

    def _materializeLazy(self, e: _Entry):
        launch = e.lazy
        e.lazy = None
        launch()

    def _flushAllDx(self, transients: str = "copy"):
        self._flushFwd()
        for e in list(self._pendingDx.values()):
            self._flushDx(e)
        self._flushAllCopies(transients)
        self._flushDw()

    # The weight gradient of `linear` is dW (+)= dY^T.X: a small output (out x in) contracted over every row. Each has
    # too few output tiles to fill the GPU, so each is cut along K into slices, with a clear before, partial sums
    # combined in L2 and a last wave of its own. Up to eight of them (the projections of a layer) are launched together
    # as one grouped product (gt_gemm_grouped): their tiles share the SMs and one split-K factor. A closure notes its
    # (dY, X, dW); the group is launched when it is full, before anything else touches one of its gradients, and at
    # every point where buffers may be recycled or gradients are handed over (sync, region end, graph cut, optimizer).
    def _deferDw(self, ew: _Entry, gw: int, accum: int, rows: int, outDim: int, inDim: int, dy: int, x: int):
        if self._pendingDw and (self._pendingDwRows != rows or len(self._pendingDw) == 8):
            self._flushDw()
        self._pendingDwRows = rows
        self._pendingDw.append((dy, x, gw, accum, outDim, inDim, ew))
        ew.pendingDw = True

    def _flushDw(self):
        parts = self._pendingDw
        if not parts:
            return
        self._pendingDw = []
        rows = self._pendingDwRows
        for p in parts:
            p[6].pendingDw = False
        n = len(parts)
        if n == 1:
            dy, x, gw, acc, outDim, inDim, _e = parts[0]
            self._gemm("TN", acc, outDim, inDim, rows, dy, x, gw)
            return
        Ms = (C.c_int32 * n)(*[p[4] for p in parts])
        Ns = (C.c_int32 * n)(*[p[5] for p in parts])
        As = (C.c_uint64 * n)(*[p[0] for p in parts])
        Bs = (C.c_uint64 * n)(*[p[1] for p in parts])
        Cs = (C.c_uint64 * n)(*[p[2] for p in parts])
        acc = (C.c_int32 * n)(*[p[3] for p in parts])
        self._check(self.lib.gt_gemm_grouped(self.ctx, _KIND["TN"], n, Ms, Ns, rows, As, Bs, Cs, acc))

    def flushDeferred(self):
        """Launch everything whose launch was put off (merged input gradients, grouped weight gradients, copies):
        called by whoever is about to use gradients outside the ops, e.g. an optimizer step or a gradient exchange."""
        self._flushAllDx("keep")

    def _gradTarget(self, t: Tensor, e: _Entry):
        """(grad address or 0, accum flag) for a backward kernel about to write into t's gradient."""
        if e.grad == 0 or (e.external and not t.requiresGrad):
            return 0, 0
        if e.pendingDw:
            self._flushDw()             # an earlier product into this gradient goes first
        if e.copyFrom:
            self._materializeCopy(e)
        if e.pendingDx is not None:
            self._flushDx(e)
        acc = 1 if e.gradLive else 0
        e.gradLive = True
        return e.grad, acc

    def _gradSource(self, e: _Entry) -> int:
        """The upstream gradient of an op output. Never written means it is exactly zero."""
        if e.pendingDw:
            self._flushDw()
        if e.pendingDx is not None:
            self._flushDx(e)           # (a gradient that is still a view gets its copy made first: _flushDx writes into it)
        if e.copyFrom:
            return e.copyFrom          # still exactly the upstream buffer of an `add`: read it there, no copy
        if not e.gradLive:
            self._check(self.lib.gt_zero(self.ctx, e.grad, e.bytes))
            self.gradClearsIssued += 1
            e.gradLive = True
        return e.grad

    # ------------------------------------------------------------------ data movement
    def uploadParams(self, tensors: Sequence[Tensor]):
        """webgpu.ts:406-411."""
        for t in tensors:
            e = self._entryFor(t)
            self._write(e.data, t.data)

    def reserveGradArena(self, tensors: Sequence[Tensor]) -> tuple:
        """Give the listed trainable tensors gradient buffers carved, in order, from one contiguous
        block, so a data-parallel step can sum them across ranks in a few large buckets.
        Returns (address, element count, [offset per tensor])."""
        total = 0
        offs = []
        for t in tensors:
            if t in self._entries:
                raise _lib.GtError(4, "reserveGradArena must run before the tensors are first used")
            offs.append(total)
            total += (t.size + 63) // 64 * 64   # 256-byte aligned slices
        base = self.createStateBuffer(total * 4)
        for t, off in zip(tensors, offs):
            nbytes = t.size * 4
            e = _Entry(self._acquirePersistent(nbytes), base + off * 4, nbytes, True, t.size)
            self._entries[t] = e
            self._write(e.data, t.data)
        return base, total, offs

    def sync(self, reads: Sequence[Tensor] = ()):
        """webgpu.ts:419-576: flush, copy back `reads` and the gradients of every touched external that
        requires grad and is not kept on device, recycle the transients."""
        if self._capturing:
            raise _lib.GtError(4, "sync() inside a graph capture")
        self._readback = 0
        self._flushAllDx("drop")
        self._flushPendingActs(only=list(reads))
        self._pendingAct.clear()
        self._pendingAdd.clear()
        seen = set()
        for t in reads:
            if id(t) in seen:
                continue
            seen.add(id(t))
            e = self._entries.get(t)
            if e is None:
                continue
            if e.lazy is not None:
                self._materializeLazy(e)
            self._read(e.data, t.data)
        for t in list(self._touched.values()):
            e = self._entries.get(t)
            if e is None:
                continue
            if t.requiresGrad and e.grad:
                if not e.gradLive:
                    # touched by a forward, never written by a backward: the reference's cleared buffer
                    self._check(self.lib.gt_zero(self.ctx, e.grad, e.bytes))
                    self.gradClearsIssued += 1
                if t not in self._keptOnDevice:
                    self._read(e.grad, t.grad)
            e.gradLive = False   # the next graph's first writer overwrites (the deferred clear)
        self._check(self.lib.gt_sync(self.ctx))
        self.lastSyncReadbackBytes = self._readback
        for addr, _size in self._transients:
            self._check(self.lib.gt_free(self.ctx, addr))
        self._transients = []
        for addr, _size in self._regionFree:
            self._check(self.lib.gt_free(self.ctx, addr))
        self._regionFree = []
        self._touched.clear()
        self._backwardBegun = False
        if self._graphOpen:                    # (a sync with no graph behind it, e.g. after building an optimizer, arms nothing)
            self._graphSynced = True
        self._graphOpen = False
        self._regionRecs.clear()
        self._curRec = None
        self._regionDepth = 0

    def reclaimStepTransients(self, keep: Sequence[Tensor] = ()):
        """webgpu.ts:612-633: recycle this micro-batch's transients without the readback."""
        self._flushAllDx()
        keepBufs = set()
        for t in keep:
            e = self._entries.get(t)
            if e is not None:
                keepBufs.add(e.data)
        retained = []
        for tr in self._transients:
            if tr[0] in keepBufs:
                retained.append(tr)
            else:
                self._check(self.lib.gt_free(self.ctx, tr[0]))
        self._transients = retained
        for addr, _size in self._regionFree:
            self._check(self.lib.gt_free(self.ctx, addr))
        self._regionFree = []

    # ------------------------------------------------------------------ regions (RegionBackend)
    def beginRegion(self) -> int:
        self._regionsOpened += 1
        self._regionDepth += 1
        if self._regionDepth == 1 and self.keepAttentionAcrossRecompute:
            self._curRec = {"id": self._nextRegionId, "saved": [], "pos": 0, "replay": False}
            self._nextRegionId += 1
        else:
            if self._curRec is not None:             # a region inside a region: nothing is kept for either
                self._regionRecs.pop(self._curRec["id"], None)
            self._curRec = None
        return len(self._transients)

    # Optional extension of RegionBackend, used by `checkpoint` when present. A recompute region runs its forward
    # twice; the attention inside it is the one op whose second run costs real time (a quarter of a layer's forward)
    # while its result is, by construction, bit-identical to the first. So the first run's attention outputs (O and
    # the row statistics) survive the region's end, and the replay, told which region it repeats, takes them instead
    # of launching the kernel again. Everything else of the region is still freed and recomputed.
    def regionToken(self) -> Optional[int]:
        """Identity of the outermost region just opened (None when nothing will be kept for it)."""
        rec = self._curRec
        if rec is None or rec["replay"]:
            return None
        self._regionRecs[rec["id"]] = rec
        return rec["id"]

    def replayOf(self, token: Optional[int]):
        """The region just opened repeats the forward of region `token`."""
        rec = self._regionRecs.get(token) if token is not None else None
        if rec is not None and self._regionDepth == 1:
            rec["replay"], rec["pos"] = True, 0
            self._curRec = rec

    def regionCount(self) -> int:
        return self._regionsOpened

    def endRegion(self, mark: int, keep: Sequence[Tensor]):
        """webgpu.ts:659-702."""
        if mark > len(self._transients):
            raise RuntimeError(
                f"endRegion: mark {mark} is past the {len(self._transients)} live transients; "
                f"a sync() or reclaim ran inside the region")
        self._flushAllDx()
        self._flushPendingActs(only=list(keep))
        keepBufs = set()
        for t in keep:
            e = self._entries.get(t)
            if e is not None:
                keepBufs.add(e.data)
                keepBufs.add(e.grad)
        rec = self._curRec if self._regionDepth == 1 else None
        self._regionDepth = max(0, self._regionDepth - 1)
        release = set()
        if rec is not None:
            self._curRec = None
            held = {b for item in rec["saved"] for b in item[:2]}
            if rec["replay"]:
                release = held                       # the replay and its backward are over: the kept outputs go too
                self._regionRecs.pop(rec["id"], None)
            elif rec["id"] in self._regionRecs:
                keepBufs |= held                     # first run, and `checkpoint` asked for a token: keep them
        retained = []
        for tr in self._transients[:mark]:
            if tr[0] in release:
                self._regionFree.append(tr)
            else:
                retained.append(tr)
        for tr in self._transients[mark:]:
            if tr[0] in keepBufs:
                retained.append(tr)
            else:
                self._regionFree.append(tr)
        self._transients = retained

    def seedGradFrom(self, dst: Tensor, src: Tensor):
        """webgpu.ts:748-761."""
        self._ensureBackwardBegun()
        ed, es = self._entryOf(dst), self._entryOf(src)
        if ed is None or es is None:
            raise RuntimeError("seedGradFrom: tensor has no GPU buffers")
        if dst.size != src.size:
            raise RuntimeError(f"seedGradFrom: size mismatch {dst.size} vs {src.size}")
        self._check(self.lib.gt_copy(self.ctx, ed.grad, self._gradSource(es), src.size * 4))
        ed.gradLive = True

    def seedGradFromHost(self, t: Tensor):
        """webgpu.ts:1432-1437."""
        self._ensureBackwardBegun()
        e = self._entryOf(t)
        if e is None:
            raise RuntimeError("seedGradFromHost: tensor has no GPU buffers")
        self._write(e.grad, t.grad)
        e.gradLive = True

    def _beginForwardOp(self, keepPending: bool = False):
        """Every forward op starts here. Unless the op launches nothing itself (`keepPending`), projections noted but
        not launched yet go first, so no kernel can read an output that does not exist yet."""
        if self._pendingFwd and not keepPending:
            self._flushFwd()
        self._backwardBegun = False
        self._graphSynced = False
        self._graphOpen = True

    def _ensureBackwardBegun(self):
        """webgpu.ts:1397-1429. A sync() between a graph's forward and its backward recycled the graph's
        buffers; refuse to accumulate into them."""
        if self._pendingFwd:
            self._flushFwd()
        if self._backwardBegun:
            return
        if self._graphSynced:
            raise RuntimeError(
                "backward over a graph built before a sync(): that sync recycled the graph's "
                "gradient buffers and discarded their clears, so this backward would "
                "accumulate into pool garbage")
        self._backwardBegun = True

    # ------------------------------------------------------------------ raw buffers (optimizers, checkpoints)
    def buffersFor(self, t: Tensor):
        e = self._entryFor(t)
        if e.copyFrom:                  # the caller is about to look at the gradient buffer itself
            self._materializeCopy(e)
        return {"data": e.data, "grad": e.grad}

    def keepGradOnDevice(self, t: Tensor):
        self._keptOnDevice.add(t)

    def createStateBuffer(self, nbytes: int) -> int:
        out = C.c_uint64()
        self._check(self.lib.gt_alloc_state(self.ctx, nbytes, C.byref(out)))
        self._stateBufs[int(out.value)] = nbytes
        return int(out.value)

    def writeStateBuffer(self, buf: int, f32: np.ndarray):
        self._write(buf, np.ascontiguousarray(f32, dtype=np.float32))

    def readStateBuffer(self, buf: int, n: int) -> np.ndarray:
        out = np.empty(n, np.float32)
        self._read(buf, out)
        return out

    # ------------------------------------------------------------------ asynchronous reads (checkpoints)
    def readAsync(self, addr: int, nbytes: int) -> int:
        """Start copying `nbytes` at `addr`, as of the work enqueued so far, to pinned host memory on a copy stream
        that runs beside later compute. Returns a ticket for `readFinish`."""
        t = C.c_uint64()
        self._check(self.lib.gt_read_async(self.ctx, addr, nbytes, C.byref(t)))
        return int(t.value)

    def readFence(self):
        """Later compute waits (on the device) for every read started so far: call before work that overwrites their
        sources. The optimizers call it at the top of `recordStep`."""
        self._check(self.lib.gt_read_fence(self.ctx))

    def readFinish(self, ticket: int, out: np.ndarray):
        assert out.flags["C_CONTIGUOUS"]
        self._check(self.lib.gt_read_finish(self.ctx, ticket, out.ctypes.data, out.nbytes))

    # ------------------------------------------------------------------ graph capture
    def beginCapture(self, seed: float = 1.0, accumulate: bool = True):
        """Start recording device work into a replayable graph. Run the same work once eagerly first:
        recording cannot allocate (the pool, RoPE tables and scratch must already be warm).
        `seed` is the loss seed the recorded backward uses. With `accumulate` the recorded backward adds
        into the parameter gradients (replay it once per micro-batch after zeroing them); without, its
        first write to each parameter gradient overwrites (one replay per step)."""
        if self._capturing:
            raise _lib.GtError(4, "beginCapture: already capturing")
        if self._seedBuf == 0:
            self._seedBuf = self.createStateBuffer(4)
        self._write(self._seedBuf, np.array([seed], np.float32))
        for t, e in list(self._entries.items()):
            if e.external and e.grad:
                e.gradLive = bool(accumulate)
        self._check(self.lib.gt_graph_begin(self.ctx))
        self._capturing = True
        self._captureInputs = []
        self._captureSegments = []
        self._captureMark = len(self._transients)

    def cutCapture(self) -> int:
        """Close the graph recorded so far and start the next one: the place where the replayer will issue work from
        the host between two segments. Returns the number of segments closed so far."""
        if not self._capturing:
            raise _lib.GtError(4, "cutCapture: not capturing")
        self._flushAllDx("keep")
        h = C.c_uint64()
        self._check(self.lib.gt_graph_end(self.ctx, C.byref(h)))
        self._captureSegments.append(int(h.value))
        self._check(self.lib.gt_graph_begin(self.ctx))
        return len(self._captureSegments)

    def endCapture(self, outputs: Optional[Dict[str, Tensor]] = None) -> CapturedGraph:
        h = C.c_uint64()
        self._flushAllDx("drop")
        self._capturing = False
        self._check(self.lib.gt_graph_end(self.ctx, C.byref(h)))
        owned = self._transients[self._captureMark:] + self._regionFree
        self._transients = self._transients[:self._captureMark]
        self._regionFree = []
        owned = owned + [(a, n * 4) for a, n, _r, _b in self._captureInputs]
        outs = {}
        for name, t in (outputs or {}).items():
            e = self._entries[t]
            outs[name] = (e.data, t.size)
        g = CapturedGraph(self, int(h.value), list(self._captureInputs), owned, outs, earlier=self._captureSegments)
        self._captureInputs = []
        self._captureSegments = []
        # externals touched while recording keep their accumulate-or-overwrite state as recorded
        return g

    def readGraphOutput(self, g: CapturedGraph, name: str) -> np.ndarray:
        addr, n = g.outputs[name]
        out = np.empty(n, np.float32)
        self._read(addr, out)
        return out

    # ------------------------------------------------------------------ events
    def recordEvent(self, slot: int):
        self._check(self.lib.gt_event_record(self.ctx, slot))

    def elapsedMs(self, a: int, b: int) -> float:
        ms = C.c_float()
        self._check(self.lib.gt_event_elapsed_ms(self.ctx, a, b, C.byref(ms)))
        return float(ms.value)

    # ------------------------------------------------------------------ ops (OpsBackend)
    def _gemm(self, kind: str, accum: int, M: int, N: int, K: int, a: int, b: int, c: int):
        self._check(self.lib.gt_gemm(self.ctx, _KIND[kind], accum, M, N, K, a, b, c))

    def _gemm2(self, kind: str, accum: int, M: int, N: int, K: int, a: int, b: int, K2: int, a2: int, b2: int, c: int):
        self._check(self.lib.gt_gemm2(self.ctx, _KIND[kind], accum, M, N, K, a, b, K2, a2, b2, c))

    def linear(self, x: Tensor, w: Tensor) -> Tensor:
        """webgpu.ts:884-903."""
        self._beginForwardOp(keepPending=True)
        T, inDim = x.shape
        outDim = w.shape[0]
        ex, ew = self._entryFor(x), self._entryFor(w)
        out, eo = self._makeOut([T, outDim], [x, w])
        if self.groupForward:
            self._deferLinear(ex, ew, eo, T, inDim, outDim)
        else:
            self._flushFwd()
            self._gemm("NT", 0, T, outDim, inDim, ex.data, ew.data, eo.data)

        def _bw():
            self._ensureBackwardBegun()
            go = self._gradSource(eo)
            if ex.grad and not (ex.external and not x.requiresGrad):
                self._deferDx(ex, T, inDim, go, ew.data, outDim)
            if w.requiresGrad:
                gw, aw = self._gradTarget(w, ew)
                if gw:
                    # (a product with many output tiles, the readout's, fills the GPU alone and is launched as it comes)
                    if self.groupWeightGradients and ((outDim + 255) // 256) * ((inDim + 191) // 192) <= 64:
                        self._deferDw(ew, gw, aw, T, outDim, inDim, go, ex.data)
                    else:
                        self._gemm("TN", aw, outDim, inDim, T, go, ex.data, gw)

        out._backward = _bw
        return out

    def loraLinear(self, x: Tensor, w: Tensor, a: Tensor, b: Tensor, scale: float) -> Tensor:
        """The adapter-carrying projection of autograd.ts:311-319, y = x·Wᵀ + scale·((x·Aᵀ)·Bᵀ), as one op. Recorded as
        `add(linear(x,w), scale(linear(linear(x,a),b), scale))` it costs two more passes over [T, out] in forward
        (scale, add) and two in backward; here the factor is applied to the [T, r] intermediate instead and the
        low-rank product is r more columns of the wide product's contraction (`gt_gemm2`), so [T, out] is written
        once and not read back. (scale·t)·Bᵀ equals scale·(t·Bᵀ) up to rounding, exactly when scale is a power of two, e.g. the
        usual alpha/r = 2.) Gradients: dx += g·W + (scale·(g·B))·A, dB += gᵀ·(scale·t), dA += (scale·(g·B))ᵀ·x,
        and dW += gᵀ·x when the base weight is not frozen."""
        self._beginForwardOp(keepPending=self.groupForward)
        T, inDim = x.shape
        outDim, r = w.shape[0], a.shape[0]
        ex, ew, ea, eb = self._entryFor(x), self._entryFor(w), self._entryFor(a), self._entryFor(b)
        out, eo = self._makeOut([T, outDim], [x, w, a, b])
        small = T * r * 4
        ts, dt = self._acquireRecycled(small), self._acquireRecycled(small)
        s = float(scale)
        kNT, kNN = _KIND["NT"], _KIND["NN"]
        if self.groupForward:
            # noted, not launched: projections of the same input (q, k, v; gate, up) form their thin products
            # ts = scale·(x·Aᵀ) in one grouped launch, which reads x once (_flushFwd)
            first = self._pendingFwd[0] if self._pendingFwd else None
            if first is not None and ("lora" not in first or first["ex"] is not ex or first["r"] != r or first["s"] != s
                                      or len(self._pendingFwd) == 8):
                self._flushFwd()
            self._pendingFwd.append(dict(lora=True, ex=ex, ew=ew, ea=ea, eb=eb, eo=eo, ts=ts, T=T, inDim=inDim, outDim=outDim, r=r, s=s))
            eo.pendingFwd = True
        else:
            # ts = scale·(x·Aᵀ): the factor rides on the product's epilogue (gt_gemm_scaled), no pass of its own
            self._check(self.lib.gt_gemm_scaled(self.ctx, kNT, 0, T, r, inDim, ex.data, ea.data, ts, s))
            self._gemm2("NT", 0, T, outDim, inDim, ex.data, ew.data, r, ts, eb.data, eo.data)

        def _bw():
            self._ensureBackwardBegun()
            go = self._gradSource(eo)
            wantDx = bool(ex.grad) and not (ex.external and not x.requiresGrad)
            self._check(self.lib.gt_gemm_scaled(self.ctx, kNN, 0, T, r, outDim, go, eb.data, dt, s))   # dt = scale·(g·B)
            # dB = gᵀ·ts and dA = dtᵀ·x: thin outputs contracted over every row, bound by reading g and x; the fourteen of a
            # layer go out as two grouped launches (_deferDw) instead of one launch each
            if b.requiresGrad:
                gb, ab = self._gradTarget(b, eb)
                if gb:
                    if self.groupWeightGradients:
                        self._deferDw(eb, gb, ab, T, outDim, r, go, ts)
                    else:
                        self._gemm("TN", ab, outDim, r, T, go, ts, gb)
            if a.requiresGrad:
                ga, aa = self._gradTarget(a, ea)
                if ga:
                    if self.groupWeightGradients:
                        self._deferDw(ea, ga, aa, T, r, inDim, dt, ex.data)
                    else:
                        self._gemm("TN", aa, r, inDim, T, dt, ex.data, ga)
            if wantDx:      # g·W + dt·A: two more K ranges of x's input-gradient product
                self._deferDx(ex, T, inDim, go, ew.data, outDim)
                self._deferDx(ex, T, inDim, dt, ea.data, r)
            if w.requiresGrad:
                gw, aw = self._gradTarget(w, ew)
                if gw:
                    self._gemm("TN", aw, outDim, inDim, T, go, ex.data, gw)

        out._backward = _bw
        return out

    def _elementwise(self, op: str, a: Tensor, b: Optional[Tensor], c: float) -> Tensor:
        self._beginForwardOp()
        ea = self._entryFor(a)
        eb = self._entryFor(b) if b is not None else None
        out, eo = self._makeOut(a.shape, [a, b] if b is not None else [a])
        n = a.size
        code = _EW[op]
        self._check(self.lib.gt_ew_fwd(self.ctx, code, n, ea.data, eb.data if eb else 0, c, eo.data))

        def _bw():
            self._ensureBackwardBegun()
            go = self._gradSource(eo)
            if eb is not None and eb is ea:
                # add(t,t) / mul(t,t): both contributions land in one buffer, summed in one write
                ga, aa = self._gradTarget(a, ea)
                self._check(self.lib.gt_ew_bwd(self.ctx, code, n, ea.data, ea.data, c, go, ga, aa, ga, aa))
                return
            ga, aa = self._gradTarget(a, ea)
            gb, ab = self._gradTarget(b, eb) if eb is not None else (0, 0)
            self._check(self.lib.gt_ew_bwd(self.ctx, code, n, ea.data, eb.data if eb else 0, c, go, ga, aa, gb, ab))

        out._backward = _bw
        return out

    def add(self, a, b):
        """webgpu.ts:905-960. Not launched when recorded: if the first use of the sum is a norm (every residual
        connection of a block), one kernel forms the sum and normalises it (gt_add_rmsnorm_fwd); any other use
        launches the plain add then. Backward launches nothing where it can (see _materializeCopy)."""
        if a is b or not self.fuseResidualNorm or a.shape != b.shape:
            return self._elementwise("add", a, b, 0.0)
        self._beginForwardOp(keepPending=True)
        ea, eb = self._entryFor(a), self._entryFor(b)
        out = Tensor.zeros(a.shape)
        out._prev = [a, b]
        self._pendingAdd[id(out)] = (out, a, b)
        n = a.size

        def _bw():
            eo = self._entries.get(out)
            if eo is None:
                return          # never used by anything: no gradient reaches it
            self._ensureBackwardBegun()
            go = self._gradSource(eo)
            for t, e, first in ((a, ea, True), (b, eb, False)):
                if e.grad == 0 or (e.external and not t.requiresGrad):
                    continue
                if e.pendingDx is not None:
                    self._flushDx(e)
                if e.gradLive or e.copyFrom:
                    g, acc = self._gradTarget(t, e)
                    self._check(self.lib.gt_ew_bwd(self.ctx, _EW["add"], n, ea.data, eb.data, 0.0, go,
                                                   g if first else 0, acc, 0 if first else g, acc))
                else:
                    e.copyFrom = go
                    self._pendingCopy[id(e)] = e

        out._backward = _bw
        return out

    def _newEntry(self, t: Tensor) -> _Entry:
        nbytes = t.size * 4
        e = _Entry(self._acquireRecycled(nbytes), self._acquireRecycled(nbytes), nbytes, False, t.size)
        self._entries[t] = e
        return e

    def _materializeAdd(self, t: Tensor) -> _Entry:
        _t, a, b = self._pendingAdd.pop(id(t))
        ea, eb = self._entries[a], self._entries[b]
        self._flushFwd()
        e = self._newEntry(t)
        self._check(self.lib.gt_ew_fwd(self.ctx, _EW["add"], t.size, ea.data, eb.data, 0.0, e.data))
        return e

    def mul(self, a, b):
        if a is not b:
            for act, other in ((a, b), (b, a)):
                if id(act) in self._pendingAct and id(other) not in self._pendingAct:
                    return self._gatedUnit(act, other)
        return self._elementwise("mul", a, b, 0.0)

    def silu(self, x):
        return self._activation("silu", x)

    def gelu(self, x):
        return self._activation("gelu", x)

    # An activation is not launched when it is recorded: if its only use turns out to be a product (the gated FFN
    # unit silu(gate)*up / gelu(gate)*up), one fused kernel does both and the activated gate is never written. Any
    # other use (another op, a sync that reads it, the end of a recompute region) launches it then, unchanged.
    def _activation(self, op: str, x: Tensor) -> Tensor:
        if not self.fuseGatedUnits:
            return self._elementwise(op, x, None, 0.0)
        self._beginForwardOp(keepPending=True)
        e0 = self._entries.get(x)
        if e0 is None or not e0.pendingFwd:      # (a projection still waiting to be launched stays waiting: see _gatedUnit)
            self._entryFor(x)
        t = Tensor.zeros(x.shape)
        t._prev = [x]
        self._pendingAct[id(t)] = (t, _EW[op], x)

        def _bw():
            e = self._entries.get(t)
            if e is None or not (e.gradLive or e.copyFrom or e.pendingDx is not None):
                return          # consumed only by fused products, which sent their gradient straight to x
            self._ensureBackwardBegun()
            ex = self._entryOf(x)
            go = self._gradSource(e)
            gx, ax = self._gradTarget(x, ex)
            self._check(self.lib.gt_ew_bwd(self.ctx, _EW[op], x.size, ex.data, 0, 0.0, go, gx, ax, 0, 0))

        t._backward = _bw
        return t

    def _materializeAct(self, t: Tensor) -> _Entry:
        _t, code, x = self._pendingAct.pop(id(t))
        ex = self._entries[x]
        self._flushFwd()
        if ex.lazy is not None:
            self._materializeLazy(ex)
        nbytes = t.size * 4
        e = _Entry(self._acquireRecycled(nbytes), self._acquireRecycled(nbytes), nbytes, False, t.size)
        self._entries[t] = e
        self._check(self.lib.gt_ew_fwd(self.ctx, code, t.size, ex.data, 0, 0.0, e.data))
        return e

    def _flushPendingActs(self, only=None):
        for key in list(self._pendingAct.keys()):
            t = self._pendingAct[key][0]
            if only is None or any(t is o for o in only):
                self._materializeAct(t)
        for key in list(self._pendingAdd.keys()):
            t = self._pendingAdd[key][0]
            if only is None or any(t is o for o in only):
                self._materializeAdd(t)

    def _gatedUnit(self, act: Tensor, u: Tensor) -> Tensor:
        _t, code, x = self._pendingAct[id(act)]
        self._beginForwardOp(keepPending=True)
        ex, eu = self._entries[x], self._entries.get(u)
        pend = self._pendingFwd
        if (eu is not None and len(pend) == 2 and ex.pendingFwd and eu.pendingFwd and ex is not eu
                and {id(pend[0]["eo"]), id(pend[1]["eo"])} == {id(ex), id(eu)} and pend[0]["outDim"] == pend[1]["outDim"]
                and "rope" not in pend[0] and "rope" not in pend[1] and "lora" not in pend[0]):
            # gate and up are the two projections waiting to be launched: one launch writes both and the gated unit
            pg, pu = (pend[0], pend[1]) if pend[0]["eo"] is ex else (pend[1], pend[0])
            self._pendingFwd = []
            ex.pendingFwd = eu.pendingFwd = False
            out, eo = self._makeOut(act.shape, [act, u])
            self._check(self.lib.gt_glu_linear_fwd(self.ctx, code, pg["T"], pg["outDim"], pg["inDim"], pg["ex"].data, pg["ew"].data,
                                                   pu["ew"].data, ex.data, eu.data, eo.data))
        else:
            self._flushFwd()
            if ex.lazy is not None:
                self._materializeLazy(ex)
            eu = self._entryFor(u)
            out, eo = self._makeOut(act.shape, [act, u])
            self._check(self.lib.gt_glu_fwd(self.ctx, code, act.size, ex.data, eu.data, eo.data))
        n = act.size

        def _bw():
            self._ensureBackwardBegun()
            go = self._gradSource(eo)
            gx, ax = self._gradTarget(x, ex)
            gu, au = self._gradTarget(u, eu)
            if gx and gx == gu:      # act(x) * x: one buffer takes both terms, in two passes
                self._check(self.lib.gt_glu_bwd(self.ctx, code, n, ex.data, eu.data, go, gx, ax, 0, 0))
                self._check(self.lib.gt_glu_bwd(self.ctx, code, n, ex.data, eu.data, go, 0, 0, gu, 1))
            else:
                self._check(self.lib.gt_glu_bwd(self.ctx, code, n, ex.data, eu.data, go, gx, ax, gu, au))

        out._backward = _bw
        return out

    def scale(self, x, c):
        return self._elementwise("scale", x, None, float(c))

    def _rmsNormRows(self, x: Tensor, w: Tensor, rows: int, d: int, eps: float, shape, heads=None) -> Tensor:
        """webgpu.ts:1673-1701. `heads` = (T, H): a per-head norm that may wait for the rotary embedding after it."""
        self._beginForwardOp(keepPending=heads is not None)
        ew = self._entryFor(w)
        if id(x) in self._pendingAdd and x not in self._entries:
            # x = a + b has not been launched and this norm is its first use: one kernel writes both
            _t, a, b = self._pendingAdd.pop(id(x))
            ea, eb = self._entries[a], self._entries[b]
            ex = self._newEntry(x)
            out, eo = self._makeOut(shape, [x, w])
            rinv = self._acquireRecycled(rows * 4)
            self._check(self.lib.gt_add_rmsnorm_fwd(self.ctx, rows, d, ea.data, eb.data, ew.data, eps, ex.data, eo.data, rinv))
        else:
            ex = self._entryFor(x)
            out, eo = self._makeOut(shape, [x, w])
            rinv = self._acquireRecycled(rows * 4)
            if heads is not None:
                self._deferHeadNorm(ex, ew, eo, rinv, heads[0], heads[1], d, eps)
            else:
                self._check(self.lib.gt_rmsnorm_fwd(self.ctx, rows, d, ex.data, ew.data, eps, eo.data, rinv))

        def _bw():
            self._ensureBackwardBegun()
            go = self._gradSource(eo)
            wantX = bool(ex.grad) and not (ex.external and not x.requiresGrad)
            if wantX and ex.pendingDx is not None:
                self._flushDx(ex)
            gw, aw = self._gradTarget(w, ew) if w.requiresGrad else (0, 0)
            if wantX and ex.copyFrom and not ex.gradLive:
                # the gradient so far is an `add`'s upstream buffer: dx = that buffer + this term, written in one pass
                gadd = ex.copyFrom
                ex.copyFrom = 0
                self._pendingCopy.pop(id(ex), None)
                ex.gradLive = True
                self._check(self.lib.gt_rmsnorm_bwd_add(self.ctx, rows, d, ex.data, ew.data, rinv, go, gadd, ex.grad, gw, aw))
                return
            gx, ax = self._gradTarget(x, ex)
            self._check(self.lib.gt_rmsnorm_bwd(self.ctx, rows, d, ex.data, ew.data, rinv, go, gx, ax, gw, aw))

        out._backward = _bw
        return out

    def rmsNorm(self, x, weight, eps):
        T, d = x.shape
        return self._rmsNormRows(x, weight, T, d, eps, [T, d])

    def rmsNormHeads(self, x, weight, T, H, hd, eps):
        wait = self.fuseRope and hd in (64, 128, 256) and not (id(x) in self._pendingAdd and x not in self._entries)
        return self._rmsNormRows(x, weight, T * H, hd, eps, [T, H * hd], heads=(T, H) if wait else None)

    def embedding(self, weight: Tensor, ids) -> Tensor:
        """webgpu.ts:1090-1108."""
        self._beginForwardOp()
        d = weight.shape[1]
        T = len(ids)
        ew = self._entryFor(weight)
        idBuf = self._uploadU32(ids, "ids", weight.shape[0])
        out, eo = self._makeOut([T, d], [weight])
        self._check(self.lib.gt_embedding_fwd(self.ctx, T, d, ew.data, idBuf, eo.data))

        def _bw():
            self._ensureBackwardBegun()
            if not weight.requiresGrad or not ew.grad:
                return
            go = self._gradSource(eo)
            if ew.pendingDw:
                self._flushDw()
            if ew.pendingDx is not None:
                self._flushDx(ew)
            if ew.copyFrom:
                self._materializeCopy(ew)
            if not ew.gradLive:
                self._check(self.lib.gt_zero(self.ctx, ew.grad, ew.bytes))
                self.gradClearsIssued += 1
                ew.gradLive = True
            self._check(self.lib.gt_embedding_bwd(self.ctx, T, d, go, idBuf, ew.grad))

        out._backward = _bw
        return out

    def _checkT(self, T: int, rows: int, where: str):
        b, sl = self._batch
        if b and T != b * sl:
            raise ValueError(f"{where}: T={T} but the batch is {b} x {sl}")
        if not b and T != rows:
            raise ValueError(f"{where}: T={T} but the tensor has {rows} rows")

    def rope(self, x: Tensor, T: int, H: int, hd: int, base: float, posOffset: int = 0) -> Tensor:
        """webgpu.ts:1110-1123. Where the input is a projection that has not been launched yet (`rope(linear(x, Wq))`, the
        llama block) and the heads are 64 wide, the rotation is applied by the projection's launch as its tiles are
        written (gt_linear_rope_grouped); where it is a per-head norm that has not been launched yet (the Qwen3 and
        Gemma 3 blocks), by the norm's pass (gt_rmsnorm_heads_rope_fwd). No pass of its own runs in either case; the
        gradient side is in `attention`."""
        self._checkT(T, x.shape[0], "rope")
        e0 = self._entries.get(x)
        part = None
        if self.fuseRope and e0 is not None and e0.pendingFwd:
            part = next((p for p in self._pendingFwd if p["eo"] is e0), None)
            if part is not None and "norm" in part:
                # a per-head norm waiting to be launched: it normalises and rotates in one pass
                if "rope" in part or (part["T"], part["H"], part["hd"]) != (T, H, hd):
                    part = None
            elif part is not None:
                # a projection waiting to be launched (64-wide heads, tensor-core mode): its launch writes the rotated values
                first = next((p["rope"] for p in self._pendingFwd if "rope" in p), None)
                if ("rope" in part or "lora" in part or part["outDim"] != H * hd or hd != 64 or self.precision != "tf32" or T < 16 or
                        (first is not None and first[2:] != (hd, base, posOffset))):
                    part = None
        if part is not None:
            self._beginForwardOp(keepPending=True)
            ex = e0
            out, eo = self._makeOut([T, H * hd], [x])
            part["rope"] = (eo, H, hd, base, posOffset)
            eo.pendingFwd = True
        else:
            self._beginForwardOp()
            ex = self._entryFor(x)
            out, eo = self._makeOut([T, H * hd], [x])
            self._check(self.lib.gt_rope_fwd(self.ctx, T, H, hd, float(base), posOffset, ex.data, eo.data))
        eo.ropeOf = (x, ex, H, hd, base, posOffset)

        def _bw():
            self._ensureBackwardBegun()
            if eo.ropeFused and not (eo.gradLive or eo.copyFrom or eo.pendingDx is not None):
                return                       # attention's backward already delivered this gradient to x
            go = self._gradSource(eo)
            gx, ax = self._gradTarget(x, ex)
            self._check(self.lib.gt_rope_bwd(self.ctx, T, H, hd, float(base), posOffset, go, gx, ax))

        out._backward = _bw
        return out

    def attention(self, q: Tensor, k: Tensor, v: Tensor, T: int, Hq: int, Hkv: int, hd: int, window: int) -> Tensor:
        """webgpu.ts:1125-1192."""
        self._beginForwardOp()
        self._checkT(T, q.shape[0], "attention")
        eq, ek, ev = self._entryFor(q), self._entryFor(k), self._entryFor(v)
        rec = self._curRec
        nbytes = T * Hq * hd * 4
        if rec is not None and rec["replay"] and rec["pos"] < len(rec["saved"]) and rec["saved"][rec["pos"]][2] == nbytes:
            # replay of a recompute region: the first run's output and row statistics, no launch
            data, lse, _n = rec["saved"][rec["pos"]]
            rec["pos"] += 1
            out = Tensor.zeros([T, Hq * hd])
            out._prev = [q, k, v]
            eo = _Entry(data, self._acquireRecycled(nbytes), nbytes, False, out.size)
            self._entries[out] = eo
        else:
            out, eo = self._makeOut([T, Hq * hd], [q, k, v])
            lse = self._acquireRecycled(Hq * T * 4)
            self._check(self.lib.gt_attention_fwd(self.ctx, T, Hq, Hkv, hd, window, eq.data, ek.data, ev.data, eo.data, lse))
            if rec is not None and not rec["replay"]:
                rec["saved"].append((eo.data, lse, nbytes))

        def _bw():
            self._ensureBackwardBegun()
            go = self._gradSource(eo)
            rq, rk = eq.ropeOf, ek.ropeOf
            fresh = lambda e: not (e.gradLive or e.copyFrom or e.pendingDx is not None)
            if (self.fuseRope and rq is not None and rk is not None and eq is not ek and rq[3:] == rk[3:] and rq[3] == hd
                    and rq[2] == Hq and rk[2] == Hkv and hd in (64, 128) and T >= 64 and self.precision == "tf32"
                    and fresh(eq) and fresh(ek)):
                # q and k came out of rotary embeddings and nothing else has written their gradients: the kernels rotate
                # dQ and dK back as they store them, into the gradients of the embeddings' inputs
                gq, aq = self._gradTarget(rq[0], rq[1])
                gk, ak = self._gradTarget(rk[0], rk[1])
                gv, av = self._gradTarget(v, ev)
                self._check(self.lib.gt_attention_bwd_rope(self.ctx, T, Hq, Hkv, hd, window, eq.data, ek.data, ev.data, eo.data,
                                                           lse, go, gq, aq, gk, ak, gv, av, float(rq[4]), rq[5]))
                eq.ropeFused = ek.ropeFused = True
                return
            gq, aq = self._gradTarget(q, eq)
            gk, ak = self._gradTarget(k, ek)
            gv, av = self._gradTarget(v, ev)
            self._check(self.lib.gt_attention_bwd(self.ctx, T, Hq, Hkv, hd, window, eq.data, ek.data, ev.data, eo.data,
                                                  lse, go, gq, aq, gk, ak, gv, av))

        out._backward = _bw
        return out

    def _nseq(self) -> int:
        return self._batch[0] if self._batch[0] else 1

    def _lossOut(self, prev):
        """The scalar loss tensor plus its device-side companions: [1+nseq] losses and [nseq] 1/kept."""
        nseq = self._nseq()
        loss = Tensor.zeros([1])
        loss._prev = list(prev)
        e = _Entry(self._acquireRecycled((1 + nseq) * 4), self._acquireRecycled(4), 4, False, 1)
        self._entries[loss] = e
        invKept = self._acquireRecycled(nseq * 4)
        return loss, e, invKept

    def _lossGrad(self, loss: Tensor, e: _Entry) -> int:
        """backward(loss, seed) wrote the seed into the HOST grad array; push it to the device
        (webgpu.ts:1316-1320). A captured graph instead reads the seed from a fixed buffer that
        beginCapture filled, since a host write cannot be replayed."""
        if self._capturing:
            return self._seedBuf
        if not e.gradLive:
            self._write(e.grad, loss.grad[:1])
            e.gradLive = True
        return e.grad

    def crossEntropy(self, logits: Tensor, targets, kept: int) -> Tensor:
        """webgpu.ts:1295-1329. `kept` was counted above the dispatch; the device derives the same
        count from the uploaded targets, so nothing host-computed is baked into a replayable graph."""
        self._beginForwardOp()
        T, V = logits.shape
        el = self._entryFor(logits)
        tgt = self._uploadU32(targets, "targets", V)
        stats = self._acquireRecycled(T * 16)
        loss, eo, invKept = self._lossOut([logits])
        self._check(self.lib.gt_ce_fwd(self.ctx, T, V, el.data, tgt, stats, eo.data, invKept))

        def _bw():
            self._ensureBackwardBegun()
            seed = self._lossGrad(loss, eo)
            gl, al = self._gradTarget(logits, el)
            self._check(self.lib.gt_ce_bwd(self.ctx, T, V, el.data, tgt, stats, invKept, seed, gl, al))

        loss._backward = _bw
        return loss

    def fusedCrossEntropy(self, hidden: Tensor, w: Tensor, targets, chunk: int, kept: int) -> Tensor:
        """webgpu.ts:1214-1278: per vocab span, logits = hidden·W[span]ᵀ then online (max, sum, target
        logit); backward recomputes each span, forms dlogits in place and feeds the two products."""
        self._beginForwardOp()
        T, H = hidden.shape
        V = w.shape[0]
        eh, ew = self._entryFor(hidden), self._entryFor(w)
        tgt = self._uploadU32(targets, "targets", V)
        run = self._acquireRecycled(T * 12)
        width = min(chunk, V)
        ch = self._acquireRecycled(T * width * 4)
        loss, eo, invKept = self._lossOut([hidden, w])
        for v0 in range(0, V, chunk):
            n = min(chunk, V - v0)
            self._gemm("NT", 0, T, n, H, eh.data, ew.data + v0 * H * 4, ch)
            self._check(self.lib.gt_ce_chunk_stats(self.ctx, T, n, v0, 1 if v0 == 0 else 0, ch, tgt, run))
        self._check(self.lib.gt_ce_loss_from_stats(self.ctx, T, run, tgt, eo.data, invKept))

        def _bw():
            self._ensureBackwardBegun()
            seed = self._lossGrad(loss, eo)
            gh, ah = self._gradTarget(hidden, eh)
            gw, aw = self._gradTarget(w, ew) if w.requiresGrad else (0, 0)
            for v0 in range(0, V, chunk):
                n = min(chunk, V - v0)
                self._gemm("NT", 0, T, n, H, eh.data, ew.data + v0 * H * 4, ch)
                self._check(self.lib.gt_ce_chunk_grad(self.ctx, T, n, v0, ch, tgt, run, invKept, seed))
                if gh:
                    self._gemm("NN", ah, T, H, n, ch, ew.data + v0 * H * 4, gh)
                    ah = 1
                if gw:
                    # rows [v0, v0+n) of dW; each span is written by exactly one product
                    self._gemm("TN", aw, n, H, T, ch, eh.data, gw + v0 * H * 4)

        loss._backward = _bw
        return loss

    def softCrossEntropy(self, logits: Tensor, teacherIds, teacherProbs, k: int, kept: int) -> Tensor:
        """webgpu.ts:1331-1378."""
        self._beginForwardOp()
        T, V = logits.shape
        el = self._entryFor(logits)
        ids = self._uploadU32(teacherIds, "teacher", V)
        probs = self._uploadF32(teacherProbs)
        stats = self._acquireRecycled(T * 16)
        loss, eo, invKept = self._lossOut([logits])
        self._check(self.lib.gt_soft_ce_fwd(self.ctx, T, V, k, el.data, ids, probs, stats, eo.data, invKept))

        def _bw():
            self._ensureBackwardBegun()
            seed = self._lossGrad(loss, eo)
            gl, al = self._gradTarget(logits, el)
            self._check(self.lib.gt_soft_ce_bwd(self.ctx, T, V, k, el.data, ids, probs, stats, invKept, seed, gl, al))

        loss._backward = _bw
        return loss

    # ------------------------------------------------------------------ per-sequence losses of a batched call
    def sequenceLosses(self, loss: Tensor) -> np.ndarray:
        """The per-sequence losses behind a loss tensor produced under setBatch (blocks)."""
        e = self._entries[loss]
        out = np.empty(1 + self._nseq(), np.float32)
        self._read(e.data, out)
        return out[1:]


def _destroy_ctx(lib, ctx):
    try:
        lib.gt_destroy(ctx)
    except Exception:
        pass


def initCuda(device: int = 0, precision: str = "fp32") -> Optional[CudaBackend]:
    """`initWebGPU()` (webgpu.ts:1812-1870): a backend, or None when there is no GPU so suites can SKIP."""
    try:
        return CudaBackend(device, precision)
    except _lib.GtError:
        return None


def requireGPU(purpose: str, device: int = 0, precision: str = "fp32") -> CudaBackend:
    """webgpu.ts:1872-1888."""
    gpu = initCuda(device, precision)
    if gpu is None:
        raise RuntimeError(f"no GPU adapter found, and {purpose} needs one")
    return gpu
