"""Device-resident optimizers with the public methods of the reference's `AdamWGpu`
(src/backend/adamw-gpu.ts:131-251) and `MuonGpu` (src/backend/muon-gpu.ts:351-470): `setLrScale`,
`zeroGrad`, `recordStep`, `syncWeightsToHost`, `exportState`, `importState`, plus the `.optstate`
byte format (muon-gpu.ts:293-349). The WGSL-specific `prepareDispatch` plumbing is replaced by the
native `gt_adamw_step` / `gt_muon_step`.
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np

from .autograd import Tensor
from .backend import CudaBackend

OPT_MAGIC = 0x4F505431  # "OPT1"


class PendingCheckpoint:
    """Weights and optimizer state on their way to the host while training goes on (`beginCheckpoint`). The copies
    were ordered after the optimizer step that preceded the call and run on a copy stream beside the next step's
    forward and backward; that step's optimizer waits for them on the device before it overwrites anything.
    `finish()` blocks until they have landed, fills every parameter's host `data` (what `syncWeightsToHost` does) and
    returns the state dict (what `exportState` returns)."""

    def __init__(self, gpu: CudaBackend):
        self.gpu = gpu
        self._weights = []      # (tensor, ticket)
        self._state = []        # (key, ticket, size)
        self._scalars = {}
        self._lists = []        # keys that are lists even when empty

    def addWeight(self, t: Tensor):
        self._weights.append((t, self.gpu.readAsync(self.gpu.buffersFor(t)["data"], t.size * 4)))

    def addState(self, key: str, addr: int, size: int):
        self._state.append((key, self.gpu.readAsync(addr, size * 4), size))

    def finish(self):
        for t, ticket in self._weights:
            self.gpu.readFinish(ticket, t.data)
        out: Dict[str, list] = {}
        for key, ticket, size in self._state:
            a = np.empty(size, np.float32)
            self.gpu.readFinish(ticket, a)
            out.setdefault(key, []).append(a)
        for key in self._lists:
            out.setdefault(key, [])
        out.update(self._scalars)
        self._weights, self._state = [], []
        return out


class AdamWGpu:
    def __init__(self, gpu: CudaBackend, params: Sequence[Tensor], lr: float, beta1: float = 0.9, beta2: float = 0.999,
                 eps: float = 1e-8, weightDecay: float = 0.0, clip: float = 1.0):
        self.gpu = gpu
        self.params = list(params)
        self.baseLr = lr
        n = len(self.params)
        data = (C.c_uint64 * max(n, 1))()
        grad = (C.c_uint64 * max(n, 1))()
        sizes = (C.c_uint64 * max(n, 1))()
        for i, p in enumerate(self.params):
            if not p.requiresGrad:
                raise ValueError("AdamWGpu: every parameter must require grad")
            b = gpu.buffersFor(p)
            gpu.keepGradOnDevice(p)
            data[i], grad[i], sizes[i] = b["data"], b["grad"], p.size
        h = C.c_uint64()
        gpu._check(gpu.lib.gt_adamw_create(gpu.ctx, n, data, grad, sizes, lr, beta1, beta2, eps, weightDecay, clip,
                                           C.byref(h)))
        self.handle = int(h.value)

    def setLrScale(self, scale: float):
        self.gpu._check(self.gpu.lib.gt_adamw_set_lr(self.gpu.ctx, self.handle, self.baseLr * scale))

    def zeroGrad(self):
        """No-op: gradients are device-resident and restart at the next step's first write."""

    def recordStep(self):
        self.gpu.flushDeferred()  # gradient products whose launch was put off
        self.gpu.readFence()      # a checkpoint still being copied out reads the values this step overwrites
        self.gpu._check(self.gpu.lib.gt_adamw_step(self.gpu.ctx, self.handle))

    def syncWeightsToHost(self):
        self.gpu.sync(self.params)

    def beginCheckpoint(self, into: Optional[PendingCheckpoint] = None, keys=("m", "v", "t")) -> PendingCheckpoint:
        """`syncWeightsToHost` + `exportState` without stopping the device: see PendingCheckpoint."""
        ck = into or PendingCheckpoint(self.gpu)
        for i, p in enumerate(self.params):
            ck.addWeight(p)
            m, v = self._state(i)
            ck.addState(keys[0], m, p.size)
            ck.addState(keys[1], v, p.size)
        t = C.c_int32()
        self.gpu._check(self.gpu.lib.gt_adamw_get_t(self.gpu.ctx, self.handle, C.byref(t)))
        ck._scalars[keys[2]] = int(t.value)
        ck._lists.extend(keys[:2])
        return ck

    def _state(self, i):
        m, v = C.c_uint64(), C.c_uint64()
        self.gpu._check(self.gpu.lib.gt_adamw_state(self.gpu.ctx, self.handle, i, C.byref(m), C.byref(v)))
        return int(m.value), int(v.value)

    def exportState(self):
        ms, vs = [], []
        for i, p in enumerate(self.params):
            m, v = self._state(i)
            ms.append(self.gpu.readStateBuffer(m, p.size))
            vs.append(self.gpu.readStateBuffer(v, p.size))
        t = C.c_int32()
        self.gpu._check(self.gpu.lib.gt_adamw_get_t(self.gpu.ctx, self.handle, C.byref(t)))
        return {"m": ms, "v": vs, "t": int(t.value)}

    def importState(self, s):
        if len(s["m"]) != len(self.params) or len(s["v"]) != len(self.params):
            raise ValueError(f"adam moment count mismatch: {len(s['m'])} vs {len(self.params)}")
        for i, p in enumerate(self.params):
            if s["m"][i].size != p.size or s["v"][i].size != p.size:
                raise ValueError(f"adam moment {i} has {s['m'][i].size} elements, parameter has {p.size}")
            m, v = self._state(i)
            self.gpu.writeStateBuffer(m, s["m"][i])
            self.gpu.writeStateBuffer(v, s["v"][i])
        self.gpu._check(self.gpu.lib.gt_adamw_set_t(self.gpu.ctx, self.handle, int(s["t"])))


class MuonGpu:
    """Muon on the hidden matrices, AdamW on the aux group (muon-gpu.ts:351-437)."""

    def __init__(self, gpu: CudaBackend, muonParams: Sequence[Tensor], auxParams: Sequence[Tensor], lr: float,
                 momentum: float = 0.95, nesterov: bool = True, nsSteps: int = 5, aux: Optional[dict] = None,
                 shardOverRanks: bool = False):
        self.gpu = gpu
        self.muonParams = list(muonParams)
        self.auxParams = list(auxParams)
        self.baseLr = lr
        self.aux = AdamWGpu(gpu, self.auxParams, **(aux or {"lr": lr}))
        n = len(self.muonParams)
        data = (C.c_uint64 * max(n, 1))()
        grad = (C.c_uint64 * max(n, 1))()
        rows = (C.c_int32 * max(n, 1))()
        cols = (C.c_int32 * max(n, 1))()
        for i, p in enumerate(self.muonParams):
            if len(p.shape) != 2:
                raise ValueError("Muon param must be 2-D")
            b = gpu.buffersFor(p)
            gpu.keepGradOnDevice(p)
            data[i], grad[i], rows[i], cols[i] = b["data"], b["grad"], p.shape[0], p.shape[1]
        h = C.c_uint64()
        gpu._check(gpu.lib.gt_muon_create(gpu.ctx, n, data, grad, rows, cols, lr, momentum, 1 if nesterov else 0,
                                          nsSteps, C.byref(h)))
        self.handle = int(h.value)
        if shardOverRanks:
            # data parallel (gt_dp_init has run, every rank steps alike): each rank runs the Newton-Schulz iterations of
            # its share of the matrices and the results are all-gathered
            gpu._check(gpu.lib.gt_muon_set_sharded(gpu.ctx, self.handle, 1))

    def setLrScale(self, scale: float):
        self.gpu._check(self.gpu.lib.gt_muon_set_lr(self.gpu.ctx, self.handle, self.baseLr * scale))
        self.aux.setLrScale(scale)

    def zeroGrad(self):
        self.aux.zeroGrad()

    def recordStep(self):
        self.gpu.flushDeferred()
        self.gpu.readFence()
        self.gpu._check(self.gpu.lib.gt_muon_step(self.gpu.ctx, self.handle))
        self.aux.recordStep()

    def syncWeightsToHost(self):
        self.gpu.sync(self.muonParams + self.auxParams)

    def beginCheckpoint(self) -> PendingCheckpoint:
        """`syncWeightsToHost` + `exportState` (muon-gpu.ts:440-470) without stopping the device."""
        ck = PendingCheckpoint(self.gpu)
        ck._lists.append("muonMomentum")
        for i, p in enumerate(self.muonParams):
            ck.addWeight(p)
            ck.addState("muonMomentum", self._momentum(i), p.size)
        return self.aux.beginCheckpoint(ck, keys=("adamM", "adamV", "adamT"))

    def _momentum(self, i) -> int:
        b = C.c_uint64()
        self.gpu._check(self.gpu.lib.gt_muon_state(self.gpu.ctx, self.handle, i, C.byref(b)))
        return int(b.value)

    def exportState(self):
        mm = [self.gpu.readStateBuffer(self._momentum(i), p.size) for i, p in enumerate(self.muonParams)]
        a = self.aux.exportState()
        return {"muonMomentum": mm, "adamM": a["m"], "adamV": a["v"], "adamT": a["t"]}

    def importState(self, s):
        if len(s["muonMomentum"]) != len(self.muonParams):
            raise ValueError(f"muon momentum count mismatch: {len(s['muonMomentum'])} vs {len(self.muonParams)}")
        for i in range(len(self.muonParams)):
            self.gpu.writeStateBuffer(self._momentum(i), s["muonMomentum"][i])
        self.aux.importState({"m": s["adamM"], "v": s["adamV"], "t": s["adamT"]})


def serializeOptState(s) -> bytes:
    """muon-gpu.ts:293-320: u32 LE header [magic, adamT, (count, lens...) x3] then f32 data in order
    muonMomentum, adamM, adamV."""
    groups = [s["muonMomentum"], s["adamM"], s["adamV"]]
    head = [OPT_MAGIC, int(s["adamT"])]
    for g in groups:
        head.append(len(g))
        head.extend(int(a.size) for a in g)
    out = [struct.pack(f"<{len(head)}I", *head)]
    for g in groups:
        for a in g:
            out.append(np.ascontiguousarray(a, dtype="<f4").tobytes())
    return b"".join(out)


def deserializeOptState(data: bytes):
    """muon-gpu.ts:323-349."""
    o = 0
    (magic,) = struct.unpack_from("<I", data, o)
    if magic != OPT_MAGIC:
        raise ValueError("bad optstate magic")
    o += 4
    (adamT,) = struct.unpack_from("<I", data, o)
    o += 4
    lens = []
    for _ in range(3):
        (count,) = struct.unpack_from("<I", data, o)
        o += 4
        ls = list(struct.unpack_from(f"<{count}I", data, o))
        o += 4 * count
        lens.append(ls)
    f32 = np.frombuffer(data, dtype="<f4", offset=o)
    fo = 0
    groups = []
    for ls in lens:
        g = []
        for L in ls:
            g.append(f32[fo:fo + L].copy())
            fo += L
        groups.append(g)
    return {"muonMomentum": groups[0], "adamM": groups[1], "adamV": groups[2], "adamT": adamT}


def newtonSchulzGpu(gpu: CudaBackend, g: np.ndarray, m: int, n: int, steps: int) -> np.ndarray:
    """muon-gpu.ts:258-282 (test support): the device Newton-Schulz on raw row-major data."""
    g = np.ascontiguousarray(g, dtype=np.float32).reshape(-1)
    src = gpu.createStateBuffer(g.nbytes)
    dst = gpu.createStateBuffer(g.nbytes)
    gpu.writeStateBuffer(src, g)
    gpu._check(gpu.lib.gt_newton_schulz(gpu.ctx, m, n, steps, src, dst))
    out = gpu.readStateBuffer(dst, m * n)
    gpu._check(gpu.lib.gt_free(gpu.ctx, src))
    gpu._check(gpu.lib.gt_free(gpu.ctx, dst))
    return out.reshape(m, n)
