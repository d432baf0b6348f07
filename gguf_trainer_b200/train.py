"""Step loops. `trainLMGpuResident` mirrors src/backend/train-gpu.ts:162-258 call for call (rng order,
masks, two syncs per step, checkpoint cadence). `CudaStep` is the batched form for this backend:
the B sequences of a step travel as one [B*T]-row call, the forward+backward is captured once as a
CUDA graph and replayed, and with several ranks (`DataParallel`) the gradients are summed over NCCL
before the optimizer step. `drawWindows` consumes the rng in the reference's order, so a given seed
draws the same windows in both loops.
"""
from __future__ import annotations

import math
import time
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from . import autograd as ag
from .autograd import Tensor, backward, crossEntropy, fusedCrossEntropy
from .backend import CudaBackend, _as_u32
from .qk_clip import applyQKClip


def sequenceLoss(model, inputIds, targetIds, lossChunk: int = 0) -> Tensor:
    """src/train/loss.ts:104-115."""
    if lossChunk > 0 and hasattr(model, "forwardToReadout"):
        r = model.forwardToReadout(inputIds)
        return fusedCrossEntropy(r["hidden"], r["readout"], targetIds, lossChunk)
    return crossEntropy(model.forward(inputIds), targetIds)


def freezeForScoring(model) -> None:
    """src/train/loss.ts:52-54: a model that is only scored gets no gradient buffers and stages nothing back."""
    for p in model.params():
        p.requiresGrad = False


def maskWindow(targetIds: np.ndarray, supervised: np.ndarray, start: int) -> np.ndarray:
    """src/train/trainer.ts:45-49: in place, target -> -1 where the supervision mask is 0."""
    m = supervised[start:start + len(targetIds)]
    targetIds[m == 0] = -1
    return targetIds


def trainLMGpuResident(model, gpu: CudaBackend, tokens: np.ndarray, seqLen: int, steps: int, batchPerStep: int,
                       optimizer, logEvery: int = 20, rng: Optional[Callable[[], float]] = None,
                       onLog=None, schedule=None, qkClipTau: float = 0.0, onStepTime=None,
                       supervised: Optional[np.ndarray] = None, checkpointEvery: int = 0,
                       checkpointEveryMs: float = 0.0, onCheckpoint=None, reclaimTransients: bool = False,
                       lossChunk: int = 0):
    """src/backend/train-gpu.ts:162-258."""
    import random
    rng = rng or random.random
    tokens = np.asarray(tokens)
    maxStart = len(tokens) - seqLen - 1
    if maxStart <= 0:
        raise ValueError("Not enough tokens for one training window")
    history = []
    lastCheckpointAt = time.perf_counter()
    normTensors: List[Tensor] = []
    if qkClipTau:
        qk = model.qkNorms() if hasattr(model, "qkNorms") else None
        for L in (qk["pairs"] if qk else []):
            normTensors.extend([L["qNorm"], L["kNorm"]])
    gpu.install()
    try:
        for step in range(steps):
            t0 = time.perf_counter()
            if schedule:
                optimizer.setLrScale(schedule(step))
            optimizer.zeroGrad()
            losses: List[Tensor] = []
            for b in range(batchPerStep):
                start = math.floor(rng() * maxStart)
                inputIds = tokens[start:start + seqLen].astype(np.int64)
                targetIds = tokens[start + 1:start + 1 + seqLen].astype(np.int64)
                if supervised is not None:
                    maskWindow(targetIds, supervised, start + 1)
                loss = sequenceLoss(model, inputIds, targetIds, lossChunk)
                backward(loss, 1 / batchPerStep)
                losses.append(loss)
                if reclaimTransients and b < batchPerStep - 1:
                    gpu.reclaimStepTransients(losses)
            gpu.sync(losses)
            readback = gpu.lastSyncReadbackBytes
            t1 = time.perf_counter()
            optimizer.recordStep()
            gpu.sync(normTensors)
            if qkClipTau:
                applyQKClip(model, qkClipTau)
                gpu.uploadParams(normTensors)
            if onStepTime:
                onStepTime((t1 - t0) * 1e3, (time.perf_counter() - t1) * 1e3, readback)
            avg = float(sum(float(l.data[0]) for l in losses) / batchPerStep)
            if step % logEvery == 0 or step == steps - 1:
                history.append({"step": step, "loss": avg})
                if onLog:
                    onLog(step, avg)
            dueByStep = bool(checkpointEvery) and step % checkpointEvery == 0
            dueByTime = bool(checkpointEveryMs) and (time.perf_counter() - lastCheckpointAt) * 1e3 >= checkpointEveryMs
            if onCheckpoint and step > 0 and (dueByStep or dueByTime):
                optimizer.syncWeightsToHost()
                onCheckpoint(step)
                lastCheckpointAt = time.perf_counter()
    finally:
        gpu.uninstall()
    optimizer.syncWeightsToHost()
    return history


class DataParallel:
    """One process per GPU. Rank r runs micro-batches [r*B, (r+1)*B) of each step's global draw order;
    the only exchange is an f32 sum of the gradient arena over NCCL, in buckets, on a side stream."""

    def __init__(self, gpu: CudaBackend, rank: int, world: int, unique_id: bytes, commCtas: int = 0):
        """`commCtas` > 0 caps the collective's kernel at that many CTAs (NCCL_MAX_CTAS, unless the environment already
        sets it) and makes the step leave as many SMs free for it while a reduction is in flight (`reserve`)."""
        import ctypes as C
        import os
        self.gpu, self.rank, self.world = gpu, rank, world
        self.commCtas = commCtas if world > 1 else 0
        if self.commCtas > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(self.commCtas))
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        gpu._check(gpu.lib.gt_dp_init(gpu.ctx, rank, world, buf))

    def reserve(self, on: bool):
        if self.commCtas > 0:
            self.gpu._check(self.gpu.lib.gt_dp_reserve_sms(self.gpu.ctx, self.commCtas if on else 0))

    @staticmethod
    def uniqueId() -> bytes:
        import ctypes as C
        from . import _lib
        lib = _lib.load()
        buf = (C.c_uint8 * 128)()
        st = lib.gt_dp_unique_id(buf)
        if st != 0:
            raise _lib.GtError(st, lib.gt_last_error(None).decode())
        return bytes(buf)

    def allreduce(self, addr: int, count: int, bucketElems: int = 8 << 20):
        """Sum `count` f32 at `addr` across ranks in buckets, then make the compute stream wait."""
        off = 0
        while off < count:
            n = min(bucketElems, count - off)
            self.gpu._check(self.gpu.lib.gt_dp_allreduce_start(self.gpu.ctx, addr + off * 4, n))
            off += n
        self.gpu._check(self.gpu.lib.gt_dp_wait(self.gpu.ctx))

    def start(self, addr: int, count: int):
        self.gpu._check(self.gpu.lib.gt_dp_allreduce_start(self.gpu.ctx, addr, count))

    def wait(self):
        self.gpu._check(self.gpu.lib.gt_dp_wait(self.gpu.ctx))


def drawWindows(rng, n: int, maxStart: int) -> List[int]:
    """`floor(rng() * maxStart)` n times, the reference's draw (train-gpu.ts:206)."""
    return [math.floor(rng() * maxStart) for _ in range(n)]


class CudaStep:
    """The forward+backward of one step recorded once and replayed: `batch` sequences of `seqLen` rows in
    a single [batch*seqLen]-row call. Each sequence's loss is its own mean over kept rows and the step
    loss is their mean, so gradients equal `batch` reference micro-batches seeded with 1/batch."""

    def __init__(self, model, gpu: CudaBackend, batch: int, seqLen: int, lossChunk: int = 0, world: int = 1,
                 capture: bool = True, dp: Optional["DataParallel"] = None, arena=None, layersPerBucket: int = 6,
                 source=None):
        """`dp` + `arena` turn on the gradient exchange: `arena` is what `reserveGradArena(list(reversed(params)))`
        returned, i.e. the parameter gradients in the order backward completes them (last layer first, the tied
        embedding last). The arena is cut into buckets of `layersPerBucket` layers; each bucket's all-reduce is started
        on the side stream the moment backward leaves its first layer, so it runs under the rest of backward, and the
        compute stream only joins it after the last bucket. A captured step is cut into one graph per bucket boundary and
        the NCCL calls are issued from the host between the segments (they are not recorded into the graphs)."""
        self.model, self.gpu, self.batch, self.seqLen, self.lossChunk = model, gpu, batch, seqLen, lossChunk
        self.world = world
        self.capture = capture
        self.dp, self.arena, self.layersPerBucket = dp, arena, max(1, layersPerBucket)
        self.graph = None
        self.lossTensor: Optional[Tensor] = None
        self.launchesPerReplay = 0
        # `source` (an ingest.DeviceTokenSource) switches the step's input from ids/targets arrays to window starts:
        # `runWindows(starts)` gathers ids and targets on the device as the first kernel of the (recorded) step.
        self.source = source
        self._winBufs = None

    def bucketPlan(self):
        """[(first layer of the bucket, arena offset, element count)] in the order the buckets complete, the last entry
        reaching the end of the arena (first layers, output norm, embedding)."""
        base, total, offs = self.arena
        L = len(self.model.layers)
        perLayer = len(self.model.params()) - (3 if self.model.output is not None else 2)
        perLayer //= max(L, 1)
        # arena order is reversed(params): entry j of the arena list is params[-1 - j]; layer l starts at list index (L-1-l)*perLayer
        plan = []
        l_hi = L
        while l_hi > 0:
            l_lo = max(0, l_hi - self.layersPerBucket)
            start = offs[(L - l_hi) * perLayer]
            end = offs[(L - l_lo) * perLayer] if l_lo > 0 else total
            plan.append((l_lo, start, end - start))
            l_hi = l_lo
        return plan

    def _once(self, ids: np.ndarray, targets: np.ndarray, seed: float) -> Tensor:
        loss = sequenceLoss(self.model, ids, targets, self.lossChunk)
        if self.dp is not None and self.arena is not None:
            base = self.arena[0]
            plan = self.bucketPlan()
            outs = self.model.layerOutputs
            for l_lo, start, count in plan[:-1]:
                # backward reaches the closure of layer l_lo's input only after every closure of layers >= l_lo has run
                t = outs[l_lo - 1]
                orig = t._backward

                def hooked(orig=orig, start=start, count=count):
                    if self.gpu._capturing:
                        self.gpu.cutCapture()         # the replayer starts this bucket's reduction here
                    else:
                        self.gpu.flushDeferred()      # the bucket's gradients must all have been launched
                        self.dp.start(base + start * 4, count)
                    self.dp.reserve(True)             # what follows runs (and is recorded) beside a reduction
                    orig()

                t._backward = hooked
            backward(loss, seed)
            _l, start, count = plan[-1]
            if not self.gpu._capturing:
                self.gpu.flushDeferred()
                self.dp.start(base + start * 4, count)
                self.dp.wait()
            self.dp.reserve(False)
        else:
            backward(loss, seed)
        return loss

    def run(self, ids: np.ndarray, targets: np.ndarray) -> None:
        """Enqueue forward+backward for ids/targets of shape [batch*seqLen]; gradients overwrite."""
        gpu = self.gpu
        seed = 1.0 / self.world
        gpu.install()
        gpu.setBatch(self.batch, self.seqLen)
        try:
            if not self.capture:
                # eager form of the same step: the previous step's transients go back to the pool and the parameter
                # gradients restart (sync() re-arms their first-write-overwrites state)
                gpu.sync([])
                self.lossTensor = self._once(ids, targets, seed)
                return
            if self.graph is None:
                # eager once (warms the pool, RoPE tables, scratch), then record
                warm = self._once(ids, targets, seed)
                gpu.sync([warm])
                before = gpu.kernelLaunches()
                gpu.beginCapture(seed=seed, accumulate=False)
                loss = self._once(ids, targets, seed)
                self.graph = gpu.endCapture({"loss": loss})
                self.launchesPerReplay = gpu.kernelLaunches() - before
                self.lossTensor = loss
            self.graph.writeInputs(self.graphInputs(ids, targets))   # range-checked like the eager ops' inputs
            self.replay()
        finally:
            gpu.setBatch(0)
            gpu.uninstall()

    def runWindows(self, starts: Sequence[int]) -> None:
        """The same step fed by `batch` window starts into the device-resident corpus (`source`): 8 bytes per sequence
        cross the bus instead of 8 bytes per token."""
        from .ingest import DeviceInts
        src, gpu, B, T = self.source, self.gpu, self.batch, self.seqLen
        if src is None:
            raise ValueError("runWindows needs a DeviceTokenSource (CudaStep(..., source=...))")
        if len(starts) != B:
            raise ValueError(f"{len(starts)} window starts for a batch of {B}")
        seed = 1.0 / self.world
        gpu.install()
        gpu.setBatch(B, T)
        try:
            if not self.capture:
                gpu.sync([])
                ids, tg = src.gather(starts, T)
                self.lossTensor = self._once(ids, tg, seed)
                return
            if self.graph is None:
                sbuf = src.writeStarts(starts, T)
                ids = DeviceInts(gpu._acquirePersistent(B * T * 4), B * T, src.vocabSize)
                tg = DeviceInts(gpu._acquirePersistent(B * T * 4), B * T, src.vocabSize)
                self._winBufs = (sbuf, ids, tg)
                src.gatherInto(sbuf, B, T, ids.addr, tg.addr)
                warm = self._once(ids, tg, seed)
                gpu.sync([warm])
                before = gpu.kernelLaunches()
                gpu.beginCapture(seed=seed, accumulate=False)
                src.gatherInto(sbuf, B, T, ids.addr, tg.addr)        # first node of the recorded step
                loss = self._once(ids, tg, seed)
                self.graph = gpu.endCapture({"loss": loss})
                self.launchesPerReplay = gpu.kernelLaunches() - before
                self.lossTensor = loss
            src.writeStarts(starts, T)        # range-checked; lands in the buffer the recorded gather reads
            self.replay()
        finally:
            gpu.setBatch(0)
            gpu.uninstall()

    def graphInputs(self, ids, targets):
        return [ids, targets]

    def replay(self) -> None:
        """Enqueue the recorded step again on the inputs already on the device (plus the gradient exchange)."""
        if self.dp is None or self.arena is None:
            self.graph.replay()
            return
        base = self.arena[0]
        plan = self.bucketPlan()
        between = [(lambda s=s, c=c: self.dp.start(base + s * 4, c)) for _l, s, c in plan[:-1]]
        self.graph.replay(between)
        _l, s, c = plan[-1]
        self.dp.start(base + s * 4, c)
        self.dp.wait()

    def lossesBegin(self) -> int:
        """Start reading the last run's losses without waiting for them: the copy is queued behind everything enqueued
        so far and lands in pinned memory while the host goes on to enqueue the next step (whose loss kernel waits, on
        the device, for this copy). Returns a ticket for `lossesEnd`. A loop that reads each step's loss after it has
        enqueued the next step never leaves the device idle between steps."""
        gpu = self.gpu
        e = gpu._entries[self.lossTensor]
        ticket = gpu.readAsync(e.data, (1 + self.batch) * 4)
        gpu.readFence()
        return ticket

    def lossesEnd(self, ticket: int) -> np.ndarray:
        """[mean over sequences, per-sequence...] of the run `ticket` was taken after (blocks until that copy landed)."""
        out = np.empty(1 + self.batch, np.float32)
        self.gpu.readFinish(ticket, out)
        return out

    def losses(self) -> np.ndarray:
        """[mean over sequences, per-sequence...] of the last run (blocks)."""
        gpu = self.gpu
        e = gpu._entries[self.lossTensor]
        out = np.empty(1 + self.batch, np.float32)
        gpu._read(e.data, out)
        return out
