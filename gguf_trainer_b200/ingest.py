"""Token and mask ingest on the device. The corpus (`.tokens`) and the supervision mask (`.mask`) live in HBM exactly
as they are on disk, bare little-endian u16 or u32 values (src/data/tokens.ts:12-14, 158-185; the mask is read with the
token width, src/commands/pretrain.ts:416). A step then sends B window starts (8 bytes each) instead of B*T ids and B*T
targets, and one integer kernel forms both arrays where the model reads them: ids = tokens[start : start+T], targets =
tokens[start+1 : start+1+T] with -1 where the mask is 0 (maskWindow, src/train/trainer.ts:45-49), windows drawn as
floor(rng() * maxStart) (src/backend/train-gpu.ts:206-208). The values never pass through host number arrays."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib
from .backend import CudaBackend


def tokenBytes(vocabSize: int) -> int:
    """src/data/tokens.ts:35-37: 2 bytes per token when the vocabulary fits u16, else 4."""
    return 2 if vocabSize <= 0x10000 else 4


class DeviceInts:
    """Integer op inputs (ids or targets) that are already on the device. `bound` is the exclusive upper bound their
    producer vouches for, checked once when the corpus was uploaded; ops accept them where they accept host arrays."""

    __slots__ = ("addr", "count", "bound")

    def __init__(self, addr: int, count: int, bound: int):
        self.addr, self.count, self.bound = addr, count, bound

    def __len__(self) -> int:
        return self.count


class DeviceTokenSource:
    """A token file (and optionally its mask) resident on the device: the `TokenSource` of src/data/tokens.ts:25-33
    for this backend. `length` and the range check of `window` keep their meaning; `gather` replaces B pairs of
    `window()` calls plus `maskWindow` by one kernel."""

    def __init__(self, gpu: CudaBackend, tokens: np.ndarray, vocabSize: int, supervised: Optional[np.ndarray] = None):
        bpt = tokenBytes(vocabSize)
        dt = np.dtype("<u2") if bpt == 2 else np.dtype("<u4")
        tokens = np.asarray(tokens)
        if tokens.dtype.kind not in "iu":
            raise ValueError("token corpus must be an integer array")
        if tokens.size and (int(tokens.min()) < 0 or int(tokens.max()) >= (1 << (8 * bpt))):
            raise ValueError(f"token values do not fit {bpt} bytes per token")
        self.gpu, self.vocabSize, self.bytesPerToken = gpu, vocabSize, bpt
        self.length = int(tokens.size)
        raw = np.ascontiguousarray(tokens.astype(dt, copy=False))
        self.tokens = gpu.createStateBuffer(max(raw.nbytes, 4))
        gpu._write(self.tokens, raw.view(np.uint8))
        self.mask = 0
        if supervised is not None:
            supervised = np.asarray(supervised)
            if supervised.size != self.length:
                # src/commands/pretrain.ts:417-419
                raise ValueError(f"mask has {supervised.size} tokens, corpus has {self.length}")
            m = np.ascontiguousarray(supervised.astype(dt, copy=False))
            self.mask = gpu.createStateBuffer(max(m.nbytes, 4))
            gpu._write(self.mask, m.view(np.uint8))
        # the corpus must fit the vocabulary (assertCorpusFitsVocab does this on the host when a file is opened);
        # checked once here on the device, so no window needs a per-step range check afterwards
        mx = C.c_uint32()
        gpu._check(gpu.lib.gt_tokens_max(gpu.ctx, self.tokens, bpt, self.length, C.byref(mx)))
        if int(mx.value) >= vocabSize:
            raise ValueError(
                f"corpus holds token id {int(mx.value)}, which is not in [0,{vocabSize}). "
                f"A corpus tokenized with a different vocab than the checkpoint is the usual cause.")
        self._starts = {}   # B -> device buffer of B u64

    def startsBuffer(self, B: int) -> int:
        if B not in self._starts:
            self._starts[B] = self.gpu.createStateBuffer(8 * B)
        return self._starts[B]

    def writeStarts(self, starts: Sequence[int], T: int) -> int:
        """Range-check the window starts like `window()` (src/data/tokens.ts:166-168) and put them on the device."""
        s = np.asarray(starts, dtype=np.int64)
        bad = np.nonzero((s < 0) | (s + T + 1 > self.length))[0]
        if bad.size:
            b = int(s[bad[0]])
            raise ValueError(f"window [{b},{b + T + 1}) out of range 0..{self.length}")
        buf = self.startsBuffer(len(s))
        self.gpu._write(buf, s.astype("<u8"))
        return buf

    def gatherInto(self, startsBuf: int, B: int, T: int, ids: int, targets: int):
        g = self.gpu
        g._check(g.lib.gt_gather_windows(g.ctx, self.tokens, self.mask, self.bytesPerToken, self.length, startsBuf, B, T,
                                         ids, targets))

    def gather(self, starts: Sequence[int], T: int):
        """(ids, targets) as `DeviceInts` of B*T elements each, in transient buffers of the current graph."""
        B = len(starts)
        buf = self.writeStarts(starts, T)
        g = self.gpu
        ids, tg = g._acquireTransient(B * T * 4), g._acquireTransient(B * T * 4)
        self.gatherInto(buf, B, T, ids, tg)
        return DeviceInts(ids, B * T, self.vocabSize), DeviceInts(tg, B * T, self.vocabSize)

    def window(self, start: int, length: int) -> np.ndarray:
        """`TokenSource.window` (blocking read; for tests and tools, the step loop uses `gather`)."""
        if start < 0 or start + length > self.length:
            raise ValueError(f"window [{start},{start + length}) out of range 0..{self.length}")
        dt = np.dtype("<u2") if self.bytesPerToken == 2 else np.dtype("<u4")
        out = np.empty(length, dt)
        self.gpu._check(self.gpu.lib.gt_read(self.gpu.ctx, self.tokens + start * self.bytesPerToken, out.ctypes.data, out.nbytes))
        return out.astype(np.int64)

    def close(self):
        for b in [self.tokens, self.mask] + list(self._starts.values()):
            if b:
                self.gpu._check(self.gpu.lib.gt_free(self.gpu.ctx, b))
        self.tokens = self.mask = 0
        self._starts = {}
