"""Host-side tape and op interface: the Python mirror of src/model/autograd.ts.

Same names, argument meaning and error behaviour as the reference so that the parity tests read
like its own: `Tensor`, `backward`, `checkpoint`, `setOpsBackend`, `setLoraAdapters`, the 14 ops and
the validators that run ABOVE the backend dispatch. Unlike the reference there are no CPU
implementations here: with no backend installed every op raises. The device work lives behind
`OpsBackend` (see backend.CudaBackend).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

_tensors_created = 0


class Tensor:
    """src/model/autograd.ts:20-51. `data`/`grad` are host f32 arrays; with a device backend they are
    stale until `sync()` copies them back."""

    __slots__ = ("data", "grad", "shape", "requiresGrad", "_backward", "_prev", "seq", "__weakref__")

    def __init__(self, data: np.ndarray, shape: Sequence[int], requiresGrad: bool = False):
        global _tensors_created
        data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        n = 1
        for s in shape:
            n *= int(s)
        if data.size != n:
            raise ValueError(f"data length {data.size} != shape {list(shape)}")
        self.data = data
        self.shape = [int(s) for s in shape]
        self.requiresGrad = requiresGrad
        self.grad = np.zeros(n, dtype=np.float32)
        self._backward: Callable[[], None] = _noop
        self._prev: List["Tensor"] = []
        self.seq = _tensors_created
        _tensors_created += 1

    @staticmethod
    def zeros(shape: Sequence[int], requiresGrad: bool = False) -> "Tensor":
        n = 1
        for s in shape:
            n *= int(s)
        return Tensor(np.zeros(n, dtype=np.float32), shape, requiresGrad)

    def zeroGrad(self):
        self.grad.fill(0)

    @property
    def size(self) -> int:
        return self.data.size


def _noop():
    return None


def backward(loss: Tensor, seed: float = 1.0):
    """src/model/autograd.ts:81-93: reverse topological walk seeded with loss.grad[0] = seed."""
    topo: List[Tensor] = []
    seen = set()
    stack = [(loss, 0)]
    seen.add(id(loss))
    while stack:
        t, i = stack.pop()
        if i < len(t._prev):
            stack.append((t, i + 1))
            p = t._prev[i]
            if id(p) not in seen:
                seen.add(id(p))
                stack.append((p, 0))
        else:
            topo.append(t)
    loss.grad[0] = seed
    for t in reversed(topo):
        t._backward()


# ---------------------------------------------------------------------------
# backend dispatch (autograd.ts:103-164, 275-279)
# ---------------------------------------------------------------------------
_ops_backend = None
_checkpointing = False


def setOpsBackend(b):
    global _ops_backend
    _ops_backend = b


def opsBackend():
    return _ops_backend


def _need_backend():
    if _ops_backend is None:
        raise RuntimeError(
            "no ops backend installed: this package has no CPU implementation of the ops. "
            "Create a CudaBackend and call install().")
    return _ops_backend


def setCheckpointing(on: bool):
    """autograd.ts:178-180."""
    global _checkpointing
    _checkpointing = bool(on)


def _assert_self_contained(out: Tensor, inputs: List[Tensor], born: int):
    """autograd.ts:198-215."""
    seen = {id(t) for t in inputs}
    if id(out) in seen:
        raise RuntimeError("checkpoint: fn returned one of its inputs; there is nothing to recompute")
    stack = [out]
    while stack:
        t = stack.pop()
        if id(t) in seen:
            continue
        seen.add(id(t))
        if len(t._prev) > 0 and t.seq < born:
            raise RuntimeError(
                "checkpoint: the block reads a computed tensor it did not create. Pass it in `inputs`, "
                "or move its computation inside the block (docs/adding-an-architecture.md).")
        stack.extend(t._prev)


def checkpoint(inputs: List[Tensor], fn: Callable[[], Tensor]) -> Tensor:
    """autograd.ts:234-273: run `fn` without keeping its interior and replay it in backward."""
    if not _checkpointing:
        return fn()
    rb = _ops_backend if (_ops_backend is not None and hasattr(_ops_backend, "beginRegion")) else None
    born = _tensors_created
    mark = rb.beginRegion() if rb else 0
    tok = rb.regionToken() if (rb is not None and hasattr(rb, "regionToken")) else None   # optional backend extension
    out = fn()
    _assert_self_contained(out, inputs, born)
    if rb:
        rb.endRegion(mark, [out])
    out._prev = list(inputs)

    def _bw():
        mark2 = rb.beginRegion() if rb else 0
        if tok is not None:
            rb.replayOf(tok)
        replay = fn()
        if rb:
            rb.seedGradFrom(replay, out)
        else:
            replay.grad[:] = out.grad
        topo: List[Tensor] = []
        seen = {id(t) for t in inputs}
        stack = []
        if id(replay) not in seen:
            seen.add(id(replay))
            stack.append((replay, 0))
        while stack:
            t, i = stack.pop()
            if i < len(t._prev):
                stack.append((t, i + 1))
                p = t._prev[i]
                if id(p) not in seen:
                    seen.add(id(p))
                    stack.append((p, 0))
            else:
                topo.append(t)
        for t in reversed(topo):
            t._backward()
        if rb:
            rb.endRegion(mark2, [])

    out._backward = _bw
    return out


# ---------------------------------------------------------------------------
# LoRA routing (autograd.ts:286-319)
# ---------------------------------------------------------------------------
class LoraAdapter:
    __slots__ = ("a", "b", "scale")

    def __init__(self, a: Tensor, b: Tensor, scale: float):
        self.a, self.b, self.scale = a, b, scale


_lora: Dict[int, LoraAdapter] = {}


def setLoraAdapters(m: Dict[int, LoraAdapter]):
    """Keys are `id(weight_tensor)`."""
    global _lora
    _lora = m


def linear(x: Tensor, w: Tensor) -> Tensor:
    """y = x·Wᵀ, plus the low-rank update when `w` carries an adapter (autograd.ts:311-319)."""
    if _lora:
        ad = _lora.get(id(w))
        if ad is not None:
            be = _need_backend()
            if getattr(be, "fuseLora", False):       # optional backend extension: the same sum as one recorded op
                if x.shape[1] != w.shape[1] or x.shape[1] != ad.a.shape[1] or ad.b.shape[1] != ad.a.shape[0]:
                    raise ValueError(f"linear dim mismatch: x is {x.shape}, w is {w.shape}, adapter A {ad.a.shape}, B {ad.b.shape}")
                return be.loraLinear(x, w, ad.a, ad.b, ad.scale)
            return add(_linear_raw(x, w), scale(_linear_raw(_linear_raw(x, ad.a), ad.b), ad.scale))
    return _linear_raw(x, w)


def _linear_raw(x: Tensor, w: Tensor) -> Tensor:
    in_dim = x.shape[1]
    in_dim2 = w.shape[1]
    if in_dim != in_dim2:
        raise ValueError(
            f"linear dim mismatch: x is [{', '.join(map(str, x.shape))}] and w is [{', '.join(map(str, w.shape))}], "
            f"so the contracted dimension is {in_dim} on one side and {in_dim2} on the other. "
            f"A projection wired to the wrong config field is the usual cause.")
    return _need_backend().linear(x, w)


def add(a: Tensor, b: Tensor) -> Tensor:
    return _need_backend().add(a, b)


def mul(a: Tensor, b: Tensor) -> Tensor:
    return _need_backend().mul(a, b)


def silu(x: Tensor) -> Tensor:
    return _need_backend().silu(x)


def gelu(x: Tensor) -> Tensor:
    return _need_backend().gelu(x)


def scale(x: Tensor, c: float) -> Tensor:
    return _need_backend().scale(x, c)


def rmsNorm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    return _need_backend().rmsNorm(x, weight, eps)


def rmsNormHeads(x: Tensor, weight: Tensor, T: int, H: int, hd: int, eps: float) -> Tensor:
    return _need_backend().rmsNormHeads(x, weight, T, H, hd, eps)


def _is_int(v) -> bool:
    return isinstance(v, (int, np.integer)) or (isinstance(v, float) and v.is_integer())


def assertRank(t: Tensor, rank: int, name: str, where: str):
    """autograd.ts:835-839."""
    if len(t.shape) != rank:
        raise ValueError(f"{where}: {name} must be {rank}-D, got [{', '.join(map(str, t.shape))}]")


def assertMatrix(t: Tensor, name: str, where: str):
    assertRank(t, 2, name, where)


def assertIdsInTable(ids, V: int, where: str):
    """autograd.ts:813-823. Every embedding id must be a row of the table."""
    arr = np.asarray(ids)
    if arr.dtype.kind in "iu":
        bad = np.nonzero((arr < 0) | (arr >= V))[0]
        if bad.size:
            t = int(bad[0])
            raise ValueError(
                f"{where}: id {int(arr[t])} at position {t} is not an integer in [0,{V}). "
                f"A corpus tokenized with a different vocab than the checkpoint is the usual cause.")
        return
    for t, v in enumerate(ids):
        if not _is_int(v) or v < 0 or v >= V:
            raise ValueError(
                f"{where}: id {v} at position {t} is not an integer in [0,{V}). "
                f"A corpus tokenized with a different vocab than the checkpoint is the usual cause.")


def keptRowsInVocab(targets, T: int, V: int, where: str) -> int:
    """autograd.ts:875-894: count kept rows, refusing any target that is not -1 or a vocab row."""
    if len(targets) != T:
        raise ValueError(
            f"{where}: {len(targets)} targets for {T} logit rows. The loss sums T rows and means "
            f"over the targets it counts, so a mismatch reports a plausible wrong loss.")
    arr = np.asarray(targets)
    if arr.dtype.kind in "iu":
        bad = np.nonzero((arr < -1) | (arr >= V))[0]
        if bad.size:
            t = int(bad[0])
            raise ValueError(
                f"{where}: target {int(arr[t])} at position {t} is not -1 (ignore) or an integer in [0,{V}). "
                f"A corpus tokenized with a different vocab than the checkpoint is the usual cause.")
        return int((arr >= 0).sum())
    kept = 0
    for t, g in enumerate(targets):
        if not _is_int(g) or g < -1 or g >= V:
            raise ValueError(
                f"{where}: target {g} at position {t} is not -1 (ignore) or an integer in [0,{V}). "
                f"A corpus tokenized with a different vocab than the checkpoint is the usual cause.")
        if g >= 0:
            kept += 1
    return kept


def keptTeacherRows(teacherIds, teacherProbs, T: int, k: int, V: int) -> int:
    """autograd.ts:760-791."""
    if k < 1:
        raise ValueError(f"softCrossEntropy: k must be >= 1, got {k}")
    if len(teacherIds) != T * k or len(teacherProbs) != T * k:
        raise ValueError(
            f"softCrossEntropy: teacher arrays must be [T*k]={T * k}, got {len(teacherIds)}/{len(teacherProbs)}")
    kept = 0
    for t in range(T):
        if teacherIds[t * k] == -1:
            continue
        for j in range(k):
            i = teacherIds[t * k + j]
            if not _is_int(i) or i < 0 or i >= V:
                raise ValueError(
                    f"softCrossEntropy: teacher id {i} at slot {j} of row {t} is not an "
                    f"integer in [0,{V}). Only -1 in the first slot marks an ignored row. "
                    f"A teacher file built against a different vocab than the checkpoint is "
                    f"the usual cause.")
        kept += 1
    return kept


def _on_device(values, V: int, where: str) -> bool:
    """Integer inputs produced on the device (the window gather) carry the bound their producer checked once; the
    per-element validators have nothing on the host to read."""
    bound = getattr(values, "bound", None)
    if bound is None or not hasattr(values, "addr"):
        return False
    if bound > V:
        raise ValueError(f"{where}: device-resident ids were checked against a vocabulary of {bound}, this table has {V} rows")
    return True


def embedding(weight: Tensor, ids) -> Tensor:
    assertMatrix(weight, "weight", "embedding")
    if not _on_device(ids, weight.shape[0], "embedding"):
        assertIdsInTable(ids, weight.shape[0], "embedding")
    return _need_backend().embedding(weight, ids)


def rope(x: Tensor, T: int, H: int, hd: int, base: float, posOffset: int = 0) -> Tensor:
    return _need_backend().rope(x, T, H, hd, base, posOffset)


def attention(q: Tensor, k: Tensor, v: Tensor, T: int, Hq: int, Hkv: int, hd: int, window: int = 0) -> Tensor:
    return _need_backend().attention(q, k, v, T, Hq, Hkv, hd, window)


def crossEntropy(logits: Tensor, targets) -> Tensor:
    """autograd.ts:897-952 (validation above the dispatch; `kept` passed down)."""
    assertMatrix(logits, "logits", "crossEntropy")
    T, V = logits.shape
    if _on_device(targets, V, "crossEntropy"):
        if len(targets) != T:
            raise ValueError(f"crossEntropy: {len(targets)} targets for {T} logit rows.")
        kept = -1      # counted on the device from the targets themselves
    else:
        kept = keptRowsInVocab(targets, T, V, "crossEntropy")
    return _need_backend().crossEntropy(logits, targets, kept)


def fusedCrossEntropy(hidden: Tensor, w: Tensor, targets, chunk: int) -> Tensor:
    """autograd.ts:968-1055."""
    assertMatrix(hidden, "hidden", "fusedCrossEntropy")
    assertMatrix(w, "w", "fusedCrossEntropy")
    T, H = hidden.shape
    V, H2 = w.shape
    if H != H2:
        raise ValueError(f"fusedCrossEntropy dim mismatch {H} vs {H2}")
    if chunk <= 0:
        raise ValueError(f"fusedCrossEntropy chunk must be positive, got {chunk}")
    if id(w) in _lora:
        raise ValueError(
            "fusedCrossEntropy: the readout weight carries a LoRA adapter, which this "
            "path cannot apply. Put the readout in the aux param group, or use --loss-chunk 0.")
    if _on_device(targets, V, "fusedCrossEntropy"):
        if len(targets) != T:
            raise ValueError(f"fusedCrossEntropy: {len(targets)} targets for {T} hidden rows.")
        kept = -1
    else:
        kept = keptRowsInVocab(targets, T, V, "fusedCrossEntropy")
    return _need_backend().fusedCrossEntropy(hidden, w, targets, chunk, kept)


def softCrossEntropy(logits: Tensor, teacherIds, teacherProbs, k: int) -> Tensor:
    """autograd.ts:1076-1138."""
    assertMatrix(logits, "logits", "softCrossEntropy")
    T, V = logits.shape
    kept = keptTeacherRows(teacherIds, teacherProbs, T, k, V)
    return _need_backend().softCrossEntropy(logits, teacherIds, teacherProbs, k, kept)
