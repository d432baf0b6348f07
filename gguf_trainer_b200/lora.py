"""LoRA adapters attached through `linear` (src/train/lora.ts:46-120): freeze everything, give every
Muon-group matrix A ~ N(0, 1/in) [rank, in] and B = 0 [out, rank], route them to AdamW."""
from __future__ import annotations

import math
from typing import Dict, List

import numpy as np

from . import autograd as ag
from .arch import param
from .autograd import LoraAdapter, Tensor
from .rng import Mulberry32

_installed = False


class LoraHandle:
    def __init__(self, model, rank, alpha, adapters, aux):
        self.rank = rank
        self.scale = alpha / rank
        self.adapters = adapters          # [(w, LoraAdapter)]
        self.groups = {"muon": [], "aux": aux}
        self.adapted = len(adapters)
        self.frozen = len(model.params())
        self.trainable = sum(t.size for t in aux)

    def _fold(self, sign: float):
        """Host fold W += sign * scale * B·A, f64 accumulate, f32 store (lora.ts:81-96)."""
        for w, ad in self.adapters:
            outDim, inDim = w.shape
            b = ad.b.data.reshape(outDim, self.rank).astype(np.float64)
            a = ad.a.data.reshape(self.rank, inDim).astype(np.float64)
            w.data[:] = (w.data.reshape(outDim, inDim).astype(np.float64) + sign * self.scale * (b @ a)).astype(
                np.float32).reshape(-1)

    def merge(self):
        self._fold(1.0)

    def unmerge(self):
        self._fold(-1.0)


def applyLora(model, rank: int, alpha: float, rng: Mulberry32) -> LoraHandle:
    global _installed
    if rank <= 0:
        raise ValueError(f"applyLora: rank must be positive, got {rank}")
    if alpha <= 0:
        raise ValueError(f"applyLora: alpha must be positive, got {alpha}")
    if _installed:
        raise RuntimeError("applyLora: adapters are already installed; call clearLora() first")
    base = model.paramGroups()["muon"]
    for t in model.params():
        t.requiresGrad = False
    table: Dict[int, LoraAdapter] = {}
    adapters = []
    aux: List[Tensor] = []
    sc = alpha / rank
    for w in base:
        if len(w.shape) != 2:
            continue
        outDim, inDim = w.shape
        a = param([rank, inDim], 1 / math.sqrt(inDim), rng)
        b = Tensor.zeros([outDim, rank], True)
        ad = LoraAdapter(a, b, sc)
        table[id(w)] = ad
        adapters.append((w, ad))
        aux.extend([a, b])
    ag.setLoraAdapters(table)
    _installed = True
    return LoraHandle(model, rank, alpha, adapters, aux)


def clearLora(model=None):
    global _installed
    ag.setLoraAdapters({})
    _installed = False
    if model is not None:
        for t in model.params():
            t.requiresGrad = True
