"""QK-logit control on the host (src/train/qk-clip.ts:35-64): cap each layer's logit-scale proxy at tau
by rescaling qNorm/kNorm. Operates on the host copies; the step loop re-uploads the clipped norms."""
from __future__ import annotations

import math

import numpy as np


def qkLogitScale(qNorm: np.ndarray, kNorm: np.ndarray, headDim: int) -> float:
    p = qNorm[:headDim].astype(np.float64) * kNorm[:headDim].astype(np.float64)
    return math.sqrt(float((p * p).sum())) / math.sqrt(headDim)


def applyQKClip(model, tau: float) -> int:
    if not (tau > 0):
        raise ValueError("qk-clip tau must be > 0")
    qk = model.qkNorms() if hasattr(model, "qkNorms") else None
    if not qk:
        return 0
    hd = qk["headDim"]
    clipped = 0
    for L in qk["pairs"]:
        s = qkLogitScale(L["qNorm"].data, L["kNorm"].data, hd)
        if s > tau:
            f = math.sqrt(tau / s)
            L["qNorm"].data[:hd] = (L["qNorm"].data[:hd].astype(np.float64) * f).astype(np.float32)
            L["kNorm"].data[:hd] = (L["kNorm"].data[:hd].astype(np.float64) * f).astype(np.float32)
            clipped += 1
    return clipped
