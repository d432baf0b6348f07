"""Warmup-Stable-Decay learning-rate multiplier (src/train/schedule.ts:20-36)."""
from __future__ import annotations

import math


def wsdSchedule(warmupSteps: int, stableSteps: int, cooldownSteps: int, minScale: float = 0.0):
    warmup = max(0, math.floor(warmupSteps))
    stable = max(0, math.floor(stableSteps))
    cooldown = max(0, math.floor(cooldownSteps))
    cooldownStart = warmup + stable
    total = cooldownStart + cooldown

    def f(step: int) -> float:
        if warmup > 0 and step < warmup:
            return (step + 1) / warmup
        if step < cooldownStart:
            return 1.0
        if cooldown > 0 and step < total:
            frac = (step - cooldownStart + 1) / cooldown
            return 1 - (1 - minScale) * frac
        return 1.0 if step < total else minScale

    return f
