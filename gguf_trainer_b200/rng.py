"""`mulberry32` and Box-Muller `randn` with the reference's exact draw order
(src/model/autograd.ts:61-78), vectorised: the generator's state is a counter
(a += 0x6d2b79f5 per draw), so draw n is a pure function of (seed, n)."""
from __future__ import annotations

import math

import numpy as np

_INC = 0x6D2B79F5


class Mulberry32:
    def __init__(self, seed: int):
        self.a = seed & 0xFFFFFFFF

    def __call__(self) -> float:
        self.a = (self.a + _INC) & 0xFFFFFFFF
        a = self.a
        t = ((a ^ (a >> 15)) * (1 | a)) & 0xFFFFFFFF
        t = ((t + (((t ^ (t >> 7)) * (61 | t)) & 0xFFFFFFFF)) & 0xFFFFFFFF) ^ t
        return ((t ^ (t >> 14)) & 0xFFFFFFFF) / 4294967296.0

    def draws(self, n: int) -> np.ndarray:
        """The next n uniforms as float64, advancing the state."""
        k = np.arange(1, n + 1, dtype=np.uint64)
        a = ((np.uint64(self.a) + k * np.uint64(_INC)) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
        self.a = int(a[-1]) if n else self.a
        with np.errstate(over="ignore"):
            t = (a ^ (a >> np.uint32(15))) * (np.uint32(1) | a)
            t = (t + (t ^ (t >> np.uint32(7))) * (np.uint32(61) | t)) ^ t
            r = t ^ (t >> np.uint32(14))
        return r.astype(np.float64) / 4294967296.0

    def randn(self, shape, scale: float = 1.0) -> np.ndarray:
        """`randn(rng) * scale` per element, rounded to f32 like a Float32Array store."""
        n = int(np.prod(shape))
        start = self.a
        u = self.draws(2 * n)
        if (u == 0).any():  # a zero draw is redrawn by the reference: replay that path exactly
            self.a = start
            out = np.empty(n, np.float32)
            for i in range(n):
                a = b = 0.0
                while a == 0:
                    a = self()
                while b == 0:
                    b = self()
                out[i] = math.sqrt(-2 * math.log(a)) * math.cos(2 * math.pi * b) * scale
            return out.reshape(shape)
        z = np.sqrt(-2 * np.log(u[0::2])) * np.cos(2 * np.pi * u[1::2])
        return (z * scale).astype(np.float32).reshape(shape)

    def uniform_pm1(self, shape) -> np.ndarray:
        n = int(np.prod(shape))
        return (self.draws(n) * 2 - 1).astype(np.float32).reshape(shape)

    def randint(self, n: int, hi: int) -> np.ndarray:
        return np.floor(self.draws(n) * hi).astype(np.int64)
