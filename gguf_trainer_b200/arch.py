"""The three architectures' forward passes, parameter order and optimizer groups, mirroring
src/arch/llama.ts:138-222, src/arch/qwen3.ts:87-195 and src/arch/gemma3.ts:102-223.

In a deployment these stay in TypeScript unchanged; this module is the Python driver of the same
op sequence so the backend can be exercised and measured without a JS runtime. GGUF export,
config-from-flags and the llama Q/K row permutation are export-side and not part of this path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import numpy as np

from .autograd import (Tensor, add, attention, checkpoint, embedding, gelu, linear, mul, rmsNorm, rmsNormHeads, rope,
                       scale, silu)
from .rng import Mulberry32


@dataclass
class ModelConfig:
    arch: str                 # "llama" | "qwen3" | "gemma3"
    vocabSize: int
    hiddenSize: int
    nLayers: int
    nHeads: int
    nKVHeads: int
    headDim: int
    ffnDim: int
    ropeBase: float
    rmsEps: float
    ropeBaseLocal: float = 10_000.0   # gemma3 sliding-window layers
    slidingWindow: int = 0            # gemma3
    swaPattern: int = 0               # gemma3: layer il is global iff il % swaPattern == swaPattern - 1
    tieEmbeddings: bool = True
    maxSeq: int = 8192
    init: str = "reference"           # "reference": embeddings 0.02, matrices 1/sqrt(fan_in); "n002": every matrix N(0, 0.02)

    def oracle_dict(self) -> dict:
        """The same config in the CPU oracle's vocabulary (tests only)."""
        return dict(arch=self.arch, vocab=self.vocabSize, hidden=self.hiddenSize, layers=self.nLayers,
                    heads=self.nHeads, kv_heads=self.nKVHeads, head_dim=self.headDim, ffn=self.ffnDim,
                    rope_base=self.ropeBase, rope_base_local=self.ropeBaseLocal, eps=self.rmsEps,
                    window=self.slidingWindow, swa_pattern=self.swaPattern, tie=self.tieEmbeddings, init=self.init)


def param(shape, std: float, rng: Mulberry32) -> Tensor:
    """src/model/autograd.ts:54-58."""
    return Tensor(rng.randn(shape, std), shape, True)


def ones(shape) -> Tensor:
    """src/arch/common.ts `ones`: a norm gain starts at 1."""
    n = int(np.prod(shape))
    return Tensor(np.ones(n, np.float32), shape, True)


class Layer:
    __slots__ = ("attnNorm", "qProj", "kProj", "vProj", "oProj", "qNorm", "kNorm", "postAttnNorm", "ffnNorm", "gate",
                 "up", "down", "postFfnNorm")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)


def isGlobalLayer(c: ModelConfig, il: int) -> bool:
    """src/arch/gemma3.ts:75-77."""
    return c.swaPattern > 0 and il % c.swaPattern == c.swaPattern - 1


class LanguageModel:
    """One class for the three architectures; `cfg.arch` selects the differences, which are exactly the
    ones the reference lists: QK-norm (qwen3, gemma3), sandwich norms, GeGLU, embedding scale, two RoPE
    bases and sliding windows (gemma3)."""

    def __init__(self, cfg: ModelConfig, rng: Mulberry32):
        self.cfg = cfg
        c = cfg
        h = c.hiddenSize
        qDim, kvDim = c.nHeads * c.headDim, c.nKVHeads * c.headDim
        sd = (lambda fan: 0.02) if c.init == "n002" else (lambda fan: 1 / math.sqrt(fan))
        self.tokenEmbd = param([c.vocabSize, h], 0.02, rng)
        self.outputNorm = ones([h])
        self.output = None if c.tieEmbeddings else param([c.vocabSize, h], 0.02, rng)
        self.layers: List[Layer] = []
        qk = c.arch in ("qwen3", "gemma3")
        g3 = c.arch == "gemma3"
        for _ in range(c.nLayers):
            L = Layer()
            L.attnNorm = ones([h])
            L.qProj = param([qDim, h], sd(h), rng)
            L.kProj = param([kvDim, h], sd(h), rng)
            L.vProj = param([kvDim, h], sd(h), rng)
            L.oProj = param([h, qDim], sd(qDim), rng)
            if qk:
                L.qNorm = ones([c.headDim])
                L.kNorm = ones([c.headDim])
            if g3:
                L.postAttnNorm = ones([h])
            L.ffnNorm = ones([h])
            L.gate = param([c.ffnDim, h], sd(h), rng)
            L.up = param([c.ffnDim, h], sd(h), rng)
            L.down = param([h, c.ffnDim], sd(c.ffnDim), rng)
            if g3:
                L.postFfnNorm = ones([h])
            self.layers.append(L)

    def _layerParams(self, L: Layer) -> List[Tensor]:
        a = self.cfg.arch
        if a == "llama":
            return [L.attnNorm, L.qProj, L.kProj, L.vProj, L.oProj, L.ffnNorm, L.gate, L.up, L.down]
        if a == "qwen3":
            return [L.attnNorm, L.qProj, L.kProj, L.vProj, L.oProj, L.qNorm, L.kNorm, L.ffnNorm, L.gate, L.up, L.down]
        return [L.attnNorm, L.qProj, L.kProj, L.vProj, L.oProj, L.qNorm, L.kNorm, L.postAttnNorm, L.ffnNorm, L.gate,
                L.up, L.down, L.postFfnNorm]

    def params(self) -> List[Tensor]:
        ps = [self.tokenEmbd, self.outputNorm]
        if self.output is not None:
            ps.append(self.output)
        for L in self.layers:
            ps.extend(self._layerParams(L))
        return ps

    def paramGroups(self) -> Dict[str, List[Tensor]]:
        muon: List[Tensor] = []
        aux: List[Tensor] = [self.tokenEmbd, self.outputNorm]
        if self.output is not None:
            aux.append(self.output)
        a = self.cfg.arch
        for L in self.layers:
            muon.extend([L.qProj, L.kProj, L.vProj, L.oProj, L.gate, L.up, L.down])
            if a == "llama":
                aux.extend([L.attnNorm, L.ffnNorm])
            elif a == "qwen3":
                aux.extend([L.attnNorm, L.qNorm, L.kNorm, L.ffnNorm])
            else:
                aux.extend([L.attnNorm, L.qNorm, L.kNorm, L.postAttnNorm, L.ffnNorm, L.postFfnNorm])
        return {"muon": muon, "aux": aux}

    def qkNorms(self):
        if self.cfg.arch == "llama":
            return None
        return {"headDim": self.cfg.headDim, "pairs": [{"qNorm": L.qNorm, "kNorm": L.kNorm} for L in self.layers]}

    def _block(self, hIn: Tensor, il: int, T: int) -> Tensor:
        c = self.cfg
        L = self.layers[il]
        g3 = c.arch == "gemma3"
        glob = (not g3) or isGlobalLayer(c, il)
        window = 0 if glob else c.slidingWindow
        ropeB = c.ropeBase if glob else c.ropeBaseLocal
        h = hIn
        n1 = rmsNorm(h, L.attnNorm, c.rmsEps)
        q = linear(n1, L.qProj)
        k = linear(n1, L.kProj)
        v = linear(n1, L.vProj)
        if L.qNorm is not None:
            q = rmsNormHeads(q, L.qNorm, T, c.nHeads, c.headDim, c.rmsEps)
            k = rmsNormHeads(k, L.kNorm, T, c.nKVHeads, c.headDim, c.rmsEps)
        q = rope(q, T, c.nHeads, c.headDim, ropeB)
        k = rope(k, T, c.nKVHeads, c.headDim, ropeB)
        a = attention(q, k, v, T, c.nHeads, c.nKVHeads, c.headDim, window)
        attnOut = linear(a, L.oProj)
        if g3:
            attnOut = rmsNorm(attnOut, L.postAttnNorm, c.rmsEps)
        h = add(h, attnOut)
        n2 = rmsNorm(h, L.ffnNorm, c.rmsEps)
        g = gelu(linear(n2, L.gate)) if g3 else silu(linear(n2, L.gate))
        u = linear(n2, L.up)
        down = linear(mul(g, u), L.down)
        if g3:
            down = rmsNorm(down, L.postFfnNorm, c.rmsEps)
        return add(h, down)

    def forwardToReadout(self, ids):
        c = self.cfg
        T = len(ids)
        h = embedding(self.tokenEmbd, ids)
        if c.arch == "gemma3":
            h = scale(h, math.sqrt(c.hiddenSize))
        self.layerOutputs = []
        for il in range(c.nLayers):
            hIn = h
            h = checkpoint([hIn], (lambda hIn=hIn, il=il: self._block(hIn, il, T)))
            self.layerOutputs.append(h)
        hidden = rmsNorm(h, self.outputNorm, c.rmsEps)
        self.lastHidden = hidden
        return {"hidden": hidden, "readout": self.output if self.output is not None else self.tokenEmbd}

    def forward(self, ids) -> Tensor:
        r = self.forwardToReadout(ids)
        return linear(r["hidden"], r["readout"])


def buildModel(cfg: ModelConfig, seed: int) -> LanguageModel:
    """`arch.build(cfg, mulberry32(seed))` (src/commands/pretrain.ts:431-436 uses seed 1234)."""
    return LanguageModel(cfg, Mulberry32(seed))


def paramCount(cfg: ModelConfig) -> int:
    m = 0
    h, q, kv, f = cfg.hiddenSize, cfg.nHeads * cfg.headDim, cfg.nKVHeads * cfg.headDim, cfg.ffnDim
    per = q * h + 2 * kv * h + h * q + 3 * f * h + 2 * h
    if cfg.arch in ("qwen3", "gemma3"):
        per += 2 * cfg.headDim
    if cfg.arch == "gemma3":
        per += 2 * h
    m = cfg.vocabSize * h * (1 if cfg.tieEmbeddings else 2) + h + cfg.nLayers * per
    return m


# The configurations the benchmark and parity tests are quoted on.
def tinyLlama() -> ModelConfig:
    return ModelConfig("llama", 512, 128, 2, 4, 2, 32, 384, 10_000.0, 1e-5, init="n002")


def smolLM2_135M() -> ModelConfig:
    return ModelConfig("llama", 49152, 576, 30, 9, 3, 64, 1536, 100_000.0, 1e-5, init="n002")


def gemma3_95M() -> ModelConfig:
    return ModelConfig("gemma3", 32768, 640, 12, 4, 1, 256, 2048, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0,
                       slidingWindow=512, swaPattern=6, init="n002")


def qwen3_0_6B() -> ModelConfig:
    return ModelConfig("qwen3", 151936, 1024, 28, 16, 8, 128, 3072, 1_000_000.0, 1e-6, init="n002")
