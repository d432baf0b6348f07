"""Optimizer parity on a B200 (tests/gpu-parity.ts:974-1093): Newton-Schulz in every orientation, Muon
with momentum over two steps, AdamW over three steps with the clip triggering, and the .optstate
round trip through device buffers."""
import numpy as np
import pytest

from gpu_harness import compare

pytestmark = pytest.mark.gpu

from gguf_trainer_b200.autograd import Tensor
from gguf_trainer_b200.optim import (AdamWGpu, MuonGpu, deserializeOptState, newtonSchulzGpu, serializeOptState)


@pytest.fixture()
def gpu():
    from gguf_trainer_b200.backend import requireGPU
    g = requireGPU("the parity suite")
    yield g
    g.destroy()


@pytest.mark.parametrize("m,n", [(6, 10), (10, 6), (8, 8), (5, 7), (192, 576), (160, 96)])
def test_newton_schulz(gpu, oracle, m, n):
    G = oracle.Mulberry32(0x5EED).randn((m, n), 1.0)
    want = oracle.newton_schulz(G, 5)
    got = newtonSchulzGpu(gpu, G, m, n, 5)
    assert np.abs(got - want).max() < 2e-5   # the reference measures about 7e-7 on its shapes
    compare("newtonSchulz", got, want, dict(atol=2e-5, rtol=1e-4), 1e-5)


def _set_grad(gpu, p, g):
    gpu.writeStateBuffer(gpu.buffersFor(p)["grad"], g)


def test_adamw_three_steps_with_clip(gpu, oracle):
    rng = oracle.Mulberry32(0xABCD)
    shapes = [(7, 5), (33,), (20, 16)]
    ps = [Tensor(rng.randn(s, 0.5), list(s), True) for s in shapes]
    ref_w = [p.data.copy().reshape(s) for p, s in zip(ps, shapes)]
    ref_m = [np.zeros(s, np.float32) for s in shapes]
    ref_v = [np.zeros(s, np.float32) for s in shapes]
    opt = AdamWGpu(gpu, ps, lr=1e-2, beta1=0.9, beta2=0.95, weightDecay=0.1, clip=1.0)
    for t in range(1, 4):
        scale = [2.0, 0.01, 0.5][t - 1]   # norm above the clip at steps 1 and 3, below at step 2
        gs = [rng.randn(s, scale) for s in shapes]
        for p, g in zip(ps, gs):
            _set_grad(gpu, p, g)
        opt.recordStep()
        oracle.adamw_step_arrays(ref_w, [g.copy() for g in gs], ref_m, ref_v, t, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1.0)
    gpu.sync(ps)
    for p, w in zip(ps, ref_w):
        compare("adamw weight", p.data, w, dict(atol=1e-6, rtol=1e-5), 1e-6)
    st = opt.exportState()
    assert st["t"] == 3
    for a, b in zip(st["m"], ref_m):
        compare("adam m", a, b, dict(atol=1e-7, rtol=1e-5), 1e-6)
    for a, b in zip(st["v"], ref_v):
        compare("adam v", a, b, dict(atol=1e-9, rtol=1e-5), 1e-6)


@pytest.mark.parametrize("rows,cols", [(12, 20), (20, 12), (16, 16)])
def test_muon_two_steps_momentum(gpu, oracle, rows, cols):
    rng = oracle.Mulberry32(0x4D4D)
    p = Tensor(rng.randn((rows, cols), 0.5), [rows, cols], True)
    w = p.data.copy().reshape(rows, cols)
    buf = np.zeros((rows, cols), np.float32)
    opt = MuonGpu(gpu, [p], [], lr=0.05, momentum=0.95, nesterov=True, nsSteps=5, aux={"lr": 1e-3})
    for _ in range(2):
        g = rng.randn((rows, cols), 0.3)
        _set_grad(gpu, p, g)
        opt.recordStep()
        oracle.muon_step_array(w, g, buf, 0.05, 0.95, True, 5)
    gpu.sync([p])
    compare("muon weight", p.data, w, dict(atol=2e-5, rtol=1e-4), 1e-5)
    st = opt.exportState()
    compare("muon momentum", st["muonMomentum"][0], buf, dict(atol=1e-6, rtol=1e-5), 1e-6)


def test_optstate_round_trip_through_device(gpu, oracle):
    rng = oracle.Mulberry32(1)
    mp = [Tensor(rng.randn((6, 4), 0.5), [6, 4], True)]
    ap = [Tensor(rng.randn((9,), 0.5), [9], True), Tensor(rng.randn((3, 5), 0.5), [3, 5], True)]
    opt = MuonGpu(gpu, mp, ap, lr=0.02, aux={"lr": 1e-3})
    for p in mp + ap:
        _set_grad(gpu, p, rng.randn((p.size,), 0.1))
    opt.recordStep()
    s1 = opt.exportState()
    blob = serializeOptState(s1)
    opt2 = MuonGpu(gpu, [Tensor(t.data.copy(), t.shape, True) for t in mp], [Tensor(t.data.copy(), t.shape, True) for t in ap],
                   lr=0.02, aux={"lr": 1e-3})
    opt2.importState(deserializeOptState(blob))
    s2 = opt2.exportState()
    assert s2["adamT"] == s1["adamT"] == 1
    for k in ("muonMomentum", "adamM", "adamV"):
        for a, b in zip(s1[k], s2[k]):
            assert np.array_equal(a, b)
    assert serializeOptState(s2) == blob
