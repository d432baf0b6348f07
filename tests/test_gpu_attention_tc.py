"""Tensor-core (tcgen05, TF32) attention through the op interface against the CPU oracle: head dims 32/64/128 and
256 (the last as pairs of CTAs holding half a head each), GQA groups, sliding windows, ragged sequence lengths,
batched sequences. Bound: relative L2 <= 2e-3."""
import numpy as np
import pytest

from gpu_harness import REL_L2_TC, rand_tensor, rel_l2, upstream

pytestmark = pytest.mark.gpu

from gguf_trainer_b200 import autograd as ag


@pytest.fixture(scope="module")
def gpu():
    from gguf_trainer_b200.backend import requireGPU
    g = requireGPU("the tensor-core suite", precision="tf32")
    yield g
    g.destroy()


CASES = [(64, 2, 1, 64, 0), (130, 4, 2, 64, 0), (193, 4, 1, 32, 0), (300, 9, 3, 64, 0), (257, 4, 2, 128, 0),
         (200, 4, 2, 64, 33), (300, 2, 1, 32, 100), (513, 2, 2, 64, 512), (640, 3, 1, 128, 70),
         (64, 1, 1, 256, 0), (257, 4, 1, 256, 0), (300, 4, 2, 256, 100), (640, 2, 1, 256, 512)]


@pytest.mark.parametrize("T,Hq,Hkv,hd,window", CASES)
def test_attention_tf32(gpu, oracle, T, Hq, Hkv, hd, window):
    rng = oracle.Mulberry32(T + hd)
    q = rand_tensor(rng, [T, Hq * hd]); k = rand_tensor(rng, [T, Hkv * hd]); v = rand_tensor(rng, [T, Hkv * hd])
    for t in (q, k, v):
        t.zeroGrad()
    launches = gpu.kernelLaunches()
    gpu.install()
    try:
        out = ag.attention(q, k, v, T, Hq, Hkv, hd, window)
        r = upstream(oracle, out.size)
        out.grad[:] = r
        gpu.seedGradFromHost(out)
        out._backward()
        gpu.sync([out])
    finally:
        gpu.uninstall()
    assert gpu.kernelLaunches() > launches
    ref_out, probs = oracle.attention_fwd(q.data, k.data, v.data, T, Hq, Hkv, hd, window)
    gq, gk, gv = oracle.attention_bwd(q.data, k.data, v.data, probs, r, T, Hq, Hkv, hd, window)
    assert np.isfinite(out.data).all()
    e = rel_l2(out.data, ref_out)
    assert e <= REL_L2_TC, f"out: relative L2 {e:.3e}"
    for name, got, want in (("dq", q.grad, gq), ("dk", k.grad, gk), ("dv", v.grad, gv)):
        assert np.isfinite(got).all()
        e = rel_l2(got, want)
        assert e <= REL_L2_TC, f"{name}: relative L2 {e:.3e}"


@pytest.mark.parametrize("B,T,Hq,Hkv,hd", [(3, 150, 4, 2, 64), (2, 150, 2, 1, 256)])
def test_attention_tf32_batched_sequences_do_not_see_each_other(gpu, oracle, B, T, Hq, Hkv, hd):
    rng = oracle.Mulberry32(9)
    q = rand_tensor(rng, [B * T, Hq * hd]); k = rand_tensor(rng, [B * T, Hkv * hd]); v = rand_tensor(rng, [B * T, Hkv * hd])
    gpu.install()
    gpu.setBatch(B, T)
    try:
        out = ag.attention(q, k, v, B * T, Hq, Hkv, hd, 0)
        r = upstream(oracle, out.size)
        out.grad[:] = r
        gpu.seedGradFromHost(out)
        out._backward()
        gpu.sync([out])
    finally:
        gpu.setBatch(0)
        gpu.uninstall()
    Q, K, V = (t.data.reshape(B, T, -1) for t in (q, k, v))
    R = r.reshape(B, T, -1)
    for b in range(B):
        ref_out, probs = oracle.attention_fwd(Q[b], K[b], V[b], T, Hq, Hkv, hd, 0)
        gq, gk, gv = oracle.attention_bwd(Q[b], K[b], V[b], probs, R[b], T, Hq, Hkv, hd, 0)
        assert rel_l2(out.data.reshape(B, T, -1)[b], ref_out) <= REL_L2_TC
        for got, want in ((q.grad, gq), (k.grad, gk), (v.grad, gv)):
            assert rel_l2(got.reshape(B, T, -1)[b], want) <= REL_L2_TC
