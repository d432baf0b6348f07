"""Shared pieces of the GPU parity tests: the `opCase` harness of the reference's
tests/gpu-parity.ts:90-126 (same random upstream gradient from mulberry32(0xbeef) on both sides),
its element tolerances, and the relative-L2 bound this backend states for its strict-f32 mode."""
import numpy as np

from gguf_trainer_b200.autograd import Tensor

FWD = dict(atol=2e-4, rtol=2e-3)   # tests/gpu-parity.ts:55-56
BWD = dict(atol=1e-3, rtol=1e-2)
REL_L2_FP32 = 1e-5                 # strict-f32 mode
REL_L2_TC = 2e-3                   # TF32 / BF16 tensor-core modes


def rel_l2(got, want):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    den = np.linalg.norm(want)
    if den == 0:
        return float(np.linalg.norm(got))
    return float(np.linalg.norm(got - want) / den)


def compare(label, got, want, tol, l2=REL_L2_FP32):
    got = np.asarray(got, np.float32).ravel()
    want = np.asarray(want, np.float32).ravel()
    assert got.shape == want.shape, f"{label}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{label}: non-finite values"
    err = np.abs(got - want)
    bound = tol["atol"] + tol["rtol"] * np.maximum(np.abs(got), np.abs(want))
    bad = np.nonzero(err > bound)[0]
    assert bad.size == 0, f"MISMATCH {label}[{bad[0]}]: gpu={got[bad[0]]} ref={want[bad[0]]}"
    if l2 is not None:
        r = rel_l2(got, want)
        assert r <= l2, f"{label}: relative L2 {r:.3e} > {l2:.1e}"


def rand_tensor(rng, shape, scale=0.8, requires_grad=True):
    """tests/gpu-parity.ts:60-64 randTensor, drawing from an oracle Mulberry32."""
    return Tensor(rng.randn(tuple(shape), scale), shape, requires_grad)


def upstream(oracle, n):
    """tests/gpu-parity.ts:103-105: 1 for a scalar, else rng()*2-1 from mulberry32(0xbeef)."""
    if n == 1:
        return np.ones(1, np.float32)
    return oracle.Mulberry32(0xBEEF).uniform_pm1((n,))


def op_case(gpu, oracle, name, inputs, fwd, ref, l2=REL_L2_FP32, fwd_tol=FWD, bwd_tol=BWD):
    """Run `fwd()` through the installed backend, seed the output gradient, run that op's backward
    closure, sync, and compare output and input gradients with `ref(upstream) -> (out, [grads])`."""
    for t in inputs:
        t.zeroGrad()
    gpu.install()
    try:
        out = fwd()
        r = upstream(oracle, out.size)
        out.grad[:] = r
        if out.size > 1:
            gpu.seedGradFromHost(out)
        out._backward()
        gpu.sync([out])
    finally:
        gpu.uninstall()
    ref_out, ref_grads = ref(r)
    compare(f"{name}.out", out.data, ref_out, fwd_tol, l2)
    for k, (t, g) in enumerate(zip(inputs, ref_grads)):
        if g is None:
            continue
        compare(f"{name}.dInput{k}", t.grad, g, bwd_tol, l2)
    return out
