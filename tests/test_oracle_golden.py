"""Pins the CPU oracle to the reference's own known-answer tests (no GPU).

Every case restates a check from gguf-trainer's tests/gradcheck.ts or
tests/gpu-parity.ts: closed forms, identities and golden values that do not need
the TypeScript runtime to evaluate.
"""
import math

import numpy as np
import pytest


def _mulberry32_py(seed):
    """Independent restatement of src/model/autograd.ts:69-78 with Python ints."""
    a = seed & 0xFFFFFFFF

    def nxt():
        nonlocal a
        a = (a + 0x6D2B79F5) & 0xFFFFFFFF
        t = ((a ^ (a >> 15)) * (1 | a)) & 0xFFFFFFFF
        t = ((t + (((t ^ (t >> 7)) * (61 | t)) & 0xFFFFFFFF)) & 0xFFFFFFFF) ^ t
        return ((t ^ (t >> 14)) & 0xFFFFFFFF) / 4294967296

    return nxt


@pytest.mark.parametrize("seed", [0, 1, 7, 1234, 0xBEEF, 0xFFFFFFFF])
def test_mulberry32_matches_integer_restatement(oracle, seed):
    r = oracle.Mulberry32(seed)
    p = _mulberry32_py(seed)
    for _ in range(200):
        assert r() == p()


def test_randn_is_box_muller_of_the_stream(oracle):
    r = oracle.Mulberry32(1234)
    p = _mulberry32_py(1234)
    got = r.randn((64,), 0.8)
    for i in range(64):
        u = 0.0
        while u == 0:
            u = p()
        v = 0.0
        while v == 0:
            v = p()
        want = np.float32(math.sqrt(-2 * math.log(u)) * math.cos(2 * math.pi * v) * 0.8)
        assert got[i] == want


# tests/gradcheck.ts:321-330
@pytest.mark.parametrize("gap", [1, 10, 30, 60, 90])
def test_ce_closed_form_at_big_gaps(oracle, gap):
    row = np.array([[gap, 0, 0, -3]], np.float32)
    exact = math.log(math.exp(gap) + 2 + math.exp(-3)) + 3
    loss, _ = oracle.ce_fwd(row, [3])
    assert abs(float(loss) - exact) < 1e-4
    soft, _ = oracle.soft_ce(row, [3], [0.6], 1)
    assert abs(float(soft) - 0.6 * exact) < 1e-4


# tests/gradcheck.ts:692-723
def test_mean_times_kept_is_summed_nll(oracle):
    rng = oracle.Mulberry32(42)
    T, H, V = 7, 5, 23
    hid = rng.randn((T, H), 0.8)
    w = rng.randn((V, H), 0.8)
    targets = [-1, -1, -1, 4, 9, 2, 17]
    kept = 4
    logits = oracle.linear_fwd(hid, w)
    expected = 0.0
    for t in range(T):
        if targets[t] < 0:
            continue
        z = logits[t].astype(np.float64)
        mx = z.max()
        expected += math.log(np.exp(z - mx).sum()) + mx - z[targets[t]]
    loss, _ = oracle.ce_fwd(logits, targets)
    worst = abs(float(loss) * kept - expected)
    for chunk in (4, 8, 100):
        fl, _, _ = oracle.fused_ce(hid, w, targets, chunk)
        worst = max(worst, abs(float(fl) * kept - expected))
    assert worst < 1e-4


# tests/gradcheck.ts:742-768
def test_soft_ce_summed_nll(oracle):
    T, V, K = 4, 9, 2
    logits = oracle.Mulberry32(0x5F7A).randn((T, V), 0.8)
    ids = [1, 4, -1, 0, 7, 2, 3, 3]
    q = [0.6, 0.3, 0.0, 0.0, 0.5, 0.2, 0.25, 0.25]
    kept = 3
    expected = 0.0
    for t in range(T):
        if ids[t * K] < 0:
            continue
        z = logits[t].astype(np.float64)
        mx = z.max()
        s = np.exp(z - mx).sum()
        for j in range(K):
            wgt = float(np.float32(q[t * K + j]))
            if wgt == 0:
                continue
            expected += wgt * (math.log(s) + mx - z[ids[t * K + j]])
    loss, _ = oracle.soft_ce(logits, ids, q, K)
    assert abs(float(loss) * kept - expected) < 1e-4


# tests/gradcheck.ts:854-877
@pytest.mark.parametrize("chunk", [3, 8, 64])
def test_fused_ce_equals_dense(oracle, chunk):
    rng = oracle.Mulberry32(77)
    T, H, V = 6, 8, 19
    hid = rng.randn((T, H), 0.8)
    w = rng.randn((V, H), 0.8)
    targets = [3, -1, 18, 0, 7, -1]
    logits = oracle.linear_fwd(hid, w)
    loss, probs = oracle.ce_fwd(logits, targets)
    gl = oracle.ce_bwd(probs, targets, 1.0)
    gh, gw = oracle.linear_bwd(hid, w, gl)
    fl, fgh, fgw = oracle.fused_ce(hid, w, targets, chunk, loss_grad=1.0)
    assert abs(float(fl) - float(loss)) <= 1e-5
    assert np.abs(fgh - gh).max() <= 1e-5
    assert np.abs(fgw - gw).max() <= 1e-5


# tests/gpu-parity.ts:2419-2502
def test_all_ignored_batch_is_exactly_zero(oracle):
    rng = oracle.Mulberry32(5)
    logits = rng.randn((4, 11), 0.8)
    loss, probs = oracle.ce_fwd(logits, [-1] * 4)
    assert float(loss) == 0.0
    assert not oracle.ce_bwd(probs, [-1] * 4).any()
    fl, gh, gw = oracle.fused_ce(rng.randn((4, 6)), rng.randn((11, 6)), [-1] * 4, 4, loss_grad=1.0)
    assert float(fl) == 0.0 and not gh.any() and not gw.any()
    sl, g = oracle.soft_ce(logits, [-1, 0] * 4, [0.5, 0.5] * 4, 2, loss_grad=1.0)
    assert float(sl) == 0.0 and not g.any()


# tests/gradcheck.ts:1038-1051, tests/gpu-parity.ts:1163
def test_wsd_golden_values(oracle):
    got = [oracle.wsd(4, 3, 4, 0.1, s) for s in range(12)]
    want = [0.25, 0.5, 0.75, 1, 1, 1, 1, 0.775, 0.55, 0.325, 0.1, 0.1]
    assert np.allclose(got, want, atol=1e-6)
    assert oracle.wsd(0, 2, 2, 0.0, 0) == 1
    assert oracle.wsd(0, 2, 0, 0.0, 1) == 1 and oracle.wsd(0, 2, 0, 0.0, 2) == 0
    assert np.allclose([oracle.wsd(2, 0, 2, 0.1, s) for s in range(4)], [0.5, 1, 0.55, 0.1], atol=1e-9)


GEMMA_TINY = dict(arch="gemma3", vocab=13, hidden=8, layers=2, heads=2, kv_heads=1, head_dim=4, ffn=16,
                  rope_base=1_000_000, rope_base_local=10_000, eps=1e-6, window=16, swa_pattern=2, tie=True)


# tests/gradcheck.ts:1057-1108
def test_muonclip_lands_on_tau(oracle):
    m = oracle.Model(GEMMA_TINY, 99)
    names = [m.info(i) for i in range(m.nparams())]
    # gemma3 params(): tokenEmbd, outputNorm, then 13 per layer; qNorm/kNorm are slots 5 and 6
    q0, k0 = m.data(2 + 5), m.data(2 + 6)
    assert names[2 + 5]["shape"] == (4,)
    assert abs(oracle.qk_logit_scale(q0, k0, 4) - 1) < 1e-6
    q0[:] = 3
    k0[:] = 2
    before = oracle.qk_logit_scale(q0, k0, 4)
    assert abs(before - 6) < 1e-6
    qb, kb = q0.copy(), k0.copy()
    assert m.qk_clip(0.5) == 2
    assert abs(oracle.qk_logit_scale(q0, k0, 4) - 0.5) < 1e-6
    f = math.sqrt(0.5 / before)
    assert np.allclose(q0, qb * f, atol=1e-6) and np.allclose(k0, kb * f, atol=1e-6)
    m.qk_clip(0.5)
    assert oracle.qk_logit_scale(q0, k0, 4) <= 0.5 + 1e-6


LLAMA_TINY = dict(arch="llama", vocab=23, hidden=8, layers=2, heads=2, kv_heads=1, head_dim=4, ffn=16,
                  rope_base=100_000, eps=1e-5, tie=True)
QWEN_TINY = dict(arch="qwen3", vocab=23, hidden=8, layers=2, heads=2, kv_heads=1, head_dim=4, ffn=16,
                 rope_base=1_000_000, eps=1e-6, tie=True)
GEMMA_T23 = dict(GEMMA_TINY, vocab=23, window=4)


# tests/gradcheck.ts:786-806 (checkpoint on == off, bit-exact)
@pytest.mark.parametrize("cfg", [LLAMA_TINY, QWEN_TINY, GEMMA_T23], ids=lambda c: c["arch"])
def test_checkpoint_is_bit_exact(oracle, cfg):
    ids = oracle.Mulberry32(3).randint(9, cfg["vocab"])
    tg = oracle.Mulberry32(4).randint(9, cfg["vocab"])
    outs = []
    for on in (False, True):
        oracle.set_checkpointing(on)
        m = oracle.Model(cfg, 1234)
        loss = m.loss_backward(ids, tg)
        outs.append((loss, [m.grad(i).copy() for i in range(m.nparams())]))
        m.close()
    oracle.set_checkpointing(False)
    assert outs[0][0] == outs[1][0]
    for a, b in zip(outs[0][1], outs[1][1]):
        assert np.array_equal(a, b)


# tests/gradcheck.ts:53-55, 919-992 (directional finite difference on the whole model)
@pytest.mark.parametrize("cfg", [LLAMA_TINY, QWEN_TINY, GEMMA_T23], ids=lambda c: c["arch"])
@pytest.mark.parametrize("chunk", [0, 5])
def test_model_directional_finite_difference(oracle, cfg, chunk):
    ids = oracle.Mulberry32(3).randint(9, cfg["vocab"])
    tg = oracle.Mulberry32(4).randint(9, cfg["vocab"])
    m = oracle.Model(cfg, 1234)
    m.loss_backward(ids, tg, loss_chunk=chunk)
    n = m.nparams()
    dir_rng = oracle.Mulberry32(777)
    base = [m.data(i).copy() for i in range(n)]
    fails = 0
    for _trial in range(4):
        dirs = [dir_rng.randn(m.info(i)["shape"], 1.0).astype(np.float64) for i in range(n)]
        norm = math.sqrt(sum(float((d * d).sum()) for d in dirs))
        dirs = [d / norm for d in dirs]
        dot = sum(float((m.grad(i).astype(np.float64) * dirs[i]).sum()) for i in range(n))
        eps = 2e-3

        def loss_at(sign):
            for i in range(n):
                m.data(i)[...] = (base[i] + sign * eps * dirs[i]).astype(np.float32)
            return float(m.loss_backward(ids, tg, loss_chunk=chunk, seed=0.0))

        fd = (loss_at(1) - loss_at(-1)) / (2 * eps)
        rel = abs(fd - dot) / max(abs(fd), abs(dot), 1e-12)
        if rel > 5e-2 and abs(fd - dot) > 1e-3:
            fails += 1
    assert fails == 0


def test_op_finite_difference(oracle):
    """Per-op FD on the ops with closed backward formulas (tests/gradcheck.ts:174-247)."""
    rng = oracle.Mulberry32(2024)
    T, Hq, Hkv, hd = 6, 4, 2, 4
    q = rng.randn((T, Hq * hd), 0.8); k = rng.randn((T, Hkv * hd), 0.8); v = rng.randn((T, Hkv * hd), 0.8)
    up = rng.uniform_pm1((T, Hq * hd))
    for window in (0, 3):
        out, probs = oracle.attention_fwd(q, k, v, T, Hq, Hkv, hd, window)
        gq, gk, gv = oracle.attention_bwd(q, k, v, probs, up, T, Hq, Hkv, hd, window)
        eps = 1e-2
        for arr, g in ((q, gq), (k, gk), (v, gv)):
            for idx in [(0, 1), (3, 5), (5, 7)]:
                a2 = arr.copy(); a2[idx] += eps
                a3 = arr.copy(); a3[idx] -= eps
                args = lambda z: (z if arr is q else q, z if arr is k else k, z if arr is v else v)
                f1 = (oracle.attention_fwd(*args(a2), T, Hq, Hkv, hd, window)[0].astype(np.float64) * up).sum()
                f0 = (oracle.attention_fwd(*args(a3), T, Hq, Hkv, hd, window)[0].astype(np.float64) * up).sum()
                fd = (f1 - f0) / (2 * eps)
                assert abs(fd - g[idx]) <= 2e-3 + 1.5e-2 * max(abs(fd), abs(g[idx]))
    # rmsNorm
    x = rng.randn((5, 7), 0.8); w = (1 + 0.3 * rng.randn((7,), 1.0)).astype(np.float32)
    upn = rng.uniform_pm1((5, 7))
    y, rinv = oracle.rmsnorm_fwd(x, w, 1e-6)
    gx, gw = oracle.rmsnorm_bwd(x, w, rinv, upn)
    for idx in [(0, 0), (2, 3), (4, 6)]:
        a2 = x.copy(); a2[idx] += 1e-2
        a3 = x.copy(); a3[idx] -= 1e-2
        fd = ((oracle.rmsnorm_fwd(a2, w, 1e-6)[0].astype(np.float64) * upn).sum()
              - (oracle.rmsnorm_fwd(a3, w, 1e-6)[0].astype(np.float64) * upn).sum()) / 2e-2
        assert abs(fd - gx[idx]) <= 2e-3 + 1.5e-2 * max(abs(fd), abs(gx[idx]))
    # silu / gelu
    for op in ("silu", "gelu"):
        xv = rng.randn((35,), 1.5)
        _, ga, _ = oracle.elementwise(op, xv, gy=np.ones(35, np.float32))
        fp = oracle.elementwise(op, xv + np.float32(1e-2))[0].astype(np.float64)
        fm = oracle.elementwise(op, xv - np.float32(1e-2))[0].astype(np.float64)
        fd = (fp - fm) / 2e-2
        assert np.all(np.abs(fd - ga) <= 2e-3 + 1.5e-2 * np.maximum(np.abs(fd), np.abs(ga)))


def test_newton_schulz_orthogonalises(oracle):
    """Five quintic iterations push singular values into the band the coefficients target
    (src/train/muon.ts:26-29); both orientations and a square case."""
    rng = oracle.Mulberry32(0x5EED)
    for m, n in ((6, 10), (10, 6), (8, 8), (5, 7)):
        G = rng.randn((m, n), 1.0)
        X = oracle.newton_schulz(G, 5)
        s = np.linalg.svd(X.astype(np.float64), compute_uv=False)
        assert s.max() < 1.3 and s.min() > 0.3
        # zero steps = plain Frobenius normalisation
        X0 = oracle.newton_schulz(G, 0)
        assert np.allclose(X0, G / (np.linalg.norm(G.astype(np.float64)) + 1e-7), atol=1e-7)


def test_adamw_matches_closed_form_first_step(oracle):
    """At t=1 with wd=0 and no clip, update = g/(|g|+eps) (src/train/adam.ts:64-81)."""
    rng = oracle.Mulberry32(0xABCD)
    w = rng.randn((3, 5), 1.0); g = rng.randn((3, 5), 0.01)
    m = np.zeros_like(w); v = np.zeros_like(w)
    w0 = w.copy()
    oracle.adamw_step_arrays([w], [g.copy()], [m], [v], 1, 1e-3, clip=0.0)
    want = w0 - 1e-3 * g / (np.abs(g) + 1e-8)
    assert np.allclose(w, want, atol=1e-7)
    # clip triggers: norm > clip scales the gradient itself
    g2 = rng.randn((3, 5), 2.0)
    gin = g2.copy()
    oracle.adamw_step_arrays([w], [gin], [m], [v], 2, 1e-3, clip=1.0)
    nrm = np.linalg.norm(g2.astype(np.float64))
    assert np.allclose(gin, g2 * (1.0 / (nrm + 1e-12)), atol=1e-6)
