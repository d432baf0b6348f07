"""Per-op parity of the CUDA backend against the CPU oracle, through the C ABI, on a B200.
Cases follow the reference's tests/gpu-parity.ts (shapes, seeds, tolerances); strict-f32 mode."""
import numpy as np
import pytest

from gpu_harness import BWD, FWD, REL_L2_FP32, compare, op_case, rand_tensor, rel_l2

pytestmark = pytest.mark.gpu

from gguf_trainer_b200 import autograd as ag
from gguf_trainer_b200.autograd import Tensor


@pytest.fixture(scope="module")
def gpu():
    from gguf_trainer_b200.backend import requireGPU
    g = requireGPU("the parity suite")
    yield g
    g.destroy()


# tests/gpu-parity.ts:654-672 plus config-scale shapes
@pytest.mark.parametrize("T,i,o", [(5, 7, 6), (33, 48, 37), (70, 83, 75), (256, 576, 192), (300, 1536, 576)])
def test_linear(gpu, oracle, T, i, o):
    rng = oracle.Mulberry32(1234)
    x = rand_tensor(rng, [T, i]); w = rand_tensor(rng, [o, i])

    def ref(r):
        X, W = x.data.reshape(T, i), w.data.reshape(o, i)
        y = oracle.linear_fwd(X, W)
        gx, gw = oracle.linear_bwd(X, W, r.reshape(T, o))
        return y, [gx, gw]

    op_case(gpu, oracle, f"linear {T}x{i}.{o}x{i}T", [x, w], lambda: ag.linear(x, w), ref)


def test_linear_frozen_weight_skips_dw(gpu, oracle):
    rng = oracle.Mulberry32(8)
    x = rand_tensor(rng, [9, 12]); w = rand_tensor(rng, [7, 12], requires_grad=False)

    def ref(r):
        X, W = x.data.reshape(9, 12), w.data.reshape(7, 12)
        gx, _ = oracle.linear_bwd(X, W, r.reshape(9, 7), want_dw=False)
        return oracle.linear_fwd(X, W), [gx, None]

    op_case(gpu, oracle, "linear frozen", [x, w], lambda: ag.linear(x, w), ref)
    assert not w.grad.any()


@pytest.mark.parametrize("op", ["add", "mul", "silu", "gelu", "scale"])
@pytest.mark.parametrize("shape", [(4, 6), (5, 7), (129, 515)])
def test_elementwise(gpu, oracle, op, shape):
    rng = oracle.Mulberry32(99)
    sc = 1.5 if op in ("silu", "gelu") else 0.8
    a = rand_tensor(rng, shape, sc)
    b = rand_tensor(rng, shape, sc) if op in ("add", "mul") else None
    c = 0.37

    def ref(r):
        out, ga, gb = oracle.elementwise(op, a.data, None if b is None else b.data, c, r)
        return out, [ga] + ([gb] if b is not None else [])

    f = {"add": lambda: ag.add(a, b), "mul": lambda: ag.mul(a, b), "silu": lambda: ag.silu(a),
         "gelu": lambda: ag.gelu(a), "scale": lambda: ag.scale(a, c)}[op]
    op_case(gpu, oracle, op, [a] + ([b] if b is not None else []), f, ref)


# tests/gpu-parity.ts:2166-2173: the same tensor on both sides
@pytest.mark.parametrize("op", ["add", "mul"])
def test_aliased_binary(gpu, oracle, op):
    rng = oracle.Mulberry32(5)
    t = rand_tensor(rng, [6, 10])

    def ref(r):
        out, ga, gb = oracle.elementwise(op, t.data, t.data, 0.0, r)
        return out, [ga + gb]

    op_case(gpu, oracle, f"{op}(t,t)", [t], (lambda: ag.add(t, t)) if op == "add" else (lambda: ag.mul(t, t)), ref)


@pytest.mark.parametrize("T,d", [(5, 7), (64, 576), (33, 640), (17, 1024), (3, 1500)])
def test_rmsnorm(gpu, oracle, T, d):
    rng = oracle.Mulberry32(21)
    x = rand_tensor(rng, [T, d])
    w = Tensor((1 + 0.3 * rng.randn((d,), 1.0)).astype(np.float32), [d], True)

    def ref(r):
        y, rinv = oracle.rmsnorm_fwd(x.data.reshape(T, d), w.data, 1e-6)
        gx, gw = oracle.rmsnorm_bwd(x.data.reshape(T, d), w.data, rinv, r.reshape(T, d))
        return y, [gx, gw]

    op_case(gpu, oracle, f"rmsNorm {T}x{d}", [x, w], lambda: ag.rmsNorm(x, w, 1e-6), ref)


# tests/gpu-parity.ts:690-702 uses rows = 65600 to cross a dispatch limit; kept as a many-rows case
@pytest.mark.parametrize("T,H,hd", [(6, 3, 8), (8200, 8, 4), (40, 4, 256), (50, 16, 128), (37, 9, 64)])
def test_rmsnorm_heads(gpu, oracle, T, H, hd):
    rng = oracle.Mulberry32(22)
    x = rand_tensor(rng, [T, H * hd])
    w = Tensor((1 + 0.3 * rng.randn((hd,), 1.0)).astype(np.float32), [hd], True)

    def ref(r):
        y, rinv = oracle.rmsnorm_fwd(x.data, w.data, 1e-6)
        gx, gw = oracle.rmsnorm_bwd(x.data, w.data, rinv, r)
        return y, [gx, gw]

    op_case(gpu, oracle, f"rmsNormHeads {T}x{H}x{hd}", [x, w], lambda: ag.rmsNormHeads(x, w, T, H, hd, 1e-6), ref)


def test_embedding_is_bit_exact_gather_and_scatter_adds_duplicates(gpu, oracle):
    rng = oracle.Mulberry32(31)
    V, d, T = 50, 24, 40
    w = rand_tensor(rng, [V, d])
    ids = oracle.Mulberry32(32).randint(T, 7)  # heavy duplicates

    def ref(r):
        return oracle.embedding_fwd(w.data.reshape(V, d), ids), [oracle.embedding_bwd(r.reshape(T, d), ids, V)]

    out = op_case(gpu, oracle, "embedding", [w], lambda: ag.embedding(w, ids), ref)
    assert np.array_equal(out.data.reshape(T, d), w.data.reshape(V, d)[ids])  # gather is bit-exact


@pytest.mark.parametrize("T,H,hd,base,off", [(7, 2, 8, 10_000.0, 0), (130, 9, 64, 100_000.0, 0),
                                            (33, 4, 256, 1_000_000.0, 5), (2048, 1, 32, 10_000.0, 0), (5, 3, 12, 10_000.0, 2)])
def test_rope(gpu, oracle, T, H, hd, base, off):
    rng = oracle.Mulberry32(41)
    x = rand_tensor(rng, [T, H * hd])

    def ref(r):
        return oracle.rope_fwd(x.data, T, H, hd, base, off), [oracle.rope_bwd(r, T, H, hd, base, off)]

    op_case(gpu, oracle, f"rope T{T} hd{hd}", [x], lambda: ag.rope(x, T, H, hd, base, off), ref)


# tests/gpu-parity.ts:872-930: T=67/130/193, hd 6/12/24/32/64, GQA groups 1/2/4, sliding windows
ATTN = [(9, 4, 2, 8, 0), (67, 2, 2, 6, 0), (130, 4, 2, 12, 0), (193, 4, 1, 24, 0), (67, 4, 2, 32, 0), (130, 2, 1, 64, 0),
        (40, 4, 1, 256, 0), (70, 16, 8, 128, 0), (67, 4, 2, 8, 16), (130, 4, 2, 32, 64), (193, 2, 1, 64, 33),
        (300, 9, 3, 64, 0)]


@pytest.mark.parametrize("T,Hq,Hkv,hd,window", ATTN)
def test_attention(gpu, oracle, T, Hq, Hkv, hd, window):
    rng = oracle.Mulberry32(51)
    q = rand_tensor(rng, [T, Hq * hd]); k = rand_tensor(rng, [T, Hkv * hd]); v = rand_tensor(rng, [T, Hkv * hd])

    def ref(r):
        out, probs = oracle.attention_fwd(q.data, k.data, v.data, T, Hq, Hkv, hd, window)
        gq, gk, gv = oracle.attention_bwd(q.data, k.data, v.data, probs, r, T, Hq, Hkv, hd, window)
        return out, [gq, gk, gv]

    op_case(gpu, oracle, f"attention T{T} {Hq}/{Hkv} hd{hd} w{window}", [q, k, v],
            lambda: ag.attention(q, k, v, T, Hq, Hkv, hd, window), ref)


@pytest.mark.parametrize("T,V", [(7, 23), (33, 512), (5, 49152), (64, 1000)])
def test_cross_entropy(gpu, oracle, T, V):
    rng = oracle.Mulberry32(61)
    logits = rand_tensor(rng, [T, V], 2.0)
    targets = oracle.Mulberry32(62).randint(T, V)
    targets[::3] = -1

    def ref(r):
        loss, probs = oracle.ce_fwd(logits.data.reshape(T, V), targets)
        return [loss], [oracle.ce_bwd(probs, targets, 1.0)]

    op_case(gpu, oracle, f"crossEntropy {T}x{V}", [logits], lambda: ag.crossEntropy(logits, targets), ref)


# tests/gradcheck.ts:321-330 on the device
@pytest.mark.parametrize("gap", [1, 10, 30, 60, 90])
def test_ce_closed_form_on_device(gpu, gap):
    import math
    logits = Tensor(np.array([gap, 0, 0, -3], np.float32), [1, 4], True)
    gpu.install()
    try:
        loss = ag.crossEntropy(logits, [3])
        soft = ag.softCrossEntropy(logits, [3], [0.6], 1)
        gpu.sync([loss, soft])
    finally:
        gpu.uninstall()
    exact = math.log(math.exp(gap) + 2 + math.exp(-3)) + 3
    assert abs(float(loss.data[0]) - exact) < 1e-4
    assert abs(float(soft.data[0]) - 0.6 * exact) < 1e-4


# tests/gpu-parity.ts:2419-2502: an all-ignored batch is exactly 0, not NaN
def test_all_ignored_is_exactly_zero(gpu, oracle):
    rng = oracle.Mulberry32(71)
    logits = rand_tensor(rng, [4, 11]); hid = rand_tensor(rng, [4, 6]); w = rand_tensor(rng, [11, 6])
    gpu.install()
    try:
        l1 = ag.crossEntropy(logits, [-1] * 4)
        l2 = ag.fusedCrossEntropy(hid, w, [-1] * 4, 4)
        l3 = ag.softCrossEntropy(logits, [-1, 0] * 4, [0.5, 0.5] * 4, 2)
        for l in (l1, l2, l3):
            ag.backward(l, 1.0)
        gpu.sync([l1, l2, l3])
    finally:
        gpu.uninstall()
    for l in (l1, l2, l3):
        assert float(l.data[0]) == 0.0
    for t in (logits, hid, w):
        assert not t.grad.any() and np.isfinite(t.grad).all()


# tests/gpu-parity.ts:174-207: four shapes including a ragged last chunk
@pytest.mark.parametrize("T,H,V,chunk", [(7, 5, 23, 8), (130, 32, 200, 70), (16, 64, 512, 512), (33, 48, 300, 7)])
def test_fused_cross_entropy(gpu, oracle, T, H, V, chunk):
    rng = oracle.Mulberry32(81)
    hid = rand_tensor(rng, [T, H]); w = rand_tensor(rng, [V, H], 0.3)
    targets = oracle.Mulberry32(82).randint(T, V)
    targets[1::4] = -1

    def ref(r):
        loss, gh, gw = oracle.fused_ce(hid.data.reshape(T, H), w.data.reshape(V, H), targets, chunk, loss_grad=1.0)
        return [loss], [gh, gw]

    op_case(gpu, oracle, f"fusedCE {T}x{H}x{V}/{chunk}", [hid, w], lambda: ag.fusedCrossEntropy(hid, w, targets, chunk), ref)


def test_soft_cross_entropy(gpu, oracle):
    T, V, K = 6, 19, 3
    logits = rand_tensor(oracle.Mulberry32(91), [T, V], 1.5)
    idr = oracle.Mulberry32(92)
    ids = idr.randint(T * K, V)
    ids[K * 2] = -1  # row 2 ignored
    q = np.abs(oracle.Mulberry32(93).uniform_pm1((T * K,))).astype(np.float32) / K
    q[K * 4 + 1] = 0.0  # a pad inside a kept row

    def ref(r):
        loss, g = oracle.soft_ce(logits.data.reshape(T, V), ids, q, K, loss_grad=1.0)
        return [loss], [g]

    op_case(gpu, oracle, "softCE", [logits], lambda: ag.softCrossEntropy(logits, list(ids), list(q), K), ref)


# tests/gpu-parity.ts:2203-2290: malformed inputs are refused above the dispatch with a backend installed
def test_refusals_happen_above_the_dispatch(gpu, oracle):
    rng = oracle.Mulberry32(3)
    w = rand_tensor(rng, [4, 3]); logits = rand_tensor(rng, [3, 6])
    launches = gpu.kernelLaunches()
    gpu.install()
    try:
        with pytest.raises(ValueError, match=r"embedding: id 6 at position 1 is not an integer in \[0,4\)"):
            ag.embedding(w, [0, 6])
        with pytest.raises(ValueError, match=r"crossEntropy: target 6 at position 2"):
            ag.crossEntropy(logits, [0, -1, 6])
        with pytest.raises(ValueError, match=r"crossEntropy: 2 targets for 3 logit rows"):
            ag.crossEntropy(logits, [0, 1])
        with pytest.raises(ValueError, match=r"target -2 at position 0"):
            ag.crossEntropy(logits, [-2, 1, 1])
        with pytest.raises(ValueError, match="linear dim mismatch"):
            ag.linear(logits, w)
        with pytest.raises(ValueError, match="fusedCrossEntropy chunk must be positive"):
            ag.fusedCrossEntropy(rand_tensor(rng, [3, 3]), w, [0, 1, 2], 0)
        with pytest.raises(ValueError, match=r"teacher id 9 at slot 1 of row 0"):
            ag.softCrossEntropy(logits, [0, 9, 1, 1, 2, 2], [0.5] * 6, 2)
    finally:
        gpu.uninstall()
    assert gpu.kernelLaunches() == launches


def test_backward_after_sync_is_refused(gpu, oracle):
    """tests/gpu-parity.ts:1848,1892."""
    rng = oracle.Mulberry32(4)
    x = rand_tensor(rng, [4, 5]); w = rand_tensor(rng, [3, 5])
    gpu.install()
    try:
        y = ag.linear(x, w)
        gpu.sync([y])
        with pytest.raises(RuntimeError, match="graph built before a sync"):
            y._backward()
    finally:
        gpu.uninstall()


def test_gemm_is_deterministic_run_to_run(gpu, oracle):
    rng = oracle.Mulberry32(1234)
    x = rand_tensor(rng, [70, 83]); w = rand_tensor(rng, [75, 83])
    outs = []
    for _ in range(2):
        gpu.install()
        try:
            y = ag.linear(x, w)
            gpu.sync([y])
        finally:
            gpu.uninstall()
        outs.append(y.data.copy())
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("kind", ["NT", "NN", "TN"])
def test_gemm_scaled_and_gemm2_strict_f32(gpu, oracle, kind):
    """The two extra product entry points in strict-f32 mode: C (+)= alpha*A.B and C (+)= A.B + A2.B2, ragged sizes,
    against f64 products of the same f32 inputs (relative L2 <= 1e-5); and their argument checks."""
    from gguf_trainer_b200._lib import GtError
    M, N, K, K2, alpha = 37, 29, 53, 8, 0.75
    rng = oracle.Mulberry32(99)
    A, B = rng.randn((M, K), 0.5), rng.randn((N, K), 0.5)
    A2, B2 = rng.randn((M, K2), 0.5), rng.randn((N, K2), 0.5)
    C0 = rng.randn((M, N), 0.5)
    sa = (lambda X: X if kind != "TN" else np.ascontiguousarray(X.T))
    sb = (lambda X: X if kind == "NT" else np.ascontiguousarray(X.T))
    kinds = {"NT": 0, "NN": 1, "TN": 2}

    def dev(a):
        b = gpu.createStateBuffer(a.nbytes)
        gpu.writeStateBuffer(b, a)
        return b

    da, db, da2, db2 = dev(sa(A)), dev(sb(B)), dev(sa(A2)), dev(sb(B2))
    AB = A.astype(np.float64) @ B.astype(np.float64).T
    AB2 = A2.astype(np.float64) @ B2.astype(np.float64).T
    for accum in (0, 1):
        base = C0.astype(np.float64) if accum else 0.0
        dc = dev(C0)
        gpu._check(gpu.lib.gt_gemm_scaled(gpu.ctx, kinds[kind], accum, M, N, K, da, db, dc, alpha))
        assert rel_l2(gpu.readStateBuffer(dc, M * N).reshape(M, N), alpha * AB + base) <= REL_L2_FP32
        gpu.writeStateBuffer(dc, C0)
        gpu._check(gpu.lib.gt_gemm2(gpu.ctx, kinds[kind], accum, M, N, K, da, db, K2, da2, db2, dc))
        assert rel_l2(gpu.readStateBuffer(dc, M * N).reshape(M, N), AB + AB2 + base) <= REL_L2_FP32
        gpu._check(gpu.lib.gt_free(gpu.ctx, dc))
    dc = dev(C0)
    with pytest.raises(GtError, match="empty product"):
        gpu._check(gpu.lib.gt_gemm2(gpu.ctx, kinds[kind], 0, M, N, K, da, db, 0, da2, db2, dc))
    with pytest.raises(GtError, match="null operand"):
        gpu._check(gpu.lib.gt_gemm2(gpu.ctx, kinds[kind], 0, M, N, K, da, db, K2, 0, db2, dc))
    gpu.sync([])
    for b in (da, db, da2, db2, dc):
        gpu._check(gpu.lib.gt_free(gpu.ctx, b))


def test_residual_add_feeding_a_norm_is_one_kernel_and_its_backward_copies_nothing(gpu, oracle):
    """`n = rmsNorm(add(a, b), w)`, the residual connection of every block (src/arch/llama.ts:203-208): the forward is
    one launch that writes the sum and the normalised row; in backward the `add` hands its upstream gradient to both
    inputs without a copy kernel (readers read it in place; a second writer would add on top of it). Values equal the
    two reference ops."""
    rng = oracle.Mulberry32(71)
    T, d = 37, 96
    a = rand_tensor(rng, [T, d]); b = rand_tensor(rng, [T, d]); w = rand_tensor(rng, [d], 0.5)
    for t in (a, b, w):
        t.zeroGrad()
    up = oracle.Mulberry32(0xBEEF).uniform_pm1((T * d,))
    up2 = oracle.Mulberry32(0xF00D).uniform_pm1((T * d,))
    gpu.install()
    try:
        gpu.sync([])
        l0 = gpu.kernelLaunches()
        s = ag.add(a, b)
        n = ag.rmsNorm(s, w, 1e-5)
        assert gpu.kernelLaunches() - l0 == 1
        z = ag.add(s, n)                       # the sum has a second consumer, like the residual stream
        z.grad[:] = up
        gpu.seedGradFromHost(z)
        l1 = gpu.kernelLaunches()
        z._backward()                          # add: s and n take the upstream gradient as views
        n._backward()                          # norm: dx = (view of z's gradient) + term, written into s's own buffer
        s._backward()                          # add: a and b take s's gradient as views
        assert gpu.kernelLaunches() - l1 == 1, "only the norm's backward may launch"
        gpu.sync([s, n, z])
    finally:
        gpu.uninstall()
    sw = a.data.astype(np.float64) + b.data
    y, rinv = oracle.rmsnorm_fwd(sw.astype(np.float32).reshape(T, d), w.data, 1e-5)
    compare("sum", s.data, sw, FWD)
    compare("norm", n.data, y, FWD)
    compare("z", z.data, sw + y.reshape(-1), FWD)
    gx, gw = oracle.rmsnorm_bwd(sw.astype(np.float32).reshape(T, d), w.data, rinv, up.reshape(T, d))
    want = up.astype(np.float64) + gx.reshape(-1)
    compare("d a", a.grad, want, BWD)
    compare("d b", b.grad, want, BWD)
    compare("d w", w.grad, gw, BWD)
