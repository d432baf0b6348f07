"""The tcgen05 (TF32, f32 accumulate) matrix product through the C ABI against an f64 product of the same
f32 inputs: all three operand layouts, ragged edges, accumulate, split-K; and a whole training step in
tf32 mode against the CPU oracle. Bound: relative L2 <= 2e-3 (the tensor-core modes' stated tolerance)."""
import numpy as np
import pytest

from gpu_harness import REL_L2_TC, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from gguf_trainer_b200.backend import requireGPU
    g = requireGPU("the tensor-core suite", precision="tf32")
    yield g
    g.destroy()


def _dev(gpu, a):
    b = gpu.createStateBuffer(a.nbytes)
    gpu.writeStateBuffer(b, a)
    return b


SHAPES = [(128, 128, 32), (128, 192, 64), (256, 192, 576), (300, 200, 100), (2048, 576, 576), (1000, 1536, 576),
          (576, 1536, 2048), (192, 576, 4096), (2048, 64, 1536), (130, 16, 576), (4096, 576, 16),
          (16, 1024, 4096), (16, 200, 300), (24, 64, 2048), (48, 576, 16)]   # rank-16 adapter gradients: M below one tile


@pytest.mark.parametrize("kind", ["NT", "NN", "TN"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_tf32(gpu, oracle, kind, M, N, K):
    rng = oracle.Mulberry32(M * 7 + N * 3 + K)
    A = rng.randn((M, K), 0.5)
    B = rng.randn((N, K), 0.5)
    C0 = rng.randn((M, N), 0.5)
    want = A.astype(np.float64) @ B.astype(np.float64).T
    a_store = A if kind != "TN" else np.ascontiguousarray(A.T)        # TN: A is [K, M]
    b_store = B if kind == "NT" else np.ascontiguousarray(B.T)        # NN, TN: B is [K, N]
    da, db = _dev(gpu, a_store), _dev(gpu, b_store)
    launches = gpu.kernelLaunches()
    for accum in (0, 1):
        dc = _dev(gpu, C0)
        gpu._gemm(kind, accum, M, N, K, da, db, dc)
        got = gpu.readStateBuffer(dc, M * N).reshape(M, N)
        ref = want + (C0.astype(np.float64) if accum else 0.0)
        r = rel_l2(got, ref)
        assert np.isfinite(got).all()
        assert r <= REL_L2_TC, f"{kind} {M}x{N}x{K} accum={accum}: relative L2 {r:.3e}"
        gpu._check(gpu.lib.gt_free(gpu.ctx, dc))
    gpu.sync([])   # surfaces a pipeline-wait flag if one was raised
    assert gpu.kernelLaunches() > launches
    for b in (da, db):
        gpu._check(gpu.lib.gt_free(gpu.ctx, b))


@pytest.mark.parametrize("kind", ["NT", "NN", "TN"])
@pytest.mark.parametrize("M,N,K,K2", [(2048, 3072, 1024, 16), (300, 200, 100, 16), (1000, 576, 70, 40), (64, 1536, 4096, 8),
                                      (4096, 192, 576, 576)])
def test_gemm2_two_products_into_one_tile(gpu, oracle, kind, M, N, K, K2):
    """gt_gemm2: C (+)= A.B + A2.B2 with the second product's K blocks following the first's in one launch (the
    projection with a rank-16 adapter and its input gradient), ragged K on both, split-K, accumulate."""
    rng = oracle.Mulberry32(M + 3 * N + 5 * K + 7 * K2)
    A, B = rng.randn((M, K), 0.5), rng.randn((N, K), 0.5)
    A2, B2 = rng.randn((M, K2), 0.5), rng.randn((N, K2), 0.5)
    C0 = rng.randn((M, N), 0.5)
    want = A.astype(np.float64) @ B.astype(np.float64).T + A2.astype(np.float64) @ B2.astype(np.float64).T
    sa = (lambda X: X if kind != "TN" else np.ascontiguousarray(X.T))
    sb = (lambda X: X if kind == "NT" else np.ascontiguousarray(X.T))
    bufs = [_dev(gpu, sa(A)), _dev(gpu, sb(B)), _dev(gpu, sa(A2)), _dev(gpu, sb(B2))]
    for accum in (0, 1):
        dc = _dev(gpu, C0)
        gpu._gemm2(kind, accum, M, N, K, bufs[0], bufs[1], K2, bufs[2], bufs[3], dc)
        got = gpu.readStateBuffer(dc, M * N).reshape(M, N)
        ref = want + (C0.astype(np.float64) if accum else 0.0)
        r = rel_l2(got, ref)
        assert np.isfinite(got).all()
        assert r <= REL_L2_TC, f"{kind} {M}x{N}x({K}+{K2}) accum={accum}: relative L2 {r:.3e}"
        gpu._check(gpu.lib.gt_free(gpu.ctx, dc))
    gpu.sync([])
    for b in bufs:
        gpu._check(gpu.lib.gt_free(gpu.ctx, b))


@pytest.mark.parametrize("kind", ["NT", "NN", "TN"])
@pytest.mark.parametrize("M,N,Ks", [(2048, 576, (576, 192, 192)), (300, 200, (100, 16, 40, 8)), (1000, 1536, (64,) * 8),
                                    (16384, 576, (1536, 1536))])
def test_gemm_multi_sums_products_in_one_launch(gpu, oracle, kind, M, N, Ks):
    """gt_gemm_multi: C (+)= sum_p A_p.B_p, the K blocks of each product following the previous one's in one main loop
    (dX = dQ.Wq + dK.Wk + dV.Wv of the activation that feeds three projections; dGate.Wg + dUp.Wu), ragged K, up to
    eight products, accumulate."""
    import ctypes as C
    rng = oracle.Mulberry32(M + 3 * N + sum(Ks))
    As = [rng.randn((M, K), 0.5) for K in Ks]
    Bs = [rng.randn((N, K), 0.5) for K in Ks]
    C0 = rng.randn((M, N), 0.5)
    want = sum(a.astype(np.float64) @ b.astype(np.float64).T for a, b in zip(As, Bs))
    sa = (lambda X: X if kind != "TN" else np.ascontiguousarray(X.T))
    sb = (lambda X: X if kind == "NT" else np.ascontiguousarray(X.T))
    da, db = [_dev(gpu, sa(a)) for a in As], [_dev(gpu, sb(b)) for b in Bs]
    n = len(Ks)
    kinds = {"NT": 0, "NN": 1, "TN": 2}
    launches = gpu.kernelLaunches()
    for accum in (0, 1):
        dc = _dev(gpu, C0)
        gpu._check(gpu.lib.gt_gemm_multi(gpu.ctx, kinds[kind], accum, M, N, n, (C.c_int32 * n)(*Ks), (C.c_uint64 * n)(*da),
                                         (C.c_uint64 * n)(*db), dc))
        got = gpu.readStateBuffer(dc, M * N).reshape(M, N)
        r = rel_l2(got, want + (C0.astype(np.float64) if accum else 0.0))
        assert np.isfinite(got).all() and r <= REL_L2_TC, f"{kind} {M}x{N}x{Ks} accum={accum}: relative L2 {r:.3e}"
        gpu._check(gpu.lib.gt_free(gpu.ctx, dc))
    gpu.sync([])
    assert gpu.kernelLaunches() - launches == 2, "each call must be a single launch on the tensor-core path"
    for b in da + db:
        gpu._check(gpu.lib.gt_free(gpu.ctx, b))


@pytest.mark.parametrize("kind,M,N,K,accum", [("NT", 2048, 16, 1024, 0), ("NN", 300, 16, 200, 1), ("TN", 576, 1536, 4096, 1),
                                              ("NT", 513, 200, 96, 0)])
def test_gemm_scaled(gpu, oracle, kind, M, N, K, accum):
    """gt_gemm_scaled: C (+)= alpha * A.B with the factor applied in the epilogue (thin adapter products, split-K too)."""
    alpha = 1.25
    rng = oracle.Mulberry32(3 * M + N + 9 * K)
    A, B, C0 = rng.randn((M, K), 0.5), rng.randn((N, K), 0.5), rng.randn((M, N), 0.5)
    want = alpha * (A.astype(np.float64) @ B.astype(np.float64).T) + (C0.astype(np.float64) if accum else 0.0)
    a_store = A if kind != "TN" else np.ascontiguousarray(A.T)
    b_store = B if kind == "NT" else np.ascontiguousarray(B.T)
    da, db, dc = _dev(gpu, a_store), _dev(gpu, b_store), _dev(gpu, C0)
    kinds = {"NT": 0, "NN": 1, "TN": 2}
    gpu._check(gpu.lib.gt_gemm_scaled(gpu.ctx, kinds[kind], accum, M, N, K, da, db, dc, alpha))
    got = gpu.readStateBuffer(dc, M * N).reshape(M, N)
    gpu.sync([])
    r = rel_l2(got, want)
    assert r <= REL_L2_TC, f"{kind} {M}x{N}x{K}: relative L2 {r:.3e}"
    for b in (da, db, dc):
        gpu._check(gpu.lib.gt_free(gpu.ctx, b))


@pytest.mark.parametrize("frozen_base", [True, False])
def test_lora_projection_as_one_op_tf32(gpu, oracle, frozen_base):
    """`loraLinear` on the tensor-core path (gt_gemm2 forward and input gradient, 16-row adapter gradient) against
    f64 formulas of y = x.W^T + s.(x.A^T).B^T, with a scale that is not a power of two."""
    from gpu_harness import rand_tensor, upstream
    from gguf_trainer_b200 import autograd as ag
    T, din, dout, r, s = 200, 96, 80, 16, 1.25
    rng = oracle.Mulberry32(77)
    x = rand_tensor(rng, [T, din]); w = rand_tensor(rng, [dout, din], 0.3, requires_grad=not frozen_base)
    la = rand_tensor(rng, [r, din], 0.3); lb = rand_tensor(rng, [dout, r], 0.3)
    for t in (x, w, la, lb):
        t.zeroGrad()
    ag.setLoraAdapters({id(w): ag.LoraAdapter(la, lb, s)})
    gpu.install()
    try:
        y = ag.linear(x, w)
        g = upstream(oracle, y.size)
        y.grad[:] = g
        gpu.seedGradFromHost(y)
        y._backward()
        gpu.sync([y])
    finally:
        gpu.uninstall()
        ag.setLoraAdapters({})
    X, W, A, B = (t.data.astype(np.float64).reshape(t.shape) for t in (x, w, la, lb))
    G = g.astype(np.float64).reshape(T, dout)
    t1 = X @ A.T
    want = {"y": X @ W.T + s * (t1 @ B.T), "dx": G @ W + s * (G @ B) @ A, "dA": s * (G @ B).T @ X, "dB": s * G.T @ t1}
    got = {"y": y.data, "dx": x.grad, "dA": la.grad, "dB": lb.grad}
    if not frozen_base:
        want["dW"], got["dW"] = G.T @ X, w.grad
    else:
        assert not w.grad.any()
    for k in want:
        e = rel_l2(got[k], want[k])
        assert e <= REL_L2_TC, f"{k}: relative L2 {e:.3e}"


def test_muon_step_tf32_batched_shapes(gpu, oracle):
    """The Muon step on the tensor-core path: same-shape matrices batched, tall ones iterated as stored (Gram matrix
    X^T.X, update X.B'^T) and wide ones as X.X^T, B'.X; the applied update against the CPU oracle. Five Newton-Schulz
    iterations compound the products' error, so the bound on the update is 5e-3 relative L2."""
    from gguf_trainer_b200.autograd import Tensor
    from gguf_trainer_b200.optim import MuonGpu
    rng = oracle.Mulberry32(0x4D4E)
    shapes = [(160, 64), (160, 64), (64, 160), (96, 96)]
    ps = [Tensor(rng.randn(s, 0.5), list(s), True) for s in shapes]
    ws = [p.data.copy().reshape(s) for p, s in zip(ps, shapes)]
    w0 = [w.copy() for w in ws]
    bufs = [np.zeros(s, np.float32) for s in shapes]
    opt = MuonGpu(gpu, ps, [], lr=0.05, momentum=0.95, nesterov=True, nsSteps=5, aux={"lr": 1e-3})
    for _ in range(2):
        for p, w, b, s in zip(ps, ws, bufs, shapes):
            g = rng.randn(s, 0.3)
            gpu.writeStateBuffer(gpu.buffersFor(p)["grad"], g)
            oracle.muon_step_array(w, g, b, 0.05, 0.95, True, 5)
        opt.recordStep()
    gpu.sync(ps)
    for p, w, z, s in zip(ps, ws, w0, shapes):
        r = rel_l2(p.data.reshape(s) - z, w - z)
        assert r <= 5e-3, f"{s}: update relative L2 {r:.3e}"


TILES = ["1,192", "1,128", "2,256", "2,192", "3,192", "3,256"]   # rows per CTA x columns; 3 = a CTA pair (cta_group::2)


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("kind,M,N,K,accum", [("NT", 1000, 1536, 576, 0), ("NN", 2048, 576, 1536, 1), ("TN", 576, 1536, 4096, 0),
                                              ("TN", 300, 200, 2048, 1), ("NT", 513, 49, 96, 0)])
def test_gemm_every_tile_shape(gpu, oracle, monkeypatch, tile, kind, M, N, K, accum):
    """Each tile shape of the dispatcher forced in turn (the cost model would otherwise pick one per product):
    ragged edges, accumulate, split-K, all layouts."""
    monkeypatch.setenv("GT_GEMM_TILE", tile)
    rng = oracle.Mulberry32(M + 11 * N + 5 * K)
    A, B, C0 = rng.randn((M, K), 0.5), rng.randn((N, K), 0.5), rng.randn((M, N), 0.5)
    want = A.astype(np.float64) @ B.astype(np.float64).T + (C0.astype(np.float64) if accum else 0.0)
    a_store = A if kind != "TN" else np.ascontiguousarray(A.T)
    b_store = B if kind == "NT" else np.ascontiguousarray(B.T)
    da, db, dc = _dev(gpu, a_store), _dev(gpu, b_store), _dev(gpu, C0)
    gpu._gemm(kind, accum, M, N, K, da, db, dc)
    got = gpu.readStateBuffer(dc, M * N).reshape(M, N)
    gpu.sync([])
    r = rel_l2(got, want)
    assert np.isfinite(got).all() and r <= REL_L2_TC, f"tile {tile} {kind} {M}x{N}x{K}: relative L2 {r:.3e}"
    assert r > 1e-6, "the strict-f32 kernel answered: the forced tile shape was not used"
    for b in (da, db, dc):
        gpu._check(gpu.lib.gt_free(gpu.ctx, b))


def test_tf32_products_differ_from_strict_f32(gpu, oracle):
    """Guards against the tensor-core path silently falling through to the f32 kernel."""
    rng = oracle.Mulberry32(5)
    M, N, K = 256, 192, 576
    A, B = rng.randn((M, K), 0.5), rng.randn((N, K), 0.5)
    da, db = _dev(gpu, A), _dev(gpu, B)
    outs = {}
    for mode in ("tf32", "fp32"):
        gpu.setPrecision(mode)
        dc = gpu.createStateBuffer(M * N * 4)
        gpu._gemm("NT", 0, M, N, K, da, db, dc)
        outs[mode] = gpu.readStateBuffer(dc, M * N)
    gpu.setPrecision("tf32")
    want = (A.astype(np.float64) @ B.astype(np.float64).T).ravel()
    assert rel_l2(outs["fp32"], want) < 1e-6
    assert 1e-5 < rel_l2(outs["tf32"], want) <= REL_L2_TC


def test_config1_step_in_tf32_mode(gpu, oracle):
    """Tiny llama (hidden 128, 2 layers, seq 128): loss and every gradient in tf32 mode vs the oracle."""
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.arch import buildModel, tinyLlama
    from gguf_trainer_b200.train import sequenceLoss
    cfg = tinyLlama()
    om = oracle.Model(cfg.oracle_dict(), 1234)
    m = buildModel(cfg, 1234)
    for i, p in enumerate(m.params()):
        p.data[:] = om.data(i).reshape(-1)
    ids = oracle.Mulberry32(3).randint(128, cfg.vocabSize)
    tg = oracle.Mulberry32(4).randint(128, cfg.vocabSize)
    ref = float(om.loss_backward(ids, tg))
    gpu.install()
    try:
        loss = sequenceLoss(m, ids, tg)
        ag.backward(loss, 1.0)
        gpu.sync([loss])
    finally:
        gpu.uninstall()
    assert abs(float(loss.data[0]) - ref) <= 2e-3 * abs(ref)
    for i, p in enumerate(m.params()):
        r = rel_l2(p.grad, om.grad(i))
        assert r <= REL_L2_TC, f"grad[{i}] {p.shape}: relative L2 {r:.3e}"


def test_muon_batched_groups_in_tf32_mode(gpu, oracle):
    """Three 192x576 and two 576x192 matrices: each shape is orthogonalised as one batch on the tensor cores."""
    from gguf_trainer_b200.autograd import Tensor
    from gguf_trainer_b200.optim import MuonGpu
    rng = oracle.Mulberry32(0x4D4D)
    shapes = [(192, 576), (576, 192), (192, 576), (576, 192), (192, 576)]
    ps = [Tensor(rng.randn(s, 0.05), list(s), True) for s in shapes]
    ws = [p.data.copy().reshape(s) for p, s in zip(ps, shapes)]
    w0 = [w.copy() for w in ws]
    bufs = [np.zeros(s, np.float32) for s in shapes]
    opt = MuonGpu(gpu, ps, [], lr=0.05, momentum=0.95, nesterov=True, nsSteps=5, aux={"lr": 1e-3})
    for _ in range(2):
        gs = [rng.randn(s, 0.3) for s in shapes]
        for p, g in zip(ps, gs):
            gpu.writeStateBuffer(gpu.buffersFor(p)["grad"], g)
        opt.recordStep()
        for w, g, b in zip(ws, gs, bufs):
            oracle.muon_step_array(w, g, b, 0.05, 0.95, True, 5)
    gpu.sync(ps)
    for i, (p, w) in enumerate(zip(ps, ws)):
        r = rel_l2(p.data, w)
        assert r <= REL_L2_TC, f"matrix {i} {shapes[i]}: relative L2 {r:.3e}"
        # the update itself (15 chained tf32 products per step) is held to 1e-2
        d = rel_l2(p.data.reshape(shapes[i]) - w0[i], w - w0[i])
        assert d <= 1e-2, f"matrix {i} {shapes[i]}: update relative L2 {d:.3e}"


def test_fused_cross_entropy_large_vocab_tf32(gpu, oracle):
    """The chunked readout loss on the tensor-core path at a large vocabulary: V = 40000 in chunks of 16384 (two full
    spans and a ragged one of 7232), a third of the rows masked out, against the f64 dense formula: loss, dHidden and
    dW (webgpu.ts:1214-1278 is the op; the case follows tests/gpu-parity.ts:174-207 at a size where spans are real)."""
    from gpu_harness import rand_tensor
    from gguf_trainer_b200 import autograd as ag
    T, H, V, chunk = 192, 128, 40000, 16384
    rng = oracle.Mulberry32(0xCE)
    hidden = rand_tensor(rng, [T, H], 1.0)
    w = rand_tensor(rng, [V, H], 0.05)
    targets = oracle.Mulberry32(9).randint(T, V)
    targets[::3] = -1
    targets[5] = V - 1                     # a target inside the ragged last span
    for t in (hidden, w):
        t.zeroGrad()
    gpu.install()
    try:
        loss = ag.fusedCrossEntropy(hidden, w, targets, chunk)
        ag.backward(loss, 1.0)
        gpu.sync([loss])
    finally:
        gpu.uninstall()
    Hd, W = hidden.data.astype(np.float64).reshape(T, H), w.data.astype(np.float64).reshape(V, H)
    z = Hd @ W.T
    z -= z.max(axis=1, keepdims=True)
    p = np.exp(z)
    p /= p.sum(axis=1, keepdims=True)
    kept = targets >= 0
    rows = np.nonzero(kept)[0]
    ref_loss = -np.log(p[rows, targets[rows]]).mean()
    dz = p.copy()
    dz[rows, targets[rows]] -= 1.0
    dz[~kept] = 0.0
    dz /= kept.sum()
    assert abs(float(loss.data[0]) - ref_loss) <= REL_L2_TC * ref_loss
    for name, got, want in (("dHidden", hidden.grad, dz @ W), ("dW", w.grad, dz.T @ Hd)):
        r = rel_l2(got, want)
        assert r <= REL_L2_TC, f"{name}: relative L2 {r:.3e}"
    assert not hidden.grad.reshape(T, H)[~kept].any()      # masked rows get exactly no gradient


@pytest.mark.parametrize("tile", ["", "1,192", "2,192"])
@pytest.mark.parametrize("kind,K,shapes", [
    ("TN", 2048, [(576, 576), (192, 576), (192, 576), (576, 576), (1536, 576), (1536, 576), (576, 1536)]),   # a layer's dW
    ("TN", 300, [(100, 200), (16, 64), (132, 36)]),
    ("NT", 96, [(513, 200), (64, 48)]),
    ("NN", 1024, [(256, 192), (256, 192), (128, 576), (40, 24), (300, 100), (16, 16), (700, 64), (64, 700)])])
def test_gemm_grouped_products_in_one_launch(gpu, oracle, monkeypatch, tile, kind, K, shapes):
    """gt_gemm_grouped: independent products of one layout and one K, each with its own extents, operands and
    accumulate flag, as one launch (the weight gradients of a layer's projections). Both tile shapes forced in turn
    and the dispatcher's own choice; every other product accumulates."""
    import ctypes as C
    if tile:
        monkeypatch.setenv("GT_GEMM_TILE", tile)
    rng = oracle.Mulberry32(K + 17 * len(shapes))
    As = [rng.randn((M, K), 0.5) for M, _N in shapes]
    Bs = [rng.randn((N, K), 0.5) for _M, N in shapes]
    C0 = [rng.randn(s, 0.5) for s in shapes]
    accs = [g % 2 for g in range(len(shapes))]
    sa = (lambda X: X if kind != "TN" else np.ascontiguousarray(X.T))
    sb = (lambda X: X if kind == "NT" else np.ascontiguousarray(X.T))
    da, db, dc = [_dev(gpu, sa(a)) for a in As], [_dev(gpu, sb(b)) for b in Bs], [_dev(gpu, c) for c in C0]
    n = len(shapes)
    launches = gpu.kernelLaunches()
    gpu._check(gpu.lib.gt_gemm_grouped(gpu.ctx, {"NT": 0, "NN": 1, "TN": 2}[kind], n, (C.c_int32 * n)(*[s[0] for s in shapes]),
                                       (C.c_int32 * n)(*[s[1] for s in shapes]), K, (C.c_uint64 * n)(*da), (C.c_uint64 * n)(*db),
                                       (C.c_uint64 * n)(*dc), (C.c_int32 * n)(*accs)))
    got = [gpu.readStateBuffer(c, s[0] * s[1]).reshape(s) for c, s in zip(dc, shapes)]
    gpu.sync([])
    assert gpu.kernelLaunches() - launches == 1
    for g, (a, b, c0, acc) in enumerate(zip(As, Bs, C0, accs)):
        want = a.astype(np.float64) @ b.astype(np.float64).T + (c0.astype(np.float64) if acc else 0.0)
        r = rel_l2(got[g], want)
        assert np.isfinite(got[g]).all() and r <= REL_L2_TC, f"product {g} {shapes[g]} accum={acc}: relative L2 {r:.3e}"
        assert r > 1e-7, "the strict-f32 kernel answered"
    for b in da + db + dc:
        gpu._check(gpu.lib.gt_free(gpu.ctx, b))


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("T,din,ffn", [(300, 96, 200), (2048, 576, 1536), (130, 64, 96), (257, 64, 224)])
def test_gated_ffn_is_two_launches_forward_and_four_backward(gpu, oracle, act, T, din, ffn):
    """`linear(mul(act(linear(x, Wg)), linear(x, Wu)), Wd)`, the FFN of every block (src/arch/llama.ts:209-212). Forward:
    the gate and up projections and the gated unit are ONE launch (gt_glu_linear_fwd: each output tile holds 96 gate and
    the matching 96 up columns), then the down projection. Backward: the down projection's input gradient, the unit's
    backward, the three weight gradients as one grouped launch, the input gradient of gate and up as one launch over
    both K ranges. Values and every gradient against f64 formulas, ragged widths included."""
    from gpu_harness import rand_tensor, upstream
    from gguf_trainer_b200 import autograd as ag
    rng = oracle.Mulberry32(T + 3 * din + 7 * ffn)
    x = rand_tensor(rng, [T, din]); wg = rand_tensor(rng, [ffn, din], 0.2); wu = rand_tensor(rng, [ffn, din], 0.2)
    wd = rand_tensor(rng, [din, ffn], 0.2)
    for t in (x, wg, wu, wd):
        t.zeroGrad()
    f = ag.silu if act == "silu" else ag.gelu
    gpu.install()
    try:
        gpu.sync([])
        l0 = gpu.kernelLaunches()
        gate = ag.linear(x, wg)
        up = ag.linear(x, wu)
        hidden = ag.mul(f(gate), up)
        assert gpu.kernelLaunches() - l0 == 1, "projections and gated unit must be one launch"
        y = ag.linear(hidden, wd)
        g = upstream(oracle, y.size)
        y.grad[:] = g
        gpu.seedGradFromHost(y)                    # (launches the down projection)
        l1 = gpu.kernelLaunches()
        # closures in reverse creation order: down, product, activation (a no-op here), up, gate
        y._backward(); hidden._backward(); hidden._prev[0]._backward(); up._backward(); gate._backward()
        gpu.sync([y, hidden, gate, up])
        assert gpu.kernelLaunches() - l1 == 4, gpu.kernelLaunches() - l1
    finally:
        gpu.uninstall()
    X, Wg, Wu, Wd = (t.data.astype(np.float64).reshape(t.shape) for t in (x, wg, wu, wd))
    G, U = X @ Wg.T, X @ Wu.T
    if act == "silu":
        sig = 1 / (1 + np.exp(-G))
        A, dA = G * sig, sig + G * sig * (1 - sig)
    else:
        k, a = 0.7978845608028654, 0.044715
        th = np.tanh(k * (G + a * G ** 3))
        A, dA = 0.5 * G * (1 + th), 0.5 * (1 + th) + 0.5 * G * (1 - th ** 2) * k * (1 + 3 * a * G ** 2)
    Hh = A * U
    gy = g.astype(np.float64).reshape(T, din)
    go = gy @ Wd
    dG, dU = go * U * dA, go * A
    want = {"gate": G, "up": U, "hidden": Hh, "y": Hh @ Wd.T, "dx": dG @ Wg + dU @ Wu, "dWg": dG.T @ X, "dWu": dU.T @ X, "dWd": gy.T @ Hh}
    got = {"gate": gate.data, "up": up.data, "hidden": hidden.data, "y": y.data, "dx": x.grad, "dWg": wg.grad, "dWu": wu.grad, "dWd": wd.grad}
    for k_ in want:
        e = rel_l2(got[k_], want[k_])
        assert np.isfinite(np.asarray(got[k_])).all() and e <= REL_L2_TC, f"{k_}: relative L2 {e:.3e}"


def test_projections_of_one_input_are_one_grouped_launch(gpu, oracle):
    """q, k and v of the same normed input: three `linear` calls, one launch (the products are noted and launched when
    the first output is needed), results as three separate products."""
    from gpu_harness import rand_tensor
    from gguf_trainer_b200 import autograd as ag
    rng = oracle.Mulberry32(404)
    T, din = 513, 576
    x = rand_tensor(rng, [T, din])
    ws = [rand_tensor(rng, [o, din], 0.1) for o in (576, 192, 192)]
    gpu.install()
    try:
        gpu.sync([])
        l0 = gpu.kernelLaunches()
        outs = [ag.linear(x, w) for w in ws]
        assert gpu.kernelLaunches() == l0                       # nothing launched yet
        gpu.sync(outs)
        assert gpu.kernelLaunches() - l0 == 1
    finally:
        gpu.uninstall()
    X = x.data.astype(np.float64).reshape(T, din)
    for o, w in zip(outs, ws):
        e = rel_l2(o.data, X @ w.data.astype(np.float64).reshape(w.shape).T)
        assert e <= REL_L2_TC and e > 1e-7, f"relative L2 {e:.3e}"


def _attention_block(gpu, oracle, T, B, din, Hq, Hkv, hd, window, fuse, read_q=False, head_norm=False):
    """q = rope(linear(x, Wq)), k = rope(linear(x, Wk)), v = linear(x, Wv), a = attention(q, k, v), the attention half
    of a llama block (src/arch/llama.ts:195-201), forward and backward with a fixed upstream gradient. Returns the
    launch counts and every value a caller can observe."""
    from gpu_harness import rand_tensor, upstream
    from gguf_trainer_b200 import autograd as ag
    rng = oracle.Mulberry32(T + 7 * din + 13 * Hq + hd)
    rows = T * max(B, 1)
    x = rand_tensor(rng, [rows, din])
    wq, wk, wv = (rand_tensor(rng, [h * hd, din], 0.1) for h in (Hq, Hkv, Hkv))
    nq, nk = rand_tensor(rng, [hd], 0.5), rand_tensor(rng, [hd], 0.5)
    for t in (x, wq, wk, wv, nq, nk):
        t.zeroGrad()
    gpu.fuseRope = fuse
    gpu.install()
    if B:
        gpu.setBatch(B, T)
    try:
        gpu.sync([])
        l0 = gpu.kernelLaunches()
        q0, k0 = ag.linear(x, wq), ag.linear(x, wk)
        v = ag.linear(x, wv)
        q1, k1 = q0, k0
        if head_norm:            # the Qwen3 / Gemma 3 block: per-head norms between the projections and the rotations
            q1, k1 = ag.rmsNormHeads(q0, nq, rows, Hq, hd, 1e-6), ag.rmsNormHeads(k0, nk, rows, Hkv, hd, 1e-6)
        q, k = ag.rope(q1, rows, Hq, hd, 10000.0), ag.rope(k1, rows, Hkv, hd, 10000.0)
        a = ag.attention(q, k, v, rows, Hq, Hkv, hd, window)
        fwd = gpu.kernelLaunches() - l0
        g = upstream(oracle, a.size)
        a.grad[:] = g
        gpu.seedGradFromHost(a)
        l1 = gpu.kernelLaunches()
        a._backward(); k._backward(); q._backward()
        if head_norm:
            k1._backward(); q1._backward()
        v._backward(); k0._backward(); q0._backward()
        reads = [a, q, k, v] + ([q0, q1] if read_q else [])
        gpu.sync(reads)
        bwd = gpu.kernelLaunches() - l1
    finally:
        gpu.setBatch(0)
        gpu.uninstall()
        gpu.fuseRope = True
    vals = {"a": a.data.copy(), "q": q.data.copy(), "k": k.data.copy(), "v": v.data.copy(), "dx": x.grad.copy(),
            "dWq": wq.grad.copy(), "dWk": wk.grad.copy(), "dWv": wv.grad.copy()}
    if head_norm:
        vals["dnq"], vals["dnk"] = nq.grad.copy(), nk.grad.copy()
    if read_q:
        vals["q0"], vals["q1"] = q0.data.copy(), q1.data.copy()
    return fwd, bwd, vals


@pytest.mark.parametrize("T,B,din,Hq,Hkv,hd,window", [(256, 0, 192, 4, 2, 64, 0), (200, 2, 576, 9, 3, 64, 0), (192, 3, 128, 2, 1, 64, 96),
                                                     (128, 2, 256, 2, 2, 128, 0), (160, 0, 96, 4, 1, 32, 0)])
def test_rotary_embedding_runs_inside_its_neighbours(gpu, oracle, T, B, din, Hq, Hkv, hd, window):
    """`rope` between `linear` and `attention`: with 64-wide heads the q/k/v launch writes q and k already rotated, and
    for head sizes 64 and 128 attention's backward rotates dQ and dK back as it stores them, so neither rotation is
    a launch of its own. Every observable value against the same block with the rotations launched separately (which
    the op tests hold to the oracle). The rotated values themselves agree to f32 rounding (1e-6). What then passes through
    another TF32 product (the attention output, dx, dW) can differ more: an operand that moved by a few f32 units in the last
    place, as a difference of two rotated terms does, can fall on the other side of a TF32 truncation (2^-11 on that
    element). Measured 3e-5 at most; bound 1e-4, a twentieth of the mode's own tolerance."""
    _attention_block(gpu, oracle, T, B, din, Hq, Hkv, hd, window, False)     # (builds the angle table of this shape: one more launch)
    f_fwd, f_bwd, fused = _attention_block(gpu, oracle, T, B, din, Hq, Hkv, hd, window, True)
    p_fwd, p_bwd, plain = _attention_block(gpu, oracle, T, B, din, Hq, Hkv, hd, window, False)
    assert p_fwd == 4 and p_bwd == 3 + 2 + 2, (p_fwd, p_bwd)      # q/k/v, 2 rotations, attention; D, dKV, dQ, 2 rotations, dW, dX
    assert f_fwd == (2 if hd == 64 else 4), f_fwd
    assert f_bwd == (5 if hd >= 64 else 7), f_bwd
    for name in plain:
        e = rel_l2(fused[name], plain[name])
        assert np.isfinite(fused[name]).all() and e <= (1e-6 if name in ("q", "k", "v") else 1e-4), f"{name}: relative L2 {e:.3e}"


@pytest.mark.parametrize("T,B,din,Hq,Hkv,hd,window", [(200, 2, 256, 4, 2, 128, 0), (128, 2, 128, 2, 1, 256, 96), (192, 0, 192, 4, 2, 64, 0)])
def test_per_head_norm_and_rotary_embedding_are_one_pass(gpu, oracle, T, B, din, Hq, Hkv, hd, window):
    """`rope(rmsNormHeads(linear(x, W)))`, the q and k of the Qwen3 and Gemma 3 blocks: the norm waits for its first
    reader and, when that is the rotation, one pass normalises and rotates; attention's backward delivers dQ and dK to
    the norms' outputs (head sizes 64 and 128). Against the same block with every op launched."""
    _attention_block(gpu, oracle, T, B, din, Hq, Hkv, hd, window, False, head_norm=True)
    f_fwd, f_bwd, fused = _attention_block(gpu, oracle, T, B, din, Hq, Hkv, hd, window, True, head_norm=True)
    p_fwd, p_bwd, plain = _attention_block(gpu, oracle, T, B, din, Hq, Hkv, hd, window, False, head_norm=True)
    assert (p_fwd, p_bwd) == (6, 9), (p_fwd, p_bwd)
    assert f_fwd == 4 and f_bwd == (7 if hd <= 128 else 9), (f_fwd, f_bwd)
    for name in plain:
        e = rel_l2(fused[name], plain[name])
        assert np.isfinite(fused[name]).all() and e <= (1e-6 if name in ("q", "k", "v") else 1e-4), f"{name}: relative L2 {e:.3e}"


@pytest.mark.parametrize("head_norm", [False, True])
def test_tensor_consumed_rotated_is_still_readable(gpu, oracle, head_norm):
    """The unrotated projection (or per-head norm) is not written when its only reader took it rotated; a later reader
    (here a sync that asks for it) gets it from a launch made then."""
    _f, _b, fused = _attention_block(gpu, oracle, 256, 0, 192, 4, 2, 64, 0, True, read_q=True, head_norm=head_norm)
    _f, _b, plain = _attention_block(gpu, oracle, 256, 0, 192, 4, 2, 64, 0, False, read_q=True, head_norm=head_norm)
    for name in ("q0", "q1"):
        assert np.abs(plain[name]).max() > 0
        assert rel_l2(fused[name], plain[name]) <= 1e-6
