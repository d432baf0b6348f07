"""The host side (`autograd.py` tape + `backend.py` bookkeeping) driven on a CPU-only machine: `CudaBackend` talks to a
numpy stand-in for the C ABI (`tests/fake_cabi.py`) and whole small models are held to the CPU oracle, once with every
launch-merging decision of the backend switched on and once with every op launched as recorded. What this pins down
without a GPU: which entry points the backend calls and how often, the accumulate flags and addresses it passes (a
wrong one shows as a wrong gradient, an unwritten buffer reads as NaN), the projections and norms it leaves unwritten
until asked, and that recompute regions replay through the same decisions.

The shape of the whole-model check follows the reference's parity case (tests/gpu-parity.ts:333-392), as the GPU depth
suite does; the stand-in computes in f64 and stores f32 like the oracle, so the bound is the strict one (1e-5)."""
import numpy as np
import pytest

import fake_cabi
from depth_cases import run_case
from gguf_trainer_b200.arch import ModelConfig

L = 2
CONFIGS = {
    "llama": (ModelConfig("llama", 96, 128, L, 2, 1, 64, 192, 10_000.0, 1e-5), 64),
    "qwen3": (ModelConfig("qwen3", 96, 128, L, 2, 1, 64, 192, 1_000_000.0, 1e-6), 64),
    "gemma3": (ModelConfig("gemma3", 96, 128, 3, 2, 1, 64, 192, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0, slidingWindow=8,
                           swaPattern=3), 64),
}
FLAGS = ("mergeInputGradients", "fuseResidualNorm", "groupWeightGradients", "groupForward", "fuseGatedUnits", "fuseRope", "fuseLora")


@pytest.fixture
def dev(monkeypatch):
    fake = fake_cabi.install(monkeypatch)
    from gguf_trainer_b200.backend import CudaBackend
    gpu = CudaBackend(0, "tf32")
    yield gpu, fake
    gpu.destroy()


def check(res, what, bound=1e-5):
    got, ref = res["loss"]
    assert res["finite"], f"{what}: a gradient is not finite (something read a buffer nobody wrote)"
    assert abs(got - ref) <= bound * abs(ref), f"{what}: loss {got} vs {ref}"
    for l, e in enumerate(res["layers"]):
        assert e <= bound, f"{what}: output of layer {l}: relative L2 {e:.3e}"
    for i, (shape, e) in enumerate(res["grads"]):
        assert e <= bound, f"{what}: gradient {i} {shape}: relative L2 {e:.3e}"


@pytest.mark.parametrize("arch", list(CONFIGS))
@pytest.mark.parametrize("merged", [True, False])
@pytest.mark.parametrize("recompute", [False, True])
def test_whole_model_against_the_oracle(dev, oracle, arch, merged, recompute):
    gpu, fake = dev
    cfg, T = CONFIGS[arch]
    for f in FLAGS:
        setattr(gpu, f, merged)
    check(run_case(gpu, oracle, cfg, T, adamw=False, recompute=recompute), f"{arch}, merged launches {merged}, recompute {recompute}")
    if merged and not recompute:
        # what a merged step must not contain: rotations, residual adds, gated units and gradient copies of their own
        for name in ("gt_rope_fwd", "gt_copy", "gt_glu_fwd"):
            assert fake.count(name) == 0, (name, fake.count(name))
        assert not [c for c in fake.calls("gt_ew_fwd") if c["op"] == 0], "a residual add was launched on its own"
        assert fake.count("gt_glu_linear_fwd") == cfg.nLayers
        assert fake.count("gt_gemm_multi") == 2 * cfg.nLayers          # dX of q/k/v and of gate/up, one product each
        assert fake.count("gt_add_rmsnorm_fwd") >= 2 * cfg.nLayers - 1
        if arch == "llama":
            assert fake.count("gt_linear_rope_grouped") == cfg.nLayers and fake.count("gt_attention_bwd_rope") == cfg.nLayers
            assert fake.count("gt_rope_bwd") == 0
        else:
            assert fake.count("gt_rmsnorm_heads_rope_fwd") == 2 * cfg.nLayers and fake.count("gt_attention_bwd_rope") == cfg.nLayers
    if not merged:
        assert fake.count("gt_rope_fwd") == 2 * cfg.nLayers * (2 if recompute else 1)
        for name in ("gt_gemm_multi", "gt_gemm_grouped", "gt_linear_rope_grouped", "gt_glu_linear_fwd", "gt_add_rmsnorm_fwd",
                     "gt_rmsnorm_bwd_add", "gt_attention_bwd_rope", "gt_rmsnorm_heads_rope_fwd"):
            assert fake.count(name) == 0, (name, fake.count(name))


@pytest.mark.parametrize("merged", [True, False])
def test_adapters_on_a_frozen_base(dev, oracle, merged):
    """Rank-4 adapters on all seven projections of the Qwen3 block, half of the targets masked, recompute on: the
    adapter gradients against the oracle; merged, the thin products of projections that share an input are one grouped
    launch and the adapters' own gradients go through the grouped weight-gradient launch."""
    gpu, fake = dev
    cfg, T = CONFIGS["qwen3"]
    for f in FLAGS:
        setattr(gpu, f, merged)
    check(run_case(gpu, oracle, cfg, T, adamw=False, lora=(4, 8.0), mask_frac=0.5, recompute=True), f"adapters, merged {merged}")
    if merged:
        assert fake.count("gt_gemm_grouped_scaled") == 2 * cfg.nLayers * 2      # q/k/v and gate/up, forward and replay
        assert not [c for c in fake.calls("gt_gemm") if c["kind"] == fake_cabi.TN], "an adapter gradient was launched on its own"
    else:
        assert fake.count("gt_gemm_grouped_scaled") == 0 and fake.count("gt_gemm2") == 0


def test_projection_left_unwritten_is_written_when_read(dev, oracle):
    """`rope(linear(x, W))` merged into one launch never writes the projection itself; a later reader gets it from a
    product launched then, and the values are the projection's."""
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.autograd import Tensor
    gpu, fake = dev
    rng = np.random.default_rng(3)
    T, din, H, hd = 32, 48, 2, 64
    x = Tensor(rng.standard_normal(T * din).astype(np.float32), [T, din], True)
    wq = Tensor((rng.standard_normal(H * hd * din) * 0.1).astype(np.float32), [H * hd, din], True)
    wv = Tensor((rng.standard_normal(H * hd * din) * 0.1).astype(np.float32), [H * hd, din], True)
    gpu.install()
    try:
        q0, v = ag.linear(x, wq), ag.linear(x, wv)
        q = ag.rope(q0, T, H, hd, 10_000.0)
        assert fake.launches == 0                                 # three ops recorded, nothing launched yet
        gpu.sync([q, v])
        assert fake.count("gt_linear_rope_grouped") == 1 and fake.count("gt_gemm") == 0
        assert np.isnan(fake.f32(gpu._entries[q0].data, T, H * hd)).all()   # the unrotated projection: never written
    finally:
        gpu.uninstall()
    X, W = x.data.astype(np.float64).reshape(T, din), wq.data.astype(np.float64).reshape(H * hd, din)
    gpu.install()
    try:
        q0, v = ag.linear(x, wq), ag.linear(x, wv)
        q = ag.rope(q0, T, H, hd, 10_000.0)
        gpu.sync([q, q0])                                         # this time someone asks for it
        assert fake.count("gt_gemm") == 1
        assert np.allclose(q0.data.reshape(T, H * hd), X @ W.T, rtol=1e-6, atol=1e-6)
    finally:
        gpu.uninstall()


def test_precision_names_and_refusals(dev):
    gpu, _fake = dev
    gpu.setPrecision("fp32")
    assert gpu.precision == "fp32"
    with pytest.raises(KeyError):
        gpu.setPrecision("bf16")                                  # not a mode of this library
    assert gpu.precision == "fp32"


def test_batched_step_is_the_mean_of_its_sequences(dev, oracle):
    """`CudaStep` (eager form) over 3 sequences of 64 tokens: per-sequence losses equal the oracle's loss of each sequence
    run alone, and every gradient is the mean of the three single-sequence gradients (the loss seed is 1/sequences per
    sequence, as the reference's accumulation over micro-batches scales it, src/backend/train-gpu.ts:206-215)."""
    from gguf_trainer_b200.arch import buildModel
    from gguf_trainer_b200.train import CudaStep
    gpu, fake = dev
    cfg, T = CONFIGS["llama"]
    B = 3
    om = oracle.Model(cfg.oracle_dict(), 77)
    m = buildModel(cfg, 77)
    ps = m.params()
    for i, p in enumerate(ps):
        p.data[:] = om.data(i).reshape(-1)
        gpu.keepGradOnDevice(p)
    ids = oracle.Mulberry32(3).randint(B * T, cfg.vocabSize)
    tg = oracle.Mulberry32(4).randint(B * T, cfg.vocabSize)
    tg[5], tg[T + 9] = -1, -1
    step = CudaStep(m, gpu, B, T, capture=False)
    step.run(ids, tg)
    losses = step.losses().copy()
    grads = [gpu.readStateBuffer(gpu.buffersFor(p)["grad"], p.size) for p in ps]
    gpu.sync([])
    want_losses = []
    for s in range(B):   # the oracle's gradients accumulate over calls, as the reference's do over micro-batches
        want_losses.append(float(om.loss_backward(ids[s * T:(s + 1) * T], tg[s * T:(s + 1) * T], seed=1.0 / B)))
    want_grads = [om.grad(i).astype(np.float64).reshape(-1) for i in range(len(ps))]
    om.close()
    assert np.allclose(losses[1:], want_losses, rtol=1e-5, atol=0)
    assert abs(losses[0] - np.mean(want_losses)) <= 1e-5 * abs(np.mean(want_losses))
    for p, g, w in zip(ps, grads, want_grads):
        e = float(np.linalg.norm(g - w) / max(np.linalg.norm(w), 1e-30))
        assert e <= 1e-5, f"gradient {tuple(p.shape)}: relative L2 {e:.3e}"
    assert fake.count("gt_copy") == 0


def test_the_stand_in_follows_the_header():
    """Every entry point the stand-in offers is declared in include/gguftrain.h with the same number of parameters, so a
    call the backend makes against it is a call the library accepts."""
    import inspect
    from gguf_trainer_b200 import _lib
    declared = {name: len(types) for name, _ret, types in _lib.declared_functions()}
    mine = [n for n in dir(fake_cabi.FakeLib) if n.startswith("gt_")]
    assert len(mine) >= 45
    for n in mine:
        assert n in declared, f"{n} is not in the header"
        params = [p for p in inspect.signature(getattr(fake_cabi.FakeLib, n)).parameters.values()
                  if p.name != "self" and not p.name.startswith("_")]
        assert len(params) == declared[n], f"{n}: {len(params)} parameters here, {declared[n]} in the header"


def test_forward_only_caller_gets_no_gradient_work(dev, oracle):
    """A frozen model scored window by window (the evaluation loop, src/train/eval.ts): no backward, so no gradient
    buffer is cleared, nothing but the loss comes back, and the logits are the oracle's."""
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.arch import buildModel
    from gguf_trainer_b200.train import freezeForScoring, sequenceLoss
    gpu, fake = dev
    cfg, T = CONFIGS["qwen3"]
    om = oracle.Model(cfg.oracle_dict(), 5)
    m = buildModel(cfg, 5)
    for i, p in enumerate(m.params()):
        p.data[:] = om.data(i).reshape(-1)
    freezeForScoring(m)
    ids = oracle.Mulberry32(3).randint(T, cfg.vocabSize)
    tg = oracle.Mulberry32(4).randint(T, cfg.vocabSize)
    want = float(om.loss_backward(ids, tg))
    om.close()
    gpu.install()
    try:
        for _ in range(2):
            loss = sequenceLoss(m, ids, tg)
            gpu.sync([loss])
            assert abs(float(loss.data[0]) - want) <= 1e-5 * abs(want)
    finally:
        gpu.uninstall()
    assert gpu.gradClearsIssued == 0 and fake.count("gt_zero") == 0
    assert gpu.lastSyncReadbackBytes == 4
    assert all(fake.count(n) == 0 for n in ("gt_attention_bwd", "gt_attention_bwd_rope", "gt_ce_bwd", "gt_rmsnorm_bwd"))


@pytest.mark.parametrize("arch", ["llama", "gemma3"])
def test_readout_loss_over_vocabulary_spans(dev, oracle, arch):
    """`fusedCrossEntropy` with spans of 40 over a vocabulary of 96 (a ragged last span of 16) and a third of the targets
    ignored: loss and every gradient against the oracle's chunked loss; the [T, V] logits are never formed."""
    gpu, fake = dev
    cfg, T = CONFIGS[arch]
    check(run_case(gpu, oracle, cfg, T, adamw=False, loss_chunk=40, mask_frac=0.33), f"{arch}, readout in spans")
    assert fake.count("gt_ce_fwd") == 0 and fake.count("gt_ce_chunk_stats") == 3 and fake.count("gt_ce_chunk_grad") == 3
    assert [c["n"] for c in fake.calls("gt_ce_chunk_stats")] == [40, 40, 16]
    assert not [c for c in fake.calls("gt_gemm") if c["N"] == cfg.vocabSize or c["M"] == cfg.vocabSize]


def test_step_with_adamw_matches_the_oracle_weights(dev, oracle):
    """Forward, backward and one AdamW step (lr 1e-3, betas 0.9 / 0.95, weight decay 0.1, clip 1.0) through `AdamWGpu`: the
    optimizer flushes whatever launches were still put off before it reads the gradients, and the weights after the
    step are the oracle's."""
    gpu, fake = dev
    cfg, T = CONFIGS["llama"]
    res = run_case(gpu, oracle, cfg, T, adamw=True)
    check(res, "llama with adamw")
    for i, (shape, e) in enumerate(res["weights"]):
        assert e <= 1e-5, f"weight {i} {shape} after the step: relative L2 {e:.3e}"
    assert fake.count("gt_adamw_step") == 1
    order = [n for n, _kw in fake.log]
    assert max(i for i, n in enumerate(order) if n in ("gt_gemm_grouped", "gt_gemm_multi")) < order.index("gt_adamw_step")


def test_recorded_step_replays_to_the_eager_steps_results(dev, oracle):
    """`CudaStep` with recording: the first call runs eagerly once and records, later calls only rewrite the inputs and
    replay. Losses and gradients of three different batches equal the eager form's bit for bit (same arithmetic, same
    order), the replay records nothing new, and ids outside the vocabulary are refused before they reach the recording."""
    from gguf_trainer_b200.arch import buildModel
    from gguf_trainer_b200.train import CudaStep
    gpu, fake = dev
    cfg, T = CONFIGS["qwen3"]
    B = 2
    batches = [(oracle.Mulberry32(10 + i).randint(B * T, cfg.vocabSize), oracle.Mulberry32(20 + i).randint(B * T, cfg.vocabSize)) for i in range(3)]
    results = {}
    for capture in (False, True):
        m = buildModel(cfg, 9)
        for p in m.params():
            gpu.keepGradOnDevice(p)
        step = CudaStep(m, gpu, B, T, capture=capture)
        out = []
        for ids, tg in batches:
            before = len(fake.log)
            step.run(ids, tg)
            out.append((step.losses().copy(), [gpu.readStateBuffer(gpu.buffersFor(p)["grad"], p.size) for p in m.params()], len(fake.log) - before))
        gpu.sync([])
        results[capture] = out
        if capture:
            assert step.launchesPerReplay > 0
            bad = batches[0][0].copy()
            bad[3] = cfg.vocabSize
            with pytest.raises(ValueError, match="not an integer in \\[0,96\\)"):
                step.run(bad, batches[0][1])
    for (la, ga, _na), (lb, gb, _nb) in zip(results[False], results[True]):
        assert np.array_equal(la, lb)
        for a, b in zip(ga, gb):
            assert np.array_equal(a, b) and np.isfinite(a).all()
    # the first call ran the step eagerly and then replayed its recording; later calls only replay
    assert results[True][1][2] == results[True][2][2] and results[True][0][2] == 2 * results[True][1][2]


@pytest.mark.parametrize("capture", [False, True])
def test_gradient_exchange_in_buckets_leaves_the_single_process_gradients(dev, oracle, capture):
    """The data-parallel step as one of two ranks holding the same batch: the loss is seeded with 1/2, the gradient arena
    is summed bucket by bucket (one bucket per layer, each started when backward leaves the bucket's first layer; the
    stand-in's sum over two equal ranks is a doubling), and the result is bit for bit the gradient of the plain step.
    Recorded, the step is one graph per bucket boundary and the exchange is issued between the segments."""
    from gguf_trainer_b200.arch import buildModel
    from gguf_trainer_b200.train import CudaStep, DataParallel
    gpu, fake = dev
    cfg, T = CONFIGS["gemma3"]
    B = 2
    batches = [(oracle.Mulberry32(10 + i).randint(B * T, cfg.vocabSize), oracle.Mulberry32(20 + i).randint(B * T, cfg.vocabSize)) for i in range(2)]

    def run(with_dp):
        m = buildModel(cfg, 9)
        ps = m.params()
        arena = gpu.reserveGradArena(list(reversed(ps))) if with_dp else None
        if not with_dp:
            for p in ps:
                gpu.keepGradOnDevice(p)
        dp = DataParallel(gpu, 0, 2, DataParallel.uniqueId()) if with_dp else None
        step = CudaStep(m, gpu, B, T, world=2 if with_dp else 1, capture=capture, dp=dp, arena=arena, layersPerBucket=1)
        out = []
        for ids, tg in batches:
            before = len(fake.log)
            step.run(ids, tg)
            grads = [gpu.readStateBuffer(gpu.buffersFor(p)["grad"], p.size) for p in ps]
            out.append((step.losses().copy(), grads, [n for n, _kw in fake.log[before:]]))
        gpu.sync([])
        return out, (step.bucketPlan() if with_dp else None)

    plain, _ = run(False)
    exchanged, plan = run(True)
    assert len(plan) == cfg.nLayers and sum(c for _l, _s, c in plan) == sum(p.size + (-p.size) % 64 for p in buildModel(cfg, 9).params())
    for (la, ga, _), (lb, gb, names) in zip(plain, exchanged):
        assert np.array_equal(la, lb)
        for a, b in zip(ga, gb):
            assert np.array_equal(a, b) and np.isfinite(a).all()
    names = exchanged[1][2]
    starts = [i for i, n in enumerate(names) if n == "gt_dp_allreduce_start"]
    assert len(starts) == cfg.nLayers and names.count("gt_dp_wait") == 1
    # the first reduction starts while backward still has work to launch; the wait comes after the last one
    assert any(n.startswith("gt_attention_bwd") for n in names[starts[0]:]) and names.index("gt_dp_wait") > starts[-1]


@pytest.mark.parametrize("capture", [False, True])
def test_step_fed_by_window_starts(dev, oracle, capture):
    """`CudaStep.runWindows(starts)` over a corpus resident on the device equals `run(ids, targets)` on the windows the
    host would have cut (`window` twice + `maskWindow`, src/data/tokens.ts:158-185, src/train/trainer.ts:45-49), bit for
    bit; starts past the end and a corpus outside the vocabulary are refused on the host."""
    from gguf_trainer_b200.arch import buildModel
    from gguf_trainer_b200.ingest import DeviceTokenSource
    from gguf_trainer_b200.train import CudaStep, maskWindow
    gpu, fake = dev
    cfg, T = CONFIGS["llama"]
    B = 2
    rng = np.random.default_rng(5)
    tokens = rng.integers(0, cfg.vocabSize, 400)
    supervised = (rng.random(400) < 0.6).astype(np.int64)
    with pytest.raises(ValueError, match="not in \\[0,90\\)"):
        DeviceTokenSource(gpu, np.concatenate([tokens, [95]]), 90)

    def host_windows(starts):
        ids, tgs = [], []
        for s in starts:
            ids.append(np.array(tokens[s:s + T], dtype=np.int64))
            t = np.array(tokens[s + 1:s + 1 + T], dtype=np.int64)
            maskWindow(t, supervised, s + 1)
            tgs.append(t)
        return np.concatenate(ids), np.concatenate(tgs)

    out = []
    for windows in (False, True):
        m = buildModel(cfg, 9)
        for p in m.params():
            gpu.keepGradOnDevice(p)
        src = DeviceTokenSource(gpu, tokens, cfg.vocabSize, supervised) if windows else None
        step = CudaStep(m, gpu, B, T, capture=capture, source=src)
        res = []
        for starts in ([5, 300], [0, 400 - T - 1]):
            if windows:
                step.runWindows(starts)
            else:
                step.run(*host_windows(starts))
            res.append((step.losses().copy(), [gpu.readStateBuffer(gpu.buffersFor(p)["grad"], p.size) for p in m.params()]))
        gpu.sync([])
        out.append(res)
        if windows:
            with pytest.raises(ValueError, match="out of range"):
                step.runWindows([0, 400 - T])
    for (la, ga), (lb, gb) in zip(out[0], out[1]):
        assert np.array_equal(la, lb)
        for a, b in zip(ga, gb):
            assert np.array_equal(a, b)


@pytest.mark.parametrize("rows,cols", [(12, 20), (20, 12), (16, 16)])
def test_muon_host_side_two_steps_and_state(dev, oracle, rows, cols):
    """`MuonGpu` (src/backend/muon-gpu.ts:351-470) over two steps against the oracle's Muon (momentum 0.95, Nesterov, five
    Newton-Schulz steps), its auxiliary AdamW group, and the .optstate round trip through device buffers
    (tests/gpu-parity.ts:1040-1093)."""
    from gguf_trainer_b200.autograd import Tensor
    from gguf_trainer_b200.optim import MuonGpu, deserializeOptState, serializeOptState
    gpu, fake = dev
    rng = oracle.Mulberry32(0x4D4D)
    p = Tensor(rng.randn((rows, cols), 0.5), [rows, cols], True)
    aux = Tensor(rng.randn((9,), 0.5), [9], True)
    w = p.data.copy().reshape(rows, cols)
    buf = np.zeros((rows, cols), np.float32)
    opt = MuonGpu(gpu, [p], [aux], lr=0.05, momentum=0.95, nesterov=True, nsSteps=5, aux={"lr": 1e-3})
    for _ in range(2):
        g = rng.randn((rows, cols), 0.3)
        gpu.writeStateBuffer(gpu.buffersFor(p)["grad"], g)
        gpu.writeStateBuffer(gpu.buffersFor(aux)["grad"], rng.randn((9,), 0.1))
        opt.recordStep()
        oracle.muon_step_array(w, g, buf, 0.05, 0.95, True, 5)
    gpu.sync([p, aux])
    assert np.linalg.norm(p.data.reshape(rows, cols) - w) <= 1e-5 * np.linalg.norm(w)
    st = opt.exportState()
    assert np.allclose(st["muonMomentum"][0].reshape(rows, cols), buf, rtol=1e-5, atol=1e-6) and st["adamT"] == 2
    blob = serializeOptState(st)
    opt2 = MuonGpu(gpu, [Tensor(p.data.copy(), p.shape, True)], [Tensor(aux.data.copy(), aux.shape, True)], lr=0.05, aux={"lr": 1e-3})
    opt2.importState(deserializeOptState(blob))
    assert serializeOptState(opt2.exportState()) == blob
    assert fake.count("gt_muon_step") == 2 and fake.count("gt_adamw_step") == 2


def _trajectory(oracle, gpu, cfg, reclaim, loss_chunk=0, recompute=False, steps=3, seq=8, batch=3):
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.arch import buildModel
    from gguf_trainer_b200.optim import MuonGpu
    from gguf_trainer_b200.train import trainLMGpuResident
    rng_tok = oracle.Mulberry32(0x5EC1)
    tokens = np.array([int(rng_tok() * cfg.vocabSize) for _ in range(160)])
    ag.setCheckpointing(recompute)
    try:
        m = buildModel(cfg, 5)
        g = m.paramGroups()
        opt = MuonGpu(gpu, g["muon"], g["aux"], lr=0.02, momentum=0.95, aux={"lr": 3e-3, "weightDecay": 0.0, "clip": 1.0})
        hist = trainLMGpuResident(m, gpu, tokens, seq, steps, batch, opt, logEvery=1, rng=oracle.Mulberry32(7),
                                  reclaimTransients=reclaim, lossChunk=loss_chunk)
    finally:
        ag.setCheckpointing(False)
    return hist, [p.data.copy() for p in m.params()]


def test_training_loop_reclaim_recompute_and_chunked_loss(dev, oracle):
    """The step loop of src/backend/train-gpu.ts:162-258 (`trainLMGpuResident`: three Muon + AdamW steps of three
    micro-batches each, windows drawn as floor(rng() * maxStart)) on the stand-in, following tests/gpu-parity.ts:438-564:
    reclaiming the transients at every micro-batch boundary changes nothing, recompute gives the plain run's losses and
    parameters bit for bit, and the chunked loss follows the dense one."""
    gpu, _fake = dev
    cfg = ModelConfig("gemma3", 50, 32, 2, 4, 2, 8, 64, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0, slidingWindow=32, swaPattern=2)
    off = _trajectory(oracle, gpu, cfg, False)
    assert len(off[0]) == 3 and all(np.isfinite(h["loss"]) for h in off[0]) and off[0][-1]["loss"] < off[0][0]["loss"]
    for name, run in (("reclaim", _trajectory(oracle, gpu, cfg, True)), ("recompute", _trajectory(oracle, gpu, cfg, False, 0, True)),
                      ("recompute + reclaim", _trajectory(oracle, gpu, cfg, True, 0, True))):
        for a, b in zip(run[0], off[0]):
            assert a["loss"] == b["loss"], f"{name}, step {a['step']}: {a['loss']} vs {b['loss']}"
        for i, (a, b) in enumerate(zip(run[1], off[1])):
            assert np.array_equal(a, b), f"{name} changed parameter {i}"
    chunked = _trajectory(oracle, gpu, cfg, True, 16)
    for a, b in zip(chunked[0], off[0]):
        assert abs(a["loss"] - b["loss"]) <= 1e-5 * abs(b["loss"])
    for a, b in zip(chunked[1], off[1]):
        assert np.linalg.norm(a - b) <= 1e-4 * max(np.linalg.norm(b), 1e-30)


def test_checkpoint_taken_while_the_next_step_runs(oracle, monkeypatch):
    """`beginCheckpoint` after step k, `finish` after step k + 1 (src/backend/muon-gpu.ts:440-470 through the asynchronous
    read): the weights and the .optstate bytes are those of step k, although step k + 1 has overwritten both."""
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.arch import buildModel
    from gguf_trainer_b200.backend import CudaBackend
    from gguf_trainer_b200.optim import MuonGpu, deserializeOptState, serializeOptState
    from gguf_trainer_b200.train import sequenceLoss
    cfg = ModelConfig("gemma3", 50, 32, 2, 4, 2, 8, 64, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0, slidingWindow=32, swaPattern=2)
    tokens = oracle.Mulberry32(23).randint(400, cfg.vocabSize)

    def run(overlapped):
        fake_cabi.install(monkeypatch)
        gpu = CudaBackend(0, "fp32")
        try:
            m = buildModel(cfg, 5)
            g = m.paramGroups()
            opt = MuonGpu(gpu, g["muon"], g["aux"], lr=0.02, aux={"lr": 1e-2, "clip": 1.0, "weightDecay": 0.0})
            T, rng = 9, oracle.Mulberry32(7)

            def step():
                gpu.install()
                try:
                    st = int(rng() * (len(tokens) - T - 1))
                    loss = sequenceLoss(m, tokens[st:st + T], tokens[st + 1:st + 1 + T])
                    ag.backward(loss, 1.0)
                    gpu.sync([loss])
                finally:
                    gpu.uninstall()
                opt.recordStep()

            step(); step()
            if overlapped:
                ck = opt.beginCheckpoint()
                step()
                state = ck.finish()
            else:
                opt.syncWeightsToHost()
                state = opt.exportState()
            return [p.data.copy() for p in m.params()], serializeOptState(state)
        finally:
            gpu.destroy()

    w_sync, s_sync = run(False)
    w_late, s_late = run(True)
    for i, (a, b) in enumerate(zip(w_late, w_sync)):
        assert np.array_equal(a, b), f"weight {i}"
    assert s_late == s_sync and deserializeOptState(s_late)["adamT"] == 2


def test_clears_and_the_refusal_of_a_late_backward(dev):
    """tests/gpu-parity.ts:1752-1900: a training window clears fewer gradient buffers than there are parameters (first
    writers overwrite), a frozen model clears none, a forward-only window clears only what its sync stages back, and a
    backward over a graph that a sync has already recycled is refused."""
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.arch import buildModel
    from gguf_trainer_b200.train import freezeForScoring, sequenceLoss
    gpu, _fake = dev
    cfg = ModelConfig("gemma3", 64, 64, 2, 4, 2, 16, 256, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0, slidingWindow=16, swaPattern=2)
    ids = np.array([(i * 11 + 5) % cfg.vocabSize for i in range(33)])
    out = {}
    for freeze in (False, True):
        m = buildModel(cfg, 5)
        if freeze:
            freezeForScoring(m)
        gpu.install()
        try:
            gpu.uploadParams(m.params())

            def window():
                loss = sequenceLoss(m, ids[:-1], ids[1:], 0)
                ag.backward(loss, 1.0)
                gpu.sync([loss])
                return float(loss.data[0])

            window()
            before = gpu.gradClearsIssued
            out[freeze] = (window(), gpu.gradClearsIssued - before, len(m.params()))
        finally:
            gpu.uninstall()
    assert out[False][1] < out[False][2] and out[True][1] == 0 and out[False][0] == out[True][0]
    m = buildModel(cfg, 5)
    gpu.install()
    try:
        before = gpu.gradClearsIssued
        loss = sequenceLoss(m, ids[:-1], ids[1:], 0)
        gpu.sync([loss])
        assert gpu.gradClearsIssued - before == len(m.params())
        with pytest.raises(RuntimeError, match="graph built before a sync"):
            ag.backward(loss, 1.0)
    finally:
        gpu.uninstall()
