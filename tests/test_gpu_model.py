"""Whole-model parity on a B200: loss, per-layer activations, every gradient and post-step weights
against the CPU oracle on the same seed, inputs and weights; plus the behaviours the reference gates
(micro-batch accumulation, recompute bit-identity, LoRA, chunked loss, readback volume)."""
import numpy as np
import pytest

from gpu_harness import BWD, FWD, compare, rel_l2

pytestmark = pytest.mark.gpu

from gguf_trainer_b200 import autograd as ag
from gguf_trainer_b200.arch import ModelConfig, buildModel, tinyLlama
from gguf_trainer_b200.optim import AdamWGpu, MuonGpu
from gguf_trainer_b200.train import CudaStep, sequenceLoss, trainLMGpuResident


@pytest.fixture()
def gpu():
    from gguf_trainer_b200.backend import requireGPU
    g = requireGPU("the parity suite")
    yield g
    ag.setCheckpointing(False)
    g.destroy()


def micro_gemma():
    """tests/gpu-parity.ts:307-325 microConfig."""
    return ModelConfig("gemma3", 50, 32, 2, 4, 2, 8, 64, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0, slidingWindow=32,
                       swaPattern=2)


def tiny(arch, vocab=23):
    if arch == "llama":
        return ModelConfig("llama", vocab, 8, 2, 2, 1, 4, 16, 100_000.0, 1e-5)
    if arch == "qwen3":
        return ModelConfig("qwen3", vocab, 8, 2, 2, 1, 4, 16, 1_000_000.0, 1e-6)
    return ModelConfig("gemma3", vocab, 8, 2, 2, 1, 4, 16, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0, slidingWindow=4,
                       swaPattern=2)


def paired(oracle, cfg, seed):
    """An oracle model and a backend-side model holding the same weights."""
    om = oracle.Model(cfg.oracle_dict(), seed)
    m = buildModel(cfg, seed)
    ps = m.params()
    assert len(ps) == om.nparams()
    for i, p in enumerate(ps):
        assert tuple(p.shape) == om.info(i)["shape"]
        p.data[:] = om.data(i).reshape(-1)
    return om, m


def check_grads(om, m, l2=1e-5, tol=BWD):
    for i, p in enumerate(m.params()):
        compare(f"grad[{i}] {p.shape}", p.grad, om.grad(i), tol, l2)


@pytest.mark.parametrize("arch", ["llama", "qwen3", "gemma3"])
@pytest.mark.parametrize("chunk", [0, 5])
def test_tiny_model_loss_activations_grads(gpu, oracle, arch, chunk):
    cfg = tiny(arch)
    om, m = paired(oracle, cfg, 99)
    ids = oracle.Mulberry32(3).randint(9, cfg.vocabSize)
    tg = oracle.Mulberry32(4).randint(9, cfg.vocabSize)
    tg[2] = -1
    ref_loss = om.loss_backward(ids, tg, loss_chunk=chunk)
    gpu.install()
    try:
        loss = sequenceLoss(m, ids, tg, chunk)
        ag.backward(loss, 1.0)
        gpu.sync([loss] + m.layerOutputs + [m.lastHidden])
    finally:
        gpu.uninstall()
    assert abs(float(loss.data[0]) - float(ref_loss)) <= 1e-5 * max(1.0, abs(float(ref_loss)))
    for l, t in enumerate(m.layerOutputs + [m.lastHidden]):
        compare(f"layer {l} output", t.data, om.layer_out(l, 9), FWD)
    check_grads(om, m)


def test_config1_tiny_llama_full_step(gpu, oracle):
    """hidden 128, 2 layers, 4/2 heads, hd 32, ffn 384, vocab 512, batch 4 x seq 128, one forward +
    backward + AdamW step (lr 1e-3, betas 0.9/0.95, wd 0.1, clip 1.0): loss, every gradient, post-step weights."""
    cfg = tinyLlama()
    om, m = paired(oracle, cfg, 1234)
    B, T = 4, 128
    stream = oracle.Mulberry32(99).randint(B * (T + 1) * 2, cfg.vocabSize)
    rng = oracle.Mulberry32(7)
    starts = [int(rng() * (len(stream) - T - 1)) for _ in range(B)]
    om.make_optimizer("adamw", lr=1e-3, beta1=0.9, beta2=0.95, wd=0.1, clip=1.0)
    om.opt_zero_grad()
    ref_losses = [om.loss_backward(stream[s:s + T], stream[s + 1:s + 1 + T], seed=1.0 / B) for s in starts]
    opt = AdamWGpu(gpu, m.params(), lr=1e-3, beta1=0.9, beta2=0.95, weightDecay=0.1, clip=1.0)
    gpu.install()
    try:
        losses = []
        for s in starts:
            loss = sequenceLoss(m, stream[s:s + T], stream[s + 1:s + 1 + T])
            ag.backward(loss, 1.0 / B)
            losses.append(loss)
        gpu.sync(losses)
        assert gpu.lastSyncReadbackBytes == 4 * B   # tests/gpu-parity.ts:1671-1735: only the loss scalars
        grads = [gpu.readStateBuffer(gpu.buffersFor(p)["grad"], p.size) for p in m.params()]
        opt.recordStep()
        gpu.sync(m.params())
    finally:
        gpu.uninstall()
    for a, b in zip(losses, ref_losses):
        assert abs(float(a.data[0]) - float(b)) <= 1e-5 * abs(float(b))
    for i, g in enumerate(grads):
        compare(f"grad[{i}]", g, om.grad(i), BWD)
    om.opt_step()
    # AdamW's first update is g/(|g|+eps), a sign function wherever |g| >> 1e-8: an element whose gradient
    # sits at the f32 rounding floor of its own accumulation can land on either side, which moves that
    # weight by up to 2*lr whatever the kernels do. Gradients above are held to 1e-5; the stepped weights
    # to the element tolerances and 5e-5 relative L2 (tests/test_gpu_optim.py holds the update itself to
    # 1e-6 when both sides are fed identical gradients).
    for i, p in enumerate(m.params()):
        compare(f"post-step weight[{i}]", p.data, om.data(i), FWD, 5e-5)


def test_two_micro_batch_accumulation(gpu, oracle):
    """tests/gpu-parity.ts:395-428."""
    cfg = micro_gemma()
    om, m = paired(oracle, cfg, 5)
    rng = oracle.Mulberry32(23)
    T = 9
    batches = [(rng.randint(T, cfg.vocabSize), rng.randint(T, cfg.vocabSize)) for _ in range(2)]
    for ids, tg in batches:
        om.loss_backward(ids, tg, seed=0.5)
    gpu.install()
    try:
        for ids, tg in batches:
            ag.backward(ag.crossEntropy(m.forward(ids), tg), 0.5)
        gpu.sync([])
    finally:
        gpu.uninstall()
    check_grads(om, m)


@pytest.mark.parametrize("arch", ["llama", "qwen3", "gemma3"])
def test_recompute_is_bit_identical(gpu, oracle, arch):
    """tests/gpu-parity.ts:536-564, 1299-1338."""
    cfg = tiny(arch)
    ids = oracle.Mulberry32(3).randint(12, cfg.vocabSize)
    tg = oracle.Mulberry32(4).randint(12, cfg.vocabSize)
    outs = []
    for on in (False, True):
        _, m = paired(oracle, cfg, 77)
        ag.setCheckpointing(on)
        regions = gpu.regionCount()
        gpu.install()
        try:
            loss = sequenceLoss(m, ids, tg)
            ag.backward(loss, 1.0)
            gpu.sync([loss])
        finally:
            gpu.uninstall()
            ag.setCheckpointing(False)
        assert (gpu.regionCount() > regions) == on
        outs.append((loss.data.copy(), [p.grad.copy() for p in m.params()]))
    assert np.array_equal(outs[0][0], outs[1][0])
    for a, b in zip(outs[0][1], outs[1][1]):
        compare("recompute grad", b, a, BWD, 1e-6)


def test_recompute_keeps_attention_outputs(gpu, oracle):
    """A recompute region's replay takes the first run's attention output instead of launching the kernel again:
    one launch fewer per layer, same loss bit for bit and the same gradients as the replay that recomputes everything."""
    cfg = tiny("qwen3")
    ids = oracle.Mulberry32(5).randint(12, cfg.vocabSize)
    tg = oracle.Mulberry32(6).randint(12, cfg.vocabSize)
    was = gpu.keepAttentionAcrossRecompute
    outs, launches = [], []
    try:
        for keep in (False, True):
            gpu.keepAttentionAcrossRecompute = keep
            _, m = paired(oracle, cfg, 78)
            ag.setCheckpointing(True)
            before = gpu.kernelLaunches()
            gpu.install()
            try:
                loss = sequenceLoss(m, ids, tg)
                ag.backward(loss, 1.0)
                gpu.sync([loss])
            finally:
                gpu.uninstall()
                ag.setCheckpointing(False)
            launches.append(gpu.kernelLaunches() - before)
            outs.append((loss.data.copy(), [p.grad.copy() for p in m.params()]))
    finally:
        gpu.keepAttentionAcrossRecompute = was
    saved = launches[0] - launches[1]
    # (the first of the two runs may also build a RoPE table once)
    assert len(m.layers) <= saved <= len(m.layers) + 2, f"launches {launches}, layers {len(m.layers)}"
    assert np.array_equal(outs[0][0], outs[1][0])
    for a, b in zip(outs[0][1], outs[1][1]):
        compare("gradient with kept attention outputs", b, a, BWD, 1e-6)   # (f32 atomics in dw: not bit-stable run to run)


@pytest.mark.parametrize("fused,alpha", [(True, 8.0), (False, 8.0), (True, 5.0)])
def test_lora_parity_and_frozen_base(gpu, oracle, fused, alpha):
    """tests/gpu-parity.ts:2037-2138: adapters train, the base stays frozen and gets no gradient. Both recordings of
    the adapter-carrying projection: as one op (with a scale that is, and one that is not, a power of two) and as
    the reference's four."""
    from gguf_trainer_b200.lora import applyLora, clearLora
    from gguf_trainer_b200.rng import Mulberry32
    cfg = tiny("qwen3")
    om, m = paired(oracle, cfg, 31)
    n_ad = om.apply_lora(4, alpha, 4321)
    h = applyLora(m, 4, alpha, Mulberry32(4321))
    was = gpu.fuseLora
    gpu.fuseLora = fused
    try:
        assert len(h.groups["aux"]) == n_ad
        base_n = len(m.params())
        rng = oracle.Mulberry32(17)
        for j, t in enumerate(h.groups["aux"]):
            if j % 2 == 1:  # B starts at zero; give it values so both factors see gradient
                t.data[:] = rng.randn((t.size,), 0.05)
            om.data(base_n + j)[...] = t.data.reshape(om.info(base_n + j)["shape"])
        ids = oracle.Mulberry32(3).randint(10, cfg.vocabSize)
        tg = oracle.Mulberry32(4).randint(10, cfg.vocabSize)
        ref = om.loss_backward(ids, tg)
        gpu.install()
        try:
            loss = sequenceLoss(m, ids, tg)
            ag.backward(loss, 1.0)
            gpu.sync([loss])
        finally:
            gpu.uninstall()
        assert abs(float(loss.data[0]) - float(ref)) <= 1e-5 * abs(float(ref))
        for j, t in enumerate(h.groups["aux"]):
            compare(f"adapter grad {j}", t.grad, om.grad(base_n + j), BWD)
        for p in m.params():
            assert not p.grad.any()
        # merge/unmerge drift (gpu-parity.ts:2120-2138)
        before = [p.data.copy() for p in m.params()]
        h.merge(); h.unmerge()
        for a, p in zip(before, m.params()):
            assert np.abs(a - p.data).max() <= 1e-5
    finally:
        gpu.fuseLora = was
        clearLora(m)


def test_batched_call_equals_sequential_micro_batches(gpu, oracle):
    """B sequences as one [B*T]-row call give the reference's B micro-batches seeded 1/B, including
    per-sequence loss denominators under a loss mask, and a replayed graph gives the same numbers."""
    cfg = tiny("gemma3", vocab=40)
    B, T = 3, 10
    om, m = paired(oracle, cfg, 11)
    rng = oracle.Mulberry32(2)
    ids = rng.randint(B * T, cfg.vocabSize)
    tg = rng.randint(B * T, cfg.vocabSize)
    tg[0:4] = -1          # sequences keep 6, 10, 7 rows
    tg[2 * T + 1:2 * T + 4] = -1
    ref_losses = [om.loss_backward(ids[b * T:(b + 1) * T], tg[b * T:(b + 1) * T], seed=1.0 / B) for b in range(B)]
    for capture in (False, True):
        _, m = paired(oracle, cfg, 11)
        for p in m.params():
            gpu.keepGradOnDevice(p)
        step = CudaStep(m, gpu, B, T, capture=capture)
        step.run(ids, tg)
        if capture:
            step.run(ids, tg)   # second call is a pure replay
        got = step.losses()
        assert abs(got[0] - np.mean([float(x) for x in ref_losses])) <= 1e-5
        for b in range(B):
            assert abs(got[1 + b] - float(ref_losses[b])) <= 1e-5 * abs(float(ref_losses[b]))
        for i, p in enumerate(m.params()):
            g = gpu.readStateBuffer(gpu.buffersFor(p)["grad"], p.size)
            compare(f"batched grad[{i}] capture={capture}", g, om.grad(i), BWD)
        gpu.sync([])


def test_muon_trajectory_matches_reference_loop(gpu, oracle):
    """tests/gpu-parity.ts:1104-1289: 4 steps of Muon + AdamW under a WSD schedule against the CPU loop."""
    from gguf_trainer_b200.schedule import wsdSchedule
    cfg = micro_gemma()
    om, m = paired(oracle, cfg, 5)
    T, B, steps = 9, 2, 4
    tokens = oracle.Mulberry32(23).randint(200, cfg.vocabSize)
    sched = wsdSchedule(2, 0, 2, 0.1)
    om.make_optimizer("muon", lr=0.02, aux_lr=1e-2, clip=1.0, wd=0.0)
    ref_hist = []
    r = oracle.Mulberry32(7)
    maxStart = len(tokens) - T - 1
    for s in range(steps):
        om.opt_set_lr_scale(sched(s))
        om.opt_zero_grad()
        tot = 0.0
        for _ in range(B):
            st = int(r() * maxStart)
            tot += float(om.loss_backward(tokens[st:st + T], tokens[st + 1:st + 1 + T], seed=1.0 / B))
        om.opt_step()
        ref_hist.append(tot / B)
    g = m.paramGroups()
    opt = MuonGpu(gpu, g["muon"], g["aux"], lr=0.02, aux={"lr": 1e-2, "clip": 1.0, "weightDecay": 0.0})
    hist = trainLMGpuResident(m, gpu, tokens, T, steps, B, opt, logEvery=1, rng=oracle.Mulberry32(7), schedule=sched)
    for h, want in zip(hist, ref_hist):
        assert abs(h["loss"] - want) <= 1e-3 + 1e-3 * abs(want)   # gpu-parity.ts:1141-1142
    for i, p in enumerate(m.params()):
        compare(f"weight[{i}] after {steps} steps", p.data, om.data(i), dict(atol=2e-3, rtol=2e-2), None)


@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_gated_unit_fusion_matches_the_two_op_form(gpu, oracle, act):
    """silu(g)*u / gelu(g)*u run as one kernel; the result must be what the two reference ops give, including when
    the activated gate is also used elsewhere and when both factors are the same tensor."""
    from gpu_harness import rand_tensor
    rng = oracle.Mulberry32(61)
    g = rand_tensor(rng, [37, 50], 1.5); u = rand_tensor(rng, [37, 50])
    f = ag.silu if act == "silu" else ag.gelu
    up = oracle.Mulberry32(0xBEEF).uniform_pm1((g.size,))
    act_v, dact, _ = oracle.elementwise(act, g.data, gy=np.ones(g.size, np.float32))
    # plain gated unit
    launches = gpu.kernelLaunches()
    gpu.install()
    try:
        out = ag.mul(f(g), u)
        out.grad[:] = up
        gpu.seedGradFromHost(out)
        # run the closures in reverse creation order: product first, then the activation
        out._backward()
        out._prev[0]._backward()
        gpu.sync([out])
    finally:
        gpu.uninstall()
    assert gpu.kernelLaunches() - launches == 2          # one fused forward, one fused backward
    compare("glu out", out.data, act_v.astype(np.float64) * u.data, FWD)
    compare("glu d gate", g.grad, up.astype(np.float64) * u.data * dact, BWD)
    compare("glu d up", u.grad, up.astype(np.float64) * act_v, BWD)
    # the activated gate has a second consumer: it is materialised and its own backward carries that share
    g.zeroGrad(); u.zeroGrad()
    gpu.install()
    try:
        a = f(g)
        out = ag.add(ag.mul(a, u), a)
        loss_up = up
        out.grad[:] = loss_up
        gpu.seedGradFromHost(out)
        out._backward()                  # add
        out._prev[0]._backward()         # fused product
        a._backward()                    # activation (share from the add)
        gpu.sync([out])
    finally:
        gpu.uninstall()
    compare("shared out", out.data, act_v.astype(np.float64) * u.data + act_v, FWD)
    compare("shared d gate", g.grad, up.astype(np.float64) * (u.data + 1.0) * dact, BWD)
    compare("shared d up", u.grad, up.astype(np.float64) * act_v, BWD)
