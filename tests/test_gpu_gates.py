"""Device-behaviour gates of the backend that no numeric comparison can see: what a forward-only window stages and
allocates (tests/gpu-parity.ts:1430-1487), what `reclaimStepTransients` and recompute do to trajectories and to the
pool (:438-565, :1363-1421), how many gradient clears a window issues (:1752-1900), the per-label profiler (:134-156),
checkpoints copied out while the next step runs (muon-gpu.ts:440-470), and run-to-run bit equality in strict-f32
mode."""
import numpy as np
import pytest

from gpu_harness import BWD, compare

pytestmark = pytest.mark.gpu

from gguf_trainer_b200 import autograd as ag
from gguf_trainer_b200.arch import ModelConfig, buildModel
from gguf_trainer_b200.backend import requireGPU
from gguf_trainer_b200.optim import AdamWGpu, MuonGpu, deserializeOptState, serializeOptState
from gguf_trainer_b200.train import freezeForScoring, sequenceLoss, trainLMGpuResident


def gemma3_config(vocab, hidden, heads, ffn, head_dim, layers=2):
    """tests/gpu-parity.ts gemma3Config(vocab, hidden, heads, ffn, headDim)."""
    return ModelConfig("gemma3", vocab, hidden, layers, heads, max(1, heads // 2), head_dim, ffn, 1_000_000.0, 1e-6,
                       ropeBaseLocal=10_000.0, slidingWindow=16, swaPattern=2)


def micro_gemma():
    return ModelConfig("gemma3", 50, 32, 2, 4, 2, 8, 64, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0, slidingWindow=32,
                       swaPattern=2)


@pytest.mark.parametrize("loss_chunk", [0, 64])
def test_forward_only_window_reads_back_four_bytes_and_allocates_no_gradients(loss_chunk):
    """tests/gpu-parity.ts:1430-1487 (eval-loss): frozen, a scoring window stages only the loss scalar and the pool is
    smaller by about the model; the score does not move."""
    cfg = gemma3_config(64, 64, 4, 256, 16)
    ids = np.array([(i * 11 + 5) % cfg.vocabSize for i in range(65)])

    def arm(freeze):
        gpu = requireGPU("the freeze gate")
        m = buildModel(cfg, 5)
        try:
            if freeze:
                freezeForScoring(m)     # before uploadParams on purpose: the entry is sized on first use
            gpu.install()
            gpu.uploadParams(m.params())
            loss = sequenceLoss(m, ids[:-1], ids[1:], loss_chunk)
            gpu.sync([loss])
            return dict(readback=gpu.lastSyncReadbackBytes, pool=gpu.residentBytes()["pool"], loss=float(loss.data[0]),
                        paramBytes=sum(t.size * 4 for t in m.params()), clears=gpu.gradClearsIssued)
        finally:
            gpu.destroy()

    hot, cold = arm(False), arm(True)
    assert hot["readback"] >= hot["paramBytes"]                 # the unfrozen arm stages a model of gradients
    assert cold["readback"] == 4                                 # frozen: the loss scalar only
    assert cold["pool"] < hot["pool"] - 0.9 * hot["paramBytes"]  # and the accumulators are not allocated
    assert hot["loss"] == cold["loss"]
    assert cold["clears"] == 0                                   # a forward-only frozen window zeroes nothing


def test_decode_loop_reads_back_only_the_last_logits():
    """tests/gpu-parity.ts:1497-1551 (generate): a greedy decode loop syncs once per token; frozen, each sync stages the
    logits it asked for and nothing else, and the generated ids do not move."""
    cfg = gemma3_config(64, 64, 4, 256, 16)
    prompt, max_new = [3, 11, 29, 5], 3

    def arm(freeze):
        gpu = requireGPU("the generate gate")
        m = buildModel(cfg, 5)
        try:
            if freeze:
                freezeForScoring(m)
            gpu.install()
            gpu.uploadParams(m.params())
            ctx = list(prompt)
            for _ in range(max_new):
                logits = m.forward(np.array(ctx))
                gpu.sync([logits])
                last = logits.data.reshape(len(ctx), cfg.vocabSize)[-1]
                ctx.append(int(np.argmax(last)))
            return dict(readback=gpu.lastSyncReadbackBytes, pool=gpu.residentBytes()["pool"], ids=ctx,
                        paramBytes=sum(t.size * 4 for t in m.params()))
        finally:
            gpu.destroy()

    hot, cold = arm(False), arm(True)
    last_logits = (len(prompt) + max_new - 1) * cfg.vocabSize * 4
    assert hot["readback"] >= hot["paramBytes"]
    assert cold["readback"] == last_logits
    assert cold["pool"] < hot["pool"] - 0.9 * hot["paramBytes"]
    assert hot["ids"] == cold["ids"]


def test_clears_per_window_and_late_backward_refusal():
    """tests/gpu-parity.ts:1752-1900. This backend never clears a buffer whose first writer can overwrite it, so a
    training window issues no clear per parameter or per intermediate at all: only a gradient that is read before
    anything wrote it (none in a language-model step) or scatter-added into first (the embedding table when it is not
    tied to the readout). A forward-only window clears nothing but the accumulators of trainable parameters that its
    sync is about to stage back unwritten (one each, none when frozen), and a backward over a graph that a sync has
    already recycled is refused."""
    cfg = gemma3_config(64, 64, 4, 256, 16)
    ids = np.array([(i * 11 + 5) % cfg.vocabSize for i in range(33)])
    out = {}
    for freeze in (False, True):
        gpu = requireGPU("the clear gate")
        m = buildModel(cfg, 5)
        try:
            if freeze:
                freezeForScoring(m)
            gpu.install()
            gpu.uploadParams(m.params())

            def window():
                loss = sequenceLoss(m, ids[:-1], ids[1:], 0)
                ag.backward(loss, 1.0)
                gpu.sync([loss])
                return float(loss.data[0])

            window()
            before = gpu.gradClearsIssued
            loss = window()
            out[freeze] = (gpu.gradClearsIssued - before, loss, len(m.params()))
        finally:
            gpu.destroy()
    hot, cold = out[False], out[True]
    assert hot[0] < hot[2], f"{hot[0]} clears for {hot[2]} parameters: the first writer should overwrite instead"
    assert cold[0] == 0
    assert hot[1] == cold[1]
    # forward only, then a backward after the sync that recycled the graph
    gpu = requireGPU("the clear gate")
    m = buildModel(cfg, 5)
    try:
        gpu.install()
        before = gpu.gradClearsIssued
        loss = sequenceLoss(m, ids[:-1], ids[1:], 0)
        gpu.sync([loss])
        assert gpu.gradClearsIssued - before == len(m.params())      # staged-back accumulators only: no intermediate
        with pytest.raises(RuntimeError, match="graph built before a sync"):
            ag.backward(loss, 1.0)
    finally:
        gpu.destroy()
    # an optimizer built and synced with no graph at all must not arm that refusal
    gpu = requireGPU("the clear gate")
    m = buildModel(cfg, 5)
    try:
        gpu.install()
        g = m.paramGroups()
        MuonGpu(gpu, g["muon"], g["aux"], lr=0.01, aux={"lr": 3e-3, "weightDecay": 0.0, "clip": 1.0})
        gpu.sync([])
        gpu.seedGradFromHost(g["muon"][0])
    finally:
        gpu.destroy()


def _trajectory(oracle, gpu, cfg, reclaim, loss_chunk=0, recompute=False, steps=4, seq=8, batch=3):
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


def test_reclaim_and_recompute_trajectories(oracle):
    """tests/gpu-parity.ts:438-564: four Muon steps of three micro-batches. Reclaiming transients at every micro-batch
    boundary changes nothing; the chunked loss across those boundaries matches the dense one; and with recompute the
    loss trajectory is BIT-identical to the plain run (strict-f32 mode: every reduction has a fixed order)."""
    cfg = micro_gemma()
    gpu = requireGPU("the trajectory gate")
    try:
        off = _trajectory(oracle, gpu, cfg, False)
        on = _trajectory(oracle, gpu, cfg, True)
        for a, b in zip(on[0], off[0]):
            assert a["loss"] == b["loss"], f"step {a['step']}: reclaim on {a['loss']} vs off {b['loss']}"
        for i, (a, b) in enumerate(zip(on[1], off[1])):
            assert np.array_equal(a, b), f"reclaim changed parameter {i}"
        ch_off = _trajectory(oracle, gpu, cfg, False, 16)
        ch_on = _trajectory(oracle, gpu, cfg, True, 16)
        for a, b, c in zip(ch_off[0], ch_on[0], off[0]):
            assert a["loss"] == b["loss"]
            assert abs(a["loss"] - c["loss"]) <= 1e-3 + 1e-3 * abs(c["loss"])
        for i, (a, b, c) in enumerate(zip(ch_off[1], ch_on[1], off[1])):
            assert np.array_equal(a, b)
            compare(f"chunked vs dense parameter {i}", a, c, BWD, None)
        rc_off = _trajectory(oracle, gpu, cfg, False, 0, True)
        rc_on = _trajectory(oracle, gpu, cfg, True, 0, True)
        for a, b, c in zip(rc_off[0], rc_on[0], off[0]):
            assert a["loss"] == c["loss"], f"step {a['step']}: recompute {a['loss']} vs plain {c['loss']}"
            assert b["loss"] == c["loss"], f"step {b['step']}: recompute + reclaim {b['loss']} vs plain {c['loss']}"
        for i, (a, c) in enumerate(zip(rc_on[1], off[1])):
            assert np.array_equal(a, c), f"recompute changed parameter {i}"
    finally:
        gpu.destroy()


@pytest.mark.parametrize("arch", ["llama", "qwen3", "gemma3"])
def test_strict_f32_step_is_bit_identical_run_to_run(oracle, arch):
    """Two runs of the same three steps x two micro-batches (recompute off and on) end in the same bits: losses and
    every parameter. No reduction in strict-f32 mode depends on scheduling (the reference's one-owner-per-gradient-
    element rule, src/backend/webgpu.ts:21-26)."""
    cfg = {"llama": ModelConfig("llama", 97, 64, 3, 4, 2, 16, 192, 100_000.0, 1e-5),
           "qwen3": ModelConfig("qwen3", 97, 64, 3, 4, 2, 16, 192, 1_000_000.0, 1e-6),
           "gemma3": ModelConfig("gemma3", 97, 64, 3, 4, 2, 16, 192, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0,
                                 slidingWindow=24, swaPattern=3)}[arch]
    tokens = oracle.Mulberry32(0xD37).randint(4000, cfg.vocabSize)
    # repeated ids inside a window (the ordered scatter-add) and rows >> CTAs (the ordered dw reduction)
    tokens[::3] = 7
    runs = []
    for recompute in (False, False, True):
        gpu = requireGPU("the determinism gate")
        try:
            ag.setCheckpointing(recompute)
            m = buildModel(cfg, 11)
            opt = AdamWGpu(gpu, m.params(), lr=1e-3, beta1=0.9, beta2=0.95, weightDecay=0.1, clip=1.0)
            hist = trainLMGpuResident(m, gpu, tokens, 1100, 3, 2, opt, logEvery=1, rng=oracle.Mulberry32(7))
            runs.append(([h["loss"] for h in hist], [p.data.copy() for p in m.params()]))
        finally:
            ag.setCheckpointing(False)
            gpu.destroy()
    for other, what in ((runs[1], "second run"), (runs[2], "recompute run")):
        assert runs[0][0] == other[0], f"{what}: losses {other[0]} vs {runs[0][0]}"
        for i, (a, b) in enumerate(zip(runs[0][1], other[1])):
            assert np.array_equal(a, b), f"{what}: parameter {i} differs"


def test_recompute_pool_is_flat_in_steps_and_micro_batches(oracle):
    """tests/gpu-parity.ts:1363-1421: with recompute the pool does not grow with the step count (sync drains it) nor
    with the micro-batch count under reclaim, and it is smaller than the dense run's."""
    cfg = gemma3_config(64, 64, 4, 256, 16)
    tokens = np.array([(i * 7 + 3) % cfg.vocabSize for i in range(8192)])

    def pool_for(recompute, reclaim, steps, batch):
        gpu = requireGPU("the memory gate")
        ag.setCheckpointing(recompute)
        try:
            m = buildModel(cfg, 5)
            g = m.paramGroups()
            opt = MuonGpu(gpu, g["muon"], g["aux"], lr=0.01, momentum=0.95, aux={"lr": 3e-3, "weightDecay": 0.0, "clip": 1.0})
            trainLMGpuResident(m, gpu, tokens, 128, steps, batch, opt, logEvery=100, rng=oracle.Mulberry32(7),
                               reclaimTransients=reclaim)
            return gpu.residentBytes()["pool"]
        finally:
            ag.setCheckpointing(False)
            gpu.destroy()

    s2, s6 = pool_for(True, False, 2, 2), pool_for(True, False, 6, 2)
    assert s6 <= s2 * 1.01, f"pool grows with steps: {s2} -> {s6}"
    b2, b4 = pool_for(True, True, 3, 2), pool_for(True, True, 3, 4)
    assert b4 <= b2 * 1.05, f"pool grows with micro-batches under reclaim: {b2} -> {b4}"
    dense = pool_for(False, True, 3, 2)
    assert b2 < 0.9 * dense, f"recompute pool {b2} not under dense {dense}"


def test_resident_bytes_counts_pool_and_state_separately():
    """webgpu.ts:774-777: pooled bytes and optimizer/state bytes are reported apart and add up."""
    gpu = requireGPU("the residency gate")
    try:
        r0 = gpu.residentBytes()
        a = gpu._acquirePersistent(1000)          # pooled: rounded to 256-byte buckets
        b = gpu.createStateBuffer(5000)           # state: never pooled
        r1 = gpu.residentBytes()
        assert r1["pool"] - r0["pool"] == 1024 and r1["state"] - r0["state"] == 5120
        assert r1["total"] == r1["pool"] + r1["state"]
        gpu._check(gpu.lib.gt_free(gpu.ctx, a))
        assert gpu.residentBytes()["pool"] == r1["pool"]      # a high-water mark: freed blocks stay pooled
        gpu._check(gpu.lib.gt_free(gpu.ctx, b))
        assert gpu.residentBytes()["state"] == r0["state"]
    finally:
        gpu.destroy()


def test_profiler_attributes_time_to_entry_points(oracle):
    """tests/gpu-parity.ts:134-156: a profiled forward attributes time to the right labels with sane counts, and
    profiling does not change results."""
    from gpu_harness import rand_tensor
    gpu = requireGPU("the profiler gate")
    try:
        x = rand_tensor(oracle.Mulberry32(5), [40, 48])
        w = rand_tensor(oracle.Mulberry32(6), [40, 48])
        gpu.install()
        y0 = ag.silu(ag.linear(x, w))
        gpu.sync([y0])
        gpu.startProfile()
        y = ag.silu(ag.linear(x, w))
        gpu.sync([y])
        prof = gpu.stopProfile()
        labels = set(prof)
        assert any(k.startswith("gt_gemm") for k in labels) and "gt_ew_fwd" in labels
        assert all(v["ms"] >= 0 and v["count"] > 0 for v in prof.values())
        assert np.array_equal(y.data, y0.data)
        assert gpu.stopProfile() == {}            # closed: nothing more is attributed
    finally:
        gpu.destroy()


def test_checkpoint_copied_out_while_the_next_step_runs(oracle):
    """muon-gpu.ts:440-470 (syncWeightsToHost + exportState) through gt_read_async: a checkpoint started after step k
    and finished after step k+1 has been enqueued holds exactly the weights and optimizer state of step k, byte for
    byte in the .optstate format, although step k+1 has overwritten both on the device meanwhile."""
    cfg = micro_gemma()
    tokens = oracle.Mulberry32(23).randint(400, cfg.vocabSize)

    def run(async_ckpt):
        gpu = requireGPU("the checkpoint gate")
        try:
            m = buildModel(cfg, 5)
            g = m.paramGroups()
            opt = MuonGpu(gpu, g["muon"], g["aux"], lr=0.02, aux={"lr": 1e-2, "clip": 1.0, "weightDecay": 0.0})
            T = 9
            rng = oracle.Mulberry32(7)

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
            if async_ckpt:
                ck = opt.beginCheckpoint()     # as of step 2
                step()                         # step 3 runs (and overwrites weights and moments) while it is copied out
                state = ck.finish()
            else:
                opt.syncWeightsToHost()
                state = opt.exportState()
            return [p.data.copy() for p in m.params()], serializeOptState(state)
        finally:
            gpu.destroy()

    w_sync, s_sync = run(False)
    w_async, s_async = run(True)
    for i, (a, b) in enumerate(zip(w_async, w_sync)):
        assert np.array_equal(a, b), f"weight {i} of the overlapped checkpoint differs from the one taken at a sync"
    assert s_async == s_sync
    back = deserializeOptState(s_async)
    assert back["adamT"] == 2


def test_scratch_growth_keeps_captured_graphs_valid(oracle):
    """A recorded graph has the address of the context's scratch block (attention backward's per-row dot products)
    in its kernel nodes. When a later, larger shape makes that block grow, the old block is retired, not freed, so
    replaying the graph still reads and writes memory that is its own."""
    import ctypes as C
    gpu = requireGPU("the scratch gate")
    lib, ctx = gpu.lib, gpu.ctx
    try:
        T, Hq, Hkv, hd = 64, 4, 2, 16
        rng = oracle.Mulberry32(21)

        def dev(a):
            b = gpu.createStateBuffer(a.nbytes)
            gpu.writeStateBuffer(b, a)
            return b

        q, k, v = rng.randn((T, Hq * hd), 0.8), rng.randn((T, Hkv * hd), 0.8), rng.randn((T, Hkv * hd), 0.8)
        go = rng.uniform_pm1((T, Hq * hd))
        dq, dk, dv, dgo = dev(q), dev(k), dev(v), dev(go)
        out, lse = gpu.createStateBuffer(q.nbytes), gpu.createStateBuffer(Hq * T * 4)
        gq, gk, gv = (gpu.createStateBuffer(x.nbytes) for x in (q, k, v))
        bwd = lambda: gpu._check(lib.gt_attention_bwd(ctx, T, Hq, Hkv, hd, 0, dq, dk, dv, out, lse, dgo, gq, 0, gk, 0, gv, 0))
        gpu._check(lib.gt_attention_fwd(ctx, T, Hq, Hkv, hd, 0, dq, dk, dv, out, lse))
        bwd()                                                   # eager once: the scratch block exists
        want = [gpu.readStateBuffer(b, x.size) for b, x in ((gq, q), (gk, k), (gv, v))]
        gpu._check(lib.gt_graph_begin(ctx))
        bwd()
        h = C.c_uint64()
        gpu._check(lib.gt_graph_end(ctx, C.byref(h)))
        # a shape whose dot products (rows * Hq floats) outgrow the 8 MiB block: 256 sequences of 128 rows, 80 heads
        B2, T2, H2 = 256, 128, 80
        rows = B2 * T2
        big = gpu.createStateBuffer(rows * H2 * 8 * 4)
        stat = gpu.createStateBuffer(H2 * rows * 4)
        gbig = gpu.createStateBuffer(rows * H2 * 8 * 4)
        gpu.setBatch(B2, T2)
        gpu._check(lib.gt_attention_fwd(ctx, rows, H2, H2, 8, 0, big, big, big, gbig, stat))
        gpu._check(lib.gt_attention_bwd(ctx, rows, H2, H2, 8, 0, big, big, big, gbig, stat, big, gbig, 0, 0, 0, 0, 0))
        gpu.setBatch(0)
        gpu.sync([])
        for b, x in ((gq, q), (gk, k), (gv, v)):
            gpu._check(lib.gt_zero(ctx, b, x.nbytes))
        gpu._check(lib.gt_graph_launch(ctx, int(h.value)))
        got = [gpu.readStateBuffer(b, x.size) for b, x in ((gq, q), (gk, k), (gv, v))]
        gpu.sync([])
        for a, b in zip(got, want):
            assert np.array_equal(a, b)
        gpu._check(lib.gt_graph_destroy(ctx, int(h.value)))
    finally:
        gpu.destroy()


def test_bf16_mode_is_refused_not_relabelled():
    """GT_PREC_BF16 is reserved in the header; asking for it answers GT_ERR_UNSUPPORTED and leaves the mode alone."""
    gpu = requireGPU("the precision gate", precision="tf32")
    try:
        st = gpu.lib.gt_set_precision(gpu.ctx, 2)
        assert st == 6 and b"no BF16 kernels" in gpu.lib.gt_last_error(gpu.ctx)
        with pytest.raises(KeyError):
            gpu.setPrecision("bf16")
        assert gpu.precision == "tf32"
    finally:
        gpu.destroy()


def test_replayed_inputs_are_range_checked(oracle):
    """The recorded kernels index the embedding table and the logits with the replayed integers and have no bound of
    their own: an id outside the vocabulary, or a target that is neither -1 nor a vocabulary row, is refused on the
    host before anything is written (the eager ops' checks, src/model/autograd.ts:813-823, 875-894)."""
    from gguf_trainer_b200.train import CudaStep
    cfg = ModelConfig("llama", 23, 8, 2, 2, 1, 4, 16, 100_000.0, 1e-5)
    gpu = requireGPU("the replay gate")
    try:
        m = buildModel(cfg, 3)
        for p in m.params():
            gpu.keepGradOnDevice(p)
        step = CudaStep(m, gpu, 2, 6)
        ids = oracle.Mulberry32(3).randint(12, cfg.vocabSize)
        tg = oracle.Mulberry32(4).randint(12, cfg.vocabSize)
        step.run(ids, tg)
        good = step.losses().copy()
        for bad_ids, bad_tg, msg in ((np.where(np.arange(12) == 5, 23, ids), tg, "id 23 at position 5"),
                                     (np.where(np.arange(12) == 0, -1, ids), tg, "id -1 at position 0"),
                                     (ids, np.where(np.arange(12) == 7, 23, tg), "value 23 at position 7"),
                                     (ids, np.where(np.arange(12) == 2, -2, tg), "value -2 at position 2")):
            with pytest.raises(ValueError, match=msg):
                step.run(bad_ids, bad_tg)
        tg2 = tg.copy(); tg2[3] = -1                               # -1 stays a legal target
        step.run(ids, tg2)
        step.run(ids, tg)
        assert np.array_equal(step.losses(), good)                 # and a refused call left the recorded inputs untouched
        gpu.sync([])
    finally:
        gpu.destroy()


def test_bounded_wait_expires_and_is_reported_at_the_next_sync():
    """Every mbarrier wait in the tensor-core kernels gives up after a time limit, raises a device flag and lets the
    kernel return; gt_sync turns the flag into an error. Exercised on a barrier nothing arrives on, with a 2 ms limit:
    the kernel returns by itself, the sync reports the expiry once, and the context works afterwards."""
    import time
    from gguf_trainer_b200 import _lib
    gpu = requireGPU("the bounded-wait gate", precision="tf32")
    try:
        gpu.sync([])
        t0 = time.perf_counter()
        gpu._check(gpu.lib.gt_selftest_bounded_wait(gpu.ctx, 2000))
        with pytest.raises(_lib.GtError, match="a pipeline wait expired \\(code 99\\)"):
            gpu.sync([])
        assert time.perf_counter() - t0 < 1.0          # gave up after ~2 ms, not after the kernels' 2 s
        gpu.sync([])                                    # reported once; the flag is clear again
        a = gpu.createStateBuffer(64 * 64 * 4)
        c = gpu.createStateBuffer(64 * 64 * 4)
        gpu.writeStateBuffer(a, np.eye(64, dtype=np.float32))
        gpu._gemm("NT", 0, 64, 64, 64, a, a, c)         # and the tensor-core path still runs
        assert np.allclose(gpu.readStateBuffer(c, 64 * 64).reshape(64, 64), np.eye(64), atol=2e-3)
        gpu.sync([])
    finally:
        gpu.destroy()


def test_exchange_wait_on_the_host_returns_when_the_reductions_are_done():
    """gt_dp_wait_host on a communicator of one rank: the reductions complete, so it returns GT_OK well inside its
    limit. (Its other outcome, aborting the communicator when a rank is missing, needs a stuck collective on the GPU
    and is not run here.)"""
    from gguf_trainer_b200.train import DataParallel
    gpu = requireGPU("the exchange gate")
    try:
        DataParallel(gpu, 0, 1, DataParallel.uniqueId())
        buf = gpu.createStateBuffer(4096 * 4)
        gpu.writeStateBuffer(buf, np.arange(4096, dtype=np.float32))
        gpu._check(gpu.lib.gt_dp_allreduce_start(gpu.ctx, buf, 4096))
        gpu._check(gpu.lib.gt_dp_wait_host(gpu.ctx, 20000))
        assert np.array_equal(gpu.readStateBuffer(buf, 4096), np.arange(4096, dtype=np.float32))
    finally:
        gpu.destroy()
