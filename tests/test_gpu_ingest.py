"""Token and mask ingest on the device against the reference's host path, bit for bit: `window(start, T)` +
`window(start + 1, T)` + `maskWindow` (src/data/tokens.ts:158-185, src/train/trainer.ts:45-49,
src/backend/train-gpu.ts:206-208) restated in numpy. Both token widths, with and without a mask, starts at both ends
of the corpus, the benchmark's batch size; the refusals; and a training step fed by window starts."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from gguf_trainer_b200 import _lib
from gguf_trainer_b200.arch import ModelConfig, buildModel
from gguf_trainer_b200.backend import requireGPU
from gguf_trainer_b200.ingest import DeviceTokenSource, tokenBytes
from gguf_trainer_b200.train import CudaStep, maskWindow


@pytest.fixture()
def gpu():
    g = requireGPU("the ingest suite")
    yield g
    g.destroy()


def host_windows(tokens, supervised, starts, T):
    """The reference's per-micro-batch ingest: two windows and the in-place mask."""
    ids, tgs = [], []
    for s in starts:
        ids.append(np.array(tokens[s:s + T], dtype=np.int64))
        t = np.array(tokens[s + 1:s + 1 + T], dtype=np.int64)
        if supervised is not None:
            maskWindow(t, supervised, s + 1)
        tgs.append(t)
    return np.concatenate(ids), np.concatenate(tgs)


def read_u32(gpu, dev):
    out = np.empty(dev.count, np.uint32)
    gpu._check(gpu.lib.gt_read(gpu.ctx, dev.addr, out.ctypes.data, out.nbytes))
    return out


@pytest.mark.parametrize("vocab", [512, 49152, 151936])
@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("B,T", [(1, 7), (3, 130), (8, 2048)])
def test_gather_matches_the_host_windows_bit_for_bit(gpu, oracle, vocab, masked, B, T):
    n = max(4 * T, B * T // 2 + T + 5)
    rng = np.random.default_rng(vocab + B * 131 + T)
    tokens = rng.integers(0, vocab, n)
    tokens[0], tokens[-1] = vocab - 1, vocab - 1
    supervised = (rng.random(n) < 0.5).astype(np.int64) if masked else None
    src = DeviceTokenSource(gpu, tokens, vocab, supervised)
    assert src.bytesPerToken == tokenBytes(vocab) == (2 if vocab <= 65536 else 4) and src.length == n
    max_start = n - T - 1
    draw = oracle.Mulberry32(7)
    starts = [int(draw() * max_start) for _ in range(B)]    # floor(rng() * maxStart), train-gpu.ts:206
    starts[0] = 0
    starts[-1] = max_start                                  # the last window the corpus holds
    ids, tg = src.gather(starts, T)
    want_ids, want_tg = host_windows(tokens, supervised, starts, T)
    got_ids = read_u32(gpu, ids).astype(np.int64)
    got_tg = read_u32(gpu, tg).astype(np.int64)
    got_tg[got_tg == 0xFFFFFFFF] = -1
    gpu.sync([])
    assert np.array_equal(got_ids, want_ids)
    assert np.array_equal(got_tg, want_tg)
    assert np.array_equal(src.window(starts[-1], T), want_ids[-T:])
    src.close()


def test_refusals(gpu):
    tokens = np.arange(100) % 50
    with pytest.raises(ValueError, match="not in \\[0,40\\)"):
        DeviceTokenSource(gpu, tokens, 40)                       # the corpus does not fit the vocabulary
    with pytest.raises(ValueError, match="mask has 99 tokens, corpus has 100"):
        DeviceTokenSource(gpu, tokens, 50, np.ones(99))
    src = DeviceTokenSource(gpu, tokens, 50)
    with pytest.raises(ValueError, match="out of range 0..100"):
        src.gather([0, 92], 8)                                   # window [92, 101)
    with pytest.raises(ValueError, match="out of range"):
        src.gather([-1], 8)
    # a bad start that reaches the kernel anyway (the C ABI called directly) reads nothing and is reported at the sync
    buf = src.startsBuffer(1)
    gpu._write(buf, np.array([95], "<u8"))
    out = gpu.createStateBuffer(8 * 4 * 2)
    src.gatherInto(buf, 1, 8, out, out + 32)
    with pytest.raises(_lib.GtError, match="window start past corpus length"):
        gpu.sync([])
    got = gpu.readStateBuffer(out, 16).view(np.uint32)
    assert (got[4:8] == 0).all() and (got[12:16] == 0xFFFFFFFF).all()   # rows past the end: id 0, target ignored
    gpu.sync([])                                                 # the flag was cleared by the failed sync


@pytest.mark.parametrize("capture", [False, True])
def test_step_fed_by_window_starts_equals_step_fed_by_arrays(gpu, oracle, capture):
    """`CudaStep.runWindows(starts)` (the gather is the first kernel of the recorded step; 8 bytes per sequence cross
    the bus) gives the losses and gradients of `CudaStep.run(ids, targets)` on the host-built windows, bit for bit."""
    cfg = ModelConfig("qwen3", 300, 32, 2, 4, 2, 8, 64, 1_000_000.0, 1e-6)
    B, T = 3, 24
    rng = np.random.default_rng(5)
    tokens = rng.integers(0, cfg.vocabSize, 500)
    supervised = (rng.random(500) < 0.6).astype(np.int64)
    out = []
    for windows in (False, True):
        m = buildModel(cfg, 9)
        for p in m.params():
            gpu.keepGradOnDevice(p)
        src = DeviceTokenSource(gpu, tokens, cfg.vocabSize, supervised) if windows else None
        step = CudaStep(m, gpu, B, T, capture=capture, source=src)
        res = []
        for starts in ([5, 100, 475], [0, 17, 300]):           # the second call is a pure replay when capturing
            if windows:
                step.runWindows(starts)
            else:
                step.run(*host_windows(tokens, supervised, starts, T))
            res.append((step.losses().copy(), [gpu.readStateBuffer(gpu.buffersFor(p)["grad"], p.size) for p in m.params()]))
        gpu.sync([])
        out.append(res)
    for (la, ga), (lb, gb) in zip(out[0], out[1]):
        assert np.array_equal(la, lb)
        for a, b in zip(ga, gb):
            assert np.array_equal(a, b)
    if capture:
        with pytest.raises(ValueError, match="out of range"):
            step.runWindows([0, 1, 476])


@pytest.mark.parametrize("capture", [False, True])
def test_losses_read_one_step_late_are_the_steps_own(gpu, oracle, capture):
    """`lossesBegin` after a step and `lossesEnd` after the NEXT step has been enqueued (the loop that keeps the device
    busy between steps) returns the first step's losses, not the second's: the copy is ordered behind the first step and
    the second step's loss kernel waits for it."""
    cfg = ModelConfig("qwen3", 300, 32, 2, 4, 2, 8, 64, 1_000_000.0, 1e-6)
    B, T = 3, 24
    rng = np.random.default_rng(11)
    tokens = rng.integers(0, cfg.vocabSize, 500)
    m = buildModel(cfg, 9)
    for p in m.params():
        gpu.keepGradOnDevice(p)
    step = CudaStep(m, gpu, B, T, capture=capture)
    batches = [host_windows(tokens, None, starts, T) for starts in ([5, 100, 475], [0, 17, 300], [9, 200, 31])]
    blocking = []
    for ids, tg in batches:
        step.run(ids, tg)
        blocking.append(step.losses().copy())
    late, pending = [], None
    for ids, tg in batches:
        step.run(ids, tg)
        ticket = step.lossesBegin()
        if pending is not None:
            late.append(step.lossesEnd(pending))
        pending = ticket
    late.append(step.lossesEnd(pending))
    gpu.sync([])
    assert not np.array_equal(blocking[0], blocking[1])
    for a, b in zip(blocking, late):
        assert np.array_equal(a, b)
