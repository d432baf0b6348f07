"""Data parallel on real GPUs. Two ranks (needs two GPUs), each with its own micro-batches and the bucketed NCCL
gradient sum started inside backward, against one process running the same global batch: weights stay replicated,
losses are the same per sequence, the stepped weights agree to f32 summation order; and the same with the north-star
optimizer split (Muon on the hidden matrices, AdamW on the rest) over a 20-step loss trajectory.
On one GPU, a world of one rank still goes through the communicator, the bucket hooks and the segmented graph replay,
and must equal the step without any of it bit for bit."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _gpus():
    try:
        out = subprocess.check_output(["nvidia-smi", "-L"], text=True)
        return len([l for l in out.splitlines() if l.startswith("GPU ")])
    except Exception:
        return 0


def _run(world, rank, work, steps, B, capture, optimizer="adamw"):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    return subprocess.Popen([sys.executable, os.path.join(HERE, "dp_worker.py"), str(rank), str(world), work, str(steps), str(B),
                             "1" if capture else "0", optimizer], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


def _finish(procs, timeout=240):
    """Outputs of the children; whatever happens, none of them is left running on a shared GPU."""
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=timeout)[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
                p.wait()
    return outs


@pytest.mark.parametrize("capture", [False, True])
def test_two_ranks_match_one_process(tmp_path, capture):
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    work = str(tmp_path)
    steps, B = 3, 2
    procs = [_run(2, r, work, steps, B, capture) for r in range(2)]
    outs = _finish(procs)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    single = _run(1, 0, work, steps, 2 * B, capture)
    so = _finish([single])[0]
    assert single.returncode == 0, so
    r0, r1, one = (np.load(os.path.join(work, f)) for f in ("out_adamw_2_0.npz", "out_adamw_2_1.npz", "out_adamw_1_0.npz"))
    n = len([k for k in r0.files if k.startswith("arr_")])
    for i in range(n):
        assert np.array_equal(r0[f"arr_{i}"], r1[f"arr_{i}"]), f"ranks diverged on parameter {i}"
        a, b = r0[f"arr_{i}"], one[f"arr_{i}"]
        assert np.abs(a - b).max() <= 2e-5 * max(1.0, np.abs(b).max()), f"parameter {i} differs from the single-process run"
    both = np.concatenate([r0["losses"], r1["losses"]], axis=1)      # [steps, 2B] in global draw order
    assert np.allclose(both, one["losses"], rtol=2e-5, atol=2e-6)


def test_muon_two_ranks_20_step_trajectory_matches_one_process(tmp_path):
    """Muon (5 Newton-Schulz iterations, momentum 0.95) on the hidden matrices + AdamW on embeddings and norms, data
    parallel on two ranks, 20 replayed steps, against one process at the same global batch: the loss trajectory within
    1e-3 + 1e-3*|ref| (tests/gpu-parity.ts:1141-1142), replicated weights identical across ranks, stepped weights close
    (src/backend/muon-gpu.ts:351-437 is the optimizer being replicated)."""
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    work = str(tmp_path)
    steps, B = 20, 2
    procs = [_run(2, r, work, steps, B, True, "muon") for r in range(2)]
    outs = _finish(procs)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    single = _run(1, 0, work, steps, 2 * B, True, "muon")
    so = _finish([single])[0]
    assert single.returncode == 0, so
    r0, r1, one = (np.load(os.path.join(work, f)) for f in ("out_muon_2_0.npz", "out_muon_2_1.npz", "out_muon_1_0.npz"))
    both = np.concatenate([r0["losses"], r1["losses"]], axis=1).mean(axis=1)     # the step loss: mean over the global batch
    ref = one["losses"].mean(axis=1)
    assert both.shape == (steps,)
    assert (np.abs(both - ref) <= 1e-3 + 1e-3 * np.abs(ref)).all(), f"trajectories:\n{both}\n{ref}"
    n = len([k for k in r0.files if k.startswith("arr_")])
    for i in range(n):
        assert np.array_equal(r0[f"arr_{i}"], r1[f"arr_{i}"]), f"ranks diverged on parameter {i}"
        a, b = r0[f"arr_{i}"], one[f"arr_{i}"]
        assert np.abs(a - b).max() <= 2e-3 + 2e-2 * np.abs(b).max(), f"parameter {i} differs from the single-process run"


@pytest.mark.parametrize("capture", [False, True])
@pytest.mark.parametrize("optimizer", ["adamw", "muon"])
def test_world_of_one_goes_through_the_exchange_and_changes_nothing(capture, optimizer):
    """One GPU: a communicator of one rank (gt_dp_init), the gradient arena, the per-bucket hooks in backward, the
    recorded step cut into one graph per bucket with the all-reduce calls issued between the segments, gt_dp_wait before
    the optimizer. A sum over one rank is the identity, so losses and stepped weights must equal the plain step's
    bit for bit."""
    from gguf_trainer_b200.arch import ModelConfig, buildModel
    from gguf_trainer_b200.backend import requireGPU
    from gguf_trainer_b200.optim import AdamWGpu, MuonGpu
    from gguf_trainer_b200.rng import Mulberry32
    from gguf_trainer_b200.train import CudaStep, DataParallel, drawWindows
    cfg = ModelConfig("llama", 61, 32, 4, 4, 2, 8, 64, 1e5, 1e-5)
    T, B, steps = 24, 3, 4
    tokens = Mulberry32(99).randint(400, cfg.vocabSize)
    results = []
    for with_dp in (False, True):
        gpu = requireGPU("the data-parallel test")
        try:
            dp = DataParallel(gpu, 0, 1, DataParallel.uniqueId()) if with_dp else None
            m = buildModel(cfg, 1234)
            arena = gpu.reserveGradArena(list(reversed(m.params())))
            if optimizer == "muon":
                g = m.paramGroups()
                opt = MuonGpu(gpu, g["muon"], g["aux"], lr=0.02, aux={"lr": 1e-2, "beta1": 0.9, "beta2": 0.95, "clip": 1.0},
                              shardOverRanks=with_dp)       # one rank: its share is everything, the all-gather is skipped
            else:
                opt = AdamWGpu(gpu, m.params(), lr=1e-2, clip=1.0)
            step = CudaStep(m, gpu, B, T, world=1, capture=capture, dp=dp, arena=arena if dp else None, layersPerBucket=1)
            rng = Mulberry32(7)
            losses = []
            for _ in range(steps):
                mine = drawWindows(rng, B, len(tokens) - T - 1)
                ids = np.concatenate([tokens[a:a + T] for a in mine])
                tg = np.concatenate([tokens[a + 1:a + 1 + T] for a in mine])
                step.run(ids, tg)
                opt.recordStep()
                losses.append(step.losses().copy())
            if with_dp and capture:
                assert len(step.graph.handles) == len(step.bucketPlan()), "the recorded step was not cut at the bucket boundaries"
            gpu.sync(m.params())
            results.append((np.array(losses), [p.data.copy() for p in m.params()]))
        finally:
            gpu.destroy()
    assert np.array_equal(results[0][0], results[1][0])
    for i, (a, b) in enumerate(zip(results[0][1], results[1][1])):
        assert np.array_equal(a, b), f"parameter {i}"
