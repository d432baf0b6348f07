"""Data parallel on real GPUs (needs two): two ranks, each with its own micro-batches and the bucketed NCCL gradient
sum started inside backward, against one process running the same global batch. Weights stay replicated, losses are the
same per sequence, and the stepped weights agree to f32 summation order."""
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


def _run(world, rank, work, steps, B, capture):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    return subprocess.Popen([sys.executable, os.path.join(HERE, "dp_worker.py"), str(rank), str(world), work, str(steps), str(B),
                             "1" if capture else "0"], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


@pytest.mark.parametrize("capture", [False, True])
def test_two_ranks_match_one_process(tmp_path, capture):
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    work = str(tmp_path)
    steps, B = 3, 2
    procs = [_run(2, r, work, steps, B, capture) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    single = _run(1, 0, work, steps, 2 * B, capture)
    so = single.communicate(timeout=240)[0]
    assert single.returncode == 0, so
    r0, r1, one = (np.load(os.path.join(work, f)) for f in ("out_2_0.npz", "out_2_1.npz", "out_1_0.npz"))
    n = len([k for k in r0.files if k.startswith("arr_")])
    for i in range(n):
        assert np.array_equal(r0[f"arr_{i}"], r1[f"arr_{i}"]), f"ranks diverged on parameter {i}"
        a, b = r0[f"arr_{i}"], one[f"arr_{i}"]
        assert np.abs(a - b).max() <= 2e-5 * max(1.0, np.abs(b).max()), f"parameter {i} differs from the single-process run"
    both = np.concatenate([r0["losses"], r1["losses"]], axis=1)      # [steps, 2B] in global draw order
    assert np.allclose(both, one["losses"], rtol=2e-5, atol=2e-6)
