"""Child process of tests/test_gpu_dp.py: one data-parallel rank on its own GPU.
usage: dp_worker.py RANK WORLD WORKDIR STEPS BATCH_PER_RANK CAPTURE [OPTIMIZER]
OPTIMIZER: adamw (default) or muon = Muon (5 Newton-Schulz iterations, momentum 0.95, Nesterov) on the hidden matrices
and AdamW on embeddings and norms, the split of `paramGroups()` (src/backend/muon-gpu.ts:351-437)."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from gguf_trainer_b200.arch import ModelConfig, buildModel  # noqa: E402
from gguf_trainer_b200.backend import requireGPU  # noqa: E402
from gguf_trainer_b200.optim import AdamWGpu, MuonGpu  # noqa: E402
from gguf_trainer_b200.rng import Mulberry32  # noqa: E402
from gguf_trainer_b200.train import CudaStep, DataParallel, drawWindows  # noqa: E402

CFG = ModelConfig("llama", 61, 32, 4, 4, 2, 8, 64, 1e5, 1e-5)
T = 24


def main():
    rank, world, work, steps, B, capture = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4]), int(sys.argv[5]), sys.argv[6] == "1"
    optimizer = sys.argv[7] if len(sys.argv) > 7 else "adamw"
    gpu = requireGPU("the data-parallel test", device=rank if world > 1 else 0)
    dp = None
    if world > 1:
        idf = os.path.join(work, "nccl_id")
        if rank == 0:
            uid = DataParallel.uniqueId()
            with open(idf + ".tmp", "wb") as f:
                f.write(uid)
            os.rename(idf + ".tmp", idf)
        else:
            t0 = time.time()
            while not os.path.exists(idf):
                if time.time() - t0 > 60:
                    raise SystemExit("rank 0 never published the NCCL id")
                time.sleep(0.05)
            uid = open(idf, "rb").read()
        dp = DataParallel(gpu, rank, world, uid)
    m = buildModel(CFG, 1234)
    arena = gpu.reserveGradArena(list(reversed(m.params())))
    for p in m.params():
        gpu.keepGradOnDevice(p)
    if optimizer == "muon":
        g = m.paramGroups()
        opt = MuonGpu(gpu, g["muon"], g["aux"], lr=0.02, momentum=0.95, nesterov=True, nsSteps=5,
                      aux={"lr": 1e-2, "beta1": 0.9, "beta2": 0.95, "weightDecay": 0.0, "clip": 1.0},
                      shardOverRanks=dp is not None)       # each rank orthogonalises its share of the matrices
    else:
        opt = AdamWGpu(gpu, m.params(), lr=1e-2, clip=1.0)
    tokens = Mulberry32(99).randint(400, CFG.vocabSize)
    rng = Mulberry32(7)
    step = CudaStep(m, gpu, B, T, world=world, capture=capture, dp=dp, arena=arena if dp else None, layersPerBucket=1)
    losses = []
    for s in range(steps):
        draws = drawWindows(rng, B * world, len(tokens) - T - 1)
        mine = draws[rank * B:(rank + 1) * B]
        ids = np.concatenate([tokens[a:a + T] for a in mine])
        tg = np.concatenate([tokens[a + 1:a + 1 + T] for a in mine])
        step.run(ids, tg)
        opt.recordStep()
        losses.append(step.losses()[1:].copy())
    gpu.sync(m.params())
    np.savez(os.path.join(work, f"out_{optimizer}_{world}_{rank}.npz"), losses=np.array(losses), *[p.data for p in m.params()])
    gpu.destroy()


if __name__ == "__main__":
    main()
