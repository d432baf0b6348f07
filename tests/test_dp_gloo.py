"""The data-parallel host logic on CPU with two gloo ranks (no GPU): rank r takes draws [r*B, (r+1)*B) of each
step's global draw order and seeds its losses with 1/(B*world); summing the ranks' gradients must reproduce a
single process running the same global batch. The per-rank compute engine here is the CPU oracle (a checker),
the exchange is torch.distributed all_reduce over gloo in place of the NCCL sum the library issues on GPUs."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(arch="llama", vocab=31, hidden=8, layers=2, heads=2, kv_heads=1, head_dim=4, ffn=16, rope_base=1e5, eps=1e-5, tie=True)
B, T, STEPS, WORLD = 2, 9, 2, 2


def _windows(step, rank, world):
    """The draw partition the benchmark and `CudaStep` under `DataParallel` use."""
    sys.path.insert(0, ROOT)
    from gguf_trainer_b200.rng import Mulberry32
    from gguf_trainer_b200.train import drawWindows
    rng = Mulberry32(7)
    maxStart = 200 - T - 1
    draws = drawWindows(rng, (step + 1) * B * world, maxStart)[step * B * world:]
    return draws[rank * B:(rank + 1) * B], draws


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from oracle import oracle as orc
    orc.set_threads(1)
    tokens = orc.Mulberry32(99).randint(200, CFG["vocab"])
    m = orc.Model(CFG, 1234)           # same seed on every rank: replicated weights
    m.make_optimizer("adamw", lr=1e-2, clip=1.0)
    for step in range(STEPS):
        m.opt_zero_grad()
        mine, _ = _windows(step, rank, world)
        for s in mine:
            m.loss_backward(tokens[s:s + T], tokens[s + 1:s + 1 + T], seed=1.0 / (B * world))
        for i in range(m.nparams()):    # the one exchange: an f32 sum of the gradients
            g = torch.from_numpy(m.grad(i))
            dist.all_reduce(g, op=dist.ReduceOp.SUM)
        m.opt_step()
    if rank == 0:
        np.savez(out, *[m.data(i).copy() for i in range(m.nparams())])
    w0 = torch.from_numpy(m.data(3).copy())
    ws = [torch.zeros_like(w0) for _ in range(world)]
    dist.all_gather(ws, w0)
    assert all(torch.equal(ws[0], w) for w in ws), "ranks diverged"
    dist.destroy_process_group()


def test_two_ranks_match_one_process_at_the_same_global_batch(tmp_path, oracle):
    out = str(tmp_path / "dp.npz")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(WORLD, port, out), nprocs=WORLD, join=True)
    got = np.load(out)
    oracle.set_threads(1)
    tokens = oracle.Mulberry32(99).randint(200, CFG["vocab"])
    m = oracle.Model(CFG, 1234)
    m.make_optimizer("adamw", lr=1e-2, clip=1.0)
    for step in range(STEPS):
        m.opt_zero_grad()
        _, alld = _windows(step, 0, WORLD)
        assert len(alld) == B * WORLD
        for s in alld:
            m.loss_backward(tokens[s:s + T], tokens[s + 1:s + 1 + T], seed=1.0 / (B * WORLD))
        m.opt_step()
    for i in range(m.nparams()):
        # the sum order differs (per-rank partial sums), so agreement is to f32 rounding, not bitwise
        assert np.abs(got[f"arr_{i}"] - m.data(i)).max() <= 2e-6


def test_partition_covers_the_global_draws_exactly_once():
    for step in range(3):
        parts = [_windows(step, r, 4)[0] for r in range(4)]
        alld = _windows(step, 0, 4)[1]
        assert sum(parts, []) == alld
