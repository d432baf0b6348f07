"""Writes tests/golden/step_fixtures.json: loss, per-parameter gradient sums of squares and post-AdamW-step parameter
sums for the three architectures at tiny sizes, fixed seeds, computed by the CPU oracle.

The reference itself cannot run in this repository's environment (TypeScript under Deno), so these are NOT outputs of
the reference: they freeze the oracle, which tests/test_oracle_golden.py pins to the reference's own known-answer
tests, so that a later change to the oracle or to the GPU path that moves any of these numbers is noticed.

    python tests/golden/make_fixtures.py
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

CASES = {
    "llama": dict(arch="llama", vocab=96, hidden=64, layers=2, heads=4, kv_heads=2, head_dim=16, ffn=128, rope_base=10000.0,
                  rope_base_local=10000.0, eps=1e-5, window=0, swa_pattern=0, tie=True, init="n002"),
    "qwen3": dict(arch="qwen3", vocab=96, hidden=64, layers=2, heads=4, kv_heads=2, head_dim=16, ffn=128, rope_base=1000000.0,
                  rope_base_local=10000.0, eps=1e-6, window=0, swa_pattern=0, tie=True, init="n002"),
    "gemma3": dict(arch="gemma3", vocab=96, hidden=64, layers=3, heads=4, kv_heads=1, head_dim=16, ffn=128, rope_base=1000000.0,
                   rope_base_local=10000.0, eps=1e-6, window=8, swa_pattern=3, tie=True, init="n002"),
}
T, SEED = 24, 4321


def compute(orc):
    out = {}
    for name, cfg in CASES.items():
        m = orc.Model(cfg, SEED)
        ids = orc.Mulberry32(11).randint(T, cfg["vocab"])
        tg = orc.Mulberry32(12).randint(T, cfg["vocab"])
        m.make_optimizer("adamw", lr=1e-3, beta1=0.9, beta2=0.95, wd=0.1, clip=1.0)
        loss = float(m.loss_backward(ids, tg))
        n = m.nparams()
        grads = [float(np.sum(m.grad(i).astype(np.float64) ** 2)) for i in range(n)]
        m.opt_step()
        params = [float(np.sum(m.data(j).astype(np.float64))) for j in range(n)]
        out[name] = dict(config=cfg, T=T, seed=SEED, loss=loss, grad_sumsq=grads, param_sum_after_step=params)
    return out


if __name__ == "__main__":
    from oracle import oracle as orc
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "step_fixtures.json"), "w") as f:
        json.dump(compute(orc), f, indent=1)
    print("written")
