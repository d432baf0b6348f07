"""tests/golden/step_fixtures.json (written by tests/golden/make_fixtures.py from the CPU oracle; the reference itself
cannot run here): the oracle still reproduces it exactly, and the CUDA path matches it: loss, every gradient's sum
of squares, every parameter's sum after one AdamW step, for the three architectures."""
import importlib.util
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
FIX = json.load(open(os.path.join(HERE, "golden", "step_fixtures.json")))


def _generator():
    spec = importlib.util.spec_from_file_location("make_fixtures", os.path.join(HERE, "golden", "make_fixtures.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_oracle_reproduces_the_fixtures(oracle):
    got = _generator().compute(oracle)
    for name, want in FIX.items():
        assert got[name]["loss"] == want["loss"], name
        assert got[name]["grad_sumsq"] == want["grad_sumsq"], name
        assert got[name]["param_sum_after_step"] == want["param_sum_after_step"], name


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(FIX))
def test_cuda_step_matches_the_fixtures(oracle, name):
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.arch import ModelConfig, buildModel
    from gguf_trainer_b200.backend import requireGPU
    from gguf_trainer_b200.optim import AdamWGpu
    from gguf_trainer_b200.train import sequenceLoss
    want = FIX[name]
    c = want["config"]
    cfg = ModelConfig(c["arch"], c["vocab"], c["hidden"], c["layers"], c["heads"], c["kv_heads"], c["head_dim"], c["ffn"], c["rope_base"],
                      c["eps"], ropeBaseLocal=c["rope_base_local"], slidingWindow=c["window"], swaPattern=c["swa_pattern"],
                      tieEmbeddings=c["tie"], init=c["init"])
    om = oracle.Model(cfg.oracle_dict(), want["seed"])      # only to initialise the weights identically
    m = buildModel(cfg, want["seed"])
    for i, p in enumerate(m.params()):
        p.data[:] = om.data(i).reshape(-1)
    ids = oracle.Mulberry32(11).randint(want["T"], cfg.vocabSize)
    tg = oracle.Mulberry32(12).randint(want["T"], cfg.vocabSize)
    gpu = requireGPU("the fixture check")                   # strict f32 mode
    try:
        gpu.install()
        try:
            loss = sequenceLoss(m, ids, tg)
            ag.backward(loss, 1.0)
            gpu.sync([loss])                                # brings the gradients back (no optimizer owns them yet)
            sumsq = [float(np.sum(np.asarray(p.grad, np.float64) ** 2)) for p in m.params()]
            opt = AdamWGpu(gpu, m.params(), lr=1e-3, beta1=0.9, beta2=0.95, weightDecay=0.1, clip=1.0)
            opt.recordStep()                                # the gradients are still in their device buffers
            gpu.sync(m.params())
        finally:
            gpu.uninstall()
        assert abs(float(loss.data[0]) - want["loss"]) <= 1e-5 * abs(want["loss"])
        for i, (g, w) in enumerate(zip(sumsq, want["grad_sumsq"])):
            assert abs(g - w) <= 2e-5 * max(abs(w), 1e-12), f"{name} grad[{i}]: {g} vs {w}"   # squares double the 1e-5 bound
        for i, (p, w) in enumerate(zip(m.params(), want["param_sum_after_step"])):
            got = float(np.sum(p.data.astype(np.float64)))
            scale = float(np.sum(np.abs(p.data.astype(np.float64))))
            assert abs(got - w) <= 5e-5 * max(scale, 1e-12), f"{name} param[{i}]: {got} vs {w}"
    finally:
        gpu.destroy()
