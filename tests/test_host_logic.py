"""Host-side logic of the package against the CPU oracle and the reference's golden values (no GPU)."""
import struct

import numpy as np
import pytest

from gguf_trainer_b200 import autograd as ag
from gguf_trainer_b200.arch import (ModelConfig, buildModel, gemma3_95M, paramCount, qwen3_0_6B, smolLM2_135M, tinyLlama)
from gguf_trainer_b200.optim import OPT_MAGIC, deserializeOptState, serializeOptState
from gguf_trainer_b200.qk_clip import applyQKClip, qkLogitScale
from gguf_trainer_b200.rng import Mulberry32
from gguf_trainer_b200.schedule import wsdSchedule
from gguf_trainer_b200.train import drawWindows, maskWindow


@pytest.mark.parametrize("seed", [0, 7, 1234, 0xFFFFFFFF])
def test_mulberry32_scalar_and_vector_paths_match_the_oracle(oracle, seed):
    a, b, c = Mulberry32(seed), Mulberry32(seed), oracle.Mulberry32(seed)
    v = a.draws(300)
    for i in range(300):
        x = c()
        assert b() == x and v[i] == x
    assert a.a == b.a


def test_param_init_matches_the_oracle_stream(oracle):
    a, c = Mulberry32(1234), oracle.Mulberry32(1234)
    got, want = a.randn((64, 33), 0.02), c.randn((64, 33), 0.02)
    # numpy's vector log/cos may differ from libm in the last bit of the f64, which can move an f32 store by one ulp
    assert np.abs(got - want).max() <= 4e-9 and (got != want).mean() < 0.01
    assert a() == c()   # both consumed the same number of draws


def test_model_param_order_and_groups_match_the_oracle(oracle):
    for cfg in (ModelConfig("llama", 23, 8, 2, 2, 1, 4, 16, 1e5, 1e-5),
                ModelConfig("qwen3", 23, 8, 2, 2, 1, 4, 16, 1e6, 1e-6),
                ModelConfig("gemma3", 23, 8, 2, 2, 1, 4, 16, 1e6, 1e-6, slidingWindow=4, swaPattern=2),
                ModelConfig("llama", 23, 8, 1, 2, 1, 4, 16, 1e5, 1e-5, tieEmbeddings=False, init="n002")):
        om = oracle.Model(cfg.oracle_dict(), 99)
        m = buildModel(cfg, 99)
        ps = m.params()
        assert len(ps) == om.nparams()
        muon = {id(t) for t in m.paramGroups()["muon"]}
        for i, p in enumerate(ps):
            inf = om.info(i)
            assert tuple(p.shape) == inf["shape"]
            assert ("muon" if id(p) in muon else "aux") == inf["group"]
            assert np.abs(p.data - om.data(i).reshape(-1)).max() <= 1e-7
        assert sum(p.size for p in ps) == paramCount(cfg)


def test_named_configs_have_the_stated_sizes():
    assert paramCount(smolLM2_135M()) == 134_515_008
    assert abs(paramCount(gemma3_95M()) - 87.9e6) < 0.2e6
    assert abs(paramCount(qwen3_0_6B()) - 596.1e6) < 0.3e6
    assert paramCount(tinyLlama()) == 459_392


def test_wsd_golden_values():
    s = wsdSchedule(4, 3, 4, 0.1)
    assert np.allclose([s(i) for i in range(12)], [0.25, 0.5, 0.75, 1, 1, 1, 1, 0.775, 0.55, 0.325, 0.1, 0.1], atol=1e-6)
    assert wsdSchedule(0, 2, 2)(0) == 1
    nc = wsdSchedule(0, 2, 0, 0)
    assert nc(1) == 1 and nc(2) == 0
    assert np.allclose([wsdSchedule(2, 0, 2, 0.1)(i) for i in range(4)], [0.5, 1, 0.55, 0.1])


def test_wsd_matches_oracle_everywhere(oracle):
    for (w, st, c, m) in [(4, 3, 4, 0.1), (0, 0, 0, 0.0), (10, 70, 20, 0.1), (1, 0, 1, 0.5)]:
        f = wsdSchedule(w, st, c, m)
        for step in range(w + st + c + 3):
            assert f(step) == oracle.wsd(w, st, c, m, step)


def test_qk_clip_lands_on_tau(oracle):
    m = buildModel(ModelConfig("gemma3", 13, 8, 2, 2, 1, 4, 16, 1e6, 1e-6, slidingWindow=16, swaPattern=2), 99)
    L0 = m.layers[0]
    assert abs(qkLogitScale(L0.qNorm.data, L0.kNorm.data, 4) - 1) < 1e-6
    L0.qNorm.data[:] = 3
    L0.kNorm.data[:] = 2
    assert abs(qkLogitScale(L0.qNorm.data, L0.kNorm.data, 4) - 6) < 1e-6
    assert abs(oracle.qk_logit_scale(L0.qNorm.data, L0.kNorm.data, 4) - 6) < 1e-6
    assert applyQKClip(m, 0.5) == 2
    assert abs(qkLogitScale(L0.qNorm.data, L0.kNorm.data, 4) - 0.5) < 1e-6
    assert applyQKClip(buildModel(ModelConfig("llama", 13, 8, 1, 2, 1, 4, 16, 1e5, 1e-5), 1), 0.5) == 0
    with pytest.raises(ValueError):
        applyQKClip(m, 0)


def test_optstate_byte_layout():
    """src/backend/muon-gpu.ts:293-349: u32 LE header [magic, adamT, (count, lens...) x3], then f32 data."""
    s = {"muonMomentum": [np.arange(6, dtype=np.float32)], "adamM": [np.ones(2, np.float32), np.zeros(3, np.float32)],
         "adamV": [np.full(2, 2, np.float32), np.full(3, 3, np.float32)], "adamT": 17}
    b = serializeOptState(s)
    head = struct.unpack_from("<10I", b, 0)
    assert head == (OPT_MAGIC, 17, 1, 6, 2, 2, 3, 2, 2, 3)
    assert len(b) == 40 + 4 * 16
    assert np.array_equal(np.frombuffer(b, "<f4", offset=40)[:6], np.arange(6, dtype=np.float32))
    r = deserializeOptState(b)
    assert r["adamT"] == 17 and serializeOptState(r) == b
    with pytest.raises(ValueError, match="bad optstate magic"):
        deserializeOptState(b"\0" * 16)


def test_validators_speak_the_reference_messages():
    with pytest.raises(ValueError, match=r"embedding: id 9 at position 1 is not an integer in \[0,5\)"):
        ag.assertIdsInTable([0, 9], 5, "embedding")
    with pytest.raises(ValueError, match=r"id 1.5 at position 0"):
        ag.assertIdsInTable([1.5], 5, "embedding")
    assert ag.keptRowsInVocab([-1, 0, 4, -1], 4, 5, "crossEntropy") == 2
    assert ag.keptRowsInVocab(np.array([-1, 0, 4, -1]), 4, 5, "crossEntropy") == 2
    with pytest.raises(ValueError, match=r"target -2 at position 1 is not -1 \(ignore\)"):
        ag.keptRowsInVocab([0, -2], 2, 5, "crossEntropy")
    with pytest.raises(ValueError, match=r"3 targets for 2 logit rows"):
        ag.keptRowsInVocab([0, 1, 2], 2, 5, "crossEntropy")
    assert ag.keptTeacherRows([1, 4, -1, 0, 7, 2, 3, 3], [0.5] * 8, 4, 2, 9) == 3
    with pytest.raises(ValueError, match="k must be >= 1"):
        ag.keptTeacherRows([], [], 0, 0, 9)
    with pytest.raises(ValueError, match=r"weight must be 2-D, got \[6\]"):
        ag.assertMatrix(ag.Tensor(np.zeros(6, np.float32), [6]), "weight", "embedding")


def test_mask_window_and_draw_order():
    tg = np.arange(10, 20)
    mask = np.array([1, 0] * 20)
    maskWindow(tg, mask, 3)
    assert list(tg) == [-1, 11, -1, 13, -1, 15, -1, 17, -1, 19]
    a, b = Mulberry32(7), Mulberry32(7)
    assert drawWindows(a, 5, 1000) == [int(b() * 1000) for _ in range(5)]


def test_lora_fold_matches_oracle(oracle):
    from gguf_trainer_b200.lora import applyLora, clearLora
    cfg = ModelConfig("llama", 23, 8, 2, 2, 1, 4, 16, 1e5, 1e-5)
    om = oracle.Model(cfg.oracle_dict(), 31)
    m = buildModel(cfg, 31)
    n = om.apply_lora(4, 8.0, 4321)
    h = applyLora(m, 4, 8.0, Mulberry32(4321))
    try:
        assert len(h.groups["aux"]) == n and h.adapted == 14 and h.trainable == sum(t.size for t in h.groups["aux"])
        with pytest.raises(RuntimeError, match="already installed"):
            applyLora(m, 4, 8.0, Mulberry32(1))
        base = len(m.params())
        r = Mulberry32(5)
        for j, t in enumerate(h.groups["aux"]):
            assert np.abs(t.data - om.data(base + j).reshape(-1)).max() <= 1e-7   # A ~ N(0, 1/in), B = 0
            t.data[:] = r.randn((t.size,), 0.1)
            om.data(base + j)[...] = t.data.reshape(om.info(base + j)["shape"])
        for i, p in enumerate(m.params()):
            p.data[:] = om.data(i).reshape(-1)
        assert all(not p.requiresGrad for p in m.params())
        h.merge(); om.lora_fold(1.0)
        for i, p in enumerate(m.params()):
            assert np.abs(p.data - om.data(i).reshape(-1)).max() <= 1e-7
    finally:
        clearLora(m)
    assert all(p.requiresGrad for p in m.params())


def test_bucket_plan_tiles_the_gradient_arena_in_completion_order():
    from gguf_trainer_b200.train import CudaStep
    cfg = ModelConfig("qwen3", 23, 8, 5, 2, 1, 4, 16, 1e6, 1e-6)
    m = buildModel(cfg, 1)
    order = list(reversed(m.params()))
    offs, total = [], 0
    for t in order:
        offs.append(total)
        total += (t.size + 63) // 64 * 64
    step = CudaStep(m, None, 2, 8, dp=object(), arena=(0, total, offs), layersPerBucket=2)
    plan = step.bucketPlan()
    assert [p[0] for p in plan] == [3, 1, 0]                 # buckets start at layers 3, 1, 0 (5 layers, 2 per bucket)
    assert plan[0][1] == 0 and sum(p[2] for p in plan) == total
    for (_, s0, c0), (_, s1, _c1) in zip(plan, plan[1:]):
        assert s0 + c0 == s1                                 # contiguous, in the order backward finishes them
    # the first bucket begins at the last layer's last parameter and ends where layer 2 begins
    assert order[0] is m.layers[4].down
    idx_l2_down = next(i for i, t in enumerate(order) if t is m.layers[2].down)
    assert plan[1][1] == offs[idx_l2_down]
    # the last bucket reaches the end of the arena: first layer, output norm and the (tied) embedding
    assert order[-1] is m.tokenEmbd and plan[-1][1] + plan[-1][2] == total


def test_linear_routes_an_adapter_to_one_op_or_to_the_reference_four():
    """`linear` (autograd.ts:311-319) with an adapter on the weight: a backend that offers `loraLinear` gets that one
    call; any other backend gets the reference's add(linear(x,w), scale(linear(linear(x,a),b), s))."""
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.autograd import Tensor

    class Recorder:
        def __init__(self, fuse):
            self.calls = []
            if fuse:
                self.fuseLora = True

        def _out(self, name, shape):
            self.calls.append(name)
            return Tensor.zeros(shape)

        def linear(self, x, w):
            return self._out("linear", [x.shape[0], w.shape[0]])

        def scale(self, x, c):
            return self._out(f"scale {c}", x.shape)

        def add(self, a, b):
            return self._out("add", a.shape)

        def loraLinear(self, x, w, a, b, s):
            return self._out(f"loraLinear {s}", [x.shape[0], w.shape[0]])

    x, w = Tensor.zeros([5, 8]), Tensor.zeros([6, 8])
    a, b = Tensor.zeros([2, 8]), Tensor.zeros([6, 2])
    prev = ag.opsBackend()
    try:
        ag.setLoraAdapters({id(w): ag.LoraAdapter(a, b, 1.5)})
        for fuse, want in ((True, ["loraLinear 1.5"]), (False, ["linear", "linear", "linear", "scale 1.5", "add"])):
            r = Recorder(fuse)
            ag.setOpsBackend(r)
            y = ag.linear(x, w)
            assert y.shape == [5, 6] and r.calls == want
            r.calls.clear()
            ag.linear(x, Tensor.zeros([6, 8]))            # a weight without an adapter: the plain product
            assert r.calls == ["linear"]
    finally:
        ag.setLoraAdapters({})
        ag.setOpsBackend(prev)
