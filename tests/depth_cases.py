"""Depth-faithful cuts of the benchmark configurations, small enough for the CPU oracle: the layer count, head
layout, widths, windows and adapters of each configuration are kept (they are what the tensor-core kernels and the
accumulated rounding depend on); sequence length and vocabulary are cut. Used by tests/test_gpu_depth_tf32.py.

`run_case` runs one forward + backward (+ AdamW step) on the device in the requested precision and on the oracle, and
returns every comparison as numbers, so a test can assert on them and a probe can print them."""
import numpy as np

from gpu_harness import rel_l2

from gguf_trainer_b200 import autograd as ag
from gguf_trainer_b200.arch import ModelConfig, buildModel
from gguf_trainer_b200.optim import AdamWGpu
from gguf_trainer_b200.train import sequenceLoss


def smollm2_cut():
    """SmolLM2-135M shape: 30 layers, hidden 576, 9/3 heads of 64, FFN 1536; vocabulary cut to 2048."""
    return ModelConfig("llama", 2048, 576, 30, 9, 3, 64, 1536, 100_000.0, 1e-5, init="n002"), 256


def gemma3_cut():
    """gemma3 ~95M shape: 12 layers, hidden 640, 4/1 heads of 256, GeGLU 2048, window 512 on 5 of 6 layers; the
    sequence (640) is longer than the window so the windowed kernels see clipped rows; vocabulary cut to 2048."""
    return ModelConfig("gemma3", 2048, 640, 12, 4, 1, 256, 2048, 1_000_000.0, 1e-6, ropeBaseLocal=10_000.0,
                       slidingWindow=512, swaPattern=6, init="n002"), 640


def qwen3_cut():
    """Qwen3-0.6B shape: 28 layers, hidden 1024, 16/8 heads of 128, FFN 3072; vocabulary cut to 2500 so a loss chunk
    of 1024 leaves a ragged last chunk of 452."""
    return ModelConfig("qwen3", 2500, 1024, 28, 16, 8, 128, 3072, 1_000_000.0, 1e-6, init="n002"), 128


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bfloat16 precision, kept as f32 (such values are exact in tf32)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def run_case(gpu, oracle, cfg, T, seed=1234, lora=None, mask_frac=0.0, recompute=False, loss_chunk=0,
             round_weights=False, adamw=True):
    """Returns {"loss": (got, ref), "layers": [rel-L2 per layer output and the final norm], "grads": [(shape, rel-L2)],
    "weights": [(shape, rel-L2)] after one AdamW step (lr 1e-3, betas 0.9/0.95, wd 0.1, clip 1.0)}."""
    from gguf_trainer_b200.lora import applyLora, clearLora
    from gguf_trainer_b200.rng import Mulberry32
    om = oracle.Model(cfg.oracle_dict(), seed)
    m = buildModel(cfg, seed)
    ps = m.params()
    for i, p in enumerate(ps):
        w = om.data(i)
        if round_weights and w.ndim == 2:
            w[...] = bf16_round(w)
        p.data[:] = w.reshape(-1)
    trainable = ps
    handle = None
    try:
        if lora is not None:
            rank, alpha = lora
            om.apply_lora(rank, alpha, 4321)
            handle = applyLora(m, rank, alpha, Mulberry32(4321))
            rng = oracle.Mulberry32(17)
            base_n = len(ps)
            for j, t in enumerate(handle.groups["aux"]):
                if j % 2 == 1:      # B starts at zero; give it values so both factors see a gradient
                    t.data[:] = rng.randn((t.size,), 0.02)
                om.data(base_n + j)[...] = t.data.reshape(om.info(base_n + j)["shape"])
            trainable = handle.groups["aux"]
            tr_index = [base_n + j for j in range(len(trainable))]
        else:
            tr_index = list(range(len(ps)))
        ids = oracle.Mulberry32(3).randint(T, cfg.vocabSize)
        tg = oracle.Mulberry32(4).randint(T, cfg.vocabSize)
        if mask_frac > 0:
            mr = oracle.Mulberry32(5)
            for t in range(T):
                if mr() < mask_frac:
                    tg[t] = -1
        if adamw:
            om.make_optimizer("adamw", lr=1e-3, beta1=0.9, beta2=0.95, wd=0.1, clip=1.0)
        ref_loss = float(om.loss_backward(ids, tg, loss_chunk=loss_chunk))
        ref_layers = [om.layer_out(l, T).copy() for l in range(cfg.nLayers + 1)]
        ref_grads = [om.grad(i).copy() for i in tr_index]
        opt = AdamWGpu(gpu, trainable, lr=1e-3, beta1=0.9, beta2=0.95, weightDecay=0.1, clip=1.0) if adamw else None
        ag.setCheckpointing(recompute)
        gpu.install()
        try:
            loss = sequenceLoss(m, ids, tg, loss_chunk)
            ag.backward(loss, 1.0)
            # with recompute the layer interiors are gone, but the layer outputs are the regions' kept tensors
            gpu.sync([loss] + m.layerOutputs + [m.lastHidden])
            grads = [gpu.readStateBuffer(gpu.buffersFor(p)["grad"], p.size) for p in trainable]
            if opt is not None:
                opt.recordStep()
                gpu.sync(trainable)
        finally:
            gpu.uninstall()
            ag.setCheckpointing(False)
        out = {"loss": (float(loss.data[0]), ref_loss),
               "layers": [rel_l2(t.data, ref_layers[l]) for l, t in enumerate(m.layerOutputs + [m.lastHidden])],
               "grads": [(tuple(p.shape), rel_l2(g, r)) for p, g, r in zip(trainable, grads, ref_grads)],
               "finite": all(np.isfinite(g).all() for g in grads)}
        if opt is not None:
            om.opt_step()
            out["weights"] = [(tuple(p.shape), rel_l2(p.data, om.data(i))) for p, i in zip(trainable, tr_index)]
        return out
    finally:
        if handle is not None:
            clearLora(m)
        om.close()
