#!/usr/bin/env python
"""Benchmark of the training hot path on B200: tokens/s of a full step (forward + backward + optimizer)
at the SmolLM2-135M shape, batch 8 x seq 2048 per GPU, on synthetic Zipf(1.1) token ids.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--precision tf32|fp32] [--impl reference]

One process per GPU (under torchrun for N > 1). Prints ONE JSON line on rank 0:
  value      whole-job tokens/s with the step's inputs already resident in HBM (device-timed)
  e2e        the same step through the public API with host buffers: ids/targets copied from pinned
             host memory every step and the loss read back, inside the timed region
  roofline   the backward matrix products (dX = dY.W, dW = dY^T.X of one layer at this shape),
             timed live with CUDA events, against the measured tensor peak
  cpu_baseline  the CPU oracle (a port of the reference's own CPU code) on a bounded slice
`--impl reference` times that CPU port alone with every host thread.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "train tokens/s, SmolLM2-135M shape seq2048 b8"
UNIT = "tokens/s"


def zipf_tokens(n: int, vocab: int, s: float, seed: int) -> np.ndarray:
    """Zipf(s) ids over [0, vocab) by inverse CDF from mulberry32(seed) draws."""
    from gguf_trainer_b200.rng import Mulberry32
    w = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** s
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    u = Mulberry32(seed).draws(n)
    return np.minimum(np.searchsorted(cdf, u, side="left"), vocab - 1).astype(np.int64)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                          "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "src": "fallback"}


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle (port of the reference's CPU code) on a bounded slice of the same workload
# ---------------------------------------------------------------------------------------------
def cpu_slice(threads: int, T: int = 256, repeats: int = 1):
    """One T-token sequence through the SmolLM2-135M shape cut to 1 and 5 layers (tied readout, CE,
    forward + backward + AdamW over those parameters). The per-layer cost comes from the difference;
    tokens/s for the 30-layer model is extrapolated from it."""
    from oracle import oracle as orc
    from gguf_trainer_b200.arch import smolLM2_135M
    orc.build()
    orc.set_threads(threads)
    cfg = smolLM2_135M()
    ids = zipf_tokens(T + 1, cfg.vocabSize, 1.1, 99)
    times = {}
    for L in (1, 5):
        d = cfg.oracle_dict()
        d["layers"] = L
        m = orc.Model(d, 1234)
        m.make_optimizer("adamw", lr=1e-3, beta1=0.9, beta2=0.95, wd=0.1, clip=1.0)
        best = None
        for _ in range(repeats):
            m.opt_zero_grad()
            t0 = time.perf_counter()
            m.loss_backward(ids[:T], ids[1:T + 1], seed=1.0)
            m.opt_step()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        times[L] = best
        m.close()
    per_layer = max((times[5] - times[1]) / 4, 1e-9)
    base = max(times[1] - per_layer, 0.0)
    full = base + 30 * per_layer
    return {"value": T / full, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"one {T}-token sequence, 1- and 5-layer cuts of the 30-layer model + tied readout + CE, fwd+bwd+AdamW; "
                      f"measured {times[1]:.2f}s / {times[5]:.2f}s, extrapolated to 30 layers ({full:.1f}s per {T} tokens)",
            "seconds_measured": times[1] + times[5]}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    orc.build()
    threads = orc.max_threads()
    t0 = time.perf_counter()
    res = None
    steps = max(1, args.steps)
    vals = []
    for i in range(args.warmup + steps):
        r = cpu_slice(threads, T=args.cpu_tokens)
        if i >= args.warmup:
            vals.append(r["value"])
        res = r
        if time.perf_counter() - t0 > 150:   # stay within a few minutes whatever K and W are
            if not vals:
                vals.append(r["value"])
            break
    v = float(np.mean(vals))
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": len(vals),
            "warmup": args.warmup, "ms_per_step": 1e3 * 16384 / v, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64 arithmetic on f32 arrays", "data": "synthetic",
            "config": {"workload": "SmolLM2-135M shape llama step, seq 2048 x batch 8 per GPU, AdamW (CPU port on a bounded slice)"},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": res["cores"], "kind": "port", "sample": res["sample"]},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def backward_gemm_roofline(gpu, rows: int, iters: int = 5):
    """The backward matrix products of one layer at this shape as the step issues them: the weight gradients
    dW = dY^T.X of q, k, v, o, gate, up, down as ONE grouped launch, and the input gradients dX = dY.W, those of the
    activations that feed several projections as one launch each (dQ.Wq + dK.Wk + dV.Wv; dGate.Wg + dUp.Wu) and those of
    o and down on their own: 5 launches, 2 x 2 x rows x in x out flop per projection. Launched back to back between two
    events on the library's stream. Operands are far larger than L2 in aggregate (rows x 1536 f32 alone is 100 MB)."""
    import ctypes as C
    h, q, kv, f = 576, 576, 192, 1536
    bufs = []

    def buf(n):
        bufs.append(gpu.createStateBuffer(n * 4))
        return bufs[-1]

    projections = [(q, h), (kv, h), (kv, h), (h, q), (f, h), (f, h), (h, f)]      # (out, in): q k v o gate up down
    dys = [buf(rows * o) for o, _i in projections]
    xs = {h: buf(rows * h), q + 1: buf(rows * q), f: buf(rows * f)}               # n1/n2 share a width; attention out; gated unit
    x_of = [xs[h], xs[h], xs[h], xs[q + 1], xs[h], xs[h], xs[f]]
    ws = [buf(o * i) for o, i in projections]
    gws = [buf(o * i) for o, i in projections]
    gx = {0: buf(rows * h), 3: buf(rows * q), 4: buf(rows * h), 6: buf(rows * f)}
    flops = sum(2 * 2 * rows * i * o for o, i in projections)
    n = len(projections)
    Ms, Ns = (C.c_int32 * n)(*[o for o, _i in projections]), (C.c_int32 * n)(*[i for _o, i in projections])
    As, Bs, Cs, acc = (C.c_uint64 * n)(*dys), (C.c_uint64 * n)(*x_of), (C.c_uint64 * n)(*gws), (C.c_int32 * n)(*([0] * n))

    def multi(idx, inn, out):
        k = len(idx)
        Ks, A2, B2 = (C.c_int32 * k)(*[projections[j][0] for j in idx]), (C.c_uint64 * k)(*[dys[j] for j in idx]), (C.c_uint64 * k)(*[ws[j] for j in idx])
        return lambda: gpu._check(gpu.lib.gt_gemm_multi(gpu.ctx, 1, 0, rows, inn, k, Ks, A2, B2, out))

    calls = [lambda: gpu._check(gpu.lib.gt_gemm_grouped(gpu.ctx, 2, n, Ms, Ns, rows, As, Bs, Cs, acc)),
             multi((0, 1, 2), h, gx[0]), multi((3,), q, gx[3]), multi((4, 5), h, gx[4]), multi((6,), f, gx[6])]
    for c in calls:
        c()
    gpu.recordEvent(10)
    for _ in range(iters):
        for c in calls:
            c()
    gpu.recordEvent(11)
    ms = gpu.elapsedMs(10, 11) / iters
    for a in bufs:
        gpu._check(gpu.lib.gt_free(gpu.ctx, a))
    return flops, ms, len(calls)


def tf32_peak_and_comparator(rows: int, seconds: float = 3.0):
    """Harness only (never on the product's path): the TF32 rate of this GPU measured the way MEASURED_PEAKS.json
    measures BF16 (`torch.matmul` 8192^3 with allow_tf32, best of 10 and a seconds-long loop), and cuBLAS on the same 14
    backward product shapes the roofline object times, as a same-box comparator."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True

    def timed(fn, n):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / n

    N = 8192
    a, b = torch.randn(N, N, device="cuda"), torch.randn(N, N, device="cuda")
    for _ in range(3):
        a @ b
    burst = 2 * N ** 3 / min(timed(lambda: a @ b, 1) for _ in range(10)) / 1e9
    t0, tot, n = time.perf_counter(), 0.0, 0
    while time.perf_counter() - t0 < seconds:
        tot += timed(lambda: a @ b, 20) * 20
        n += 20
    sustained = 2 * N ** 3 / (tot / n) / 1e9
    del a, b
    h, q, kv, f = 576, 576, 192, 1536
    flops, ops = 0, []
    for out, inn in [(q, h), (kv, h), (kv, h), (h, q), (f, h), (f, h), (h, f)]:
        dy, x, w = torch.randn(rows, out, device="cuda"), torch.randn(rows, inn, device="cuda"), torch.randn(out, inn, device="cuda")
        ops.append((lambda dy=dy, w=w: dy @ w))
        ops.append((lambda dy=dy, x=x: dy.t() @ x))
        flops += 2 * 2 * rows * inn * out

    def layer():
        for op in ops:
            op()

    layer()
    ms = timed(layer, 5)
    torch.cuda.empty_cache()
    return {"burst": burst, "sustained": sustained, "unit": "TFLOP/s", "how": "torch.matmul allow_tf32 8192^3: best of 10, and back to back for 3 s"}, \
        flops / (ms / 1e3) / 1e12


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.arch import buildModel, gemma3_95M, qwen3_0_6B, smolLM2_135M
    from gguf_trainer_b200.backend import requireGPU
    from gguf_trainer_b200.optim import AdamWGpu, MuonGpu
    from gguf_trainer_b200.train import CudaStep, DataParallel

    # The headline workload is the SmolLM2-135M shape; the other two configurations of the parity list can be timed too.
    cfg = {"smollm2": smolLM2_135M, "gemma3": gemma3_95M, "qwen3-lora": qwen3_0_6B}[args.config]()
    # per-configuration defaults: the Qwen3 LoRA fine-tune runs batch 4 per GPU with the chunked (fused) readout loss
    B = args.batch if args.batch > 0 else (4 if args.config == "qwen3-lora" else 8)
    T = args.seq
    gpu = requireGPU("the benchmark", device=local, precision=args.precision)
    if args.plain:
        gpu.mergeInputGradients = False
        gpu.fuseResidualNorm = False
        gpu.groupWeightGradients = False
        gpu.groupForward = False
        gpu.fuseRope = False
    if args.no_rope_fusion:
        gpu.fuseRope = False
    model = buildModel(cfg, 1234)       # same seed on every rank: replicated weights
    loss_chunk = args.loss_chunk if args.loss_chunk >= 0 else (32768 if args.config == "qwen3-lora" else 0)
    mask = None
    if args.config == "qwen3-lora":      # frozen base, rank-16 adapters on the 7 projections, 50 % prompt mask, recompute
        from gguf_trainer_b200.lora import applyLora
        from gguf_trainer_b200.rng import Mulberry32 as _M
        lora = applyLora(model, 16, 32.0, _M(4321))
        ag.setCheckpointing(True)
    if args.recompute:
        ag.setCheckpointing(True)
    params = [p for p in model.params() if p.requiresGrad] if args.config != "qwen3-lora" else lora.groups["aux"]
    groups = model.paramGroups() if args.config != "qwen3-lora" else lora.groups
    # gradients in one arena, last layers first: the order backward finishes them in
    order = list(reversed(params))
    arena = gpu.reserveGradArena(order)
    for p in params:
        gpu.keepGradOnDevice(p)
    dp = None
    if world > 1:       # (before the optimizers: a sharded Muon asks the communicator for its rank)
        uid = [DataParallel.uniqueId() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        dp = DataParallel(gpu, rank, world, uid[0], commCtas=args.comm_ctas)

    def make_muon():
        return MuonGpu(gpu, groups["muon"], groups["aux"], lr=0.02, momentum=0.95, nesterov=True, nsSteps=5,
                       aux={"lr": 1e-3, "beta1": 0.9, "beta2": 0.95, "weightDecay": 0.0, "clip": 1.0},
                       shardOverRanks=dp is not None and not args.no_shard_muon)

    if args.optimizer == "muon":
        opt = make_muon()
    else:
        opt = AdamWGpu(gpu, params, lr=1e-3, beta1=0.9, beta2=0.95, weightDecay=0.1, clip=1.0)
    opts = {"cur": opt}

    # synthetic stream; rank r takes draws [r*B, (r+1)*B) of each step's B*world windows
    need = (args.steps + args.warmup + 2) * B * world
    stream = zipf_tokens(max(4 * (T + 1) * B, 1 << 20), cfg.vocabSize, 1.1, 99)
    from gguf_trainer_b200.rng import Mulberry32
    rng = Mulberry32(7)
    maxStart = len(stream) - T - 1
    starts = np.floor(rng.draws(need) * maxStart).astype(np.int64)

    if args.config == "qwen3-lora":
        mask = (Mulberry32(5).draws(len(stream)) < 0.5)

    def batch(step):
        s = starts[step * B * world + rank * B: step * B * world + (rank + 1) * B]
        ids = np.concatenate([stream[a:a + T] for a in s])
        tg = np.concatenate([stream[a + 1:a + 1 + T] for a in s])
        if mask is not None:
            keep = np.concatenate([mask[a + 1:a + 1 + T] for a in s])
            tg = np.where(keep, tg, -1)
        return ids, tg

    # pinned host staging for the e2e arm
    pin_ids = torch.empty(B * T, dtype=torch.int32).pin_memory()
    pin_tg = torch.empty(B * T, dtype=torch.int32).pin_memory()
    step = CudaStep(model, gpu, B, T, lossChunk=loss_chunk, world=world, capture=not args.no_graph, dp=dp,
                    arena=arena if dp is not None else None, layersPerBucket=args.layers_per_bucket)

    def one_step(i, resident, prepared=None):
        ids, tg = prepared if prepared is not None else batch(i)
        if resident and step.graph is not None:
            step.replay()                       # inputs already in HBM
        else:
            pin_ids.numpy()[:] = ids
            pin_tg.numpy()[:] = tg
            step.run(pin_ids.numpy(), pin_tg.numpy())
        opts["cur"].recordStep()              # the gradient exchange is part of the step (started bucket by bucket in backward)

    def barrier():
        gpu.sync([])
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def timed(resident, steps, first):
        nxt = batch(first)          # (drawn before the clock starts, as every later batch is drawn while a step runs)
        barrier()
        gpu.recordEvent(0)
        loss = None
        pending = None
        for i in range(steps):
            one_step(first + i, resident, nxt)
            if i + 1 < steps:
                nxt = batch(first + i + 1)  # the next batch is drawn on the host while this step runs on the device
            if not resident:
                # device -> host read of every step's result: started now, collected after the next step has been
                # enqueued, so the device does not wait for the host between steps
                ticket = step.lossesBegin()
                if pending is not None:
                    loss = step.lossesEnd(pending)
                pending = ticket
        if pending is not None:
            loss = step.lossesEnd(pending)
        gpu.recordEvent(1)
        ms = gpu.elapsedMs(0, 1)
        barrier()
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, loss

    for i in range(max(args.warmup, 3)):
        one_step(i, False)
        step.lossesEnd(step.lossesBegin())     # (the first asynchronous read allocates its pinned block: not in the timed region)
    barrier()
    launches0 = gpu.kernelLaunches()
    per_replay = step.launchesPerReplay
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_res, _ = timed(True, args.steps, args.warmup)
    ms_e2e, loss = timed(False, args.steps, args.warmup)
    # Beside the headline (AdamW at every N, so the driver's scaling ratio compares like with like): the same step with
    # the optimizer split of the multi-GPU configuration, Muon (5 Newton-Schulz iterations, momentum 0.95) on the hidden
    # matrices and AdamW on embeddings and norms.
    muon_line = None
    if world > 1 and args.optimizer == "adamw" and args.config != "qwen3-lora" and groups["muon"]:
        opts["cur"] = make_muon()
        for i in range(3):
            one_step(i, False)
        ms_muon, _ = timed(True, args.steps, args.warmup)
        muon_line = {"optimizer": "muon (5 Newton-Schulz iterations, momentum 0.95, Nesterov) on the hidden matrices + adamw on embeddings and norms",
                     "value": B * T * world * args.steps / (ms_muon / 1e3), "unit": UNIT, "ms_per_step": ms_muon / args.steps}
        opts["cur"] = opt
    clocks = sampler.stop() if rank == 0 else None
    eager_launches = gpu.kernelLaunches() - launches0
    tokens = B * T * world * args.steps
    value = tokens / (ms_res / 1e3)
    e2e = tokens / (ms_e2e / 1e3)

    if rank == 0:
        pk = peaks()
        flops, gms, ncalls = backward_gemm_roofline(gpu, B * T)
        achieved = flops / (gms / 1e3) / 1e12
        tf32_peak, cublas_same = (None, None)
        if not args.no_peak:
            tf32_peak, cublas_same = tf32_peak_and_comparator(B * T)
        metric = METRIC if (args.config == "smollm2" and B == 8 and T == 2048) else f"train tokens/s, {args.config} shape seq{T} b{B}"
        line = {
            "metric": metric, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_res / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"tf32": "tf32 products, f32 accumulate and storage", "fp32": "f32"}[args.precision],
            "data": "synthetic",
            "config": {"workload": {"smollm2": "SmolLM2-135M shape llama (h576 L30 9/3 heads hd64 ffn1536 V49152, tied)",
                                    "gemma3": "gemma3 ~95M shape (h640 L12 4/1 heads hd256 ffn2048 V32768, window 512 on 5 of 6 layers)",
                                    "qwen3-lora": "Qwen3-0.6B shape LoRA r16 alpha 32 on q,k,v,o,gate,up,down (h1024 L28 16/8 heads hd128 ffn3072 V151936), frozen base, 50% loss mask, recompute"}[args.config]
                                   + f", full step fwd+bwd+{args.optimizer}, "
                                   + (f"chunked readout loss (chunk {loss_chunk}), " if loss_chunk else "dense readout loss, ")
                                   + f"seq {T} x batch {B} per GPU, Zipf(1.1) ids, N(0,0.02) f32 weights",
                       "precision": args.precision, "graph_replay": not args.no_graph,
                       "l2": "per-step working set (activations > 20 GB) exceeds L2; no flush needed",
                       "parallelism": f"dp{world}"},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": 2 * B * T * 4, "d2h_bytes_per_step": 4 * (1 + B),
                    "ms_per_step": ms_e2e / args.steps, "loss": float(loss[0]) if loss is not None else None},
            "gpu_launches": int(eager_launches + per_replay * args.steps * 2 if not args.no_graph else eager_launches),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["tflops_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / pk["tflops_sustained"],
                         # dram__bytes_read.sum + dram__bytes_write.sum of these launches at rows 16384 from one ncu capture
                         # (profiles/gemm_tf32_rows16384.md: 1063.1 MB for the five), per launch; only meaningful at the default shape
                         "traffic": (1063.1e6 / ncalls) if (args.config == "smollm2" and B * T == 16384) else None,
                         "kernel": f"backward matrix products of one layer (dW of 7 projections grouped, dX merged per shared input: {ncalls} launches, rows {B * T})",
                         "peak_source": f"{pk['src']} bf16 sustained (the products run in tf32, whose own measured rate is tf32_peak)",
                         "tf32_peak": tf32_peak,
                         "frac_of_tf32_sustained": (achieved / tf32_peak["sustained"]) if tf32_peak else None,
                         "cublas_tf32_same_shapes": cublas_same},
        }
        if muon_line is not None:
            line["config3_optimizer"] = muon_line
        if args.gpus == 1 and not args.no_cpu:
            from oracle import oracle as orc
            orc.build()
            line["cpu_baseline"] = {k: v for k, v in cpu_slice(orc.max_threads(), T=args.cpu_tokens).items() if k != "seconds_measured"}
            # the reference's CPU code is single-threaded: the same slice on one thread, on a shorter sequence to stay bounded
            one = cpu_slice(1, T=64)
            line["cpu_baseline"]["single_thread"] = {"value": one["value"], "unit": UNIT, "cores": 1, "sample": one["sample"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        gpu.sync([])
        dist.destroy_process_group()


def run_profile(args):
    """One eager step at the benchmark shape with the backend's per-label profiler open: GPU time per entry point
    (and per product shape), each call bracketed by events and synchronised. Shares, not throughput."""
    from gguf_trainer_b200 import autograd as ag
    from gguf_trainer_b200.arch import buildModel, gemma3_95M, qwen3_0_6B, smolLM2_135M
    from gguf_trainer_b200.backend import requireGPU
    from gguf_trainer_b200.optim import AdamWGpu
    from gguf_trainer_b200.train import CudaStep
    cfg = {"smollm2": smolLM2_135M, "gemma3": gemma3_95M, "qwen3-lora": qwen3_0_6B}[args.config]()
    B = args.batch if args.batch > 0 else (4 if args.config == "qwen3-lora" else 8)
    T = args.seq
    loss_chunk = args.loss_chunk if args.loss_chunk >= 0 else (32768 if args.config == "qwen3-lora" else 0)
    gpu = requireGPU("the profile", precision=args.precision)
    if args.no_rope_fusion:
        gpu.fuseRope = False
    m = buildModel(cfg, 1234)
    params = m.params()
    ids = zipf_tokens(B * T + 1, cfg.vocabSize, 1.1, 99)
    tg = ids[1:]
    if args.config == "qwen3-lora":      # as in the timed run: frozen base, adapters, half of the targets masked, recompute
        from gguf_trainer_b200.lora import applyLora
        from gguf_trainer_b200.rng import Mulberry32
        params = applyLora(m, 16, 32.0, Mulberry32(4321)).groups["aux"]
        ag.setCheckpointing(True)
        tg = np.where(Mulberry32(5).draws(B * T) < 0.5, tg, -1)
    if args.recompute:
        ag.setCheckpointing(True)
    for p in params:
        gpu.keepGradOnDevice(p)
    opt = AdamWGpu(gpu, params, lr=1e-3, beta1=0.9, beta2=0.95, weightDecay=0.1, clip=1.0)
    step = CudaStep(m, gpu, B, T, lossChunk=loss_chunk, capture=False)
    for _ in range(2):
        step.run(ids[:-1], tg); opt.recordStep(); gpu.sync([])
    gpu.startProfile()
    step.run(ids[:-1], tg); opt.recordStep()
    tot = gpu.stopProfile()
    gpu.sync([])
    total = sum(v["ms"] for v in tot.values())
    print(f"# one step, {B} x {T} tokens, precision {args.precision}: {total:.2f} ms summed over {sum(v['count'] for v in tot.values())} calls")
    for k, v in sorted(tot.items(), key=lambda kv: -kv[1]["ms"]):
        print(f"{v['ms']:9.3f} ms {100 * v['ms'] / total:5.1f}%  n={v['count']:4d}  avg {1e3 * v['ms'] / v['count']:8.1f} us  {k}")


def run_micro(args):
    """One op of the step at the benchmark shape, launched `--steps` times between two events: prints its
    time and achieved algorithmic rate. Meant for `ncu` captures of a single kernel and for the per-kernel
    roofline table; `--micro-batch` shrinks the row count (default: the full 8 x 2048)."""
    from gguf_trainer_b200.backend import requireGPU
    gpu = requireGPU("the micro benchmark", precision=args.precision)
    B, T = args.micro_batch, args.seq
    rows = B * T
    h, q, kv, f, V, Hq, Hkv, hd = 576, 576, 192, 1536, 49152, 9, 3, 64
    if args.heads:                                   # attention at another head layout, e.g. 4,1,256 (gemma3)
        Hq, Hkv, hd = (int(x) for x in args.heads.split(","))
        q, kv = Hq * hd, Hkv * hd
    rng = np.random.default_rng(0)

    def buf(n, fill=True):
        b = gpu.createStateBuffer(n * 4)
        if fill:
            gpu.writeStateBuffer(b, (rng.standard_normal(n, dtype=np.float32) * 0.5))
        return b

    lib, ctx = gpu.lib, gpu.ctx
    name = args.micro
    pk = peaks()
    if name == "bwd-gemm":       # the roofline object itself: one layer's backward products, as the step issues them
        flops, ms, n = backward_gemm_roofline(gpu, rows, iters=args.steps)
        rate = flops / (ms / 1e3) / 1e12
        print(json.dumps({"micro": f"backward matrix products of one layer (grouped dW, merged dX), {n} launches", "ms": ms, "achieved": rate, "unit": "TFLOP/s",
                          "peak": pk["tflops_sustained"], "frac": rate / pk["tflops_sustained"], "rows": rows}), flush=True)
        gpu.sync([])
        return
    gpu.setBatch(B, T)
    if name == "attention":
        Q, K, Vv, O, G = buf(rows * q), buf(rows * kv), buf(rows * kv), buf(rows * q, False), buf(rows * q)
        L = buf(Hq * rows, False)
        gq, gk, gv = buf(rows * q, False), buf(rows * kv, False), buf(rows * kv, False)
        P = T * (T + 1) // 2
        gq0, gk0 = buf(rows * q, False), buf(rows * kv, False)

        def bwd_then_rope():
            st = lib.gt_attention_bwd(ctx, rows, Hq, Hkv, hd, args.window, Q, K, Vv, O, L, G, gq, 0, gk, 0, gv, 0)
            st = st or lib.gt_rope_bwd(ctx, rows, Hq, hd, 10000.0, 0, gq, gq0, 0)
            return st or lib.gt_rope_bwd(ctx, rows, Hkv, hd, 10000.0, 0, gk, gk0, 0)

        cases = [("attention fwd", lambda: lib.gt_attention_fwd(ctx, rows, Hq, Hkv, hd, args.window, Q, K, Vv, O, L), 4 * Hq * hd * P * B),
                 ("attention bwd", lambda: lib.gt_attention_bwd(ctx, rows, Hq, Hkv, hd, args.window, Q, K, Vv, O, L, G, gq, 0, gk, 0, gv, 0), 10 * Hq * hd * P * B),
                 ("attention bwd, then the rotations' backward (3 + 2 launches)", bwd_then_rope, 10 * Hq * hd * P * B),
                 ("attention bwd rotating dQ and dK as it stores them (3 launches)",
                  lambda: lib.gt_attention_bwd_rope(ctx, rows, Hq, Hkv, hd, args.window, Q, K, Vv, O, L, G, gq0, 0, gk0, 0, gv, 0, 10000.0, 0), 10 * Hq * hd * P * B)]
        unit, peak = "TFLOP/s", pk["tflops_sustained"]
    elif name == "qkv":
        # q, k, v projections of one input and the rotary embedding of q and k: one launch against three
        import ctypes as C
        x, ws = buf(rows * h), [buf(o * h) for o in (q, kv, kv)]
        ys, yr = [buf(rows * o, False) for o in (q, kv, kv)], [buf(rows * o, False) for o in (q, kv)]
        Ms, Ns = (C.c_int32 * 3)(rows, rows, rows), (C.c_int32 * 3)(q, kv, kv)
        As, Bs, Cs, acc = (C.c_uint64 * 3)(x, x, x), (C.c_uint64 * 3)(*ws), (C.c_uint64 * 3)(*ys), (C.c_int32 * 3)(0, 0, 0)
        Cr, Hs = (C.c_uint64 * 3)(yr[0], yr[1], ys[2]), (C.c_int32 * 3)(Hq, Hkv, 0)

        def sep():
            st = lib.gt_gemm_grouped(ctx, 0, 3, Ms, Ns, h, As, Bs, Cs, acc)
            st = st or lib.gt_rope_fwd(ctx, rows, Hq, hd, 10000.0, 0, ys[0], yr[0])
            return st or lib.gt_rope_fwd(ctx, rows, Hkv, hd, 10000.0, 0, ys[1], yr[1])

        fl = 2 * rows * h * (q + 2 * kv)
        cases = [("q/k/v projections, grouped launch", lambda: lib.gt_gemm_grouped(ctx, 0, 3, Ms, Ns, h, As, Bs, Cs, acc), fl),
                 ("q/k/v grouped, then the two rotations (3 launches)", sep, fl),
                 ("q/k/v grouped with the rotations applied as the tiles are written (1 launch)",
                  lambda: lib.gt_linear_rope_grouped(ctx, 3, rows, h, x, Ns, Bs, Cr, Hs, hd, 10000.0, 0), fl)]
        unit, peak = "TFLOP/s", pk["tflops_sustained"]
    elif name == "ffn":
        # the gated FFN's fused launches against their separate forms (rows x 576 -> 1536 -> 576)
        x, wg, wu, wd = buf(rows * h), buf(f * h), buf(f * h), buf(h * f)
        gate, up, hid = buf(rows * f, False), buf(rows * f, False), buf(rows * f, False)
        n = rows * f
        fl_f = 2 * 2 * rows * h * f

        def fwd_sep():
            st = lib.gt_gemm(ctx, 0, 0, rows, f, h, x, wg, gate)
            st = st or lib.gt_gemm(ctx, 0, 0, rows, f, h, x, wu, up)
            return st or lib.gt_glu_fwd(ctx, 2, n, gate, up, hid)

        cases = [("ffn entry, one launch (gate, up, gated unit)", lambda: lib.gt_glu_linear_fwd(ctx, 2, rows, f, h, x, wg, wu, gate, up, hid), fl_f),
                 ("ffn entry, three launches", fwd_sep, fl_f)]
        unit, peak = "TFLOP/s", pk["tflops_sustained"]
    elif name == "norm":
        # the HBM-bound passes around a residual connection at the benchmark shape, in bytes moved per second
        a, b2, sm, y, g, gx = buf(rows * h), buf(rows * h), buf(rows * h, False), buf(rows * h, False), buf(rows * h), buf(rows * h, False)
        w, rinv, gw = buf(h), buf(rows, False), buf(h, False)
        nb = rows * h * 4
        gpu._check(lib.gt_rmsnorm_fwd(ctx, rows, h, a, w, 1e-5, y, rinv))
        cases = [("rmsnorm forward (read x, write y)", lambda: lib.gt_rmsnorm_fwd(ctx, rows, h, a, w, 1e-5, y, rinv), 2 * nb),
                 ("residual add + rmsnorm forward (read a, b; write sum, y)", lambda: lib.gt_add_rmsnorm_fwd(ctx, rows, h, a, b2, w, 1e-5, sm, y, rinv), 4 * nb),
                 ("rmsnorm backward on top of the residual gradient (read x, g, upstream; write dx; dw)",
                  lambda: lib.gt_rmsnorm_bwd_add(ctx, rows, h, a, w, rinv, g, b2, gx, gw, 0), 4 * nb)]
        unit, peak = "TB/s", pk["hbm_gbs"] / 1e3
    elif name == "gemm":
        cases = []
        for out, inn in [(q, h), (kv, h), (f, h), (h, f)]:
            x, w, y = buf(rows * inn), buf(out * inn), buf(rows * out)
            dx, dw = buf(rows * inn, False), buf(out * inn, False)
            fl = 2 * rows * inn * out
            cases.append((f"NT {rows}x{out}x{inn}", (lambda x=x, w=w, y=y, out=out, inn=inn: lib.gt_gemm(ctx, 0, 0, rows, out, inn, x, w, y)), fl))
            cases.append((f"NN {rows}x{inn}x{out}", (lambda w=w, y=y, dx=dx, out=out, inn=inn: lib.gt_gemm(ctx, 1, 0, rows, inn, out, y, w, dx)), fl))
            cases.append((f"TN {out}x{inn}x{rows}", (lambda x=x, y=y, dw=dw, out=out, inn=inn: lib.gt_gemm(ctx, 2, 0, out, inn, rows, y, x, dw)), fl))
        # the merged input-gradient products of a layer: dX = dQ.Wq + dK.Wk + dV.Wv and dX = dGate.Wg + dUp.Wu, one launch each
        import ctypes as C
        for label, outs in (("qkv", (q, kv, kv)), ("gate+up", (f, f))):
            dys, ws = [buf(rows * o) for o in outs], [buf(o * h) for o in outs]
            dx = buf(rows * h, False)
            n = len(outs)
            Ks, As, Bs = (C.c_int32 * n)(*outs), (C.c_uint64 * n)(*dys), (C.c_uint64 * n)(*ws)
            cases.append((f"NN multi {rows}x{h}x({'+'.join(map(str, outs))}) [{label}]",
                          (lambda Ks=Ks, As=As, Bs=Bs, dx=dx, n=n: lib.gt_gemm_multi(ctx, 1, 0, rows, h, n, Ks, As, Bs, dx)), 2 * rows * h * sum(outs)))
        # the weight gradients of a layer's seven projections as one grouped launch
        shapes = [(q, h), (kv, h), (kv, h), (h, q), (f, h), (f, h), (h, f)]
        n = len(shapes)
        dys, xs, gws = [buf(rows * o) for o, _i in shapes], [buf(rows * i) for _o, i in shapes], [buf(o * i, False) for o, i in shapes]
        Ms, Ns = (C.c_int32 * n)(*[o for o, _i in shapes]), (C.c_int32 * n)(*[i for _o, i in shapes])
        As, Bs, Cs, acc = (C.c_uint64 * n)(*dys), (C.c_uint64 * n)(*xs), (C.c_uint64 * n)(*gws), (C.c_int32 * n)(*([0] * n))
        cases.append((f"TN grouped: dW of q,k,v,o,gate,up,down at rows {rows}",
                      (lambda: lib.gt_gemm_grouped(ctx, 2, n, Ms, Ns, rows, As, Bs, Cs, acc)), sum(2 * rows * o * i for o, i in shapes)))
        unit, peak = "TFLOP/s", pk["tflops_sustained"]
    else:
        raise SystemExit(f"unknown --micro {name}")
    for label, fn, work in cases:
        for _ in range(2):
            gpu._check(fn())
        gpu.recordEvent(30)
        for _ in range(args.steps):
            gpu._check(fn())
        gpu.recordEvent(31)
        ms = gpu.elapsedMs(30, 31) / args.steps
        rate = work / (ms / 1e3) / 1e12
        print(json.dumps({"micro": label, "ms": ms, "achieved": rate, "unit": unit, "peak": peak, "frac": rate / peak,
                          "precision": args.precision, "rows": rows}), flush=True)
    gpu.sync([])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="tf32", choices=["fp32", "tf32"])
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "muon"])
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU per step (default 8; 4 for qwen3-lora)")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--cpu-tokens", type=int, default=256)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--config", default="smollm2", choices=["smollm2", "gemma3", "qwen3-lora"])
    ap.add_argument("--loss-chunk", type=int, default=-1, help="vocabulary chunk of the fused readout loss; 0 = dense (default: 0; 32768 for qwen3-lora)")
    ap.add_argument("--no-peak", action="store_true", help="skip the torch.matmul TF32 peak and comparator")
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--profile", action="store_true", help="per-entry-point GPU time of one eager step")
    ap.add_argument("--micro", default="", help="time one op of the step instead: attention | gemm | bwd-gemm | ffn | qkv | norm")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--layers-per-bucket", type=int, default=6, help="data parallel: layers per gradient all-reduce bucket")
    ap.add_argument("--comm-ctas", type=int, default=0, help="data parallel: CTAs left to the collective while it overlaps backward (0 = no cap, no reservation)")
    ap.add_argument("--no-shard-muon", action="store_true", help="data parallel: every rank runs all Newton-Schulz iterations")
    ap.add_argument("--no-rope-fusion", action="store_true", help="rotary embeddings as launches of their own (for comparison)")
    ap.add_argument("--plain", action="store_true", help="launch every op as recorded: no merged input gradients, no residual add + norm fusion")
    ap.add_argument("--heads", default="", help="--micro attention: Hq,Hkv,hd instead of 9,3,64")
    args = ap.parse_args()
    if args.profile:
        run_profile(args)
    elif args.micro:
        run_micro(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
