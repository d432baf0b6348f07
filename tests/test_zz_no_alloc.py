"""The allocation-free attention backward (`gt_attention_bwd_static`) against the regular entry point.

Some callers of the library may not allocate device memory once they are running: a host that gave all of
HBM to its own arena, or a step loop that cannot take cudaMalloc's device-wide synchronisation. For them
the library keeps the one scratch array attention backward needs inside its own image. This test drives
both entry points through the C ABI on the same inputs, twice in a row (the array is shared and keeps the
previous call's contents), and checks the gradients agree; it also checks the size limit is refused with
a message rather than overrun. Collected last so a failure here cannot hide any other test's result.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_attention_backward_matches_regular_entry_point(oracle):
    from gpu_harness import BWD, compare
    from gguf_trainer_b200.backend import requireGPU

    gpu = requireGPU("the allocation-free attention test")
    lib, ctx = gpu.lib, gpu.ctx
    try:
        for call, (T, Hq, Hkv, hd, window, seed) in enumerate([(70, 4, 2, 32, 0, 11), (193, 6, 3, 64, 50, 12)]):
            rng = oracle.Mulberry32(seed)
            q = rng.randn((T, Hq * hd), 0.8); k = rng.randn((T, Hkv * hd), 0.8); v = rng.randn((T, Hkv * hd), 0.8)
            go = rng.uniform_pm1((T, Hq * hd))

            def dev(a):
                b = gpu.createStateBuffer(a.nbytes)
                gpu.writeStateBuffer(b, a)
                return b

            dq, dk, dv, dgo = dev(q), dev(k), dev(v), dev(go)
            out = gpu.createStateBuffer(q.nbytes)
            lse = gpu.createStateBuffer(Hq * T * 4)
            gpu._check(lib.gt_attention_fwd(ctx, T, Hq, Hkv, hd, window, dq, dk, dv, out, lse))
            grads = {}
            for name, fn in (("regular", lib.gt_attention_bwd), ("static", lib.gt_attention_bwd_static)):
                gq, gk, gv = (gpu.createStateBuffer(x.nbytes) for x in (q, k, v))
                before = gpu.stats()
                gpu._check(fn(ctx, T, Hq, Hkv, hd, window, dq, dk, dv, out, lse, dgo, gq, 0, gk, 0, gv, 0))
                if name == "static":
                    after = gpu.stats()
                    assert (after["pool"], after["state"]) == (before["pool"], before["state"])
                grads[name] = [gpu.readStateBuffer(b, x.size) for b, x in ((gq, q), (gk, k), (gv, v))]
            for a, b, nm in zip(grads["static"], grads["regular"], ("dq", "dk", "dv")):
                compare(f"call {call} {nm}", a, b, BWD, 1e-6)
            # and against the CPU oracle, so both cannot be wrong together
            _o, probs = oracle.attention_fwd(q, k, v, T, Hq, Hkv, hd, window)
            for a, b, nm in zip(grads["static"], oracle.attention_bwd(q, k, v, probs, go, T, Hq, Hkv, hd, window), ("dq", "dk", "dv")):
                compare(f"call {call} {nm} vs oracle", a, b, BWD)
        # beyond the built-in scratch: refused, with the limit in the message
        st = lib.gt_attention_bwd_static(ctx, 1 << 19, 4, 2, 32, 0, dq, dk, dv, out, lse, dgo, 0, 0, 0, 0, 0, 0)
        assert st == 2
        assert b"exceeds the built-in scratch" in lib.gt_last_error(ctx)
    finally:
        gpu.destroy()
