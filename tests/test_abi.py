"""The C-ABI library loads without a GPU and exports exactly what include/gguftrain.h declares."""
import ctypes as C
import os
import re
import subprocess

from gguf_trainer_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = [name for name, _ret, _args in _lib.declared_functions()]
    assert len(declared) >= 50 and len(set(declared)) == len(declared)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in gguftrain.h but not exported"


def test_no_undeclared_gt_exports():
    out = subprocess.check_output(["nm", "-D", "--defined-only", _lib.LIB_PATH], text=True)
    exported = {l.split()[-1] for l in out.splitlines() if re.search(r" T gt_\w+$", l)}
    declared = {name for name, _r, _a in _lib.declared_functions()}
    assert exported == declared, f"undeclared: {sorted(exported - declared)}, missing: {sorted(declared - exported)}"


def test_signatures_use_plain_c_types_only():
    text = open(_lib.HEADER_PATH).read()
    assert "torch" not in text and "at::" not in text and "std::" not in text
    for _name, _ret, args in _lib.declared_functions():
        for a in args:
            assert a in _lib._TYPES, f"unexpected type {a!r} in the ABI"


def test_init_without_a_gpu_fails_with_a_message_not_a_crash():
    import torch
    if torch.cuda.is_available():
        return
    lib = _lib.load()
    ctx = C.c_void_p()
    st = lib.gt_init(0, C.byref(ctx))
    assert st != 0 and not ctx.value
    assert b"no GPU adapter found" in lib.gt_last_error(None)


def test_ops_refuse_to_run_without_a_backend():
    import numpy as np
    import pytest
    from gguf_trainer_b200 import autograd as ag
    ag.setOpsBackend(None)
    x = ag.Tensor(np.zeros(6, np.float32), [2, 3])
    with pytest.raises(RuntimeError, match="no ops backend installed"):
        ag.add(x, x)


def test_product_code_never_touches_the_oracle():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "gguf_trainer_b200")
    for dirpath, _d, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle", text, re.M), f"{f} imports the oracle"
                assert "liboracle" not in text, f"{f} names the oracle library"


def test_typescript_binding_lists_every_entry_point_with_the_declared_arity():
    """integration/src/backend/cuda.ts cannot run here, but its Deno.dlopen table can be held to the header: same set
    of names, same number of parameters, pointer-like results only for gt_last_error."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "integration", "src", "backend", "cuda.ts")).read()
    table = text[text.index("const SYMBOLS = {"):text.index("} as const;")]
    bound = {}
    for m in re.finditer(r"^\s*(gt_\w+): \{ parameters: \[([^\]]*)\], result: \"(\w+)\"", table, re.M):
        params = [p for p in m.group(2).split(",") if p.strip()]
        bound[m.group(1)] = (len(params), m.group(3))
    declared = {name: (len(args), "pointer" if ret.startswith("const char") else "i32") for name, ret, args in _lib.declared_functions()}
    assert bound == declared, f"only in cuda.ts: {sorted(set(bound) - set(declared))}, missing: {sorted(set(declared) - set(bound))}"
