"""Rewrites the Deno.dlopen symbol table of integration/src/backend/cuda.ts from include/gguftrain.h, so that the
TypeScript binding cannot drift from the declared ABI. Usage: python integration/gen_symbols.py"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from gguf_trainer_b200 import _lib  # noqa: E402  (only its header parser is used; no library is loaded)

FFI = {"gt_ctx*": "pointer", "gt_ctx**": "buffer", "gt_buf": "u64", "gt_buf*": "buffer", "const gt_buf*": "buffer", "int32_t": "i32",
       "int32_t*": "buffer", "const int32_t*": "buffer", "uint64_t": "u64", "uint64_t*": "buffer", "const uint64_t*": "buffer",
       "float": "f32", "float*": "buffer", "double": "f64", "const void*": "buffer", "void*": "buffer", "char*": "buffer",
       "const uint8_t*": "buffer", "uint8_t*": "buffer", "uint32_t*": "buffer"}
# calls that wait for the device: declared nonblocking so they return Promises
BLOCKING = {"gt_sync", "gt_read", "gt_read_finish", "gt_graph_end", "gt_event_elapsed_ms", "gt_dp_wait_host", "gt_tokens_max", "gt_dp_init"}


def table() -> str:
    lines = []
    for name, ret, types in _lib.declared_functions():
        params = ", ".join(f'"{FFI[t]}"' for t in types)
        res = '"pointer"' if ret.startswith("const char") else '"i32"'
        nb = ", nonblocking: true" if name in BLOCKING else ""
        lines.append(f"  {name}: {{ parameters: [{params}], result: {res}{nb} }},")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    path = os.path.join(ROOT, "integration", "src", "backend", "cuda.ts")
    text = open(path).read()
    a = text.index("const SYMBOLS = {\n") + len("const SYMBOLS = {\n")
    b = text.index("} as const;")
    open(path, "w").write(text[:a] + table() + text[b:])
    print(f"{len(_lib.declared_functions())} entry points written to {path}")
