"""Compile libgguftrain_cuda.so for sm_100a, in-tree, with nvcc (no torch involved).

Usage: python build.py [--force] [--verbose]   (also imported by __graft_entry__.build)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "libgguftrain_cuda.so")
SOURCES = ["ctx.cu", "gemm_simt.cu", "gemm_tc.cu", "elementwise.cu", "norm.cu", "rope_embed.cu", "attention.cu",
           "attention_simt.cu", "attention_tc.cu", "loss.cu", "optim.cu", "dp.cu", "noalloc.cu", "ingest.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
EXTRA = os.environ.get("GT_NVCC_EXTRA", "").split()
FLAGS = EXTRA + ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math=false",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unknown-pragmas"]


def sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(HERE, s))]


def stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = sources() + ["common.cuh", "../../include/gguftrain.h", "build.py"] + \
        [f for f in os.listdir(HERE) if f.endswith(".cuh")]
    return any(os.path.getmtime(os.path.join(HERE, d)) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not stale():
        return OUT
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    objs = []
    procs = []
    for s in sources():
        o = os.path.join(HERE, "build", s.replace(".cu", ".o"))
        objs.append(o)
        src = os.path.join(HERE, s)
        hdr_t = max(os.path.getmtime(os.path.join(HERE, h)) for h in os.listdir(HERE) if h.endswith(".cuh"))
        hdr_t = max(hdr_t, os.path.getmtime(os.path.join(HERE, "../../include/gguftrain.h")))
        if not force and os.path.exists(o) and os.path.getmtime(o) > max(os.path.getmtime(src), hdr_t):
            continue
        cmd = [NVCC] + [f for f in FLAGS if f != "--use_fast_math=false"] + (["-Xptxas", "-v"] if verbose else []) + \
            ["-c", src, "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {s} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([NVCC, "-shared", "-o", OUT] + objs + ["-ldl"])
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(OUT)
