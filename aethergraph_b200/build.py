"""Builds libaethergpu.so (the CUDA kernels and the C ABI) for sm_100a, in-tree.

    python -m aethergraph_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU, so this runs on a CPU-only build machine;
the shared library lands beside this file and is what `aethergraph_b200._lib`
loads.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libaethergpu.so")
SOURCES = ["api.cu", "gather.cu", "sampler.cu", "synth.cu", "loader.cu", "noalloc.cu", "hetero.cu", "hop.cu", "shard.cu",
           "hetero_loader.cu", "rewrite.cu", "hot.cu", "peer_block.cu", "reorder.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libaethergpu.so cannot be built")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "aethergpu.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    objs = []
    env = dict(os.environ)
    # The image exports CC/CXX wrappers that lack some specs; use the system g++.
    host = shutil.which("g++") or "g++"
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.rsplit(".", 1)[0] + ".o")
        cmd = [nvcc, "-ccbin", host, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        procs.append((src, subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        text = out.decode(errors="replace")
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src}\n{text}\n")
        elif verbose or text.strip():
            sys.stderr.write(f"--- {src}\n{text}\n")
    if failed:
        raise RuntimeError("libaethergpu.so: compilation failed")
    link = [nvcc, "-ccbin", host, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
            "-o", LIB + ".tmp", *objs, "-lpthread"]
    r = subprocess.run(link, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if r.returncode != 0:
        raise RuntimeError("libaethergpu.so: link failed\n" + r.stdout.decode(errors="replace"))
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
