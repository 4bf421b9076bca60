"""Build libtensorlib_b200.so in-tree with nvcc for sm_100a (no GPU needed to compile).

    python -m tensorlib_b200.build [--force] [--verbose]

Objects go to tensorlib_b200/_build/, the library to tensorlib_b200/libtensorlib_b200.so.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OUT = os.path.join(PKG, "_build")
LIB = os.path.join(PKG, "libtensorlib_b200.so")
NVCC = os.environ.get("TL_NVCC", "/usr/local/cuda/bin/nvcc")

SOURCES = ["runtime.cu", "ops_refmode.cu", "device_ops.cu", "gemv.cu", "attn.cu", "attn_sm100.cu", "hgemm_sm100.cu", "skinny_sm100.cu", "decode_mega.cu", "tp_prefill.cu", "engine.cu",
           "api.cu", "tp.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr", "-Xptxas", "-v",
              "-ccbin", "g++"]


def _newer(a: str, b: str) -> bool:
    return not os.path.exists(b) or os.path.getmtime(a) > os.path.getmtime(b)


def _deps() -> list[str]:
    hdr = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".hpp", ".h"))]
    hdr.append(os.path.join(PKG, "..", "include", "tensorlib_b200.h"))
    return hdr


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    deps = _deps()
    jobs = []
    for s in srcs:
        src, obj = os.path.join(CSRC, s), os.path.join(OUT, s + ".o")
        if force or _newer(src, obj) or any(_newer(d, obj) for d in deps):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [NVCC, *NVCC_FLAGS, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = os.path.join(OUT, os.path.basename(src) + ".ptxas.log")
        with open(log, "w") as f:
            f.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    objs = [os.path.join(OUT, s + ".o") for s in srcs]
    if jobs or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-ccbin", "g++", "-Xlinker", "--no-undefined",
               "-ldl"]    # NCCL is bound at run time (csrc/tp.cu), never at link time
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
