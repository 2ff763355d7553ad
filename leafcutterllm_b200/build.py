"""Builds libleafcutter_b200.so for sm_100a with nvcc (cross-compiles without a GPU).

Usage: python -m leafcutterllm_b200.build [--force] [--verbose]
Each .cu file becomes an object in csrc/build/ (compiled in parallel), then one shared
library is linked next to this file.  The CUDA runtime is linked statically, so the
library loads on a machine without a driver (every compute entry point then reports
LC_ERR_CUDA).
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libleafcutter_b200.so")
SOURCES = ["common.cu", "dequant.cu", "scan.cu", "sampler.cu", "synth.cu", "ops.cu", "qgemv.cu", "qgemv_mma.cu", "qgemv_mma_q6k.cu", "qgemv_kq.cu", "qgemm_umma.cu", "moe.cu", "dist.cu", "attention.cu", "attention_stream.cu", "attention_prefill.cu", "engine.cu", "gguf.cu", "shard_engine.cu"]
HEADERS = ["lc_common.cuh", "lc_quant.cuh", "lc_kernels.h", "lc_synth.h", "lc_tma.cuh", "lc_planes.cuh", "lc_attn.cuh", os.path.join("..", "..", "include", "leafcutter_b200.h")]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-ffp-contract=off,-fno-fast-math",
    "-ccbin", "/usr/bin/g++",
]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(os.path.join(CSRC, "build"), exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, "build", src.replace(".cu", ".o"))
        objs.append(o)
        if force or not _newer(o, [s] + hdrs):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr + "\n")
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or force or not _newer(OUT, objs):
        cmd = [NVCC, "-shared", "-o", OUT] + objs + ["-cudart", "static", "-ccbin", "/usr/bin/g++", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr + "\n")
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
