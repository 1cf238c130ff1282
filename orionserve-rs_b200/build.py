"""Builds ``liborion_cuda.so`` (sm_100a only) from ``csrc/`` with nvcc, in-tree."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "liborion_cuda.so")
SOURCES = ["elementwise.cu", "attention.cu", "attention_prefill.cu", "attention_prefill_tc.cu", "gemm_simt.cu", "tp_fused.cu", "gemm_tc.cu", "model.cu", "c_api.cu",
           "tp_nccl.cpp", "driver.cpp", "driver_sched.cpp", "driver_api.cpp", "checkpoint.cpp", "selftest.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
         "-I", "/usr/include"]


if os.environ.get("ORION_EXTRA_NVCC_FLAGS"):  # e.g. -DNAME for a compile-time A/B (rebuild with --force)
    FLAGS.extend(os.environ["ORION_EXTRA_NVCC_FLAGS"].split())
if os.environ.get("ORION_TRACE"):  # phase traces of the GEMM and the hand-over kernels (rebuild with --force)
    FLAGS.append("-DORION_TRACE")


def _newer(a: str, b: str) -> bool:
    return (not os.path.exists(b)) or os.path.getmtime(a) > os.path.getmtime(b)


def _deps() -> list[str]:
    root = os.path.dirname(HERE)
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return hdrs + [os.path.join(root, "include", "orion_cuda.h"), os.path.join(root, "include", "orion_driver.h")]


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    deps = _deps()
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src + ".o")
        if force or _newer(s, o) or any(_newer(h, o) for h in deps):
            extra = ["-Xptxas", "-v"] if verbose else []
            lang = ["-x", "cu"] if src.endswith(".cpp") else []
            jobs.append((src, [NVCC, *FLAGS, *extra, *lang, "-c", s, "-o", o]))

    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return name, r.returncode, r.stdout

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for name, rc, out in ex.map(run, jobs):
            if verbose or rc != 0:
                sys.stderr.write(f"--- {name}\n{out}\n")
            if rc != 0:
                raise RuntimeError(f"nvcc failed on {name}")
    objs = [os.path.join(OBJ, s + ".o") for s in SOURCES]
    if force or jobs or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-ldl", "-lpthread"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
