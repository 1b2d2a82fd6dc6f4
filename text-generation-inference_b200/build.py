"""Builds csrc/*.cu into the in-tree C-ABI shared libraries with nvcc for sm_100a only.

`python text-generation-inference_b200/build.py [--force] [--verbose] [--seq]`
  libb200_tgis.so  every source: the whole C ABI of include/b200_tgis.h
  libb200_seq.so   the sources the hybrid decoder families need (seq_*.cu + the block allocator and the runtime pieces); a
                   process that serves only such a model builds and loads this one (`--seq`, `build(target="seq")`)
Objects are shared between the two.  The libraries are git-ignored; they are built in the tree at first use.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libb200_tgis.so")
SEQ_LIB = os.path.join(HERE, "libb200_seq.so")
SEQ_EXTRA_SOURCES = ("runtime.cu", "kv_alloc.cu", "gemm_f16.cu")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the B200 path cannot be built (there is no CPU fallback)")
    return nvcc


def sources(target: str = "all"):
    every = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    if target == "seq":
        return [f for f in every if f.startswith("seq_") or f in SEQ_EXTRA_SOURCES]
    return every


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, target: str = "all") -> str:
    """target "all": both libraries; "seq": libb200_seq.so only (compiles nothing else)."""
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "b200_tgis.h"))
    headers = [h for h in headers if os.path.exists(h)]
    jobs = []
    for src in sources(target):
        obj = os.path.join(OBJ, src[:-3] + ".o")
        if force or _stale(obj, [os.path.join(CSRC, src)] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-I", os.path.join(os.path.dirname(HERE), "include"), "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(compile_one, jobs):
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError(f"nvcc failed on {src}")
            if verbose:
                sys.stderr.write(f"== {src}\n{r.stderr}\n")
            with open(os.path.join(OBJ, src[:-3] + ".ptxas.txt"), "w") as f:
                f.write(r.stderr)
    for lib, which in ((LIB, "all"), (SEQ_LIB, "seq")):
        if target == "seq" and which == "all":
            continue
        objs = [os.path.join(OBJ, s[:-3] + ".o") for s in sources(which)]
        if force or _stale(lib, objs):
            part = f"{lib}.{os.getpid()}.part"  # linked aside and renamed: a concurrent first use never loads half a file
            cmd = [nvcc, "-shared", "-o", part, *objs, "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError("link failed")
            os.replace(part, lib)
    return SEQ_LIB if target == "seq" else LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, target="seq" if "--seq" in sys.argv else "all"))
