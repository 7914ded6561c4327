"""Build ``libteletron_b200.so`` in-tree with nvcc for sm_100a.

``python -m teletron_b200.build`` compiles every ``csrc/*.cu`` with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and links one shared library next to the
sources (``teletron_b200/lib/``).  The library has no PyTorch dependency: Python reaches it through
``ctypes`` (:mod:`teletron_b200.ops._lib`), so a build takes seconds and the binary travels with the
source tree.  Files are rebuilt only when a source or header is newer than its object.
"""

from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "lib")
LIB = os.path.join(OUT, "libteletron_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "--expt-relaxed-constexpr"]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _needs(obj: str, deps) -> bool:
    if not os.path.isfile(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    nvcc = find_nvcc()
    os.makedirs(OUT, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(SRC, "*.cu")))
    headers = glob.glob(os.path.join(SRC, "*.cuh")) + glob.glob(os.path.join(SRC, "*.h"))
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    jobs = []
    for src in sources:
        obj = os.path.join(OUT, os.path.basename(src)[:-3] + ".o")
        if force or ptxas_info or _needs(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc] + flags + ["-I", SRC, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(compile_one, jobs):
            if verbose or ptxas_info or r.returncode:
                sys.stderr.write(f"[nvcc] {os.path.basename(src)}\n{r.stdout}{r.stderr}")
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
    objs = [os.path.join(OUT, os.path.basename(s)[:-3] + ".o") for s in sources]
    if jobs or not os.path.isfile(LIB):
        cmd = [nvcc, "-shared", "-o", LIB] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
