"""Build libb200tm.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m lmdeploy_b200.build [--force]

Sources: lmdeploy_b200/csrc/*.cu  ->  lmdeploy_b200/lib/libb200tm.so
Objects are cached under build/obj and rebuilt when a source or header is newer.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(ROOT)
CSRC = os.path.join(ROOT, "csrc")
LIBDIR = os.path.join(ROOT, "lib")
OBJDIR = os.path.join(REPO, "build", "obj")
LIB = os.path.join(LIBDIR, "libb200tm.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-DB200_BUILD",
]


def _newest_header():
    t = 0.0
    for d in (CSRC, os.path.join(REPO, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def build(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr_t = _newest_header()
    jobs = []
    objs = []
    for s in srcs:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJDIR, s[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_t):
            jobs.append([NVCC, *FLAGS, "-c", src, "-o", obj])

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        return r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run([NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
             "-Xcompiler", "-fPIC", "-lcudart", "-lcuda" if os.environ.get("B200_LINK_LIBCUDA") else "-lcudart"])
    return LIB


HYBRID_SRC = os.path.join(CSRC, "hybrid", "hybrid_ops.cu")
HYBRID_LIB = os.path.join(LIBDIR, "libb200hybrid.so")


def build_hybrid(force=False):
    """lmdeploy_b200/csrc/hybrid/hybrid_ops.cu -> lmdeploy_b200/lib/libb200hybrid.so (the operators of hybrid decoders; one
    translation unit, independent of libb200tm.so so that serving such a model compiles nothing else).  Rebuilt when the
    source or its header is newer; concurrent builders write to a private name and rename."""
    hdr = os.path.join(REPO, "include", "b200_hybrid.h")
    hdir = os.path.dirname(HYBRID_SRC)
    newest = max([os.path.getmtime(hdr)] + [os.path.getmtime(os.path.join(hdir, f)) for f in os.listdir(hdir) if f.endswith((".cu", ".cuh"))])
    if not force and os.path.exists(HYBRID_LIB) and os.path.getmtime(HYBRID_LIB) >= newest:
        return HYBRID_LIB
    os.makedirs(LIBDIR, exist_ok=True)
    tmp = f"{HYBRID_LIB}.{os.getpid()}.tmp"
    cmd = [NVCC, *FLAGS, "-shared", "-o", tmp, HYBRID_SRC, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, HYBRID_LIB)
    return HYBRID_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
    print(build_hybrid(force="--force" in sys.argv))
