"""Builds libancora_b200.so in-tree with nvcc for sm_100a.

    python -m ancora_cutile_b200.build          # incremental
    python -m ancora_cutile_b200.build --force
    python -m ancora_cutile_b200.build --profile   # libancora_b200_prof.so: stall accounting compiled
                                                   # into the Newton-Schulz chain kernel (profile_chain.py)

nvcc cross-compiles without a GPU.  The library links the static CUDA runtime only;
the driver's tensor-map encoder and NCCL are looked up at run time, so the shared
object loads on a machine without a GPU (its compute calls then fail with a status).
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libancora_b200.so")
SOURCES = ["runtime.cu", "adamw.cu", "muon_elem.cu", "ns_gemm.cu", "muon_plan.cu", "grad_prod.cu", "zero1.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--ftz=false", "--prec-div=true",
              "--prec-sqrt=true", "--fmad=true"]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build libancora_b200.so")
    return exe


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


PROF_LIB = os.path.join(PKG, "libancora_b200_prof.so")


def build(force=False, verbose=False, profile=False):
    nvcc = _nvcc()
    global OBJ, LIB
    if profile:
        saved = OBJ, LIB
        OBJ, LIB = os.path.join(PKG, "build_prof"), PROF_LIB
        try:
            return _build(nvcc, force, verbose, ["-DANC_CHAIN_PROFILE"])
        finally:
            OBJ, LIB = saved
    return _build(nvcc, force, verbose, [])


def _build(nvcc, force, verbose, extra):
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, "anc_internal.h"),
               os.path.join(PKG, "..", "include", "ancora_b200.h")]
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            jobs.append([nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=6) as ex:
        logs = list(ex.map(run, jobs))
    if verbose:
        for l in logs:
            sys.stderr.write(l)
    if jobs or force or _stale(LIB, objs):
        run([nvcc, "-shared", "-o", LIB] + objs + ["-cudart", "static", "-ldl", "-lpthread", "-lrt"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, profile="--profile" in sys.argv))
