"""Builds libgraphop_b200.so (the C ABI of include/graphop_b200.h) in-tree with nvcc for sm_100a.

``python -m custom_op_benchmark_b200.build`` compiles the translation units in parallel and
links them next to this file.  nvcc cross-compiles, so no GPU is needed to build.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libgraphop_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
UNITS = ["graphop_capi_f32.cu", "graphop_capi_f64.cu", "graphop_capi_bf16.cu", "graphop_capi_attn_f32.cu",
         "graphop_capi_attn_f64.cu", "graphop_capi_attn_bf16.cu", "graphop_capi_misc.cu", "graphop_capi_static.cu"]
NVCC_FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-Xcompiler", "-fPIC"]


def _sources():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    deps.append(os.path.join(HERE, "..", "include", "graphop_b200.h"))
    return deps


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def build(force=False, verbose=False, ptxas_info=False):
    """Compile and link the library if any source is newer than it.  Returns the library path."""
    deps = _sources()
    if not force and not _stale(LIB, deps):
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])

    def compile_one(unit):
        obj = os.path.join(OBJ_DIR, unit.replace(".cu", ".o"))
        if not force and not _stale(obj, deps):
            return obj, ""
        cmd = [nvcc] + flags + ["-c", os.path.join(CSRC, unit), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (unit, res.stdout + res.stderr))
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=len(UNITS)) as pool:
        results = list(pool.map(compile_one, UNITS))
    if verbose or ptxas_info:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    cmd = [nvcc, "-shared", "-o", LIB] + [o for o, _ in results] + ["-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
