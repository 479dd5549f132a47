"""Builds libgraphop_b200.so (the C ABI of include/graphop_b200.h) in-tree with nvcc for sm_100a, and
libgraphop_b200_bench.so, the instrumented twin bench.py uses to time single kernels (the same sources for
the element types the benchmark runs, compiled with -DGK_BENCH_HOOKS, plus csrc/bench/graphop_bench.cu).

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
BENCH_LIB = os.path.join(HERE, "libgraphop_b200_bench.so")
OBJ_DIR = os.path.join(HERE, "build")
UNITS = ["graphop_capi_f32.cu", "graphop_capi_f64.cu", "graphop_capi_bf16.cu", "graphop_capi_attn_f32.cu",
         "graphop_capi_attn_f64.cu", "graphop_capi_attn_bf16.cu", "graphop_capi_misc.cu", "graphop_capi_static.cu"]
# the instrumented twin: what bench.py's workloads call, plus the hooks themselves
BENCH_UNITS = ["graphop_capi_f32.cu", "graphop_capi_attn_f32.cu", "graphop_capi_attn_bf16.cu", "graphop_capi_misc.cu",
               os.path.join("bench", "graphop_bench.cu")]
BENCH_FLAG = "-DGK_BENCH_HOOKS"
# -fno-gnu-unique: the twin library holds the same templates as the product library; without it the dynamic linker
# merges their function-local statics (the "shared memory limit already raised" flags) across the two libraries
NVCC_FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fno-gnu-unique"]


def _sources():
    deps = []
    for root, _, files in os.walk(CSRC):
        deps += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".h"))]
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


def build(force=False, verbose=False, ptxas_info=False, bench=True):
    """Compile and link the library (and, with bench=True, its instrumented twin) if any source is newer.
    Returns the library path."""
    deps = _sources()
    targets = [(LIB, UNITS, [], "")] + ([(BENCH_LIB, BENCH_UNITS, [BENCH_FLAG], "bench_")] if bench else [])
    todo = [t for t in targets if force or _stale(t[0], deps)]
    if not todo:
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])

    def compile_one(job):
        unit, extra, prefix = job
        obj = os.path.join(OBJ_DIR, prefix + os.path.basename(unit).replace(".cu", ".o"))
        if not force and not _stale(obj, deps):
            return obj, ""
        cmd = [nvcc] + flags + extra + ["-c", os.path.join(CSRC, unit), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (unit, res.stdout + res.stderr))
        return obj, res.stderr

    jobs = [(u, extra, prefix) for _, units, extra, prefix in todo for u in units]
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 4))) as pool:
        results = list(pool.map(compile_one, jobs))
    if verbose or ptxas_info:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    at = 0
    for lib, units, _, _ in todo:
        objs = [o for o, _ in results[at:at + len(units)]]
        at += len(units)
        # -Bsymbolic: the twin defines the same entry points as the product library; each binds to its own
        cmd = [nvcc, "-shared", "-Xlinker", "-Bsymbolic", "-o", lib] + objs + ["-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv,
                bench="--no-bench" not in sys.argv))
