"""Builds libgraphop_b200.so (the C ABI of include/graphop_b200.h) in-tree with nvcc for sm_100a,
libgraphop_b200_bench.so, the instrumented twin bench.py uses to time single kernels (the same sources for
the element types the benchmark runs, compiled with -DGK_BENCH_HOOKS, plus csrc/bench/graphop_bench.cu), and
ext/graphop.<abi>.so, the compiled Python module `graphop` (csrc/binding/graphop_module.cpp, g++ against torch's
headers, linked to libgraphop_b200.so).

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
         "graphop_capi_attn_f64.cu", "graphop_capi_attn_bf16.cu", "graphop_capi_misc.cu", "graphop_capi_static.cu",
         "graphop_capi_dlpack.cu", "graphop_capi_prep.cu"]
# the instrumented twin: what bench.py's workloads call, plus the hooks themselves
BENCH_UNITS = ["graphop_capi_f32.cu", "graphop_capi_attn_f32.cu", "graphop_capi_attn_bf16.cu", "graphop_capi_misc.cu",
               os.path.join("bench", "graphop_bench.cu")]
BENCH_FLAG = "-DGK_BENCH_HOOKS"
# -fno-gnu-unique: the twin library holds the same templates as the product library; without it the dynamic linker
# merges their function-local statics (the "shared memory limit already raised" flags) across the two libraries
NVCC_FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fno-gnu-unique"]


MODULE_SRC = os.path.join(CSRC, "binding", "graphop_module.cpp")
MODULE_DIR = os.path.join(HERE, "ext")


def module_path():
    import sysconfig
    return os.path.join(MODULE_DIR, "graphop" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_module(force=False):
    """Compile the pybind module `graphop` next to the library (needs torch's headers; no GPU).  Returns its path."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    out = module_path()
    deps = [MODULE_SRC, LIB, os.path.join(HERE, "..", "include", "graphop_b200.h"),
            os.path.join(HERE, "..", "include", "graphop_dlpack.h")]
    if not force and not _stale(out, deps):
        return out
    os.makedirs(MODULE_DIR, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-DTORCH_EXTENSION_NAME=graphop", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]:
        cmd += ["-isystem", inc]
    cmd += [MODULE_SRC, "-o", out, "-L" + HERE, "-lgraphop_b200", "-Wl,-rpath,$ORIGIN/.."]
    for lib_dir in ce.library_paths():
        cmd += ["-L" + lib_dir]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed for the graphop module:\n" + res.stdout + res.stderr)
    return out


def _sources():
    deps = []
    for root, _, files in os.walk(CSRC):
        deps += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "graphop_b200.h"))
    deps.append(os.path.join(HERE, "..", "include", "graphop_dlpack.h"))
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
    if "--no-module" not in sys.argv:
        print(build_module(force="--force" in sys.argv))
