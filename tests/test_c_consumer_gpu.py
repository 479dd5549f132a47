"""The C ABI used the way a non-Python host would: tests/c_consumer_gpu.c (C99, CUDA runtime only) is compiled with
gcc against include/graphop_b200.h, linked to the shared library and run on the GPU."""
import os
import subprocess

import pytest

from helpers import ROOT
from custom_op_benchmark_b200 import _capi

pytestmark = pytest.mark.gpu


def test_c_program_runs_an_op_through_the_c_abi(tmp_path):
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    lib = _capi.LIB_PATH
    exe = tmp_path / "c_consumer_gpu"
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(cuda, "include"), os.path.join(ROOT, "tests", "c_consumer_gpu.c"), "-o", str(exe),
           "-L" + os.path.dirname(lib), "-l:" + os.path.basename(lib), "-Wl,-rpath," + os.path.dirname(lib),
           "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-lm"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and run.stdout.strip().endswith("ok"), (run.returncode, run.stdout, run.stderr)
