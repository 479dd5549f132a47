"""The C-ABI shared library loads and exports every symbol include/graphop_b200.h and include/graphop_dlpack.h declare.
No compute call is made here (no GPU needed)."""
import os
import re
import subprocess

from helpers import ROOT
from custom_op_benchmark_b200 import _capi


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "graphop_b200.h")).read()
    body = text[text.index("#define GRAPHOP_DECLARE(SUF"):text.index("GRAPHOP_DECLARE(f32_i32")]
    ops = re.findall(r"int (graphop_\w+)_##SUF", body)
    suffixes = re.findall(r"^GRAPHOP_DECLARE\((\w+),", text, re.M)
    names = ["%s_%s" % (op, s) for op in ops for s in suffixes]
    planned = text[text.index("#define GRAPHOP_DECLARE_PLANNED"):text.index("#define GRAPHOP_DECLARE(SUF")]
    pops = re.findall(r"int (graphop_\w+)_##SUF", planned)
    psuf = re.findall(r"^GRAPHOP_DECLARE_PLANNED\((\w+),", text, re.M)
    names += ["%s_%s" % (op, s) for op in pops for s in psuf]
    names += re.findall(r"^(?:int|size_t|long long|const char\*) (graphop_\w+)\(", text, re.M)
    dl = open(os.path.join(ROOT, "include", "graphop_dlpack.h")).read()
    names += re.findall(r"^int (graphop_dl_\w+)\(", dl, re.M)
    return sorted(set(names))


def test_header_and_binding_agree():
    assert _header_symbols() == sorted(_capi.exported_symbols())
    assert len(_header_symbols()) == 12 * 6 + 10 * 3 + 21 + 10


def test_product_library_carries_no_benchmark_hooks():
    """Launch accounting, per-kernel timing and the gather probe live in the benchmark's instrumented twin only."""
    out = subprocess.run(["nm", "-D", "--defined-only", _capi.LIB_PATH], capture_output=True, text=True).stdout
    assert not re.findall(r"graphop_bench_\w+|graphop_profile_\w+|graphop_launch_count|graphop_gather_probe", out)
    twin = os.path.join(os.path.dirname(_capi.LIB_PATH), "libgraphop_b200_bench.so")
    if os.path.exists(twin):
        sym = subprocess.run(["nm", "-D", "--defined-only", twin], capture_output=True, text=True).stdout
        for name in ("graphop_bench_launch_count", "graphop_bench_profile_begin", "graphop_bench_profile_end",
                     "graphop_bench_gather_probe_i32", "graphop_attention_forward_f32_i32"):
            assert " T %s" % name in sym, name


def test_library_exports_every_declared_symbol():
    assert os.path.exists(_capi.LIB_PATH), "build with python -m custom_op_benchmark_b200.build"
    out = subprocess.run(["nm", "-D", "--defined-only", _capi.LIB_PATH], capture_output=True, text=True).stdout
    exported = set(re.findall(r" T (graphop_\w+)", out))
    missing = [s for s in _header_symbols() if s not in exported]
    assert not missing, missing


def test_library_loads_and_answers_host_only_queries():
    lib = _capi.lib()
    assert lib.graphop_version() >= 100
    assert lib.graphop_error_string(0) == b"ok"
    assert b"workspace" in lib.graphop_error_string(_capi.ERR_WORKSPACE)
    small = lib.graphop_workspace_bytes(_capi.OP_SPMM_FWD, 1000, 100, 4, 32, 4, 4)
    big = lib.graphop_workspace_bytes(_capi.OP_SPMM_FWD, 1_000_000, 100, 4, 32, 4, 4)
    assert 0 < small < big
    # int64 indices need room for the 32-bit copies
    assert lib.graphop_workspace_bytes(_capi.OP_SPMM_FWD, 1000, 100, 4, 32, 4, 8) > small
    assert lib.graphop_workspace_bytes(99, 1000, 100, 4, 32, 4, 4) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest
    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _capi.lib()


C_CONSUMER = r"""
#include <stdio.h>
#include <string.h>
#include "graphop_b200.h"
#include "graphop_dlpack.h"

int main(void) {
  /* host-only calls: none of them needs a GPU */
  if (graphop_version() < 100) return 1;
  if (!graphop_error_string(GRAPHOP_OK) || !graphop_error_string(GRAPHOP_ERR_INVALID_ARGUMENT)) return 2;
  if (strcmp(graphop_error_string(GRAPHOP_OK), graphop_error_string(GRAPHOP_ERR_WORKSPACE)) == 0) return 3;
  if (graphop_workspace_bytes(GRAPHOP_OP_SPMM_FWD, 1000, 100, 4, 32, 4, 4) == 0) return 4;
  if (graphop_plan_bytes(1000, 100, 100, 4) < sizeof(graphop_plan_t)) return 5;
  /* argument checks come before any CUDA call: a null graph is refused, not dereferenced */
  if (graphop_vector_spmm_forward_f32_i32(NULL, NULL, NULL, NULL, NULL, NULL, NULL, 4, 10, 5, 5, 1, -3, NULL, 0, NULL)
      == GRAPHOP_OK) return 6;
  {
    graphop_dltensor_t t;
    memset(&t, 0, sizeof t);
    if (sizeof t != 48 && sizeof t != 40) return 7;   /* DLTensor's layout: 48 bytes on LP64 */
  }
  printf("ok %d\n", graphop_version());
  return 0;
}
"""


def test_a_plain_c_program_compiles_links_and_runs_against_the_headers(tmp_path):
    """The boundary is a C ABI: a C99 translation unit includes both headers (no C++, no torch), links the shared
    library and calls its host-only entry points."""
    lib = _capi.LIB_PATH
    assert os.path.exists(lib)
    src = tmp_path / "consumer.c"
    src.write_text(C_CONSUMER)
    exe = tmp_path / "consumer"
    inc = os.path.join(ROOT, "include")
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I" + inc, str(src), "-o", str(exe),
           "-L" + os.path.dirname(lib), "-l:" + os.path.basename(lib), "-Wl,-rpath," + os.path.dirname(lib)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.startswith("ok "), (run.returncode, run.stdout, run.stderr)
