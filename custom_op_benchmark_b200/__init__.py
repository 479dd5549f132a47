"""graphop for NVIDIA B200: sparse graph-attention operators (masked matmul on CSR edges,
sparse row softmax, node-edge multiply, vector SpMM, and their fused chain), forward and
backward, as hand-written sm_100a CUDA kernels behind the reference extension's Python
surface.

    from custom_op_benchmark_b200.graphop import *      # the 8 ops of the reference module
    from custom_op_benchmark_b200.wrapper import *      # the autograd Functions
    from custom_op_benchmark_b200.part_csr import partition_csr

    custom_op_benchmark_b200.compiled_graphop()         # the compiled module, importable as `graphop` afterwards
"""
from .part_csr import partition_csr, unchunked_rows  # noqa: F401

__version__ = "0.2.0"


def compiled_graphop():
    """Loads the compiled Python module `graphop` (csrc/binding/graphop_module.cpp: the eight functions of the
    reference's graphop/graphop.cpp:216-225, bound with pybind11 on top of the C ABI) and registers it in
    ``sys.modules`` under the reference's name, so that code written against the reference - its wrapper.py does
    ``import graphop`` - runs on it unchanged.  Raises ImportError when the module has not been built."""
    import importlib.util
    import os
    import sys
    import torch  # noqa: F401  (the module links against torch's libraries: they must be loaded first)
    from . import build as _build
    path = _build.module_path()
    if not os.path.exists(path):
        raise ImportError("%s is missing: build it with `python -m custom_op_benchmark_b200.build`" % path)
    loaded = sys.modules.get("graphop")
    if loaded is not None and getattr(loaded, "__file__", None) == path:
        return loaded
    spec = importlib.util.spec_from_file_location("graphop", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules["graphop"] = module
    return module
