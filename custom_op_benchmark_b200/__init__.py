"""graphop for NVIDIA B200: sparse graph-attention operators (masked matmul on CSR edges,
sparse row softmax, node-edge multiply, vector SpMM, and their fused chain), forward and
backward, as hand-written sm_100a CUDA kernels behind the reference extension's Python
surface.

    from custom_op_benchmark_b200.graphop import *      # the 8 ops of the reference module
    from custom_op_benchmark_b200.wrapper import *      # the autograd Functions
    from custom_op_benchmark_b200.part_csr import partition_csr
"""
from .part_csr import partition_csr, unchunked_rows  # noqa: F401

__version__ = "0.1.0"
