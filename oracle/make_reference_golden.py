"""Golden vectors from the reference itself.  TEST INFRASTRUCTURE ONLY.

Runs the reference's CUDA extension (built unmodified by oracle/build_reference.py into
oracle/_ref) on a GPU, on small seeded graphs whose rows span several partition_csr chunks, and
stores inputs and outputs of all eight ops under tests/golden/reference_cuda_*.npz.  The tests
compare the CPU oracle and the CUDA kernels of this package with these files; nothing reads the
reference at test time.

    python oracle/make_reference_golden.py [output_dir]        (needs a CUDA device)
"""
import os
import sys

import numpy as np
import torch as th

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from custom_op_benchmark_b200 import graphs  # noqa: E402
from custom_op_benchmark_b200.part_csr import partition_csr  # noqa: E402
from oracle.build_reference import load_reference  # noqa: E402

CASES = [
    # name, nodes, degree list maker, heads, dim, dtype, chunk size
    ("f32_h2_d8", 150, 2, 8, th.float32, 32),
    ("f32_h1_d16", 120, 1, 16, th.float32, 32),
    ("f64_h4_d4", 90, 4, 4, th.float64, 8),
]


def make_graph(n, seed):
    g = th.Generator().manual_seed(seed)
    deg = th.randint(0, 12, (n,), generator=g)
    deg[th.rand(n, generator=g) < 0.2] = 0
    deg[3] = 300          # ten chunks of 32: the reference's cross-chunk atomic path
    deg[n // 2] = 77
    dst = th.repeat_interleave(th.arange(n), deg)
    # sources from the first third of the nodes only: the transposed CSR then has fewer chunks than the
    # row CSR, which the reference's dx launch needs to be complete (graphop_kernel.cu:566, 588)
    src = th.randint(0, n // 3, (int(deg.sum()),), generator=g)
    return graphs.coo_to_graph(dst, src, n, index_dtype=th.int64)


def main(out_dir):
    ref = load_reference()
    if ref is None:
        raise SystemExit("oracle/_ref holds no build of the reference; run oracle/build_reference.py first")
    dev = "cuda:0"
    for ci, (name, n, h, d, dtype, cs) in enumerate(CASES):
        gr = make_graph(n, 100 + ci)
        e = gr.n_edges
        row, ptr = partition_csr(gr.indptr, cs)
        col, ptr_t = partition_csr(gr.indptr_t, cs)
        gen = th.Generator().manual_seed(200 + ci)
        node = lambda: (th.rand(n, h, d, generator=gen, dtype=th.float64) - 0.3).to(dtype)
        edge = lambda: th.rand(e, h, generator=gen, dtype=th.float64).to(dtype)
        A, B, X, dY = node(), node(), node(), node()
        w, x_e, dy_e = edge(), edge() * 4 - 2, edge() - 0.5
        Be = (th.rand(e, d, generator=gen, dtype=th.float64) - 0.5).to(dtype)
        if h == 1:
            A, B, X, dY = (t.view(n, d) for t in (A, B, X, dY))
            w, x_e, dy_e = (t.view(e) for t in (w, x_e, dy_e))
        c = lambda t: t.to(dev)
        R = [c(row), c(ptr), c(gr.eid), c(gr.indices)]
        C = [c(col), c(ptr_t), c(gr.eid_t), c(gr.indices_t)]
        out = {}
        out["mm_y"] = ref.maskedmm_csr_forward(*R, c(A), c(B))
        out["mm_dA"], out["mm_dB"] = ref.maskedmm_csr_backward(*R, *C, c(A), c(B), c(dy_e))
        out["nme_y"] = ref.node_mul_edge_forward(*R[:3], c(A), c(Be))
        out["nme_dA"], out["nme_dB"] = ref.node_mul_edge_backward(*R[:3], c(A), c(Be), c(dy_e))
        out["sm_y"] = ref.sparse_softmax_forward(*R[:3], c(x_e))
        out["sm_dx"] = ref.sparse_softmax_backward(*R[:3], out["sm_y"], c(dy_e))
        out["sm_y_t"] = ref.sparse_softmax_forward(*C[:3], c(x_e))
        out["spmm_y"] = ref.vector_spmm_forward(*R, c(w), c(X))
        out["spmm_dw"], out["spmm_dx"] = ref.vector_spmm_backward(*R, *C, c(w), c(dY), c(X))
        th.cuda.synchronize()
        # the reference sizes the grid of its dx kernel by the row CSR's chunk count
        # (graphop_kernel.cu:566, 588): dx is complete only when the transposed CSR has no more chunks
        dx_complete = col.numel() <= row.numel()
        arrays = {k: v.cpu().numpy() for k, v in out.items()}
        arrays.update(indptr=gr.indptr.numpy(), indices=gr.indices.numpy(), chunk_size=np.int64(cs),
                      A=A.numpy(), B=B.numpy(), X=X.numpy(), dY=dY.numpy(), w=w.numpy(), x_e=x_e.numpy(),
                      dy_e=dy_e.numpy(), Be=Be.numpy(), dx_complete=np.bool_(dx_complete),
                      chunks=np.array([row.numel(), col.numel()]))
        path = os.path.join(out_dir, "reference_cuda_%s.npz" % name)
        np.savez_compressed(path, **arrays)
        print("wrote", path, os.path.getsize(path), "bytes; dx complete:", dx_complete)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden"))
