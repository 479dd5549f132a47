"""Regenerates tests/golden/partition_csr.json by running the reference's own partition_csr
(part_csr.py:13-27) on the CPU.  Needs the reference checkout; pass its directory as argv[1].
The committed JSON is what the tests read; this script never runs under pytest."""
import importlib.util
import json
import os
import sys

import torch as th


def main(ref_dir):
    spec = importlib.util.spec_from_file_location("ref_part_csr", os.path.join(ref_dir, "part_csr.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    cases = [
        ([0, 4, 8, 10], 4),          # the example in the reference's own __main__
        ([0, 4, 8, 10], 3),
        ([0, 4, 8, 10], 32),
        ([0, 0, 5, 5, 6], 2),        # empty rows are skipped
        ([0, 0, 0], 2),              # no edges at all
        ([0, 1, 2, 3, 4], 1),
        ([0, 33, 33, 100, 164, 165], 32),
        ([3, 7, 7, 12], 2),          # first position is not 0
        ([0, 64], 32),
        ([0, 65], 32),
        ([5], 4),                    # no rows
    ]
    g = th.Generator().manual_seed(0)
    for n, hi, cs in [(40, 9, 4), (25, 70, 32), (60, 3, 2), (10, 200, 32), (50, 40, 7)]:
        deg = th.randint(0, hi, (n,), generator=g)
        deg[th.rand(n, generator=g) < 0.3] = 0
        ip = th.cat([th.zeros(1, dtype=th.long), th.cumsum(deg, 0)]).tolist()
        cases.append((ip, cs))
    out = []
    for ip, cs in cases:
        row, ptr = mod.partition_csr(th.tensor(ip, dtype=th.long), chunk_size=cs)
        out.append({"indptr": ip, "chunk_size": cs, "row": [int(v) for v in row.tolist()],
                    "row_dtype": str(row.dtype), "indptr_": ptr.tolist(), "indptr_dtype": str(ptr.dtype)})
    # int32 input still gives int64 output
    row, ptr = mod.partition_csr(th.tensor([0, 4, 8, 10], dtype=th.int32), chunk_size=3)
    out.append({"indptr": [0, 4, 8, 10], "chunk_size": 3, "input_dtype": "torch.int32",
                "row": row.tolist(), "row_dtype": str(row.dtype), "indptr_": [int(v) for v in ptr.tolist()],
                "indptr_dtype": str(ptr.dtype)})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "partition_csr.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=0)
    print("wrote", path, len(out), "cases")


if __name__ == "__main__":
    main(sys.argv[1])
