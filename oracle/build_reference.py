"""Builds the reference's own CUDA extension as a checker.  TEST INFRASTRUCTURE ONLY.

Compiles graphop/graphop.cpp and graphop/graphop_kernel.cu of the reference checkout, unmodified
and from where they lie, into oracle/_ref/graphop_ref*.so for sm_100a, with oracle/ref_shim on
the include path to stand in for the THC headers torch no longer ships.  The result is a torch
extension module exporting the reference's eight functions; tests and the golden-vector script
load it with `load_reference()`.  Nothing in the product package touches it.

    python oracle/build_reference.py [reference_dir]

The reference checkout is found, in this order, from the command line, from the environment
variable GRAPHOP_REFERENCE_DIR, or as a directory named `reference` beside this repository.
"""
import glob
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "graphop_ref"


def default_reference_dir():
    return os.environ.get("GRAPHOP_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_dir=None, verbose=False):
    from torch.utils.cpp_extension import load
    ref_dir = ref_dir or default_reference_dir()
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    src = os.path.join(ref_dir, "graphop")
    return load(name=NAME, sources=[os.path.join(src, "graphop.cpp"), os.path.join(src, "graphop_kernel.cu")],
                extra_include_paths=[os.path.join(HERE, "ref_shim")],
                extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-O3"],
                extra_cflags=["-O2", "-w"], build_directory=OUT, verbose=verbose)


def load_reference():
    """The prebuilt module, or None when oracle/_ref holds no build."""
    import torch  # noqa: F401  (the extension links against libtorch)
    hits = glob.glob(os.path.join(OUT, NAME + "*.so"))
    if not hits:
        return None
    spec = importlib.util.spec_from_file_location(NAME, hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else default_reference_dir()
    if not os.path.isdir(ref):
        print("reference checkout not found at", ref)
        sys.exit(0)
    m = build(ref, verbose="-v" in sys.argv)
    print("built", [n for n in dir(m) if n.endswith("ward")])
