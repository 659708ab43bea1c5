"""Build oracle/_ref/forge_ref_kernels.so: the reference's own solver-path CUDA kernels for sm_100a.

Test infrastructure.  The five .cu files are compiled where they lie in the reference checkout (nothing is copied
into this repository); the only source of ours is the pybind stub oracle/ref_binding.cpp.  The reference builds the
same files with torch.utils.cpp_extension.load at import time (forge/backend/cuda/__init__.py:48-75); this recipe
does the same with an explicit sm_100a arch and an in-tree output folder, so that the library travels to the GPU
machine next to our own.  Without the reference checkout the build is skipped (returns None).

    python oracle/ref_build.py [path-to-reference-checkout]
"""
from __future__ import annotations

import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
NAME = "forge_ref_kernels"
KERNEL_FILES = ("quant_grid.cu", "solver.cu", "solver_sparsegptq14.cu", "bitpacking_sparsegptq14.cu", "sparse14_gemm.cu")


def built_path():
    p = os.path.join(OUT_DIR, NAME + ".so")
    return p if os.path.exists(p) else None


def build(reference_root: str, verbose: bool = False):
    src_dir = os.path.join(reference_root, "forge", "backend", "cuda")
    if not all(os.path.exists(os.path.join(src_dir, f)) for f in KERNEL_FILES):
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    load(name=NAME, sources=[os.path.join(HERE, "ref_binding.cpp")] + [os.path.join(src_dir, f) for f in KERNEL_FILES],
         extra_cflags=["-O3"], extra_cuda_cflags=["-O3"], build_directory=OUT_DIR, verbose=verbose, is_python_module=False)
    return built_path()


def load_built():
    """Import the built library (torch must be importable).  None when it has not been built."""
    p = built_path()
    if p is None:
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FORGE_REFERENCE_ROOT", "")
    print(build(root, verbose=True))
