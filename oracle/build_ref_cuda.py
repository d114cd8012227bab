#!/usr/bin/env python3
"""Compile the reference's own CUDA extension (its three translation units, unmodified, read where they lie in the
read-only reference tree) into oracle/_ref/crispybits_ref_C.so for sm_100a.  TEST / BASELINE INFRASTRUCTURE ONLY.

    python oracle/build_ref_cuda.py [path/to/reference]        (default: $CRISPYBITS_REFERENCE, else the tree beside the build)

The sources are Crispybits/Kernel/csrc/{bindings.cpp, packed_gemv.cu, packed_gemm.cu} (the list of the reference's
Crispybits/Kernel/setup.py:11-16, with its flags -O3 -std=c++17 -lineinfo); they are compiled with torch's generic
extension builder (nvcc + g++ + ninja), not with the reference's build script, and nothing is copied: only the
built module lands in oracle/_ref/, which git ignores and which travels to the GPU box like the library's own .so.
bench.py loads the module, when it is there, to time the reference's kernels on the same GPU beside this library's
(`reference_cuda` object of the bench line).  The product never loads it.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "crispybits_ref_C"
REF_ROOT = os.environ.get("CRISPYBITS_REFERENCE", os.path.join(os.sep, "root", "reference"))


def sources_present(ref_root=None):
    """True when the reference tree with its CUDA sources is on this machine."""
    return os.path.isdir(os.path.join(ref_root or REF_ROOT, "Crispybits", "Kernel", "csrc"))


def build(ref_root=None, verbose=False):
    src = os.path.join(ref_root or REF_ROOT, "Crispybits", "Kernel", "csrc")
    files = [os.path.join(src, f) for f in ("bindings.cpp", "packed_gemv.cu", "packed_gemm.cu")]
    if not all(os.path.exists(f) for f in files):
        raise FileNotFoundError(f"reference sources not found under {src}")
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    load(name=NAME, sources=files, build_directory=OUT, extra_cflags=["-O3", "-std=c++17"],
         extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo"], is_python_module=False, verbose=verbose)
    return os.path.join(OUT, NAME + ".so")


def load_module():
    """The built module (None when it has not been built): functions packed_gemv, packed_gemm, fused_gate_up,
    fused_qkv, sm_count, tile_n, max_rho with the reference's signatures (Crispybits/Kernel/csrc/bindings.cpp:32-40)."""
    path = os.path.join(OUT, NAME + ".so")
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True))
