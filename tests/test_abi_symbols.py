"""The C-ABI library loads on a machine without a GPU and exports every function that
include/crispybits_b200.h declares (no compute is attempted here)."""
import ctypes
import os
import re

from conftest import PKG, ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "crispybits_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("cb_packed_gemv", "cb_packed_gemm", "cb_fused_qkv", "cb_fused_gate_up", "cb_unpack_codes",
                 "cb_gemv_scratch_bytes", "cb_sm_count", "cb_tile_n", "cb_max_rho", "cb_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(os.path.join(PKG, "lib", "libcrispybits_b200.so"))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    lib.cb_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.cb_version()
    assert lib.cb_tile_n() == 16
    lib.cb_gemv_scratch_bytes.restype = ctypes.c_size_t
    lib.cb_gemv_scratch_bytes.argtypes = [ctypes.c_int64] * 3
    assert lib.cb_gemv_scratch_bytes(1, 4096, 1) == 0
    # fixed region of 65536 arrival counters + 3 partial planes of 4096 floats
    assert lib.cb_gemv_scratch_bytes(1, 4096, 3) == 65536 * 4 + 3 * 4096 * 4


def test_product_package_does_not_reach_into_the_oracle():
    """The shipped package must not import or execute anything under oracle/."""
    for dirpath, _, files in os.walk(PKG):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "cb_oracle" not in src and "import oracle" not in src and "from oracle" not in src, f
