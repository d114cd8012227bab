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


def test_decode_plan_is_host_arithmetic_and_stays_inside_an_sm():
    """cb_decode_plan needs no GPU.  Every plan covers all rows, fits the 227 KB a CTA may ask for, and a plan meant to
    share an SM between two CTAs fits half of it."""
    lib = ctypes.CDLL(os.path.join(PKG, "lib", "libcrispybits_b200.so"))
    lib.cb_decode_plan.argtypes = [ctypes.c_int] + [ctypes.c_int64] * 5 + [ctypes.c_int, ctypes.POINTER(ctypes.c_longlong)]
    out = (ctypes.c_longlong * 7)()
    shapes = [(4096, 4096), (11008, 4096), (4096, 11008), (22016, 4096), (12288, 4096), (512, 4096), (32000, 4096),
              (64, 256), (2, 256), (130, 512), (4096, 14336), (28672, 8192)]
    seen_two_per_sm = False
    for n, k in shapes:
        for bits in (2, 3, 4):
            for batch in (1, 2, 5, 8):
                for split_k in (1, 2, 4):
                    for rho in (0, 1, 2, 4):
                        for sms in (148, 132, 8):
                            rc = lib.cb_decode_plan(bits, batch, n, k, split_k, rho, sms, out)
                            assert rc == 0, (n, k, bits, batch, split_k, rho, sms)
                            grid, smem, split, rpp, slots, passes, slabs = (int(v) for v in out)
                            assert grid == slabs * split and grid >= 1
                            assert split >= min(split_k, k // 256) and 16 <= rpp <= 32 and rpp % 2 == 0
                            assert 1 <= slots <= passes
                            assert slabs * passes * rpp >= n, "the passes of all slabs cover every row"
                            assert smem <= 227 * 1024
                            if grid > sms and split == 1:
                                assert smem <= 112 * 1024
                                seen_two_per_sm = True
                            if grid > 2 * sms and split == 1:
                                assert smem <= 75 * 1024 and passes == 1, "three CTAs per SM: a third of the shared memory, one pass"
    assert seen_two_per_sm
    # outside the kernel's domain: K not a multiple of 256, batch above 8
    assert lib.cb_decode_plan(4, 1, 4096, 4096 + 128, 1, 1, 148, out) != 0
    assert lib.cb_decode_plan(4, 9, 4096, 4096, 1, 1, 148, out) != 0


def test_python_struct_mirrors_match_the_c_header(tmp_path):
    """The ctypes mirrors in crispybits_kernels/_C.py lay cb_weight and cb_scatter out exactly as a C compiler lays out
    the header's declarations (size and the offset of every field)."""
    import subprocess
    import sys

    sys.path.insert(0, PKG)
    from crispybits_kernels import _C

    mirrors = {"cb_weight": _C._Weight, "cb_scatter": _C._Scatter}
    lines = []
    for cname, cls in mirrors.items():
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for field, _ in cls._fields_:
            lines.append(f'printf("{cname}.{field} %zu\\n", offsetof({cname}, {field}));')
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "crispybits_b200.h"\nint main(void) {\n'
                   + "\n".join(lines) + "\nreturn 0; }\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True,
                                                       text=True).stdout.splitlines())
    for cname, cls in mirrors.items():
        assert int(got[cname]) == ctypes.sizeof(cls), cname
        for field, _ in cls._fields_:
            assert int(got[f"{cname}.{field}"]) == getattr(cls, field).offset, (cname, field)
    # and the header declares no field that the mirror lacks
    text = open(os.path.join(ROOT, "include", "crispybits_b200.h")).read()
    for cname, cls in mirrors.items():
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        declared = re.findall(r"(\w+)(?:\[\d+\])?\s*;", body)
        assert declared == [f for f, _ in cls._fields_], cname
