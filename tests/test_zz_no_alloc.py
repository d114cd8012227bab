"""cb_packed_gemv_static_scratch: the decode GEMV for callers that cannot allocate device memory.

A serving loop that owns all device memory through its own arena, or a plugin that runs under a
foreign allocator, cannot hand the library a fresh scratch buffer (and must not have the library call
cudaMalloc behind its back).  For them the library carries the Split-K scratch itself, in a fixed
device array.  This file checks, straight through the C ABI, that the variant returns what the
ordinary entry point returns -- twice in a row, so that what the first call left in the shared array
cannot leak into the second -- and that it refuses requests larger than the array.

It is named to be collected last: a run that stops at the first failure has then already run
everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import make, ref_linear, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lib():
    from crispybits_kernels import _C
    lib = _C._lib
    lib.cb_packed_gemv_static_scratch.restype = ctypes.c_int
    lib.cb_packed_gemv_static_scratch.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(_C._Weight),
                                                  ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int64,
                                                  ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                                  ctypes.c_void_p]
    lib.cb_static_scratch_bytes.restype = ctypes.c_size_t
    return _C, lib


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_static_scratch_matches_ordinary_entry_point_twice(bits):
    _C, lib = _lib()
    n, k, B, split_k = 1000, 1536, 3, 6
    w, wd, bd = make(n, k, bits, torch.float16, DEV, bias=True, seed=40 + bits)
    rec = _C._Weight(w.packed.data_ptr(), w.scales.data_ptr(), w.zeros.data_ptr(), w.bias.data_ptr(), n)
    stream = torch.cuda.current_stream().cuda_stream
    own = torch.zeros(lib.cb_gemv_scratch_bytes(B, n, split_k), dtype=torch.uint8, device=DEV)
    gen = torch.Generator(DEV).manual_seed(bits)
    for call in range(2):                       # two calls in a row share the library's array
        x = torch.randn(B, k, device=DEV, dtype=torch.float16, generator=gen)
        want = torch.empty(B, n, device=DEV, dtype=torch.float16)
        got = torch.full((B, n), float("nan"), device=DEV, dtype=torch.float16)
        rc = lib.cb_packed_gemv(x.data_ptr(), B, ctypes.byref(rec), want.data_ptr(), k, bits, 128, 1, split_k, 1, 2,
                                own.data_ptr(), own.numel(), stream)
        assert rc == 0, lib.cb_last_error()
        rc = lib.cb_packed_gemv_static_scratch(x.data_ptr(), B, ctypes.byref(rec), got.data_ptr(), k, bits, 128, 1,
                                               split_k, 1, 2, stream)
        assert rc == 0, lib.cb_last_error()
        torch.cuda.synchronize()
        assert rel_err(got, want.float()) < 2e-3, f"call {call}"
        assert rel_err(got, ref_linear(x, wd, bd, "silu")) < 2e-3, f"call {call}"


def test_static_scratch_without_split_and_limits():
    _C, lib = _lib()
    assert lib.cb_static_scratch_bytes() == 65536 * 4 + (1 << 20)
    n, k = 4096, 4096
    w, wd, _ = make(n, k, 3, torch.float16, DEV, seed=77, std=0.02)
    rec = _C._Weight(w.packed.data_ptr(), w.scales.data_ptr(), w.zeros.data_ptr(), 0, n)
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.randn(1, k, device=DEV, dtype=torch.float16)
    out = torch.empty(1, n, device=DEV, dtype=torch.float16)
    for split_k in (1, 4, 64):                 # 64 * 1 * 4096 floats = exactly the array's room
        rc = lib.cb_packed_gemv_static_scratch(x.data_ptr(), 1, ctypes.byref(rec), out.data_ptr(), k, 3, 128, 1,
                                               split_k, 1, 0, stream)
        assert rc == 0, lib.cb_last_error()
        torch.cuda.synchronize()
        assert rel_err(out, ref_linear(x, wd)) < 2e-3
    rc = lib.cb_packed_gemv_static_scratch(x.data_ptr(), 1, ctypes.byref(rec), out.data_ptr(), k, 3, 128, 1, 65, 1, 0,
                                           stream)
    assert rc == 1 and b"built-in array" in lib.cb_last_error()
    x8 = torch.randn(8, k, device=DEV, dtype=torch.float16)
    out8 = torch.empty(8, n, device=DEV, dtype=torch.float16)
    rc = lib.cb_packed_gemv_static_scratch(x8.data_ptr(), 8, ctypes.byref(rec), out8.data_ptr(), k, 3, 128, 1, 9, 1, 0,
                                           stream)
    assert rc == 1
    rc = lib.cb_packed_gemv_static_scratch(x8.data_ptr(), 8, ctypes.byref(rec), out8.data_ptr(), k, 3, 128, 1, 8, 1, 0,
                                           stream)
    assert rc == 0, lib.cb_last_error()
    torch.cuda.synchronize()
    assert rel_err(out8, ref_linear(x8, wd)) < 2e-3


@pytest.mark.parametrize("dtype,gs", [(torch.float32, 128), (torch.float16, 64)])
def test_static_scratch_split_k_through_the_generic_kernel_twice(dtype, gs):
    """fp32 activations, or a group size other than 128, take the shape-generic decode kernel: its Split-K partial
    sums and arrival counters then live in the library's array.  Two calls in a row, against the ordinary entry point
    with the caller's own buffer."""
    _C, lib = _lib()
    n, k, B, split_k, bits = 520, 1024, 2, 5, 3
    w, wd, bd = make(n, k, bits, dtype, DEV, bias=True, seed=91, gs=gs)
    rec = _C._Weight(w.packed.data_ptr(), w.scales.data_ptr(), w.zeros.data_ptr(), w.bias.data_ptr(), n)
    stream = torch.cuda.current_stream().cuda_stream
    own = torch.zeros(lib.cb_gemv_scratch_bytes(B, n, split_k), dtype=torch.uint8, device=DEV)
    code = {torch.float32: 0, torch.float16: 1}[dtype]
    gen = torch.Generator(DEV).manual_seed(5)
    for call in range(2):
        x = torch.randn(B, k, device=DEV, dtype=dtype, generator=gen)
        want = torch.empty(B, n, device=DEV, dtype=dtype)
        got = torch.full((B, n), float("nan"), device=DEV, dtype=dtype)
        rc = lib.cb_packed_gemv(x.data_ptr(), B, ctypes.byref(rec), want.data_ptr(), k, bits, gs, code, split_k, 1, 0,
                                own.data_ptr(), own.numel(), stream)
        assert rc == 0, lib.cb_last_error()
        rc = lib.cb_packed_gemv_static_scratch(x.data_ptr(), B, ctypes.byref(rec), got.data_ptr(), k, bits, gs, code,
                                               split_k, 1, 0, stream)
        assert rc == 0, lib.cb_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}"          # same kernel, same split order
        assert rel_err(got, ref_linear(x, wd, bd)) < (1e-4 if dtype == torch.float32 else 2e-3), f"call {call}"


def test_static_scratch_refuses_more_tiles_than_counters():
    _C, lib = _lib()
    # ceil(N/16) > 65536 with a K split: documented as CB_ERR_INVALID (nothing is launched, pointers are not read)
    rec = _C._Weight(16, 16, 16, 0, 16 * 65536 + 16)
    rc = lib.cb_packed_gemv_static_scratch(16, 1, ctypes.byref(rec), 16, 64, 4, 32, 1, 2, 1, 0, None)
    assert rc == 1 and b"arrival counters" in lib.cb_last_error()
