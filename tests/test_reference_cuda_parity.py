"""This library against the reference's OWN CUDA kernels on the same GPU and the same inputs.

oracle/build_ref_cuda.py compiles the reference's extension (Crispybits/Kernel/csrc/{bindings.cpp, packed_gemv.cu,
packed_gemm.cu}, unmodified) for sm_100a into oracle/_ref/.  Where that module is present both are called with identical
positional arguments (the seven entry points share their signatures, Crispybits/Kernel/csrc/bindings.cpp:32-40) and
the outputs must agree to fp16 rounding; the reference's output is also held against the CPU oracle, which pins the
oracle to the reference as it runs on this hardware.  Skipped where the module has not been built.
"""
import pytest
import torch

from helpers import make, rel_err, rope_tables
from oracle import build_ref_cuda

pytestmark = pytest.mark.gpu
DEV = "cuda"
H = torch.float16


@pytest.fixture(scope="module")
def ref():
    mod = build_ref_cuda.load_module()
    if mod is None:
        pytest.skip("oracle/_ref/crispybits_ref_C.so is not built (python oracle/build_ref_cuda.py)")
    return mod


def _parts(w):
    bias = w.bias if w.bias is not None else torch.empty(0, device=DEV, dtype=w.scales.dtype)
    return w.packed, w.scales, w.zeros, bias


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("n,k", [(4096, 4096), (300, 200), (1000, 1536)])
def test_decode_gemv_matches_the_reference_kernel(ref, bits, n, k):
    from crispybits_kernels import _C
    w, wd, bd = make(n, k, bits, H, DEV, True, 40 + bits)
    ws_a, ws_b = (torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(2))
    for B in (1, 3):
        x = torch.randn(B, k, device=DEV, dtype=H, generator=torch.Generator(DEV).manual_seed(B))
        for split_k in (1, 3):
            for act in (0, 1, 2):
                theirs = ref.packed_gemv(x, *_parts(w), bits, k, 128, split_k, 1, act, ws_a)
                ours = _C.packed_gemv(x, *_parts(w), bits, k, 128, split_k, 1, act, ws_b)
                assert rel_err(ours, theirs.float()) < 1e-3, (B, split_k, act)
        fp32 = x.float() @ wd.T + bd
        assert rel_err(ref.packed_gemv(x, *_parts(w), bits, k, 128, 1, 1, 0, ws_a), fp32) < 2e-3    # reference vs oracle
    assert ws_a.tolist() == [0, 0] and ws_b.tolist() == [0, 0]


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("M", [33, 320])
def test_prefill_gemm_matches_the_reference_kernel(ref, bits, M):
    from crispybits_kernels import _C
    n, k = 512, 1024
    w, wd, bd = make(n, k, bits, H, DEV, True, 50 + bits, 128, 0.02)
    x = torch.randn(M, k, device=DEV, dtype=H, generator=torch.Generator(DEV).manual_seed(M))
    for tc in (True, False):
        for act in (0, 2):
            theirs = ref.packed_gemm(x, *_parts(w), bits, k, 128, act, tc)
            ours = _C.packed_gemm(x, *_parts(w), bits, k, 128, act, tc)
            # the tensor-core paths multiply fp16-rounded weights; summation order differs between wmma and tcgen05
            assert rel_err(ours, theirs.float()) < 1.5e-3, (tc, act)
    fp32 = x.float() @ wd.T + bd
    assert rel_err(ref.packed_gemm(x, *_parts(w), bits, k, 128, 0, False), fp32) < 2e-3


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_fused_gate_up_matches_the_reference_kernel(ref, bits):
    from crispybits_kernels import _C
    n, k = 1376, 1024
    g, gd, _ = make(n, k, bits, H, DEV, False, 60 + bits, 128, 0.03)
    u, ud, _ = make(n, k, bits, H, DEV, False, 70 + bits, 128, 0.03)
    ws_a, ws_b = (torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(2))
    for B in (1, 4):
        x = torch.randn(B, k, device=DEV, dtype=H, generator=torch.Generator(DEV).manual_seed(9 + B))
        for split_k in (1, 2):
            theirs = ref.fused_gate_up(x, g.packed, g.scales, g.zeros, u.packed, u.scales, u.zeros, bits, k, 128, split_k, 1, ws_a)
            ours = _C.fused_gate_up(x, g.packed, g.scales, g.zeros, u.packed, u.scales, u.zeros, bits, k, 128, split_k, 1, ws_b)
            assert rel_err(ours, theirs.float()) < 1e-3, (B, split_k)
        fp32 = torch.nn.functional.silu(x.float() @ gd.T) * (x.float() @ ud.T)
        assert rel_err(theirs, fp32) < 2e-3


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("rope", [False, True])
def test_fused_qkv_matches_the_reference_kernel(ref, bits, rope):
    from crispybits_kernels import _C, permute_for_rope
    k, hd = 1024, 64
    q, _, _ = make(512, k, bits, H, DEV, True, 80 + bits)
    kk, _, _ = make(256, k, bits, H, DEV, True, 90 + bits)
    v, _, _ = make(256, k, bits, H, DEV, False, 100 + bits)
    if rope:
        q, kk = permute_for_rope(q, hd), permute_for_rope(kk, hd)
    x = torch.randn(2, k, device=DEV, dtype=H, generator=torch.Generator(DEV).manual_seed(3))
    cos, sin = rope_tables(2, hd, DEV) if rope else (torch.empty(0, device=DEV), torch.empty(0, device=DEV))
    ws_a, ws_b = (torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(2))
    args = (x, *_parts(q), *_parts(kk), *_parts(v), cos, sin, hd if rope else 0, hd if rope else 0, bits, k, 128)
    for split_k in (1, 2):
        theirs = ref.fused_qkv(*args, split_k, 1, ws_a)
        ours = _C.fused_qkv(*args, split_k, 1, ws_b)
        for a, b in zip(ours, theirs):
            assert rel_err(a, b.float()) < 1e-3, split_k
