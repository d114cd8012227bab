"""GPU parity tests: the CUDA path, called through the package API and the C ABI underneath, against
the CPU oracle on identical seeded inputs.

Integer work (unpacked codes) must be bit-exact.  Floating outputs are compared with the
fp32-accumulated dequantise-then-matmul of the oracle's weight; fp16 must stay within 2e-3 maximum
relative error (max|y-ref| / max|ref|), bf16 within 2e-2, fp32 within 1e-4.  Case lists follow the
reference's Crispybits/Kernel/tests/test_correctness.py.
"""
import functools
import os

import numpy as np
import pytest
import torch

from helpers import NAME, TOL, close, make, make_dict, ref_linear, rel_err, rope_tables, to_weight
from oracle import cb_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True, scope="module")
def _cuda_backend():
    from crispybits_kernels import ops
    assert ops._CUDA is not None, f"native library missing: {ops._IMPORT_ERROR}"
    ops.set_backend("cuda")
    yield


@functools.lru_cache(maxsize=64)
def cached(n, k, bits, dtype, bias=False, seed=0, gs=128, std=0.05):
    return make(n, k, bits, dtype, DEV, bias, seed, gs, std)


def test_library_reports_b200_geometry():
    import crispybits_kernels as ck
    from crispybits_kernels import _C
    assert "sm_100a" in _C.version()
    assert ck.sm_count() == torch.cuda.get_device_properties(0).multi_processor_count
    assert ck.tile_n() == 16
    for kind in ("gemv", "qkv", "gate_up"):
        assert ck.max_rho(3, kind) >= 1
    with pytest.raises(RuntimeError):
        ck.max_rho(3, "nope")


# ------------------------------------------------------------------ integer layout, bit-exact
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("n,k", [(7, 32), (5, 200), (64, 4096), (33, 4128), (3, 11008)])
def test_unpack_codes_bit_exact(bits, n, k):
    from crispybits_kernels import _C
    rng = np.random.default_rng(bits * 1000 + k)
    q = rng.integers(0, 1 << bits, size=(n, k), dtype=np.int32)
    packed = O.pack_codes(q, bits)
    got = _C.unpack_codes(torch.from_numpy(packed).to(DEV), bits, k).cpu().numpy()
    assert np.array_equal(got, q)


def test_unpack_golden_bit_exact(golden):
    from crispybits_kernels import _C
    for tag in [c for c in golden["cases"].tolist() if c.startswith("lin_")]:
        bits, k = int(tag.split("_")[1][1:]), int(tag.split("_")[2].split("x")[1])
        got = _C.unpack_codes(torch.from_numpy(golden[f"{tag}/packed"]).to(DEV), bits, k).cpu().numpy()
        assert np.array_equal(got, golden[f"{tag}/unpacked"]), tag


# ------------------------------------------------------------------ golden fixtures through the C ABI
TD = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
GOLD_TOL = {"float16": 2e-3, "bfloat16": 1.6e-2, "float32": 1e-4}


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def test_golden_gemv_and_gemm(golden):
    from crispybits_kernels import _C
    for tag in [c for c in golden["cases"].tolist() if c.startswith("lin_")]:
        _, wb, nk, g, dname = tag.split("_")
        bits, k, gs, dt = int(wb[1:]), int(nk.split("x")[1]), int(g[1:]), TD[dname]
        p, s, z = _t(golden[f"{tag}/packed"]), _t(golden[f"{tag}/scales"], dt), _t(golden[f"{tag}/zeros"], dt)
        bias = _t(golden[f"{tag}/bias"], dt) if f"{tag}/bias" in golden else torch.empty(0, device=DEV, dtype=dt)
        x, xm = _t(golden[f"{tag}/x"], dt), _t(golden[f"{tag}/xm"], dt)
        ws = torch.zeros(2, dtype=torch.int32, device=DEV)
        for split_k in (1, 3):
            for act in (0, 1, 2):
                y = _C.packed_gemv(x, p, s, z, bias, bits, k, gs, split_k, 1, act, ws)
                assert rel_err(y, _t(golden[f"{tag}/gemv_s{split_k}_a{act}"])) < GOLD_TOL[dname], (tag, split_k, act)
        for tc in (True, False):
            for act in (0, 2):
                y = _C.packed_gemm(xm, p, s, z, bias, bits, k, gs, act, tc)
                assert rel_err(y, _t(golden[f"{tag}/gemm_tc{int(tc)}_a{act}"])) < GOLD_TOL[dname], (tag, tc, act)
        assert ws.tolist() == [0, 0]


def test_golden_fused_ops(golden):
    from crispybits_kernels import _C
    h = torch.float16
    empty = torch.empty(0, device=DEV, dtype=h)
    ws = torch.zeros(2, dtype=torch.int32, device=DEV)
    for bits in (2, 3, 4):
        t = f"gu_w{bits}"
        g = [_t(golden[f"{t}/gate/packed"]), _t(golden[f"{t}/gate/scales"], h), _t(golden[f"{t}/gate/zeros"], h)]
        u = [_t(golden[f"{t}/up/packed"]), _t(golden[f"{t}/up/scales"], h), _t(golden[f"{t}/up/zeros"], h)]
        x = _t(golden[f"{t}/x"], h)
        for split_k in (1, 2):
            y = _C.fused_gate_up(x, *g, *u, bits, 256, 128, split_k, 1, ws)
            assert rel_err(y, _t(golden[f"{t}/out_s{split_k}"])) < 2e-3

        t, hd = f"qkv_w{bits}", 64
        x = _t(golden[f"{t}/x"], h)
        prj = {n: [_t(golden[f"{t}/{n}/packed"]), _t(golden[f"{t}/{n}/scales"], h), _t(golden[f"{t}/{n}/zeros"], h),
                   _t(golden[f"{t}/{n}/bias"], h)] for n in "qkv"}
        outs = _C.fused_qkv(x, *prj["q"], *prj["k"], *prj["v"], empty, empty, 0, 0, bits, 256, 128, 2, 1, ws)
        for n, o in zip("qkv", outs):
            assert rel_err(o, _t(golden[f"{t}/plain_{n}"])) < 2e-3, (t, n)
        for n in "qk":
            order = torch.from_numpy(golden[f"{t}/order_{n}"]).to(DEV)
            prj[n] = [a[order].contiguous() for a in prj[n]]
        outs = _C.fused_qkv(x, *prj["q"], *prj["k"], *prj["v"], _t(golden[f"{t}/cos"]), _t(golden[f"{t}/sin"]),
                            hd, hd, bits, 256, 128, 1, 1, ws)
        for n, o in zip("qkv", outs):
            assert rel_err(o, _t(golden[f"{t}/rope_{n}"])) < 2e-3, (t, n)


# ------------------------------------------------------------------ decode GEMV
SHAPES = [(128, 256), (300, 200), (4096, 4096), (1024, 5120), (5120, 1024), (33, 4128)]


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("B", [1, 3])
def test_gemv(bits, n, k, B):
    from crispybits_kernels import max_rho, packed_linear
    w, wd, _ = cached(n, k, bits, torch.float16)
    x = torch.randn(B, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(B))
    ref = ref_linear(x, wd)
    for split_k in (1, 2, 7, None):
        for rho in sorted({0, 1, max(1, max_rho(bits))}):
            close(packed_linear(x, w, split_k, rho), ref, torch.float16)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("B", [2, 4, 8, 11])
def test_gemv_batches_share_one_weight_pass(bits, B):
    from crispybits_kernels import packed_linear
    w, wd, bd = cached(1000, 1536, bits, torch.float16, True)
    x = torch.randn(B, 1536, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(7))
    for split_k in (1, 5, None):
        y = packed_linear(x, w, split_k, 1, decode_threshold=16)
        close(y, ref_linear(x, wd, bd), torch.float16)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("act", [None, "relu", "silu"])
@pytest.mark.parametrize("split_k", [1, 4])
def test_gemv_bias_act_dtypes(dtype, act, split_k):
    from crispybits_kernels import packed_linear
    w, wd, bd = cached(1000, 768, 3, dtype, True)
    x = torch.randn(2, 768, device=DEV, dtype=dtype)
    close(packed_linear(x, w, split_k, 2, act), ref_linear(x, wd, bd, act), dtype)


@pytest.mark.parametrize("gs", [32, 64, 256])
def test_group_sizes(gs):
    from crispybits_kernels import packed_linear
    w, wd, _ = cached(200, 640, 3, torch.float16, False, 0, gs)
    x = torch.randn(1, 640, device=DEV, dtype=torch.float16)
    close(packed_linear(x, w, 3, 1), ref_linear(x, wd), torch.float16)


def test_workspace_stays_zero_over_mixed_calls():
    from crispybits_kernels import new_workspace, packed_linear
    w, wd, _ = cached(5120, 1024, 3, torch.float16)
    x = torch.randn(1, 1024, device=DEV, dtype=torch.float16)
    ws = new_workspace(DEV)
    for pk, rho in [(1, 1), (4, 2), (1, 0), (7, 1), (1, 3)] * 3:
        y = packed_linear(x, w, pk, rho, workspace=ws)
        assert torch.isfinite(y).all()
        close(y, ref_linear(x, wd), torch.float16)
    torch.cuda.synchronize()
    assert ws.tolist() == [0, 0]


def test_split_k_scratch_counters_are_left_zero():
    from crispybits_kernels import _C, packed_linear
    w, wd, _ = cached(1024, 5120, 4, torch.float16)
    x = torch.randn(3, 5120, device=DEV, dtype=torch.float16)
    for pk in (2, 9, 160):
        close(packed_linear(x, w, pk, 1), ref_linear(x, wd), torch.float16)
    torch.cuda.synchronize()
    st = torch.cuda.current_stream().cuda_stream
    buf = _C._scratch[(torch.cuda.current_device(), st)]
    assert int(buf[: 65536 * 4].view(torch.int32).abs().sum()) == 0     # the fixed counter region


def test_results_do_not_depend_on_arrival_order():
    """The Split-K fix-up adds partial sums in split order: repeated calls are bit-identical."""
    from crispybits_kernels import packed_linear
    w, _, _ = cached(4096, 4096, 3, torch.float16)
    x = torch.randn(2, 4096, device=DEV, dtype=torch.float16)
    first = packed_linear(x, w, 6, 2)
    for _ in range(5):
        assert torch.equal(packed_linear(x, w, 6, 2), first)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("mode", ["gemv", "gate_up", "qkv_rope"])
def test_streamlined_kernel_agrees_with_generic_kernel(bits, mode):
    """Same call through both decode kernels (option 1 forces the generic one)."""
    from crispybits_kernels import _C, fused_gate_up, fused_qkv, packed_linear, permute_for_rope
    K = 2048
    x = torch.randn(3, K, device=DEV, dtype=torch.float16)

    def run():
        if mode == "gemv":
            w, _, _ = cached(1000, K, bits, torch.float16, True, 4)
            return [packed_linear(x, w, sk, 1, "silu") for sk in (1, 3)]
        if mode == "gate_up":
            g_, _, _ = cached(1376, K, bits, torch.float16, False, 1)
            u_, _, _ = cached(1376, K, bits, torch.float16, False, 2)
            return [fused_gate_up(x, g_, u_, sk, 1) for sk in (1, 2)]
        q, _, _ = cached(1024, K, bits, torch.float16, True, 1)
        k, _, _ = cached(256, K, bits, torch.float16, True, 2)
        v, _, _ = cached(256, K, bits, torch.float16, False, 3)
        q, k = permute_for_rope(q, 128), permute_for_rope(k, 128)
        cos, sin = rope_tables(3, 128, DEV)
        return [o for sk in (1, 4) for o in fused_qkv(x, q, k, v, sk, 1, rope=(cos, sin, 128))]

    outs = {}
    try:
        for which in (0, 1):           # option 5: operand form of the ring kernel (0 fp16 subnormals, 1 the 1024 offset)
            _C.set_option(5, which)
            outs[which] = run()
        _C.set_option(5, 0)
        _C.set_option(1, 1)
        slow = run()
    finally:
        _C.set_option(1, 0)
        _C.set_option(5, 0)
    for which in (0, 1):
        for a, b in zip(outs[which], slow):
            assert rel_err(a, b.float()) < 1e-3, which
    assert _C.decode_status() == 0


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("mode", ["gemv", "gate_up", "qkv_rope"])
def test_bf16_ring_kernel_agrees_with_generic_kernel(bits, mode):
    """bfloat16 decode through the ring kernel (bf16 MMA, 0x4300 magic-number unpack) against the generic fp32-FMA
    kernel on the same call and against the fp32 dequantise-then-matmul."""
    from crispybits_kernels import _C, fused_gate_up, fused_qkv, packed_linear, permute_for_rope
    K = 2048
    x = torch.randn(3, K, device=DEV, dtype=torch.bfloat16)

    def run():
        if mode == "gemv":
            w, _, _ = cached(1000, K, bits, torch.bfloat16, True, 4)
            return [packed_linear(x, w, sk, 1, "silu") for sk in (1, 3)]
        if mode == "gate_up":
            g_, _, _ = cached(1376, K, bits, torch.bfloat16, False, 1)
            u_, _, _ = cached(1376, K, bits, torch.bfloat16, False, 2)
            return [fused_gate_up(x, g_, u_, sk, 1) for sk in (1, 2)]
        q, _, _ = cached(1024, K, bits, torch.bfloat16, True, 1)
        k, _, _ = cached(256, K, bits, torch.bfloat16, True, 2)
        v, _, _ = cached(256, K, bits, torch.bfloat16, False, 3)
        q, k = permute_for_rope(q, 128), permute_for_rope(k, 128)
        cos, sin = rope_tables(3, 128, DEV)
        return [o for sk in (1, 4) for o in fused_qkv(x, q, k, v, sk, 1, rope=(cos, sin, 128))]

    fast = run()
    _C.set_option(1, 1)
    try:
        slow = run()
    finally:
        _C.set_option(1, 0)
    for a, b in zip(fast, slow):
        assert a.dtype == torch.bfloat16
        assert rel_err(a, b.float()) < 8e-3          # two bf16 output roundings apart at most
    if mode == "gemv":
        w, wd, bd = cached(1000, K, bits, torch.bfloat16, True, 4)
        close(fast[0], ref_linear(x, wd, bd, "silu"), torch.bfloat16)
    assert _C.decode_status() == 0


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("B", [1, 5, 8])
def test_ring_kernel_full_size_both_operand_forms(bits, B):
    """Ragged last slab, several passes per CTA, uneven K slices (K = 11008 is 86 groups over 8 warps), bias and SiLU,
    in both operand forms of the fp16 ring kernel (option 5): packed fields as fp16 subnormals, and fields OR-ed into
    1024.0 with the offset removed per group -- the error study of the second form at W2 and long K is this test."""
    from crispybits_kernels import _C, packed_linear
    w, wd, bd = cached(5000, 11008, bits, torch.float16, True, 21, 128, 0.02)
    x = torch.randn(B, 11008, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(B))
    try:
        for form in (0, 1):
            _C.set_option(5, form)
            close(packed_linear(x, w, None, 1, "silu", decode_threshold=8), ref_linear(x, wd, bd, "silu"), torch.float16)
    finally:
        _C.set_option(5, 0)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("B", [1, 3, 8])
@pytest.mark.parametrize("rho", [1, -1])
@pytest.mark.parametrize("n,k", [(20000, 4096), (2100, 11008)])
def test_ring_kernel_plans(bits, B, rho, n, k):
    """Both orders of the ring kernel's plan search at sizes with several passes per CTA: two CTAs per SM with a single
    32-row slot or 16-row passes (rho >= 0), one CTA per SM with a ring two to six slots deep (rho < 0); ragged last
    slab and last pass."""
    from crispybits_kernels import _C, packed_linear
    plan = _C.decode_plan(bits, B, n, k, 1, rho, _C.sm_count())
    assert plan is not None and (plan["passes"] >= 2 or k > 4096)
    w, wd, bd = cached(n, k, bits, torch.float16, True, 31, 128, 0.02)
    x = torch.randn(B, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(7 * B))
    close(packed_linear(x, w, 1, rho, decode_threshold=8), ref_linear(x, wd, bd), torch.float16)
    assert _C.decode_status() == 0


def test_remembered_weight_checks_follow_the_tensors():
    """The shim remembers weights that passed their checks by tensor identity.  Swapping a tensor's storage in place, or
    passing a bad tensor after good ones, must not be served from that memory."""
    from dataclasses import replace
    from crispybits_kernels import packed_linear
    w, wd, _ = cached(256, 512, 4, torch.float16, False, 77)
    x = torch.randn(1, 512, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(2))
    w = replace(w, scales=w.scales.clone())                       # own tensors: this test changes them
    y0 = packed_linear(x, w)
    close(y0, ref_linear(x, wd), torch.float16)
    assert torch.equal(packed_linear(x, w), y0)                   # second call: served from the remembered record
    w.scales.data = (w.scales * 2).contiguous()                   # same Python object, new storage
    close(packed_linear(x, w), 2 * ref_linear(x, wd), torch.float16)
    with pytest.raises(RuntimeError):
        packed_linear(x, replace(w, scales=w.scales.float()))     # metadata dtype must match x
    with pytest.raises(RuntimeError):
        packed_linear(x, replace(w, packed=w.packed[:, :-1].contiguous()))


def test_decode_status_word_is_clean_after_the_suite_so_far():
    from crispybits_kernels import _C
    assert _C.decode_status() == 0


# ------------------------------------------------------------------ prefill GEMM
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("M", [5, 33, 130])
@pytest.mark.parametrize("act", [None, "relu"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_prefill_gemm(bits, M, act, dtype):
    from crispybits_kernels import packed_linear
    w, wd, bd = cached(260, 400, bits, dtype, True)
    x = torch.randn(M, 400, device=DEV, dtype=dtype)
    tol = TOL[torch.bfloat16] if dtype == torch.bfloat16 else 3e-3   # reference bound for the rounded-weight path
    close(packed_linear(x, w, act=act), ref_linear(x, wd, bd, act), dtype, tol)
    close(packed_linear(x, w, act=act, use_tensor_cores=False), ref_linear(x, wd, bd, act), dtype,
          TOL[torch.bfloat16] if dtype == torch.bfloat16 else 2e-3)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("M,n,k", [(5, 256, 64), (130, 520, 1024), (300, 4096, 4096), (1024, 1000, 11008)])
def test_prefill_gemm_tensor_core_kernel(bits, M, n, k):
    """Shapes inside the tcgen05 kernel's domain (fp16, K a multiple of 64): parity with the
    rounded-weight arithmetic of the reference's tensor-core path, ragged M and N tiles, bias, SiLU."""
    from crispybits_kernels import _C, packed_linear
    w, wd, bd = cached(n, k, bits, torch.float16, True, 9, 128, 0.02)
    x = torch.randn(M, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(M))
    y = packed_linear(x, w, act="silu", decode_threshold=0)
    rounded = torch.nn.functional.silu(x.float() @ wd.half().float().T + bd)     # packed_gemm.cu:56,60
    assert rel_err(y, rounded) < 1e-3
    close(y, ref_linear(x, wd, bd, "silu"), torch.float16, 3e-3)                 # and the reference's bound vs fp32 weights
    _C.set_option(1, 1)
    try:
        slow = packed_linear(x, w, act="silu", decode_threshold=0)               # CUDA-core kernel, same numerics
    finally:
        _C.set_option(1, 0)
    assert rel_err(y, slow.float()) < 1e-3
    # both tcgen05 kernels on the same call: operands in shared memory (1), expanded weights in tensor memory (2)
    both = []
    try:
        for which in (1, 2):
            _C.set_option(3, which)
            both.append(packed_linear(x, w, act="silu", decode_threshold=0))
    finally:
        _C.set_option(3, 0)
    for o in both:
        assert rel_err(o, rounded) < 1e-3
    # same products, different summation order (inside the MMA; across K partitions when the call splits): the fp16
    # outputs may differ by one unit in the last place, which is at most 2^-10 of the largest output
    assert rel_err(both[0], both[1].float()) < 1e-3
    assert _C.decode_status() == 0


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("M,n,k,gs", [(129, 8, 128, 128), (257, 136, 256, 64), (513, 2048, 384, 128), (700, 264, 896, 64),
                                      (2049, 1032, 1152, 128)])
def test_prefill_gemm_edge_shapes_of_the_weight_stationary_kernel(bits, M, n, k, gs):
    """Just above 128 tokens, ragged token and weight-row tiles, two to eighteen pipeline stages (the rings wrap at
    six stages and four packed slots), group 64 (a scale change inside a packed super-block), several tiles per
    CTA at M = 2049: the weights-in-TMEM kernel against the rounded-weight product and against the CUDA-core kernel."""
    from crispybits_kernels import _C, packed_linear
    w, wd, bd = cached(n, k, bits, torch.float16, True, 11, gs, 0.02)
    x = torch.randn(M, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(M + k))
    _C.set_option(3, 2)
    try:
        y = packed_linear(x, w, act="relu", decode_threshold=0)
    finally:
        _C.set_option(3, 0)
    rounded = torch.relu(x.float() @ wd.half().float().T + bd)
    assert rel_err(y, rounded) < 1e-3
    _C.set_option(1, 1)
    try:
        slow = packed_linear(x, w, act="relu", decode_threshold=0)
    finally:
        _C.set_option(1, 0)
    assert rel_err(y, slow.float()) < 1e-3
    assert _C.decode_status() == 0


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("M,n,k,gs", [(5, 264, 256, 128), (130, 520, 1024, 64), (300, 4096, 4096, 128), (1024, 1000, 11008, 128)])
def test_prefill_gemm_bf16_tensor_core_kernel(bits, M, n, k, gs):
    """bfloat16 through the weights-in-TMEM kernel: the expanded weight is round_bf16((q - zero) * scale) as in the
    reference's tensor-core path (packed_gemm.cu:56,60), fp32 accumulation, bf16 output."""
    from crispybits_kernels import _C, packed_linear
    w, wd, bd = cached(n, k, bits, torch.bfloat16, True, 13, gs, 0.02)
    x = torch.randn(M, k, device=DEV, dtype=torch.bfloat16, generator=torch.Generator(DEV).manual_seed(M))
    y = packed_linear(x, w, act="silu", decode_threshold=0)
    assert y.dtype == torch.bfloat16
    rounded = torch.nn.functional.silu(x.float() @ wd.bfloat16().float().T + bd)
    assert rel_err(y, rounded) < 8e-3                        # one bf16 output rounding
    close(y, ref_linear(x, wd, bd, "silu"), torch.bfloat16)   # the reference's bf16 bound against fp32 weights
    _C.set_option(1, 1)
    try:
        slow = packed_linear(x, w, act="silu", decode_threshold=0)     # CUDA-core kernel, same rounded-weight numerics
    finally:
        _C.set_option(1, 0)
    assert rel_err(y, slow.float()) < 8e-3
    assert _C.decode_status() == 0


BENCH_PREFILL = [(1024, 4096, 4096), (1024, 12288, 4096), (1024, 22016, 4096), (1024, 4096, 11008),
                 (128, 4096, 4096), (512, 4096, 4096), (4096, 4096, 4096),
                 (128, 12288, 4096), (512, 22016, 4096), (4096, 4096, 11008)]


@pytest.mark.parametrize("bits", [3, 4])
@pytest.mark.parametrize("M,n,k", BENCH_PREFILL)
def test_prefill_gemm_at_the_benchmark_shapes(bits, M, n, k):
    """The prefill configuration's own (M, N, K): the tensor-core result against the fp32-accumulated product with the
    ORACLE's dequantised weight at the stated fp16 tolerance of 2e-3 (Crispybits/Kernel/tests/test_correctness.py:72-81
    with the tighter bound), against the CUDA-core kernel with the same rounded-weight numerics, and linearity in x
    (a size-independent property: f(2x) = 2 f(x) bit for bit, except where f(x) is an fp16 subnormal, whose rounding
    step does not scale -- hence the 2^-23 allowance)."""
    from crispybits_kernels import _C, packed_linear
    w, wd, _ = cached(n, k, bits, torch.float16, False, 17, 128, 0.02)
    x = (torch.randn(M, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(M)) * 0.25)
    y = packed_linear(x, w, decode_threshold=0)
    close(y, ref_linear(x, wd), torch.float16, 2e-3)
    twice = packed_linear(x * 2, w, decode_threshold=0)
    assert (twice.float() - 2 * y.float()).abs().max().item() <= 2.0 ** -23
    _C.set_option(1, 1)
    try:
        slow = packed_linear(x, w, decode_threshold=0)
    finally:
        _C.set_option(1, 0)
    assert rel_err(y, slow.float()) < 1e-3
    assert _C.decode_status() == 0


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("M,n,k,gs", [(64, 1024, 2048, 128), (130, 2048, 4096, 128), (300, 1024, 4096, 64), (512, 4096, 4096, 128),
                                      (257, 1032, 2048, 128)])
def test_prefill_gemm_k_split(bits, M, n, k, gs):
    """Few tokens against a narrow matrix: the weights-in-TMEM kernel splits K over otherwise idle SMs (fp32 partial
    sums in the stream's scratch, a second kernel adds them in order).  Against the oracle's dequantised weight at the
    fp16 tolerance, against the unsplit CUDA-core kernel, and bit for bit against itself on a second launch."""
    from crispybits_kernels import _C, packed_linear
    w, wd, bd = cached(n, k, bits, torch.float16, True, 23, gs, 0.02)
    x = torch.randn(M, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(M + n))
    assert _C._lib.cb_gemm_scratch_bytes(M, n, k) > 0, "this shape is meant to split"
    y = packed_linear(x, w, act="silu", decode_threshold=0)
    close(y, ref_linear(x, wd, bd, "silu"), torch.float16, 2e-3)
    assert torch.equal(packed_linear(x, w, act="silu", decode_threshold=0), y)
    _C.set_option(1, 1)
    try:
        slow = packed_linear(x, w, act="silu", decode_threshold=0)
    finally:
        _C.set_option(1, 0)
    assert rel_err(y, slow.float()) < 1e-3
    assert _C.decode_status() == 0


def test_prefill_gemm_k_split_is_skipped_without_scratch():
    """Straight through the C ABI: cb_packed_gemm (no scratch) and cb_packed_gemm_scratch agree within one rounding."""
    import ctypes
    from crispybits_kernels import _C
    M, n, k, bits = 256, 2048, 4096, 4
    w, wd, _ = cached(n, k, bits, torch.float16, False, 29, 128, 0.02)
    x = torch.randn(M, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(4))
    rec = _C._Weight(w.packed.data_ptr(), w.scales.data_ptr(), w.zeros.data_ptr(), 0, n)
    stream = torch.cuda.current_stream().cuda_stream
    a = torch.empty(M, n, device=DEV, dtype=torch.float16)
    b = torch.empty_like(a)
    lib = _C._lib
    assert lib.cb_packed_gemm(x.data_ptr(), M, ctypes.byref(rec), a.data_ptr(), k, bits, 128, 1, 0, 1, stream) == 0
    need = lib.cb_gemm_scratch_bytes(M, n, k)
    assert need == 4 * M * n * 4 or need == 2 * M * n * 4 or need == 8 * M * n * 4
    scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
    assert lib.cb_packed_gemm_scratch(x.data_ptr(), M, ctypes.byref(rec), b.data_ptr(), k, bits, 128, 1, 0, 1,
                                      scratch.data_ptr(), need, stream) == 0
    torch.cuda.synchronize()
    close(a, ref_linear(x, wd), torch.float16, 2e-3)
    close(b, ref_linear(x, wd), torch.float16, 2e-3)
    assert rel_err(a, b.float()) < 1e-3


@pytest.mark.parametrize("M,n,k", [(300, 4096, 4096), (1024, 1000, 11008)])
def test_prefill_gemm_is_stable_over_repeated_launches(M, n, k):
    """Shapes with fewer tiles than SMs, where the kernel's roles run at other relative speeds than in the large
    cases, launched 150 times: every launch reproduces the first one bit for bit and agrees with the CUDA-core
    kernel.  (An early version handed shared-memory slots back too soon and failed this in a few percent of runs.)"""
    from crispybits_kernels import _C, packed_linear
    w, _, _ = cached(n, k, 4, torch.float16, False, 9, 128, 0.02)
    x = torch.randn(M, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(7))
    _C.set_option(1, 1)
    try:
        slow = packed_linear(x, w, decode_threshold=0)
    finally:
        _C.set_option(1, 0)
    for which in (1, 2):
        _C.set_option(3, which)
        try:
            first = packed_linear(x, w, decode_threshold=0)
            assert rel_err(first, slow.float()) < 1e-3
            for _ in range(150):
                assert torch.equal(packed_linear(x, w, decode_threshold=0), first)
        finally:
            _C.set_option(3, 0)
    assert _C.decode_status() == 0


@pytest.mark.parametrize("bits", [2, 4])
def test_fused_prefill_kernels_are_stable_over_repeated_launches(bits):
    """The fused gate/up and Q/K/V forms of the prefill kernel, 100 launches each on a shape with several tiles per
    CTA and one with fewer tiles than SMs: every launch reproduces the first bit for bit."""
    from crispybits_kernels import fused_gate_up, fused_qkv, permute_for_rope
    for M, n, k in ((1024, 11008, 1024), (300, 1024, 2048)):
        g, _, _ = cached(n, k, bits, torch.float16, False, 1, 128, 0.02)
        u, _, _ = cached(n, k, bits, torch.float16, False, 2, 128, 0.02)
        x = torch.randn(M, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(3))
        first = fused_gate_up(x, g, u, decode_threshold=0)
        for _ in range(100):
            assert torch.equal(fused_gate_up(x, g, u, decode_threshold=0), first)
    from crispybits_kernels import _C
    for M, nq, nkv, k in ((1024, 32, 8, 1024), (300, 4, 2, 2048)):
        q, _, _ = cached(nq * 128, k, bits, torch.float16, True, 1, 128, 0.02)
        kk, _, _ = cached(nkv * 128, k, bits, torch.float16, True, 2, 128, 0.02)
        v, _, _ = cached(nkv * 128, k, bits, torch.float16, True, 3, 128, 0.02)
        q, kk = permute_for_rope(q, 128), permute_for_rope(kk, 128)
        x = torch.randn(M, k, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(4))
        rope = rope_tables(M, 128, DEV) + (128,)
        first = fused_qkv(x, q, kk, v, rope=rope, decode_threshold=0)
        for _ in range(100):
            again = fused_qkv(x, q, kk, v, rope=rope, decode_threshold=0)
            assert all(torch.equal(a, b) for a, b in zip(again, first))
    assert _C.decode_status() == 0


# ------------------------------------------------------------------ fused gate/up and QKV
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("B", [1, 4])
@pytest.mark.parametrize("split_k", [1, 3, None])
def test_fused_gate_up(bits, B, split_k):
    from crispybits_kernels import fused_gate_up
    g, gd, _ = cached(1376, 512, bits, torch.float16, False, 1)
    u, ud, _ = cached(1376, 512, bits, torch.float16, False, 2)
    x = torch.randn(B, 512, device=DEV, dtype=torch.float16)
    ref = torch.nn.functional.silu(x.float() @ gd.T) * (x.float() @ ud.T)
    close(fused_gate_up(x, g, u, split_k, 2), ref, torch.float16)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,n,k,gs", [(9, 384, 256, 128), (300, 1376, 4096, 128), (1024, 1000, 1152, 64)])
def test_fused_gate_up_prefill_kernel(bits, dtype, M, n, k, gs):
    """silu(x Wg^T) * (x Wu^T) for a prefill batch in ONE tcgen05 launch (gate and up rows interleaved as neighbouring
    tensor-memory lanes): against the fp32 reference and against the two-GEMM route it replaces; ragged 64-column
    tiles (n = 1376 = 21.5 tiles, n = 1000), group 64, fp16 and bf16."""
    from crispybits_kernels import _C, fused_gate_up
    g, gd, _ = cached(n, k, bits, dtype, False, 1, gs, 0.02)
    u, ud, _ = cached(n, k, bits, dtype, False, 2, gs, 0.02)
    x = torch.randn(M, k, device=DEV, dtype=dtype, generator=torch.Generator(DEV).manual_seed(M + n))
    direct = _C.fused_gate_up_gemm(x, g.packed, g.scales, g.zeros, u.packed, u.scales, u.zeros, bits, k, gs)
    assert direct is not None and direct.shape == (M, n) and direct.dtype == dtype     # the fused kernel took the call
    y = fused_gate_up(x, g, u, decode_threshold=0)
    assert torch.equal(y, direct)
    ref = torch.nn.functional.silu(x.float() @ gd.T) * (x.float() @ ud.T)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3                       # a product of two rounded-weight GEMMs
    assert rel_err(y, ref) < tol
    _C.set_option(1, 1)                                                   # CUDA-core kernels: two GEMMs and a product
    try:
        two = fused_gate_up(x, g, u, decode_threshold=0)
    finally:
        _C.set_option(1, 0)
    assert rel_err(y, two.float()) < (2e-2 if dtype == torch.bfloat16 else 3e-3)
    assert _C.decode_status() == 0


def test_fused_gate_up_prefill_route():
    from crispybits_kernels import fused_gate_up
    g, gd, _ = cached(384, 256, 4, torch.float16, False, 1)
    u, ud, _ = cached(384, 256, 4, torch.float16, False, 2)
    x = torch.randn(9, 256, device=DEV, dtype=torch.float16)
    ref = torch.nn.functional.silu(x.float() @ gd.T) * (x.float() @ ud.T)
    close(fused_gate_up(x, g, u), ref, torch.float16, 3e-3)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("B", [1, 3, 6])
@pytest.mark.parametrize("split_k", [1, 5])
@pytest.mark.parametrize("rope,head_dim", [(False, 0), (False, 128), (True, 128), (True, 64)])
@pytest.mark.parametrize("bias", [False, True])
def test_fused_qkv_gqa(bits, B, split_k, rope, head_dim, bias):
    from crispybits_kernels import apply_rope_reference, fused_qkv, permute_for_rope
    K, nq, nkv, hd = 1024, 8, 2, (head_dim or 128)
    q, qd, qb = cached(nq * hd, K, bits, torch.float16, bias, 1)
    k, kd, kb = cached(nkv * hd, K, bits, torch.float16, bias, 2)
    v, vd, vb = cached(nkv * hd, K, bits, torch.float16, bias, 3)
    if head_dim:
        q, k = permute_for_rope(q, head_dim), permute_for_rope(k, head_dim)
    x = torch.randn(B, K, device=DEV, dtype=torch.float16)
    rq, rk, rv = ref_linear(x, qd, qb), ref_linear(x, kd, kb), ref_linear(x, vd, vb)
    r = None
    if rope:
        cos, sin = rope_tables(B, head_dim, DEV)
        rq = apply_rope_reference(rq, cos, sin, head_dim)
        rk = apply_rope_reference(rk, cos, sin, head_dim)
        r = (cos, sin, head_dim)
    oq, ok, ov = fused_qkv(x, q, k, v, split_k, 2, rope=r)
    tol = 3e-3 if B > 4 else None      # B=6 routes to the prefill GEMM (rounded weights)
    close(oq, rq, torch.float16, tol); close(ok, rk, torch.float16, tol); close(ov, rv, torch.float16, tol)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,nq,nkv,head_dim,rope,bias", [
    (9, 256, 2, 1, 128, True, True),
    (300, 1024, 8, 2, 128, True, False),
    (300, 1024, 8, 2, 64, True, True),
    (700, 2048, 4, 4, 128, False, True),       # permuted, no rotation
    (64, 512, 3, 1, 0, False, False),          # natural order
])
def test_fused_qkv_prefill_kernel(bits, dtype, M, K, nq, nkv, head_dim, rope, bias):
    """Q, K, V of a prefill batch in ONE tcgen05 launch (bias, RoPE and the un-permuted store in the epilogue): against
    the fp32 reference and against the route it replaces (three GEMMs, a column gather, a separate rotation); GQA
    widths, head_dim 64 and 128, several token tiles, a ragged last token tile."""
    from crispybits_kernels import _C, apply_rope_reference, fused_qkv, permute_for_rope
    hd = head_dim or 128
    q, qd, qb = cached(nq * hd, K, bits, dtype, bias, 1, 128, 0.02)
    k, kd, kb = cached(nkv * hd, K, bits, dtype, bias, 2, 128, 0.02)
    v, vd, vb = cached(nkv * hd, K, bits, dtype, bias, 3, 128, 0.02)
    if head_dim:
        q, k = permute_for_rope(q, head_dim), permute_for_rope(k, head_dim)
    x = torch.randn(M, K, device=DEV, dtype=dtype, generator=torch.Generator(DEV).manual_seed(M + K))
    rq, rk, rv = ref_linear(x, qd, qb), ref_linear(x, kd, kb), ref_linear(x, vd, vb)
    r, cos, sin = None, None, None
    if rope:
        cos, sin = rope_tables(M, head_dim, DEV)
        rq = apply_rope_reference(rq, cos, sin, head_dim)
        rk = apply_rope_reference(rk, cos, sin, head_dim)
        r = (cos, sin, head_dim)
    e = torch.empty(0, device=DEV, dtype=dtype)
    direct = _C.fused_qkv_gemm(x, q.packed, q.scales, q.zeros, q.bias if bias else e,
                               k.packed, k.scales, k.zeros, k.bias if bias else e,
                               v.packed, v.scales, v.zeros, v.bias if bias else e,
                               cos, sin, head_dim if rope else 0, head_dim, bits, K, 128)
    assert direct is not None                                             # the fused kernel took the call
    got = fused_qkv(x, q, k, v, rope=r, decode_threshold=0)
    tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
    for y, d, ref in zip(got, direct, (rq, rk, rv)):
        assert y.dtype == dtype and torch.equal(y, d)
        assert rel_err(y, ref) < tol
    _C.set_option(1, 1)                                                   # CUDA-core kernels: the unfused route
    try:
        three = fused_qkv(x, q, k, v, rope=r, decode_threshold=0)
    finally:
        _C.set_option(1, 0)
    for y, t in zip(got, three):
        assert rel_err(y, t.float()) < tol
    assert _C.decode_status() == 0


def test_fused_qkv_prefill_outside_domain_falls_back():
    """A projection whose row count is not a multiple of 128 takes the three-GEMM route, with the same results."""
    from crispybits_kernels import _C, apply_rope_reference, fused_qkv, permute_for_rope
    K, hd = 512, 64
    q, qd, _ = cached(3 * hd, K, 4, torch.float16, False, 1)
    k, kd, _ = cached(hd, K, 4, torch.float16, False, 2)
    v, vd, _ = cached(hd, K, 4, torch.float16, False, 3)
    q, k = permute_for_rope(q, hd), permute_for_rope(k, hd)
    x = torch.randn(40, K, device=DEV, dtype=torch.float16)
    cos, sin = rope_tables(40, hd, DEV)
    e = torch.empty(0, device=DEV, dtype=torch.float16)
    assert _C.fused_qkv_gemm(x, q.packed, q.scales, q.zeros, e, k.packed, k.scales, k.zeros, e,
                             v.packed, v.scales, v.zeros, e, cos, sin, hd, hd, 4, K, 128) is None
    oq, ok, ov = fused_qkv(x, q, k, v, rope=(cos, sin, hd))
    close(oq, apply_rope_reference(ref_linear(x, qd, None), cos, sin, hd), torch.float16, 3e-3)
    close(ok, apply_rope_reference(ref_linear(x, kd, None), cos, sin, hd), torch.float16, 3e-3)
    close(ov, ref_linear(x, vd, None), torch.float16, 3e-3)


def test_prefill_kernels_on_seeded_random_shapes():
    """Plain, fused gate/up and fused Q/K/V forms of the prefill kernel on 16 seeded random problems: token counts
    around the 256-token tile edges, K from one super-block (128) up, head_dim 64 / 128, GQA widths, ragged gate/up
    widths, fp16 and bf16, with and without bias and rotation; each against the fp32 reference."""
    import random
    from crispybits_kernels import _C, apply_rope_reference, fused_gate_up, packed_linear, permute_for_rope
    rnd = random.Random(1)
    for _ in range(16):
        bits, dtype = rnd.choice([2, 3, 4]), rnd.choice([torch.float16, torch.bfloat16])
        K, M = 128 * rnd.randint(1, 12), rnd.choice([129, 130, 255, 256, 257, 300, 511, 513, 777, 1025])
        hd = rnd.choice([64, 128])
        nq, nkv = rnd.randint(1, 6) * (128 // hd), rnd.randint(1, 3) * (128 // hd)
        bias, rope = rnd.random() < 0.5, rnd.random() < 0.7
        tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
        tag = (bits, dtype, M, K, hd, nq, nkv, bias, rope)
        q, qd, qb = make(nq * hd, K, bits, dtype, DEV, bias, 1, 128, 0.02)
        k, kd, kb = make(nkv * hd, K, bits, dtype, DEV, bias, 2, 128, 0.02)
        v, vd, vb = make(nkv * hd, K, bits, dtype, DEV, bias, 3, 128, 0.02)
        q, k = permute_for_rope(q, hd), permute_for_rope(k, hd)
        x = torch.randn(M, K, device=DEV, dtype=dtype, generator=torch.Generator(DEV).manual_seed(M + K))
        refs = [ref_linear(x, qd, qb), ref_linear(x, kd, kb), ref_linear(x, vd, vb)]
        cos = sin = None
        if rope:
            cos, sin = rope_tables(M, hd, DEV)
            refs[0], refs[1] = apply_rope_reference(refs[0], cos, sin, hd), apply_rope_reference(refs[1], cos, sin, hd)
        e = torch.empty(0, device=DEV, dtype=dtype)
        outs = _C.fused_qkv_gemm(x, q.packed, q.scales, q.zeros, q.bias if bias else e,
                                 k.packed, k.scales, k.zeros, k.bias if bias else e,
                                 v.packed, v.scales, v.zeros, v.bias if bias else e,
                                 cos, sin, hd if rope else 0, hd, bits, K, 128)
        assert outs is not None, tag
        for o, r in zip(outs, refs):
            assert rel_err(o, r) < tol, tag
        n = rnd.choice([64, 100, 1000, 1376, 2048])
        g, gd, _ = make(n, K, bits, dtype, DEV, False, 4, 128, 0.02)
        u, ud, _ = make(n, K, bits, dtype, DEV, False, 5, 128, 0.02)
        ref = torch.nn.functional.silu(x.float() @ gd.T) * (x.float() @ ud.T)
        assert rel_err(fused_gate_up(x, g, u, decode_threshold=0), ref) < (2e-2 if dtype == torch.bfloat16 else 4e-3), tag
        w, wd, wb = make(n - n % 8, K, bits, dtype, DEV, True, 6, 128, 0.02)
        assert rel_err(packed_linear(x, w, act="silu", decode_threshold=0), ref_linear(x, wd, wb, "silu")) < tol, tag
    assert _C.decode_status() == 0


# ------------------------------------------------------------------ error behaviour
def test_argument_errors():
    import crispybits_kernels as ck
    from crispybits_kernels import _C
    w, _, _ = cached(256, 256, 3, torch.float16)
    x = torch.randn(1, 256, device=DEV, dtype=torch.float16)
    cos, sin = rope_tables(1, 128, DEV)
    with pytest.raises(ValueError):
        ck.fused_qkv(x, w, w, w, rope=(cos, sin, 128))
    with pytest.raises(ValueError):
        ck.packed_linear(x, ck.permute_for_rope(w, 128))
    e = torch.empty(0, device=DEV, dtype=torch.float16)
    ws = torch.zeros(2, dtype=torch.int32, device=DEV)
    bad = [
        lambda: _C.packed_gemv(x.cpu(), w.packed, w.scales, w.zeros, e, 3, 256, 128, 1, 1, 0, ws),     # CPU x
        lambda: _C.packed_gemv(x, w.packed, w.scales, w.zeros, e, 5, 256, 128, 1, 1, 0, ws),           # bits
        lambda: _C.packed_gemv(x, w.packed, w.scales, w.zeros, e, 3, 256, 48, 1, 1, 0, ws),            # group size
        lambda: _C.packed_gemv(x, w.packed, w.scales, w.zeros, e, 3, 256, 128, 0, 1, 0, ws),           # split_k
        lambda: _C.packed_gemv(x, w.packed, w.scales, w.zeros, e, 3, 256, 128, 1, 1, 3, ws),           # act
        lambda: _C.packed_gemv(x, w.packed, w.scales.float(), w.zeros.float(), e, 3, 256, 128, 1, 1, 0, ws),
        lambda: _C.packed_gemv(x, w.packed[:, :-1].contiguous(), w.scales, w.zeros, e, 3, 256, 128, 1, 1, 0, ws),
        lambda: _C.packed_gemv(x, w.packed, w.scales, w.zeros, e[:0].new_zeros(7), 3, 256, 128, 1, 1, 0, ws),
        lambda: _C.packed_gemm(x[:, :100].contiguous(), w.packed, w.scales, w.zeros, e, 3, 256, 128, 0, True),
        lambda: _C.fused_qkv(x, w.packed, w.scales, w.zeros, e, w.packed, w.scales, w.zeros, e, w.packed, w.scales,
                             w.zeros, e, cos, sin, 128, 0, 3, 256, 128, 1, 1, ws),                      # rope w/o perm
        lambda: _C.fused_qkv_gemm(x, w.packed, w.scales, w.zeros, e, w.packed, w.scales, w.zeros, e, w.packed, w.scales,
                                  w.zeros, e, cos, sin, 128, 0, 3, 256, 128),                           # rope w/o perm
        lambda: _C.fused_qkv_gemm(x, w.packed, w.scales, w.zeros, e, w.packed, w.scales, w.zeros, e, w.packed, w.scales,
                                  w.zeros, e, cos[:, :64], sin, 128, 128, 3, 256, 128),                 # cos/sin shapes
        lambda: _C.fused_qkv_gemm(x, w.packed, w.scales, w.zeros, e, w.packed, w.scales, w.zeros, e, w.packed, w.scales,
                                  w.zeros, e, None, None, 0, 6, 3, 256, 128),                           # rows not a multiple of head_dim
        lambda: _C.fused_gate_up_gemm(x, w.packed, w.scales, w.zeros, w.packed[:128], w.scales[:128], w.zeros[:128],
                                      3, 256, 128),                                                     # gate/up shapes
    ]
    for call in bad:
        with pytest.raises(RuntimeError):
            call()
    assert _C.packed_gemv(x[:0], w.packed, w.scales, w.zeros, e, 3, 256, 128, 1, 1, 0, ws).shape == (0, 256)


def test_c_abi_reports_errors_by_code():
    """Straight ctypes call, no Python-side checks in between."""
    import ctypes
    from crispybits_kernels import _C
    w, _, _ = cached(256, 256, 3, torch.float16)
    x = torch.randn(1, 256, device=DEV, dtype=torch.float16)
    out = torch.empty(1, 256, device=DEV, dtype=torch.float16)
    rec = _C._Weight(w.packed.data_ptr(), w.scales.data_ptr(), w.zeros.data_ptr(), 0, 256)
    rc = _C._lib.cb_packed_gemv(x.data_ptr(), 1, ctypes.byref(rec), out.data_ptr(), 256, 7, 128, 1, 1, 1, 0, 0, 0, 0)
    assert rc == 1 and b"bits" in _C._lib.cb_last_error()
    rc = _C._lib.cb_packed_gemv(x.data_ptr(), 1, ctypes.byref(rec), out.data_ptr(), 256, 3, 128, 1, 4, 1, 0, 0, 0, 0)
    assert rc == 1 and b"scratch" in _C._lib.cb_last_error()
    rc = _C._lib.cb_packed_gemv(x.data_ptr(), 1, ctypes.byref(rec), out.data_ptr(), 256, 3, 128, 1, 1, 1, 0, 0, 0,
                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()


# ------------------------------------------------------------------ streams and graphs
def test_non_default_stream():
    from crispybits_kernels import packed_linear
    w, wd, _ = cached(512, 512, 3, torch.float16)
    x = torch.randn(1, 512, device=DEV, dtype=torch.float16)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        y = packed_linear(x, w, 3, 1)
    s.synchronize()
    close(y, ref_linear(x, wd), torch.float16)


@pytest.mark.parametrize("split_k", [1, 4])
def test_cuda_graph_capture(split_k):
    from crispybits_kernels import new_workspace, packed_linear
    w, wd, _ = cached(4096, 4096, 3, torch.float16)
    x = torch.randn(1, 4096, device=DEV, dtype=torch.float16)
    ws = new_workspace(DEV)
    packed_linear(x, w, split_k, 1, workspace=ws)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = packed_linear(x, w, split_k, 1, workspace=ws)
    for _ in range(3):
        x.copy_(torch.randn_like(x)); g.replay(); torch.cuda.synchronize()
        close(y, ref_linear(x, wd), torch.float16)


# ------------------------------------------------------------------ full benchmark sizes: properties
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008)])
def test_full_size_properties(bits, n, k):
    """At the benchmark's sizes (weights ~ N(0, 0.02)): parity for batch 1..8, exact unpack of the whole
    matrix, and linearity y(a + b) = y(a) + y(b) up to output rounding."""
    from crispybits_kernels import _C, packed_linear
    w, wd, _ = cached(n, k, bits, torch.float16, False, 0, 128, 0.02)
    codes = _C.unpack_codes(w.packed, bits, k)
    assert np.array_equal(codes.cpu().numpy(), O.unpack_codes(w.packed.cpu().numpy(), bits, k))
    gen = torch.Generator(DEV).manual_seed(n + k + bits)
    for B in (1, 2, 4, 8):
        x = torch.randn(B, k, device=DEV, dtype=torch.float16, generator=gen)
        close(packed_linear(x, w, None, 1, decode_threshold=8), ref_linear(x, wd), torch.float16)
    a = torch.randn(1, k, device=DEV, dtype=torch.float16, generator=gen)
    b = torch.randn(1, k, device=DEV, dtype=torch.float16, generator=gen)
    lhs = packed_linear((a.float() + b.float()).half(), w).float()
    rhs = packed_linear(a, w).float() + packed_linear(b, w).float()
    assert rel_err(lhs, rhs) < 4e-3


@pytest.mark.parametrize("bits", [3, 4])
def test_config3_fused_equals_concatenated(bits):
    """Fused QKV / gate-up at Llama-2-7B widths against one GEMV over the row-concatenated matrix."""
    from crispybits_kernels import PackedLinearWeight, fused_gate_up, fused_qkv, packed_linear
    K = 4096
    ws = [cached(4096, K, bits, torch.float16, False, s, 128, 0.02)[0] for s in (1, 2, 3)]
    x = torch.randn(1, K, device=DEV, dtype=torch.float16)
    cat = PackedLinearWeight(torch.cat([w.packed for w in ws]), torch.cat([w.scales for w in ws]),
                             torch.cat([w.zeros for w in ws]), bits, 128, K, 3 * 4096)
    y = packed_linear(x, cat)
    for i, o in enumerate(fused_qkv(x, *ws)):
        assert rel_err(o, y[:, i * 4096:(i + 1) * 4096].float()) < 1e-3
    g, gd, _ = cached(11008, K, bits, torch.float16, False, 5, 128, 0.02)
    u, ud, _ = cached(11008, K, bits, torch.float16, False, 6, 128, 0.02)
    ref = torch.nn.functional.silu(x.float() @ gd.T) * (x.float() @ ud.T)
    close(fused_gate_up(x, g, u), ref, torch.float16)
