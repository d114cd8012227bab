"""Host-side logic of the package on CPU: routing, policy, permutation helpers, error types.

`ops._C` is pointed at the oracle-backed stand-in (tests/oracle_backend.py), the way the reference's
suite runs against its emulator (Crispybits/Kernel/tests/conftest.py).  Numerics here are the oracle's;
what is being tested is everything in ops.py around the binding calls.
"""
import pytest
import torch

import oracle_backend
from helpers import close, make, ref_linear, rope_tables

import crispybits_kernels as ck
from crispybits_kernels import ops


@pytest.fixture(autouse=True)
def oracle_env():
    prev = ops._C
    ops.set_backend(oracle_backend)
    ops._sm_count_for.cache_clear()
    yield "cpu"
    ops.set_backend(prev if prev is not None else "cuda")
    ops._sm_count_for.cache_clear()


def test_backend_switch():
    assert ops.backend_name() == "emulator"
    ops.set_backend("cuda")
    assert ops.backend_name() == "cuda" and ops._C is ops._CUDA
    with pytest.raises(RuntimeError):
        ops.set_backend("emulator")
    with pytest.raises(ValueError):
        ops.set_backend("rocm")
    ops.set_backend(oracle_backend)


def test_cuda_shim_refuses_cpu_tensors():
    if ops._CUDA is None:
        pytest.skip("library not built")
    w, _, _ = make(64, 128, 3, torch.float16, "cpu")
    x = torch.randn(1, 128).half()
    e = torch.empty(0, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        ops._CUDA.packed_gemv(x, w.packed, w.scales, w.zeros, e, 3, 128, 128, 1, 1, 0, torch.zeros(2, dtype=torch.int32))


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("n,k", [(128, 256), (300, 200), (33, 1056)])
@pytest.mark.parametrize("B", [1, 3])
@pytest.mark.parametrize("split_k", [1, 2, 7, None])
def test_gemv_routing(bits, n, k, B, split_k):
    w, wd, _ = make(n, k, bits, torch.float16, "cpu")
    x = torch.randn(B, k).half()
    for rho in (0, 1, 2):
        close(ck.packed_linear(x, w, split_k, rho), ref_linear(x, wd), torch.float16)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("act", [None, "relu", "silu"])
def test_bias_act_dtypes(dtype, act):
    w, wd, bd = make(100, 160, 3, dtype, "cpu", bias=True)
    x = torch.randn(2, 160).to(dtype)
    close(ck.packed_linear(x, w, 4, 2, act), ref_linear(x, wd, bd, act), dtype)


def test_leading_dims_and_threshold_routing(monkeypatch):
    w, wd, _ = make(64, 96, 4, torch.float16, "cpu")
    calls = []
    monkeypatch.setattr(oracle_backend, "packed_gemv", lambda *a: (calls.append("gemv"), _orig_gemv(*a))[1])
    monkeypatch.setattr(oracle_backend, "packed_gemm", lambda *a: (calls.append("gemm"), _orig_gemm(*a))[1])
    x = torch.randn(2, 2, 96).half()
    y = ck.packed_linear(x, w)
    assert y.shape == (2, 2, 64) and calls == ["gemv"]
    ck.packed_linear(torch.randn(5, 96).half(), w)
    ck.packed_linear(torch.randn(8, 96).half(), w, decode_threshold=8)
    assert calls == ["gemv", "gemm", "gemv"]
    close(y.reshape(4, 64), ref_linear(x.reshape(4, 96), wd), torch.float16)


_orig_gemv, _orig_gemm = oracle_backend.packed_gemv, oracle_backend.packed_gemm


@pytest.mark.parametrize("B", [1, 4, 9])
def test_fused_gate_up(B):
    g, gd, _ = make(96, 128, 3, torch.float16, "cpu", seed=1)
    u, ud, _ = make(96, 128, 3, torch.float16, "cpu", seed=2)
    x = torch.randn(B, 128).half()
    ref = torch.nn.functional.silu(x.float() @ gd.T) * (x.float() @ ud.T)
    close(ck.fused_gate_up(x, g, u, 2, 1), ref, torch.float16, 3e-3)
    g4, _, _ = make(96, 128, 4, torch.float16, "cpu", seed=1)
    with pytest.raises(ValueError):
        ck.fused_gate_up(x, g4, u)


@pytest.mark.parametrize("B", [1, 3, 6])
@pytest.mark.parametrize("rope,head_dim", [(False, 0), (False, 64), (True, 64)])
@pytest.mark.parametrize("bias", [False, True])
def test_fused_qkv(B, rope, head_dim, bias):
    K, hd = 128, (head_dim or 64)
    q, qd, qb = make(4 * hd, K, 3, torch.float16, "cpu", bias, 1)
    k, kd, kb = make(2 * hd, K, 3, torch.float16, "cpu", bias, 2)
    v, vd, vb = make(2 * hd, K, 3, torch.float16, "cpu", bias, 3)
    if head_dim:
        q, k = ck.permute_for_rope(q, head_dim), ck.permute_for_rope(k, head_dim)
    x = torch.randn(B, K).half()
    rq, rk, rv = ref_linear(x, qd, qb), ref_linear(x, kd, kb), ref_linear(x, vd, vb)
    r = None
    if rope:
        cos, sin = rope_tables(B, head_dim, "cpu")
        rq, rk = ck.apply_rope_reference(rq, cos, sin, head_dim), ck.apply_rope_reference(rk, cos, sin, head_dim)
        r = (cos, sin, head_dim)
    oq, ok, ov = ck.fused_qkv(x, q, k, v, 3, 2, rope=r)
    for o, ref in ((oq, rq), (ok, rk), (ov, rv)):
        close(o, ref, torch.float16, 3e-3)


def test_value_errors():
    q, _, _ = make(128, 128, 3, torch.float16, "cpu")
    x = torch.randn(1, 128).half()
    cos, sin = rope_tables(1, 64, "cpu")
    with pytest.raises(ValueError):
        ck.fused_qkv(x, q, q, q, rope=(cos, sin, 64))
    with pytest.raises(ValueError):
        ck.packed_linear(x, ck.permute_for_rope(q, 64))
    with pytest.raises(ValueError):
        ck.permute_for_rope(ck.permute_for_rope(q, 64), 32)
    with pytest.raises(ValueError):
        ck.fused_qkv(x, ck.permute_for_rope(q, 64), q, q)
    with pytest.raises(ValueError):
        ops.rope_row_order(100, 64)
    with pytest.raises(ValueError):
        ck.virtual_rows("conv", 3)
    with pytest.raises(RuntimeError):
        ck.max_rho(3, "nope")


@pytest.mark.parametrize("hd", [64, 128])
def test_row_permutation_helpers(hd):
    from oracle import cb_oracle as O
    n = 4 * hd
    order = ops.rope_row_order(n, hd)
    assert order.tolist() == O.unperm_index(n, hd).tolist()       # the kernel's un-permute is the host order
    inv = ops.rope_inverse_order(n, hd)
    assert torch.equal(order[inv], torch.arange(n))
    for p in range(0, n, 2):                                      # stored neighbours are RoPE partners
        a, b = int(order[p]), int(order[p + 1])
        assert b - a == hd // 2 and a // hd == b // hd


def test_policy_rules():
    s, bn = ck.sm_count(), ck.tile_n()
    assert ck.candidate_split_k(1, bn * 4, bn, s, 1) == max(1, -(-s // 4))
    assert ck.candidate_split_k(64, 4096, bn, s, 1) == 1
    assert ck.candidate_split_k(1, 10 ** 6, bn, s, 1) == 1
    assert ck.candidate_split_k(1, bn * 4, bn, s, 1, max_split=8) == 8
    assert ck.virtual_rows("qkv", 4096, 1024, 1024) == 6144 and ck.virtual_rows("gate_up", 11008) == 22016
    # balanced rule: never below the underfill answer, never starves a split of chunks
    for n, k in ((4096, 4096), (11008, 4096), (4096, 11008), (512, 4096), (12288, 4096), (22016, 4096)):
        for b in (1, 4, 8, 16):
            nch = -(-k // 32)
            p = ck.balanced_split_k(b, n, 16, 148, 1, nch)
            base = ck.candidate_split_k(-(-b // 8), n, 16, 148, 1)
            assert base <= p <= max(base, 32) and p <= nch
            units = -(-b // 8) * -(-n // 16) * p
            eff = units / (-(-units // 148) * 148)
            assert eff >= 0.85 or p == base, (n, k, b, p, eff)
    assert ops._resolve(1000, 1, 1, 4096, 4096, torch.device("cpu")) == 128     # clamped to the chunk count
    assert ops._resolve(None, 1, 1, 4096, 4096, torch.device("cpu")) >= 1


def test_packed_linear_module_and_io(tmp_path):
    from oracle import cb_oracle as O
    from crispybits_kernels.io import from_packed_dict
    w, wd, bd = make(48, 64, 4, torch.float32, "cpu", bias=True)
    m = ck.PackedLinear(w, split_k=2, rho=1, act="relu")
    x = torch.randn(3, 64)
    close(m(x), ref_linear(x, wd, bd, "relu"), torch.float32)
    assert m.workspace.tolist() == [0, 0] and "W4" in m.extra_repr()
    assert set(dict(m.named_buffers())) >= {"packed", "scales", "zeros", "bias"}
    m.permute_for_rope_(16)
    assert m.rope_perm_head_dim == 16 and m.weight_spec().rope_perm_head_dim == 16
    # the on-disk dict layout of the reference (reference.py:70-76) round-trips through torch.save
    d = O.pack_linear_dict(torch.randn(8, 64).numpy(), 3, 32, None, "float16")
    td = {k: (torch.from_numpy(v) if hasattr(v, "dtype") else v) for k, v in d.items() if k != "dtype"}
    torch.save({"proj": td}, tmp_path / "block_000_w3.pt")
    back = torch.load(tmp_path / "block_000_w3.pt", weights_only=False)["proj"]
    pw = from_packed_dict(back, "cpu", torch.float16)
    assert pw.bits == 3 and pw.group_size == 32 and pw.packed.dtype == torch.int32 and pw.scales.dtype == torch.float16
