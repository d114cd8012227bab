"""Input factories and comparison helpers shared by the test modules.

Inputs follow the reference's tests (Crispybits/Kernel/tests/test_correctness.py:13-37): seeded CPU
generator, W ~ N(0,1)*std, optional bias ~ N(0,1)*0.1, quantised group-wise by the oracle, and the
check value is the fp32 product with the dequantised weight; the metric is max|y-ref| / max|ref|.
"""
import numpy as np
import torch

from oracle import cb_oracle as O

NAME = {torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float32: "float32"}
# north_star tolerance for fp16: 2e-3 max relative error against an fp32-accumulated
# dequant-then-matmul; bf16 / fp32 keep the reference's own bounds (test_correctness.py:10)
TOL = {torch.float16: 2e-3, torch.bfloat16: 2e-2, torch.float32: 1e-4}


def make_dict(n, k, bits, dtype=torch.float16, bias=False, seed=0, gs=128, std=0.05):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * std
    b = torch.randn(n, generator=g) * 0.1 if bias else None
    d = O.pack_linear_dict(w.numpy(), bits, gs, None if b is None else b.numpy(), NAME[dtype])
    return d


def to_weight(d, device, dtype):
    from crispybits_kernels.io import from_packed_dict
    td = dict(d)
    for key in ("packed", "scales", "zeros", "bias"):
        td[key] = None if d[key] is None else torch.from_numpy(d[key])
    return from_packed_dict(td, device, dtype)


def make(n, k, bits, dtype, device, bias=False, seed=0, gs=128, std=0.05):
    """(PackedLinearWeight on device, dequantised fp32 weight on device, fp32 bias or None)."""
    d = make_dict(n, k, bits, dtype, bias, seed, gs, std)
    wd = torch.from_numpy(O.dequantized_weight(d)).to(device)
    bd = None if d["bias"] is None else torch.from_numpy(d["bias"]).float().to(device)
    return to_weight(d, device, dtype), wd, bd


def ref_linear(x, wd, bd=None, act=None):
    y = x.float() @ wd.T
    if bd is not None:
        y = y + bd
    if act == "relu":
        y = torch.relu(y)
    elif act == "silu":
        y = torch.nn.functional.silu(y)
    return y


def rel_err(y, ref):
    return ((y.float() - ref).abs().max() / (ref.abs().max() + 1e-6)).item()


def close(y, ref, dtype, tol=None):
    e = rel_err(y, ref)
    assert e < (tol if tol is not None else TOL[dtype]), f"rel err {e:.2e}"


def rope_tables(m, head_dim, device, seed=0):
    g = torch.Generator().manual_seed(seed)
    pos = torch.randint(0, 2048, (m,), generator=g).float()
    inv = 1.0 / (10000 ** (torch.arange(0, head_dim, 2).float() / head_dim))
    f = pos[:, None] * inv[None]
    emb = torch.cat([f, f], -1)
    return emb.cos().to(device), emb.sin().to(device)
