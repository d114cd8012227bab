#!/usr/bin/env python3
"""Generate the golden fixtures in this directory from the reference's own Python code.

Run on a machine that holds the reference tree (it is imported, never copied):

    python tests/golden/make_golden.py path/to/reference/Crispybits/Kernel

The script imports the reference's ``crispybits_kernels.reference`` (quantizer,
bitstream) and ``crispybits_kernels.emulator`` (decode / prefill arithmetic),
feeds them seeded inputs, and stores inputs and outputs as float32/int32 numpy
arrays in ``golden_v1.npz``.  The fixtures travel with the repository; the
reference does not.  ``tests/test_oracle_golden.py`` replays them through the
numpy oracle and the C oracle, ``tests/test_gpu_parity.py`` through the CUDA kernels.
"""
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py <path to the reference's Crispybits/Kernel directory>")
REF = sys.argv[1]
sys.dont_write_bytecode = True
sys.path.insert(0, REF)
from crispybits_kernels import emulator as E  # noqa: E402
from crispybits_kernels import reference as R  # noqa: E402
from crispybits_kernels.ops import apply_rope_reference, rope_row_order  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_v1.npz")
TD = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
store = {}


def f32(t):
    return t.detach().float().cpu().numpy().astype(np.float32)


def put(name, t):
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().numpy() if t.dtype in (torch.int32, torch.int64) else f32(t)
    store[name] = np.ascontiguousarray(t)


def make(tag, n, k, bits, gs, dtype, seed, bias=False, std=0.02):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * std
    b = torch.randn(n, generator=g) * 0.1 if bias else None
    q, s, z = R.quantize_affine(w, bits, gs)
    d = R.pack_linear_dict(w, bits, gs, b, TD[dtype])
    put(f"{tag}/w", w); put(f"{tag}/q", q); put(f"{tag}/scale32", s); put(f"{tag}/zero32", z)
    put(f"{tag}/packed", d["packed"]); put(f"{tag}/scales", d["scales"]); put(f"{tag}/zeros", d["zeros"])
    if bias:
        put(f"{tag}/bias", d["bias"])
    put(f"{tag}/unpacked", R.unpack_codes(d["packed"], bits, k))
    put(f"{tag}/wdq", R.dequantized_weight(d))
    return d, g


def ws():
    return torch.zeros(2, dtype=torch.int32)


cases = []
# ---- quantizer / bitstream / GEMV / GEMM, per bit-width, aligned and ragged K, three dtypes
for bits in (2, 3, 4):
    for (n, k, gs, dtype, bias) in ((24, 256, 128, "float16", True), (19, 200, 128, "float16", False),
                                    (16, 640, 64, "bfloat16", True), (20, 416, 32, "float32", True)):
        tag = f"lin_w{bits}_{n}x{k}_g{gs}_{dtype}"
        d, g = make(tag, n, k, bits, gs, dtype, seed=100 * bits + n, bias=bias)
        t = TD[dtype]
        x = torch.randn(3, k, generator=g).to(t)
        put(f"{tag}/x", x)
        sc, ze = d["scales"], d["zeros"]
        bi = d["bias"] if bias else torch.empty(0, dtype=t)
        for split_k in (1, 3):
            for act in (0, 1, 2):
                y = E.packed_gemv(x, d["packed"], sc, ze, bi, bits, k, gs, split_k, 1, act, ws())
                put(f"{tag}/gemv_s{split_k}_a{act}", y)
        xm = torch.randn(9, k, generator=g).to(t)
        put(f"{tag}/xm", xm)
        for tc in (True, False):
            for act in (0, 2):
                y = E.packed_gemm(xm, d["packed"], sc, ze, bi, bits, k, gs, act, tc)
                put(f"{tag}/gemm_tc{int(tc)}_a{act}", y)
        cases.append(tag)

# ---- fused gate-up and fused QKV (GQA widths, bias, permutation, RoPE), fp16
for bits in (2, 3, 4):
    tag = f"gu_w{bits}"
    dg, g = make(tag + "/gate", 48, 256, bits, 128, "float16", seed=700 + bits)
    du, _ = make(tag + "/up", 48, 256, bits, 128, "float16", seed=800 + bits)
    x = torch.randn(2, 256, generator=g).half()
    put(f"{tag}/x", x)
    for split_k in (1, 2):
        y = E.fused_gate_up(x, dg["packed"], dg["scales"], dg["zeros"], du["packed"], du["scales"], du["zeros"],
                            bits, 256, 128, split_k, 1, ws())
        put(f"{tag}/out_s{split_k}", y)
    cases.append(tag)

    hd, nq, nkv, k = 64, 2, 1, 256
    tag = f"qkv_w{bits}"
    ds = []
    for nm, n, seed in (("q", nq * hd, 1), ("k", nkv * hd, 2), ("v", nkv * hd, 3)):
        d, g = make(f"{tag}/{nm}", n, k, bits, 128, "float16", seed=900 + 10 * bits + seed, bias=True)
        ds.append(d)
    x = torch.randn(3, k, generator=g).half()
    put(f"{tag}/x", x)
    pos = torch.tensor([0.0, 5.0, 1234.0])
    inv = 1.0 / (10000 ** (torch.arange(0, hd, 2).float() / hd))
    emb = torch.cat([pos[:, None] * inv[None]] * 2, -1)
    cos, sin = emb.cos(), emb.sin()
    put(f"{tag}/cos", cos); put(f"{tag}/sin", sin)
    # (a) unpermuted, no rope
    a = [(d["packed"], d["scales"], d["zeros"], d["bias"]) for d in ds]
    outs = E.fused_qkv(x, *a[0], *a[1], *a[2], torch.empty(0), torch.empty(0), 0, 0, bits, k, 128, 2, 1, ws())
    for nm, o in zip("qkv", outs):
        put(f"{tag}/plain_{nm}", o)
    # (b) Q/K stored pair-interleaved, RoPE fused
    perm = []
    for i, d in enumerate(ds):
        if i < 2:
            o = rope_row_order(d["out_features"], hd)
            perm.append((d["packed"][o].contiguous(), d["scales"][o].contiguous(), d["zeros"][o].contiguous(),
                         d["bias"][o].contiguous()))
            put(f"{tag}/order_{'qk'[i]}", o)
        else:
            perm.append(a[i])
    outs = E.fused_qkv(x, *perm[0], *perm[1], *perm[2], cos, sin, hd, hd, bits, k, 128, 1, 1, ws())
    for nm, o in zip("qkv", outs):
        put(f"{tag}/rope_{nm}", o)
    # the rotate_half formulation on the un-fused outputs, as the reference's tests check it
    wq, wk = R.dequantized_weight(ds[0]), R.dequantized_weight(ds[1])
    put(f"{tag}/ropecheck_q", apply_rope_reference(x.float() @ wq.T + ds[0]["bias"].float(), cos, sin, hd))
    put(f"{tag}/ropecheck_k", apply_rope_reference(x.float() @ wk.T + ds[1]["bias"].float(), cos, sin, hd))
    cases.append(tag)

# ---- raw bitstream round trips on uniform random codes (reference tests/test_packing.py:8-16)
for bits in (2, 3, 4):
    for k in (32, 200, 1056):
        g = torch.Generator().manual_seed(bits * 1000 + k)
        q = torch.randint(0, 1 << bits, (5, k), generator=g, dtype=torch.int32)
        p = R.pack_codes(q, bits)
        assert torch.equal(R.unpack_codes(p, bits, k), q)
        put(f"codes_w{bits}_k{k}/q", q); put(f"codes_w{bits}_k{k}/packed", p)

store["cases"] = np.array(cases)
np.savez_compressed(OUT, **store)
print(OUT, os.path.getsize(OUT), "bytes;", len(store), "arrays")
