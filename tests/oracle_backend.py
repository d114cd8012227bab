"""A stand-in for `crispybits_kernels._C` backed by the CPU oracle, for tests only.

It lets the host-side code of the package (ops.py routing and policy, integration.py module surgery,
autotune.py) run on a machine without a GPU, the way the reference's test-suite uses its emulator
(Crispybits/Kernel/tests/conftest.py:12-22).  Install it with `ops.set_backend(oracle_backend)`.
Tensors are converted to float32 numpy arrays, pushed through oracle/cb_oracle.py, and converted back.
"""
import numpy as np
import torch

from oracle import cb_oracle as O

IS_EMULATOR = True
_NAME = {torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float32: "float32"}


def sm_count():
    return 148


def tile_n():
    return 16


def max_rho(bits, kind="gemv"):
    if kind not in ("gemv", "qkv", "gate_up"):
        raise RuntimeError("kind must be 'gemv', 'qkv' or 'gate_up'")
    return 2


def _f(t):
    return None if t is None or t.numel() == 0 else t.detach().float().cpu().numpy()


def _i(t):
    return t.detach().cpu().numpy().astype(np.int32)


def _back(a, like):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device=like.device, dtype=like.dtype)


def _check_dtypes(x, *meta):
    if x.dtype not in _NAME:
        raise RuntimeError("x must be fp16/bf16/fp32")
    if not x.is_contiguous() or x.dim() != 2:
        raise RuntimeError("x must be contiguous [B, K]")
    for m in meta:
        if m.dtype != x.dtype:
            raise RuntimeError("metadata dtype must match x")


def _check_ws(ws):
    if ws is not None and ws.numel() >= 2:
        assert ws.dtype == torch.int32 and ws[:2].tolist() == [0, 0], "workspace not reset"


def packed_gemv(x, packed, scales, zeros, bias, bits, K, gs, split_k, rho, act, ws):
    _check_dtypes(x, scales, zeros); _check_ws(ws)
    if packed.dtype != torch.int32:
        raise RuntimeError("packed must be torch.int32")
    y = O.packed_gemv(_f(x), _i(packed), _f(scales), _f(zeros), _f(bias), int(bits), int(K), int(gs), int(split_k),
                      int(act), _NAME[x.dtype])
    return _back(y, x)


def packed_gemm(x, packed, scales, zeros, bias, bits, K, gs, act, use_tensor_cores):
    _check_dtypes(x, scales, zeros)
    y = O.packed_gemm(_f(x), _i(packed), _f(scales), _f(zeros), _f(bias), int(bits), int(K), int(gs), int(act),
                      bool(use_tensor_cores), _NAME[x.dtype])
    return _back(y, x)


def fused_gate_up(x, wg, sg, zg, wu, su, zu, bits, K, gs, split_k, rho, ws):
    _check_dtypes(x, sg, zg, su, zu); _check_ws(ws)
    y = O.fused_gate_up(_f(x), _i(wg), _f(sg), _f(zg), _i(wu), _f(su), _f(zu), int(bits), int(K), int(gs),
                        int(split_k), _NAME[x.dtype])
    return _back(y, x)


def fused_qkv(x, wq, sq, zq, bq, wk, sk, zk, bk, wv, sv, zv, bv, rope_cos, rope_sin, head_dim, perm_hd,
              bits, K, gs, split_k, rho, ws):
    _check_dtypes(x, sq, zq, sk, zk, sv, zv); _check_ws(ws)
    pr = [(_i(w), _f(s), _f(z), _f(b)) for w, s, z, b in ((wq, sq, zq, bq), (wk, sk, zk, bk), (wv, sv, zv, bv))]
    outs = O.fused_qkv(_f(x), pr[0], pr[1], pr[2], _f(rope_cos), _f(rope_sin), int(head_dim), int(perm_hd),
                       int(bits), int(K), int(gs), int(split_k), _NAME[x.dtype])
    return [_back(o, x) for o in outs]
