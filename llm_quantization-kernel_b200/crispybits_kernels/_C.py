"""`crispybits_kernels._C` for B200: a ctypes shim over libcrispybits_b200.so.

The reference builds a pybind11/libtorch module of this name from
Crispybits/Kernel/csrc/bindings.cpp:32-40.  This module exposes the same seven functions with the
same positional signatures, so `ops.py` calls it unchanged, but the native side is a plain C ABI
(include/crispybits_b200.h): this file checks the tensors the way
Crispybits/Kernel/csrc/host_utils.h:49-87 does (failures raise RuntimeError, as TORCH_CHECK does),
allocates outputs and Split-K scratch with torch, and passes raw device pointers plus the current
CUDA stream across the boundary.

There is no CPU path here: importing this module without the built library raises ImportError, and
calling it with CPU tensors raises RuntimeError.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from typing import Dict, List, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libcrispybits_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is not built; run `python llm_quantization-kernel_b200/build.py`")
_lib = ctypes.CDLL(LIB_PATH)

IS_EMULATOR = False
_vp, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t


class _Weight(ctypes.Structure):
    """struct cb_weight of include/crispybits_b200.h"""
    _fields_ = [("packed", _vp), ("scales", _vp), ("zeros", _vp), ("bias", _vp), ("n", _i64)]


_WP = ctypes.POINTER(_Weight)
_lib.cb_last_error.restype = ctypes.c_char_p
_lib.cb_version.restype = ctypes.c_char_p
_lib.cb_gemv_scratch_bytes.restype = _sz
_lib.cb_gemv_scratch_bytes.argtypes = [_i64, _i64, _i64]
_lib.cb_packed_gemv.argtypes = [_vp, _i64, _WP, _vp, _i64, _int, _i64, _int, _i64, _i64, _int, _vp, _sz, _vp]
_lib.cb_fused_gate_up.argtypes = [_vp, _i64, _WP, _WP, _vp, _i64, _int, _i64, _int, _i64, _i64, _vp, _sz, _vp]
_lib.cb_fused_qkv.argtypes = [_vp, _i64, _WP, _WP, _WP, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _i64,
                              _int, _i64, _i64, _vp, _sz, _vp]
_lib.cb_packed_gemm.argtypes = [_vp, _i64, _WP, _vp, _i64, _int, _i64, _int, _int, _int, _vp]
_lib.cb_packed_gemm_scratch.argtypes = [_vp, _i64, _WP, _vp, _i64, _int, _i64, _int, _int, _int, _vp, _sz, _vp]
_lib.cb_packed_gemm_scratch.restype = _int
_lib.cb_gemm_scratch_bytes.argtypes = [_i64, _i64, _i64]
_lib.cb_gemm_scratch_bytes.restype = _sz
_COUNTER_BYTES = 65536 * 4      # the decode kernels' arrival counters at the head of a stream's scratch buffer
_lib.cb_unpack_codes.argtypes = [_vp, _i64, _i64, _int, _vp, _vp]
_lib.cb_max_rho.argtypes = [_int, _int]
_lib.cb_decode_plan.argtypes = [_int, _i64, _i64, _i64, _i64, _i64, _int, ctypes.POINTER(ctypes.c_longlong)]
_lib.cb_set_option.argtypes = [_int, _int]
_lib.cb_set_option.restype = None
_lib.cb_decode_status.argtypes = [ctypes.POINTER(_int)]
for _f in ("cb_packed_gemv", "cb_fused_gate_up", "cb_fused_qkv", "cb_packed_gemm", "cb_unpack_codes",
           "cb_sm_count", "cb_tile_n", "cb_max_rho", "cb_decode_status"):
    getattr(_lib, _f).restype = _int

_DTYPE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_KIND = {"gemv": 0, "qkv": 1, "gate_up": 2}


def _fail(msg: str):
    raise RuntimeError(msg)


def _rc(code: int):
    if code != 0:
        raise RuntimeError(_lib.cb_last_error().decode() or f"libcrispybits_b200 error {code}")


def _ptr(t) -> int:
    return 0 if t is None or t.numel() == 0 else t.data_ptr()


def _check_x(x: torch.Tensor, k: int):
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        _fail("x must be a CUDA tensor (this build has no CPU path)")
    if x.dim() != 2:
        _fail("x must be [B, K]")
    if not x.is_contiguous():
        _fail("x must be contiguous")
    if x.shape[1] != k:
        _fail("x K != in_features")
    if x.dtype not in _DTYPE:
        _fail("x must be fp16/bf16/fp32")


def _check_weight(x, packed, scales, zeros, bits: int, k: int, gs: int, name: str):
    if not (packed.is_cuda and scales.is_cuda and zeros.is_cuda):
        _fail(f"{name}: tensors must be CUDA")
    if packed.device != x.device or scales.device != x.device or zeros.device != x.device:
        _fail(f"{name}: weight and activation on different devices")
    if packed.dtype != torch.int32:
        _fail(f"{name}: packed must be torch.int32")
    if packed.dim() != 2 or scales.dim() != 2:
        _fail(f"{name}: packed/scales must be 2-D")
    if not (packed.is_contiguous() and scales.is_contiguous() and zeros.is_contiguous()):
        _fail(f"{name}: weight tensors must be contiguous")
    if scales.shape != zeros.shape:
        _fail(f"{name}: scale/zero shape mismatch")
    if scales.shape[0] != packed.shape[0]:
        _fail(f"{name}: metadata rows != output rows")
    if scales.dtype != x.dtype or zeros.dtype != x.dtype:
        _fail(f"{name}: metadata dtype must match x")
    if bits not in (2, 3, 4):
        _fail(f"{name}: bits must be 2/3/4")
    if gs <= 0 or gs % 32:
        _fail(f"{name}: group_size must be a positive multiple of 32")
    if packed.shape[1] != -(-k // 32) * bits:
        _fail(f"{name}: packed row must hold exactly ceil(K/32)*bits words (rows padded to 32 codes)")
    if scales.shape[1] != -(-k // gs):
        _fail(f"{name}: expected ceil(K/group_size) groups")
    align = 16 if bits == 4 else (8 if bits == 2 else 4)
    if packed.data_ptr() % align:
        _fail(f"{name}: packed storage must be {align}-byte aligned for vector loads")


def _bias_or_none(bias, x, n: int):
    if bias is None or bias.numel() == 0:
        return None
    if not bias.is_cuda or bias.device != x.device:
        _fail("bias must be on x's device")
    if bias.numel() != n:
        _fail("bias length must equal out_features")
    if bias.dtype != x.dtype:
        _fail("bias dtype must match x")
    if not bias.is_contiguous():
        _fail("bias must be contiguous")
    return bias


def _check_workspace(ws, x):
    """The reference's 2-int job-queue workspace (host_utils.h:38-47).  The B200 kernels partition work
    statically and need no queue; a caller-supplied workspace is validated and left untouched, so it
    still reads [0, 0] afterwards."""
    if ws is None or ws.numel() < 2:
        return
    if not ws.is_cuda or ws.device != x.device:
        _fail("workspace must be on x's device")
    if ws.dtype != torch.int32 or not ws.is_contiguous():
        _fail("workspace must be contiguous int32")


def _weight(packed, scales, zeros, bias) -> _Weight:
    return _Weight(packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(), _ptr(bias), packed.shape[0])


# Weights that passed their checks, so that a model's repeated calls with the same tensors do not pay for them again:
# (identities of the four tensors, bits, K, group size, activation dtype and device) -> (weak reference to `packed`,
# the record handed to the library).  An identity can be reused after a tensor dies, hence the weak reference; a tensor
# whose storage is swapped in place (`.data = ...`) changes its data pointer, so the four pointers are compared too.
_checked: Dict[tuple, tuple] = {}


def _checked_weight(x, packed, scales, zeros, bias, bits: int, k: int, gs: int, name: str) -> _Weight:
    key = (id(packed), id(scales), id(zeros), id(bias), bits, k, gs, x.dtype, x.device)
    hit = _checked.get(key)
    if hit is not None and hit[0]() is packed:
        w = hit[1]
        if (w.packed == packed.data_ptr() and w.scales == scales.data_ptr() and w.zeros == zeros.data_ptr()
                and (w.bias or 0) == _ptr(bias)):
            return w
    _check_weight(x, packed, scales, zeros, bits, k, gs, name)
    w = _weight(packed, scales, zeros, _bias_or_none(bias, x, packed.shape[0]))
    if len(_checked) >= 8192:
        _checked.clear()
    _checked[key] = (weakref.ref(packed), w)
    return w


_COUNTER_REGION = 65536 * 4      # cb_gemv_scratch_bytes: a fixed region of arrival counters, then split_k * B * V floats


# Split-K scratch: one zero-initialised buffer per (device, stream), grown on demand and kept alive
# for the life of the process (CUDA graphs that captured its address stay valid).  The kernels reset
# the counters they use, so the buffer is zeroed only when it is created.
_scratch: Dict[Tuple[int, int], torch.Tensor] = {}
_retired: List[torch.Tensor] = []


def _scratch_for(x: torch.Tensor, stream: int, nbytes: int):
    if nbytes == 0:
        return None
    key = (x.device.index, stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _retired.append(buf)   # a captured graph may still point at it
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=x.device)
        _scratch[key] = buf
    return buf


def _decode_scratch(x, stream: int, B: int, V: int, pk: int):
    """Scratch for a decode call.  Sized for the requested split and, so that the streamlined kernel may
    raise the split when its shared-memory budget asks for it, for at least a 4-way split (the arithmetic of
    cb_gemv_scratch_bytes, done here to save two library calls per launch)."""
    return _scratch_for(x, stream, _COUNTER_REGION + max(pk, 4) * B * V * 4)


class _on_device:
    """`with torch.cuda.device(...)` only when the tensor's device is not the current one."""
    __slots__ = ("ctx",)

    def __init__(self, device):
        self.ctx = None if device.index is None or torch.cuda.current_device() == device.index else torch.cuda.device(device)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        return False


def _stream(x) -> int:
    return torch.cuda.current_stream(x.device).cuda_stream


def packed_gemv(x, packed, scales, zeros, bias, bits, in_features, group_size, split_k, rho, act, workspace):
    bits, k, gs, split_k, rho, act = int(bits), int(in_features), int(group_size), int(split_k), int(rho), int(act)
    _check_x(x, k)
    w = _checked_weight(x, packed, scales, zeros, bias, bits, k, gs, "packed_gemv")
    if split_k < 1:
        _fail("split_k must be >= 1")
    if not 0 <= act <= 2:
        _fail("act must be 0 (none), 1 (relu) or 2 (silu)")
    _check_workspace(workspace, x)
    B, n = x.shape[0], packed.shape[0]
    out = torch.empty((B, n), dtype=x.dtype, device=x.device)
    if B == 0:
        return out
    with _on_device(x.device):
        st = _stream(x)
        pk = max(1, min(split_k, -(-k // 32)))
        sc = _decode_scratch(x, st, B, n, pk)
        _rc(_lib.cb_packed_gemv(x.data_ptr(), B, ctypes.byref(w), out.data_ptr(), k, bits, gs, _DTYPE[x.dtype],
                                pk, rho, act, _ptr(sc), 0 if sc is None else sc.numel(), st))
    return out


def packed_gemm(x, packed, scales, zeros, bias, bits, in_features, group_size, act, use_tensor_cores):
    bits, k, gs, act = int(bits), int(in_features), int(group_size), int(act)
    _check_x(x, k)
    _check_weight(x, packed, scales, zeros, bits, k, gs, "packed_gemm")
    if not 0 <= act <= 2:
        _fail("act must be 0 (none), 1 (relu) or 2 (silu)")
    bias = _bias_or_none(bias, x, packed.shape[0])
    M, n = x.shape[0], packed.shape[0]
    out = torch.empty((M, n), dtype=x.dtype, device=x.device)
    if M == 0:
        return out
    with torch.cuda.device(x.device):
        w = _weight(packed, scales, zeros, bias)
        st = _stream(x)
        # scratch for a K split of few-token calls: behind the decode kernels' counter region of the stream's buffer
        need = _lib.cb_gemm_scratch_bytes(M, n, k) if use_tensor_cores else 0
        sc = _scratch_for(x, st, _COUNTER_BYTES + need) if need else None
        _rc(_lib.cb_packed_gemm_scratch(x.data_ptr(), M, ctypes.byref(w), out.data_ptr(), k, bits, gs, _DTYPE[x.dtype],
                                        act, 1 if use_tensor_cores else 0,
                                        0 if sc is None else sc.data_ptr() + _COUNTER_BYTES, need, st))
    return out


def fused_gate_up(x, wg, sg, zg, wu, su, zu, bits, in_features, group_size, split_k, rho, workspace):
    bits, k, gs, split_k, rho = int(bits), int(in_features), int(group_size), int(split_k), int(rho)
    _check_x(x, k)
    _check_weight(x, wg, sg, zg, bits, k, gs, "fused_gate_up(gate)")
    _check_weight(x, wu, su, zu, bits, k, gs, "fused_gate_up(up)")
    if wg.shape != wu.shape:
        _fail("gate/up packed shapes must match")
    if split_k < 1:
        _fail("split_k must be >= 1")
    _check_workspace(workspace, x)
    B, n = x.shape[0], wg.shape[0]
    out = torch.empty((B, n), dtype=x.dtype, device=x.device)
    if B == 0:
        return out
    with torch.cuda.device(x.device):
        st = _stream(x)
        pk = max(1, min(split_k, -(-k // 32)))
        sc = _decode_scratch(x, st, B, 2 * n, pk)
        g, u = _weight(wg, sg, zg, None), _weight(wu, su, zu, None)
        _rc(_lib.cb_fused_gate_up(x.data_ptr(), B, ctypes.byref(g), ctypes.byref(u), out.data_ptr(), k, bits, gs,
                                  _DTYPE[x.dtype], pk, rho, _ptr(sc), 0 if sc is None else sc.numel(), st))
    return out


def fused_qkv(x, wq, sq, zq, bq, wk, sk, zk, bk, wv, sv, zv, bv, rope_cos, rope_sin, head_dim, perm_hd,
              bits, in_features, group_size, split_k, rho, workspace):
    bits, k, gs, split_k, rho = int(bits), int(in_features), int(group_size), int(split_k), int(rho)
    head_dim, perm_hd = int(head_dim), int(perm_hd)
    _check_x(x, k)
    _check_weight(x, wq, sq, zq, bits, k, gs, "fused_qkv(q)")
    _check_weight(x, wk, sk, zk, bits, k, gs, "fused_qkv(k)")
    _check_weight(x, wv, sv, zv, bits, k, gs, "fused_qkv(v)")
    if split_k < 1:
        _fail("split_k must be >= 1")
    B = x.shape[0]
    if perm_hd > 0:
        if perm_hd % 2:
            _fail("perm head_dim must be even")
        if wq.shape[0] % perm_hd or wk.shape[0] % perm_hd:
            _fail("Q/K widths must be multiples of head_dim")
    rope = rope_cos is not None and rope_cos.numel() > 0
    rc = rs = None
    if rope:
        if not (perm_hd > 0 and perm_hd == head_dim):
            _fail("fused RoPE needs Q/K weights stored pair-interleaved with the same head_dim "
                  "(ops.permute_for_rope / install_bitmap(fuse_rope=True))")
        if rope_cos.shape != rope_sin.shape:
            _fail("cos/sin shape mismatch")
        if rope_cos.numel() != B * head_dim:
            _fail("cos/sin must be [B, head_dim] (one row per x row)")
        rc = rope_cos.to(device=x.device, dtype=torch.float32).contiguous()
        rs = rope_sin.to(device=x.device, dtype=torch.float32).contiguous()
    bq, bk, bv = (_bias_or_none(b, x, w.shape[0]) for b, w in ((bq, wq), (bk, wk), (bv, wv)))
    _check_workspace(workspace, x)
    outs = [torch.empty((B, w.shape[0]), dtype=x.dtype, device=x.device) for w in (wq, wk, wv)]
    if B == 0:
        return outs
    with torch.cuda.device(x.device):
        st = _stream(x)
        pk = max(1, min(split_k, -(-k // 32)))
        V = wq.shape[0] + wk.shape[0] + wv.shape[0]
        sc = _decode_scratch(x, st, B, V, pk)
        q, kk, v = _weight(wq, sq, zq, bq), _weight(wk, sk, zk, bk), _weight(wv, sv, zv, bv)
        _rc(_lib.cb_fused_qkv(x.data_ptr(), B, ctypes.byref(q), ctypes.byref(kk), ctypes.byref(v),
                              outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), _ptr(rc), _ptr(rs),
                              head_dim if rope else 0, perm_hd, k, bits, gs, _DTYPE[x.dtype], pk, rho,
                              _ptr(sc), 0 if sc is None else sc.numel(), st))
    return outs


# ------------------------------------------------------------------ column-parallel stacks (no reference counterpart)
class _Scatter(ctypes.Structure):
    """struct cb_scatter of include/crispybits_b200.h"""
    _fields_ = [("peer_out", _vp * 8), ("world", _int), ("n_gather", _i64), ("ld", _i64), ("col", _i64),
                ("sync", _int), ("rank", _int), ("peer_flags", _vp * 8), ("my_flags", _vp), ("epoch", _vp),
                ("done", _vp), ("status", _vp), ("seq", _i64), ("need", _i64)]


class PeerSync:
    """Device words of the in-kernel rank hand-shake (see struct cb_scatter): peer flag arrays, own flag array,
    launch count, CTA counter and status."""

    def __init__(self, peer_flag_ptrs, my_flags: torch.Tensor, epoch: torch.Tensor, done: torch.Tensor,
                 status: torch.Tensor, rank: int, numbered: bool = False):
        self.peer_flag_ptrs, self.rank = list(peer_flag_ptrs), int(rank)
        self.my_flags, self.epoch, self.done, self.status = my_flags, epoch, done, status
        self.numbered = bool(numbered)     # the numbered hand-shake (cb_scatter.sync == 2): seq per launch, publish, step end


_SP = ctypes.POINTER(_Scatter)
_lib.cb_packed_gemv_scatter.argtypes = [_vp, _i64, _WP, _vp, _SP, _i64, _int, _i64, _int, _i64, _i64, _int, _vp, _sz, _vp]
_lib.cb_fused_gate_up_scatter.argtypes = [_vp, _i64, _WP, _WP, _vp, _SP, _i64, _int, _i64, _int, _i64, _i64, _vp, _sz, _vp]
_lib.cb_peer_barrier.argtypes = [ctypes.POINTER(_vp), _vp, _vp, _vp, _int, _int, _vp]
_lib.cb_peer_wait.argtypes = [_SP, _vp]
_lib.cb_peer_publish.argtypes = [_SP, _vp]
_lib.cb_peer_step_end.argtypes = [_SP, _i64, _vp]
for _f in ("cb_packed_gemv_scatter", "cb_fused_gate_up_scatter", "cb_peer_barrier", "cb_peer_wait", "cb_peer_publish",
           "cb_peer_step_end"):
    getattr(_lib, _f).restype = _int


def _scatter(peer_ptrs, n_gather: int, ld: int, col: int, sync: "PeerSync | None" = None, seq: int = 0,
             need: "int | None" = None) -> _Scatter:
    sc = _Scatter()
    for i, ptr in enumerate(peer_ptrs):
        sc.peer_out[i] = ptr
    sc.world, sc.n_gather, sc.ld, sc.col = len(peer_ptrs), n_gather, ld, col
    if sync is not None:
        sc.sync, sc.rank, sc.seq = (2 if sync.numbered else 1), sync.rank, int(seq)
        sc.need = int(seq) if need is None else int(need)
        for i, ptr in enumerate(sync.peer_flag_ptrs):
            sc.peer_flags[i] = ptr
        sc.my_flags, sc.epoch = sync.my_flags.data_ptr(), sync.epoch.data_ptr()
        sc.done, sc.status = sync.done.data_ptr(), sync.status.data_ptr()
    return sc


def packed_gemv_scatter(x, packed, scales, zeros, bias, out, peer_ptrs, n_gather, ld, col, bits, in_features,
                        group_size, split_k, rho, act, sync=None, seq=0, need=None):
    """packed_gemv whose output rows < n_gather go to every rank's gathered buffer (peer pointers) at column
    `col` of a [B, ld] matrix; the other rows go to `out` [B, N].  `seq`: number of the launch within its step, for a
    numbered hand-shake."""
    bits, k, gs, split_k = int(bits), int(in_features), int(group_size), int(split_k)
    _check_x(x, k)
    _check_weight(x, packed, scales, zeros, bits, k, gs, "packed_gemv_scatter")
    bias = _bias_or_none(bias, x, packed.shape[0])
    B, n = x.shape[0], packed.shape[0]
    if out.shape != (B, n) or out.dtype != x.dtype or not out.is_contiguous() or out.device != x.device:
        _fail("packed_gemv_scatter: out must be a contiguous [B, N] tensor of x's dtype on x's device")
    with torch.cuda.device(x.device):
        st = _stream(x)
        pk = max(1, min(split_k, -(-k // 32)))
        sc = _decode_scratch(x, st, B, n, pk)
        w, s = _weight(packed, scales, zeros, bias), _scatter(peer_ptrs, int(n_gather), int(ld), int(col), sync, seq, need)
        _rc(_lib.cb_packed_gemv_scatter(x.data_ptr(), B, ctypes.byref(w), out.data_ptr(), ctypes.byref(s), k, bits, gs,
                                        _DTYPE[x.dtype], pk, int(rho), int(act), _ptr(sc), 0 if sc is None else sc.numel(), st))
    return out


def fused_gate_up_scatter(x, wg, sg, zg, wu, su, zu, out, peer_ptrs, n_gather, ld, col, bits, in_features, group_size,
                          split_k, rho, sync=None, seq=0):
    bits, k, gs, split_k = int(bits), int(in_features), int(group_size), int(split_k)
    _check_x(x, k)
    _check_weight(x, wg, sg, zg, bits, k, gs, "fused_gate_up_scatter(gate)")
    _check_weight(x, wu, su, zu, bits, k, gs, "fused_gate_up_scatter(up)")
    if wg.shape != wu.shape:
        _fail("gate/up packed shapes must match")
    B, n = x.shape[0], wg.shape[0]
    if out.shape != (B, n) or out.dtype != x.dtype or not out.is_contiguous():
        _fail("fused_gate_up_scatter: out must be a contiguous [B, N] tensor of x's dtype")
    with torch.cuda.device(x.device):
        st = _stream(x)
        pk = max(1, min(split_k, -(-k // 32)))
        sc = _decode_scratch(x, st, B, 2 * n, pk)
        g, u, s = _weight(wg, sg, zg, None), _weight(wu, su, zu, None), _scatter(peer_ptrs, int(n_gather), int(ld), int(col), sync, seq)
        _rc(_lib.cb_fused_gate_up_scatter(x.data_ptr(), B, ctypes.byref(g), ctypes.byref(u), out.data_ptr(), ctypes.byref(s),
                                          k, bits, gs, _DTYPE[x.dtype], pk, int(rho), _ptr(sc), 0 if sc is None else sc.numel(), st))
    return out


def peer_barrier(peer_flag_ptrs, my_flags: torch.Tensor, epoch: torch.Tensor, status: torch.Tensor, rank: int):
    """Launch the rank-to-rank barrier kernel on the current stream of my_flags' device."""
    world = len(peer_flag_ptrs)
    arr = (_vp * world)(*peer_flag_ptrs)
    with torch.cuda.device(my_flags.device):
        _rc(_lib.cb_peer_barrier(arr, my_flags.data_ptr(), epoch.data_ptr(), status.data_ptr(), world, int(rank),
                                 torch.cuda.current_stream(my_flags.device).cuda_stream))


def peer_publish(sync: "PeerSync", seq: int):
    """Numbered hand-shake: after scatter launch `seq` of a step, the one-CTA kernel that tells every rank it is done."""
    sc = _scatter([0] * len(sync.peer_flag_ptrs), 0, 1, 0, sync, seq)
    with _on_device(sync.my_flags.device):
        _rc(_lib.cb_peer_publish(ctypes.byref(sc), torch.cuda.current_stream(sync.my_flags.device).cuda_stream))


def peer_step_end(sync: "PeerSync", launches: int):
    """Numbered hand-shake: end of a step of `launches` launches (bounded wait for every rank, then the step base moves)."""
    sc = _scatter([0] * len(sync.peer_flag_ptrs), 0, 1, 0, sync)
    with _on_device(sync.my_flags.device):
        _rc(_lib.cb_peer_step_end(ctypes.byref(sc), int(launches), torch.cuda.current_stream(sync.my_flags.device).cuda_stream))


def peer_wait(sync: "PeerSync"):
    """Launch the bounded wait for the peers' latest hand-shake launch on the current stream."""
    sc = _scatter([0] * len(sync.peer_flag_ptrs), 0, 1, 0, sync)
    with torch.cuda.device(sync.my_flags.device):
        _rc(_lib.cb_peer_wait(ctypes.byref(sc), torch.cuda.current_stream(sync.my_flags.device).cuda_stream))


def unpack_codes(packed: torch.Tensor, bits: int, in_features: int) -> torch.Tensor:
    """int32 codes [N, K] from packed words, computed on the GPU (checked bit-for-bit in the tests)."""
    if not packed.is_cuda or packed.dtype != torch.int32 or packed.dim() != 2 or not packed.is_contiguous():
        _fail("packed must be a contiguous 2-D CUDA int32 tensor")
    k = int(in_features)
    if packed.shape[1] != -(-k // 32) * int(bits):
        _fail("packed row must hold exactly ceil(K/32)*bits words")
    out = torch.empty((packed.shape[0], k), dtype=torch.int32, device=packed.device)
    with torch.cuda.device(packed.device):
        _rc(_lib.cb_unpack_codes(packed.data_ptr(), packed.shape[0], k, int(bits), out.data_ptr(),
                                 torch.cuda.current_stream(packed.device).cuda_stream))
    return out


_lib.cb_fused_gate_up_gemm.argtypes = [_vp, _i64, _WP, _WP, _vp, _i64, _int, _i64, _int, _vp]
_lib.cb_fused_gate_up_gemm.restype = _int


def fused_gate_up_gemm(x, wg, sg, zg, wu, su, zu, bits, in_features, group_size):
    """silu(x Wg^T) * (x Wu^T) for a prefill batch in one launch, or None when the shape is outside the fused
    kernel's domain (the caller then runs two GEMMs and a product, as the reference does)."""
    bits, k, gs = int(bits), int(in_features), int(group_size)
    _check_x(x, k)
    _check_weight(x, wg, sg, zg, bits, k, gs, "fused_gate_up_gemm(gate)")
    _check_weight(x, wu, su, zu, bits, k, gs, "fused_gate_up_gemm(up)")
    if wg.shape != wu.shape:
        _fail("gate/up packed shapes must match")
    if x.dtype not in (torch.float16, torch.bfloat16) or k % 128 or gs % 64:
        return None
    M, n = x.shape[0], wg.shape[0]
    out = torch.empty((M, n), dtype=x.dtype, device=x.device)
    if M == 0:
        return out
    with torch.cuda.device(x.device):
        g, u = _weight(wg, sg, zg, None), _weight(wu, su, zu, None)
        rc = _lib.cb_fused_gate_up_gemm(x.data_ptr(), M, ctypes.byref(g), ctypes.byref(u), out.data_ptr(), k, bits, gs,
                                        _DTYPE[x.dtype], _stream(x))
    if rc == 3:          # CB_ERR_UNSUPPORTED
        return None
    _rc(rc)
    return out


_lib.cb_fused_qkv_gemm.argtypes = [_vp, _i64, _WP, _WP, _WP, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _i64, _int, _vp]
_lib.cb_fused_qkv_gemm.restype = _int


def fused_qkv_gemm(x, wq, sq, zq, bq, wk, sk, zk, bk, wv, sv, zv, bv, rope_cos, rope_sin, head_dim, perm_hd,
                   bits, in_features, group_size):
    """Q, K, V of a prefill batch (+ bias, + RoPE on Q and K, outputs in the original column order) in one launch,
    or None when the shape is outside the fused kernel's domain (every projection's rows a multiple of 128); the
    caller then runs three GEMMs and rotates afterwards, as the reference does."""
    bits, k, gs = int(bits), int(in_features), int(group_size)
    head_dim, perm_hd = int(head_dim), int(perm_hd)
    _check_x(x, k)
    _check_weight(x, wq, sq, zq, bits, k, gs, "fused_qkv_gemm(q)")
    _check_weight(x, wk, sk, zk, bits, k, gs, "fused_qkv_gemm(k)")
    _check_weight(x, wv, sv, zv, bits, k, gs, "fused_qkv_gemm(v)")
    if x.dtype not in (torch.float16, torch.bfloat16) or k % 128 or gs % 64:
        return None
    if any(w.shape[0] % 128 for w in (wq, wk, wv)):
        return None
    M = x.shape[0]
    if perm_hd > 0:
        if perm_hd % 2:
            _fail("perm head_dim must be even")
        if wq.shape[0] % perm_hd or wk.shape[0] % perm_hd:
            _fail("Q/K widths must be multiples of head_dim")
    rope = rope_cos is not None and rope_cos.numel() > 0
    rc = rs = None
    if rope:
        if not (perm_hd > 0 and perm_hd == head_dim):
            _fail("fused RoPE needs Q/K weights stored pair-interleaved with the same head_dim "
                  "(ops.permute_for_rope / install_bitmap(fuse_rope=True))")
        if rope_cos.shape != rope_sin.shape:
            _fail("cos/sin shape mismatch")
        if rope_cos.numel() != M * head_dim:
            _fail("cos/sin must be [M, head_dim] (one row per x row)")
        rc = rope_cos.to(device=x.device, dtype=torch.float32).contiguous()
        rs = rope_sin.to(device=x.device, dtype=torch.float32).contiguous()
    bq, bk, bv = (_bias_or_none(b, x, w.shape[0]) for b, w in ((bq, wq), (bk, wk), (bv, wv)))
    outs = [torch.empty((M, w.shape[0]), dtype=x.dtype, device=x.device) for w in (wq, wk, wv)]
    if M == 0:
        return outs
    with torch.cuda.device(x.device):
        q, kk, v = _weight(wq, sq, zq, bq), _weight(wk, sk, zk, bk), _weight(wv, sv, zv, bv)
        code = _lib.cb_fused_qkv_gemm(x.data_ptr(), M, ctypes.byref(q), ctypes.byref(kk), ctypes.byref(v),
                                      outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), _ptr(rc), _ptr(rs),
                                      head_dim, perm_hd, k, bits, gs, _DTYPE[x.dtype], _stream(x))
    if code == 3:        # CB_ERR_UNSUPPORTED
        return None
    _rc(code)
    return outs


_lib.cb_quantize_pack.argtypes = [_vp, _int, _i64, _i64, _int, _i64, _vp, _vp, _vp, _int, _vp]
_lib.cb_quantize_pack.restype = _int


def quantize_pack(w: torch.Tensor, bits: int, group_size: int, meta_dtype=torch.float16):
    """(packed int32 [N, ceil(K/32)*bits], scales, zeros [N, ceil(K/gs)] of meta_dtype) from a CUDA [N, K] float
    matrix, computed by the library's quantise+pack kernel (bit-identical to the reference's CPU packer)."""
    if not w.is_cuda or w.dim() != 2 or w.dtype not in _DTYPE:
        _fail("quantize_pack: w must be a 2-D CUDA tensor of float32, float16 or bfloat16")
    if meta_dtype not in _DTYPE:
        _fail("quantize_pack: scales/zeros dtype must be float32, float16 or bfloat16")
    bits, gs = int(bits), int(group_size)
    w = w.contiguous()
    n, k = w.shape
    packed = torch.empty((n, -(-k // 32) * bits), dtype=torch.int32, device=w.device)
    scales = torch.empty((n, -(-k // gs)), dtype=meta_dtype, device=w.device)
    zeros = torch.empty_like(scales)
    with torch.cuda.device(w.device):
        _rc(_lib.cb_quantize_pack(w.data_ptr(), _DTYPE[w.dtype], n, k, bits, gs, packed.data_ptr(), scales.data_ptr(),
                                  zeros.data_ptr(), _DTYPE[meta_dtype], torch.cuda.current_stream(w.device).cuda_stream))
    return packed, scales, zeros


def sm_count() -> int:
    n = _lib.cb_sm_count()
    if n < 0:
        _rc(2)
    return int(n)


def tile_n() -> int:
    return int(_lib.cb_tile_n())


def max_rho(bits: int, kind: str = "gemv") -> int:
    if kind not in _KIND:
        _fail("kind must be 'gemv', 'qkv' or 'gate_up'")
    r = _lib.cb_max_rho(int(bits), _KIND[kind])
    if r < 0:
        _rc(1)
    return int(r)


def decode_plan(bits: int, batch: int, rows: int, in_features: int, split_k: int = 1, rho: int = 1, sms: int = 148):
    """Launch plan of the ring decode kernel as a dict (host arithmetic only; no GPU needed), or None when the ring
    kernel does not take the problem."""
    out = (ctypes.c_longlong * 7)()
    if _lib.cb_decode_plan(bits, batch, rows, in_features, split_k, rho, sms, out) != 0:
        return None
    keys = ("grid", "smem_bytes", "split_k", "rows_per_pass", "ring_slots", "passes", "row_slabs")
    return dict(zip(keys, (int(v) for v in out)))


def set_option(option: int, value: int) -> None:
    """0: programmatic dependent launch on/off; 1: force the shape-generic decode kernel (A/B checks)."""
    _lib.cb_set_option(int(option), int(value))


def decode_status() -> int:
    """Synchronise, then read and clear the decode kernels' error word (0 = fine)."""
    out = _int(0)
    _rc(_lib.cb_decode_status(ctypes.byref(out)))
    return int(out.value)


def version() -> str:
    return _lib.cb_version().decode()
