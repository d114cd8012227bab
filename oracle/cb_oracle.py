"""CPU oracle for the packed W2/W3/W4 linear path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy, the algorithm of the CrispyBits reference for
the packed linear path: the group-wise affine quantizer, the little-endian
bitstream layout, and the decode GEMV / prefill GEMM / fused QKV / fused
gate-up arithmetic of the reference's CPU emulator.  It exists to check the
CUDA kernels; nothing in the shipped package may import it.  Only the test
suite, the smoke entry point and the benchmark's CPU-baseline leg use it.

Parity status: PINNED.  Every function here is compared against outputs of
the reference's own ``reference.py`` / ``emulator.py`` (imported once, on the
machine that holds the reference tree) through the fixtures in
``tests/golden/`` and against the known-answer vectors of the reference's
``tests/test_packing.py``; see ``tests/golden/make_golden.py``.

Each function cites the reference lines it follows, as
``Crispybits/Kernel/<file>:<lines>``.

Conventions.  Arrays are numpy.  Floating inputs are float32 arrays whose
values are exactly representable in the storage dtype named by ``dtype``
("float16", "bfloat16" or "float32"); results are float32 arrays rounded to
that dtype.  Integer codes are int32, packed words are int32 (two's complement
view of the 32-bit word, as the reference stores them).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

TILE_N = 32      # Crispybits/Kernel/crispybits_kernels/emulator.py:9
SM_COUNT = 108   # emulator.py:10
MAX_RHO = 4      # emulator.py:11
IS_EMULATOR = True

_F32 = np.float32


# --------------------------------------------------------------------------- dtype helpers
def round_to(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round a float32 array to `dtype` (round-to-nearest-even) and return it as float32."""
    a = np.asarray(a, dtype=_F32)
    if dtype == "float32":
        return a
    if dtype == "float16":
        with np.errstate(over="ignore"):
            return a.astype(np.float16).astype(_F32)
    if dtype == "bfloat16":
        u = a.view(np.uint32).astype(np.uint64)
        nan = np.isnan(a)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
        out = u.astype(np.uint32).view(_F32).copy()
        out[nan] = np.nan
        return out
    raise ValueError(dtype)


def _act(y: np.ndarray, act: int) -> np.ndarray:
    """0 none, 1 relu, 2 silu  (emulator.py:12; csrc/common.cuh:15-19)."""
    if act == 0:
        return y
    if act == 1:
        return np.maximum(y, _F32(0))
    if act == 2:
        return (y / (_F32(1) + np.exp(-y, dtype=_F32))).astype(_F32)
    raise RuntimeError("act must be 0 (none), 1 (relu) or 2 (silu)")


# --------------------------------------------------------------------------- quantizer
def quantize_affine(w: np.ndarray, bits: int, group_size: int = 128) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Group-wise asymmetric affine quantizer (reference.py:10-27).

    scale = max((max-min)/qmax, 1e-8), zero = clamp(round(-min/scale), 0, qmax),
    q = clamp(round(w/scale) + zero, 0, qmax); a ragged last group is padded by
    repeating the last column.  All arithmetic in float32, rounding half-to-even.
    Returns (q int32 [N,K], scale float32 [N,G], zero float32 [N,G]).
    """
    assert bits in (2, 3, 4)
    w = np.asarray(w, dtype=_F32)
    n, k = w.shape
    g = math.ceil(k / group_size)
    kp = g * group_size
    wf = np.zeros((n, kp), dtype=_F32)
    wf[:, :k] = w
    if kp != k:
        wf[:, k:] = wf[:, k - 1:k]
    grp = wf.reshape(n, g, group_size)
    qmax = _F32((1 << bits) - 1)
    mn, mx = grp.min(-1), grp.max(-1)
    scale = np.maximum((mx - mn) / qmax, _F32(1e-8)).astype(_F32)
    zero = np.clip(np.rint((-mn) / scale), _F32(0), qmax).astype(_F32)
    q = np.clip(np.rint(grp / scale[..., None]) + zero[..., None], _F32(0), qmax)
    q = q.reshape(n, kp)[:, :k].astype(np.int32)
    return q, scale, zero


def dequantize(q: np.ndarray, scales: np.ndarray, zeros: np.ndarray, group_size: int) -> np.ndarray:
    """(q - zero) * scale with per-group metadata broadcast along K (reference.py:30-34)."""
    k = q.shape[1]
    s = np.repeat(np.asarray(scales, dtype=_F32), group_size, axis=1)[:, :k]
    z = np.repeat(np.asarray(zeros, dtype=_F32), group_size, axis=1)[:, :k]
    return ((q.astype(_F32) - z) * s).astype(_F32)


# --------------------------------------------------------------------------- bit layout
def pack_codes(q: np.ndarray, bits: int) -> np.ndarray:
    """Codes -> per-row little-endian bitstream of int32 words (reference.py:37-55).

    Code k of a row sits at bit k*bits of the row's stream; K is padded with
    zero codes to a multiple of 32, so every 32-code chunk is exactly `bits`
    words.  For 3 bits, codes 10 and 21 of each chunk straddle two words.
    """
    assert bits in (2, 3, 4)
    q = np.asarray(q)
    n, k = q.shape
    c = math.ceil(k / 32)
    qq = np.zeros((n, c * 32), dtype=np.uint64)
    qq[:, :k] = q.astype(np.int64).astype(np.uint64) & np.uint64((1 << bits) - 1)
    qq = qq.reshape(n, c, 32)
    # A chunk is a 32*bits-bit integer (at most 128 bits): build it as two 64-bit halves.
    words = np.zeros((n, c, bits), dtype=np.uint64)
    for j in range(32):
        pos = j * bits
        wi, off = divmod(pos, 32)
        v = qq[:, :, j] << np.uint64(off)          # fits in 35 bits
        words[:, :, wi] |= v & np.uint64(0xFFFFFFFF)
        if off + bits > 32:
            words[:, :, wi + 1] |= v >> np.uint64(32)
    out = words.reshape(n, c * bits).astype(np.uint32).view(np.int32)
    return np.ascontiguousarray(out)


def unpack_codes(packed: np.ndarray, bits: int, k: int) -> np.ndarray:
    """Inverse of pack_codes for the first k codes of each row (reference.py:58-67)."""
    w = np.asarray(packed).astype(np.int64) & 0xFFFFFFFF
    idx = np.arange(k, dtype=np.int64)
    pos = idx * bits
    wi, off = pos // 32, pos % 32
    lo = w[:, wi] >> off
    nxt = np.minimum(wi + 1, w.shape[1] - 1)
    hi = np.where(off + bits > 32, w[:, nxt] << (32 - off), 0)
    return ((lo | hi) & ((1 << bits) - 1)).astype(np.int32)


def pack_linear_dict(weight: np.ndarray, bits: int, group_size: int = 128,
                     bias: Optional[np.ndarray] = None, dtype: str = "float16") -> Dict:
    """Quantize + pack one linear layer (reference.py:70-76).

    Scales and zeros are rounded to `dtype` AFTER the codes were computed from
    the float32 scale; the rounded values are what the kernels and the
    dequant-then-matmul check see.
    """
    q, s, z = quantize_affine(weight, bits, group_size)
    return dict(packed=pack_codes(q, bits), scales=round_to(s, dtype), zeros=round_to(z, dtype),
                bits=bits, group_size=group_size, in_features=int(weight.shape[1]),
                out_features=int(weight.shape[0]),
                bias=None if bias is None else round_to(bias, dtype), dtype=dtype)


def dequantized_weight(d: Dict) -> np.ndarray:
    """float32 weight seen by the kernels (reference.py:79-82)."""
    q = unpack_codes(d["packed"], d["bits"], d["in_features"])
    return dequantize(q, d["scales"], d["zeros"], d["group_size"])


# --------------------------------------------------------------------------- validation
def _check(x, packed, scales, zeros, bits, k, gs, name):
    """Argument rules shared by all entry points (emulator.py:29-38; csrc/host_utils.h:49-78)."""
    if not (x.ndim == 2 and x.shape[1] == k):
        raise RuntimeError(f"{name}: x must be [B, in_features]")
    if packed.dtype != np.int32 or packed.ndim != 2:
        raise RuntimeError(f"{name}: packed must be 2-D int32")
    if bits not in (2, 3, 4):
        raise RuntimeError(f"{name}: bits must be 2/3/4")
    if not (gs > 0 and gs % 32 == 0):
        raise RuntimeError(f"{name}: group_size must be a positive multiple of 32")
    if packed.shape[1] != math.ceil(k / 32) * bits:
        raise RuntimeError(f"{name}: packed row must hold ceil(K/32)*bits words")
    if scales.shape != zeros.shape or scales.shape[0] != packed.shape[0]:
        raise RuntimeError(f"{name}: scale/zero shape")
    if scales.shape[1] != math.ceil(k / gs):
        raise RuntimeError(f"{name}: expected ceil(K/group_size) groups")


def _bias(b, n):
    if b is None or np.size(b) == 0:
        return np.zeros(n, dtype=_F32)
    if np.size(b) != n:
        raise RuntimeError("bias length must equal out_features")
    return np.asarray(b, dtype=_F32).reshape(n)


# --------------------------------------------------------------------------- decode arithmetic
def split_bounds(nchunks: int, split_k: int):
    """Chunk range of each K split: [C*s/P, C*(s+1)/P)  (csrc/packed_gemv.cu:94-95; emulator.py:63-65)."""
    p = max(1, min(int(split_k), nchunks))
    return [((nchunks * s) // p, (nchunks * (s + 1)) // p) for s in range(p)]


def partials(x, rows, scales, zeros, bits, k, gs, split_k) -> np.ndarray:
    """Per-split partial sums [P, B, V] with the kernel's chunk algebra (emulator.py:48-67).

    For every 32-code chunk c of row v:  s[v,g(c)] * (sum_j x_j q_j - z[v,g(c)] * sum_j x_j),
    g(c) = 32c // group_size, everything in float32; x is zero-padded to whole chunks.
    """
    b = x.shape[0]
    c = math.ceil(k / 32)
    q = unpack_codes(rows, bits, c * 32).astype(_F32).reshape(-1, c, 32)
    xp = np.zeros((b, c * 32), dtype=_F32)
    xp[:, :k] = x
    xc = xp.reshape(b, c, 32)
    dot = np.einsum("bcj,vcj->bvc", xc, q, optimize=True).astype(_F32)
    xsum = xc.sum(-1, dtype=_F32)
    g = (np.arange(c) * 32) // gs
    s = np.asarray(scales, dtype=_F32)[:, g]
    z = np.asarray(zeros, dtype=_F32)[:, g]
    contrib = s[None] * (dot - z[None] * xsum[:, None, :])
    return np.stack([contrib[..., c0:c1].sum(-1, dtype=_F32) for c0, c1 in split_bounds(c, split_k)])


def packed_gemv(x, packed, scales, zeros, bias, bits, k, gs, split_k=1, act=0, dtype="float16") -> np.ndarray:
    """y = act(x W^T + bias), decode path (emulator.py:77-80; csrc/packed_gemv.cu:252-269, 54-58)."""
    _check(x, packed, scales, zeros, bits, k, gs, "packed_gemv")
    if split_k < 1:
        raise RuntimeError("split_k must be >= 1")
    acc = partials(x, packed, scales, zeros, bits, k, gs, split_k).sum(0, dtype=_F32)
    return round_to(_act(acc + _bias(bias, packed.shape[0])[None], int(act)), dtype)


def fused_gate_up(x, wg, sg, zg, wu, su, zu, bits, k, gs, split_k=1, dtype="float16") -> np.ndarray:
    """silu(x Wg^T) * (x Wu^T): gate row n and up row n are virtual rows 2n, 2n+1
    (emulator.py:83-93; csrc/packed_gemv.cu:33-35, 59-64, 317-337)."""
    _check(x, wg, sg, zg, bits, k, gs, "gate")
    _check(x, wu, su, zu, bits, k, gs, "up")
    if wg.shape != wu.shape:
        raise RuntimeError("gate/up packed shapes must match")
    n = wg.shape[0]
    rows = np.stack([wg, wu], 1).reshape(2 * n, -1)
    s = np.stack([sg, su], 1).reshape(2 * n, -1)
    z = np.stack([zg, zu], 1).reshape(2 * n, -1)
    acc = partials(x, rows, s, z, bits, k, gs, split_k).sum(0, dtype=_F32)
    gate, up = acc[:, 0::2], acc[:, 1::2]
    return round_to(_act(gate, 2) * up, dtype)


def unperm_index(n: int, hd: int) -> np.ndarray:
    """Stored (pair-interleaved) row -> original row (csrc/common.cuh:66-70; emulator.py:96-101)."""
    r = np.arange(n)
    if hd <= 0:
        return r
    head, p = r // hd, r % hd
    return head * hd + np.where(p % 2 == 1, p // 2 + hd // 2, p // 2)


def rope_row_order(out_features: int, head_dim: int) -> np.ndarray:
    """Host permutation: stored row p holds original row order[p]; per head (0, h/2, 1, h/2+1, ...)
    (crispybits_kernels/ops.py:91-98)."""
    if head_dim % 2 or out_features % head_dim:
        raise ValueError("out_features must be a multiple of an even head_dim")
    h = head_dim // 2
    within = np.stack([np.arange(h), np.arange(h) + h], 1).reshape(-1)
    heads = np.arange(out_features // head_dim)[:, None] * head_dim
    return (heads + within[None]).reshape(-1)


def fused_qkv(x, q: Sequence, k_: Sequence, v: Sequence, rope_cos, rope_sin, head_dim, perm_hd,
              bits, k, gs, split_k=1, dtype="float16"):
    """Three projections in one pass; bias; optional RoPE on Q/K with the partner at stored row r^1;
    outputs written at the un-permuted column (emulator.py:104-132; csrc/packed_gemv.cu:65-80, 271-315).

    q, k_, v are (packed, scales, zeros, bias-or-None) tuples; rope_cos/rope_sin are float32
    [B, head_dim] or None.
    """
    for (w, s, z, _), nm in zip((q, k_, v), "qkv"):
        _check(x, w, s, z, bits, k, gs, nm)
    rope = rope_cos is not None and np.size(rope_cos) > 0
    if perm_hd > 0 and not (perm_hd % 2 == 0 and q[0].shape[0] % perm_hd == 0 and k_[0].shape[0] % perm_hd == 0):
        raise RuntimeError("Q/K widths must be multiples of an even head_dim")
    if rope:
        if not (perm_hd > 0 and perm_hd == head_dim):
            raise RuntimeError("fused RoPE needs pair-interleaved Q/K with the same head_dim")
        if np.size(rope_cos) != x.shape[0] * head_dim or np.shape(rope_cos) != np.shape(rope_sin):
            raise RuntimeError("cos/sin must be [B, head_dim]")
    rows = np.concatenate([q[0], k_[0], v[0]])
    s = np.concatenate([q[1], k_[1], v[1]])
    z = np.concatenate([q[2], k_[2], v[2]])
    acc = partials(x, rows, s, z, bits, k, gs, split_k).sum(0, dtype=_F32)
    outs, off = [], 0
    for i, (w, _, _, b) in enumerate((q, k_, v)):
        n = w.shape[0]
        y = acc[:, off:off + n] + _bias(b, n)[None]
        off += n
        hd = perm_hd if i < 2 else 0
        orig = unperm_index(n, hd)
        if rope and i < 2:
            partner = y[:, np.arange(n) ^ 1]
            d = orig % head_dim
            c = np.asarray(rope_cos, dtype=_F32).reshape(-1, head_dim)[:, d]
            sn = np.asarray(rope_sin, dtype=_F32).reshape(-1, head_dim)[:, d]
            y = np.where(d[None] < head_dim // 2, y * c - partner * sn, y * c + partner * sn).astype(_F32)
        out = np.empty_like(y)
        out[:, orig] = y
        outs.append(round_to(out, dtype))
    return outs


def apply_rope(t: np.ndarray, cos: np.ndarray, sin: np.ndarray, head_dim: int) -> np.ndarray:
    """rotate_half RoPE on a flat [M, H*head_dim] array (crispybits_kernels/ops.py:224-231)."""
    m, w = t.shape
    th = t.astype(_F32).reshape(m, w // head_dim, head_dim)
    c, s = cos.astype(_F32)[:, None, :], sin.astype(_F32)[:, None, :]
    h = head_dim // 2
    rot = np.concatenate([-th[..., h:], th[..., :h]], axis=-1)
    return (th * c + rot * s).reshape(m, w)


# --------------------------------------------------------------------------- prefill arithmetic
def packed_gemm(x, packed, scales, zeros, bias, bits, k, gs, act=0, use_tensor_cores=True,
                dtype="float16") -> np.ndarray:
    """Prefill GEMM act(x Wdq^T + bias) (emulator.py:135-144; csrc/packed_gemm.cu:47-61, 182-203).

    On the tensor-core path with a 16-bit dtype the dequantised weight (q-z)*s is rounded to
    that dtype before the product; accumulation is float32.
    """
    _check(x, packed, scales, zeros, bits, k, gs, "packed_gemm")
    q = unpack_codes(packed, bits, k).astype(_F32)
    g = np.arange(k) // gs
    w = (q - np.asarray(zeros, dtype=_F32)[:, g]) * np.asarray(scales, dtype=_F32)[:, g]
    if use_tensor_cores and dtype in ("float16", "bfloat16"):
        w = round_to(w, dtype)
    y = np.asarray(x, dtype=_F32) @ w.T + _bias(bias, packed.shape[0])[None]
    return round_to(_act(y.astype(_F32), int(act)), dtype)


# --------------------------------------------------------------------------- policy arithmetic
def candidate_split_k(batch: int, n: int, bn: int, sms: int, rho: int, max_split: Optional[int] = None) -> int:
    """SM-underfill rule P_K = ceil(rho*S / (B*ceil(N/B_N))) when C_out < C_target, else 1
    (crispybits_kernels/ops.py:155-163)."""
    rho = max(1, int(rho))
    c_out = batch * math.ceil(n / bn)
    c_target = rho * sms
    if c_out >= c_target:
        return 1
    pk = max(1, math.ceil(c_target / c_out))
    return pk if max_split is None else min(max_split, pk)
