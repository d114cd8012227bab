"""Public operator API of the packed W2/W3/W4 linear path (B200 build).

Same names, arguments and error behaviour as the reference's
Crispybits/Kernel/crispybits_kernels/ops.py, so callers (integration.py, autotune.py, user code) do
not change: `PackedLinearWeight`, `packed_linear`, `fused_gate_up`, `fused_qkv`, `PackedLinear`, the
RoPE row-permutation helpers and the Split-K policy helpers.  Underneath, `_C` is the ctypes shim
over libcrispybits_b200.so instead of the pybind11 module; there is no CPU backend in this package
(the reference's emulator lives on as the test oracle, outside the package).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, replace
from functools import lru_cache
from math import ceil
from typing import Optional, Tuple

import torch
import torch.nn as nn

try:
    from . import _C as _CUDA
    _IMPORT_ERROR = None
except Exception as exc:  # library not built (or not loadable): every op raises, nothing falls back
    _CUDA = None
    _IMPORT_ERROR = exc

_C = _CUDA

DECODE_THRESHOLD = 4          # rows <= this use the decode GEMV, more rows the prefill GEMM (ops.py:23)
ACT = {"none": 0, None: 0, "relu": 1, "silu": 2}
KINDS = ("gemv", "qkv", "gate_up")
BATCH_BLOCK = 8               # batch rows that share one pass over the weights in the decode kernels

if os.environ.get("CRISPYBITS_BACKEND", "").lower() == "emulator":
    raise RuntimeError("CRISPYBITS_BACKEND=emulator: this build ships no CPU emulator; the packed linear "
                       "path runs on the GPU only")


def set_backend(backend):
    """Select what `_C` points at.  "cuda" is the only named backend of this build.  An object that
    provides the seven binding functions (packed_gemv, packed_gemm, fused_gate_up, fused_qkv, sm_count,
    tile_n, max_rho) may be passed instead of a name; the test-suite uses that to drive this module
    with its CPU oracle."""
    global _C
    if backend == "cuda":
        _C = _CUDA
    elif backend == "emulator":
        raise RuntimeError("no CPU emulator in this build; pass a backend object to set_backend for testing")
    elif isinstance(backend, str):
        raise ValueError(backend)
    else:
        _C = backend
    tile_n.cache_clear()


def backend_name() -> str:
    return "emulator" if (_C is not None and getattr(_C, "IS_EMULATOR", False)) else "cuda"


def _check_ext():
    if _C is None:
        raise RuntimeError(f"crispybits CUDA library is not available: {_IMPORT_ERROR}")


@dataclass
class PackedLinearWeight:
    """One packed linear layer: int32 `packed` [N, ceil(K/32)*bits], `scales`/`zeros` [N, ceil(K/group)]
    in the activation dtype, optional `bias` [N].  `rope_perm_head_dim` > 0 marks rows stored
    pair-interleaved per head for the fused RoPE epilogue."""
    packed: torch.Tensor
    scales: torch.Tensor
    zeros: torch.Tensor
    bits: int
    group_size: int
    in_features: int
    out_features: int
    bias: Optional[torch.Tensor] = None
    rope_perm_head_dim: int = 0

    def cuda(self, device=None, dtype=torch.float16):
        dev = device or "cuda"
        mv = lambda t, dt: t.to(device=dev, dtype=dt).contiguous()
        return replace(self, packed=mv(self.packed, torch.int32), scales=mv(self.scales, dtype),
                       zeros=mv(self.zeros, dtype), bias=None if self.bias is None else mv(self.bias, dtype))


_ABSENT = {}       # (device, dtype) -> the 0-element tensor that stands for "absent"; made once, not per call


def _absent(device, dtype) -> torch.Tensor:
    t = _ABSENT.get((device, dtype))
    if t is None:
        t = _ABSENT[(device, dtype)] = torch.empty(0, device=device, dtype=dtype)
    return t


def _none_like(x: torch.Tensor) -> torch.Tensor:
    """The bindings take a 0-element tensor for "absent" (ops.py:74-83)."""
    return _absent(x.device, x.dtype)


def _bias_arg(w: PackedLinearWeight, x: torch.Tensor):
    return _none_like(x) if w.bias is None else w.bias


def _ws_arg(workspace, x):
    return _absent(x.device, torch.int32) if workspace is None else workspace


def new_workspace(device) -> torch.Tensor:
    """Two zeroed int32 counters, the reference's persistent job-queue workspace.  The B200 kernels do
    not need it; it is accepted everywhere and left at [0, 0]."""
    return torch.zeros(2, dtype=torch.int32, device=device)


# ------------------------------------------------------------------ RoPE row permutation
def rope_row_order(out_features: int, head_dim: int, device=None) -> torch.Tensor:
    """order[p] = original row stored at position p: inside each head 0, h/2, 1, h/2+1, ... so that the
    two rows RoPE mixes are neighbours (p, p^1)."""
    if head_dim % 2 or out_features % head_dim:
        raise ValueError("out_features must be a multiple of an even head_dim")
    half = head_dim // 2
    lo = torch.arange(half)
    within = torch.stack((lo, lo + half), dim=1).flatten()
    base = torch.arange(0, out_features, head_dim)
    return (base[:, None] + within[None, :]).flatten().to(device)


def rope_inverse_order(out_features: int, head_dim: int, device=None) -> torch.Tensor:
    order = rope_row_order(out_features, head_dim)
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel())
    return inverse.to(device)


def permute_for_rope(w: PackedLinearWeight, head_dim: int) -> PackedLinearWeight:
    """Return `w` with rows (and bias) stored pair-interleaved for the fused RoPE epilogue."""
    if w.rope_perm_head_dim:
        if w.rope_perm_head_dim != head_dim:
            raise ValueError("weight already permuted with a different head_dim")
        return w
    order = rope_row_order(w.out_features, head_dim, w.packed.device)
    take = lambda t: t[order].contiguous()
    return replace(w, packed=take(w.packed), scales=take(w.scales), zeros=take(w.zeros),
                   bias=None if w.bias is None else take(w.bias), rope_perm_head_dim=head_dim)


def _unpermute_cols(y: torch.Tensor, w: PackedLinearWeight) -> torch.Tensor:
    """Outputs in stored-row order -> original column order (prefill path of a permuted weight)."""
    if not w.rope_perm_head_dim:
        return y
    return y.index_select(-1, rope_inverse_order(w.out_features, w.rope_perm_head_dim, y.device))


def apply_rope_reference(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, head_dim: int) -> torch.Tensor:
    """rotate_half RoPE on a flat [M, H*head_dim] tensor with cos/sin [M, head_dim] (prefill path)."""
    rows, width = t.shape
    heads = t.float().view(rows, width // head_dim, head_dim)
    half = head_dim // 2
    rotated = torch.cat((-heads[..., half:], heads[..., :half]), dim=-1)
    out = heads * cos.float()[:, None, :] + rotated * sin.float()[:, None, :]
    return out.view(rows, width).to(t.dtype)


# ------------------------------------------------------------------ Split-K policy
@lru_cache(maxsize=None)
def tile_n() -> int:
    """Virtual output rows per decode work tile (B_N of the policy)."""
    _check_ext()
    return int(_C.tile_n())


@lru_cache(maxsize=None)
def _sm_count_for(device_index: int) -> int:
    if backend_name() == "emulator":
        return int(_C.sm_count())
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def sm_count():
    _check_ext()
    return int(_C.sm_count())


def max_rho(bits: int, kind: str = "gemv"):
    _check_ext()
    return int(_C.max_rho(bits, kind))


def virtual_rows(kind: str, *out_features: int) -> int:
    """Rows the decode kernel iterates over: N, Nq+Nk+Nv, or 2N (gate and up interleaved)."""
    if kind == "gemv":
        return out_features[0]
    if kind == "qkv":
        return sum(out_features)
    if kind == "gate_up":
        return 2 * out_features[0]
    raise ValueError(kind)


def candidate_split_k(batch: int, n: int, bn: int, sms: int, rho: int, max_split: Optional[int] = None) -> int:
    """SM-underfill rule: with C_out = batch * ceil(n / bn) output tiles and a target of rho * sms
    resident CTAs, split K by ceil(C_target / C_out) when the tiles alone would leave SMs idle."""
    rho = max(1, int(rho))
    tiles, target = batch * ceil(n / bn), rho * sms
    if tiles >= target:
        return 1
    split = max(1, ceil(target / tiles))
    return split if max_split is None else min(max_split, split)


def balanced_split_k(batch: int, n: int, bn: int, sms: int, rho: int, nchunks: int,
                     min_chunks: int = 8, good: float = 0.94) -> int:
    """B200 refinement of the underfill rule.  Work units are dealt round-robin to rho*sms persistent
    CTAs, so the last wave is partly empty unless units is close to a multiple of the grid.  Starting
    from the underfill rule's answer, take the smallest split whose wave efficiency
    units / (ceil(units / grid) * grid) reaches `good`, keeping at least `min_chunks` 32-code chunks
    per split (else the one with the best efficiency).  `batch` counts blocks of up to 8 rows: the
    kernels read the weights once per block."""
    blocks = ceil(batch / BATCH_BLOCK)
    tiles = blocks * ceil(n / bn)
    grid = max(1, int(rho)) * sms
    first = candidate_split_k(blocks, n, bn, sms, rho)
    limit = max(first, min(32, max(1, nchunks // min_chunks)))
    best, best_eff = first, 0.0
    for split in range(first, limit + 1):
        units = tiles * split
        eff = units / (ceil(units / grid) * grid)
        if eff >= good:
            return split
        if eff > best_eff + 1e-9:
            best, best_eff = split, eff
    return best


def _resolve(split_k: Optional[int], rho: int, batch: int, v_rows: int, k: int, device,
             dtype=None, group_size: Optional[int] = None) -> int:
    """An explicit split_k is clamped to the chunk count; None applies the policy for this batch."""
    nchunks = ceil(k / 32)
    if split_k is not None:
        return max(1, min(int(split_k), nchunks))
    # Inside the domain of the fp16 / bf16 ring kernel (group 128, K a multiple of 256, up to 8 batch rows) no split is
    # the measured optimum on B200 at every shape tried, also for 512- and 1376-row shards (3.2 us against 5.0 us
    # with the underfill rule's split): the kernel spreads a matrix over the SMs by rows and a K split costs it
    # a partial-sum round trip through memory that is as long as the whole launch.
    if dtype in (torch.float16, torch.bfloat16) and group_size == 128 and k % 256 == 0 and batch <= BATCH_BLOCK:
        return 1
    if device.type == "cuda":
        index = device.index if device.index is not None else torch.cuda.current_device()
    else:
        index = 0
    # The decode kernels read the weights once per block of up to 8 batch rows and give every CTA an
    # equal slab of rows, so the underfill rule applies with batch counted in blocks: split K only
    # when there are fewer 16-row tiles than resident CTAs.
    split = candidate_split_k(ceil(batch / BATCH_BLOCK), v_rows, tile_n(), _sm_count_for(index), rho)
    return max(1, min(split, nchunks))


# ------------------------------------------------------------------ operators
def _rows(x: torch.Tensor) -> torch.Tensor:
    if x.dim() == 2 and x.is_contiguous():
        return x
    return x.reshape(-1, x.shape[-1]).contiguous()


def _packed_linear_raw(x, w, split_k=None, rho=1, act=None, decode_threshold=DECODE_THRESHOLD,
                       workspace=None, use_tensor_cores=True):
    lead = x.shape[:-1]
    x2 = _rows(x)
    code = ACT[act]
    if x2.shape[0] <= decode_threshold:
        split = _resolve(split_k, rho, x2.shape[0], w.out_features, w.in_features, x2.device, x2.dtype, w.group_size)
        y = _C.packed_gemv(x2, w.packed, w.scales, w.zeros, _bias_arg(w, x2), w.bits, w.in_features,
                           w.group_size, split, rho, code, _ws_arg(workspace, x2))
    else:
        y = _C.packed_gemm(x2, w.packed, w.scales, w.zeros, _bias_arg(w, x2), w.bits, w.in_features,
                           w.group_size, code, use_tensor_cores)
    return y if len(lead) == 1 else y.reshape(*lead, w.out_features)


def packed_linear(x: torch.Tensor, w: PackedLinearWeight, split_k: Optional[int] = None, rho: int = 1,
                  act: Optional[str] = None, decode_threshold: int = DECODE_THRESHOLD,
                  workspace: Optional[torch.Tensor] = None, use_tensor_cores: bool = True):
    """act(x W^T + bias).  Up to `decode_threshold` rows run the decode GEMV, more the prefill GEMM."""
    _check_ext()
    if w.rope_perm_head_dim:
        raise ValueError("this weight is stored RoPE-permuted; use fused_qkv (or _unpermute_cols)")
    return _packed_linear_raw(x, w, split_k, rho, act, decode_threshold, workspace, use_tensor_cores)


def fused_gate_up(x: torch.Tensor, gate: PackedLinearWeight, up: PackedLinearWeight,
                  split_k: Optional[int] = None, rho: int = 1, decode_threshold: int = DECODE_THRESHOLD,
                  workspace: Optional[torch.Tensor] = None):
    """silu(x Wg^T) * (x Wu^T): one decode launch up to the threshold, above it one fused tcgen05 prefill launch
    (two prefill GEMMs and a product where that kernel does not apply)."""
    _check_ext()
    if gate.bits != up.bits:
        raise ValueError("fused Gate/Up requires the same precision for Gate and Up within a block")
    x2 = _rows(x)
    if x2.shape[0] <= decode_threshold:
        split = _resolve(split_k, rho, x2.shape[0], virtual_rows("gate_up", gate.out_features),
                         gate.in_features, x2.device, x2.dtype, gate.group_size)
        y = _C.fused_gate_up(x2, gate.packed, gate.scales, gate.zeros, up.packed, up.scales, up.zeros,
                             gate.bits, gate.in_features, gate.group_size, split, rho, _ws_arg(workspace, x2))
    else:
        # one fused tcgen05 launch where the backend has it and the shape allows it; else two GEMMs and a product
        fused = getattr(_C, "fused_gate_up_gemm", None)
        y = None
        if fused is not None and gate.group_size == up.group_size and gate.in_features == up.in_features:
            y = fused(x2, gate.packed, gate.scales, gate.zeros, up.packed, up.scales, up.zeros, gate.bits,
                      gate.in_features, gate.group_size)
        if y is None:
            none = _none_like(x2)
            g = _C.packed_gemm(x2, gate.packed, gate.scales, gate.zeros, none, gate.bits, gate.in_features,
                               gate.group_size, ACT["silu"], True)
            u = _C.packed_gemm(x2, up.packed, up.scales, up.zeros, none, up.bits, up.in_features,
                               up.group_size, ACT["none"], True)
            y = g * u
    return y.reshape(*x.shape[:-1], gate.out_features)


def fused_qkv(x: torch.Tensor, q: PackedLinearWeight, k: PackedLinearWeight, v: PackedLinearWeight,
              split_k: Optional[int] = None, rho: int = 1,
              rope: Optional[Tuple[torch.Tensor, torch.Tensor, int]] = None,
              decode_threshold: int = DECODE_THRESHOLD, workspace: Optional[torch.Tensor] = None):
    """Q, K, V projections of one x in a single decode launch (GQA widths and biases allowed).
    `rope=(cos, sin, head_dim)` also rotates Q and K in the epilogue; that needs Q/K stored with
    permute_for_rope(w, head_dim).  Outputs are always in the original column order."""
    _check_ext()
    if not (q.bits == k.bits == v.bits):
        raise ValueError("Q/K/V must use the block precision")
    if q.rope_perm_head_dim != k.rope_perm_head_dim or v.rope_perm_head_dim:
        raise ValueError("Q and K must be permuted with the same head_dim; V must not be permuted")
    perm = q.rope_perm_head_dim
    lead = x.shape[:-1]
    x2 = _rows(x)
    rows = x2.shape[0]
    if rope is not None:
        cos, sin, head_dim = rope
        head_dim = int(head_dim)
        if perm != head_dim:
            raise ValueError("fused RoPE needs Q/K permuted with permute_for_rope(w, head_dim) "
                             "(install_bitmap(fuse_rope=True) does this)")
        cos2 = cos.expand(*lead, head_dim).reshape(rows, head_dim)
        sin2 = sin.expand(*lead, head_dim).reshape(rows, head_dim)
    if rows <= decode_threshold:
        total = virtual_rows("qkv", q.out_features, k.out_features, v.out_features)
        split = _resolve(split_k, rho, rows, total, q.in_features, x2.device, x2.dtype, q.group_size)
        if rope is None:
            rc, rs, hd = _none_like(x2), _none_like(x2), 0
        else:
            rc, rs, hd = cos2.float().contiguous(), sin2.float().contiguous(), head_dim
        oq, ok, ov = _C.fused_qkv(x2, q.packed, q.scales, q.zeros, _bias_arg(q, x2),
                                  k.packed, k.scales, k.zeros, _bias_arg(k, x2),
                                  v.packed, v.scales, v.zeros, _bias_arg(v, x2),
                                  rc, rs, hd, perm, q.bits, q.in_features, q.group_size, split, rho,
                                  _ws_arg(workspace, x2))
    else:
        fused, fused_fn = None, getattr(_C, "fused_qkv_gemm", None)
        if fused_fn is not None:
            # one launch with bias, rotation and un-permuted stores in the epilogue (None outside its domain)
            fused = fused_fn(x2, q.packed, q.scales, q.zeros, _bias_arg(q, x2),
                             k.packed, k.scales, k.zeros, _bias_arg(k, x2),
                             v.packed, v.scales, v.zeros, _bias_arg(v, x2),
                             None if rope is None else cos2.float().contiguous(),
                             None if rope is None else sin2.float().contiguous(),
                             0 if rope is None else head_dim, perm, q.bits, q.in_features, q.group_size)
        if fused is not None:
            oq, ok, ov = fused
        else:
            oq, ok, ov = (_unpermute_cols(_packed_linear_raw(x2, w, decode_threshold=0), w) for w in (q, k, v))
            if rope is not None:
                oq = apply_rope_reference(oq, cos2, sin2, head_dim)
                ok = apply_rope_reference(ok, cos2, sin2, head_dim)
    return (oq.reshape(*lead, q.out_features), ok.reshape(*lead, k.out_features),
            ov.reshape(*lead, v.out_features))


class PackedLinear(nn.Module):
    """nn.Linear replacement holding one packed weight; forward = packed_linear."""

    def __init__(self, w: PackedLinearWeight, split_k: Optional[int] = None, rho: int = 1,
                 act: Optional[str] = None):
        super().__init__()
        for name in ("packed", "scales", "zeros", "bias"):
            self.register_buffer(name, getattr(w, name))
        self.register_buffer("workspace", new_workspace(w.packed.device), persistent=False)
        self.bits, self.group_size = int(w.bits), int(w.group_size)
        self.in_features, self.out_features = int(w.in_features), int(w.out_features)
        self.rope_perm_head_dim = int(w.rope_perm_head_dim)
        self.split_k = None if split_k is None else int(split_k)
        self.rho = int(rho)
        self.act = act

    def weight_spec(self) -> PackedLinearWeight:
        return PackedLinearWeight(self.packed, self.scales, self.zeros, self.bits, self.group_size,
                                  self.in_features, self.out_features, self.bias, self.rope_perm_head_dim)

    def permute_for_rope_(self, head_dim: int):
        """In place: store rows pair-interleaved for the fused RoPE epilogue."""
        w = permute_for_rope(self.weight_spec(), head_dim)
        self.packed, self.scales, self.zeros, self.bias = w.packed, w.scales, w.zeros, w.bias
        self.rope_perm_head_dim = head_dim
        return self

    def forward(self, x):
        return packed_linear(x, self.weight_spec(), self.split_k, self.rho, self.act, workspace=self.workspace)

    def extra_repr(self):
        perm = f", rope_perm={self.rope_perm_head_dim}" if self.rope_perm_head_dim else ""
        return (f"in={self.in_features}, out={self.out_features}, W{self.bits}, g={self.group_size}, "
                f"split_k={self.split_k}, rho={self.rho}, act={self.act}{perm}")
