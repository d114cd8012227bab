"""Quantise / pack / unpack / dequantise and the on-disk writer under the reference's names
(Crispybits/Kernel/crispybits_kernels/reference.py), computed on the GPU by the library's kernels.

The reference's module is a CPU implementation that doubles as its test oracle; here the same functions are
the *fast packer*: `cb_quantize_pack` / `cb_unpack_codes` do the work on the device and give bit-identical
codes, words, scales and zeros (the tests compare them with the CPU oracle).  Inputs may live on the CPU or on
a GPU; they are moved to the current CUDA device for the computation.  Like the rest of the package there is
no CPU path: without the built library or without a GPU these functions raise.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Iterable, Optional

import torch


def _C():
    from . import ops
    ops._check_ext()
    from . import _C as ext
    return ext


def _dev(t: torch.Tensor) -> torch.Tensor:
    if t.is_cuda:
        return t
    if not torch.cuda.is_available():
        raise RuntimeError("crispybits_kernels.reference runs on the GPU: no CUDA device is available")
    return t.cuda()


def quantize_affine(w: torch.Tensor, bits: int, group_size: int = 128):
    """(codes int32 [N, K], scale fp32 [N, G], zero fp32 [N, G]) as reference.py:10-27, on w's device."""
    ext = _C()
    packed, s, z = ext.quantize_pack(_dev(w.detach()).float(), bits, group_size, torch.float32)
    q = ext.unpack_codes(packed, bits, w.shape[1])
    return q.to(w.device), s.to(w.device), z.to(w.device)


def dequantize(q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group_size: int) -> torch.Tensor:
    """(q - zero) * scale in fp32 with per-group metadata (reference.py:30-34)."""
    k = q.shape[1]
    s = scales.float().repeat_interleave(group_size, dim=1)[:, :k]
    z = zeros.float().repeat_interleave(group_size, dim=1)[:, :k]
    return (q.float() - z) * s


def pack_codes(q: torch.Tensor, bits: int) -> torch.Tensor:
    """Packed int32 words of already-quantised codes (reference.py:37-55): code j of a 32-code chunk at bit
    j*bits of the chunk's little-endian stream of `bits` words.  Integer torch ops on the GPU."""
    assert bits in (2, 3, 4)
    qd = _dev(q)
    n, k = qd.shape
    c = -(-k // 32)
    qq = torch.zeros(n, c * 32, dtype=torch.int64, device=qd.device)
    qq[:, :k] = qd.to(torch.int64) & ((1 << bits) - 1)
    qq = qq.view(n, c, 32)
    words = torch.zeros(n, c, bits, dtype=torch.int64, device=qd.device)
    for j in range(32):
        wi, off = divmod(j * bits, 32)
        v = qq[:, :, j] << off
        words[:, :, wi] |= v & 0xFFFFFFFF
        if off + bits > 32:
            words[:, :, wi + 1] |= v >> 32
    words = words.view(n, c * bits)
    return torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32).contiguous().to(q.device)


def unpack_codes(packed: torch.Tensor, bits: int, K: int) -> torch.Tensor:
    """int32 codes [N, K] of packed words (reference.py:58-67), returned on packed's device."""
    out = _C().unpack_codes(_dev(packed).to(torch.int32).contiguous(), bits, K)
    return out.to(packed.device)


def pack_linear_dict(weight: torch.Tensor, bits: int, group_size: int = 128,
                     bias: Optional[torch.Tensor] = None, dtype=torch.float16) -> Dict:
    """The reference's packed-weight dictionary (reference.py:70-76), tensors on the CPU."""
    packed, s, z = _C().quantize_pack(_dev(weight.detach()).float(), bits, group_size, dtype)
    return dict(packed=packed.cpu(), scales=s.cpu(), zeros=z.cpu(), bits=bits, group_size=group_size,
                in_features=weight.shape[1], out_features=weight.shape[0],
                bias=None if bias is None else bias.detach().to(dtype).cpu())


def dequantized_weight(d: Dict) -> torch.Tensor:
    """fp32 [N, K] weight a packed dictionary stands for (reference.py:79-82), on the CPU like its inputs."""
    q = unpack_codes(d["packed"], d["bits"], d["in_features"])
    return dequantize(q, d["scales"], d["zeros"], d["group_size"])


def write_packed_dir(model: torch.nn.Module, out_dir: str, bits_options: Iterable[int] = (2, 3, 4),
                     group_size: int = 128, dtype=torch.float16) -> None:
    """One `block_XXX_wB.pt` per transformer block and bit-width, each a dict {linear name: packed dictionary}
    (reference.py:85-94): the files `install_bitmap` and `io.from_packed_dict` load."""
    from .integration import _blocks
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    for i, block in enumerate(_blocks(model)):
        linears = {n: m for n, m in block.named_modules() if isinstance(m, torch.nn.Linear)}
        for b in bits_options:
            data = {n: pack_linear_dict(m.weight.detach(), b, group_size, m.bias, dtype) for n, m in linears.items()}
            torch.save(data, out / f"block_{i:03d}_w{b}.pt")
