"""Loader for one entry of a packed block file (`block_XXX_wB.pt`): the dict written by the reference's
pack_linear_dict (Crispybits/Kernel/crispybits_kernels/reference.py:70-76) -> PackedLinearWeight on a
device.  Mirrors Crispybits/Kernel/crispybits_kernels/io.py."""
import torch

from .ops import PackedLinearWeight


def from_packed_dict(d: dict, device="cuda", dtype=torch.float16) -> PackedLinearWeight:
    def meta(t):
        return t.to(device=device, dtype=dtype).contiguous()

    bias = d.get("bias")
    return PackedLinearWeight(
        packed=d["packed"].to(device=device, dtype=torch.int32).contiguous(),
        scales=meta(d["scales"]), zeros=meta(d["zeros"]),
        bits=int(d["bits"]), group_size=int(d["group_size"]),
        in_features=int(d["in_features"]), out_features=int(d["out_features"]),
        bias=None if bias is None else meta(bias))
