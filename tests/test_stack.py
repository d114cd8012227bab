"""The decode stack (packed linears of N transformer blocks, column-parallel over ranks).

CPU tests: the sharding arithmetic and the 2-rank gather (gloo) reproduce the 1-rank result with the oracle standing
in for the kernels.  GPU test: the stack on one GPU against the fp32 evaluation of the same data flow.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from conftest import PKG, ROOT


def oracle_packer(w, bits, group_size=128, dtype=torch.float16):
    """The CPU oracle's quantise + pack as a DecodeStack packer (test infrastructure)."""
    from crispybits_kernels import PackedLinearWeight
    from oracle import cb_oracle as O
    d = O.pack_linear_dict(w.float().cpu().numpy(), bits, group_size, None, "float16")
    t = lambda a: torch.from_numpy(a).to(w.device)
    return PackedLinearWeight(t(d["packed"]), t(d["scales"]).to(dtype), t(d["zeros"]).to(dtype), bits, group_size,
                              w.shape[1], w.shape[0])


def test_bitmap_draw_is_the_reference_draw():
    from crispybits_kernels.stack import sample_bitmap
    bm = sample_bitmap(32, 0)
    rng = np.random.default_rng(0)      # Crispybits/quantization/scripts/sample_bitmaps.py:11-12
    assert bm == rng.choice(np.array([2, 3, 4], dtype=np.int8), size=(1, 32), replace=True)[0].tolist()
    assert set(bm) <= {2, 3, 4} and abs(np.mean(bm) - 3.0) < 0.2


def _worker(rank, world, port, out_path):
    sys.path[:0] = [ROOT, PKG, os.path.join(ROOT, "tests")]
    import torch.distributed as dist
    import oracle_backend
    from crispybits_kernels import ops
    from crispybits_kernels.stack import DecodeStack
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ops.set_backend(oracle_backend)
    torch.manual_seed(0)
    x = torch.randn(2, 256).half()
    from test_stack import oracle_packer
    sharded = DecodeStack(2, 256, 512, bitmap=[3, 4], rank=rank, world=world, device="cpu", std=0.05, packer=oracle_packer)
    y = sharded.step(x)
    if rank == 0:
        full = DecodeStack(2, 256, 512, bitmap=[3, 4], rank=0, world=1, device="cpu", std=0.05, packer=oracle_packer)
        torch.save({"sharded": y, "full": full.step(x), "bytes": (sharded.algorithmic_bytes(2), full.algorithmic_bytes(2))},
                   out_path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_column_split_matches_one_rank(tmp_path):
    """gloo, world size 2, oracle-backed kernels: the gathered column-parallel step equals the single-rank step."""
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "res.pt")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["sharded"].shape == (2, 256)
    err = (res["sharded"].float() - res["full"].float()).abs().max() / res["full"].float().abs().max()
    assert err < 2e-3, err
    # two ranks move half of the weight bytes each (activations are replicated)
    assert res["bytes"][0] < 0.6 * res["bytes"][1]


@pytest.mark.gpu
def test_stack_on_gpu_matches_fp32_dataflow():
    from crispybits_kernels import ops
    from crispybits_kernels.stack import DecodeStack
    from oracle import cb_oracle as O
    ops.set_backend("cuda")
    st = DecodeStack(3, 512, 1024, bitmap=[4, 2, 3], device="cuda", std=0.05)
    # rebuild the full dequantised weights from the stack's own packed tensors with the oracle
    full = []
    for blk in st.blocks:
        d = {}
        for name in ("q", "k", "v", "o", "gate", "up", "down"):
            w = getattr(blk, name)
            dd = dict(packed=w.packed.cpu().numpy(), scales=w.scales.float().cpu().numpy(), zeros=w.zeros.float().cpu().numpy(),
                      bits=w.bits, group_size=w.group_size, in_features=w.in_features)
            d[name] = torch.from_numpy(O.dequantized_weight(dd)).cuda()
        full.append(d)
    for B in (1, 4, 8):
        x = torch.randn(B, 512, device="cuda", dtype=torch.float16)
        y = st.step(x)
        ref = st.reference_step(x, full)
        err = ((y.float() - ref).abs().max() / ref.abs().max()).item()
        assert err < 4e-3, (B, err)      # four chained fp16 launches
    assert st.launches_per_step() == 12
