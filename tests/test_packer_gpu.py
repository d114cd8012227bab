"""The GPU quantise+pack kernel and the reference-named module built on it: bit-identical to the CPU oracle."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(HERE, ".."), os.path.join(HERE, "..", "llm_quantization-kernel_b200")]

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("n,k,gs", [(7, 128, 128), (33, 1000, 128), (64, 4096, 128), (5, 96, 32), (3, 777, 64), (4096, 4096, 128)])
def test_quantize_pack_kernel_is_bit_identical_to_the_oracle(bits, n, k, gs):
    from crispybits_kernels import _C
    from oracle import cb_oracle as O
    g = torch.Generator().manual_seed(bits * 1000 + n + k)
    w = torch.randn(n, k, generator=g) * 0.02
    if n > 4:
        w[1] = 0.0                         # an all-equal group: scale clamps to 1e-8
        w[2, : k // 2] = w[2, : k // 2].abs()   # groups that do not straddle zero
    packed, s, z = _C.quantize_pack(w.cuda(), bits, gs, torch.float32)
    q_ref, s_ref, z_ref = O.quantize_affine(w.numpy(), bits, gs)
    assert np.array_equal(s.cpu().numpy(), s_ref)
    assert np.array_equal(z.cpu().numpy(), z_ref)
    assert np.array_equal(packed.cpu().numpy(), O.pack_codes(q_ref, bits))
    assert np.array_equal(_C.unpack_codes(packed, bits, k).cpu().numpy(), q_ref)
    # fp16 metadata is the fp32 result rounded once
    _, s16, z16 = _C.quantize_pack(w.cuda(), bits, gs, torch.float16)
    assert torch.equal(s16.cpu(), torch.from_numpy(s_ref).half())
    assert torch.equal(z16.cpu(), torch.from_numpy(z_ref).half())


def test_reference_named_module_round_trip_and_writer(tmp_path):
    import crispybits_kernels as ck
    from crispybits_kernels import reference as R
    from oracle import cb_oracle as O
    ck.set_backend("cuda")
    w = torch.randn(96, 320) * 0.05
    b = torch.randn(96)
    d = R.pack_linear_dict(w, 3, 64, b, torch.float16)
    ref = O.pack_linear_dict(w.numpy(), 3, 64)
    assert np.array_equal(d["packed"].numpy(), ref["packed"])
    assert np.array_equal(d["scales"].float().numpy(), ref["scales"]) and np.array_equal(d["zeros"].float().numpy(), ref["zeros"])
    assert d["packed"].device.type == "cpu" and d["bias"].dtype == torch.float16
    q, s, z = R.quantize_affine(w, 3, 64)
    assert torch.equal(R.unpack_codes(d["packed"], 3, 320), q)
    assert torch.equal(R.pack_codes(q, 3), d["packed"])
    wd = R.dequantized_weight(d)
    assert np.allclose(wd.numpy(), O.dequantized_weight(ref), rtol=0, atol=0)
    # the packed dictionary drives the kernels
    x = torch.randn(2, 320, device="cuda", dtype=torch.float16)
    y = ck.packed_linear(x, ck.io.from_packed_dict(d))
    want = x.float() @ wd.cuda().T + b.half().float().cuda()
    assert ((y.float() - want).abs().max() / want.abs().max()).item() < 2e-3

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(64, 32)
            self.b = torch.nn.Linear(32, 64, bias=False)

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.model = torch.nn.Module()
            self.model.layers = torch.nn.ModuleList([Block(), Block()])

    m = Tiny()
    R.write_packed_dir(m, str(tmp_path), (2, 4), 32)
    files = sorted(os.listdir(tmp_path))
    assert files == ["block_000_w2.pt", "block_000_w4.pt", "block_001_w2.pt", "block_001_w4.pt"]
    blk = torch.load(tmp_path / "block_001_w4.pt")
    assert set(blk) == {"a", "b"} and blk["a"]["bits"] == 4 and blk["b"]["bias"] is None
    ref = O.pack_linear_dict(m.model.layers[1].a.weight.detach().numpy(), 4, 32)
    assert np.array_equal(blk["a"]["packed"].numpy(), ref["packed"])
