"""Pins the CPU oracle (numpy and C) to the reference.

Every fixture in tests/golden/golden_v1.npz is an output of the reference's own reference.py /
emulator.py (see tests/golden/make_golden.py).  Integer work (codes, packed words) must match
bit-for-bit; the float32 quantizer metadata must match exactly; decode / prefill outputs must
match the emulator to within one rounding of the storage dtype.
"""
import numpy as np
import pytest

from oracle import cb_oracle as O
from oracle import cb_oracle_c as OC

# max |a-b| / max |b|: the reference's own metric (Crispybits/Kernel/tests/test_correctness.py:34-37)
def rel(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / (np.abs(b).max() + 1e-6))


# one storage-dtype rounding of the output, relative to the largest output
ULP = {"float16": 1.0e-3, "bfloat16": 8.0e-3, "float32": 2e-6}


def lin_cases(golden):
    return [c for c in golden["cases"].tolist() if c.startswith("lin_")]


def parse(tag):
    # lin_w{bits}_{n}x{k}_g{gs}_{dtype}
    _, wb, nk, g, dtype = tag.split("_")
    n, k = nk.split("x")
    return int(wb[1:]), int(n), int(k), int(g[1:]), dtype


def test_fixture_inventory(golden):
    cases = golden["cases"].tolist()
    assert len(lin_cases(golden)) == 12 and sum(c.startswith("gu_") for c in cases) == 3
    assert sum(c.startswith("qkv_") for c in cases) == 3


@pytest.mark.parametrize("impl", ["numpy", "c"])
def test_quantizer_and_bitstream_bit_exact(golden, impl):
    for tag in lin_cases(golden):
        bits, n, k, gs, dtype = parse(tag)
        w = golden[f"{tag}/w"]
        q, s, z = (O if impl == "numpy" else OC).quantize_affine(w, bits, gs)
        assert np.array_equal(q, golden[f"{tag}/q"]), tag
        assert np.array_equal(s, golden[f"{tag}/scale32"]), tag
        assert np.array_equal(z, golden[f"{tag}/zero32"]), tag
        packed = (O if impl == "numpy" else OC).pack_codes(q, bits)
        assert packed.dtype == np.int32 and np.array_equal(packed, golden[f"{tag}/packed"]), tag
        un = (O if impl == "numpy" else OC).unpack_codes(golden[f"{tag}/packed"], bits, k)
        assert np.array_equal(un, golden[f"{tag}/unpacked"]), tag


def test_pack_linear_dict_matches_reference(golden):
    for tag in lin_cases(golden):
        bits, n, k, gs, dtype = parse(tag)
        bias = golden[f"{tag}/bias"] if f"{tag}/bias" in golden else None
        d = O.pack_linear_dict(golden[f"{tag}/w"], bits, gs, bias, dtype)
        assert np.array_equal(d["packed"], golden[f"{tag}/packed"])
        assert np.array_equal(d["scales"], golden[f"{tag}/scales"])
        assert np.array_equal(d["zeros"], golden[f"{tag}/zeros"])
        assert np.array_equal(O.dequantized_weight(d), golden[f"{tag}/wdq"])
        assert np.array_equal(OC.dequantized_weight(d["packed"], d["scales"], d["zeros"], bits, k, gs),
                              golden[f"{tag}/wdq"])


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("k", [32, 200, 1056])
def test_raw_code_roundtrip(golden, bits, k):
    q, p = golden[f"codes_w{bits}_k{k}/q"], golden[f"codes_w{bits}_k{k}/packed"]
    for impl in (O, OC):
        assert np.array_equal(impl.pack_codes(q, bits), p)
        assert np.array_equal(impl.unpack_codes(p, bits, k), q)


def test_w3_known_answers():
    # Crispybits/Kernel/tests/test_packing.py:28-36
    for impl in (O, OC):
        p = impl.pack_codes(np.full((1, 32), 7, dtype=np.int32), 3)
        assert p.shape == (1, 3) and all((int(v) & 0xFFFFFFFF) == 0xFFFFFFFF for v in p[0])
        q = np.zeros((1, 32), dtype=np.int32)
        q[0, 10] = 0b101
        p = impl.pack_codes(q, 3)
        assert (int(p[0, 0]) & 0xFFFFFFFF) >> 30 == 0b01 and (int(p[0, 1]) & 1) == 1


@pytest.mark.parametrize("bits,per_word", [(2, 16), (4, 8)])
def test_codes_per_word(bits, per_word):
    # Crispybits/Kernel/tests/test_packing.py:19-25
    q = np.concatenate([np.arange(per_word) % (1 << bits), np.zeros(32 - per_word)]).astype(np.int32)[None]
    for impl in (O, OC):
        w0 = int(impl.pack_codes(q, bits)[0, 0]) & 0xFFFFFFFF
        assert [(w0 >> (bits * i)) & ((1 << bits) - 1) for i in range(per_word)] == q[0, :per_word].tolist()


def test_gemv_matches_emulator(golden):
    for tag in lin_cases(golden):
        bits, n, k, gs, dtype = parse(tag)
        x, p, s, z = golden[f"{tag}/x"], golden[f"{tag}/packed"], golden[f"{tag}/scales"], golden[f"{tag}/zeros"]
        bias = golden[f"{tag}/bias"] if f"{tag}/bias" in golden else None
        for split_k in (1, 3):
            for act in (0, 1, 2):
                want = golden[f"{tag}/gemv_s{split_k}_a{act}"]
                got = O.packed_gemv(x, p, s, z, bias, bits, k, gs, split_k, act, dtype)
                assert rel(got, want) <= ULP[dtype], (tag, split_k, act, rel(got, want))
        # C oracle: raw accumulation, compared before bias/activation
        raw = OC.gemv(x, p, s, z, bits, k, gs, 3)
        want = O.partials(x, p, s, z, bits, k, gs, 3).sum(0)
        assert rel(raw, want) < 2e-6, tag
        parts_c = OC.gemv_partials(x, p, s, z, bits, k, gs, 3)
        parts_np = O.partials(x, p, s, z, bits, k, gs, 3)
        assert parts_c.shape == parts_np.shape and rel(parts_c, parts_np) < 2e-6


def test_gemm_matches_emulator(golden):
    for tag in lin_cases(golden):
        bits, n, k, gs, dtype = parse(tag)
        x, p, s, z = golden[f"{tag}/xm"], golden[f"{tag}/packed"], golden[f"{tag}/scales"], golden[f"{tag}/zeros"]
        bias = golden[f"{tag}/bias"] if f"{tag}/bias" in golden else None
        for tc in (True, False):
            for act in (0, 2):
                want = golden[f"{tag}/gemm_tc{int(tc)}_a{act}"]
                got = O.packed_gemm(x, p, s, z, bias, bits, k, gs, act, tc, dtype)
                assert rel(got, want) <= ULP[dtype], (tag, tc, act, rel(got, want))
        wdq = OC.dequantized_weight(p, s, z, bits, k, gs)
        assert rel(OC.matmul_nt(x, wdq), x @ wdq.T) < 2e-6


def test_fused_gate_up_matches_emulator(golden):
    for bits in (2, 3, 4):
        t = f"gu_w{bits}"
        g = [golden[f"{t}/gate/{n}"] for n in ("packed", "scales", "zeros")]
        u = [golden[f"{t}/up/{n}"] for n in ("packed", "scales", "zeros")]
        for split_k in (1, 2):
            got = O.fused_gate_up(golden[f"{t}/x"], *g, *u, bits, 256, 128, split_k, "float16")
            assert rel(got, golden[f"{t}/out_s{split_k}"]) <= ULP["float16"]


def test_fused_qkv_matches_emulator(golden):
    hd = 64
    for bits in (2, 3, 4):
        t = f"qkv_w{bits}"
        x = golden[f"{t}/x"]
        prj = {n: tuple(golden[f"{t}/{n}/{f}"] for f in ("packed", "scales", "zeros", "bias")) for n in "qkv"}
        outs = O.fused_qkv(x, prj["q"], prj["k"], prj["v"], None, None, 0, 0, bits, 256, 128, 2, "float16")
        for n, o in zip("qkv", outs):
            assert rel(o, golden[f"{t}/plain_{n}"]) <= ULP["float16"], (t, n)
        perm = dict(prj)
        for n in "qk":
            order = golden[f"{t}/order_{n}"]
            assert np.array_equal(order, O.rope_row_order(prj[n][0].shape[0], hd))
            assert np.array_equal(O.unperm_index(len(order), hd), order)
            perm[n] = tuple(a[order] for a in prj[n])
        outs = O.fused_qkv(x, perm["q"], perm["k"], perm["v"], golden[f"{t}/cos"], golden[f"{t}/sin"], hd, hd,
                           bits, 256, 128, 1, "float16")
        for n, o in zip("qkv", outs):
            assert rel(o, golden[f"{t}/rope_{n}"]) <= ULP["float16"], (t, n)
        # the fused rotation equals rotate_half on the plain projections
        wq = O.dequantize(golden[f"{t}/q/unpacked"], prj["q"][1], prj["q"][2], 128)
        ref = O.apply_rope(x @ wq.T + prj["q"][3], golden[f"{t}/cos"], golden[f"{t}/sin"], hd)
        assert rel(ref, golden[f"{t}/ropecheck_q"]) < 1e-5
        assert rel(outs[0], golden[f"{t}/ropecheck_q"]) < 2e-3


def test_split_bounds_law():
    # Crispybits/Kernel/tests/test_device_logic.py:84-88
    for c in (1, 7, 128, 161):
        for p in range(1, min(c, 40) + 1):
            b = O.split_bounds(c, p)
            assert b[0][0] == 0 and b[-1][1] == c
            assert all(lo < hi for lo, hi in b) and all(b[i][1] == b[i + 1][0] for i in range(p - 1))


def test_policy_rule():
    # Crispybits/Kernel/tests/test_correctness.py:159-163
    for s, bn in ((148, 16), (108, 32)):
        assert O.candidate_split_k(1, bn * 4, bn, s, 1) == max(1, -(-s // 4))
        assert O.candidate_split_k(64, 4096, bn, s, 1) == 1
        assert O.candidate_split_k(1, 10 ** 6, bn, s, 1) == 1
