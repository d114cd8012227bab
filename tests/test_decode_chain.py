"""Captured chains of decode launches (`-m gpu`).

Inside stream capture, back-to-back decode calls on one stream order themselves only after the earlier calls whose
operands overlap theirs; calls with disjoint operands overlap on the GPU.  Whatever the schedule, replaying the graph
must give bit for bit what the same calls give when issued one by one outside capture -- for dependent, independent
and mixed sequences, for every bit-width, and again on every replay.
"""
import ctypes

import pytest
import torch

from helpers import make

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _stats():
    from crispybits_kernels import _C
    a = (ctypes.c_longlong * 4)()
    assert _C._lib.cb_chain_stats(a) == 0
    return list(a)


def _weights(bits, n, k, count, std=0.02):
    return [make(n, k, bits, torch.float16, DEV, False, 300 + 7 * i + bits, 128, std)[0] for i in range(count)]


def _sequence(ws, x0, pattern):
    from crispybits_kernels import packed_linear
    outs, x = [], x0
    for i, w in enumerate(ws):
        if pattern == "dependent":
            x = packed_linear(x, w, 1, 1, decode_threshold=8)
            outs.append(x)
        elif pattern == "independent":
            outs.append(packed_linear(x0, w, 1, 1, decode_threshold=8))
        elif pattern == "mixed":
            if i % 3 == 2:
                outs.append(packed_linear(x0, w, 1, 1, decode_threshold=8))
            else:
                x = packed_linear(x, w, 1, 1, decode_threshold=8)
                outs.append(x)
        else:                                # "two_back": reads the output of the launch before the previous one
            src = outs[-2] if len(outs) >= 2 else x0
            outs.append(packed_linear(src, w, 1, 1, decode_threshold=8))
    return outs


def _capture_and_compare(fn, replays=12):
    from crispybits_kernels import _C
    _C.set_option(4, 0)
    try:
        eager = [y.clone() for y in fn()]
    finally:
        _C.set_option(4, 1)
    torch.cuda.synchronize()
    before = _stats()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ys = fn()
    delta = [b - a for a, b in zip(before, _stats())]
    for r in range(replays):
        g.replay()
        if r % 4 == 3 or r == 0:
            torch.cuda.synchronize()
            for i, (a, b) in enumerate(zip(eager, ys)):
                assert torch.isfinite(a.float()).all(), f"launch {i}: the test data overflowed"
                assert torch.equal(a, b), f"replay {r}, launch {i}"
    torch.cuda.synchronize()
    assert _C.decode_status() == 0
    return delta


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("B", [1, 3, 8])
@pytest.mark.parametrize("pattern", ["dependent", "independent", "mixed", "two_back"])
def test_captured_chain_replays_equal_eager_launches(bits, B, pattern):
    ws = _weights(bits, 1024, 1024, 20, std=0.03)
    x0 = torch.randn(B, 1024, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(B))
    heads, links, ordered, free = _capture_and_compare(lambda: _sequence(ws, x0, pattern))
    assert heads >= 1 and heads + links == 20 and ordered + free == links
    if pattern == "dependent":
        assert ordered == links               # every follower reads its predecessor's output
    if pattern == "independent":
        assert free == links
    if pattern == "two_back":
        assert free >= 1 and ordered >= 1     # a launch runs free when what it reads was written before the last ordered launch


@pytest.mark.parametrize("bits", [3, 4])
def test_captured_chain_at_benchmark_width(bits):
    ws = _weights(bits, 4096, 4096, 10)
    x0 = torch.randn(1, 4096, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(1))
    _capture_and_compare(lambda: _sequence(ws, x0, "dependent"), replays=8)
    _capture_and_compare(lambda: _sequence(ws, x0, "independent"), replays=8)


@pytest.mark.parametrize("B", [1, 4])
def test_captured_mlp_chain(B):
    """fused gate/up -> down projection -> fused gate/up ...: a chain of launches of different modes and shapes."""
    from crispybits_kernels import fused_gate_up, packed_linear
    d, f, bits = 1024, 2816, 3
    gate = make(f, d, bits, torch.float16, DEV, False, 401, 128, 0.02)[0]
    up = make(f, d, bits, torch.float16, DEV, False, 402, 128, 0.02)[0]
    down = make(d, f, bits, torch.float16, DEV, False, 403, 128, 0.02)[0]
    x0 = torch.randn(B, d, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(9))

    def mlp():
        outs, x = [], x0
        for _ in range(4):
            h = fused_gate_up(x, gate, up, 1, 1, decode_threshold=8)
            x = packed_linear(h, down, 1, 1, decode_threshold=8)
            outs += [h, x]
        return outs

    heads, links, ordered, _ = _capture_and_compare(mlp)
    assert heads + links == 8 and ordered == links


def test_chain_is_broken_by_other_work_and_by_split_k():
    """A torch kernel between two decode calls ends the chain (the next call starts a new one); launches that share the
    Split-K scratch are ordered one after the other."""
    from crispybits_kernels import packed_linear
    ws = _weights(4, 1024, 1024, 6, std=0.03)
    x0 = torch.randn(2, 1024, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(3))

    def broken():
        outs, x = [], x0
        for i, w in enumerate(ws):
            x = packed_linear(x, w, 1, 1, decode_threshold=8)
            if i % 2 == 1:
                x = x * 0.5                       # a kernel of another library
            outs.append(x)
        return outs

    heads, links, _, _ = _capture_and_compare(broken)
    assert heads == 3 and links == 3

    def split():
        return [packed_linear(x0, w, 4, 1, decode_threshold=8) for w in ws]

    heads, links, ordered, free = _capture_and_compare(split)
    assert heads + links == 6 and ordered == links and free == 0


def test_long_independent_run_is_interrupted_by_an_ordered_launch():
    """More free launches in a row than the host keeps operand records for: the chain inserts an ordered launch."""
    ws = _weights(4, 512, 512, 6, std=0.03)
    x0 = torch.randn(1, 512, device=DEV, dtype=torch.float16, generator=torch.Generator(DEV).manual_seed(5))
    from crispybits_kernels import packed_linear
    heads, links, ordered, free = _capture_and_compare(
        lambda: [packed_linear(x0, ws[i % 6], 1, 1) for i in range(140)], replays=4)
    assert heads + links == 140 and ordered >= 2 and free >= 120
