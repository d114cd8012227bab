"""The autotuner and the staged ablation on a GPU (`-m gpu`): the exhaustive (rho, split_k) sweep of each decode
operator (Crispybits/Kernel/crispybits_kernels/autotune.py:55-169) and the seven-stage block ablation
(Crispybits/Kernel/scripts/ablation_decode.py:66-103), through the public operators."""
import pytest
import torch

from helpers import make, ref_linear, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check_report(rep):
    assert rep.regret >= 0.0
    policy = [r for r in rep.results if r.policy]
    assert policy and all(rep.best.ms <= r.ms for r in policy)
    assert all(rep.oracle.ms <= r.ms for r in rep.results)
    assert len({(r.rho, r.split_k) for r in rep.results}) == len(rep.results)
    assert any(not r.policy for r in rep.results)          # the exhaustive grid added points the policy never picks


@pytest.mark.parametrize("bits", [2, 4])
def test_tune_gemv_exhaustive(bits):
    from crispybits_kernels import packed_linear
    from crispybits_kernels.autotune import tune_gemv
    w, wd, _ = make(1024, 2048, bits, torch.float16, DEV, False, 3, 128, 0.02)
    x = torch.randn(1, 2048, device=DEV, dtype=torch.float16)
    rep = tune_gemv(x, w, warmup=2, iters=32, exhaustive=True)
    _check_report(rep)
    for r in (rep.best, rep.oracle):                      # the chosen points give the oracle-checked result
        assert rel_err(packed_linear(x, w, r.split_k, r.rho), ref_linear(x, wd)) < 2e-3


def test_tune_qkv_and_gate_up_exhaustive():
    from crispybits_kernels import fused_gate_up, fused_qkv
    from crispybits_kernels.autotune import tune_gate_up, tune_qkv
    q, qd, _ = make(1024, 1024, 3, torch.float16, DEV, False, 1, 128, 0.02)
    k, kd, _ = make(256, 1024, 3, torch.float16, DEV, False, 2, 128, 0.02)
    v, vd, _ = make(256, 1024, 3, torch.float16, DEV, False, 3, 128, 0.02)
    x = torch.randn(2, 1024, device=DEV, dtype=torch.float16)
    rep = tune_qkv(x, q, k, v, warmup=2, iters=32, exhaustive=True)
    _check_report(rep)
    for o, d in zip(fused_qkv(x, q, k, v, rep.oracle.split_k, rep.oracle.rho), (qd, kd, vd)):
        assert rel_err(o, ref_linear(x, d)) < 2e-3
    g, gd, _ = make(1408, 1024, 3, torch.float16, DEV, False, 5, 128, 0.02)
    u, ud, _ = make(1408, 1024, 3, torch.float16, DEV, False, 6, 128, 0.02)
    rep = tune_gate_up(x, g, u, warmup=2, iters=32, exhaustive=True)
    _check_report(rep)
    ref = torch.nn.functional.silu(x.float() @ gd.T) * (x.float() @ ud.T)
    assert rel_err(fused_gate_up(x, g, u, rep.oracle.split_k, rep.oracle.rho), ref) < 2e-3


def test_staged_ablation_runs_on_a_small_block():
    from crispybits_kernels.ablation import format_table, run_ablation
    res = run_ablation(3, DEV, warmup=1, iters=16, shapes=dict(hidden=1024, ffn=2816, heads=8, kv_heads=8))
    names = [n for n, _ in res["rows"]]
    assert len(names) == 9 and names[0].startswith("1 ") and names[-1].startswith("7 ")
    assert all(ms > 0 for _, ms in res["rows"]) and res["fp16_ms"] > 0
    assert res["rows"][-1][1] <= 1.5 * min(ms for _, ms in res["rows"])      # the fastest points are (about) fastest
    assert all(v >= 0 for v in res["regret"].values())
    assert "| 7 fastest measured" in format_table(res)
