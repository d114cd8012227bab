"""Staged decode ablation of one transformer block's projections, through the public operators only.

The B200 counterpart of the reference's Crispybits/Kernel/scripts/ablation_decode.py:66-103: the same seven
stages (separate projections -> fused projections -> persistent grid -> occupancy-aware rho -> fixed Split-K ->
the policy's (split_k, rho) -> the fastest measured (split_k, rho)), each timed as one block's decode launches at
batch 1, beside the fp16 cuBLAS block.  On B200 several stages coincide by construction -- the ring kernel sizes
its own grid, so rho only chooses between one and two CTAs per SM, and the policy's split is 1 inside that
kernel's domain -- and the table says so with equal numbers instead of hiding the stages.

    python -m crispybits_kernels.ablation [--bits 3] [--iters 50]        (needs a GPU)
"""
from __future__ import annotations

import argparse
from typing import Callable, Dict, List, Tuple

import torch

from .autotune import _time, tune_gate_up, tune_gemv, tune_qkv
from .ops import PackedLinearWeight, fused_gate_up, fused_qkv, new_workspace, packed_linear
from .reference import pack_linear_dict
from .io import from_packed_dict

LLAMA2_7B = dict(hidden=4096, ffn=11008, heads=32, kv_heads=32)
SEEDS = dict(q=1, k=2, v=3, o=4, gate=5, up=6, down=7)       # seed convention of the reference's script (:18-22)


def _weight(n: int, k: int, bits: int, seed: int, device) -> Tuple[PackedLinearWeight, torch.Tensor]:
    w = torch.randn(n, k, generator=torch.Generator().manual_seed(seed)) * 0.02
    return from_packed_dict(pack_linear_dict(w, bits, 128, None, torch.float16), device, torch.float16), w.to(device).half()


def run_ablation(bits: int = 3, device="cuda", warmup: int = 5, iters: int = 50, shapes: Dict = LLAMA2_7B) -> Dict:
    H, I = shapes["hidden"], shapes["ffn"]
    hd = H // shapes["heads"]
    dims = dict(q=(shapes["heads"] * hd, H), k=(shapes["kv_heads"] * hd, H), v=(shapes["kv_heads"] * hd, H), o=(H, H),
                gate=(I, H), up=(I, H), down=(H, I))
    made = {name: _weight(n, k, bits, SEEDS[name], device) for name, (n, k) in dims.items()}
    pw = {name: m[0] for name, m in made.items()}
    dense = {name: m[1] for name, m in made.items()}
    xh = torch.randn(1, H, device=device, dtype=torch.float16)
    xi = torch.randn(1, I, device=device, dtype=torch.float16)
    ws = {name: new_workspace(device) for name in list(dims) + ["qkv", "gu"]}

    def separate(setting: Callable[[str], Tuple[int, int]]):
        for name in ("q", "k", "v", "o"):
            packed_linear(xh, pw[name], *setting(name), workspace=ws[name])
        g = packed_linear(xh, pw["gate"], *setting("gate"), workspace=ws["gate"])
        u = packed_linear(xh, pw["up"], *setting("up"), workspace=ws["up"])
        torch.nn.functional.silu(g) * u
        packed_linear(xi, pw["down"], *setting("down"), workspace=ws["down"])

    def fused(setting: Callable[[str], Tuple[int, int]]):
        fused_qkv(xh, pw["q"], pw["k"], pw["v"], *setting("qkv"), workspace=ws["qkv"])
        packed_linear(xh, pw["o"], *setting("o"), workspace=ws["o"])
        fused_gate_up(xh, pw["gate"], pw["up"], *setting("gu"), workspace=ws["gu"])
        packed_linear(xi, pw["down"], *setting("down"), workspace=ws["down"])

    def fp16_block():
        for name in ("q", "k", "v", "o"):
            torch.nn.functional.linear(xh, dense[name])
        torch.nn.functional.silu(torch.nn.functional.linear(xh, dense["gate"])) * torch.nn.functional.linear(xh, dense["up"])
        torch.nn.functional.linear(xi, dense["down"])

    def tune(name: str, exhaustive: bool = False, max_split=None):
        opts = dict(warmup=warmup, iters=max(16, iters // 2), exhaustive=exhaustive, max_split=max_split)
        if name == "qkv":
            return tune_qkv(xh, pw["q"], pw["k"], pw["v"], **opts)
        if name == "gu":
            return tune_gate_up(xh, pw["gate"], pw["up"], **opts)
        return tune_gemv(xi if name == "down" else xh, pw[name], **opts)

    t = lambda fn: _time(fn, warmup, iters)
    modules = ("qkv", "o", "gu", "down")
    rows: List[Tuple[str, float]] = [
        ("1 separate projections (rho=0, split_k=1)", t(lambda: separate(lambda n: (1, 0)))),
        ("2 + projection fusion", t(lambda: fused(lambda n: (1, 0)))),
        ("3 + persistent grid (rho=1)", t(lambda: fused(lambda n: (1, 1)))),
    ]
    best_rho = {m: tune(m, max_split=1).best.rho for m in modules}
    rows.append(("4 + occupancy-aware rho", t(lambda: fused(lambda n: (1, best_rho[n])))))
    for pk in (2, 4, 8):
        rows.append((f"5 fixed Split-K, split_k={pk}", t(lambda pk=pk: fused(lambda n: (pk, best_rho[n])))))
    reports = {m: tune(m, exhaustive=True) for m in modules}
    policy = {m: (r.best.split_k, r.best.rho) for m, r in reports.items()}
    fastest = {m: (r.oracle.split_k, r.oracle.rho) for m, r in reports.items()}
    rows.append(("6 policy (split_k, rho) per module", t(lambda: fused(lambda n: policy[n]))))
    rows.append(("7 fastest measured (split_k, rho) per module", t(lambda: fused(lambda n: fastest[n]))))
    return {"bits": bits, "rows": rows, "fp16_ms": t(fp16_block), "policy": policy, "fastest": fastest,
            "regret": {m: r.regret for m, r in reports.items()}}


def format_table(res: Dict) -> str:
    base, fp = res["rows"][0][1], res["fp16_ms"]
    lines = [f"W{res['bits']}, batch 1, one block's projections (us per block; 16 blocks captured per CUDA graph)",
             "| stage | us | vs stage 1 | vs fp16 cuBLAS |", "|---|---|---|---|"]
    for name, ms in res["rows"]:
        lines.append(f"| {name} | {ms * 1e3:.1f} | {base / ms:.2f}x | {fp / ms:.2f}x |")
    lines.append(f"| fp16 cuBLAS (dense weights) | {fp * 1e3:.1f} | {base / fp:.2f}x | 1.00x |")
    lines.append("")
    lines.append("per module (split_k, rho): policy -> fastest measured, regret of the policy")
    for m in res["policy"]:
        lines.append(f"  {m:5s} {res['policy'][m]} -> {res['fastest'][m]}   {res['regret'][m]:+.1%}")
    return "\n".join(lines)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--bits", type=int, choices=[2, 3, 4], default=3)
    ap.add_argument("--iters", type=int, default=50)
    a = ap.parse_args()
    print(format_table(run_ablation(a.bits, iters=a.iters)))
