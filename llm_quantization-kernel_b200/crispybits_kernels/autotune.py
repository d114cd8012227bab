"""Timing-based choice of (rho, split_k) per decode operator.

Mirrors Crispybits/Kernel/crispybits_kernels/autotune.py: for every occupancy level rho in
1..max_rho the policy's split_k is timed; optionally an exhaustive grid of split factors is timed too
so that the policy's regret against the best measured point can be reported.  The candidate grid
was re-chosen for 148 SMs and 16-row tiles (the reference's grid targets 108 SMs and 32-row tiles).
"""
from __future__ import annotations

import time
from dataclasses import asdict, dataclass
from math import ceil
from typing import Callable, Dict, List, Optional

import torch

from .ops import (BATCH_BLOCK, PackedLinear, PackedLinearWeight, balanced_split_k, candidate_split_k,
                  fused_gate_up, fused_qkv, max_rho, new_workspace, packed_linear, sm_count, tile_n,
                  virtual_rows)

# split factors tried by an exhaustive sweep
EXHAUSTIVE_PK = (1, 2, 3, 4, 5, 6, 8, 10, 12, 16, 20, 24, 32)


@dataclass
class TuneResult:
    rho: int
    split_k: int
    ms: float
    c_out: int
    c_target: int
    policy: bool = True   # produced by the policy rule (as opposed to the exhaustive grid)


@dataclass
class TuneReport:
    best: TuneResult      # fastest point the policy can produce
    oracle: TuneResult    # fastest point measured at all
    results: List[TuneResult]

    @property
    def regret(self) -> float:
        return self.best.ms / self.oracle.ms - 1.0


GRAPH_REPS = 16     # calls captured into one CUDA graph when timing on a GPU


def _time(fn: Callable[[], object], warmup: int, iters: int) -> float:
    """Milliseconds per call.  On a GPU the call is captured GRAPH_REPS times into a CUDA graph and the graph is
    replayed, timed with CUDA events on the current stream: a decode launch is a few microseconds, far below the
    cost of issuing it from Python, so eager timing would measure the host.  Falls back to eager CUDA-event
    timing if the capture fails, and to the wall clock without a GPU."""
    for _ in range(warmup):
        fn()
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        torch.cuda.synchronize()
        graph, reps = None, 1
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                keep = [fn() for _ in range(GRAPH_REPS)]
            reps = GRAPH_REPS
            graph.replay()
            torch.cuda.synchronize()
        except Exception:
            graph, reps = None, 1
            torch.cuda.synchronize()
        rounds = max(1, iters // reps)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(rounds):
            if graph is not None:
                graph.replay()
            else:
                fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / (rounds * reps)
    start = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - start) * 1e3 / iters


def _tune(run: Callable[[int, int], object], B: int, V: int, K: int, bits: int, kind: str,
          warmup: int, iters: int, max_split: Optional[int], exhaustive: bool = False) -> TuneReport:
    sms, bn = sm_count(), tile_n()
    levels = max(1, max_rho(bits, kind))
    nchunks = ceil(K / 32)
    c_out = ceil(B / BATCH_BLOCK) * ceil(V / bn)
    results: List[TuneResult] = []
    index: Dict[tuple, TuneResult] = {}

    def measure(rho: int, split: int, from_policy: bool):
        split = max(1, min(split, nchunks))
        if max_split is not None:
            split = min(split, max_split)
        key = (split, min(c_out * split, rho * sms))       # same grid and split = same launch
        hit = index.get(key)
        if hit is not None:
            hit.policy = hit.policy or from_policy
            return
        ms = _time(lambda: run(split, rho), warmup, iters)
        index[key] = TuneResult(rho, split, ms, c_out, rho * sms, from_policy)
        results.append(index[key])

    for rho in range(1, levels + 1):
        measure(rho, candidate_split_k(ceil(B / BATCH_BLOCK), V, bn, sms, rho, max_split), True)
        measure(rho, balanced_split_k(B, V, bn, sms, rho, nchunks), True)
        measure(rho, 1, True)      # what ops._resolve picks inside the fp16 ring kernel's domain
    if exhaustive:
        for rho in range(1, levels + 1):
            for split in EXHAUSTIVE_PK:
                if max_split is None or split <= max_split:
                    measure(rho, split, False)
    best = min((r for r in results if r.policy), key=lambda r: r.ms)
    oracle = min(results, key=lambda r: r.ms)
    return TuneReport(best, oracle, results)


def _batch(x) -> int:
    return x.reshape(-1, x.shape[-1]).shape[0]


def tune_gemv(x: torch.Tensor, w: PackedLinearWeight, warmup: int = 10, iters: int = 50,
              max_split: Optional[int] = None, act: Optional[str] = None, exhaustive: bool = False) -> TuneReport:
    ws = new_workspace(x.device)
    return _tune(lambda pk, rho: packed_linear(x, w, pk, rho, act, workspace=ws), _batch(x),
                 virtual_rows("gemv", w.out_features), w.in_features, w.bits, "gemv",
                 warmup, iters, max_split, exhaustive)


def tune_qkv(x, q: PackedLinearWeight, k: PackedLinearWeight, v: PackedLinearWeight,
             warmup: int = 10, iters: int = 50, max_split: Optional[int] = None,
             exhaustive: bool = False) -> TuneReport:
    ws = new_workspace(x.device)
    rows = virtual_rows("qkv", q.out_features, k.out_features, v.out_features)
    return _tune(lambda pk, rho: fused_qkv(x, q, k, v, pk, rho, workspace=ws), _batch(x), rows,
                 q.in_features, q.bits, "qkv", warmup, iters, max_split, exhaustive)


def tune_gate_up(x, gate: PackedLinearWeight, up: PackedLinearWeight, warmup: int = 10, iters: int = 50,
                 max_split: Optional[int] = None, exhaustive: bool = False) -> TuneReport:
    ws = new_workspace(x.device)
    return _tune(lambda pk, rho: fused_gate_up(x, gate, up, pk, rho, workspace=ws), _batch(x),
                 virtual_rows("gate_up", gate.out_features), gate.in_features, gate.bits, "gate_up",
                 warmup, iters, max_split, exhaustive)


@torch.no_grad()
def tune_model(model: torch.nn.Module, batch: int = 1, warmup: int = 10, iters: int = 50,
               max_split: Optional[int] = None, dtype=torch.float16, verbose: bool = False,
               exhaustive: bool = False) -> Dict[str, Dict]:
    """Tune every packed operator of an installed model (identical shapes are measured once), write the
    chosen (split_k, rho) into the modules and return {"block.i.<name>": {"split_k", "rho"}}."""
    from .integration import FusedLlamaMLP, FusedQKV, _blocks
    memo: Dict[tuple, TuneReport] = {}
    tuning: Dict[str, Dict] = {}
    opts = dict(warmup=warmup, iters=iters, max_split=max_split, exhaustive=exhaustive)

    def probe(k_in, device):
        return torch.randn(batch, k_in, device=device, dtype=dtype)

    def best_of(key, make) -> TuneResult:
        if key not in memo:
            memo[key] = make()
        return memo[key].best

    def apply(mod, entry, r: TuneResult):
        mod.split_k, mod.rho = r.split_k, r.rho
        tuning[entry] = {"split_k": r.split_k, "rho": r.rho}

    for i, block in enumerate(_blocks(model)):
        fused_children = set()
        for m in block.modules():
            if isinstance(m, FusedQKV):
                fused_children |= {id(m.q), id(m.k), id(m.v)}
            elif isinstance(m, FusedLlamaMLP):
                fused_children |= {id(m.gate_proj), id(m.up_proj)}
        for name, mod in block.named_modules():
            if isinstance(mod, FusedQKV):
                q, k, v = (m.weight_spec() for m in (mod.q, mod.k, mod.v))
                key = ("qkv", q.bits, q.in_features, q.out_features, k.out_features, v.out_features)
                apply(mod, f"block.{i}.self_attn.qkv",
                      best_of(key, lambda: tune_qkv(probe(q.in_features, q.packed.device), q, k, v, **opts)))
            elif isinstance(mod, FusedLlamaMLP):
                g, u = mod.gate_proj.weight_spec(), mod.up_proj.weight_spec()
                key = ("gate_up", g.bits, g.in_features, g.out_features)
                apply(mod, f"block.{i}.mlp.gate_up",
                      best_of(key, lambda: tune_gate_up(probe(g.in_features, g.packed.device), g, u, **opts)))
            elif isinstance(mod, PackedLinear) and id(mod) not in fused_children:
                w = mod.weight_spec()
                key = ("gemv", w.bits, w.in_features, w.out_features, w.bias is not None, mod.act)
                apply(mod, f"block.{i}.{name}",
                      best_of(key, lambda: tune_gemv(probe(w.in_features, w.packed.device), w, act=mod.act, **opts)))
        if verbose:
            print(f"block {i} tuned")
    if verbose:
        for key, rep in memo.items():
            print(key, "best", asdict(rep.best), "oracle", asdict(rep.oracle), f"regret {rep.regret:+.1%}")
    return tuning
