#!/usr/bin/env python3
"""Benchmark of the packed W2/W3/W4 linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload gemv|stack]

Prints ONE JSON line.  Workload at N=1 (`gemv`): batch-1 decode GEMVs over 4096x4096 group-128 weights
at W4, W3 and W2 -- the shapes the headline metric is quoted on.  A step is one pass over COPIES
distinct weight matrices per bit-width (3*COPIES launches); the matrices of one step add up to more
than twice the 126 MB L2, so every launch streams its weights from HBM.  `value` is the algorithmic
bytes of all launches divided by the device time of the timed steps (CUDA events on the launching
stream around CUDA-graph replays of a step, so Python launch overhead is not in the number).  `e2e`
times the same GEMVs through the public API with the activations starting in pinned host memory and
the result read back to the host every call.  `roofline` describes the dominant kernel (the W4 GEMV):
algorithmic bytes per launch over its average launch duration, against the measured HBM copy
bandwidth in MEASURED_PEAKS.json.  `cpu_baseline` is the C oracle (OpenMP, all host threads) timed on
a bounded sample of the same GEMVs on the host cores.

`--impl reference` times only that CPU implementation and prints the same line shape with
"impl": "reference".

Algorithmic bytes per GEMV: N*ceil(K/32)*bits*4 (packed) + N*ceil(K/128)*2*2 (fp16 scales and zeros)
+ B*K*2 (x) + B*N*2 (y), weights counted once for any batch.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "llm_quantization-kernel_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

N_OUT, K_IN, GROUP = 4096, 4096, 128
BITS = (4, 3, 2)
COPIES = 48                 # distinct weight matrices per bit-width and step (about 1 GB in all)
E2E_STREAMS = 5             # streams the end-to-end step is pipelined over
FALLBACK_HBM_GBS = 6650.0   # earlier measurement on this pool, used only without MEASURED_PEAKS.json
FALLBACK_TFLOPS = 1590.0
METRIC = "packed W2/3/4 decode GEMV effective HBM bandwidth (4096x4096, group 128, batch 1)"
COMM_TEXT = {
    "nccl": "NCCL all-gather after each launch",
    "p2p": "all-gather fused into the decode kernel: peer stores over NVLink and an in-kernel rank hand-shake",
    "p2p_barrier": "all-gather fused into the decode kernel's epilogue as peer stores over NVLink, "
                   "one-CTA flag barrier kernel (programmatic dependent launch) after each launch",
}
METRIC_STACK = "packed mixed-precision decode stack effective HBM bandwidth (Llama-2-7B shapes, 32 blocks)"
# dram__bytes_read + dram__bytes_write per W4 4096x4096 launch, from the ncu capture summarised under profiles/
NCU_TRAFFIC_W4 = 8958464


def gemv_bytes(n, k, bits, batch=1, group=GROUP):
    return n * -(-k // 32) * bits * 4 + n * -(-k // group) * 4 + batch * k * 2 + batch * n * 2


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_TFLOPS, "fallback"


# ------------------------------------------------------------------ synthetic inputs
def synth_weight_numpy(bits, seed, n=N_OUT, k=K_IN):
    """W ~ N(0, 0.02) from a seeded CPU generator, quantised and packed by the oracle (test infrastructure,
    used here only to PRODUCE inputs and as the CPU baseline)."""
    from oracle import cb_oracle_c as OC
    from oracle import cb_oracle as O
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).numpy()
    q, s, z = OC.quantize_affine(w, bits, GROUP)
    return dict(packed=OC.pack_codes(q, bits), scales=O.round_to(s, "float16"), zeros=O.round_to(z, "float16"),
                bits=bits, group_size=GROUP, in_features=k, out_features=n, bias=None)


def device_copies(d, device, copies):
    """`copies` distinct device matrices with the statistics of `d`: the first is d itself, the others are
    row rotations of it (different addresses and contents, same value distribution)."""
    from crispybits_kernels import PackedLinearWeight
    p = torch.from_numpy(d["packed"]).to(device)
    s = torch.from_numpy(d["scales"]).to(device=device, dtype=torch.float16)
    z = torch.from_numpy(d["zeros"]).to(device=device, dtype=torch.float16)
    out = []
    for c in range(copies):
        sh = 97 * c
        out.append(PackedLinearWeight(torch.roll(p, sh, 0).contiguous(), torch.roll(s, sh, 0).contiguous(),
                                      torch.roll(z, sh, 0).contiguous(), d["bits"], GROUP, d["in_features"],
                                      d["out_features"]))
    return out


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read-only NVML
    queries from a background thread every ~2 ms; falls back to an `nvidia-smi -lms` child process)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.path = gpu_index, None, None
        self.thread, self.stop_flag, self.samples, self.mask, self.max_mhz = None, False, [], 0, None

    def _nvml_loop(self, handle, nv):
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(handle))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
                handle = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                handle = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(handle, nv), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            if self.samples:
                out.update(sm_mhz=float(statistics.median(self.samples)), sm_max_mhz=self.max_mhz,
                           reasons=sorted(n for bit, n in self.REASONS.items() if self.mask & bit),
                           samples=len(self.samples), source="nvml")
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       source="nvidia-smi")
        return out


# ------------------------------------------------------------------ CPU arm
def cpu_gemv_sample(seconds_per_bits=3.0, min_iters=3, copies=2):
    """Time the C oracle's decode GEMV (OpenMP over output rows, all host threads) on the benchmark's
    three 4096x4096 matrices.  Returns (GB/s over the sample, per-bits ms, threads, description)."""
    from oracle import cb_oracle_c as OC
    threads = OC.num_threads()
    g = torch.Generator().manual_seed(123)
    x = torch.randn(1, K_IN, generator=g).half().float().numpy()
    total_bytes, total_s, per = 0, 0.0, {}
    for bits in BITS:
        ws = [synth_weight_numpy(bits, 10 * bits + c) for c in range(copies)]
        OC.gemv(x, ws[0]["packed"], ws[0]["scales"], ws[0]["zeros"], bits, K_IN, GROUP, 1)   # warm-up
        it, t0 = 0, time.perf_counter()
        while it < min_iters or time.perf_counter() - t0 < seconds_per_bits:
            d = ws[it % copies]
            OC.gemv(x, d["packed"], d["scales"], d["zeros"], bits, K_IN, GROUP, 1)
            it += 1
        dt = time.perf_counter() - t0
        per[f"w{bits}_ms"] = dt / it * 1e3
        total_bytes += it * gemv_bytes(N_OUT, K_IN, bits)
        total_s += dt
    sample = (f"C oracle cbo_gemv (OpenMP, {threads} threads), 4096x4096 batch-1 GEMV at W4/W3/W2, "
              f"{copies} matrices per bit-width, >= {seconds_per_bits:.0f} s per bit-width")
    return total_bytes / total_s / 1e9, per, threads, sample


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    per_step = max(0.5, min(3.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_gemv_sample(per_step / 3, 1)
    vals, pers = [], []
    for _ in range(args.steps):
        v, per, threads, sample = cpu_gemv_sample(per_step / 3, 1)
        vals.append(v); pers.append(per)
    value = float(np.mean(vals))
    wall = time.perf_counter() - t0
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemv_4096x4096_w4_w3_w2_b1", "group_size": GROUP,
                   "note": "CPU implementation of the reference's decode arithmetic on the host cores"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "per_bits_ms": {k: float(np.mean([p[k] for p in pers])) for k in pers[0]},
        "gpu_launches": 0, "wall_s": wall,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ GPU arm: GEMV workload
def timed_graph_replays(graphs, steps, warmup, barrier):
    """Replay each graph once per step; returns per-graph total ms over the timed steps and total ms."""
    for _ in range(warmup):
        for g in graphs:
            g.replay()
    barrier()
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(graphs) + 1)] for _ in range(steps)]
    for s in range(steps):
        ev[s][0].record()
        for i, g in enumerate(graphs):
            g.replay()
            ev[s][i + 1].record()
    torch.cuda.synchronize()
    barrier()
    per = [sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(steps)) for i in range(len(graphs))]
    total = ev[0][0].elapsed_time(ev[steps - 1][len(graphs)])
    return per, total


def run_gemv_workload(args, rank, world, device, barrier, reduce_max):
    import crispybits_kernels as ck
    from crispybits_kernels import ops
    if ops._CUDA is None:
        raise RuntimeError(f"native library not loaded: {ops._IMPORT_ERROR}")
    hbm_peak, tf_peak, peak_kind = peaks()
    weights = {b: device_copies(synth_weight_numpy(b, b), device, COPIES) for b in BITS}
    g = torch.Generator().manual_seed(1)
    x_host = torch.randn(1, K_IN, generator=g).half().pin_memory()
    x = x_host.to(device)
    ws = ck.new_workspace(device)

    # correctness gate before timing (the reference's benchmark does the same, scripts/bench_gemv.py:22-24)
    from oracle import cb_oracle as O
    for b in BITS:
        d = synth_weight_numpy(b, b)
        ref = x_host.float().numpy() @ O.dequantized_weight(d).T
        y = ck.packed_linear(x, weights[b][0], workspace=ws).float().cpu().numpy()
        err = float(np.abs(y - ref).max() / np.abs(ref).max())
        assert err < 2e-3, f"W{b} GEMV off by {err:.2e}; not timing"

    # one CUDA graph per bit-width: COPIES back-to-back GEMVs over distinct matrices
    side = torch.cuda.Stream(device)
    graphs, outs = [], []
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for b in BITS:
            for w in weights[b]:
                ck.packed_linear(x, w, workspace=ws)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for b in BITS:
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            outs.append([ck.packed_linear(x, w, workspace=ws) for w in weights[b]])
        graphs.append(gr)

    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    per_ms, total_ms = timed_graph_replays(graphs, args.steps, max(3, args.warmup), barrier)
    clocks = sampler.stop() if rank == 0 else {}
    total_ms = reduce_max(total_ms)
    per_ms = [reduce_max(v) for v in per_ms]

    step_bytes = sum(COPIES * gemv_bytes(N_OUT, K_IN, b) for b in BITS)
    value = world * step_bytes * args.steps / (total_ms * 1e-3) / 1e9
    gemv = {}
    for b, ms in zip(BITS, per_ms):
        us = ms * 1e3 / (args.steps * COPIES)
        gbs = gemv_bytes(N_OUT, K_IN, b) / (us * 1e-6) / 1e9
        gemv[f"w{b}"] = {"us": us, "gbs": gbs, "frac_of_hbm_peak": gbs / hbm_peak,
                         "split_k": ops._resolve(None, 1, 1, N_OUT, K_IN, torch.device(device))}
    top = gemv["w4"]
    roofline = {"bound": "hbm", "achieved": top["gbs"], "peak": hbm_peak, "unit": "GB/s",
                "frac": top["gbs"] / hbm_peak, "traffic": NCU_TRAFFIC_W4, "kernel": "decode GEMV W4 4096x4096 b1",
                "algorithmic_bytes_per_launch": gemv_bytes(N_OUT, K_IN, 4), "peak_kind": f"of {peak_kind}"}

    # end to end: activations start in pinned host memory, results are read back, every call
    y_host = torch.empty(1, N_OUT, dtype=torch.float16).pin_memory()

    def e2e_step():
        for b in BITS:
            for w in weights[b]:
                xd = x_host.to(device, non_blocking=True)
                y = ck.packed_linear(xd, w, workspace=ws)
                y_host.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    def time_e2e(step):
        for _ in range(3):
            step()
        barrier()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        return reduce_max(max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3))

    eager_ms = time_e2e(e2e_step)
    # The same calls the way a serving loop issues them: the step -- every host-to-device copy, every packed_linear
    # call and every read-back -- is captured once into a CUDA graph (the reference tests capture of its operators,
    # tests/test_correctness.py:178-191) and replayed; the copies still run, from and to the same pinned buffers, on
    # every replay.  Eager issue of the same step is reported beside it: there the Python call path is the bound.
    graph_ms = None
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            e2e_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for b in BITS:
                for w in weights[b]:
                    xd = x_host.to(device, non_blocking=True)
                    y = ck.packed_linear(xd, w, workspace=ws)
                    y_host.copy_(y, non_blocking=True)

        def graph_step():
            g.replay()
            torch.cuda.synchronize()

        graph_ms = time_e2e(graph_step)
    except Exception as exc:       # capture of pinned copies is not available everywhere: keep the eager figure
        print(f"[bench] e2e graph capture failed: {type(exc).__name__}: {exc}", file=sys.stderr)
        torch.cuda.synchronize()
    # The calls of a step are independent of one another, so a serving loop can pipeline them: the same step captured
    # over E2E_STREAMS streams (call i on stream i mod E2E_STREAMS, each call with its own pinned result row and each
    # stream with its own workspace), so that the copies of one call overlap the kernels of others.  Every copy still
    # runs on every replay.
    piped_ms = None
    if graph_ms is not None:
        try:
            streams = [torch.cuda.Stream(device) for _ in range(E2E_STREAMS)]
            wss = [ck.new_workspace(torch.device(device)) for _ in range(E2E_STREAMS)]
            y_rows = torch.empty(len(BITS) * COPIES, N_OUT, dtype=torch.float16).pin_memory()

            def piped_issue():
                cur = torch.cuda.current_stream()
                for st in streams:
                    st.wait_stream(cur)
                i = 0
                for b in BITS:
                    for w in weights[b]:
                        with torch.cuda.stream(streams[i % E2E_STREAMS]):
                            xd = x_host.to(device, non_blocking=True)
                            y = ck.packed_linear(xd, w, workspace=wss[i % E2E_STREAMS])
                            y_rows[i:i + 1].copy_(y, non_blocking=True)
                        i += 1
                for st in streams:
                    cur.wait_stream(st)

            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                piped_issue()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            serial_last = y_host.clone()
            gp = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gp):
                piped_issue()

            def piped_step():
                gp.replay()
                torch.cuda.synchronize()

            piped_step()
            if not torch.equal(y_rows[-1:], serial_last):
                raise RuntimeError("pipelined step disagrees with the serial one")
            piped_ms = time_e2e(piped_step)
        except Exception as exc:
            print(f"[bench] pipelined e2e capture failed: {type(exc).__name__}: {exc}", file=sys.stderr)
            torch.cuda.synchronize()
    e2e_ms = min(m for m in (piped_ms, graph_ms, eager_ms) if m is not None)
    gbs = lambda ms: world * step_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e = {"value": gbs(e2e_ms), "unit": "GB/s",
           "h2d_bytes_per_step": 3 * COPIES * K_IN * 2, "d2h_bytes_per_step": 3 * COPIES * N_OUT * 2,
           "eager_value": gbs(eager_ms),
           "one_stream_graph_value": None if graph_ms is None else gbs(graph_ms),
           "pipelined_graph_value": None if piped_ms is None else gbs(piped_ms),
           "api": "crispybits_kernels.packed_linear; per call x is copied from pinned host memory and y copied back to "
                  "pinned host memory; packed weights resident on the device as in install_bitmap; "
                  + (f"the step's calls and copies are captured in a CUDA graph over {E2E_STREAMS} streams (the calls "
                     "of a step are independent, so the copies of one overlap the kernels of others) and replayed "
                     "(one_stream_graph_value: the same step captured on one stream; eager_value: issued call by call "
                     "from Python)" if piped_ms is not None and piped_ms <= e2e_ms else
                     "the step's calls and copies are captured in a CUDA graph and replayed (eager_value: the same "
                     "step issued call by call from Python)" if graph_ms is not None else "issued call by call from Python")}

    extra = {}
    if rank == 0 and not args.no_gemm:
        extra["gemm"] = bench_gemm(device, tf_peak, peak_kind)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, per, threads, sample = cpu_gemv_sample()
        cpu = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample, **per}

    return {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemv_4096x4096_w4_w3_w2_b1", "group_size": GROUP, "copies_per_bits": COPIES,
                   "l2": f"inputs larger than L2: each step streams {step_bytes / 1e6:.0f} MB of distinct weights "
                         f"(126 MB L2)", "launch": "CUDA graph replay, one graph per bit-width",
                   "multi_gpu": "independent replicas (single matmuls stay on one GPU)" if world > 1 else "n/a"},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gemv": gemv, "clocks": clocks,
        "gpu_launches": args.steps * 3 * COPIES, **extra,
    }


# ------------------------------------------------------------------ GPU arm: decode stack workload
def run_stack_workload(args, rank, world, device, barrier, reduce_max, sub=False):
    """One step = the 128 packed decode launches of a Llama-2-7B-shaped 32-block stack (per-block bit-widths
    from the seeded {2,3,4} draw), column-parallel over `world` GPUs with an all-gather after each launch."""
    import crispybits_kernels as ck
    from crispybits_kernels.stack import DecodeStack
    hbm_peak, _, peak_kind = peaks()
    batch = args.batch
    st = DecodeStack(rank=rank, world=world, device=device, comm=args.comm)
    g = torch.Generator().manual_seed(2)
    x_host = torch.randn(batch, st.d_model, generator=g).half().pin_memory()
    x = x_host.to(device)
    comm_note = None
    try:
        for _ in range(2):
            y = st.step(x)
        torch.cuda.synchronize()
        ok = 1.0
    except Exception as exc:      # e.g. peer-mapped memory cannot be set up on this box
        comm_note = f"{type(exc).__name__}: {exc}"[:200]
        ok = 0.0
    if world > 1 and st.comm != "nccl":
        # every rank must take the same path: if the peer-memory set-up failed anywhere, all ranks use NCCL, and the
        # line says so
        all_ok = -reduce_max(-ok)
        if all_ok < 1.0:
            print(f"[bench] rank {rank}: peer-store gather unavailable ({comm_note}); using the NCCL gather", file=sys.stderr)
            st.comm = "nccl"
            comm_note = comm_note or "peer set-up failed on another rank"
            for _ in range(2):
                y = st.step(x)
            torch.cuda.synchronize()
        else:
            comm_note = None
    elif ok < 1.0:
        raise RuntimeError(comm_note)
    assert torch.isfinite(y.float()).all(), "decode stack produced non-finite values"
    graph, mode = None, "eager launches"
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            st.step(x)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y = st.step(x)
        graph.replay()
        torch.cuda.synchronize()
        mode = "CUDA graph replay of the whole step"
    except Exception as exc:   # NCCL inside a capture is not available everywhere: time eager launches instead
        graph = None
        mode = f"eager launches (graph capture failed: {type(exc).__name__})"
        torch.cuda.synchronize()

    def one_step():
        if graph is not None:
            graph.replay()
        else:
            st.step(x)

    warm = max(3, args.warmup)
    for _ in range(warm):
        one_step()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0 and not sub:
        sampler.start()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        one_step()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop() if (rank == 0 and not sub) else {}
    total_ms = reduce_max(e0.elapsed_time(e1))
    my_bytes = st.algorithmic_bytes(batch)
    all_bytes = reduce_sum(float(my_bytes)) if world > 1 else float(my_bytes)
    value = all_bytes * args.steps / (total_ms * 1e-3) / 1e9

    if st.peer_status() != 0:
        raise RuntimeError(f"rank {rank}: peer {st.peer_status() - 1} was not heard from in time")
    y_host = torch.empty(batch, st.d_model, dtype=torch.float16).pin_memory()

    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        one_step()
        y_host.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_ms = reduce_max((time.perf_counter() - t0) * 1e3)
    res = {
        "metric": METRIC_STACK, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": total_ms / args.steps, "us_per_launch": total_ms * 1e3 / args.steps / st.launches_per_step(),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "decode_stack_llama2_7b_32blocks", "batch": batch, "bitmap_seed": 0,
                   "mean_bits": float(np.mean(st.bitmap)), "parallelism": (f"column-parallel N over {world} GPUs, " + COMM_TEXT[st.comm]
                                   + (f" [requested {args.comm}: {comm_note}]" if comm_note else "")) if world > 1 else "single GPU",
                   "l2": f"inputs larger than L2: {my_bytes / 1e6:.0f} MB of weights per rank and step", "launch": mode},
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": hbm_peak, "unit": "GB/s",
                     "frac": value / world / hbm_peak, "traffic": None, "kernel": "decode step, per GPU",
                     "algorithmic_bytes_per_launch": my_bytes / st.launches_per_step(), "peak_kind": f"of {peak_kind}"},
        "e2e": {"value": all_bytes * args.steps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": batch * st.d_model * 2, "d2h_bytes_per_step": batch * st.d_model * 2,
                "api": "DecodeStack.step: hidden state from pinned host memory, result copied back, every step"},
        "cpu_baseline": None, "clocks": clocks, "gpu_launches": args.steps * st.launches_per_step(),
    }
    del st
    torch.cuda.empty_cache()
    return res


_REDUCE_SUM = [None]


def reduce_sum(v):
    return _REDUCE_SUM[0](v) if _REDUCE_SUM[0] is not None else float(v)


def _graph_timed_us(call, iters):
    """Microseconds per call of `call(i)`: `iters` calls captured in one CUDA graph and replayed three times between
    CUDA events (the host-side cost of a call -- Python, ctypes, tensor-map encoding -- is comparable to a 40 us
    kernel and would otherwise be part of the figure); issued eagerly if the capture fails."""
    for i in range(3):
        call(i)
    torch.cuda.synchronize()
    replay = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            call(0)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                call(i)
        replay = g.replay
    except Exception as exc:
        print(f"[bench] gemm graph capture failed: {type(exc).__name__}: {exc}", file=sys.stderr)
        torch.cuda.synchronize()
    reps = 3
    if replay is not None:
        replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        if replay is not None:
            replay()
        else:
            for i in range(iters):
                call(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * reps)


def bench_gemm(device, tf_peak, peak_kind, m=1024, iters=10):
    """Prefill GEMM at M=1024 (TFLOP/s = 2*M*N*K / t): the 4096x4096 matrix at W4 and W3, and at W4 the other
    three (N, K) shapes of the prefill configuration."""
    import crispybits_kernels as ck
    out = {}
    for (n, k, b) in ((N_OUT, K_IN, 4), (N_OUT, K_IN, 3), (12288, 4096, 4), (22016, 4096, 4), (4096, 11008, 4)):
        x = torch.randn(m, k, device=device, dtype=torch.float16, generator=torch.Generator(device).manual_seed(5))
        ws = device_copies(synth_weight_numpy(b, b, n, k), device, 2)
        us = _graph_timed_us(lambda i: ck.packed_linear(x, ws[i % 2]), iters)
        tf = 2.0 * m * n * k / (us * 1e-6) / 1e12
        out[f"m{m}_{n}x{k}_w{b}"] = {"us": us, "tflops": tf, "frac_of_dense_peak": tf / tf_peak,
                                     "peak_kind": f"of {peak_kind}"}
        del ws, x

    # the fused forms: gate/up (silu(g) * u in the epilogue) and Q/K/V (bias-free, RoPE and un-permuted stores in
    # the epilogue), both at K = 4096; FLOPs are those of the projections alone
    def timed(fn, flops):
        us = _graph_timed_us(lambda i: fn(), iters)
        tf = flops / (us * 1e-6) / 1e12
        return {"us": us, "tflops": tf, "frac_of_dense_peak": tf / tf_peak, "peak_kind": f"of {peak_kind}"}

    k, hd = 4096, 128
    x = torch.randn(m, k, device=device, dtype=torch.float16, generator=torch.Generator(device).manual_seed(6))
    gate = device_copies(synth_weight_numpy(4, 11, 11008, k), device, 1)[0]
    up = device_copies(synth_weight_numpy(4, 12, 11008, k), device, 1)[0]
    out[f"m{m}_gate_up_11008x{k}_w4"] = timed(lambda: ck.fused_gate_up(x, gate, up), 2.0 * m * 2 * 11008 * k)
    del gate, up
    q, kk, v = (device_copies(synth_weight_numpy(4, 13 + i, 4096, k), device, 1)[0] for i in range(3))
    q, kk = ck.permute_for_rope(q, hd), ck.permute_for_rope(kk, hd)
    pos = torch.arange(m, device=device, dtype=torch.float32)[:, None]
    inv = 10000.0 ** (-torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd)
    ang = torch.cat([pos * inv, pos * inv], dim=1)
    rope = (ang.cos().contiguous(), ang.sin().contiguous(), hd)
    out[f"m{m}_qkv_rope_12288x{k}_w4"] = timed(lambda: ck.fused_qkv(x, q, kk, v, rope=rope), 2.0 * m * 12288 * k)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "gemv", "stack"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-gemm", action="store_true", help="skip the prefill GEMM figures")
    ap.add_argument("--no-stack", action="store_true", help="skip the 1-GPU decode-stack figures at N=1")
    ap.add_argument("--comm", default="p2p_barrier", choices=["nccl", "p2p", "p2p_barrier"],
                    help="how the column-parallel stack gathers its activations at N > 1")
    ap.add_argument("--batch", type=int, default=1, help="decode batch of the stack workload (1..8)")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference_arm(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    torch.backends.cuda.matmul.allow_tf32 = False
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(device))

    def barrier():
        if dist is not None:
            dist.barrier()

    def reduce_max(v):
        if dist is None:
            return float(v)
        t = torch.tensor([float(v)], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum_impl(v):
        if dist is None:
            return float(v)
        t = torch.tensor([float(v)], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    _REDUCE_SUM[0] = reduce_sum_impl
    # N = 1: the 4096x4096 GEMVs the headline metric is quoted on (plus, as extra objects, the prefill GEMM
    # and the 1-GPU decode stack).  N > 1: single matmuls stay on one GPU, so the path that shards -- the
    # decode stack -- is what runs; the "stack" object of the N = 1 line is its 1-GPU point.
    workload = args.workload or ("gemv" if world == 1 else "stack")
    if workload == "stack":
        line = run_stack_workload(args, rank, world, device, barrier, reduce_max)
    else:
        line = run_gemv_workload(args, rank, world, device, barrier, reduce_max)
        if world == 1 and not args.no_stack:
            sub = run_stack_workload(args, rank, world, device, barrier, reduce_max, sub=True)
            line["stack"] = {k: sub[k] for k in ("metric", "value", "unit", "ms_per_step", "us_per_launch", "config", "roofline", "e2e")}
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
