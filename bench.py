#!/usr/bin/env python3
"""Benchmark of the packed W2/W3/W4 linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  Top-level workload at every N: batch-1 decode GEMVs over 4096x4096 group-128 weights
at W4, W3 and W2 -- the shapes the headline metric is quoted on; at N > 1 every rank runs its own replica
(single matmuls stay on one GPU, so the top-level figure scales weakly and has no collective).  The path that
shards -- the 32-block decode stack, column-parallel over the N GPUs -- is the `stack` object of the same
line at every N, with its own correctness check, the 1-GPU time measured in the same run, and the speed-up.
Further objects: `gemv_sweep` (bit-width x shape x batch sweep of the decode GEMV), `fused_decode` (fused
QKV / gate-up at batch 1, API form and concatenated form), `gemm` (prefill GEMM sweep).  A step is one pass over COPIES
distinct weight matrices per bit-width (3*COPIES launches); the matrices of one step add up to more
than twice the 126 MB L2, so every launch streams its weights from HBM.  `value` is the algorithmic
bytes of all launches divided by the device time of the timed steps (CUDA events on the launching
stream around CUDA-graph replays of a step, so Python launch overhead is not in the number).  `e2e`
times the same GEMVs through the public API with the activations starting in pinned host memory and
the results read back to the host: its `value` is the step captured on ONE stream with one copy of the step's
activations in and one copy of the step's results out (what a decode loop does); the stricter constructions with
copies around every call (one stream, five streams, eager) are reported beside it.  `reference_cuda` times the
reference's own CUDA kernels (oracle/_ref, when built) on the same GPU with the same harness.  `roofline` describes the dominant kernel (the W4 GEMV):
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
COPIES = 96                 # distinct weight matrices per bit-width and step (about 2 GB in all; a 7B decode step is 128 launches)
E2E_STREAMS = 5             # streams the end-to-end step is pipelined over
FALLBACK_HBM_GBS = 6650.0   # used only without MEASURED_PEAKS.json
FALLBACK_TFLOPS = 1590.0
METRIC = "packed W2/3/4 decode GEMV effective HBM bandwidth (4096x4096, group 128, batch 1)"
COMM_TEXT = {
    "nccl": "NCCL all-gather after each launch",
    "p2p": "all-gather fused into the decode kernel: peer stores over NVLink and an in-kernel rank hand-shake",
    "p2p_barrier": "all-gather fused into the decode kernel's epilogue as peer stores over NVLink, "
                   "one-CTA flag barrier kernel (programmatic dependent launch) after each launch",
    "p2p_seq": "all-gather fused into the decode kernel's epilogue as peer stores over NVLink; launches numbered within "
               "the step, each waits in the kernel for its predecessor's flag from every rank (no completion event on its "
               "own GPU; a block's QKV launch, which reads the step's input, for the one before that), a one-CTA kernel after "
               "each launch publishes its completion",
}
METRIC_STACK = "packed mixed-precision decode stack effective HBM bandwidth (Llama-2-7B shapes, 32 blocks)"
# dram__bytes_read + dram__bytes_write per W4 4096x4096 launch, from the ncu capture summarised under profiles/
# (profiles/gemv_stream_w4_4096x4096_b1.md: the ring kernel's loads are one bulk copy per packed row plus the
# scales and zeros, each byte once)
NCU_TRAFFIC_W4 = 8979328
L2_BYTES = 126e6


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
    threads = OC.use_all_host_threads()        # a launcher may have exported OMP_NUM_THREADS=1
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
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
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
                         "split_k": ops._resolve(None, 1, 1, N_OUT, K_IN, torch.device(device), torch.float16, GROUP)}
    # The same launches as a chain in which every launch reads the previous launch's output (what consecutive layers of a
    # decode step do): each launch then waits for its predecessor's completion.
    dep_graphs = []
    for b in BITS:
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            cur, keep = x, []
            for w in weights[b]:
                cur = ck.packed_linear(cur, w, workspace=ws)
                keep.append(cur)
        dep_graphs.append((gr, keep))
    dep_ms, _ = timed_graph_replays([g_ for g_, _ in dep_graphs], args.steps, 3, barrier)
    for b, ms in zip(BITS, dep_ms):
        us = reduce_max(ms) * 1e3 / (args.steps * COPIES)
        gbs = gemv_bytes(N_OUT, K_IN, b) / (us * 1e-6) / 1e9
        gemv[f"w{b}"]["dependent_chain"] = {"us": us, "gbs": gbs, "frac_of_hbm_peak": gbs / hbm_peak}
    del dep_graphs
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
    # The step the way a decode loop moves data: ONE host-to-device copy of the step's activations (a row per call,
    # from pinned memory), the step's calls on one stream, ONE device-to-host copy of the step's results -- captured
    # and replayed; both copies run on every replay.
    step_ms = None
    if graph_ms is not None:
        try:
            ncalls = len(BITS) * COPIES
            x_rows_host = x_host.repeat(ncalls, 1).contiguous().pin_memory()
            x_rows = torch.empty(ncalls, K_IN, dtype=torch.float16, device=device)
            y_rows_host = torch.empty(ncalls, N_OUT, dtype=torch.float16).pin_memory()
            all_weights = [w for b in BITS for w in weights[b]]

            def step_issue():
                x_rows.copy_(x_rows_host, non_blocking=True)
                outs = [ck.packed_linear(x_rows[i:i + 1], w, workspace=ws) for i, w in enumerate(all_weights)]
                y_rows_host.copy_(torch.cat(outs), non_blocking=True)
                return outs

            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_issue()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            gs = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gs):
                keep_outs = step_issue()

            def step_copies_step():
                gs.replay()
                torch.cuda.synchronize()

            graph_step()                                   # y_host now holds the last call's result of the per-call step
            step_copies_step()
            if not torch.equal(y_rows_host[-1:], y_host):
                raise RuntimeError("the step with per-step copies disagrees with the per-call one")
            step_ms = time_e2e(step_copies_step)
            del keep_outs
        except Exception as exc:
            print(f"[bench] per-step-copies e2e capture failed: {type(exc).__name__}: {exc}", file=sys.stderr)
            torch.cuda.synchronize()
    # The headline is the step as the contract words it -- the step's inputs copied in, the step's results read back,
    # every step -- on one stream.  The stricter per-call constructions are reported beside it.
    e2e_ms = step_ms if step_ms is not None else (graph_ms if graph_ms is not None else eager_ms)
    gbs = lambda ms: world * step_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e = {"value": gbs(e2e_ms), "unit": "GB/s",
           "h2d_bytes_per_step": 3 * COPIES * K_IN * 2, "d2h_bytes_per_step": 3 * COPIES * N_OUT * 2,
           "step_copies_graph_value": None if step_ms is None else gbs(step_ms),
           "eager_value": gbs(eager_ms),
           "one_stream_graph_value": None if graph_ms is None else gbs(graph_ms),
           "pipelined_graph_value": None if piped_ms is None else gbs(piped_ms),
           "api": "crispybits_kernels.packed_linear; packed weights resident on the device as in install_bitmap.  value = "
                  "step_copies_graph_value: per step one copy of all calls' activations from pinned host memory, the "
                  f"step's {3 * COPIES} calls (each on its own row) on one stream, one copy of all results back to pinned host "
                  "memory, captured in a CUDA graph and replayed.  one_stream_graph_value: x copied in and y copied "
                  "back around EVERY call, same stream, captured; eager_value: that per-call step issued call by call "
                  f"from Python; pipelined_graph_value: the per-call step captured over {E2E_STREAMS} streams.  All "
                  "move the same bytes per step"}

    extra = {}
    if rank == 0 and not args.no_sweeps:
        extra["gemv_sweep"] = bench_gemv_sweep(device, hbm_peak, peak_kind)
        extra["fused_decode"] = bench_fused_decode(device, hbm_peak, peak_kind)
    if rank == 0 and not args.no_gemm:
        extra["gemm"] = bench_gemm(device, tf_peak, peak_kind)
    if rank == 0 and not args.no_sweeps:
        try:
            rc = bench_reference_cuda(device, hbm_peak, tf_peak)
        except Exception as exc:      # the reference's kernels are a comparison, not a dependency of this line
            rc = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.synchronize()
        extra["reference_cuda"] = rc if rc is not None else {"unavailable": "oracle/_ref/crispybits_ref_C.so is not built (python oracle/build_ref_cuda.py)"}
        if isinstance(rc, dict) and "gemv_w4_4096x4096_b1" in rc:
            extra["speedup_vs_reference_cuda"] = {f"gemv_w{b}": round(rc[f"gemv_w{b}_4096x4096_b1"]["us"] / gemv[f"w{b}"]["us"], 2) for b in BITS}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, per, threads, sample = cpu_gemv_sample()
        cpu = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample, **per}

    return {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "gemv_4096x4096_w4_w3_w2_b1", "group_size": GROUP, "copies_per_bits": COPIES,
                   "l2": f"inputs larger than L2: each step streams {step_bytes / 1e6:.0f} MB of distinct weights "
                         f"(126 MB L2)", "launch": "CUDA graph replay, one graph per bit-width; the calls of a graph "
                         "read the same x and write their own outputs, so inside the captured chain they overlap "
                         "(gemv.wN.dependent_chain: the same launches with each one reading its predecessor's output)",
                   "multi_gpu": "independent replicas (single matmuls stay on one GPU)" if world > 1 else "n/a"},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gemv": gemv, "clocks": clocks,
        "gpu_launches": args.steps * 3 * COPIES, **extra,
    }


# ------------------------------------------------------------------ GPU arm: decode stack workload
def _stack_parity(args, rank, world, device, comm):
    """A 3-block stack of the same shapes, sharded like the timed one: (1) with more than one rank the requested gather
    must give bit for bit what the NCCL gather gives; (2) the result must match the fp32 evaluation of the same data
    flow from the full (un-sharded) weights, which rank 0 rebuilds with the library's unpack kernel.  Returns the
    maximum relative error of (2) on rank 0."""
    import torch.distributed as dist
    from crispybits_kernels import _C
    from crispybits_kernels.stack import DecodeStack, sample_bitmap
    bm = sample_bitmap(32, 0)[:3]
    x = torch.randn(args.batch, 4096, generator=torch.Generator().manual_seed(11)).half().to(device)
    st = DecodeStack(n_blocks=3, bitmap=bm, rank=rank, world=world, device=device, comm=comm)
    y = st.step(x).clone()
    torch.cuda.synchronize()
    if world > 1 and st.comm != "nccl":
        requested, st.comm = st.comm, "nccl"
        y_nccl = st.step(x).clone()
        st.comm = requested
        torch.cuda.synchronize()
        if not torch.equal(y, y_nccl):
            raise RuntimeError(f"rank {rank}: the {requested} gather and the NCCL gather disagree")
    err = 0.0
    if rank == 0:
        one = DecodeStack(n_blocks=3, bitmap=bm, rank=0, world=1, device=device) if world > 1 else st
        full = []
        for blk in one.blocks:
            dq = {}
            for name in ("q", "k", "v", "o", "gate", "up", "down"):
                w = getattr(blk, name)
                codes = _C.unpack_codes(w.packed.contiguous(), w.bits, w.in_features).float()
                sc = w.scales.float().repeat_interleave(w.group_size, 1)[:, :w.in_features]
                zc = w.zeros.float().repeat_interleave(w.group_size, 1)[:, :w.in_features]
                dq[name] = (codes - zc) * sc
            full.append(dq)
        ref = one.reference_step(x, full)
        err = float((y.float() - ref).abs().max() / ref.abs().max())
        if not err < 4e-3:              # four chained fp16 launches per block
            raise RuntimeError(f"decode stack off by {err:.2e} against the fp32 data flow; not timing")
        del one, full
    del st
    torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
    return err


def _time_stack(st, x, args, barrier, reduce_max):
    """ms per step (device time, max over ranks), the graph or eager callable that was timed, and how it was launched."""
    graph, mode = None, "eager launches"
    try:
        side = torch.cuda.Stream(x.device)
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
        y = st.step(x)

    def one_step():
        if graph is not None:
            graph.replay()
        else:
            st.step(x)

    for _ in range(max(3, args.warmup)):
        one_step()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        one_step()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return reduce_max(e0.elapsed_time(e1)) / args.steps, one_step, y, mode


def run_stack_workload(args, rank, world, device, barrier, reduce_max):
    """One step = the 128 packed decode launches of a Llama-2-7B-shaped 32-block stack (per-block bit-widths
    from the seeded {2,3,4} draw), column-parallel over `world` GPUs with a gather after each launch."""
    from crispybits_kernels.stack import DecodeStack
    hbm_peak, _, peak_kind = peaks()
    batch = args.batch
    st = DecodeStack(rank=rank, world=world, device=device, comm=args.comm)
    x_host = torch.randn(batch, st.d_model, generator=torch.Generator().manual_seed(2)).half().pin_memory()
    x = x_host.to(device)
    comm_note = None
    try:
        for _ in range(2):
            st.step(x)
        torch.cuda.synchronize()
        ok = 1.0
    except Exception as exc:      # e.g. peer-mapped memory cannot be set up on this box
        comm_note = f"{type(exc).__name__}: {exc}"[:200]
        ok = 0.0
    if world > 1 and st.comm != "nccl":
        # every rank must take the same path: if the peer-memory set-up failed anywhere, all ranks use NCCL
        if -reduce_max(-ok) < 1.0:
            print(f"[bench] rank {rank}: peer-store gather unavailable ({comm_note}); using the NCCL gather", file=sys.stderr)
            st.comm = "nccl"
            comm_note = comm_note or "peer set-up failed on another rank"
        else:
            comm_note = None
    elif ok < 1.0:
        raise RuntimeError(comm_note)
    parity_err = _stack_parity(args, rank, world, device, st.comm)

    ms, one_step, y, mode = _time_stack(st, x, args, barrier, reduce_max)
    my_bytes = st.algorithmic_bytes(batch)
    all_bytes = reduce_sum(float(my_bytes)) if world > 1 else float(my_bytes)
    value = all_bytes / (ms * 1e-3) / 1e9
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
    e2e_ms = reduce_max((time.perf_counter() - t0) * 1e3) / args.steps
    launches, comm_used, bitmap = st.launches_per_step(), st.comm, list(st.bitmap)
    del st, one_step, y
    torch.cuda.empty_cache()

    # the same step on ONE GPU, timed in this run on rank 0 (at N = 1 that is the figure above)
    single_ms = ms
    if world > 1:
        if rank == 0:
            one = DecodeStack(rank=0, world=1, device=device)
            single_ms = _time_stack(one, x, args, lambda: None, float)[0]
            del one
            torch.cuda.empty_cache()
        barrier()
    res = {
        "metric": METRIC_STACK, "value": value, "unit": "GB/s", "n_gpus": world, "ms_per_step": ms,
        "us_per_launch": ms * 1e3 / (4 * 32), "scaling": "strong",
        "single_gpu_ms_per_step": single_ms, "speedup_vs_1gpu": single_ms / ms,
        "parity_checked": True, "parity_max_rel_err_vs_fp32_dataflow": parity_err,
        "parity_note": "3-block stack of the same shapes before timing: " + ("requested gather == NCCL gather bit for bit on every rank; " if world > 1 and comm_used != "nccl" else "")
                       + "rank 0 against the fp32 evaluation of the data flow from the full weights (bound 4e-3)",
        "config": {"workload": "decode_stack_llama2_7b_32blocks", "batch": batch, "bitmap_seed": 0,
                   "mean_bits": float(np.mean(bitmap)), "parallelism": (f"column-parallel N over {world} GPUs, " + COMM_TEXT[comm_used]
                                   + (f" [requested {args.comm}: {comm_note}]" if comm_note else "")) if world > 1 else "single GPU",
                   "l2": f"inputs larger than L2: {my_bytes / 1e6:.0f} MB of weights per rank and step", "launch": mode},
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": hbm_peak, "unit": "GB/s",
                     "frac": value / world / hbm_peak, "traffic": None, "kernel": "decode step, per GPU",
                     "algorithmic_bytes_per_launch": my_bytes / (4 * 32), "peak_kind": f"of {peak_kind}"},
        "e2e": {"value": all_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": batch * 4096 * 2, "d2h_bytes_per_step": batch * 4096 * 2,
                "api": "DecodeStack.step: hidden state from pinned host memory, result copied back, every step"},
        "gpu_launches_per_step": launches,
    }
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
            keep = [call(i) for i in range(iters)]      # every call keeps its own outputs, as the calls of a model do
        replay = g.replay
    except Exception as exc:
        print(f"[bench] gemm graph capture failed: {type(exc).__name__}: {exc}", file=sys.stderr)
        torch.cuda.synchronize()
    reps = 5
    if replay is not None:
        for _ in range(2):
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


def _oracle_dequant(d):
    """fp32 [N, K] weight the packed dictionary stands for, by the C oracle (the check value of the gates below)."""
    from oracle import cb_oracle_c as OC
    return OC.dequantized_weight(d["packed"], d["scales"], d["zeros"], d["bits"], d["in_features"], GROUP)


def _gate(name, y, ref, tol=2e-3):
    err = float((y.float() - ref).abs().max() / ref.abs().max())
    if not err < tol:
        raise RuntimeError(f"{name}: off by {err:.2e} against the oracle's dequantised weight; not timing")
    return err


def _copies_beyond_l2(nbytes, floor=2):
    return max(floor, int(np.ceil(2.2 * L2_BYTES / nbytes)))


SWEEP_SHAPES = ((4096, 4096), (11008, 4096), (4096, 11008))


def bench_gemv_sweep(device, hbm_peak, peak_kind, iters_per_graph=1):
    """Decode GEMV over bits {2,3,4} x (N,K) in {(4096,4096), (11008,4096), (4096,11008)} x batch {1,2,4,8}: us per
    launch, algorithmic GB/s and fraction of the HBM peak.  Each case walks enough distinct matrices to exceed twice
    the L2 (so every launch streams from HBM), captured back to back in one CUDA graph; each (bits, shape) is first
    checked against the oracle's dequantised weight for every batch size."""
    import crispybits_kernels as ck
    out = {}
    for (n, k) in SWEEP_SHAPES:
        for b in BITS:
            d = synth_weight_numpy(b, 40 + b, n, k)
            ws = device_copies(d, device, _copies_beyond_l2(gemv_bytes(n, k, b)))
            wd = torch.from_numpy(_oracle_dequant(d)).to(device)
            for batch in (1, 2, 4, 8):
                x = torch.randn(batch, k, device=device, dtype=torch.float16, generator=torch.Generator(device).manual_seed(batch))
                err = _gate(f"gemv w{b} {n}x{k} b{batch}", ck.packed_linear(x, ws[0], decode_threshold=8), x.float() @ wd.T)
                us = _graph_timed_us(lambda i: ck.packed_linear(x, ws[i % len(ws)], decode_threshold=8),
                                     len(ws) * -(-96 // len(ws)))       # about a hundred launches per graph
                gbs = gemv_bytes(n, k, b, batch) / (us * 1e-6) / 1e9
                out[f"w{b}_{n}x{k}_b{batch}"] = {"us": round(us, 3), "gbs": round(gbs, 1), "frac": round(gbs / hbm_peak, 4),
                                                 "err": float(f"{err:.2e}")}
            del ws, wd
            torch.cuda.empty_cache()
    out["note"] = (f"fraction of the HBM copy peak {hbm_peak:.0f} GB/s ({peak_kind}); L2-cold: each graph walks more "
                   "than twice the L2 of distinct matrices; err = max relative error against the oracle")
    return out


def bench_fused_decode(device, hbm_peak, peak_kind):
    """W3, batch 1: the fused Q/K/V and gate/up decode launches in the API's form (three / two weights, three / one
    outputs) and as one GEMV over the row-concatenated matrix."""
    import crispybits_kernels as ck
    from crispybits_kernels import PackedLinearWeight
    out, b, k = {}, 3, 4096
    x = torch.randn(1, k, device=device, dtype=torch.float16, generator=torch.Generator(device).manual_seed(3))

    def cat(ws):
        return PackedLinearWeight(torch.cat([w.packed for w in ws]), torch.cat([w.scales for w in ws]),
                                  torch.cat([w.zeros for w in ws]), b, GROUP, k, sum(w.out_features for w in ws))

    def entry(us, nbytes):
        gbs = nbytes / (us * 1e-6) / 1e9
        return {"us": round(us, 3), "gbs": round(gbs, 1), "frac": round(gbs / hbm_peak, 4)}

    # Q/K/V: 3 x (4096, 4096), seeds 1, 2, 3
    dq = [synth_weight_numpy(b, s, 4096, k) for s in (1, 2, 3)]
    ncopy = _copies_beyond_l2(3 * gemv_bytes(4096, k, b))
    sets = list(zip(*[device_copies(d, device, ncopy) for d in dq]))
    refs = [x.float() @ torch.from_numpy(_oracle_dequant(d)).to(device).T for d in dq]
    for o, r, nm in zip(ck.fused_qkv(x, *sets[0]), refs, "qkv"):
        _gate(f"fused_qkv {nm}", o, r)
    nbytes = gemv_bytes(12288, k, b)
    out["qkv_12288x4096_w3_fused_api"] = entry(_graph_timed_us(lambda i: ck.fused_qkv(x, *sets[i % ncopy]), ncopy * -(-48 // ncopy)), nbytes)
    cats = [cat(st) for st in sets]
    _gate("concatenated qkv", ck.packed_linear(x, cats[0]), torch.cat(refs, 1))
    out["qkv_12288x4096_w3_concatenated"] = entry(_graph_timed_us(lambda i: ck.packed_linear(x, cats[i % ncopy]), ncopy * -(-48 // ncopy)), nbytes)
    del sets, cats, refs
    torch.cuda.empty_cache()
    # gate/up: 2 x (11008, 4096), seeds 5, 6
    dg = [synth_weight_numpy(b, s, 11008, k) for s in (5, 6)]
    ncopy = _copies_beyond_l2(2 * gemv_bytes(11008, k, b))
    sets = list(zip(*[device_copies(d, device, ncopy) for d in dg]))
    rg, ru = (x.float() @ torch.from_numpy(_oracle_dequant(d)).to(device).T for d in dg)
    _gate("fused_gate_up", ck.fused_gate_up(x, *sets[0]), torch.nn.functional.silu(rg) * ru)
    out["gate_up_2x11008x4096_w3_fused_api"] = entry(_graph_timed_us(lambda i: ck.fused_gate_up(x, *sets[i % ncopy]), ncopy * -(-48 // ncopy)),
                                                     2 * gemv_bytes(11008, k, b) - k * 2 - 11008 * 2)
    cats = [cat(st) for st in sets]
    _gate("concatenated gate/up", ck.packed_linear(x, cats[0]), torch.cat([rg, ru], 1))
    out["gate_up_22016x4096_w3_concatenated"] = entry(_graph_timed_us(lambda i: ck.packed_linear(x, cats[i % ncopy]), ncopy * -(-48 // ncopy)),
                                                      gemv_bytes(22016, k, b))
    out["note"] = f"fraction of the HBM copy peak {hbm_peak:.0f} GB/s ({peak_kind}); L2-cold as the sweep"
    return out


def bench_reference_cuda(device, hbm_peak, tf_peak):
    """The reference's OWN CUDA kernels (Crispybits/Kernel/csrc/packed_gemv.cu, packed_gemm.cu, compiled unmodified for
    sm_100a by oracle/build_ref_cuda.py) timed on this GPU with the harness used for this library: the 4096x4096 batch-1
    GEMV at W4/W3/W2 (L2-cold, captured back to back) with the reference's Split-K rule and with split_k = 1, and the
    M = 1024 prefill GEMM.  None when the module has not been built."""
    from oracle import build_ref_cuda
    ref = build_ref_cuda.load_module()
    if ref is None:
        return None
    out = {}
    e16 = torch.empty(0, device=device, dtype=torch.float16)
    sms, bn = int(ref.sm_count()), int(ref.tile_n())
    for b in BITS:
        d = synth_weight_numpy(b, b)
        ws = device_copies(d, device, _copies_beyond_l2(gemv_bytes(N_OUT, K_IN, b)))
        wd = torch.from_numpy(_oracle_dequant(d)).to(device)
        x = torch.randn(1, K_IN, device=device, dtype=torch.float16, generator=torch.Generator(device).manual_seed(1))
        wsp = torch.zeros(2, dtype=torch.int32, device=device)
        tiles = -(-N_OUT // bn)
        rule = 1 if tiles >= sms else -(-sms // tiles)          # SM-underfill rule, rho = 1 (ops.py:144-153 of the reference)
        best = None
        for split in sorted({1, rule}):
            call = lambda i, split=split: ref.packed_gemv(x, ws[i % len(ws)].packed, ws[i % len(ws)].scales, ws[i % len(ws)].zeros,
                                                           e16, b, K_IN, GROUP, split, 1, 0, wsp)
            _gate(f"reference CUDA gemv w{b} split_k={split}", call(0), x.float() @ wd.T, 3e-3)
            us = _graph_timed_us(call, len(ws) * -(-96 // len(ws)))
            if best is None or us < best[0]:
                best = (us, split)
        gbs = gemv_bytes(N_OUT, K_IN, b) / (best[0] * 1e-6) / 1e9
        out[f"gemv_w{b}_4096x4096_b1"] = {"us": round(best[0], 3), "gbs": round(gbs, 1), "frac": round(gbs / hbm_peak, 4),
                                          "split_k": best[1], "rule_split_k": rule}
        if b != 2:
            xm = torch.randn(1024, K_IN, device=device, dtype=torch.float16, generator=torch.Generator(device).manual_seed(6))
            call = lambda i: ref.packed_gemm(xm, ws[i % 2].packed, ws[i % 2].scales, ws[i % 2].zeros, e16, b, K_IN, GROUP, 0, True)
            _gate(f"reference CUDA gemm w{b}", call(0)[:256], xm[:256].float() @ wd.T, 3e-3)
            us = _graph_timed_us(call, 4)
            tf = 2.0 * 1024 * N_OUT * K_IN / (us * 1e-6) / 1e12
            out[f"gemm_m1024_4096x4096_w{b}"] = {"us": round(us, 2), "tflops": round(tf, 1), "frac_of_dense_peak": round(tf / tf_peak, 4)}
        del ws, wd
        torch.cuda.empty_cache()
    out["note"] = ("the reference's CUDA extension built unmodified for sm_100a and run on this GPU; same inputs, same CUDA-graph "
                   "timing as this library's figures; GEMV: the faster of the reference's Split-K rule and split_k = 1")
    return out


GEMM_SHAPES = ((4096, 4096), (12288, 4096), (22016, 4096), (4096, 11008))
GEMM_TOKENS = (128, 512, 1024, 4096)


def bench_gemm(device, tf_peak, peak_kind, iters=10):
    """Prefill GEMM (TFLOP/s = 2*M*N*K / t) for W4 and W3, M in {128, 512, 1024, 4096}, the four Llama-2-7B (N, K)
    shapes, plus the fused gate/up and Q/K/V forms at M = 1024.  Every figure is preceded by a check of the same
    call against the fp32 product with the oracle's dequantised weight (2e-3)."""
    import crispybits_kernels as ck
    out = {}
    for (n, k) in GEMM_SHAPES:
        for b in (4, 3):
            d = synth_weight_numpy(b, 60 + b, n, k)
            ws = device_copies(d, device, 2)
            wd = torch.from_numpy(_oracle_dequant(d)).to(device)
            for m in GEMM_TOKENS:
                x = torch.randn(m, k, device=device, dtype=torch.float16, generator=torch.Generator(device).manual_seed(5 + m))
                y = ck.packed_linear(x, ws[0])
                rows = min(m, 512)                 # the check covers the first 512 tokens of the call (every weight row)
                err = _gate(f"gemm w{b} m{m} {n}x{k}", y[:rows], x[:rows].float() @ wd.T)
                us = _graph_timed_us(lambda i: ck.packed_linear(x, ws[i % 2]), iters if m <= 1024 else 4)
                tf = 2.0 * m * n * k / (us * 1e-6) / 1e12
                out[f"m{m}_{n}x{k}_w{b}"] = {"us": round(us, 2), "tflops": round(tf, 1), "frac_of_dense_peak": round(tf / tf_peak, 4),
                                             "err": float(f"{err:.2e}")}
                del x, y
            del ws, wd
            torch.cuda.empty_cache()

    # the fused forms at M = 1024, K = 4096: gate/up (silu(g) * u in the epilogue) and Q/K/V (RoPE and un-permuted
    # stores in the epilogue); FLOPs are those of the projections alone
    def timed(fn, flops):
        us = _graph_timed_us(lambda i: fn(), iters)
        tf = flops / (us * 1e-6) / 1e12
        return {"us": round(us, 2), "tflops": round(tf, 1), "frac_of_dense_peak": round(tf / tf_peak, 4)}

    m, k, hd = 1024, 4096, 128
    x = torch.randn(m, k, device=device, dtype=torch.float16, generator=torch.Generator(device).manual_seed(6))
    dgs = [synth_weight_numpy(4, s, 11008, k) for s in (11, 12)]
    gate, up = (device_copies(d, device, 1)[0] for d in dgs)
    rg, ru = (x[:256].float() @ torch.from_numpy(_oracle_dequant(d)).to(device).T for d in dgs)
    _gate("fused gate/up gemm", ck.fused_gate_up(x, gate, up)[:256], torch.nn.functional.silu(rg) * ru, 3e-3)
    out[f"m{m}_gate_up_11008x{k}_w4"] = timed(lambda: ck.fused_gate_up(x, gate, up), 2.0 * m * 2 * 11008 * k)
    del gate, up, rg, ru
    dqs = [synth_weight_numpy(4, 13 + i, 4096, k) for i in range(3)]
    q, kk, v = (device_copies(d, device, 1)[0] for d in dqs)
    plain = ck.fused_qkv(x, q, kk, v)
    for o, d, nm in zip(plain, dqs, "qkv"):
        _gate(f"fused qkv gemm {nm}", o[:256], x[:256].float() @ torch.from_numpy(_oracle_dequant(d)).to(device).T)
    from crispybits_kernels.ops import apply_rope_reference as ops_rope
    qp, kp = ck.permute_for_rope(q, hd), ck.permute_for_rope(kk, hd)
    pos = torch.arange(m, device=device, dtype=torch.float32)[:, None]
    inv = 10000.0 ** (-torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd)
    ang = torch.cat([pos * inv, pos * inv], dim=1)
    rope = (ang.cos().contiguous(), ang.sin().contiguous(), hd)
    roped = ck.fused_qkv(x, qp, kp, v, rope=rope)
    for o, base, nm in zip(roped[:2], plain[:2], "qk"):      # rotation of the checked plain result, in fp32
        want = ops_rope(base.float(), rope[0], rope[1], hd)
        _gate(f"fused qkv gemm rope {nm}", o, want.float(), 4e-3)
    out[f"m{m}_qkv_rope_12288x{k}_w4"] = timed(lambda: ck.fused_qkv(x, qp, kp, v, rope=rope), 2.0 * m * 12288 * k)
    out["note"] = (f"fraction of the dense tensor peak {tf_peak:.0f} TFLOP/s (cuBLAS bf16, {peak_kind}); graph replay of "
                   "back-to-back calls; err = max relative error against the oracle's dequantised weight")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-gemm", action="store_true", help="skip the prefill GEMM figures")
    ap.add_argument("--no-sweeps", action="store_true", help="skip the decode sweep and the fused decode figures")
    ap.add_argument("--no-stack", action="store_true", help="skip the decode-stack figures")
    ap.add_argument("--comm", default="p2p_seq", choices=["nccl", "p2p", "p2p_barrier", "p2p_seq"],
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
    # Top level at every N: the 4096x4096 GEMVs the headline metric is quoted on, one replica per rank (single
    # matmuls stay on one GPU).  The path that shards -- the decode stack -- is the "stack" object at every N.
    line = run_gemv_workload(args, rank, world, device, barrier, reduce_max)
    if not args.no_stack:
        line["stack"] = run_stack_workload(args, rank, world, device, barrier, reduce_max)
        line["gpu_launches"] += args.steps * line["stack"]["gpu_launches_per_step"]
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
