#!/usr/bin/env python
"""Benchmark of the 27B-shape int4 decode / verify step (5 rows: 1 token + 4 MTP drafts) at context 32000.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One process per GPU (under torchrun for N > 1); every GPU runs a full model replica on its own request slot (the
path shards by independent slots: no data-path collective), so the scaling is weak and the value is the sum over
ranks. Rank 0 prints one JSON line:
  value     verified rows per second with the step's inputs resident on the device (CUDA-graph replays only)
  e2e       the same through the public host API with host buffers: qb_model_step (token upload, graph replay) and
            qb_model_argmax (device -> host read of the greedy tokens) every step
  roofline  the dominant kernel (the W4A16 GEMV): its algorithmic bytes / its average launch time, measured here with
            CUDA events over a replayed graph of the step's 257 products alone, against the measured HBM copy peak
  cpu_baseline  the fp32 CPU restatement of the step, timed on a bounded sample on rank 0's host cores
--impl reference times that CPU restatement alone (the reference's CUDA path cannot run here: its Marlin kernels end
with an illegal-instruction fault on B200, so the reference arm is its CPU check path's method, as a port).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS = 5
POSITION = 32000
METRIC = "27B-shape int4 decode tok/s (5-row MTP verify)"


NCU_TRAFFIC_RATIO = 43.35 / 43.2538  # measured DRAM bytes / algorithmic bytes of the captured launch


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi SM clock and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def workload(layers: int) -> str:
    return (f"full 27B-shape hybrid decoder verify step ({layers} layers, int4 g128 weights, int8 KV): 5 rows (1 token + 4 "
            f"MTP drafts) at context {POSITION}, one slot per GPU (the benchmark's full-step configuration)")


def cpu_baseline(seconds: float):
    from oracle import cpu_step
    # every host core this process may use (torchrun sets OMP_NUM_THREADS=1 for its workers; the baseline is the CPU
    # path with all the threads it can have)
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    r = cpu_step.time_baseline(seconds=seconds, threads=cores)
    return {"value": r["rows_per_s"], "unit": "tok/s", "cores": r["cores"], "kind": "port", "sample": r["sample"],
            "ms_per_step": r["step_s"] * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.time()
    # each "step" is one bounded sample of the workload; K + W of them within a few minutes
    per = max(2.0, min(20.0, 150.0 / max(1, args.steps + args.warmup)))
    vals = []
    for i in range(args.warmup + args.steps):
        b = cpu_baseline(per)
        if i >= args.warmup:
            vals.append(b)
    v = statistics.mean(x["value"] for x in vals)
    ms = statistics.mean(x["ms_per_step"] for x in vals)
    line = {"metric": METRIC, "value": v, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": {"workload": workload(args.layers),
                       "rows_per_step": ROWS, "note": "reference CUDA path unavailable on B200 (its Marlin kernels "
                       "fault with an illegal instruction); CPU port of its fp32 check path, one 4-layer block x16"},
            "cpu_baseline": {"value": v, "unit": "tok/s", "cores": vals[-1]["cores"], "kind": "port",
                             "sample": vals[-1]["sample"]},
            "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": time.time() - t0}
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from qwenny_b200 import model as M
    from qwenny_b200.ops import Context

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    ctx = Context(local)
    ctx.set_pdl(not args.no_pdl)
    model = M.synthetic(ctx, nlayers=args.layers, slots=1, max_ctx=32768, position=POSITION, seed=rank)
    toks = [(1000 + 7919 * i % 20000, 0, POSITION + i) for i in range(ROWS)]  # the reference's synthetic stream
    out = list(range(ROWS))
    stream = model.stream

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (captures the graph), then K device-resident replays
    for _ in range(max(3, args.warmup)):
        model.step(toks, out)
        model.argmax()
    launches0 = model.launches
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        model.run()
    e1.record(stream)
    barrier()
    ms_dev = e0.elapsed_time(e1) / args.steps
    launches = (model.launches - launches0) // args.steps

    # ---- end to end through the host API: token upload + replay + greedy tokens back, every step
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.step(toks, out)
        tokens = model.argmax()
    torch.cuda.synchronize()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    barrier()

    # ---- the dominant kernel alone: the step's 257 int4 products replayed as one graph
    gemm_bytes, gemm_us, ngemm = 0, None, 0
    if rank == 0:
        xs = {k: torch.randn(ROWS, k, device="cuda").half() for k in (5120, 6144, 17408)}
        ys = {}

        def products():
            nb, n = 0, 0
            for l in model.layers:
                for name, epi in (("in_proj", "plain"), ("out", "plain"), ("gate_up", "silu"), ("down", "plain")):
                    w = l[name]
                    if (w.n, epi) not in ys:
                        ys[(w.n, epi)] = torch.empty(ROWS, w.n // 2, dtype=torch.float16, device="cuda") \
                            if epi == "silu" else torch.empty(ROWS, w.n, device="cuda")
                    ctx.marlin_gemm(xs[w.k], w.words, w.scales, epi=epi, y=ys[(w.n, epi)])
                    nb += int(w.n * w.k * 0.515625)
                    n += 1
            return nb, n
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            products()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                gemm_bytes, ngemm = products()
            g.replay(); torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 3
            a.record(side)
            for _ in range(reps):
                g.replay()
            b.record(side); torch.cuda.synchronize()
            gemm_us = a.elapsed_time(b) * 1e3 / reps / ngemm

    # ---- max over ranks
    from qwenny_b200 import replicas
    ms_dev, ms_e2e = replicas.slowest_ms(ms_dev, "cuda"), replicas.slowest_ms(ms_e2e, "cuda")
    err = ctx.device_error()
    if err:
        raise SystemExit(f"a kernel gave up a bounded wait (code {err})")

    if rank == 0:
        peak, peak_kind = measured_peak()
        step_bytes = model.step_bytes(POSITION)
        bytes_per_launch = gemm_bytes / ngemm
        achieved = bytes_per_launch / gemm_us / 1e3  # GB/s
        line = {
            "metric": METRIC, "value": replicas.job_throughput(ROWS, ms_dev, world), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_dev, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload(args.layers),
                       "rows_per_step": ROWS, "steps_per_s_per_gpu": 1e3 / ms_dev, "position": POSITION,
                       "cuda_graph": True, "programmatic_dependent_launch": not args.no_pdl,
                       "l2": "inputs larger than L2: 14.4 GB of weights, KV and state stream per step",
                       "tok": "verified rows; steps/s = tok/s / 5"},
            "e2e": {"value": replicas.job_throughput(ROWS, ms_e2e, world), "unit": "tok/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": int(model_step_h2d_bytes()), "d2h_bytes_per_step": ROWS * 8},
            "gpu_launches": int(launches * args.steps),
            "launches_per_step": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         # dram__bytes_read + write of one ncu capture of this kernel (16384 x 5120 product: 43.35 MB
                         # against 43.25 MB algorithmic), scaled to the average launch by the bytes streamed
                         "traffic": bytes_per_launch * NCU_TRAFFIC_RATIO, "traffic_source":
                         "ncu capture of the 16384 x 5120 launch, scaled by algorithmic bytes (profiles/w4a16_gemv.md)",
                         "kernel": "w4a16_gemv_kernel", "peak_kind": f"{peak_kind} copy bandwidth",
                         "bytes_per_launch": bytes_per_launch, "us_per_launch": gemm_us, "launches_timed": ngemm},
            "step_roofline": {"bytes_per_step": step_bytes, "achieved_gbs": step_bytes / ms_dev / 1e6,
                              "frac_of_measured": step_bytes / ms_dev / 1e6 / peak,
                              "frac_of_8tbs": step_bytes / ms_dev / 1e6 / 8000.0},
            "clocks": clocks,
            "greedy_tokens": tokens,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(args.cpu_seconds)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def model_step_h2d_bytes():
    # the step arrays of one upload: one pinned block copied per step (qb_model_upload)
    MAX_TOK, MAX_OUT = 2048, 64
    ints = 7 * MAX_TOK + MAX_TOK + 2 * MAX_TOK + MAX_TOK + MAX_OUT + (MAX_TOK + 8 * MAX_OUT) + (MAX_TOK + 4)
    return ints * 4 + ROWS * 12  # + the caller's token array


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
