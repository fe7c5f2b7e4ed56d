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
  cpu_baseline  the CPU oracle of the step (CpuModel.step: the real op arithmetic), timed on a bounded sample on rank
            0's host cores
  reference_kernels  the reference's own compiled kernels that run on this part (attention decode, the DeltaNet trio, the
            16-bit in-projection), timed next to the library's on the same buffers (N = 1 only)
  greedy_256  256 greedy tokens decoded with verify steps of 1 + 4 drafts (some right, then wrong) against one token
            per step from the same state: identical or not, and where they first differ
  prefill   the 32768-token prompt in 2048-row chunks through the same model (N = 1 only)
--impl reference times the CPU oracle alone (the reference's whole CUDA step cannot run here: its Marlin kernels end
with an illegal-instruction fault on B200; its kernels that do run are timed in reference_kernels).
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


_CPU_MODEL = None


def cpu_baseline(seconds: float):
    """CpuModel.step of the oracle on one [DeltaNet x3, attention] block (x16) + the output layer, all host threads."""
    global _CPU_MODEL
    from oracle import cpu_step
    # every host core this process may use (torchrun sets OMP_NUM_THREADS=1 for its workers; the baseline is the CPU
    # path with all the threads it can have)
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    import torch
    torch.set_num_threads(cores)
    if _CPU_MODEL is None:
        _CPU_MODEL = cpu_step.host_block_model(position=POSITION)
    r = cpu_step.time_step_baseline(seconds=seconds, threads=cores, position=POSITION, model=_CPU_MODEL)
    return {"value": r["rows_per_s"], "unit": "tok/s", "cores": r["cores"], "kind": "port", "sample": r["sample"],
            "ms_per_step": r["step_s"] * 1e3}


def greedy_256(model, torch, tokens_wanted: int = 256, k: int = 4):
    """The reference's speccheck (src/checks.rs:892-937) on the benchmark's model from the benchmark's state: 256 greedy
    tokens one per step, then again from the same saved state with verify steps of 1 + k drafts of which step % (k + 1)
    are right and the rest wrong (a restart inside the step follows). The two token streams must be identical."""
    image, pos0 = model.save_state(0)
    first = 1000

    def single():
        out = [first]
        for i in range(tokens_wanted):
            model.step([(out[-1], 0, pos0 + i)], [0])
            out.append(model.argmax()[0])
        return out
    reference = single()
    model.load_state(0, image, pos0)
    got, steps = [first], 0
    while len(got) < len(reference):
        good = steps % (k + 1)
        steps += 1
        d = [reference[len(got) + j] if j < good and len(got) + j < len(reference) else 7 + j for j in range(k)]
        toks = [(t, 0, pos0 + len(got) - 1 + j) for j, t in enumerate([got[-1]] + d)]
        model.step(toks, list(range(len(toks))))
        am = model.argmax()
        for j, t in enumerate(am):
            got.append(t)
            if j >= len(d) or d[j] != t:
                break
    got = got[:len(reference)]
    same = next((i for i, (a, b) in enumerate(zip(got, reference)) if a != b), None)
    model.load_state(0, image, pos0)
    return {"steps": tokens_wanted, "verify_steps": steps, "rows_per_verify_step": k + 1, "identical": same is None,
            "first_divergence": same, "against": "one token per step on the same device, from the same saved state"}


def _time_us(torch, fn, reps=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / reps


def reference_kernels(ctx, torch):
    """The reference's own compiled kernels (oracle/_ref, built unmodified from its sources) next to the library's on the
    same buffers, CUDA events, launches back to back: the part of the reference's CUDA path that runs on this GPU."""
    import math
    import numpy as np
    from oracle import ref_cuda
    from oracle import ref_ops as R
    if not ref_cuda.available():
        return {"unavailable": "oracle/_ref is not built"}
    ref = ref_cuda.RefModule()
    g = torch.Generator(device="cuda").manual_seed(3)
    res = {"how": "CUDA events around 20 launches back to back on the default stream, after 3 warm-up launches"}
    # ---- attention, the benchmark's configuration: 5 causal rows over a 32768-token int8 cache
    n, cap, pos0 = 5, 32768, 32763
    kc = torch.randint(1, 256, (R.NKV * cap * R.HD,), generator=g, dtype=torch.uint8, device="cuda")
    vc = torch.randint(1, 256, (R.NKV * cap * R.HD,), generator=g, dtype=torch.uint8, device="cuda")
    ks = (torch.randn(R.NKV * cap, generator=g, device="cuda") * 0.05).abs()
    vs = (torch.randn(R.NKV * cap, generator=g, device="cuda") * 0.05).abs()
    q = torch.randn(n, R.NH, R.HD, generator=g, device="cuda") * (math.log2(math.e) / 16)
    gate = torch.sigmoid(torch.randn(n, R.MIX, generator=g, device="cuda"))
    st = R.build_step([(0, 0, pos0 + i) for i in range(n)], list(range(n)))
    dv = ref_cuda.upload_step(st)
    ml = torch.zeros(64 * 128 * R.NH * 2, device="cuda")
    acc = torch.zeros(64 * 128 * R.NH * R.HD, device="cuda")
    out = gate.clone()
    mix = torch.zeros(n, R.MIX, dtype=torch.float16, device="cuda")
    ours = _time_us(torch, lambda: ctx.attn_decode(q, kc, vc, ks, vs, dv, st, cap, ml, acc, out, mix))
    theirs = _time_us(torch, lambda: ref.attn_decode(q, kc, vc, ks, vs, st, dv, cap, ml, acc, out))
    res["attention_decode_5rows_32768keys"] = {"ours_us": ours, "reference_us": theirs,
                                               "reference": "attn_mq2 + attn_combine", "bytes": R.NKV * 520 * (pos0 + n)}
    # ---- the DeltaNet mixer, the benchmark's configuration: 5 sequential rows, f32 state [48, 128, 128]
    sst = (R.SLOT_FLOATS + 1023) // 1024 * 1024
    part = torch.randn(1, n, R.DELTA_IN, generator=g, device="cuda")
    ba = torch.randn(1, n, 2 * R.LV_HEADS, generator=g, device="cuda")
    conv_w = torch.randn(R.LQKV, 4, generator=g, device="cuda") * 0.3
    a_log = torch.randn(R.LV_HEADS, generator=g, device="cuda") * 0.5
    dt_bias = torch.randn(R.LV_HEADS, generator=g, device="cuda") * 0.5
    norm_w = 1 + torch.randn(R.LVD, generator=g, device="cuda") * 0.02
    mems = [torch.randn(sst, generator=g, device="cuda") * 0.01 for _ in range(24)]  # states in rotation (3 MB each)
    meta = torch.tensor([[32000, 32000, 0, 0]], dtype=torch.int32, device="cuda")
    st2 = R.build_step([(0, 0, 32000 + i) for i in range(n)], [0])
    dv2 = ref_cuda.upload_step(st2)
    cv = torch.zeros(n, R.CVW, device="cuda")
    o = torch.zeros(n, R.MIX, device="cuda")
    y = torch.zeros(n, R.MIX, dtype=torch.float16, device="cuda")
    i = [0]

    def ours_mixer():
        meta.copy_(torch.tensor([[32000, 32000, 0, 0]], dtype=torch.int32), non_blocking=True)
        ctx.delta_mixer(part, 1, n, ba, 1, conv_w, a_log, dt_bias, norm_w, mems[i[0] % 24], sst, meta, None, y, dv2, 1)
        i[0] += 1

    def their_mixer():
        meta.copy_(torch.tensor([[32000, 32000, 0, 0]], dtype=torch.int32), non_blocking=True)
        ref.delta(part, 1, n, ba, 1, conv_w, a_log, dt_bias, norm_w, mems[i[0] % 24], sst, meta, cv, o, y, st2, dv2)
        i[0] += 1
    ours, theirs = _time_us(torch, ours_mixer), _time_us(torch, their_mixer)
    res["deltanet_mixer_5rows"] = {"ours_us": ours, "reference_us": theirs,
                                   "reference": "delta_conv + delta_rule + delta_norm (three launches)",
                                   "ours": "one launch (qb_delta_mixer)", "bytes": 2 * R.SLOT_STATE * 4,
                                   "note": "both include a 16-byte metadata reset per launch"}
    # ---- the DeltaNet prompt path: the reference's sequential delta_rule against the chunked scan, 2048 rows
    T = 2048
    part_l = torch.randn(1, T, R.DELTA_IN, generator=g, device="cuda")
    qq = torch.nn.functional.normalize(torch.randn(T, R.LK_HEADS, R.LKD, generator=g, device="cuda"), dim=-1)
    kk = torch.nn.functional.normalize(torch.randn(T, R.LK_HEADS, R.LKD, generator=g, device="cuda"), dim=-1)
    cv_l = torch.cat([(qq / R.LKD ** 0.5).reshape(T, -1), kk.reshape(T, -1),
                      torch.randn(T, R.LV_HEADS * R.LVD, generator=g, device="cuda"),
                      torch.exp(-torch.nn.functional.softplus(torch.randn(T, R.LV_HEADS, generator=g, device="cuda"))),
                      torch.sigmoid(torch.randn(T, R.LV_HEADS, generator=g, device="cuda"))], dim=1).contiguous()
    st3 = R.build_step([(0, 0, i) for i in range(T)], [0])
    dv3 = ref_cuda.upload_step(st3)
    o_l = torch.zeros(T, R.MIX, device="cuda")
    meta0 = torch.tensor([[-1, 0, 0, 0]], dtype=torch.int32, device="cuda")
    ours = _time_us(torch, lambda: ctx.delta_rule(part_l, 1, T, cv_l, mems[0], sst, meta0, o_l, dv3, 1), reps=5)
    theirs = _time_us(torch, lambda: ref.delta(part_l, 1, T, None, 0, None, None, None, None, mems[1], sst, meta0, cv_l,
                                                o_l, None, st3, dv3, which=("rule",)), reps=5)
    res["deltanet_rule_2048rows"] = {"ours_us": ours, "reference_us": theirs, "reference": "delta_rule (sequential)",
                                     "ours": "chunked scan, chunk 64, 3 x TF32 (two launches)"}
    # ---- the 16-bit in-projection of a DeltaNet layer (in_proj_b / in_proj_a, 96 x 5120)
    K, rows = 5120, 96
    wp = (torch.randn(rows // 16, K // 16, 32, 8, generator=g, device="cuda") * 0.02).half()
    x = torch.randn(n, K, generator=g, device="cuda").half()
    split = R.split_for(rows // 16, K, 16, 1024)
    yo = torch.zeros(split, n, rows, device="cuda")
    ours = _time_us(torch, lambda: ctx.gemm_f16_plain(wp, x, n, K, rows // 16, K // split, y=yo))
    theirs = _time_us(torch, lambda: ref.gemm_f16_plain(wp, x, yo, n, K, rows // 16))
    res["in_ba_96x5120_5rows"] = {"ours_us": ours, "reference_us": theirs, "reference": "gemm_f16_t8_plain"}
    # ---- prompt attention: 2048 rows at the end of the 32768-token cache (the last prompt chunk)
    T, pos0 = 2048, cap - 2048
    qp = torch.randn(T, R.NH, R.HD, generator=g, device="cuda") * (math.log2(math.e) / 16)
    gp = torch.sigmoid(torch.randn(T, R.MIX, generator=g, device="cuda"))
    st4 = R.build_step([(0, 0, pos0 + i) for i in range(T)], [0], short=0)
    dv4 = ref_cuda.upload_step(st4)
    op = gp.clone()
    mixp = torch.zeros(T, R.MIX, dtype=torch.float16, device="cuda")
    ours = _time_us(torch, lambda: ctx.attn_prefill(qp, kc, vc, ks, vs, dv4, st4, cap, ml, acc, op, mixp), reps=3)
    theirs = _time_us(torch, lambda: ref.attn_prefill(qp, kc, vc, ks, vs, st4, dv4, cap, ml, acc, op), reps=3)
    res["attention_prompt_2048rows_32768keys"] = {
        "ours_us": ours, "reference_us": theirs, "reference": "attn_prefill (mma.sync)", "ours": "tcgen05, S / P / O in tensor memory",
        "flops": 4.0 * R.HD * R.NH * sum(pos0 + i + 1 for i in range(T))}
    res["not_timed"] = "marlin_* (the W4A16 products): they end in an illegal-instruction fault on this GPU and are not launched"
    torch.cuda.synchronize()
    return res


def prefill_record(model, ctx, torch, prompt: int = 32768, chunk: int = 2048):
    """The benchmark's prefill configuration on the same model: a 32768-token prompt of uniform token ids in 2048-row
    chunks (slot 0 restarts at position 0; the decode measurements are finished). Device time per chunk by CUDA events."""
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 151936, (prompt,), generator=g).tolist()
    chunks = [(a, min(prompt, a + chunk)) for a in range(0, prompt, chunk)]
    ms = []
    for rep in range(2):  # the first pass warms up (kernel attributes, the chunked scan's scratch)
        times = []
        for a, b in chunks:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(model.stream)
            model.step([(ids[i], 0, i) for i in range(a, b)], [b - a - 1])
            e1.record(model.stream)
            times.append((e0, e1))
        model.argmax()
        ms = [x.elapsed_time(y) for x, y in times]
    tot = sum(ms)
    # linear layers: 2 flops per weight and token; causal attention: 4 * HD flops per (row, key, head)
    weights = sum(l[name].n * l[name].k for l in model.layers for name in ("in_proj", "out", "gate_up", "down"))
    attn_layers = sum(1 for l in model.layers if l["kind"] == "attn")
    flops = 2.0 * weights * prompt + attn_layers * 4.0 * 256 * 24 * (prompt * (prompt + 1) / 2)
    peak = None
    pth = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pth):
        with open(pth) as f:
            peak = float(json.load(f).get("bf16_tflops_sustained", 0)) or None
    tf = flops / tot / 1e9
    return {"metric": "prefill tok/s, 32768-token prompt in 2048-row chunks", "value": prompt / tot * 1e3, "unit": "tok/s",
            "ms_total": tot, "ms_first_chunk": ms[0], "ms_last_chunk": ms[-1], "tflops": tf,
            "frac_of_measured_bf16_sustained": tf / peak if peak else None, "peak_tflops": peak,
            "device_error": ctx.device_error()}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.time()
    # each "step" is one bounded sample of the workload; K + W of them within a few minutes
    per = max(3.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
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
                       "rows_per_step": ROWS, "note": "the reference's whole CUDA step is unavailable on B200 (its "
                       "Marlin kernels fault with an illegal instruction); this arm is the CPU oracle of the step "
                       "(CpuModel.step, real op arithmetic), one 4-layer block x16 + the output layer"},
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
    sampler = ClockSampler(local)
    # K steps take a few tenths of a second: the K-step region is timed `regions` times back to back (each bracketed by
    # a barrier and a device synchronisation on both sides) so that the clock record has samples, and the median
    # region is reported
    model.run()
    barrier()
    t0 = time.perf_counter()
    model.run()
    torch.cuda.synchronize()
    regions = max(3, min(40, int(1.5 / max(1e-4, (time.perf_counter() - t0) * args.steps)) + 1))
    barrier()
    launches0 = model.launches
    sampler.start()
    dev_ms = []
    for _ in range(regions):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            model.run()
        e1.record(stream)
        barrier()
        dev_ms.append(e0.elapsed_time(e1) / args.steps)
    ms_dev = statistics.median(dev_ms)
    launches = (model.launches - launches0) // (args.steps * regions)

    # ---- end to end through the host API: token upload + replay + greedy tokens back, every step
    e2e_ms = []
    for _ in range(regions):
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            model.step(toks, out)
            tokens = model.argmax()
        torch.cuda.synchronize()
        e2e_ms.append((time.perf_counter() - t0) * 1e3 / args.steps)
    ms_e2e = statistics.median(e2e_ms)
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
                       "timed_regions": regions, "region": "K steps between barriers; the median region is reported",
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
        if world == 1 and not args.no_extras:
            line["greedy_256"] = greedy_256(model, torch)
            line["reference_kernels"] = reference_kernels(ctx, torch)
            line["prefill"] = prefill_record(model, ctx, torch)
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
    ap.add_argument("--no-extras", action="store_true", help="skip greedy_256, reference_kernels and prefill")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
