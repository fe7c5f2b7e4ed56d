"""Small drivers for timing and profiling one kernel or a short step on one GPU.

    python -m qwenny_b200.microbench gemv N K [--rows 5] [--epi plain|silu|argmax] [--reps 24] [--tune cg,kg,stages,ctas]
    python -m qwenny_b200.microbench attn [--context 32000] [--rows 5] [--reps 20]
    python -m qwenny_b200.microbench step [--layers 8] [--steps 3] [--rows 5] [--no-graph] [--no-pdl] [--lora 16]
    python -m qwenny_b200.microbench prefill [--layers 64] [--prompt 32768] [--chunk 2048]
    python -m qwenny_b200.microbench delta [--rows 2048 | --rows 5]
    python -m qwenny_b200.microbench draft [--k 4] [--draft-rows 65536]
    python -m qwenny_b200.microbench session [--layers 64] [--context 32768]
    python -m qwenny_b200.microbench sampler [--rows 5] [--top-k 50] [--top-p 0.95] [--penalty 1.1] [--draft-rows 0]

Each prints CUDA-event timings (launches replayed from a CUDA graph, inputs larger than L2 where the shape allows)
and is small enough to sit under `ncu` (-k <kernel> -s <warm-up launches> -c <few>). Synthetic inputs, seeded.
"""
from __future__ import annotations

import argparse
import math

import numpy as np
import torch

from . import model as M
from .ops import Context


def _time_graph(fn, stream, reps):
    with torch.cuda.stream(stream):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for _ in range(reps):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def gemv(args):
    ctx = Context(0)
    ctx.set_pdl(not args.no_pdl)
    if args.tune:
        ctx.tune(*[int(v) for v in args.tune.split(",")])
    if args.probe:
        from ._lib import lib
        lib().qb_marlin_probe(ctx.h, args.probe)
    n, k, m = args.n, args.k, args.rows
    nbuf = max(2, min(8, int(300e6 / (n * k * 0.516)) + 1))  # weight buffers in rotation: more than L2 in total
    if args.hot:
        nbuf = 1  # the same weights every launch: L2-resident when they fit
    g = torch.Generator(device="cuda").manual_seed(0)
    bufs = [M.Marlin.random(n, k, g) for _ in range(nbuf)]
    x = torch.randn(m, k, generator=g, device="cuda").half()
    y = torch.empty(m, n // 2, dtype=torch.float16, device="cuda") if args.epi == "silu" else torch.empty(m, n, device="cuda")
    keys = torch.zeros(64, dtype=torch.int64, device="cuda")
    i = [0]

    def one():
        w = bufs[i[0] % nbuf]
        i[0] += 1
        ctx.marlin_gemm(x, w.words, w.scales, epi=args.epi, y=y, keys=keys if args.epi == "argmax" else None)
    if args.plain:
        for _ in range(args.reps):
            one()
        torch.cuda.synchronize()
        print(f"gemv N={n} K={k} rows={m} epi={args.epi}: {args.reps} plain launches done, device error {ctx.device_error()}")
        return
    us = _time_graph(one, torch.cuda.Stream(), args.reps)
    by = n * k * 0.515625
    print(f"gemv N={n} K={k} rows={m} epi={args.epi}: {us:.2f} us/launch, {by / us / 1e3:.0f} GB/s of {by / 1e6:.1f} MB, "
          f"{2.0 * m * n * k / us / 1e6:.1f} TFLOP/s; device error {ctx.device_error()}")


def attn(args):
    ctx = Context(0)
    NH, NKV, HD, MIX = M.NH, M.NKV, M.HD, M.MIX
    n, pos0 = args.rows, args.context
    cap = (pos0 + n + 63) // 64 * 64
    g = torch.Generator(device="cuda").manual_seed(75)
    kc = torch.randint(1, 256, (NKV * cap * HD,), generator=g, dtype=torch.uint8, device="cuda")
    vc = torch.randint(1, 256, (NKV * cap * HD,), generator=g, dtype=torch.uint8, device="cuda")
    ks = (torch.randn(NKV * cap, generator=g, device="cuda") * 0.05).abs()
    vs = (torch.randn(NKV * cap, generator=g, device="cuda") * 0.05).abs()
    q = torch.randn(n, NH, HD, generator=g, device="cuda") * (math.log2(math.e) / 16)
    gate = torch.sigmoid(torch.randn(n, MIX, generator=g, device="cuda"))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    dev = dict(dseg=i32([0, n]), dtok=i32(list(range(n))), dkeys=i32([pos0 + n] * n), tok_slot=i32([0] * n),
               tok_pos=i32([pos0 + i for i in range(n)]))
    st = dict(ndseg=1, ndec=n, dmax=n, dec_max_pos=pos0 + n - 1)
    ml = torch.zeros(64 * 128 * NH * 2, device="cuda")
    acc = torch.zeros(64 * 128 * NH * HD, device="cuda")
    out = gate.clone()
    mix = torch.zeros(n, MIX, dtype=torch.float16, device="cuda")

    if n > 8:  # a prompt segment: tiles of 10 tokens
        tiles = []
        for o in range(0, n, 10):
            tiles += [o, min(10, n - o)]
        dev["ptile"] = i32(tiles)
        st = dict(ntile=len(tiles) // 2, tile_max_pos=pos0 + n - 1)

    def one():
        if n > 8:
            ctx.attn_prefill(q, kc, vc, ks, vs, dev, st, cap, ml, acc, out, mix)
        else:
            ctx.attn_decode(q, kc, vc, ks, vs, dev, st, cap, ml, acc, out, mix)
    if args.plain:
        for _ in range(args.reps):
            one()
        torch.cuda.synchronize()
        print(f"attn context={pos0} rows={n}: {args.reps} plain launches done, device error {ctx.device_error()}")
        return
    us = _time_graph(one, torch.cuda.Stream(), args.reps)
    by = NKV * 520 * (pos0 + n)
    if n > 8:
        fl = 4.0 * HD * NH * sum(pos0 + i + 1 for i in range(n))  # causal: row i sees pos0 + i + 1 keys
        print(f"attn context={pos0} rows={n}: {us:.1f} us per prompt attention, {fl / us / 1e6:.1f} TFLOP/s; "
              f"device error {ctx.device_error()}")
        return
    print(f"attn context={pos0} rows={n}: {us:.2f} us per decode + combine, {by / us / 1e3:.0f} GB/s of {by / 1e6:.1f} MB; "
          f"device error {ctx.device_error()}")


def step(args):
    ctx = Context(0)
    ctx.set_pdl(not args.no_pdl)
    m = M.synthetic(ctx, nlayers=args.layers, position=args.context, max_ctx=32768)
    m.use_graphs(not args.no_graph)
    m.use_fork(not args.no_fork)
    if args.lora:  # a LoRA of that rank on every product of every layer; the step's slot uses it
        M.synthetic_adapter(m, rank=args.lora)
        m.set_slot_scale(0, 2.0)
    toks = [(1000 + i, 0, args.context + i) for i in range(args.rows)]
    out = list(range(args.rows)) if args.rows <= 16 else [args.rows - 1]  # a prompt chunk wants its last row only
    for _ in range(2):
        m.step(toks, out)
    m.argmax()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(m.stream)
    for _ in range(args.steps):
        m.step(toks, out)
    e1.record(m.stream)
    tok = m.argmax()
    ms = e0.elapsed_time(e1) / args.steps
    print(f"step layers={args.layers} rows={args.rows} context={args.context} lora={args.lora}: {ms * 1e3:.1f} us/step, "
          f"{m.step_kernels} kernels, greedy {tok}, device error {ctx.device_error()}")


def prefill(args):
    """A whole prompt through the full model in chunks (the prefill configuration of the benchmark: 32768 tokens in
    2048-row chunks, 64 layers); reports the time of every chunk and the prompt's tok/s."""
    ctx = Context(0)
    ctx.set_pdl(True)
    m = M.synthetic(ctx, nlayers=args.layers, max_ctx=args.prompt, vocab=151936)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 151936, (args.prompt,), generator=g).tolist()
    chunks = [(a, min(args.prompt, a + args.chunk)) for a in range(0, args.prompt, args.chunk)]
    for rep in range(2):  # the first pass warms up (kernel attributes, caches); the DeltaNet states restart at position 0
        times = []
        for a, b in chunks:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(m.stream)
            m.step([(ids[i], 0, i) for i in range(a, b)], [b - a - 1])
            e1.record(m.stream)
            times.append((e0, e1))
        tok = m.argmax()
        ms = [x.elapsed_time(y) for x, y in times]
    tot = sum(ms)
    print(f"prefill layers={args.layers} prompt={args.prompt} chunk={args.chunk}: {tot:.1f} ms = {args.prompt / tot * 1e3:.0f} tok/s; "
          f"first chunk {ms[0]:.1f} ms, last chunk {ms[-1]:.1f} ms; greedy {tok}, device error {ctx.device_error()}")


def draft(args):
    """The MTP draft chain: k greedy drafts for one sequence after a verify step (one target layer stands in for the
    stack: the chain's cost does not depend on it). MTP layer at the 27B widths, context as given, draft head of
    --draft-rows rows (0: the whole output layer)."""
    ctx = Context(0)
    ctx.set_pdl(True)
    m = M.synthetic(ctx, nlayers=1, position=args.context, max_ctx=32768, pattern=("attn",), mtp=True,
                    draft_rows=args.draft_rows)
    toks = [(1000 + i, 0, args.context + i) for i in range(5)]
    m.step(toks, list(range(5)))
    got = m.argmax()
    mt = [(got[i], 0, args.context + i + 1) for i in range(5)]
    for _ in range(3):
        d = m.draft(mt, list(range(5)), [4], args.k)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(m.stream)
    for _ in range(args.reps):
        d = m.draft(mt, list(range(5)), [4], args.k)
    e1.record(m.stream)
    torch.cuda.synchronize()
    print(f"draft chain k={args.k} context={args.context} draft_rows={args.draft_rows}: "
          f"{e0.elapsed_time(e1) / args.reps * 1e3:.1f} us per chain (host round trip included), drafts {d}, "
          f"device error {ctx.device_error()}")


def sampler(args):
    """qb_sample_rows over --rows logit rows of the 27B vocabulary (or qb_draft_sample over a draft head of
    --draft-rows columns): seeded logits with a few likely tokens, 200 tokens seen per slot."""
    ctx = Context(0)
    ctx.set_pdl(True)
    V, n, QD, QCAP = 248320, args.rows, 16, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    W = args.draft_rows or V
    logits = torch.randn(n, W, generator=g, device="cuda") * (1 if args.top_k == 0 else 2)
    logits[:, ::9973] += 14 if args.top_k == 0 else 6  # top_k 0: as peaked as a language model's, the cut among the candidates
    out_rows = torch.arange(n, dtype=torch.int32, device="cuda")
    tok_slot = torch.zeros(n, dtype=torch.int32, device="cuda")
    ids = torch.randint(0, V, (n,), generator=g, device="cuda", dtype=torch.int32)
    row_first = torch.zeros(n, dtype=torch.int32, device="cuda")
    seen = torch.zeros(V // 32, dtype=torch.int32, device="cuda")
    seen[torch.randint(0, V // 32, (200,), generator=g, device="cuda")] = 1 << 7
    outs = seen.clone()
    qtok = torch.full((QD,), -1, dtype=torch.int32, device="cuda")
    qn = torch.zeros(QD, dtype=torch.int32, device="cuda")
    qid = torch.zeros(QD * QCAP, dtype=torch.int32, device="cuda")
    qp = torch.zeros(QD * QCAP, dtype=torch.float32, device="cuda")
    params = torch.tensor([[args.temperature, args.top_k, args.top_p, args.penalty, 0.37 + 0.1 * j, 0.5, -1, 0.0]
                           for j in range(n)], dtype=torch.float32, device="cuda")
    tok = torch.zeros(n, dtype=torch.int32, device="cuda")
    acc = torch.zeros(n, dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    if args.draft_rows:
        hid = torch.arange(W, dtype=torch.int32, device="cuda") * 3
        params[:, 5] = 0
        one = torch.zeros(1, dtype=torch.int32, device="cuda")  # rows of one launch may not share a (slot, t)
        fn = lambda: ctx.draft_sample(logits, W, W, hid, V, 1, one, tok_slot, seen, outs, params, tok, qtok, qn, qid,
                                      qp)
    else:
        fn = lambda: ctx.sample_rows(logits, V, n, out_rows, tok_slot, ids, row_first, seen, outs, params, qtok, qn,
                                     qid, qp, tok, acc)
    if args.plain:
        with torch.cuda.stream(stream):
            for _ in range(args.reps):
                fn()
        torch.cuda.synchronize()
        us = float("nan")
    else:
        us = _time_graph(fn, stream, args.reps)
    print(f"sampler rows={1 if args.draft_rows else n} width={W} top_k={args.top_k} top_p={args.top_p} "
          f"penalty={args.penalty}: {us:.1f} us per launch, tokens {tok.tolist()}, device error {ctx.device_error()}")


def session(args):
    """A slot's saved images at the 27B shapes: save_kv / load_kv of positions [0, context) and save_state /
    load_state, host side in pinned memory; wall-clock per call (each call waits for its copy)."""
    import time
    ctx = Context(0)
    ctx.set_pdl(True)
    m = M.synthetic(ctx, nlayers=args.layers, position=args.context - 8, max_ctx=args.context)
    from ._lib import lib
    n = lib().qb_model_kv_bytes(m.h, 0, args.context)
    pinned = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    buf = pinned.numpy()
    res = {}
    for name, fn in (("save_kv", lambda: m.save_kv(0, 0, args.context, out=buf)),
                     ("load_kv", lambda: m.load_kv(0, 0, args.context, buf)),
                     ("save_state", lambda: m.save_state(0)),):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.reps):
            r = fn()
        torch.cuda.synchronize()
        res[name] = (time.perf_counter() - t0) / args.reps
    st, pos = r
    t0 = time.perf_counter()
    for _ in range(args.reps):
        m.load_state(0, st, pos)
    res["load_state"] = (time.perf_counter() - t0) / args.reps
    print(f"session layers={args.layers} context={args.context}: kv image {n / 1e6:.1f} MB (host side pinned), state "
          f"image {len(st) / 1e6:.1f} MB (host side pageable); " +
          ", ".join(f"{k} {v * 1e3:.2f} ms ({(n if 'kv' in k else len(st)) / v / 1e9:.1f} GB/s)" for k, v in res.items()) +
          f"; device error {ctx.device_error()}")


def delta(args):
    """The DeltaNet kernels of one prompt segment: conv once, then the rule kernel timed alone."""
    ctx = Context(0)
    n = args.rows
    g = torch.Generator(device="cuda").manual_seed(0)
    LQKV, DELTA_IN, LVH, CVW, MIX = 10240, 16384, 48, 10336, 6144
    sst = (2 * 48 * 128 * 128 + 2 * 16 * 8288 + 32 * LQKV + 1023) // 1024 * 1024
    part = torch.randn(1, n, DELTA_IN, generator=g, device="cuda")
    ba = torch.randn(1, n, 2 * LVH, generator=g, device="cuda")
    conv_w = torch.randn(LQKV, 4, generator=g, device="cuda") * 0.3
    a_log, dt_bias = torch.randn(LVH, generator=g, device="cuda") * 0.5, torch.randn(LVH, generator=g, device="cuda") * 0.5
    mem = torch.zeros(sst, device="cuda")
    meta = torch.tensor([[-1, 0, 0, 0]], dtype=torch.int32, device="cuda")
    dev = {k: torch.zeros(n + 8, dtype=torch.int32, device="cuda") for k in ("tok_slot", "seg_start", "seg_slot", "seg_pos0")}
    dev["tok_pos"] = torch.arange(n + 8, dtype=torch.int32, device="cuda")
    dev["seg_len"] = torch.full((8,), n, dtype=torch.int32, device="cuda")
    cv = torch.zeros(n, CVW, device="cuda")
    o = torch.zeros(n, MIX, device="cuda")
    if n <= 29:
        # a decode / verify step: the one-launch mixer, continuing a sequence at position 1000
        from ._lib import lib
        norm_w = torch.ones(128, device="cuda")
        dev["tok_pos"] = torch.arange(1000, 1000 + n + 8, dtype=torch.int32, device="cuda")
        dev["seg_pos0"] = torch.full((8,), 1000, dtype=torch.int32, device="cuda")
        mems = [torch.randn(sst, device="cuda") * 0.01 for _ in range(20)]  # states in rotation: 3 MB each
        y = torch.zeros(n, MIX, dtype=torch.float16, device="cuda")
        i = [0]

        def one():
            meta.copy_(torch.tensor([[1000, 1000, 0, 0]], dtype=torch.int32))
            ctx.delta_mixer(part, 1, n, ba, 1, conv_w, a_log, dt_bias, norm_w, mems[i[0] % 20], sst, meta, None, y, dev, 1)
            i[0] += 1
        for _ in range(3):
            one()
        torch.cuda.synchronize()
        buf = torch.zeros(4096, dtype=torch.int64, device="cuda")
        lib().qb_marlin_trace(ctx.h, buf.data_ptr())
        one()
        torch.cuda.synchronize()
        lib().qb_marlin_trace(ctx.h, None)
        t = buf[:96 * 10].view(96, 10).cpu().numpy().astype(np.float64)
        t0 = t[:, 0].min()
        names = ["start", "dependencies done", "loads", "conv", "l2 norm", "kq, bank, ring", "recurrence", "norm + write", "state stored"]
        for j, nm in enumerate(names):
            c = t[:, j] - t0
            print(f"  {nm:18s} min {c.min() / 1e3:6.2f}  median {np.median(c) / 1e3:6.2f}  max {c.max() / 1e3:6.2f} us")
        print("device error", ctx.device_error())
        return
    norm_w = torch.ones(128, device="cuda")
    y = torch.zeros(n, MIX, dtype=torch.float16, device="cuda")
    meta2 = meta.clone()

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / args.reps
    us_conv = timed(lambda: ctx.delta_conv(part, 1, n, ba, 1, conv_w, a_log, dt_bias, mem, sst, cv, dev))
    us = timed(lambda: ctx.delta_rule(part, 1, n, cv, mem, sst, meta, o, dev, 1))
    us_norm = timed(lambda: ctx.delta_norm(part, 1, n, norm_w, o, y, meta2, dev, 1))
    print(f"delta rows={n}: conv {us_conv:.1f} us, rule {us:.1f} us = {us * 1e3 / n:.0f} ns/token, norm {us_norm:.1f} us; "
          f"device error {ctx.device_error()}")


def main():
    ap = argparse.ArgumentParser(prog="python -m qwenny_b200.microbench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("gemv")
    a.add_argument("n", type=int); a.add_argument("k", type=int)
    a.add_argument("--rows", type=int, default=5); a.add_argument("--epi", default="plain")
    a.add_argument("--reps", type=int, default=24); a.add_argument("--tune", default="")
    a.add_argument("--no-pdl", action="store_true"); a.add_argument("--plain", action="store_true")
    a.add_argument("--probe", type=int, default=0, help="1: time the copy pipeline alone (no arithmetic)")
    a.add_argument("--hot", action="store_true", help="one weight buffer: L2-resident weights")
    a.set_defaults(fn=gemv)
    b = sub.add_parser("attn")
    b.add_argument("--context", type=int, default=32000); b.add_argument("--rows", type=int, default=5)
    b.add_argument("--reps", type=int, default=20); b.add_argument("--plain", action="store_true")
    b.set_defaults(fn=attn)
    c = sub.add_parser("step")
    c.add_argument("--layers", type=int, default=8); c.add_argument("--steps", type=int, default=3)
    c.add_argument("--rows", type=int, default=5); c.add_argument("--context", type=int, default=32000)
    c.add_argument("--no-graph", action="store_true"); c.add_argument("--no-pdl", action="store_true")
    c.add_argument("--no-fork", action="store_true", help="the 16-bit in-projection in line instead of on a second stream")
    c.add_argument("--lora", type=int, default=0, help="rank of an unmerged LoRA on every layer (0: none)")
    c.set_defaults(fn=step)
    f = sub.add_parser("prefill")
    f.add_argument("--layers", type=int, default=64); f.add_argument("--prompt", type=int, default=32768)
    f.add_argument("--chunk", type=int, default=2048)
    f.set_defaults(fn=prefill)
    h = sub.add_parser("draft")
    h.add_argument("--k", type=int, default=4); h.add_argument("--context", type=int, default=32000)
    h.add_argument("--draft-rows", type=int, default=65536); h.add_argument("--reps", type=int, default=20)
    h.set_defaults(fn=draft)
    e = sub.add_parser("delta")
    e.add_argument("--rows", type=int, default=2048); e.add_argument("--reps", type=int, default=5)
    e.set_defaults(fn=delta)
    ss = sub.add_parser("session")
    ss.add_argument("--layers", type=int, default=64); ss.add_argument("--context", type=int, default=32768)
    ss.add_argument("--reps", type=int, default=3)
    ss.set_defaults(fn=session)
    sp = sub.add_parser("sampler")
    sp.add_argument("--rows", type=int, default=5); sp.add_argument("--top-k", type=int, default=50)
    sp.add_argument("--top-p", type=float, default=0.95); sp.add_argument("--penalty", type=float, default=1.1)
    sp.add_argument("--temperature", type=float, default=0.8); sp.add_argument("--draft-rows", type=int, default=0)
    sp.add_argument("--reps", type=int, default=20); sp.add_argument("--plain", action="store_true")
    sp.set_defaults(fn=sampler)
    args = ap.parse_args()
    args.fn(args)


if __name__ == "__main__":
    main()
