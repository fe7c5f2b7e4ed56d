"""Parity of the gated int8-KV attention kernels: library vs CPU oracle vs the reference's own kernels (oracle/_ref) on
the same device buffers. Tolerances: quantisation codes bit-exact; outputs 1e-2 relative / 2e-3 absolute after
rounding to bf16 (the benchmark's stated tolerance)."""
import math

import numpy as np
import pytest
import torch

from oracle import ref_cuda
from oracle import ref_ops as R
from qwenny_b200 import synth

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 2e-3
QSCALE = math.log2(math.e) / 16.0


def bf16(a):
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def close(a, b):
    a, b = bf16(a), bf16(b)
    return np.abs(a - b) <= ATOL + RTOL * np.abs(b)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_cache(slots, cap, g, filled):
    """Random cache: code bytes uniform in 1..255 (code + 128, i.e. -127..127), scales |N(0, 0.05)|."""
    kc = torch.randint(1, 256, (slots * R.NKV * cap * R.HD,), generator=g, dtype=torch.uint8)
    vc = torch.randint(1, 256, (slots * R.NKV * cap * R.HD,), generator=g, dtype=torch.uint8)
    ks = (torch.randn(slots * R.NKV * cap, generator=g) * 0.05).abs()
    vs = (torch.randn(slots * R.NKV * cap, generator=g) * 0.05).abs()
    return kc, vc, ks, vs


@pytest.mark.parametrize("splits", [1, 2])
def test_attn_prep(ctx, ref, splits):
    g = synth.gen(60 + splits)
    n, slots, cap = 5, 2, 1024
    part = torch.randn(splits, n, R.ATTN_IN, generator=g)
    qn, kn = 1 + torch.randn(R.HD, generator=g) * 0.02, 1 + torch.randn(R.HD, generator=g) * 0.02
    inv = torch.from_numpy(R.rope_inv_freq())
    toks = [(0, 1, 700 + i) for i in range(n)]
    st = R.build_step(toks, list(range(n)))
    dv = ref_cuda.upload_step(st)
    outs = []
    for impl in (ctx, ref):
        q = torch.zeros(n, R.NH, R.HD, device="cuda")
        o = torch.zeros(n, R.MIX, device="cuda")
        kc = torch.zeros(slots * R.NKV * cap * R.HD, dtype=torch.uint8, device="cuda")
        vc = torch.zeros_like(kc)
        ks = torch.zeros(slots * R.NKV * cap, device="cuda")
        vs = torch.zeros_like(ks)
        impl.attn_prep(part.cuda(), splits, n, qn.cuda(), kn.cuda(), inv.cuda(), QSCALE, q, o, kc, vc, ks, vs,
                       dv["tok_slot"], dv["tok_pos"], cap)
        outs.append([t.cpu().numpy() for t in (q, o, kc, vc, ks, vs)])
    mine, theirs = outs
    # against the reference's kernel: the quantisation codes are bit-exact; scales and q agree to an f32 ulp (the two
    # compilations contract the RoPE rotation into FMAs differently)
    assert np.array_equal(mine[2], theirs[2]) and np.array_equal(mine[3], theirs[3])
    assert np.allclose(mine[4], theirs[4], rtol=2e-7, atol=0) and np.array_equal(mine[5], theirs[5])
    assert np.allclose(mine[0], theirs[0], rtol=1e-6, atol=1e-7) and np.array_equal(mine[1], theirs[1])
    # against the CPU oracle
    qo, go, k, v = R.attn_prep(part.numpy(), qn.numpy(), kn.numpy(), inv.numpy(), QSCALE, st["tok_pos"])
    assert np.allclose(mine[0], qo, rtol=1e-4, atol=1e-5) and np.allclose(mine[1], go, rtol=1e-5, atol=1e-6)
    kc0 = np.zeros(slots * R.NKV * cap * R.HD, dtype=np.uint8); vc0 = kc0.copy()
    ks0 = np.zeros(slots * R.NKV * cap, dtype=np.float32); vs0 = ks0.copy()
    R.kv_store(kc0, vc0, ks0, vs0, k, v, st["tok_slot"], st["tok_pos"], cap)
    assert np.allclose(mine[4], ks0, rtol=1e-5) and np.allclose(mine[5], vs0, rtol=1e-6)
    # the oracle norms in f64: a code may differ by one where the value sits on a rounding boundary
    for a, b in ((mine[2], kc0), (mine[3], vc0)):
        d = np.abs(a.astype(np.int32) - b.astype(np.int32))
        assert d.max() <= 1 and (d > 0).mean() < 1e-3
    # untouched cache bytes stay zero: exactly n * NKV * HD bytes written per cache
    assert (mine[2] != 0).sum() <= n * R.NKV * R.HD and (mine[3] != 0).sum() <= n * R.NKV * R.HD


def run_decode(impl, q, gate, cache, st, dv, cap, n, mix=False):
    kc, vc, ks, vs = cache
    out = gate.clone()
    ml = torch.zeros(64 * 128 * R.NH * 2, device="cuda")
    acc = torch.zeros(64 * 128 * R.NH * R.HD, device="cuda")
    if isinstance(impl, ref_cuda.RefModule):
        impl.attn_decode(q, kc, vc, ks, vs, st, dv, cap, ml, acc, out)
        return out
    m = torch.zeros(n, R.MIX, dtype=torch.float16, device="cuda") if mix else None
    impl.attn_decode(q, kc, vc, ks, vs, dv, st, cap, ml, acc, out, m)
    return (out, m) if mix else out


@pytest.mark.parametrize("pos0,n,cap", [(295, 5, 512), (0, 1, 512), (60, 8, 512), (4100, 3, 8192), (32763, 5, 32768)])
def test_attn_decode(ctx, ref, pos0, n, cap):
    """(32763, 5, 32768) is the benchmark's attention configuration: 5 causal rows over a 32768-token context."""
    g = synth.gen(70 + n)
    cache = make_cache(1, cap, g, pos0 + n)
    q = torch.randn(n, R.NH, R.HD, generator=g) * QSCALE
    gate = torch.sigmoid(torch.randn(n, R.MIX, generator=g))
    toks = [(0, 0, pos0 + i) for i in range(n)]
    st = R.build_step(toks, list(range(n)))
    dv = ref_cuda.upload_step(st)
    dc = [t.cuda() for t in cache]
    mine, mix = run_decode(ctx, q.cuda(), gate.cuda(), dc, st, dv, cap, n, mix=True)
    theirs = run_decode(ref, q.cuda(), gate.cuda(), dc, st, dv, cap, n)
    a, b = mine.cpu().numpy(), theirs.cpu().numpy()
    assert close(a, b).all()
    assert torch.equal(mix, mine.half())
    want = R.attn_decode(q.numpy(), gate.numpy(), *[t.numpy() for t in cache], st["tok_slot"], st["tok_pos"], cap)
    assert close(a, want).all() and close(b, want).all()


def test_attn_decode_row_invariance_and_two_slots(ctx):
    """A token's attention is bit-identical alone or next to drafts, and with another slot's segment in the step."""
    g = synth.gen(80)
    cap = 2048
    cache = [t.cuda() for t in make_cache(2, cap, g, 0)]
    q = (torch.randn(8, R.NH, R.HD, generator=g) * QSCALE).cuda()
    gate = torch.sigmoid(torch.randn(8, R.MIX, generator=g)).cuda()
    toks = [(0, 1, 900 + i) for i in range(5)] + [(0, 0, 130 + i) for i in range(3)]
    st = R.build_step(toks, list(range(8)))
    full = run_decode(ctx, q, gate, cache, st, ref_cuda.upload_step(st), cap, 8)
    for t in (0, 4, 6):
        st1 = R.build_step([toks[t]], [0])
        one = run_decode(ctx, q[t:t + 1].contiguous(), gate[t:t + 1].contiguous(), cache, st1,
                         ref_cuda.upload_step(st1), cap, 1)
        assert torch.equal(one[0], full[t])


def test_attn_decode_more_than_64_decode_tokens(ctx):
    """Up to 64 decode tokens in a call, the kernel requests the cache entries that lie 64 positions or more before a
    segment's last key ahead of the kernel enqueued before it; with more it waits first. 13 slots x 5 tokens = 65
    tokens (the host's planner stops at 64; the C entry point does not), with programmatic dependent launch on, against
    the CPU oracle on three of the rows, and bit for bit against the same rows run as 13 calls of 5 tokens."""
    g = synth.gen(88)
    slots, cap, n = 13, 512, 65
    cache = make_cache(slots, cap, g, 0)
    dc = [t.cuda() for t in cache]
    q = torch.randn(n, R.NH, R.HD, generator=g) * QSCALE
    gate = torch.sigmoid(torch.randn(n, R.MIX, generator=g))
    toks = [(0, s, 300 + 7 * s + i) for s in range(slots) for i in range(5)]
    st = R.build_step(toks, list(range(n)), max_dec=128)
    assert st["ndec"] == 65 and st["ntile"] == 0
    ctx.set_pdl(True)
    try:
        full = run_decode(ctx, q.cuda(), gate.cuda(), dc, st, ref_cuda.upload_step(st), cap, n)
        for s in (0, 6, 12):
            st1 = R.build_step(toks[5 * s:5 * s + 5], list(range(5)))
            one = run_decode(ctx, q[5 * s:5 * s + 5].cuda().contiguous(), gate[5 * s:5 * s + 5].cuda().contiguous(), dc, st1,
                             ref_cuda.upload_step(st1), cap, 5)
            assert torch.equal(one, full[5 * s:5 * s + 5])
    finally:
        ctx.set_pdl(False)
    rows = [0, 32, 64]
    want = R.attn_decode(q.numpy()[rows], gate.numpy()[rows], *[t.numpy() for t in cache], st["tok_slot"][rows],
                         st["tok_pos"][rows], cap)
    assert close(full.cpu().numpy()[rows], want).all()


def run_prefill(impl, q, gate, cache, st, dv, cap, n, mix=False):
    kc, vc, ks, vs = cache
    out = gate.clone()
    pairs = 256 * 16
    ml = torch.zeros(pairs * R.NH * 2, device="cuda")
    acc = torch.zeros(pairs * R.NH * R.HD, device="cuda")
    if isinstance(impl, ref_cuda.RefModule):
        impl.attn_prefill(q, kc, vc, ks, vs, st, dv, cap, ml, acc, out)
        return out
    m = torch.zeros(n, R.MIX, dtype=torch.float16, device="cuda") if mix else None
    impl.attn_prefill(q, kc, vc, ks, vs, dv, st, cap, ml, acc, out, m)
    return (out, m) if mix else out


@pytest.mark.parametrize("pos0,n,cap,check", [
    (0, 64, 512, 64),            # a prompt from position 0: the first tile sees 10 keys
    (295, 23, 512, 23),          # ragged last tile, keys cross a 64-key block inside a tile
    (4000, 100, 8192, 12),       # ten tiles, key splits
    (32700, 17, 32768, 4),       # two tiles at the end of a long context: 32 splits
    (0, 2048, 2048, 6),          # the benchmark's prompt chunk, first chunk
    (30720, 2048, 32768, 3),     # ... and its last chunk of a 32768-token prompt
])
def test_attn_prefill(ctx, ref, pos0, n, cap, check):
    """Prompt tiles against the reference's attn_prefill kernel (every row) and the CPU oracle (`check` rows spread
    over the step: the oracle walks every key of every head in numpy)."""
    g = synth.gen(90 + n)
    cache = make_cache(1, cap, g, pos0 + n)
    q = torch.randn(n, R.NH, R.HD, generator=g) * QSCALE
    gate = torch.sigmoid(torch.randn(n, R.MIX, generator=g))
    toks = [(0, 0, pos0 + i) for i in range(n)]
    st = R.build_step(toks, list(range(n)), short=0)
    assert st["ndec"] == 0 and st["ntile"] == -(-n // 10)
    dv = ref_cuda.upload_step(st)
    dc = [t.cuda() for t in cache]
    mine, mix = run_prefill(ctx, q.cuda(), gate.cuda(), dc, st, dv, cap, n, mix=True)
    theirs = run_prefill(ref, q.cuda(), gate.cuda(), dc, st, dv, cap, n)
    assert ctx.device_error() == 0
    a, b = mine.cpu().numpy(), theirs.cpu().numpy()
    assert close(a, b).all()
    assert np.array_equal(mix.cpu().numpy(), a.astype(np.float16))
    rows = sorted(set(np.linspace(0, n - 1, check).astype(int).tolist()))
    want = R.attn_decode(q.numpy()[rows], gate.numpy()[rows], *[t.numpy() for t in cache],
                         st["tok_slot"][rows], st["tok_pos"][rows], cap)
    assert close(a[rows], want).all() and close(b[rows], want).all()


def test_attn_prefill_matches_decode_rows(ctx):
    """A token's attention as part of a prompt tile and as a lone decode token agree within the output tolerance (different key
    splits round P to f16 against different running maxima), and a mixed step (one short segment, one long) runs both kernels on one `out`."""
    g = synth.gen(99)
    cap = 4096
    cache = [t.cuda() for t in make_cache(2, cap, g, 0)]
    n = 3 + 40
    q = (torch.randn(n, R.NH, R.HD, generator=g) * QSCALE).cuda()
    gate = torch.sigmoid(torch.randn(n, R.MIX, generator=g)).cuda()
    toks = [(0, 1, 2000 + i) for i in range(3)] + [(0, 0, 700 + i) for i in range(40)]
    st = R.build_step(toks, list(range(n)))
    assert st["ndec"] == 3 and st["ntile"] == 4
    dv = ref_cuda.upload_step(st)
    kc, vc, ks, vs = cache
    out = gate.clone()
    ml = torch.zeros(4096 * R.NH * 2, device="cuda")
    acc = torch.zeros(4096 * R.NH * R.HD, device="cuda")
    ctx.attn_decode(q, kc, vc, ks, vs, dv, st, cap, ml, acc, out, None)
    ctx.attn_prefill(q, kc, vc, ks, vs, dv, st, cap, ml, acc, out, None)
    for t in (0, 2, 3, 17, 42):
        st1 = R.build_step([toks[t]], [0])
        one = run_decode(ctx, q[t:t + 1].contiguous(), gate[t:t + 1].contiguous(), cache, st1,
                         ref_cuda.upload_step(st1), cap, 1)
        assert close(out[t].cpu().numpy(), one[0].cpu().numpy()).all()


def test_attn_prefill_pairs_and_segment_boundaries(ctx, ref):
    """Steps with many tiles run two tiles per block. Two prompt segments of 25 and 33 tokens (3 + 4 tiles, one split):
    tiles 0-1 and 4-5 pair up, tiles 2 and 3 belong to different sequences and run one after the other in their
    block, tile 6 is alone."""
    g = synth.gen(131)
    cap = 1024
    cache = make_cache(2, cap, g, 0)
    toks = [(0, 0, 300 + i) for i in range(25)] + [(0, 1, 40 + i) for i in range(33)]
    n = len(toks)
    q = torch.randn(n, R.NH, R.HD, generator=g) * QSCALE
    gate = torch.sigmoid(torch.randn(n, R.MIX, generator=g))
    st = R.build_step(toks, list(range(n)))
    assert st["ndec"] == 0 and st["ntile"] == 7
    dv = ref_cuda.upload_step(st)
    dc = [t.cuda() for t in cache]
    mine, mix = run_prefill(ctx, q.cuda(), gate.cuda(), dc, st, dv, cap, n, mix=True)
    theirs = run_prefill(ref, q.cuda(), gate.cuda(), dc, st, dv, cap, n)
    a, b = mine.cpu().numpy(), theirs.cpu().numpy()
    assert close(a, b).all()
    assert np.array_equal(mix.cpu().numpy(), a.astype(np.float16))
    want = R.attn_decode(q.numpy(), gate.numpy(), *[t.numpy() for t in cache], st["tok_slot"], st["tok_pos"], cap)
    assert close(a, want).all()
