"""Parity of the Gated DeltaNet kernels: library vs CPU oracle (f64 state) vs the reference's own kernels
(oracle/_ref) on the same device buffers; the rollback plan's bit-exactness property. Tolerances: f32 state within
1e-4, outputs 1e-2 relative / 2e-3 absolute after rounding to bf16."""
import numpy as np
import pytest
import torch

from oracle import ref_cuda
from oracle import ref_ops as R
from qwenny_b200 import synth

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 2e-3
SST = (R.SLOT_FLOATS + 1023) // 1024 * 1024


def bf16(a):
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def close(a, b):
    a, b = bf16(a), bf16(b)
    return np.abs(a - b) <= ATOL + RTOL * np.abs(b)


def weights(g):
    conv_w = torch.randn(R.LQKV, 4, generator=g) * 0.3
    a_log = torch.randn(R.LV_HEADS, generator=g) * 0.5
    dt_bias = torch.randn(R.LV_HEADS, generator=g) * 0.5
    norm_w = 1 + torch.randn(R.LVD, generator=g) * 0.02
    return conv_w, a_log, dt_bias, norm_w


def fresh_mem(slots, g):
    """Slot memory with a random state N(0, 0.01) in both buffers, random banks and ring."""
    mem = torch.randn(slots * SST, generator=g) * 0.01
    return mem


def test_delta_conv(ctx, ref):
    g = synth.gen(90)
    n, slots = 6, 2
    conv_w, a_log, dt_bias, _ = weights(g)
    part = torch.randn(2, n, R.DELTA_IN, generator=g)
    ba = torch.randn(3, n, 2 * R.LV_HEADS, generator=g)
    mem = fresh_mem(slots, g)
    toks = [(0, 1, 40 + i) for i in range(4)] + [(0, 0, 1), (0, 0, 2)]  # slot 0 near the sequence start
    st = R.build_step(toks, [0])
    dv = ref_cuda.upload_step(st)
    args = [t.cuda() for t in (part, ba, conv_w, a_log, dt_bias, mem)]
    cv1 = torch.zeros(n, R.CVW, device="cuda")
    cv2 = torch.zeros_like(cv1)
    ctx.delta_conv(args[0], 2, n, args[1], 3, args[2], args[3], args[4], args[5], SST, cv1, dv)
    ref.delta(args[0], 2, n, args[1], 3, args[2], args[3], args[4], None, args[5], SST, None, cv2, None, None, st, dv,
              which=("conv",))
    want = R.delta_conv(part.numpy(), ba.numpy(), conv_w.numpy(), a_log.numpy(), dt_bias.numpy(), mem.numpy(), SST,
                        st["tok_slot"], st["tok_pos"])
    a, b = cv1.cpu().numpy(), cv2.cpu().numpy()
    assert np.allclose(a, b, rtol=1e-5, atol=1e-6)
    assert np.allclose(a, want, rtol=2e-4, atol=1e-5)


def rule_inputs(g, n):
    """cv rows as delta_conv leaves them: q, k L2-normalised (q also / sqrt(128)), v N(0,1), exp(g), beta."""
    q = torch.nn.functional.normalize(torch.randn(n, R.LK_HEADS, R.LKD, generator=g), dim=-1) / R.LKD ** 0.5
    k = torch.nn.functional.normalize(torch.randn(n, R.LK_HEADS, R.LKD, generator=g), dim=-1)
    v = torch.randn(n, R.LV_HEADS * R.LVD, generator=g)
    e = torch.exp(-torch.nn.functional.softplus(torch.randn(n, R.LV_HEADS, generator=g)))
    b = torch.sigmoid(torch.randn(n, R.LV_HEADS, generator=g))
    return torch.cat([q.reshape(n, -1), k.reshape(n, -1), v, e, b], dim=1).contiguous()


def test_delta_rule_config1(ctx, ref):
    """The benchmark's DeltaNet configuration: f32 state [48,128,128] ~ N(0, 0.01), 5 sequential rows, batch 1."""
    g = synth.gen(1)
    n, p0 = 5, 32000
    mem = fresh_mem(1, g)
    cv = rule_inputs(g, n)
    part = torch.randn(1, n, R.DELTA_IN, generator=g)
    meta = torch.tensor([[p0, p0 - 5, 0, 0]], dtype=torch.int32)
    st = R.build_step([(0, 0, p0 + i) for i in range(n)], [0])
    dv = ref_cuda.upload_step(st)
    m1, m2 = mem.cuda(), mem.cuda()
    o1, o2 = torch.zeros(n, R.MIX, device="cuda"), torch.zeros(n, R.MIX, device="cuda")
    md = meta.cuda()
    ctx.delta_rule(part.cuda(), 1, n, cv.cuda(), m1, SST, md, o1, dv, 1)
    ref.delta(part.cuda(), 1, n, None, 0, None, None, None, None, m2, SST, md, cv.cuda(), o2, None, st, dv,
              which=("rule",))
    mo = mem.numpy().copy()
    want = R.delta_rule(part.numpy(), cv.numpy(), mo, SST, meta.numpy(), st["seg_start"], st["seg_len"],
                        st["seg_slot"], st["seg_pos0"])
    a, b = o1.cpu().numpy(), o2.cpu().numpy()
    assert close(a, b).all() and close(a, want).all()
    assert np.abs(a - want).max() < 1e-4
    s1, s2 = m1.cpu().numpy(), m2.cpu().numpy()
    # f32 state within 1e-4 of the f64 oracle and of the reference's kernel; banks and ring are copies: exact
    assert np.abs(s1[:2 * R.SLOT_STATE] - mo[:2 * R.SLOT_STATE]).max() < 1e-4
    assert np.abs(s1[:2 * R.SLOT_STATE] - s2[:2 * R.SLOT_STATE]).max() < 1e-4
    assert np.array_equal(s1[2 * R.SLOT_STATE:R.SLOT_FLOATS], s2[2 * R.SLOT_STATE:R.SLOT_FLOATS])
    assert np.array_equal(s1[2 * R.SLOT_STATE:R.SLOT_FLOATS], mo[2 * R.SLOT_STATE:R.SLOT_FLOATS])


def test_delta_norm(ctx, ref):
    g = synth.gen(92)
    n = 7
    _, _, _, norm_w = weights(g)
    part = torch.randn(2, n, R.DELTA_IN, generator=g)
    out = torch.randn(n, R.MIX, generator=g)
    meta = torch.tensor([[-1, 0, 0, 0], [50, 45, 1, 0]], dtype=torch.int32)
    st = R.build_step([(0, 1, 50 + i) for i in range(4)] + [(0, 0, i) for i in range(3)], [0])
    dv = ref_cuda.upload_step(st)
    y1 = torch.zeros(n, R.MIX, dtype=torch.float16, device="cuda")
    y2 = torch.zeros_like(y1)
    m1, m2 = meta.cuda(), meta.cuda()
    ctx.delta_norm(part.cuda(), 2, n, norm_w.cuda(), out.cuda(), y1, m1, dv, st["segs"])
    ref.delta(part.cuda(), 2, n, None, 0, None, None, None, norm_w.cuda(), None, SST, m2, None, out.cuda(), y2, st, dv,
              which=("norm",))
    mo = meta.numpy().copy()
    want = R.delta_norm(part.numpy(), norm_w.numpy(), out.numpy(), mo, st["seg_len"], st["seg_slot"], st["seg_pos0"])
    assert torch.equal(m1, m2) and np.array_equal(m1.cpu().numpy(), mo)
    assert np.allclose(y1.float().cpu().numpy(), y2.float().cpu().numpy(), rtol=2e-3, atol=1e-5)
    assert np.allclose(y1.float().cpu().numpy(), want.astype(np.float32), rtol=4e-3, atol=1e-4)


def layer_step(ctx, w, mem, meta, part, ba, toks):
    """One DeltaNet mixer step (conv, rule, norm) through the library; returns (mix f16, raw out)."""
    conv_w, a_log, dt_bias, norm_w = w
    n = len(toks)
    st = R.build_step(toks, [0])
    dv = ref_cuda.upload_step(st)
    cv = torch.zeros(n, R.CVW, device="cuda")
    o = torch.zeros(n, R.MIX, device="cuda")
    y = torch.zeros(n, R.MIX, dtype=torch.float16, device="cuda")
    ctx.delta_conv(part, 1, n, ba, 1, conv_w, a_log, dt_bias, mem, SST, cv, dv)
    ctx.delta_rule(part, 1, n, cv, mem, SST, meta, o, dv, st["segs"])
    ctx.delta_norm(part, 1, n, norm_w, o, y, meta, dv, st["segs"])
    return y, o


def test_rollback_equals_one_token_per_step(ctx):
    """The reference's layercheck / speccheck property: a 5-token verify step of which 2 drafts are accepted, then a
    restart at the first rejected position, leaves exactly the state and outputs of one token per step."""
    g = synth.gen(93)
    w = [t.cuda() for t in weights(g)]
    T = 12
    part = torch.randn(1, T, R.DELTA_IN, generator=g).cuda()
    ba = torch.randn(1, T, 2 * R.LV_HEADS, generator=g).cuda()
    wrong = torch.randn(1, T, R.DELTA_IN, generator=g).cuda()  # the rejected drafts' inputs
    wrong_ba = torch.randn(1, T, 2 * R.LV_HEADS, generator=g).cuda()

    def sl(t, i, j):
        return t[:, i:j].contiguous()

    # A: one token per step
    memA = torch.zeros(SST, device="cuda")
    metaA = torch.tensor([[-1, 0, 0, 0]], dtype=torch.int32, device="cuda")
    outsA = []
    for i in range(T):
        y, _ = layer_step(ctx, w, memA, metaA, sl(part, i, i + 1), sl(ba, i, i + 1), [(0, 0, i)])
        outsA.append(y[0].clone())
    # B: prompt of 4, then verify steps of 5 (1 token + 4 drafts) of which the first 3 positions are right
    memB = torch.zeros(SST, device="cuda")
    metaB = torch.tensor([[-1, 0, 0, 0]], dtype=torch.int32, device="cuda")
    outsB = [None] * T
    y, _ = layer_step(ctx, w, memB, metaB, sl(part, 0, 4), sl(ba, 0, 4), [(0, 0, i) for i in range(4)])
    for i in range(4):
        outsB[i] = y[i].clone()
    pos = 4
    while pos < T:
        nrow = min(5, T - pos)
        good = min(3, nrow)
        p = torch.cat([sl(part, pos, pos + good), sl(wrong, pos + good, pos + nrow)], dim=1).contiguous()
        b = torch.cat([sl(ba, pos, pos + good), sl(wrong_ba, pos + good, pos + nrow)], dim=1).contiguous()
        y, _ = layer_step(ctx, w, memB, metaB, p, b, [(0, 0, pos + i) for i in range(nrow)])
        for i in range(good):
            outsB[pos + i] = y[i].clone()
        pos += good
    for i in range(T):
        assert torch.equal(outsA[i], outsB[i]), f"position {i}"
    # the end states agree bit for bit (each in the buffer its metadata names)
    ma, mb = metaA.cpu().numpy()[0], metaB.cpu().numpy()[0]
    assert ma[0] == T and mb[0] >= T
    # B ended on a verify step that ran past T only if drafts were rejected at the very end; restart it at T to compare
    if mb[0] != T:
        pytest.skip("schedule ended inside a step")
    sa = memA[ma[2] * R.SLOT_STATE:(ma[2] + 1) * R.SLOT_STATE]
    sb = memB[mb[2] * R.SLOT_STATE:(mb[2] + 1) * R.SLOT_STATE]
    assert torch.equal(sa, sb)


@pytest.mark.parametrize("case", ["continue", "restart", "fresh_two_slots", "long"])
def test_fused_mixer_matches_the_three_kernels(ctx, case):
    """Same arithmetic in one launch; the two compilations contract a few multiply-adds differently, so values agree
    to an f32 ulp or two rather than bit for bit (metadata, which positions are written, exactly)."""
    g = synth.gen(95)
    w = [t.cuda() for t in weights(g)]
    slots = 2
    mem = fresh_mem(slots, g).cuda()
    if case == "continue":
        toks, meta = [(0, 1, 300 + i) for i in range(5)], [[-1, 0, 0, 0], [300, 290, 1, 0]]
    elif case == "restart":
        toks, meta = [(0, 0, 43 + i) for i in range(5)], [[45, 40, 0, 0], [-1, 0, 0, 0]]
    elif case == "fresh_two_slots":
        toks, meta = [(0, 1, i) for i in range(3)] + [(0, 0, 77 + i) for i in range(2)], [[77, 77, 1, 0], [-1, 0, 0, 0]]
    else:
        toks, meta = [(0, 0, 10 + i) for i in range(21)], [[10, 4, 1, 0], [-1, 0, 0, 0]]
    n = len(toks)
    part = torch.randn(2, n, R.DELTA_IN, generator=g).cuda()
    ba = torch.randn(3, n, 2 * R.LV_HEADS, generator=g).cuda()
    st = R.build_step(toks, [0])
    dv = ref_cuda.upload_step(st)
    conv_w, a_log, dt_bias, norm_w = w
    mem1, mem2 = mem.clone(), mem.clone()
    meta1 = torch.tensor(meta, dtype=torch.int32, device="cuda")
    meta2 = meta1.clone()
    cv = torch.zeros(n, R.CVW, device="cuda")
    o1, o2 = torch.zeros(n, R.MIX, device="cuda"), torch.zeros(n, R.MIX, device="cuda")
    y1 = torch.zeros(n, R.MIX, dtype=torch.float16, device="cuda")
    y2 = torch.zeros_like(y1)
    ctx.delta_conv(part, 2, n, ba, 3, conv_w, a_log, dt_bias, mem1, SST, cv, dv)
    ctx.delta_rule(part, 2, n, cv, mem1, SST, meta1, o1, dv, st["segs"])
    ctx.delta_norm(part, 2, n, norm_w, o1, y1, meta1, dv, st["segs"])
    ctx.delta_mixer(part, 2, n, ba, 3, conv_w, a_log, dt_bias, norm_w, mem2, SST, meta2, o2, y2, dv, st["segs"])
    assert torch.equal(meta1, meta2)
    assert torch.allclose(o1, o2, rtol=2e-6, atol=1e-7)
    assert torch.allclose(y1.float(), y2.float(), rtol=2e-3, atol=1e-6)
    assert torch.allclose(mem1, mem2, rtol=2e-6, atol=2e-6)   # far inside the 1e-4 bound on the f32 state
    assert torch.equal(mem1 != mem, mem2 != mem)              # the same places were written


def test_chunked_prompt_matches_decode_sized_steps(ctx):
    """Segments long enough run the delta rule in chunks of 64 tokens (the WY form on the tensor cores as 3 x TF32) up to
    16..79 tokens before their end, then token by token: a 150-token prompt in one step, then an 80-token step that
    restarts 10 tokens back (replay from the bank, one more chunk), against the same positions in steps of at most 50
    tokens (token form throughout). Another summation order, so not bit for bit: raw outputs inside the benchmark's
    tolerance and within 1e-4, the f32 end state within 1e-4."""
    g = synth.gen(97)
    w = [t.cuda() for t in weights(g)]
    T = 220
    part = torch.randn(1, T, R.DELTA_IN, generator=g).cuda()
    ba = torch.randn(1, T, 2 * R.LV_HEADS, generator=g).cuda()

    def sl(t, i, j):
        return t[:, i:j].contiguous()

    def run(cuts):
        mem = torch.zeros(SST, device="cuda")
        meta = torch.tensor([[-1, 0, 0, 0]], dtype=torch.int32, device="cuda")
        outs = {}
        for a, b in cuts:
            _, o = layer_step(ctx, w, mem, meta, sl(part, a, b), sl(ba, a, b), [(0, 0, i) for i in range(a, b)])
            for i in range(a, b):
                outs[i] = o[i - a].clone()
        mt = meta.cpu().numpy()[0]
        return outs, mem[mt[2] * R.SLOT_STATE:(mt[2] + 1) * R.SLOT_STATE].clone(), mt
    chunked, sf, mf = run([(0, 150), (140, 220)])
    tokens, sc, mc = run([(0, 50), (50, 100), (100, 150), (140, 190), (190, 220)])
    assert mf[0] == mc[0] == T
    a = torch.stack([chunked[i] for i in range(T)]).cpu().numpy()
    b = torch.stack([tokens[i] for i in range(T)]).cpu().numpy()
    assert close(a, b).all() and np.abs(a - b).max() < 1e-4
    assert (sf - sc).abs().max().item() < 1e-4


@pytest.mark.parametrize("start", ["fresh", "continue"])
def test_chunked_rule_2048_tokens_next_to_the_reference_kernel(ctx, ref, start):
    """The benchmark's prompt variant (T = 2048, chunk size 64): the chunked scan against the reference's sequential
    delta_rule kernel on the same buffers and against the f64 oracle; from zeros and continuing a random state. State
    within 1e-4, outputs 1e-2 / 2e-3 after bf16 rounding; the banks and the conv ring are copies and must be identical."""
    g = synth.gen(98)
    n = 2048
    p0 = 0 if start == "fresh" else 4096
    mem = fresh_mem(1, g)
    cv = rule_inputs(g, n)
    part = torch.randn(1, n, R.DELTA_IN, generator=g)
    meta = torch.tensor([[-1, 0, 0, 0]] if start == "fresh" else [[p0, p0 - 7, 1, 0]], dtype=torch.int32)
    st = R.build_step([(0, 0, p0 + i) for i in range(n)], [0])
    dv = ref_cuda.upload_step(st)
    m1, m2 = mem.cuda(), mem.cuda()
    o1, o2 = torch.zeros(n, R.MIX, device="cuda"), torch.zeros(n, R.MIX, device="cuda")
    md = meta.cuda()
    pd, cd = part.cuda(), cv.cuda()
    ctx.delta_rule(pd, 1, n, cd, m1, SST, md, o1, dv, 1)
    ref.delta(pd, 1, n, None, 0, None, None, None, None, m2, SST, md, cd, o2, None, st, dv, which=("rule",))
    torch.cuda.synchronize()
    a, b = o1.cpu().numpy(), o2.cpu().numpy()
    assert close(a, b).all()
    assert np.abs(a - b).max() < 1e-4
    s1, s2 = m1.cpu().numpy(), m2.cpu().numpy()
    assert np.abs(s1[:2 * R.SLOT_STATE] - s2[:2 * R.SLOT_STATE]).max() < 1e-4
    assert np.array_equal(s1[2 * R.SLOT_STATE:R.SLOT_FLOATS], s2[2 * R.SLOT_STATE:R.SLOT_FLOATS])
    # the f64 oracle on a sample of the heads would need the whole recurrence; hold the first 200 tokens to it instead
    mo = mem.numpy().copy()
    st2 = R.build_step([(0, 0, p0 + i) for i in range(200)], [0])
    want = R.delta_rule(part.numpy()[:, :200], cv.numpy()[:200], mo, SST, meta.numpy(), st2["seg_start"], st2["seg_len"],
                        st2["seg_slot"], st2["seg_pos0"])
    assert np.abs(a[:200] - want).max() < 1e-4


def test_rollback_after_a_chunked_prompt(ctx):
    """A 100-token prompt (one chunk, then 36 tokens in the token form), then verify steps of 5 rows of which 3 are right
    and a restart at the first rejected position, against the same prompt followed by one token per step: identical
    outputs, bit for bit (the checkpoint, the bank and the replay are all made in the token form)."""
    g = synth.gen(99)
    w = [t.cuda() for t in weights(g)]
    P, T = 100, 112
    part = torch.randn(1, T, R.DELTA_IN, generator=g).cuda()
    ba = torch.randn(1, T, 2 * R.LV_HEADS, generator=g).cuda()
    wrong = torch.randn(1, T, R.DELTA_IN, generator=g).cuda()
    wrong_ba = torch.randn(1, T, 2 * R.LV_HEADS, generator=g).cuda()

    def sl(t, i, j):
        return t[:, i:j].contiguous()

    def prompt():
        mem = torch.zeros(SST, device="cuda")
        meta = torch.tensor([[-1, 0, 0, 0]], dtype=torch.int32, device="cuda")
        layer_step(ctx, w, mem, meta, sl(part, 0, P), sl(ba, 0, P), [(0, 0, i) for i in range(P)])
        return mem, meta
    memA, metaA = prompt()
    outsA = {}
    for i in range(P, T):
        y, _ = layer_step(ctx, w, memA, metaA, sl(part, i, i + 1), sl(ba, i, i + 1), [(0, 0, i)])
        outsA[i] = y[0].clone()
    memB, metaB = prompt()
    outsB = {}
    pos = P
    while pos < T:
        nrow = min(5, T - pos)
        good = min(3, nrow)
        pp = torch.cat([sl(part, pos, pos + good), sl(wrong, pos + good, pos + nrow)], dim=1).contiguous()
        bb = torch.cat([sl(ba, pos, pos + good), sl(wrong_ba, pos + good, pos + nrow)], dim=1).contiguous()
        y, _ = layer_step(ctx, w, memB, metaB, pp, bb, [(0, 0, pos + i) for i in range(nrow)])
        for i in range(good):
            outsB[pos + i] = y[i].clone()
        pos += good
    for i in range(P, T):
        assert torch.equal(outsA[i], outsB[i]), f"position {i}"
