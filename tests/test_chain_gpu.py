"""The persistent layer kernel (qb_layer_chain: out_proj, residual + RMSNorm, gate_up with SwiGLU, down, residual +
RMSNorm, the next in-projection in one cooperative launch) against the same chain run as the separate, individually
parity-tested launches, and the whole step with and without it. Tolerance between the two: the products sum their k
groups in different orders (f32), and a value of xn / mid on an f16 rounding boundary may flip, so outputs agree to the
step tolerance rather than bit for bit; the residual stream after the first product agrees to f32 rounding."""
import numpy as np
import pytest
import torch

from qwenny_b200 import model as M

pytestmark = pytest.mark.gpu
H, MIX, FF = 5120, 6144, 17408


def rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def separate(ctx, m, mix, w, h):
    """The chain as the step runner launches it without the persistent kernel."""
    out, gu, down, nxt, post, nextn = w
    h = h.clone()
    xn = torch.empty(m, H, dtype=torch.float16, device="cuda")
    part = ctx.marlin_gemm(mix, out.words, out.scales)
    ctx.add_rmsnorm(h, part, 1, m, post, xn)
    mid = ctx.marlin_gemm(xn, gu.words, gu.scales, epi="silu")
    part = ctx.marlin_gemm(mid, down.words, down.scales)
    ctx.add_rmsnorm(h, part, 1, m, nextn, xn)
    y = ctx.marlin_gemm(xn, nxt.words, nxt.scales) if nxt is not None else None
    return h, xn, mid, y


@pytest.mark.parametrize("m,next_n", [(5, 16384), (1, 14336), (7, 16384), (3, 0)])
def test_layer_chain_matches_separate_launches(ctx, m, next_n):
    g = torch.Generator(device="cuda").manual_seed(300 + m)
    out, gu, down = M.Marlin.random(H, MIX, g), M.Marlin.random(2 * FF, H, g), M.Marlin.random(H, FF, g)
    nxt = M.Marlin.random(next_n, H, g) if next_n else None
    post = (1 + 0.02 * torch.randn(H, generator=g, device="cuda")).float()
    nextn = (1 + 0.02 * torch.randn(H, generator=g, device="cuda")).float()
    mix = torch.randn(m, MIX, generator=g, device="cuda").half()
    h0 = torch.randn(m, H, generator=g, device="cuda")
    want_h, want_xn, want_mid, want_y = separate(ctx, m, mix, (out, gu, down, nxt, post, nextn), h0)

    h, h_tmp, part_h = h0.clone(), torch.zeros(8, H, device="cuda"), torch.zeros(8, H, device="cuda")
    mid = torch.zeros(m, FF, dtype=torch.float16, device="cuda")
    xn = torch.zeros(m, H, dtype=torch.float16, device="cuda")
    part = torch.zeros(m, max(next_n, 1), device="cuda")
    for rep in range(2):  # the second launch finds the barriers and tickets as the first left them
        h.copy_(h0)
        ctx.layer_chain(m, mix, (out.words, out.scales), (gu.words, gu.scales), (down.words, down.scales),
                        (nxt.words, nxt.scales, next_n) if nxt is not None else None, post, nextn, h, h_tmp, part_h,
                        mid, xn, part)
        torch.cuda.synchronize()
        assert ctx.device_error() == 0
        assert rel(mid.float(), want_mid.float()) < 2e-3
        assert rel(h, want_h) < 1e-4
        assert rel(xn.float(), want_xn.float()) < 2e-3
        if nxt is not None:
            assert rel(part, want_y) < 2e-3
            ok = (part - want_y).abs() <= 2e-3 + 1e-2 * want_y.abs()
            assert ok.float().mean() > 0.999


def test_layer_chain_rejects(ctx):
    from qwenny_b200 import QbError
    g = torch.Generator(device="cuda").manual_seed(310)
    out = M.Marlin.random(H, MIX, g)
    z = torch.zeros(8, H, device="cuda")
    with pytest.raises(QbError):  # more rows than the resident X holds
        ctx.layer_chain(8, z.half(), (out.words, out.scales), (out.words, out.scales), (out.words, out.scales), None, z[0],
                        z[0], z, z, z, z.half(), z.half(), z)


def test_step_with_and_without_chain(ctx):
    """Greedy tokens and logits of verify steps with the persistent kernel on and off (the default)."""
    def fresh():
        return M.synthetic(ctx, nlayers=4, slots=1, max_ctx=256, vocab=2000, seed=21)
    a, b = fresh(), fresh()
    a.use_chain(True)
    seq = [(77 + 131 * i) % 2000 for i in range(40)]
    pos = 0
    while pos + 5 <= len(seq):
        toks = [(seq[pos + i], 0, pos + i) for i in range(5)]
        a.step(toks, list(range(5)))
        b.step(toks, list(range(5)))
        la, lb = a.logits(), b.logits()
        assert rel(la, lb) < 2e-3
        ta, tb = a.argmax(), b.argmax()
        srt = lb.sort(dim=1).values
        for r in range(5):
            assert ta[r] == tb[r] or float(srt[r, -1] - srt[r, -2]) < 1e-3
        pos += 3
    assert a.step_kernels < b.step_kernels


@pytest.mark.parametrize("m", [1, 5, 12])
def test_fused_residual_and_norm_products(ctx, m):
    """qb_marlin_gemm_fused: out_proj adds into the residual stream, leaves the un-normalised f16(w * h) rows and their
    sums of squares; gate_up runs on those rows and scales its result by 1 / rms; against marlin_gemm + add_rmsnorm +
    marlin_gemm. The residual stream is the same sum in another order (f32 rounding); the second product rounds its
    input to f16 before the division by the rms instead of after it (same relative precision)."""
    g = torch.Generator(device="cuda").manual_seed(400 + m)
    out, gu = M.Marlin.random(H, MIX, g), M.Marlin.random(2 * FF, H, g)
    post = (1 + 0.02 * torch.randn(H, generator=g, device="cuda")).float()
    mix = torch.randn(m, MIX, generator=g, device="cuda").half()
    h0 = torch.randn(m, H, generator=g, device="cuda")
    want_h = h0.clone()
    xn = torch.empty(m, H, dtype=torch.float16, device="cuda")
    part = ctx.marlin_gemm(mix, out.words, out.scales)
    ctx.add_rmsnorm(want_h, part, 1, m, post, xn)
    want_mid = ctx.marlin_gemm(xn, gu.words, gu.scales, epi="silu")
    h = h0.clone()
    xu = torch.zeros(m, H, dtype=torch.float16, device="cuda")
    mid = torch.zeros(m, FF, dtype=torch.float16, device="cuda")
    ctx.marlin_gemm_fused(mix, out.words, out.scales, h, m, epi="resid", norm_w_out=post, xu_out=xu)
    ctx.marlin_gemm_fused(xu, gu.words, gu.scales, mid, m, epi="silu", x_unnormed=True)
    torch.cuda.synchronize()
    assert ctx.device_error() == 0
    assert rel(h, want_h) < 1e-6
    assert torch.equal(xu, (post * h).half())
    assert rel(mid.float(), want_mid.float()) < 1e-3
    ok = (mid.float() - want_mid.float()).abs() <= 2e-3 + 1e-2 * want_mid.float().abs()
    assert ok.float().mean() > 0.9999


def test_step_with_and_without_fused_norm(ctx):
    def fresh():
        return M.synthetic(ctx, nlayers=4, slots=1, max_ctx=256, vocab=2000, seed=23)
    a, b = fresh(), fresh()
    a.use_fused_norm(True)
    seq = [(91 + 313 * i) % 2000 for i in range(40)]
    pos = 0
    while pos + 5 <= len(seq):
        toks = [(seq[pos + i], 0, pos + i) for i in range(5)]
        a.step(toks, list(range(5)))
        la, ta = a.logits(), a.argmax()
        torch.cuda.synchronize()
        b.step(toks, list(range(5)))
        lb, tb = b.logits(), b.argmax()
        torch.cuda.synchronize()
        assert rel(la, lb) < 2e-3
        srt = lb.sort(dim=1).values
        for r in range(5):
            assert ta[r] == tb[r] or float(srt[r, -1] - srt[r, -2]) < 1e-3
        pos += 3
    assert a.step_kernels < b.step_kernels
