"""The dense products of non-int4 checkpoints (qb_gemm_dec: 16-bit and int8 weights, plain / SwiGLU / argmax epilogues)
against the reference's compiled kernels gemm_{f16,i8}_t*_{plain,silu,argmax} and the CPU oracle (exact dequantised
weights, float64 product). The kernels add the k range in different orders, so the comparison is by tolerance: 1e-3
relative on f32 sums, one f16 ulp on the SwiGLU output; the argmax token must agree unless the top two are that close."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R
from qwenny_b200 import host

pytestmark = pytest.mark.gpu


def make(wt, rows, K, silu, seed):
    g = np.random.default_rng(seed)
    w = (g.standard_normal((rows, K)) * 0.04).astype(np.float32)
    order = host.row_order(rows, silu)
    if wt == "f16":
        packed = torch.from_numpy(host.pack_f16(w, order).view(np.int16)).cuda()
        scales, wd = None, w.astype(np.float16).astype(np.float32)
    else:
        codes, sc = host.pack_i8(w, order)
        packed, scales = torch.from_numpy(codes).cuda(), torch.from_numpy(sc).cuda()
        wd = R.dequant_i8(w)
    return packed, scales, wd[order]


@pytest.mark.parametrize("wt", ["f16", "i8"])
@pytest.mark.parametrize("n", [5, 13, 27])
def test_plain_with_splits(ctx, ref, wt, n):
    rows, K, kper = 512, 1024, 256
    packed, scales, wd = make(wt, rows, K, False, 1)
    x = (torch.randn(n, K, generator=torch.Generator().manual_seed(2)) * 0.5).half().cuda()
    split = K // kper
    mine = torch.zeros(split, n, rows, device="cuda")
    theirs = torch.zeros_like(mine)
    ctx.gemm_dec(packed, scales, 16 if wt == "f16" else 8, x, K, rows // 16, n, kper, 0, mine, rows)
    ref.gemm_dec(wt, "plain", packed, scales, x, theirs, n, K, rows // 16, kper, rows)
    torch.cuda.synchronize()
    want = x.float().cpu().numpy().astype(np.float64) @ wd.astype(np.float64).T
    got, rg = mine.sum(0).cpu().numpy(), theirs.sum(0).cpu().numpy()
    tol = 1e-3 * np.abs(want).max()
    assert np.abs(got - want).max() < tol and np.abs(got - rg).max() < tol
    # every split by itself
    for s in range(split):
        ws = x.float().cpu().numpy()[:, s * kper:(s + 1) * kper].astype(np.float64) @ wd[:, s * kper:(s + 1) * kper].T
        assert np.abs(mine[s].cpu().numpy() - ws).max() < tol


@pytest.mark.parametrize("wt", ["f16", "i8"])
def test_swiglu_and_gathered_rows(ctx, ref, wt):
    rows, K, n = 1024, 768, 11
    packed, scales, wd = make(wt, rows, K, True, 3)
    x = (torch.randn(20, K, generator=torch.Generator().manual_seed(4)) * 0.5).half().cuda()
    xrows = torch.tensor([19, 0, 3, 3, 7, 12, 1, 18, 5, 9, 2], dtype=torch.int32).cuda()
    mine = torch.zeros(n, rows // 2, dtype=torch.float16, device="cuda")
    theirs = torch.zeros_like(mine)
    ctx.gemm_dec(packed, scales, 16 if wt == "f16" else 8, x, K, rows // 16, n, K, 1, mine, rows // 2, xrows=xrows)
    ref.gemm_dec(wt, "silu", packed, scales, x, theirs, n, K, rows // 16, K, rows // 2, xrows=xrows)
    torch.cuda.synchronize()
    xs = x.float().cpu().numpy()[xrows.cpu().numpy()].astype(np.float64)
    y = (xs @ wd.astype(np.float64).T).reshape(n, rows // 16, 2, 8)
    want = (y[:, :, 0] / (1 + np.exp(-y[:, :, 0])) * y[:, :, 1]).reshape(n, rows // 2)
    got, rg = mine.float().cpu().numpy(), theirs.float().cpu().numpy()
    tol = 2 ** -9 * max(1.0, np.abs(want).max())
    assert np.abs(got - want).max() < tol and np.abs(got - rg).max() < tol


@pytest.mark.parametrize("wt", ["f16", "i8"])
def test_argmax(ctx, ref, wt):
    rows, K, n = 2048, 512, 6
    packed, scales, wd = make(wt, rows, K, False, 5)
    x = (torch.randn(n, K, generator=torch.Generator().manual_seed(6)) * 0.5).half().cuda()
    mine = torch.zeros(n, rows, device="cuda")
    theirs = torch.zeros_like(mine)
    km = torch.zeros(n, dtype=torch.int64, device="cuda")
    kt = torch.zeros(n, dtype=torch.int64, device="cuda")
    ctx.gemm_dec(packed, scales, 16 if wt == "f16" else 8, x, K, rows // 16, n, K, 2, mine, rows, keys=km)
    ref.gemm_dec(wt, "argmax", packed, scales, x, theirs, n, K, rows // 16, K, rows, keys=kt)
    torch.cuda.synchronize()
    want = x.float().cpu().numpy().astype(np.float64) @ wd.astype(np.float64).T
    got = mine.cpu().numpy()
    assert np.abs(got - want).max() < 1e-3 * np.abs(want).max()
    tok = [int(0xffffffff - (int(k) & 0xffffffff)) for k in km.tolist()]
    assert tok == got.argmax(1).tolist()  # the key is the argmax of the logits this kernel wrote
    rt = [int(0xffffffff - (int(k) & 0xffffffff)) for k in kt.tolist()]
    for t in range(n):
        if tok[t] != rt[t]:
            srt = np.sort(want[t])
            assert srt[-1] - srt[-2] < 1e-3 * np.abs(want).max()


def test_bad_arguments(ctx):
    from qwenny_b200._lib import QbError
    packed, scales, wd = make("f16", 64, 256, False, 7)
    x = torch.zeros(4, 256, dtype=torch.float16, device="cuda")
    y = torch.zeros(4, 64, device="cuda")
    with pytest.raises(QbError):
        ctx.gemm_dec(packed, None, 8, x, 256, 4, 4, 256, 0, y, 64)  # int8 without scales
    with pytest.raises(QbError):
        ctx.gemm_dec(packed, None, 16, x, 256, 4, 4, 128, 1, y, 64)  # SwiGLU over a split
    with pytest.raises(QbError):
        ctx.gemm_dec(packed, None, 16, x, 256, 4, 4, 256, 2, y, 64)  # argmax without keys
