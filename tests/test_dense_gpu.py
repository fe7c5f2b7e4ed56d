"""Parity of the per-token kernels and the dense f16 product: library vs CPU oracle vs the reference's own kernels
(compiled from its sources, oracle/_ref) on the same device buffers."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R
from qwenny_b200 import host, synth

pytestmark = pytest.mark.gpu
H = R.H


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_embed(ctx, ref):
    g = synth.gen(31)
    table = (torch.randn(1000, H, generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.tensor([5, 999, 0, 17, 5], dtype=torch.int32)
    td, idd = table.cuda(), ids.cuda()
    out = torch.zeros(5, H, device="cuda")
    keys = torch.full((8,), 7, dtype=torch.int64, device="cuda")
    ctx.embed(td, idd, out, keys, 3, 5)
    want = R.embed(table.float().numpy(), ids.numpy())
    assert np.array_equal(out.cpu().numpy(), want)
    assert keys.cpu().tolist() == [0, 0, 0, 7, 7, 7, 7, 7]
    out_r = torch.zeros_like(out)
    ref.embed(td, idd, out_r, keys, 0, 5)
    assert torch.equal(out, out_r)


@pytest.mark.parametrize("n", [1, 5, 16])
def test_rmsnorm_and_add_rmsnorm(ctx, ref, n):
    g = synth.gen(32 + n)
    x = torch.randn(n, H, generator=g) * 3
    w = 1 + torch.randn(H, generator=g) * 0.02
    parts = torch.randn(3, n, H, generator=g)
    xd, wd, pd = x.cuda(), w.cuda(), parts.cuda()
    y = torch.zeros(n, H, dtype=torch.float16, device="cuda")
    ctx.rmsnorm(xd, wd, y, n)
    want = R.rmsnorm(x.numpy(), w.numpy())
    yr = torch.zeros_like(y)
    ref.rmsnorm(xd, wd, yr, n)
    # one f16 ulp of slack against the f64-normed oracle; the two CUDA versions differ by summation order only
    assert np.allclose(y.float().cpu().numpy(), want.astype(np.float32), rtol=2e-3, atol=1e-6)
    assert np.allclose(y.float().cpu().numpy(), yr.float().cpu().numpy(), rtol=2e-3, atol=1e-6)
    for splits in (1, 3):
        h1, h2 = xd.clone(), xd.clone()
        y1, y2 = torch.zeros_like(y), torch.zeros_like(y)
        ctx.add_rmsnorm(h1, pd, splits, n, wd, y1)
        ref.add_rmsnorm(h2, pd, splits, n, wd, y2)
        hw, yw = R.add_rmsnorm(x.numpy(), parts.numpy()[:splits], w.numpy())
        assert torch.equal(h1, h2)  # the same additions in the same order: bit-exact residual stream
        assert np.array_equal(h1.cpu().numpy(), hw)
        assert np.allclose(y1.float().cpu().numpy(), yw.astype(np.float32), rtol=2e-3, atol=1e-6)
        assert np.allclose(y1.float().cpu().numpy(), y2.float().cpu().numpy(), rtol=2e-3, atol=1e-6)


def test_to_xin_sum_parts_gather(ctx, ref):
    g = synth.gen(40)
    x = torch.randn(5 * 6144 + 3, generator=g).cuda()
    y, yr = torch.zeros(x.numel(), dtype=torch.float16, device="cuda"), torch.zeros(x.numel(), dtype=torch.float16, device="cuda")
    ctx.to_xin(x, y, x.numel())
    ref.to_xin(x, yr, x.numel())
    assert torch.equal(y, yr) and torch.equal(y, x.half())
    parts = torch.randn(4, 5, 96, generator=g).cuda()
    s = torch.zeros(5, 96, device="cuda")
    ctx.sum_parts(parts, 4, 5, 96, s)
    want = parts[0] + parts[1] + parts[2] + parts[3]
    assert torch.equal(s, want)
    xs = torch.randn(9, 512, generator=g).half().cuda()
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    o = torch.zeros(3, 512, dtype=torch.float16, device="cuda")
    ctx.marlin_gather(xs, rows, o, 512, 3)
    assert torch.equal(o, xs[[8, 0, 3]])


def test_mark_seen(ctx, ref):
    vocab = 248320  # the reference's compile-time vocabulary
    words = vocab // 32
    seen = torch.randint(0, 2**31 - 1, (3, words), dtype=torch.int32, device="cuda")
    seen_r = seen.clone()
    mark = torch.tensor([5, 37, 248319, 64, 5], dtype=torch.int32, device="cuda")
    mark_at = torch.tensor([0, 3, 5], dtype=torch.int32, device="cuda")
    seg_slot = torch.tensor([2, 0], dtype=torch.int32, device="cuda")
    seg_pos0 = torch.tensor([0, 9], dtype=torch.int32, device="cuda")
    before = seen.cpu().numpy().view(np.uint32).copy()
    ctx.mark_seen(seen, mark, mark_at, seg_slot, seg_pos0, 2, vocab)
    ref.mark_seen(seen_r, mark, mark_at, seg_slot, seg_pos0, 2)
    assert torch.equal(seen, seen_r)
    got = seen.cpu().numpy().view(np.uint32)
    want = before.copy()
    want[2] = 0  # the segment at position 0 starts a new sequence
    for slot, ids in ((2, [5, 37, 248319]), (0, [64, 5])):
        for i in ids:
            want[slot, i >> 5] |= np.uint32(1 << (i & 31))
    assert np.array_equal(got, want)


@pytest.mark.parametrize("n", [1, 5, 8, 13])
def test_gemm_f16_in_ba(ctx, ref, n):
    """in_proj_b / in_proj_a of the 27B build: 96 x 5120 kept in 16 bits."""
    g = synth.gen(50 + n)
    K, rows = 5120, 96
    w = (torch.randn(rows, K, generator=g) * 0.02).numpy()
    x = synth.activations(n, K, g)
    wp = dev(host.pack_f16(w).view(np.int16)).view(torch.float16)
    xd = dev(x)
    kper = K // host.split_for(rows // 16, K, 16, 1024 * 8 // (8 if n <= 8 else 16))
    y = ctx.gemm_f16_plain(wp, xd, n, K, rows // 16, kper)
    got = y.sum(0).cpu().numpy()
    want = R.dense_gemm(x, w.astype(np.float16))
    assert np.allclose(got, want, rtol=1e-4, atol=1e-4)
    yr = torch.zeros_like(y)
    split = ref.gemm_f16_plain(wp, xd, yr, n, K, rows // 16)
    assert split == y.shape[0]
    assert np.allclose(got, yr.sum(0).cpu().numpy(), rtol=1e-4, atol=1e-4)
