"""The prompt-sized W4A16 product (more than 16 rows: tcgen05 / tensor-memory kernel behind qb_marlin_gemm) against
the CPU oracle and against the skinny kernel run in 16-row slabs on the same buffers."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R
from qwenny_b200 import host, synth

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 2e-3  # the benchmark's tolerance for product outputs, after rounding to bf16


def bf16(a):
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def close(a, b):
    a, b = bf16(a), bf16(b)
    return np.abs(a - b) <= ATOL + RTOL * np.abs(b)


def make(rows, cols, silu, seed, m):
    g = synth.gen(seed)
    x = synth.activations(m, cols, g)
    codes, sc = synth.int4_matrix(rows, cols, g)
    words, s16 = host.pack_marlin(codes, sc, silu=silu)
    wdq = R.dequant(codes, sc.astype(np.float16))[R.row_order(rows, silu)]
    dev = lambda a: torch.from_numpy(a).cuda()
    return x, wdq, dev(x), dev(words.view(np.int32)), dev(s16.view(np.int16)).view(torch.float16)


@pytest.mark.parametrize("m,rows,cols", [(64, 256, 128), (256, 512, 1024), (300, 512, 640), (17, 256, 256),
                                         (2048, 1024, 5120)])
def test_plain_vs_oracle_and_slabs(ctx, m, rows, cols):
    x, wdq, xd, wd, sd = make(rows, cols, False, 100 + m, m)
    y = ctx.marlin_gemm(xd, wd, sd)
    torch.cuda.synchronize()
    assert ctx.device_error() == 0
    want = R.marlin_gemm(x, wdq)
    a = y.cpu().numpy()
    assert close(a, want).all()
    # f32 sums of the same f16 products as the oracle's f64: far inside the tolerance
    assert np.abs(a - want).max() < 2e-4 * max(1.0, np.abs(want).max())
    ctx.tune(nstages=-1)  # the skinny kernel in 16-row slabs
    try:
        ys = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()
    finally:
        ctx.tune()
    assert np.abs(a - ys).max() < 2e-4 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("m,rows,cols", [(128, 512, 256), (2048, 1024, 1024)])
def test_silu_vs_oracle(ctx, m, rows, cols):
    x, wdq, xd, wd, sd = make(rows, cols, True, 200 + m, m)
    y = ctx.marlin_gemm(xd, wd, sd, epi="silu")
    torch.cuda.synchronize()
    assert ctx.device_error() == 0
    want = R.marlin_gemm(x, wdq, "silu")
    assert y.shape == (m, rows // 2)
    assert close(y.float().cpu().numpy(), want.astype(np.float32)).all()


def test_row0_and_prefill_chunk_shape(ctx):
    """Rows row0 .. of a larger X / Y, and the 27B in-projection's width at a 2048-row chunk (sampled columns)."""
    x, wdq, xd, wd, sd = make(512, 384, False, 321, 100)
    y = torch.zeros(100, 512, device="cuda")
    ctx.marlin_gemm(xd, wd, sd, y=y, row0=30, m=50)
    want = R.marlin_gemm(x[30:80], wdq)
    a = y.cpu().numpy()
    assert close(a[30:80], want).all() and np.all(a[:30] == 0) and np.all(a[80:] == 0)


@pytest.mark.parametrize("m,rows,cols,silu", [(600, 1024, 2048, False), (2048, 5120, 1024, False), (520, 512, 1536, True)])
def test_shares_of_the_tile_list_repeat_and_agree_with_whole_tiles(ctx, m, rows, cols, silu):
    """The product deals (tile, k block) pairs to a persistent grid in equal contiguous shares when there are few tiles
    per SM; tiles cut between blocks are summed in block order by the tile's last arriver, so a repeated launch gives
    the same bits, and the result agrees with the same launch run as whole tiles (only the order of the f32 sums over
    k differs) and with the oracle."""
    x, wdq, xd, wd, sd = make(rows, cols, silu, 400 + m, m)
    epi = "silu" if silu else "plain"
    ctx.tune(ctas=1000)  # equal shares whatever the shape
    try:
        a = ctx.marlin_gemm(xd, wd, sd, epi=epi)
        b = ctx.marlin_gemm(xd, wd, sd, epi=epi)
        ctx.tune(ctas=1001)  # whole tiles whatever the shape
        c = ctx.marlin_gemm(xd, wd, sd, epi=epi)
    finally:
        ctx.tune()
    torch.cuda.synchronize()
    assert ctx.device_error() == 0
    assert torch.equal(a, b)
    want = R.marlin_gemm(x, wdq, epi)
    an, cn = a.float().cpu().numpy(), c.float().cpu().numpy()
    assert close(an, want.astype(np.float32)).all() and close(cn, want.astype(np.float32)).all()
    assert np.abs(an - cn).max() <= (2e-3 if silu else 2e-4) * max(1.0, np.abs(want).max())
