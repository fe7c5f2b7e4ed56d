"""Parity of the W4A16 skinny product (qb_marlin_gemm) on the GPU: against the CPU oracle (exact dequantisation,
f64 product) and its invariants (bit-exact unpack, row-count invariance). The reference's own Marlin kernels are not
run next to it: they end with an illegal-instruction fault on B200 (see oracle/ref_cuda.py RefModule.marlin)."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R
from qwenny_b200 import host, synth

pytestmark = pytest.mark.gpu

# The benchmark's tolerance for matrix-product outputs: 1e-2 relative / 2e-3 absolute after rounding both sides to bf16
RTOL, ATOL = 1e-2, 2e-3


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


@pytest.mark.parametrize("m", [1, 2, 5, 8, 13, 16])
@pytest.mark.parametrize("rows,cols", [(512, 1024), (2560, 512), (256, 128)])
def test_plain_vs_oracle(ctx, m, rows, cols):
    x, wdq, xd, wd, sd = make(rows, cols, False, 10 + m, m)
    y = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()
    want = R.marlin_gemm(x, wdq)
    assert close(y, want).all()
    assert np.abs(y - want).max() < 2e-3 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("cfg", [(2, 4, 1), (2, 4, 2), (4, 2, 1), (4, 2, 3), (8, 1, 2), (8, 1, 1), (1, 8, 1), (4, 1, 2),
                                 (2, 4, -2), (4, 2, -2), (1, 8, -1)])
def test_every_tile_shape(ctx, cfg):
    """Every consumer-warp arrangement, clustered split K (ctas > 0, where the shape allows) and stream-K (ctas < 0)."""
    cg, kg, ctas = cfg
    x, wdq, xd, wd, sd = make(1024, 2048, False, 3, 5)
    ctx.tune(cg=cg, kg=kg, ctas=ctas)
    try:
        y = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()
        y2 = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()  # tickets left at zero: a second product works
    finally:
        ctx.tune()
    want = R.marlin_gemm(x, wdq)
    assert close(y, want).all()
    assert np.array_equal(y, y2)


def test_unpack_bit_exact(ctx):
    """X = identity rows: row t of Y is column t of the dequantised matrix, exactly (bf16 scales: (q-8)*s is exact)."""
    rows, cols = 512, 256
    g = synth.gen(5)
    codes, sc = synth.int4_matrix(rows, cols, g)
    words, s16 = host.pack_marlin(codes, sc)
    wd = torch.from_numpy(words.view(np.int32)).cuda()
    sd = torch.from_numpy(s16.view(np.int16)).cuda().view(torch.float16)
    wdq = R.dequant(codes, sc.astype(np.float16)).astype(np.float32)
    for c0 in range(0, cols, 16):
        x = np.zeros((16, cols), dtype=np.float16)
        x[np.arange(16), c0 + np.arange(16)] = 1
        y = ctx.marlin_gemm(torch.from_numpy(x).cuda(), wd, sd).cpu().numpy()
        assert np.array_equal(y, wdq[:, c0:c0 + 16].T)


def test_row_count_invariance(ctx):
    """A row's result is bit-identical alone, among 5 rows, or among 16 (the reference's speccheck property)."""
    x, wdq, xd, wd, sd = make(1024, 5120, False, 7, 16)
    y16 = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()
    y5 = ctx.marlin_gemm(xd[:5].contiguous(), wd, sd).cpu().numpy()
    assert np.array_equal(y5, y16[:5])
    for t in (0, 3, 15):
        y1 = ctx.marlin_gemm(xd[t:t + 1].contiguous(), wd, sd).cpu().numpy()
        assert np.array_equal(y1[0], y16[t])
    # row0: rows 4..8 of X written to rows 4..8 of Y
    y = torch.zeros(16, 1024, device="cuda")
    ctx.marlin_gemm(xd, wd, sd, y=y, row0=4, m=5)
    assert np.array_equal(y.cpu().numpy()[4:9], y16[4:9]) and float(y[:4].abs().max()) == 0


@pytest.mark.parametrize("rows,cols,m", [(1024, 1024, 5), (34816, 5120, 5), (512, 256, 16)])
def test_silu_vs_oracle(ctx, rows, cols, m):
    x, wdq, xd, wd, sd = make(rows, cols, True, 11, m)
    y = ctx.marlin_gemm(xd, wd, sd, epi="silu")
    want = R.marlin_gemm(x, wdq, "silu")
    assert y.shape == (m, rows // 2)
    assert close(y.float().cpu().numpy(), want.astype(np.float32)).all()


def test_argmax_vs_oracle(ctx):
    rows, cols, valid = 2048, 512, 1936
    g = synth.gen(12)
    xall = synth.activations(9, cols, g)
    codes, sc = synth.int4_matrix(rows, cols, g)
    words, s16 = host.pack_marlin(codes, sc)
    wdq = R.dequant(codes, sc.astype(np.float16))
    xd = torch.from_numpy(xall).cuda()
    wd = torch.from_numpy(words.view(np.int32)).cuda()
    sd = torch.from_numpy(s16.view(np.int16)).cuda().view(torch.float16)
    out_rows = torch.tensor([8, 2, 5], dtype=torch.int32, device="cuda")
    keys = torch.zeros(8, dtype=torch.int64, device="cuda")
    y = ctx.marlin_gemm(xd, wd, sd, epi="argmax", xrows=out_rows, keys=keys, n_valid=valid).cpu().numpy()
    want, wkeys = R.marlin_gemm(xall[[8, 2, 5]], wdq, "argmax", valid)
    assert close(y, want).all()
    got = keys.cpu().numpy().view(np.uint64)[:3]
    assert np.array_equal(R.key_token(got), R.key_token(wkeys))
    assert all(int(t) < valid for t in R.key_token(got))
    # the key's value half is the ordered logit of that token
    for r in range(3):
        tok = int(R.key_token(got)[r])
        assert int(got[r] >> np.uint64(32)) == int(R.ordered_u32(y[r:r + 1, tok:tok + 1])[0, 0])


@pytest.mark.parametrize("m", [1, 5, 16])
def test_config0_vs_oracle(ctx, m):
    """The benchmark's single-product configuration: N=17408 x K=5120, g128, seed 0."""
    x, wdq, xd, wd, sd = make(17408, 5120, False, 0, m)
    a = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()
    want = R.marlin_gemm(x, wdq)
    assert close(a, want).all()
    # f32 sums of exact products against the f64 product: far inside the tolerance
    assert np.abs(a - want).max() < 1e-4 * np.abs(want).max()


@pytest.mark.parametrize("n,k", [(16384, 5120), (14336, 5120), (5120, 6144), (5120, 17408)])
def test_model_shapes_vs_oracle(ctx, n, k):
    x, wdq, xd, wd, sd = make(n, k, False, n + k, 5)
    a = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()
    want = R.marlin_gemm(x, wdq)
    assert close(a, want).all()
    assert np.abs(a - want).max() < 1e-4 * np.abs(want).max()


def test_stages_requested_ahead_of_the_kernel_before_do_not_change_the_result(ctx):
    """qb_marlin_early: one, two or all three of a block's first stages of weights may be requested before the product
    waits for the kernel enqueued before it (here: the kernel that writes its X). Same bits every time, with programmatic
    dependent launch on, on a clustered product, on equal shares of a persistent grid and on the SwiGLU form."""
    from qwenny_b200._lib import lib
    ctx.set_pdl(True)
    try:
        for rows, cols, silu in ((16384, 5120, False), (5120, 17408, False), (2048, 1024, True)):
            x, wdq, xd, wd, sd = make(rows, cols, silu, rows + cols + 7, 5)
            x32 = xd.float()
            outs = []
            for stages in (1, 2, 3):
                ctx.early(stages)
                xk = (x32 * 1.0).half()            # a kernel right before the product writes its X
                outs.append(ctx.marlin_gemm(xk, wd, sd, epi="silu" if silu else "plain").clone())
            ctx.early(1)
            torch.cuda.synchronize()
            assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
            assert close(outs[0].float().cpu().numpy(), R.marlin_gemm(x, wdq, "silu" if silu else "plain")).all()
        assert lib().qb_marlin_early(ctx.h, 0) == 1000 and lib().qb_marlin_early(None, 1) == 1000   # QB_ERR_ARG
        assert ctx.device_error() == 0
    finally:
        ctx.early(1)
        ctx.set_pdl(False)


def test_many_rows_fall_back_to_slabs(ctx):
    x, wdq, xd, wd, sd = make(512, 512, False, 21, 40)
    y = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()
    assert close(y, R.marlin_gemm(x, wdq)).all()


@pytest.mark.parametrize("m,epi", [(1, "plain"), (5, "plain"), (13, "plain"), (5, "silu"), (5, "argmax"), (40, "plain"),
                                   (300, "silu"), (40, "argmax")])
@pytest.mark.parametrize("rows,cols", [(512, 1024), (2560, 512)])
def test_zero_point_product_vs_oracle(ctx, m, epi, rows, cols):
    """The marlin_*_z variants (asymmetric int4): w = (q - 8) * scale + (8 - z) * scale with the second table after the
    scales; against the oracle's dequantisation (the reference's single f16 rounding of the sum) in f64. More than 16
    rows run on the tensor-core product (plain, SwiGLU) or as 16-row slabs (argmax)."""
    g = synth.gen(700 + m)
    silu = epi == "silu"
    x = synth.activations(m, cols, g)
    codes, sc = synth.int4_matrix(rows, cols, g)
    zeros = torch.randint(0, 16, (rows, cols // 128), generator=g, dtype=torch.uint8).numpy()
    words, s16 = host.pack_marlin(codes, sc, silu=silu, zeros=zeros)
    off = ((8.0 - zeros.astype(np.float32)) * sc).astype(np.float16)
    wdq = R.dequant_z(codes, sc.astype(np.float16), off)[R.row_order(rows, silu)]
    dev = lambda a: torch.from_numpy(a).cuda()
    xd, wd, sd = dev(x), dev(words.view(np.int32)), dev(s16.view(np.int16)).view(torch.float16)
    want = R.marlin_gemm(x, wdq)
    if epi == "argmax":
        keys = torch.zeros(m, dtype=torch.int64, device="cuda")
        y = ctx.marlin_gemm(xd, wd, sd, epi="argmax", keys=keys, n_valid=rows - 3, zp=True).cpu().numpy()
        tok = [int(0xffffffff - (int(k) & 0xffffffff)) for k in keys.cpu().numpy()]
        assert close(y, want).all()
        for r in range(m):
            best = np.sort(want[r, :rows - 3])
            assert tok[r] == int(np.argmax(y[r, :rows - 3])) and (tok[r] == int(np.argmax(want[r, :rows - 3])) or
                                                                    best[-1] - best[-2] < 1e-3)
        return
    y = ctx.marlin_gemm(xd, wd, sd, epi=epi, zp=True).float().cpu().numpy()
    if silu:
        b = want.reshape(m, -1, 2, 8)
        want = (R.silu(b[:, :, 0, :]) * b[:, :, 1, :]).reshape(m, -1)
    assert close(y, want).all()
    # and it is not the symmetric product: the zero points matter
    ys = ctx.marlin_gemm(xd, wd, sd[:cols // 128].contiguous(), epi=epi).float().cpu().numpy()
    assert not close(ys, want).all()
