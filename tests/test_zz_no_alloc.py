"""qb_marlin_gemm_noalloc: the product for callers that cannot allocate device memory (an engine whose page pool owns
all that was free, a plugin inside someone else's process). It must give exactly what qb_marlin_gemm gives, call after
call, out of the scratch array built into the library. Collected last on purpose: a run that stops at the first failure
has then already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from qwenny_b200 import host, synth
from qwenny_b200._lib import lib

pytestmark = pytest.mark.gpu


def _p(t):
    return C.c_void_p(t.data_ptr() if t is not None else 0)


def noalloc(x, words, scales, epi, y, keys=None, n_valid=0, xrows=None, row0=0, m=None):
    k, n = x.shape[1], words.shape[1] // 2
    m = x.shape[0] if m is None else m
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib().qb_marlin_gemm_noalloc(s, _p(x), _p(words), _p(y), _p(scales), m, n, k, row0,
                                        {"plain": 0, "silu": 1, "argmax": 2}[epi], _p(xrows), _p(keys), n_valid)


def test_noalloc_matches_the_context_product_twice_in_a_row(ctx):
    g = synth.gen(77)
    rows, cols, m = 5120, 6144, 5   # the 27B out-projection: its column blocks are shared by several blocks
    x = torch.from_numpy(synth.activations(m, cols, g)).cuda()
    codes, sc = synth.int4_matrix(rows, cols, g)
    words, s16 = host.pack_marlin(codes, sc)
    wd = torch.from_numpy(words.view(np.int32)).cuda()
    sd = torch.from_numpy(s16.view(np.int16)).cuda().view(torch.float16)
    ctx.tune(ctas=-2)  # the context product on the same stream-K path
    try:
        want = ctx.marlin_gemm(x, wd, sd)
    finally:
        ctx.tune()
    clustered = ctx.marlin_gemm(x, wd, sd)
    for _ in range(2):
        y = torch.full_like(want, float("nan"))
        assert noalloc(x, wd, sd, "plain", y) == 0
        torch.cuda.synchronize()
        assert torch.equal(y, want)                                    # same path, same bits
        assert torch.allclose(y, clustered, rtol=1e-5, atol=1e-6)      # the default path sums in another order
    # the other epilogues, and a second shape right after
    rows2, cols2 = 2048, 1024
    codes2, sc2 = synth.int4_matrix(rows2, cols2, g)
    w2, s2 = host.pack_marlin(codes2, sc2, silu=True)
    w2d = torch.from_numpy(w2.view(np.int32)).cuda()
    s2d = torch.from_numpy(s2.view(np.int16)).cuda().view(torch.float16)
    x2 = torch.from_numpy(synth.activations(16, cols2, g)).cuda()
    want2 = ctx.marlin_gemm(x2, w2d, s2d, epi="silu")
    y2 = torch.zeros_like(want2)
    assert noalloc(x2, w2d, s2d, "silu", y2) == 0
    torch.cuda.synchronize()
    assert torch.allclose(y2.float(), want2.float(), rtol=2e-3, atol=1e-5)
    keys_a = torch.zeros(16, dtype=torch.int64, device="cuda")
    keys_b = torch.zeros(16, dtype=torch.int64, device="cuda")
    la = ctx.marlin_gemm(x2, w2d, s2d, epi="argmax", keys=keys_a, n_valid=2000)
    lb = torch.zeros_like(la)
    assert noalloc(x2, w2d, s2d, "argmax", lb, keys=keys_b, n_valid=2000) == 0
    torch.cuda.synchronize()
    assert torch.allclose(la, lb, rtol=1e-5, atol=1e-6)
    ta = 0xFFFFFFFF - (keys_a.cpu().numpy().view(np.uint64) & np.uint64(0xFFFFFFFF))
    tb = 0xFFFFFFFF - (keys_b.cpu().numpy().view(np.uint64) & np.uint64(0xFFFFFFFF))
    assert np.array_equal(ta, tb)
    assert lib().qb_static_device_error() == 0   # no bounded wait of these products ran out


def test_noalloc_refuses_what_does_not_fit():
    assert lib().qb_static_scratch_bytes() < 17 << 20
    x = torch.zeros(5, 128, dtype=torch.float16, device="cuda")
    y = torch.zeros(8, device="cuda")
    big_n = 64 * 4096 + 256   # more 64-output groups than the array has tickets
    w = torch.zeros(8, dtype=torch.int32, device="cuda")  # never read: the call is refused first
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib().qb_marlin_gemm_noalloc(s, _p(x), _p(w), _p(y), _p(w), 5, big_n, 128, 0, 0, None, None, 0)
    assert rc == 1003  # QB_ERR_TOO_LARGE
    rc = lib().qb_marlin_gemm_noalloc(s, _p(x), _p(w), _p(y), _p(w), 17, 256, 128, 0, 0, None, None, 0)
    assert rc == 1000  # more than 16 rows: QB_ERR_ARG


def test_noalloc_takes_every_product_of_the_27b_step(ctx):
    """The documented limit, shape by shape: every layer product of the 27B model at 5 and at 16 rows and the output
    layer at 5 and 8 rows run out of the built-in array and equal the context product on the same stream-K path; the
    output layer at 16 rows is refused before anything is enqueued."""
    from qwenny_b200 import model as M
    g = torch.Generator(device="cuda").manual_seed(5)
    shapes = [(16384, 5120, "plain"), (14336, 5120, "plain"), (5120, 6144, "plain"), (34816, 5120, "silu"),
              (5120, 17408, "plain"), (5120, 10240, "plain"), (152064, 5120, "plain")]
    for n, k, epi in shapes:
        w = M.Marlin.random(n, k, g)
        for m in (5, 16):
            x = torch.randn(m, k, generator=g, device="cuda").half()
            y = torch.zeros(m, n // 2, dtype=torch.float16, device="cuda") if epi == "silu" else torch.zeros(m, n, device="cuda")
            if n > 131072 and m > 8:
                assert noalloc(x, w.words, w.scales, epi, y) == 1003   # QB_ERR_TOO_LARGE
                m = 8
                x, y = x[:8].contiguous(), y[:8].contiguous()
            assert noalloc(x, w.words, w.scales, epi, y) == 0, (n, k, m)
            ctx.tune(ctas=-2)
            try:
                want = ctx.marlin_gemm(x, w.words, w.scales, epi=epi)
            finally:
                ctx.tune()
            torch.cuda.synchronize()
            assert torch.equal(y, want), (n, k, m)
        del w
    assert lib().qb_static_device_error() == 0


@pytest.mark.gpu
def test_a_wait_that_runs_out_is_reported_and_the_context_lives_on(ctx):
    """Every device-side wait of the library is the same bounded poll loop; when it runs out the kernel records a code
    in the context's error word and returns. Here a block waits (4096 polls) on an mbarrier that nothing arrives on:
    qb_device_error reads 99 once, then 0, and the next product on the context is right."""
    import numpy as np
    from oracle import ref_ops as R
    from qwenny_b200 import host, synth
    assert ctx.device_error() == 0
    ctx.wait_probe(1 << 12)
    torch.cuda.synchronize()
    assert ctx.device_error() == 99
    assert ctx.device_error() == 0
    g = synth.gen(5)
    x = synth.activations(5, 512, g)
    codes, sc = synth.int4_matrix(256, 512, g)
    words, s16 = host.pack_marlin(codes, sc)
    dev = lambda a: torch.from_numpy(a).cuda()
    y = ctx.marlin_gemm(dev(x), dev(words.view(np.int32)), dev(s16.view(np.int16)).view(torch.float16)).cpu().numpy()
    want = R.marlin_gemm(x, R.dequant(codes, sc.astype(np.float16)))
    assert np.abs(y - want).max() < 2e-3 * max(1.0, np.abs(want).max()) and ctx.device_error() == 0


@pytest.mark.gpu
def test_a_product_whose_stage_never_lands_gives_up_and_reports_it(ctx):
    """The skinny product's own way out: the copy warp leaves out the second stage of every block (a measurement switch),
    the consumers' wait for it runs out after 1024 polls, each warp records error 2, walks the rest of its schedule
    and the kernel ends. qb_device_error reports 2; afterwards the same product on the same context is right again
    (tickets and ring barriers are left usable)."""
    import numpy as np
    from oracle import ref_ops as R
    from qwenny_b200 import host, synth
    g = synth.gen(8)
    # (5120 x 6144, the out-projection: 480 tile stages on 296 blocks, so many blocks have a second stage)
    x = synth.activations(5, 6144, g)
    codes, sc = synth.int4_matrix(5120, 6144, g)
    words, s16 = host.pack_marlin(codes, sc)
    dev = lambda a: torch.from_numpy(a).cuda()
    xd, wd, sd = dev(x), dev(words.view(np.int32)), dev(s16.view(np.int16)).view(torch.float16)
    want = R.marlin_gemm(x, R.dequant(codes, sc.astype(np.float16)))
    assert ctx.device_error() == 0
    for ctas in (-2, 2):  # equal shares of the persistent grid, and a cluster per column block
        ctx.tune(ctas=ctas)
        try:
            lib().qb_marlin_probe(ctx.h, 2)
            ctx.marlin_gemm(xd, wd, sd)
            lib().qb_marlin_probe(ctx.h, 0)
            torch.cuda.synchronize()
            assert ctx.device_error() == 2
            for _ in range(2):
                y = ctx.marlin_gemm(xd, wd, sd).cpu().numpy()
                assert np.abs(y - want).max() < 2e-3 * max(1.0, np.abs(want).max())
            assert ctx.device_error() == 0
        finally:
            lib().qb_marlin_probe(ctx.h, 0)
            ctx.tune()
