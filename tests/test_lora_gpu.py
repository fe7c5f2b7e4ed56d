"""The unmerged LoRA kernels (qb_lora_add, qb_lora_silu) against the reference's compiled kernels (bit for bit: the
sums run in the same order) and the CPU oracle; tokens of slots without the adapter keep the base model's values."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R

pytestmark = pytest.mark.gpu
IMAX = 2 ** 31 - 1


def setup(rank, rows, n, seed, silu):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mods = 2 if silu else 3
    M = (mods * rank + 15) // 16 * 16
    split = 3
    xa = torch.randn(split, n, M, generator=g, device="cuda") * 0.3
    B = (torch.randn(rows, rank, generator=g, device="cuda") * 0.1).half()
    if silu:
        tab = [IMAX, IMAX, IMAX, IMAX, rank, 0, -1, -1]  # up's columns first, gate's after them
    else:
        tab = [rows // 4, rows // 2, IMAX, IMAX, rank, -1, 0, -1]  # the middle module is not adapted
    tab_d = torch.tensor(tab, dtype=torch.int32, device="cuda")
    tok_slot = torch.randint(0, 3, (n,), generator=g, device="cuda", dtype=torch.int32)
    slot_scale = torch.tensor([2.0, 0.0, 0.5], device="cuda")
    y = torch.randn(n, rows, generator=g, device="cuda")
    return M, split, xa, B, tab, tab_d, tok_slot, slot_scale, y


@pytest.mark.parametrize("rank", [8, 16, 32, 64])
@pytest.mark.parametrize("n", [5, 19])
def test_lora_add(ctx, ref, rank, n):
    rows = 1024 + 256
    M, split, xa, B, tab, tab_d, tok_slot, slot_scale, y = setup(rank, rows, n, 100 + rank + n, False)
    mine, theirs = y.clone(), y.clone()
    ctx.lora_add(xa, split, M, B, rows, tab_d, tok_slot, slot_scale, n, mine, rows, rank)
    ref.lora_add(rank, xa, split, M, B, rows, tab_d, tok_slot, slot_scale, n, theirs, rows)
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)
    sc = slot_scale[tok_slot.long()].cpu().numpy()
    want = y.cpu().numpy() + R.lora_delta(xa.cpu().numpy(), B.float().cpu().numpy(), tab, sc)
    np.testing.assert_allclose(mine.cpu().numpy(), want, rtol=1e-5, atol=1e-5)
    idle = np.nonzero(sc == 0)[0]
    assert len(idle) and torch.equal(mine[idle], y[idle])  # untouched, bit for bit
    mid = slice(rows // 4, rows // 2)
    assert torch.equal(mine[:, mid], y[:, mid])  # the module without an adapter


@pytest.mark.parametrize("rank", [8, 64])
@pytest.mark.parametrize("both", [True, False])
def test_lora_silu(ctx, ref, rank, both):
    rows, n = 2048, 13
    M, split, xa, B, tab, tab_d, tok_slot, slot_scale, y = setup(rank, rows, n, 200 + rank, True)
    if not both:  # only up_proj adapted
        tab[5] = -1
        tab_d = torch.tensor(tab, dtype=torch.int32, device="cuda")
    mine = torch.zeros(n, rows // 2, dtype=torch.float16, device="cuda")
    theirs = torch.zeros_like(mine)
    ctx.lora_silu(xa, split, M, B, rows, tab_d, tok_slot, slot_scale, n, y, rows, mine, rank)
    ref.lora_silu(rank, xa, split, M, B, rows, tab_d, tok_slot, slot_scale, n, y, rows, theirs)
    torch.cuda.synchronize()
    assert torch.equal(mine.view(torch.int16), theirs.view(torch.int16))
    sc = slot_scale[tok_slot.long()].cpu().numpy()
    delta = R.lora_delta(xa.cpu().numpy(), B.float().cpu().numpy(), tab, sc, silu=True)
    want = R.lora_silu(y.cpu().numpy(), delta).astype(np.float32)
    got = mine.float().cpu().numpy()
    assert np.abs(got - want).max() <= 2 ** -9 * max(1.0, np.abs(want).max())
    # tokens without the adapter: the plain SwiGLU of the product
    idle = np.nonzero(sc == 0)[0]
    plain = R.lora_silu(y.cpu().numpy(), np.zeros_like(delta)).astype(np.float32)
    assert np.abs(got[idle] - plain[idle]).max() <= 2 ** -9 * max(1.0, np.abs(plain).max())


def test_lora_rank_not_served(ctx):
    from qwenny_b200._lib import QbError
    M, split, xa, B, tab, tab_d, tok_slot, slot_scale, y = setup(16, 256, 4, 1, False)
    with pytest.raises(QbError):
        ctx.lora_add(xa, split, M, B, 256, tab_d, tok_slot, slot_scale, 4, y, 256, 12)


def _rel(a, b):
    return np.linalg.norm(a - b) / np.linalg.norm(b)


def test_steps_with_an_adapter_match_the_cpu_oracle(ctx):
    """The step runner with a LoRA on every layer (Model::set_adapter): slots 0 and 2 use it, slot 1 does not. Decode /
    verify steps and a prompt chunk (tensor-core products) against the CPU oracle of y = W x + s B (A x); the tokens of
    the slot without the adapter get the base model's values bit for bit; steps without adapter tokens run the base
    model's kernels."""
    from oracle import cpu_step
    from qwenny_b200 import model as M
    kw = dict(nlayers=2, slots=3, max_ctx=128, vocab=2000, seed=41, pattern=("delta", "attn"))
    m = M.synthetic(ctx, **kw)
    base = M.synthetic(ctx, **kw)  # the same weights, no adapter
    M.synthetic_adapter(m, rank=16, seed=7, std=0.12)
    cpu = cpu_step.CpuModel.from_device(m)
    scales = [2.0, 0.0, 0.5]
    for s, v in enumerate(scales):
        m.set_slot_scale(s, v)
    cpu.slot_scale = scales
    seq = [(13 + 29 * i) % 2000 for i in range(100)]
    # a prompt chunk of 40 + 24 + 3 tokens
    toks = [(seq[i], 0, i) for i in range(40)] + [(seq[50 + i], 1, i) for i in range(24)] + \
           [(seq[80 + i], 2, i) for i in range(3)]
    out = [39, 63, 66]
    # (the two models share one context, which serves one stream at a time: each step is read back before the next)
    m.step(toks, out)
    lg = m.logits().cpu().numpy()
    base.step(toks, out)
    blg = base.logits().cpu().numpy()
    want, greedy, h, xn = cpu.step(toks, out)
    assert _rel(lg[:, :2000], want[:, :2000]) < 3e-3
    assert np.array_equal(lg[1], blg[1])  # slot 1: the base model, bit for bit
    assert _rel(lg[0], blg[0]) > 0.03  # and the adapter does change the others (ten times the oracle tolerance)
    # verify steps: five tokens of slot 0, one of slot 1, two of slot 2
    pos = [40, 24, 3]
    for rnd in range(2):
        toks = [(seq[pos[0] + i], 0, pos[0] + i) for i in range(5)] + [(seq[70 + rnd], 1, pos[1])] + \
               [(seq[90 + i], 2, pos[2] + i) for i in range(2)]
        out = list(range(8))
        m.step(toks, out)
        lg = m.logits().cpu().numpy()
        base.step(toks, out)
        blg = base.logits().cpu().numpy()
        want, greedy, h, xn = cpu.step(toks, out)
        assert _rel(lg[:, :2000], want[:, :2000]) < 3e-3
        assert np.array_equal(lg[5], blg[5])
        pos = [pos[0] + 5, pos[1] + 1, pos[2] + 2]
    # a step of slot 1 alone: no adapter token, the base model's kernels and launch count
    m.step([(seq[75], 1, pos[1])], [0])
    lg = m.logits().cpu().numpy()
    base.step([(seq[75], 1, pos[1])], [0])
    assert np.array_equal(lg, base.logits().cpu().numpy())
    from qwenny_b200._lib import lib
    assert lib().qb_model_step_kernels(m.h) == lib().qb_model_step_kernels(base.h)
    # without the adapter again: slot 0's next step differs from the adapted one only through its caches
    m.set_adapter(0, None)
    m.set_adapter(1, None)
    m.step([(seq[pos[0]], 0, pos[0])], [0])
    assert lib().qb_model_step_kernels(m.h) == lib().qb_model_step_kernels(base.h)
    m.close()
    base.close()
