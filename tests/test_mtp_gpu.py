"""The MTP draft step: mtp_in against the reference's kernel and the CPU oracle; the
greedy draft chain through the library's host API (qb_model_draft = Engine::draft with argmax rows) against the CPU
oracle of the same chain, with the whole output layer and with a draft head."""
import numpy as np
import pytest
import torch

from oracle import cpu_step, ref_cuda
from oracle import ref_ops as R
from qwenny_b200 import model as M
from qwenny_b200 import synth

pytestmark = pytest.mark.gpu


def test_mtp_in(ctx, ref):
    g = synth.gen(501)
    n = 6
    emb = (torch.randn(n, R.H, generator=g) * 0.02).cuda()
    h = torch.randn(9, R.H, generator=g).cuda()
    rows = torch.tensor([8, 0, 3, 3, 7, 1], dtype=torch.int32).cuda()
    fw, pe, ph = [(1 + 0.02 * torch.randn(R.H, generator=g)).cuda() for _ in range(3)]
    mine = torch.zeros(n, 2 * R.H, dtype=torch.float16, device="cuda")
    theirs = torch.zeros_like(mine)
    ctx.mtp_in(emb, h, rows, fw, pe, ph, mine, n)
    import ctypes as C
    ref.launch("mtp_in", (n, 1, 1), 256, 0, [ref_cuda._ptr(emb), ref_cuda._ptr(h), ref_cuda._ptr(rows), ref_cuda._ptr(fw),
                                             ref_cuda._ptr(pe), ref_cuda._ptr(ph), ref_cuda._ptr(theirs), C.c_float(1e-6)])
    torch.cuda.synchronize()
    a, b = mine.float().cpu().numpy(), theirs.float().cpu().numpy()
    # the two kernels add a row's squares in different orders: an f16 ulp on the few values that sit on a boundary
    assert np.abs(a - b).max() <= np.abs(b).max() * 2 ** -10 and (a != b).mean() < 1e-2
    want = R.mtp_in(emb.cpu().numpy(), h.cpu().numpy(), rows.cpu().numpy(), fw.cpu().numpy(), pe.cpu().numpy(),
                    ph.cpu().numpy()).astype(np.float32)
    assert np.abs(a - want).max() <= np.abs(want).max() * 2 ** -10 and (a != want).mean() < 1e-2


def test_draft_pick(ctx):
    keys = torch.tensor([(7 << 32) | (0xffffffff - 5), (9 << 32) | (0xffffffff - 2)], dtype=torch.int64).cuda()
    ids = torch.tensor([100, 101, 102, 103, 104, 105], dtype=torch.int32).cuda()
    nxt = torch.zeros(2, dtype=torch.int32, device="cuda")
    chain = torch.zeros(2, 8, dtype=torch.int32, device="cuda")
    ctx.draft_pick(keys, ids, 2, nxt, chain, 8, 3)
    assert nxt.tolist() == [105, 102] and chain[:, 3].tolist() == [105, 102]
    ctx.draft_pick(keys, None, 2, nxt, chain, 8, 0)
    assert nxt.tolist() == [5, 2] and chain[:, 0].tolist() == [5, 2]


@pytest.mark.parametrize("draft_rows", [0, 1000])
def test_draft_chain_matches_cpu_oracle(ctx, draft_rows):
    """A verify step, then four greedy drafts per accepted row: the first MTP step on the target's hidden states, the
    rest on the MTP's own with the draft just made as the token (its id never leaves the device); with the whole
    output layer and with a 1000-row draft head. Twice, so that the second chain finds the MTP layer's cache filled."""
    m = M.synthetic(ctx, nlayers=2, slots=2, max_ctx=256, vocab=2000, seed=31, pattern=("delta", "attn"), mtp=True,
                    draft_rows=draft_rows)
    cpu = cpu_step.CpuModel.from_device(m)
    seq = [(17 + 29 * i) % 2000 for i in range(40)]
    pos = 0
    for rnd in range(2):
        toks = [(seq[pos + i], 0, pos + i) for i in range(5)] + ([(3, 1, 0)] if rnd == 0 else [(4, 1, 1)])
        out = list(range(len(toks)))
        m.step(toks, out)
        got = m.argmax()
        logits, want, h, xn = cpu.step(toks, out)
        assert got == [int(t) for t in want]
        # the MTP's tokens: each position's NEXT token (the verify step's greedy tokens), hidden states of the same rows;
        # drafts wanted for the last row of each sequence
        mt = [(got[i], toks[i][1], toks[i][2] + 1) for i in range(len(toks))]
        rows = list(range(len(toks)))
        outs = [4, 5]
        drafts = m.draft(mt, rows, outs, 4)
        want_d, want_logits = cpu.draft(mt, rows, outs, 4)
        # the last MTP step's logits, and the chains (a near-tie in the oracle's top two may flip a draft)
        last = m.logits().cpu().numpy()
        a, b = last[:, :want_logits[-1].shape[1]], want_logits[-1]
        assert np.linalg.norm(a - b) / np.linalg.norm(b) < 2e-3
        for i in range(len(outs)):
            for t in range(4):
                if drafts[i][t] != want_d[i][t]:
                    srt = np.sort(want_logits[t][i])
                    assert srt[-1] - srt[-2] < 1e-3, (i, t, drafts[i], want_d[i])
                    break
        pos += 5
