"""The GPU sampler (qb_sample_rows, qb_draft_sample) draw for draw against the reference's own compiled kernels
(oracle/_ref) on the same device buffers, and against the CPU oracle of the reference's host definition
(oracle/ref_sample.py = src/sample.rs), the way the reference's samplecheck does (src/checks.rs:685-888): its
parameter sets, histories that make the penalties matter, argmax drafts, sampled drafts with their stored q.

Tokens must be IDENTICAL to the reference kernel's (same arithmetic, same order). Against the host definition the
prefix sums are added in another order (a tree on the GPU, a sequential scan on the host), so a draw may differ only
where its uniform number sits within rounding distance of a boundary: the oracle reports that margin and the test
allows a difference only below 1e-5 (none is expected among a few hundred draws)."""
import numpy as np
import pytest
import torch

from oracle import ref_cuda
from oracle import ref_sample as S

pytestmark = pytest.mark.gpu

V = ref_cuda.VOCAB  # the reference module's compile-time vocabulary
QD, QCAP = S.QD, S.QCAP
F = np.float32

# (temperature, top_k, top_p, repetition penalty, presence penalty): src/checks.rs:703-713 and :752
SETS = [(0.0, 50, 1.0, 1.1, 0.0), (0.1, 50, 1.0, 1.1, 0.0), (0.7, 20, 0.8, 1.0, 0.0), (1.0, 1024, 0.95, 1.1, 0.0),
        (1.5, 300, 1.0, 1.0, 0.0), (0.9, 5, 0.5, 1.3, 0.0), (0.0, 20, 1.0, 1.0, 1.5), (1.0, 20, 0.95, 1.0, 1.5),
        (0.7, 20, 0.8, 1.1, 2.0)]


def bitset(tokens, vocab=V):
    w = np.zeros(vocab // 32, dtype=np.uint32)
    for t in tokens:
        w[t >> 5] |= np.uint32(1 << (t & 31))
    return w


def member(words):
    return np.unpackbits(words.view(np.uint8), bitorder="little").astype(bool)


class Rows:
    """A step's arrays as the reference's Step holds them (src/cuda/core.rs:725-760): two sequences in slots 0 and 1
    with histories whose tokens repeat, the last 20 of each counted as generated; logits with a handful of likely
    tokens among them."""

    def __init__(self, seed, whole=True, vocab=V, slots=2):
        g = np.random.default_rng(seed)
        self.vocab = vocab
        hist = [[1000 + (i * 7) % 23 for i in range(60)], [5000 + (i * 13) % 37 for i in range(40)]]
        self.hist = hist
        if whole:  # the histories as the step's tokens: those after the first count as the step's drafts
            ids = hist[0] + hist[1]
            tok_slot = [0] * 60 + [1] * 40
            out_rows, row_first = [59, 99], [0, 60]
        else:
            ids = [hist[0][-1], hist[1][-1]]
            tok_slot, out_rows, row_first = [0, 1], [0, 1], [0, 1]
        self.ids, self.tok_slot_h, self.out_rows_h, self.row_first_h = ids, tok_slot, out_rows, row_first
        self.n_out = 2
        logits = (g.standard_normal((2, vocab)) * 2.0).astype(F)
        for j in range(2):  # likely tokens, some of them in the histories
            hot = list(g.integers(0, vocab, 12)) + hist[j][:6]
            logits[j, hot] += g.uniform(4, 9, len(hot)).astype(F)
        self.logits_h = logits
        self.seen_h = np.stack([bitset(hist[0]), bitset(hist[1])])
        self.outs_h = np.stack([bitset(hist[0][-20:]), bitset(hist[1][-20:])])
        dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).astype(dt)).cuda()
        self.logits = dev(logits, F)
        self.ids_d, self.tok_slot = dev(ids, np.int32), dev(tok_slot, np.int32)
        self.out_rows, self.row_first = dev(out_rows, np.int32), dev(row_first, np.int32)
        self.seen = torch.from_numpy(self.seen_h.view(np.int32)).cuda()
        self.outs = torch.from_numpy(self.outs_h.view(np.int32)).cuda()
        self.qtok = torch.full((slots * QD,), -1, dtype=torch.int32, device="cuda")
        self.qn = torch.zeros(slots * QD, dtype=torch.int32, device="cuda")
        self.qid = torch.zeros(slots * QD * QCAP, dtype=torch.int32, device="cuda")
        self.qp = torch.zeros(slots * QD * QCAP, dtype=torch.float32, device="cuda")

    def sets(self, j):
        """seen / generated of row j as the host sees them (Step::sample_on_host, src/cuda/core.rs:1008-1016)."""
        slot = self.tok_slot_h[self.out_rows_h[j]]
        step = self.ids[self.row_first_h[j] + 1: self.out_rows_h[j] + 1]
        seen, gen = member(self.seen_h[slot]).copy(), member(self.outs_h[slot]).copy()
        seen[step] = True
        gen[step] = True
        return seen, gen

    def mine(self, ctx, params):
        p = torch.from_numpy(np.ascontiguousarray(params, dtype=F)).cuda()
        tok = torch.full((self.n_out,), -7, dtype=torch.int32, device="cuda")
        acc = torch.full((self.n_out,), -7, dtype=torch.int32, device="cuda")
        ctx.sample_rows(self.logits, self.vocab, self.n_out, self.out_rows, self.tok_slot, self.ids_d, self.row_first,
                        self.seen, self.outs, p, self.qtok, self.qn, self.qid, self.qp, tok, acc)
        torch.cuda.synchronize()
        return tok.tolist(), acc.tolist()

    def theirs(self, ref, params):
        p = torch.from_numpy(np.ascontiguousarray(params, dtype=F)).cuda()
        tok = torch.full((self.n_out,), -7, dtype=torch.int32, device="cuda")
        acc = torch.full((self.n_out,), -7, dtype=torch.int32, device="cuda")
        ref.sample_rows(self.logits, self.out_rows, self.tok_slot, self.ids_d, self.row_first, self.seen, self.outs, p,
                        self.qtok, self.qn, self.qid, self.qp, tok, acc, self.n_out)
        torch.cuda.synchronize()
        return tok.tolist(), acc.tolist()


def check_host(got_tok, got_acc, want, margin, what):
    tok, acc = want
    if (got_tok, bool(got_acc)) != (tok, acc):
        assert margin < 1e-5, f"{what}: GPU {(got_tok, got_acc)}, host {want}, margin {margin}"
        return 1
    return 0


@pytest.mark.parametrize("whole", [True, False])
def test_sample_rows_matches_reference_and_host(ctx, ref, whole):
    rows = Rows(11, whole)
    rng = S.Rng(7)
    near = total = 0
    for (temp, k, p, rep, pres) in SETS:
        for it in range(6):
            params = np.stack([S.params_row(temp, k, p, rep, pres, rng) for _ in range(2)])
            tok, acc = rows.mine(ctx, params)
            rt, ra = rows.theirs(ref, params)
            assert (tok, acc) == (rt, ra), f"{(temp, k, p, rep, pres)} draw {it}: {tok, acc} != reference {rt, ra}"
            for j in range(2):
                seen, gen = rows.sets(j)
                t, a, margin = S.sample_row(rows.logits_h[j], seen, gen, params[j], want_margin=True)
                near += check_host(tok[j], acc[j], (t, a), margin, f"{(temp, k, p, rep, pres)} row {j}")
                total += 1
    assert near <= 1, f"{near} of {total} draws sat on a boundary"


def test_argmax_drafts_accept_or_resample(ctx, ref):
    """Rows with a draft from the draft layer's argmax: accepted with p(d), else a draw without d (u2)."""
    rows = Rows(12, whole=False)
    rng = S.Rng(9)
    near = accepted = 0
    for (temp, k, p, rep, pres) in [(1.0, 1024, 1.0, 1.0, 0.0), (0.8, 20, 0.9, 1.1, 0.0), (1.5, 50, 1.0, 1.3, 0.0),
                                    (1.0, 20, 0.95, 1.0, 1.5), (0.0, 20, 1.0, 1.0, 0.0)]:
        base = np.array([temp, k, p, rep, 0, 0, -1, pres], dtype=F)
        for it in range(8):
            params = []
            for j in range(2):
                seen, gen = rows.sets(j)
                vals, idx = S.ranked(rows.logits_h[j], seen, gen, base, 4)
                d = int(idx[it % 4]) if it < 6 else 77 + it  # likely tokens, then one outside the kept set
                params.append(S.params_row(temp, k, p, rep, pres, rng, draft=d))
            params = np.stack(params)
            tok, acc = rows.mine(ctx, params)
            assert (tok, acc) == rows.theirs(ref, params)
            for j in range(2):
                seen, gen = rows.sets(j)
                t, a, margin = S.sample_row(rows.logits_h[j], seen, gen, params[j], want_margin=True)
                near += check_host(tok[j], acc[j], (t, a), margin, f"draft row {j}")
                accepted += acc[j]
    assert near <= 1 and accepted > 5


@pytest.mark.parametrize("head", [0, 65536])
def test_sampled_drafts(ctx, ref, head):
    """draft_sample over the whole output layer or a draft head's columns: the draft, the stored q (ids ascending,
    probabilities) bit for bit the reference kernel's; then the target's rows whose draft is marked sampled: accepted
    with min(1, p / q) or drawn from max(0, p - q), against the reference kernel and the host's sample_row_q."""
    g = np.random.default_rng(21)
    rng = S.Rng(5)
    near = acc_n = 0
    for (temp, k, p, rep, pres) in [(1.0, 20, 0.95, 1.0, 1.5), (0.7, 0, 0.8, 1.1, 0.0), (1.3, 50, 1.0, 1.0, 0.0)]:
        for it in range(4):
            rows = Rows(30 + it, whole=False)
            width = head or V
            ld = width + 64 if head else V
            head_ids = np.sort(g.permutation(V)[:head]).astype(np.int32) if head else None
            dl = (g.standard_normal((2, ld)) * 2.0).astype(F)
            for j in range(2):
                dl[j, g.integers(0, width, 10)] += g.uniform(3, 8, 10).astype(F)
            dlog = torch.from_numpy(dl).cuda()
            hid = None if head_ids is None else torch.from_numpy(head_ids).cuda()
            t_idx = it % 3
            chain = [int(g.integers(0, V)) for _ in range(t_idx)]  # the chain's drafts before this one
            if head_ids is not None and t_idx:
                chain[0] = int(head_ids[int(np.argmax(dl[0, :width]))])  # a draft the penalty must reach
            for s in range(2):
                rows.qtok[s * QD: s * QD + t_idx] = torch.tensor(chain, dtype=torch.int32)
            dparams = np.stack([S.draft_row(temp, k, p, rep, pres) for _ in range(2)])
            for j in range(2):
                dparams[j, 4], dparams[j, 5] = rng.next_f32(), t_idx
            dp = torch.from_numpy(dparams).cuda()
            # the reference kernel, into its own copy of the q arrays
            theirs = [x.clone() for x in (rows.qtok, rows.qn, rows.qid, rows.qp)]
            rd = torch.full((2,), -7, dtype=torch.int32, device="cuda")
            ref.draft_sample(dlog, width, ld, hid, rows.out_rows, rows.tok_slot, rows.seen, rows.outs, dp, rd, *theirs,
                             2)
            md = torch.full((2,), -7, dtype=torch.int32, device="cuda")
            ctx.draft_sample(dlog, width, ld, hid, V, 2, rows.out_rows, rows.tok_slot, rows.seen, rows.outs, dp, md,
                             rows.qtok, rows.qn, rows.qid, rows.qp)
            torch.cuda.synchronize()
            assert md.tolist() == rd.tolist()
            mine = (rows.qtok, rows.qn, rows.qid, rows.qp)
            assert torch.equal(mine[0], theirs[0]) and torch.equal(mine[1], theirs[1])
            drafts = md.tolist()
            for j in range(2):
                q = j * QD + t_idx
                n = int(rows.qn[q])
                assert 0 < n <= QCAP
                assert torch.equal(mine[2][q * QCAP: q * QCAP + n], theirs[2][q * QCAP: q * QCAP + n])
                assert torch.equal(mine[3][q * QCAP: q * QCAP + n].view(torch.int32),
                                   theirs[3][q * QCAP: q * QCAP + n].view(torch.int32))
                # the host's statement of the same draw
                seen, gen = member(rows.seen_h[j]).copy(), member(rows.outs_h[j]).copy()
                seen[chain] = True
                gen[chain] = True
                tok, qi, qv, margin = S.draft_draw(dl[j, :width], seen, gen, dparams[j], head_ids, want_margin=True)
                assert np.array_equal(qi, rows.qid[q * QCAP: q * QCAP + n].cpu().numpy())
                np.testing.assert_allclose(rows.qp[q * QCAP: q * QCAP + n].cpu().numpy(), qv, rtol=2e-5, atol=1e-9)
                if tok != drafts[j]:
                    assert margin < 1e-5
                    near += 1
            if t_idx != 0:
                continue
            # the target's step feeds the draft at index 0 of each chain: rows whose draft is marked sampled
            params = []
            for j in range(2):
                r = S.params_row(temp, k if k else 40, p, rep, pres, rng, draft=drafts[j])
                S.mark_sampled(r)
                params.append(r)
            params = np.stack(params)
            tok, acc = rows.mine(ctx, params)
            assert (tok, acc) == rows.theirs(ref, params)
            for j in range(2):
                q = j * QD
                n = int(rows.qn[q])
                seen, gen = rows.sets(j)
                r = params[j].copy()
                r[6] = drafts[j]
                t, a, margin = S.sample_row_q(rows.logits_h[j], seen, gen, r,
                                              rows.qid[q * QCAP: q * QCAP + n].cpu().numpy(),
                                              rows.qp[q * QCAP: q * QCAP + n].cpu().numpy(), want_margin=True)
                near += check_host(tok[j], acc[j], (t, a), margin, "sampled draft")
                acc_n += acc[j]
    assert near <= 1


def test_equal_logits_rank_by_index(ctx):
    """src/sample.rs:217-229 on the device: a flat row. With top_k 1024 the kept tokens are 0..1023 (ties go to the
    lower index) whatever the blocks' order of arrival, and a draw near 1 takes the last of them; top_k 0 is the
    host's row. The reference kernel keeps whichever 2048 ties its atomics reach first, so it is not the measure
    here; the host definition is."""
    rows = Rows(40, whole=False)
    rows.logits.zero_()
    flat = np.zeros(V, dtype=F)
    for u, k, want in [(0.9999, 1024, 1023), (0.5, 1024, 512), (0.9999, 50, 49), (0.0, 300, 0)]:
        params = np.array([[1, k, 1, 1, u, 0, -1, 0]] * 2, dtype=F)
        tok, acc = rows.mine(ctx, params)
        host = S.sample_row(flat, None, None, params[0])[0]
        assert tok == [host, host] and acc == [0, 0] and abs(host - want) <= 1
    tok, acc = rows.mine(ctx, np.array([[1, 0, 1, 1, 0.3, 0, -1, 0], [1, 2000, 1, 1, 0.3, 0, -1, 0]], dtype=F))
    assert acc == [-1, -1]
    # top_k 0 with a top-p cut over a flat row: the cut lies far beyond the 1024 candidates, the host's row too
    tok, acc = rows.mine(ctx, np.array([[1, 0, 0.9, 1, 0.3, 0, -1, 0]] * 2, dtype=F))
    assert acc == [-1, -1]
    # ties below distinct values: three large logits, then the flat rest
    lg = np.zeros((2, V), dtype=F)
    lg[:, [70000, 5, 200000]] = [3.0, 2.0, 1.0]
    rows.logits.copy_(torch.from_numpy(lg))
    for u in (0.1, 0.6, 0.85, 0.97, 0.9999):
        params = np.array([[1, 40, 1, 1, u, 0, -1, 0]] * 2, dtype=F)
        tok, _ = rows.mine(ctx, params)
        t, _, margin = S.sample_row(lg[0], None, None, params[0], want_margin=True)
        assert tok == [t, t] or margin < 1e-5


def test_greedy_rows_with_penalties(ctx, ref):
    rows = Rows(50, whole=True)
    for rep, pres in [(1.0, 0.0), (1.8, 0.0), (1.0, 6.0), (1.5, 3.0)]:
        for d in (-1, 3):
            params = np.array([[0, 50, 1, rep, 0, 0, d, pres], [1, 1, 1, rep, 0, 0, d, pres]], dtype=F)
            if d >= 0:
                for j in range(2):
                    seen, gen = rows.sets(j)
                    params[j, 6] = S.sample_row(rows.logits_h[j], seen, gen, params[j])[0] if j == 0 else 3
            tok, acc = rows.mine(ctx, params)
            assert (tok, acc) == rows.theirs(ref, params)
            for j in range(2):
                seen, gen = rows.sets(j)
                assert (tok[j], bool(acc[j])) == S.sample_row(rows.logits_h[j], seen, gen, params[j])


def test_small_vocabulary_and_ragged_width(ctx):
    """Widths that are not a multiple of the cluster's slices, narrower than one slice, and unaligned rows."""
    g = np.random.default_rng(60)
    for vocab, width, ld in [(2048, 2048, 2048), (4096, 1000, 1003), (32000, 31999, 32001), (64, 40, 40)]:
        n_out = 2
        logits = (g.standard_normal((n_out, ld)) * 2).astype(F)
        seen_h = np.stack([bitset(g.integers(0, vocab, 50), vocab) for _ in range(2)])
        outs_h = np.stack([bitset(g.integers(0, vocab, 20), vocab) for _ in range(2)])
        out_rows = torch.tensor([0, 1], dtype=torch.int32).cuda()
        tok_slot = torch.tensor([1, 0], dtype=torch.int32).cuda()
        qtok = torch.full((2 * QD,), -1, dtype=torch.int32, device="cuda")
        qn = torch.zeros(2 * QD, dtype=torch.int32, device="cuda")
        qid = torch.zeros(2 * QD * QCAP, dtype=torch.int32, device="cuda")
        qp = torch.zeros(2 * QD * QCAP, dtype=torch.float32, device="cuda")
        head_ids = np.sort(g.permutation(vocab)[:width]).astype(np.int32)
        dparams = np.stack([S.draft_row(0.9, 30, 0.9, 1.2, 0.5) for _ in range(n_out)])
        dparams[:, 4] = g.uniform(0, 1, n_out).astype(F)
        drafts = torch.full((n_out,), -7, dtype=torch.int32, device="cuda")
        ctx.draft_sample(torch.from_numpy(logits).cuda(), width, ld, torch.from_numpy(head_ids).cuda(), vocab, n_out,
                         out_rows, tok_slot, torch.from_numpy(seen_h.view(np.int32)).cuda(),
                         torch.from_numpy(outs_h.view(np.int32)).cuda(), torch.from_numpy(dparams).cuda(), drafts,
                         qtok, qn, qid, qp)
        torch.cuda.synchronize()
        for j in range(n_out):
            slot = [1, 0][j]
            tok, qi, qv, margin = S.draft_draw(logits[j, :width], member(seen_h[slot]), member(outs_h[slot]),
                                               dparams[j], head_ids, want_margin=True)
            assert drafts[j].item() == tok or margin < 1e-5
            n = int(qn[slot * QD])
            assert np.array_equal(qid[slot * QD * QCAP:][:n].cpu().numpy(), qi)
            np.testing.assert_allclose(qp[slot * QD * QCAP:][:n].cpu().numpy(), qv, rtol=2e-5, atol=1e-9)


def test_speed_against_the_reference_kernel(ctx, ref, capsys):
    """Five rows of the 27B vocabulary, top_k 50 with penalties: CUDA-event time of 20 launches of each kernel. The
    figure is printed; the check is only that the cluster kernel is not the slower one."""
    rows = Rows(70, whole=False)
    params = np.array([[0.8, 50, 0.95, 1.1, 0.3, 0.6, -1, 0.5]] * 2, dtype=F)
    p = torch.from_numpy(params).cuda()
    tok = torch.zeros(2, dtype=torch.int32, device="cuda")
    acc = torch.zeros(2, dtype=torch.int32, device="cuda")
    mine = lambda: ctx.sample_rows(rows.logits, V, 2, rows.out_rows, rows.tok_slot, rows.ids_d, rows.row_first,
                                   rows.seen, rows.outs, p, rows.qtok, rows.qn, rows.qid, rows.qp, tok, acc)
    theirs = lambda: ref.sample_rows(rows.logits, rows.out_rows, rows.tok_slot, rows.ids_d, rows.row_first, rows.seen,
                                     rows.outs, p, rows.qtok, rows.qn, rows.qid, rows.qp, tok, acc, 2)
    us = []
    for fn in (mine, theirs):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us.append(e0.elapsed_time(e1) * 1e3 / 20)
    with capsys.disabled():
        print(f"\nsample_rows, 2 rows x {V}: {us[0]:.1f} us here, {us[1]:.1f} us the reference kernel")
    assert us[0] < us[1]


@pytest.mark.parametrize("draft_rows", [0, 1000])
def test_model_sampling_and_sampled_draft_chain(ctx, draft_rows):
    """Through the host API, the design of the reference's samplecheck (src/checks.rs:685-818): a sequence's history
    in one step, its last row sampled under several parameter sets (device rows and host rows); then drafts drawn on
    the device from the MTP layer's distribution, fed to the target, and accepted or resampled against the stored q:
    every token is the host definition's for the logits the model produced."""
    from qwenny_b200 import model as M
    vocab = 2000
    m = M.synthetic(ctx, nlayers=2, slots=2, max_ctx=256, vocab=vocab, seed=77, pattern=("delta", "attn"), mtp=True,
                    draft_rows=draft_rows)
    vr = m.lm_head.n  # padded rows
    hist = [100 + (i * 7) % 23 for i in range(40)]
    n = len(hist)
    gen = set(hist[-12:])
    m.set_outputs(0, bitset(gen, vr))
    rng = S.Rng(13)
    m.step([(t, 0, i) for i, t in enumerate(hist)], [n - 1])
    lg = m.logits().cpu().numpy()[0, :vocab]
    seen = np.zeros(vocab, dtype=bool)
    seen[hist] = True
    genb = np.zeros(vocab, dtype=bool)
    genb[list(gen)] = True
    genb[hist[1:]] = True  # the step's tokens after its first count as drafts fed so far
    near = 0
    for (temp, k, p, rep, pres) in SETS + [(1.0, 0, 0.95, 1.1, 0.0), (1.5, 0, 1.0, 1.0, 0.7), (0.8, 1500, 0.9, 1.2, 0.0)]:
        for it in range(3):
            r = S.params_row(temp, k, p, rep, pres, rng)
            got = m.sample([r])[0]
            t, a, margin = S.sample_row(lg, seen, genb, r, want_margin=True)
            if (k == 0 and p >= 1.0) or k > QCAP:
                assert got == (t, a)  # a host row: the host definition's arithmetic, no allowance
            else:
                near += check_host(got[0], got[1], (t, a), margin, f"{(temp, k, p, rep, pres)}")
    assert near <= 1
    # sampled drafts
    head_ids = m.mtp["head_ids"].cpu().numpy()[:draft_rows] if draft_rows else None
    for (temp, k, p, rep, pres) in [(1.0, 20, 0.95, 1.0, 1.5), (0.7, 0, 0.8, 1.1, 0.0), (1.3, 50, 1.0, 1.0, 0.0)]:
        for it in range(3):
            nxt = 300 + it
            m.step([(t, 0, i) for i, t in enumerate(hist)], [n - 1])
            ds = S.draft_row(temp, k, p, rep, pres)
            u = np.array([[rng.next_f32() for _ in range(3)]], dtype=F)
            d = m.draft_sampled([(nxt, 0, n - 1)], [n - 1], [0], 3, [ds], u)[0]
            assert len(d) == 3
            # the last draft step's logits: the host's statement of its draw
            dl = m.logits().cpu().numpy()[0]
            width = draft_rows or vocab
            seen_d, gen_d = seen.copy(), np.zeros(vocab, dtype=bool)
            gen_d[list(gen)] = True
            seen_d[d[:2]] = True
            gen_d[d[:2]] = True
            r = ds.copy()
            r[4], r[5] = u[0, 2], 2
            tok, qi, qv, margin = S.draft_draw(dl[:width], seen_d, gen_d, r, head_ids, want_margin=True)
            ids2, p2, t2 = m.draft_q(0, 2)
            assert t2 == d[2] and np.array_equal(ids2, qi)
            np.testing.assert_allclose(p2, qv, rtol=2e-5, atol=1e-9)
            assert tok == d[2] or margin < 1e-5
            for t in range(3):
                ids_t, p_t, tok_t = m.draft_q(0, t)
                assert tok_t == d[t] and tok_t in ids_t and abs(p_t.sum() - 1) < 1e-4 and np.all(np.diff(ids_t) > 0)
            # the target's step over the next token and the drafts; rows 0..2 carry a sampled draft
            step = [(nxt, 0, n)] + [(d[j], 0, n + 1 + j) for j in range(3)]
            m.step(step, [0, 1, 2, 3])
            lgs = m.logits().cpu().numpy()[:, :vocab]
            rows = []
            for j in range(4):
                r = S.params_row(temp, k if k else 40, p, rep, pres, rng, draft=d[j] if j < 3 else None)
                if j < 3:
                    S.mark_sampled(r)
                rows.append(r)
            got = m.sample(rows)
            seen_t = seen.copy()
            seen_t[[nxt] + d] = True  # the steps mark all their tokens, the drafts included
            for j in range(4):
                g2 = np.zeros(vocab, dtype=bool)
                g2[list(gen)] = True
                g2[d[:j]] = True
                if j < 3:
                    ids_j, p_j, _ = m.draft_q(0, j)
                    r = rows[j].copy()
                    r[6] = d[j]
                    t, a, margin = S.sample_row_q(lgs[j], seen_t, g2, r, ids_j, p_j, want_margin=True)
                else:
                    t, a, margin = S.sample_row(lgs[j], seen_t, g2, rows[j], want_margin=True)
                near += check_host(got[j][0], got[j][1], (t, a), margin, f"sampled draft row {j}")
                if not got[j][1]:
                    break
    assert near <= 1
    m.close()


def test_whole_vocabulary_rows_with_a_top_p_cut(ctx):
    """top_k 0 with top_p < 1 (the reference sends these rows to the host): made on the device when the cut falls among
    the 1024 most likely tokens, against the mass of the whole vocabulary; the tokens are the host definition's."""
    rows = Rows(80, whole=True)
    # logits as peaked as a language model's: a few dozen likely tokens carry the mass, 248,000 unlikely ones the rest
    g = np.random.default_rng(81)
    lg = g.standard_normal((2, V)).astype(F)
    for j in range(2):
        hot = list(g.integers(0, V, 40)) + rows.hist[j][:6]
        lg[j, hot] += g.uniform(9, 16, len(hot)).astype(F)
    rows.logits_h = lg
    rows.logits.copy_(torch.from_numpy(lg))
    rng = S.Rng(21)
    near = device = 0
    for (temp, p, rep, pres) in [(1.0, 0.95, 1.1, 0.0), (0.7, 0.8, 1.0, 0.0), (1.0, 0.5, 1.3, 1.5), (1.3, 0.9, 1.0, 0.0)]:
        for it in range(5):
            d = None
            if it >= 3:  # with an argmax draft
                seen, gen = rows.sets(0)
                d = int(S.ranked(rows.logits_h[0], seen, gen, np.array([temp, 0, p, rep, 0, 0, -1, pres], dtype=F), 2)[1][it - 3])
            params = np.stack([S.params_row(temp, 0, p, rep, pres, rng, draft=d) for _ in range(2)])
            tok, acc = rows.mine(ctx, params)
            for j in range(2):
                seen, gen = rows.sets(j)
                t, a, margin = S.sample_row(rows.logits_h[j], seen, gen, params[j], want_margin=True)
                if acc[j] < 0:
                    # the host's row: its kept set must indeed be larger than the candidates
                    assert len(S.kept_dist(rows.logits_h[j], seen, gen, params[j])[1]) > QCAP - 8
                    continue
                device += 1
                near += check_host(tok[j], acc[j], (t, a), margin, f"top_k 0, top_p {p}, row {j}")
    assert device >= 30 and near <= 1


def test_many_rows_in_one_launch(ctx, ref):
    """Twenty logit rows of one sequence (a long verify step: each row's penalties see the step's tokens before it): more
    clusters than fit the SMs at once, every row the reference kernel's token."""
    n = 20
    g = np.random.default_rng(90)
    lg = (g.standard_normal((n, V)) * 2).astype(F)
    for j in range(n):
        lg[j, g.integers(0, V, 10)] += g.uniform(4, 9, 10).astype(F)
    logits = torch.from_numpy(lg).cuda()
    ids = torch.from_numpy(g.integers(0, V, n).astype(np.int32)).cuda()
    out_rows = torch.arange(n, dtype=torch.int32, device="cuda")
    zeros = torch.zeros(n, dtype=torch.int32, device="cuda")
    base = Rows(91, whole=False)
    rng = S.Rng(17)
    params = np.stack([S.params_row(*SETS[j % len(SETS)][:4], SETS[j % len(SETS)][4], rng) for j in range(n)])
    p = torch.from_numpy(params).cuda()
    res = []
    for fn in ("mine", "theirs"):
        tok = torch.full((n,), -7, dtype=torch.int32, device="cuda")
        acc = torch.full((n,), -7, dtype=torch.int32, device="cuda")
        if fn == "mine":
            ctx.sample_rows(logits, V, n, out_rows, zeros, ids, zeros, base.seen, base.outs, p, base.qtok, base.qn,
                            base.qid, base.qp, tok, acc)
        else:
            ref.sample_rows(logits, out_rows, zeros, ids, zeros, base.seen, base.outs, p, base.qtok, base.qn, base.qid,
                            base.qp, tok, acc, n)
        torch.cuda.synchronize()
        res.append((tok.tolist(), acc.tolist()))
    assert res[0] == res[1] and -7 not in res[0][0]
