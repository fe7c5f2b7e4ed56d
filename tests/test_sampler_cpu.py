"""The sampler oracle (oracle/ref_sample.py) against the known answers the reference's own unit tests hold
(src/sample.rs:213-270), its random-number generator, and the algebra the draws rest on."""
import numpy as np

from oracle import ref_sample as S

F = np.float32


def row(temp, k, p, rep, u1, u2, d, pres):
    return np.array([temp, k, p, rep, u1, u2, d, pres], dtype=F)


def test_no_top_k_reaches_the_whole_vocabulary():
    """src/sample.rs:217-229: a flat distribution reaches past any candidate cap; ties go to the lower index."""
    logits = np.zeros(5000, dtype=F)
    draw = lambda u, k: S.sample_row(logits, None, None, row(1, k, 1, 1, u, 0, -1, 0))[0]
    assert draw(0.9999, 0) == 4999
    assert draw(0.9999, 1024) < 1024
    assert draw(0.9999, 1024) == 1023  # equal values rank by index
    assert len(S.kept_dist(logits, None, None, row(1, 0, 1, 1, 0, 0, -1, 0))[1]) == 5000


def test_sampled_drafts_follow_p():
    """src/sample.rs:233-269 on a coarser grid of draws (the reference uses 400 x 400 per draft token): a draft d ~ q,
    accepted or resampled by sample_row_q, is distributed as the row's own p."""
    logits = np.array([((i * 37) % 11) * 0.4 - i * 0.02 for i in range(64)], dtype=F)
    r = row(0.9, 20, 0.9, 1, 0, 0, -1, 0)
    p, idx = S.kept_dist(logits, None, None, r)
    qlog = np.array([((i * 13) % 7) * 0.5 for i in range(64)], dtype=F)
    qp, qidx = S.kept_dist(qlog, None, None, row(1.2, 30, 1, 1, 0, 0, -1, 0))
    o = np.argsort(qidx)
    q_ids, q_p = qidx[o], qp[o]
    got = np.zeros(64)
    n = 40
    for d, qd in zip(qidx, qp):
        for a in range(n):
            for b in range(n):
                rr = r.copy()
                rr[4], rr[5], rr[6] = (a + 0.5) / n, (b + 0.5) / n, d
                t, _ = S.sample_row_q(logits, None, None, rr, q_ids, q_p)
                got[t] += float(qd) / (n * n)
    want = np.zeros(64)
    want[idx] = p
    tv = np.abs(got - want).sum() / 2
    # the grid's resolution: the distance falls as 1 / n (0.045 at n = 40, 0.014 at n = 120; the reference's bound of
    # 0.01 is for its n = 400)
    assert tv < 0.05, tv


def test_rng_is_xorshift64star():
    """src/sample.rs:71-85 by hand for the first draws of seed 7."""
    M = (1 << 64) - 1
    s = ((7 * 0x9E3779B97F4A7C15) & M) | 1
    g = S.Rng(7)
    for _ in range(5):
        s ^= s >> 12
        s ^= (s << 25) & M
        s ^= s >> 27
        want = ((s * 0x2545F4914F6CDD1D & M) >> 40) / float(1 << 24)
        got = float(g.next_f32())
        assert got == want and 0.0 <= got < 1.0


def test_penalties_and_greedy():
    logits = np.array([2.0, 1.9, -1.0, 0.5], dtype=F)
    seen = np.array([True, False, True, False])
    # repetition 2: 2.0 -> 1.0, -1.0 -> -2.0: the argmax moves to token 1
    assert S.sample_row(logits, seen, None, row(0, 0, 1, 2.0, 0, 0, -1, 0)) == (1, False)
    # presence 1.5 on token 0 only
    gen = np.array([True, False, False, False])
    vals, idx = S.ranked(logits, None, gen, row(1, 0, 1, 1, 0, 0, -1, 1.5), 0)
    assert idx.tolist() == [1, 0, 3, 2] and vals[0] == F(0.5)
    # a greedy row accepts its draft only when the draft is the argmax
    assert S.sample_row(logits, None, None, row(0, 0, 1, 1, 0, 0, 0, 0)) == (0, True)
    assert S.sample_row(logits, None, None, row(1, 1, 1, 1, 0, 0, 1, 0)) == (0, False)


def test_draft_accept_or_resample_follows_p():
    """With an argmax draft d: accepted with p(d), else drawn from p without d; over a grid of (u1, u2) the tokens are
    distributed as plain sampling (the design src/checks.rs:820-884 measures on the GPU)."""
    g = np.random.default_rng(3)
    logits = (g.standard_normal(200) * 2).astype(F)
    base = row(0.8, 20, 0.9, 1, 0, 0, -1, 0)
    p, idx = S.kept_dist(logits, None, None, base)
    d = int(idx[1])
    n = 60
    got = np.zeros(200)
    for a in range(n):
        for b in range(n):
            r = base.copy()
            r[4], r[5], r[6] = (a + 0.5) / n, (b + 0.5) / n, d
            t, acc = S.sample_row(logits, None, None, r)
            assert acc == (t == d)
            got[t] += 1.0 / (n * n)
    want = np.zeros(200)
    want[idx] = p
    assert np.abs(got - want).sum() / 2 < 0.02


def test_draft_draw_matches_kept_dist():
    g = np.random.default_rng(5)
    logits = (g.standard_normal(4096) * 3).astype(F)
    head_ids = g.permutation(100000)[:4096]
    seen = np.zeros(100000, dtype=bool)
    seen[head_ids[::7]] = True
    r = S.draft_row(0.9, 0, 0.95, 1.2, 0.0)
    r[4] = 0.37
    tok, qi, qp, margin = S.draft_draw(logits, seen, None, r, head_ids, want_margin=True)
    assert np.all(np.diff(qi) > 0) and tok in qi and abs(qp.sum() - 1) < 1e-5 and margin > 0
    # the same distribution from kept_dist over the columns
    p, idx = S.kept_dist(logits, seen[head_ids], None, r)
    assert sorted(head_ids[idx].tolist()) == qi.tolist()


def _words(tokens, vocab):
    w = np.zeros((vocab + 31) // 32, dtype=np.uint32)
    for t in tokens:
        w[t >> 5] |= np.uint32(1 << (t & 31))
    return w


def test_host_rows_of_the_library_match_the_oracle():
    """qb_host_sample_row (the rows the GPU kernel leaves to the host: top_k 0 or above 1024) against the oracle, token
    for token: both are float32 in the host definition's order, so no boundary allowance."""
    from qwenny_b200 import host
    g = np.random.default_rng(17)
    rng = S.Rng(3)
    vocab = 6000
    for trial in range(40):
        logits = (g.standard_normal(vocab) * 2.5).astype(F)
        logits[g.integers(0, vocab, 8)] += g.uniform(3, 8, 8).astype(F)
        seen_t, outs_t = g.integers(0, vocab, 80), g.integers(0, vocab, 30)
        step = list(g.integers(0, vocab, trial % 4))
        temp, k, p, rep, pres = [(1.0, 0, 0.95, 1.1, 0.0), (1.5, 0, 1.0, 1.0, 0.0), (0.7, 2000, 0.8, 1.2, 1.5),
                                 (0.9, 5, 0.5, 1.3, 0.0), (0.0, 0, 1.0, 1.3, 2.0)][trial % 5]
        top = int(np.argsort(-logits)[trial % 3])
        draft = None if trial % 3 == 0 else top
        r = S.params_row(temp, k, p, rep, pres, rng, draft=draft)
        seen = np.zeros(vocab, dtype=bool)
        gen = np.zeros(vocab, dtype=bool)
        seen[seen_t] = True
        gen[outs_t] = True
        seen[step] = True
        gen[step] = True
        want = S.sample_row(logits, seen, gen, r)
        got = host.sample_row(logits, _words(seen_t, vocab), _words(outs_t, vocab), step, r)
        assert got == want, (trial, got, want)
        if draft is not None and temp > 0:
            # the same row with its draft marked sampled from a stored q
            qp, qidx = S.kept_dist(np.roll(logits, 1), None, None, np.array([1.1, 40, 1, 1, 0, 0, -1, 0], dtype=F))
            qidx = np.concatenate([qidx, [draft]]) if draft not in qidx else qidx
            qp = np.concatenate([qp, [F(0.05)]]) if len(qp) < len(qidx) else qp
            o = np.argsort(qidx)
            r2 = r.copy()
            S.mark_sampled(r2)
            r3 = r.copy()
            want = S.sample_row_q(logits, seen, gen, r3, qidx[o], qp[o])
            got = host.sample_row(logits, _words(seen_t, vocab), _words(outs_t, vocab), step, r2, (qidx[o], qp[o]))
            assert got == want, (trial, got, want)
    # the reference's flat row (src/sample.rs:217-229)
    flat = np.zeros(5000, dtype=F)
    assert host.sample_row(flat, None, None, None, [1, 0, 1, 1, 0.9999, 0, -1, 0])[0] == 4999
    assert host.sample_row(flat, None, None, None, [1, 1024, 1, 1, 0.9999, 0, -1, 0])[0] == 1023
