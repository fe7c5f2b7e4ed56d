"""CPU restatement of the reference's sampler (src/sample.rs), in numpy float32.

TEST INFRASTRUCTURE ONLY: the parity tests put the CUDA sampler's tokens next to these, draw for draw, the way the
reference's own `samplecheck` does with its host functions (src/checks.rs:685-888). The reference's host code is the
definition the GPU kernels are checked against there, so it is the oracle here; every function cites the lines it
follows. Parity pinned: the unit tests of src/sample.rs:213-270 (tests/test_sampler_cpu.py), and on a GPU the
reference's own compiled kernels `sample_rows` / `draft_sample` (tests/test_sampler_gpu.py).

Arithmetic is float32 in the host's order: a sequential prefix sum, exp of (v - vmax) / temperature. Every function
also reports the `margin` of its decision: the smallest relative distance between a uniform draw and the boundary it
was compared with. A kernel that sums in another order (the GPU's scans are trees) can differ from the host only on
draws whose margin is of the order of the rounding error, which the tests name explicitly.
"""
from __future__ import annotations

import numpy as np

F = np.float32
QD, QCAP = 16, 1024  # kernels/sampling.cuh:73-74


class Rng:
    """xorshift64* (src/sample.rs:71-85)."""

    M = (1 << 64) - 1

    def __init__(self, seed: int):
        self.s = ((seed * 0x9E3779B97F4A7C15) & self.M) | 1

    def next_f32(self) -> np.float32:
        s = self.s
        s ^= s >> 12
        s ^= (s << 25) & self.M
        s ^= s >> 27
        self.s = s
        return F(F((s * 0x2545F4914F6CDD1D & self.M) >> 40) / F(1 << 24))


def params_row(temperature, top_k, top_p, repetition_penalty, presence_penalty, rng: Rng, draft=None):
    """Params::row (src/sample.rs:26-32)."""
    sampling = temperature > 0.0 and top_k != 1
    u1 = rng.next_f32() if sampling else F(0)
    u2 = rng.next_f32() if sampling and draft is not None else F(0)
    d = -1.0 if draft is None else float(draft)
    return np.array([temperature, top_k, top_p, repetition_penalty, u1, u2, d, presence_penalty], dtype=F)


def draft_row(temperature, top_k, top_p, repetition_penalty, presence_penalty, presence=True):
    """Params::draft_row (src/sample.rs:44-56)."""
    k = 1024 if top_k == 0 else min(top_k, 1024)
    return np.array([temperature, k, top_p, repetition_penalty, 0, 0, -1, presence_penalty if presence else 0],
                    dtype=F)


def argmax_draft_row(t):
    """src/sample.rs:60-62."""
    return np.array([1, 1, 1, 1, 0.5, t, -1, 0], dtype=F)


def mark_sampled(row):
    """src/sample.rs:65-69."""
    if row[6] >= 0:
        row[6] = -row[6] - 2.0


def ranked(logits, seen, generated, row, k):
    """src/sample.rs:88-115. seen / generated: boolean arrays over the vocabulary (or None)."""
    rep, pres = F(row[3]), F(row[7])
    vals = np.asarray(logits, dtype=F).copy()
    if rep != 1.0 and seen is not None:
        s = np.asarray(seen, dtype=bool)
        vals[s] = np.where(vals[s] > 0, vals[s] / rep, vals[s] * rep)
    if pres != 0.0 and generated is not None:
        g = np.asarray(generated, dtype=bool)
        vals[g] = vals[g] - pres
    n = len(vals)
    k = min(k, n) if k > 0 else n
    # descending by value (total order of the bits, as total_cmp), ties to the lower index
    u = vals.view(np.uint32).astype(np.int64)
    key = np.where(u & 0x80000000, (~u) & 0xFFFFFFFF, u | 0x80000000)
    if k < n:
        part = np.argpartition(-key, k - 1)[:k]
        kth = key[part].min()
        above = np.nonzero(key > kth)[0]
        equal = np.nonzero(key == kth)[0][: k - len(above)]
        idx = np.concatenate([above, equal])
    else:
        idx = np.arange(n)
    order = np.lexsort((idx, -key[idx]))
    return vals, idx[order].astype(np.int64)


def kept(vals, idx, temp, top_p):
    """src/sample.rs:119-135."""
    vmax = vals[idx[0]]
    p = np.exp(((vals[idx] - vmax) / F(temp)).astype(F)).astype(F)
    cum = np.cumsum(p, dtype=F)
    total = cum[-1]
    keep = len(idx)
    if top_p < 1.0:
        hit = np.nonzero((cum / total).astype(F) >= F(top_p))[0]
        if len(hit):
            keep = int(hit[0]) + 1
    return p, cum, keep


def _rel(a, b):
    return abs(float(a) - float(b)) / max(abs(float(b)), 1e-30)


def sample_row(logits, seen, generated, row, want_margin=False):
    """src/sample.rs:141-172: (token, draft accepted)."""
    temp, top_k, top_p, u1, u2 = F(row[0]), int(row[1]), F(row[2]), F(row[4]), F(row[5])
    draft = int(row[6]) if row[6] >= 0 else None
    greedy = temp <= 0 or top_k == 1
    vals, idx = ranked(logits, seen, generated, row, 1 if greedy else top_k)
    if greedy:
        out = (int(idx[0]), draft == int(idx[0]))
        return out + (np.inf,) if want_margin else out
    p, cum, keep = kept(vals, idx, temp, top_p)
    margin = np.inf
    if top_p < 1.0:
        total = cum[-1]
        for i in (keep - 2, keep - 1):
            if i >= 0:
                margin = min(margin, _rel(cum[i] / total, top_p))
    mass = cum[keep - 1]
    at_d = None
    if draft is not None:
        w = np.nonzero(idx[:keep] == draft)[0]
        at_d = int(w[0]) if len(w) else None
    pd = F(p[at_d] / mass) if at_d is not None else F(0)
    if draft is not None:
        if pd > 0:
            margin = min(margin, _rel(u1, pd))
        if u1 < pd:
            out = (draft, True)
            return out + (margin,) if want_margin else out
    target = F(u2 * F(mass - F(pd * mass))) if draft is not None else F(u1 * mass)
    sub = F(pd * mass)
    r = None
    for i in range(keep):
        c = cum[i] - (sub if (at_d is not None and i >= at_d) else F(0))
        if i != at_d:
            margin = min(margin, _rel(c, target))
            if r is None and c >= target:
                r = i
    if r is None:
        r = keep - 1
    if at_d is not None and r == at_d:
        r = r + 1 if r + 1 < keep else max(r - 1, 0)
    out = (int(idx[r]), False)
    return out + (margin,) if want_margin else out


def kept_dist(logits, seen, generated, row):
    """src/sample.rs:203-211: probabilities and tokens of the kept set."""
    vals, idx = ranked(logits, seen, generated, row, int(row[1]))
    p, cum, keep = kept(vals, idx, F(row[0]), F(row[2]))
    mass = cum[keep - 1]
    return (p[:keep] / mass).astype(F), idx[:keep]


def sample_row_q(logits, seen, generated, row, q_ids, q_p, want_margin=False):
    """src/sample.rs:177-200: a draft drawn from q (ascending ids q_ids, probabilities q_p)."""
    p, idx = kept_dist(logits, seen, generated, row)
    d = int(row[6])
    q_ids = np.asarray(q_ids, dtype=np.int64)
    q_p = np.asarray(q_p, dtype=F)

    def qof(t):
        i = np.searchsorted(q_ids, t)
        hit = (i < len(q_ids)) & (q_ids[np.minimum(i, len(q_ids) - 1)] == t)
        return np.where(hit, q_p[np.minimum(i, len(q_ids) - 1)], F(0)).astype(F)

    w = np.nonzero(idx == d)[0]
    pd = p[w[0]] if len(w) else F(0)
    lhs = F(F(row[4]) * F(qof(np.array([d]))[0]))
    margin = _rel(lhs, pd) if pd > 0 else np.inf
    if lhs < pd:
        out = (d, True)
        return out + (margin,) if want_margin else out
    r = np.maximum(p - qof(idx), F(0)).astype(F)
    cum = np.cumsum(r, dtype=F)
    total = cum[-1] if len(cum) else F(0)
    if total <= 0:
        out = (int(idx[0]), False)
        return out + (margin,) if want_margin else out
    target = F(F(row[5]) * total)
    live = r > 0
    for i in np.nonzero(live)[0]:
        margin = min(margin, _rel(cum[i], target))
    hit = np.nonzero(live & (cum >= target))[0]
    at = int(hit[0]) if len(hit) else int(np.nonzero(live)[0][-1])
    out = (int(idx[at]), False)
    return out + (margin,) if want_margin else out


def draft_draw(logits, seen, generated, row, head_ids=None, want_margin=False):
    """The draw of draft_sample (kernels/sampling.cuh:298-352) stated with the host's functions: the row's kept
    distribution over the draft head's columns (token head_ids[i] for column i), a draw with u = row[4]: the first kept
    token whose prefix reaches u * mass. Returns (token, q ids ascending, q probabilities[, margin])."""
    n = len(logits)
    ids = np.arange(n) if head_ids is None else np.asarray(head_ids, dtype=np.int64)
    s = None if seen is None else np.asarray(seen, dtype=bool)[ids]
    g = None if generated is None else np.asarray(generated, dtype=bool)[ids]
    top_k = int(row[1])
    r2 = np.array(row, dtype=F)
    r2[1] = min(min(top_k, n) if top_k > 0 else 1024, QCAP)
    vals, idx = ranked(logits, s, g, r2, int(r2[1]))
    p, cum, keep = kept(vals, idx, F(r2[0]), F(r2[2]))
    mass = cum[keep - 1]
    target = F(F(row[4]) * mass)
    hit = np.nonzero(cum[:keep] >= target)[0]
    at = int(hit[0]) if len(hit) else keep - 1
    margin = min(_rel(c, target) for c in cum[:keep])
    toks = ids[idx[:keep]]
    prob = (p[:keep] / mass).astype(F)
    o = np.argsort(toks, kind="stable")
    out = (int(toks[at]), toks[o], prob[o])
    return out + (margin,) if want_margin else out
