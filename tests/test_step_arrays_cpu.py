"""The host arrays of a step (qb_step_arrays = what qb_model_upload copies to the device) against the oracle's
restatement of the reference's Step::upload (src/cuda/core.rs:835-926), without a device: random mixed steps (decode
tokens, drafts, prompt chunks), the cut of short segments at multiples of 2048 positions, the marks, and every refusal."""
import ctypes as C
import random

import numpy as np
import pytest

from oracle import ref_ops as R
from qwenny_b200 import _lib
from qwenny_b200.model import QbTok

NAMES = ["ids", "tok_slot", "tok_pos", "seg_start", "seg_len", "seg_slot", "seg_pos0", "dtok", "dseg", "dkeys", "ptile",
         "out_rows", "mark", "mark_at", "mtp_rows", "row_first"]
SHAPE = ["n", "n_out", "segs", "ndec", "ntile", "ndseg", "dmax", "max_seg", "dec_max_pos", "tile_max_pos"]
SLOTS, CTX, VOCAB = 24, 40000, 248320


def arrays(toks, out, marks=None, slots=SLOTS, ctx=CTX, vocab=VOCAB, marks_at=None):
    l = _lib.lib()
    arr = (QbTok * max(1, len(toks)))()
    for i, (tid, slot, pos) in enumerate(toks):
        arr[i].id, arr[i].slot, arr[i].pos = tid, slot, pos
    o = (C.c_int * max(1, len(out)))(*out)
    h = (C.c_int * l.qb_step_ints())()
    off, shape = (C.c_longlong * 16)(), (C.c_int * 10)()
    mk = ma = None
    if marks is not None:
        flat = [t for seg in marks for t in seg]
        at = [0]
        for seg in marks:
            at.append(at[-1] + len(seg))
        at = marks_at if marks_at is not None else at
        mk, ma = (C.c_uint32 * max(1, len(flat)))(*flat), (C.c_int * len(at))(*at)
    rc = l.qb_step_arrays(arr, len(toks), o, len(out), mk, ma, slots, ctx, vocab, h, off, shape)
    return rc, np.ctypeslib.as_array(h).copy(), list(off), dict(zip(SHAPE, shape))


def same_as_the_oracle(toks, out, marks=None):
    rc, h, off, shape = arrays(toks, out, marks)
    assert rc == 0
    st = R.build_step(toks, out, marks=marks)
    for k in SHAPE:
        assert shape[k] == st[k], k
    for i, name in enumerate(NAMES):
        if name == "mtp_rows":
            continue
        want = st[name]
        got = h[off[i]:off[i] + len(want)]
        assert np.array_equal(got, want), name
    assert off == sorted(off) and all(o % 4 == 0 for o in off)  # 16-byte aligned arrays, in the documented order
    return st


def random_step(rng):
    slots = rng.sample(range(SLOTS), rng.randrange(1, 9))
    toks, budget = [], 2048
    for s in slots:
        kind = rng.random()
        ln = 1 if kind < 0.35 else rng.randrange(2, 9) if kind < 0.75 else rng.randrange(9, 400)
        ln = min(ln, budget)
        if ln == 0:
            break
        budget -= ln
        # often right below a multiple of 2048, where short segments are cut
        p0 = rng.choice([0, 2048 * rng.randrange(1, 15) - rng.randrange(0, 9), rng.randrange(0, CTX - 500)])
        toks += [(rng.randrange(VOCAB), s, max(0, p0) + i) for i in range(ln)]
    n_out = rng.randrange(0, min(64, len(toks)) + 1)
    out = sorted(rng.sample(range(len(toks)), n_out))
    return toks, out


@pytest.mark.parametrize("seed", range(8))
def test_random_steps(seed):
    rng = random.Random(seed)
    for _ in range(60):
        toks, out = random_step(rng)
        st = same_as_the_oracle(toks, out)
        if rng.random() < 0.5:
            marks = [[rng.randrange(VOCAB) for _ in range(rng.randrange(0, 12))] for _ in range(st["segs"])]
            same_as_the_oracle(toks, out, marks)


def test_the_verify_step_of_the_headline_config():
    toks = [(11 + i, 0, 32000 + i) for i in range(5)]
    st = same_as_the_oracle(toks, list(range(5)), marks=[[11]])
    assert (st["ndec"], st["ndseg"], st["dmax"], st["ntile"], st["dec_max_pos"]) == (5, 1, 5, 0, 32004)
    assert list(st["mark"]) == [11] and list(st["dkeys"]) == [32005] * 5


def test_a_short_segment_is_cut_where_the_position_crosses_2048():
    toks = [(1, 3, 2046 + i) for i in range(5)]
    st = same_as_the_oracle(toks, [4])
    assert list(st["dseg"]) == [0, 2, 2, 3] and list(st["dkeys"]) == [2048, 2048, 2051, 2051, 2051]


def test_more_than_64_decode_tokens_go_on_as_prompt_tiles():
    toks = [(1, s, 100 + i) for s in range(10) for i in range(8)]
    st = same_as_the_oracle(toks, [0])
    assert st["ndec"] == 64 and st["ntile"] == 2 and st["max_seg"] == 8


def test_largest_step_and_most_marks():
    toks = [(i % VOCAB, 0, i) for i in range(2048)]
    st = same_as_the_oracle(toks, list(range(2048 - 64, 2048)), marks=[list(range(2560))])
    assert st["ntile"] == 205 and st["tile_max_pos"] == 2047 and len(st["mark"]) == 2560


def test_refusals():
    ok = [(1, 0, 5), (2, 0, 6), (3, 1, 0)]
    assert arrays(ok, [0, 2])[0] == 0
    assert arrays([], [])[0] == 1000                                          # no tokens
    assert arrays([(1, 0, i) for i in range(2049)], [])[0] == 1000            # more than 2048 tokens
    assert arrays([(1, 0, i) for i in range(100)], list(range(65)))[0] == 1000  # more than 64 logit rows
    assert arrays(ok, [3])[0] == 1000 and arrays(ok, [-1])[0] == 1000         # a logit row that is no token of the step
    assert arrays([(1, SLOTS, 0)], [])[0] == 1000                             # slot beyond the model's
    assert arrays([(1, 0, CTX)], [])[0] == 1000                               # position beyond the context
    assert arrays([(VOCAB, 0, 0)], [])[0] == 1000                             # token beyond the vocabulary
    assert arrays([(1, 0, 5), (2, 0, 7)], [])[0] == 1000                      # positions of a slot not consecutive
    assert arrays([(1, 0, 5), (2, 1, 0), (3, 0, 6)], [])[0] == 1000           # a slot in two segments
    assert arrays(ok, [], marks=[[1], [VOCAB]])[0] == 1000                    # a mark beyond the vocabulary
    assert arrays(ok, [], marks=[list(range(2561)), []])[0] == 1000           # more marks than the step holds
    assert arrays(ok, [], marks=[[1], [2]], marks_at=[0, 2, 1])[0] == 1000    # mark ranges that run backwards
    assert arrays(ok, [], marks=[[1, 2, 3], []])[0] == 0
