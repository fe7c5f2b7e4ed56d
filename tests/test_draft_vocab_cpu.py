"""The draft head's bookkeeping (csrc/draft_vocab.h through qb_draft_vocab_*) against the known answers of the
reference's own unit tests (src/draft_vocab.rs:275-400, restated case by case), and against a plain-Python restatement
of its rules on random streams of committed tokens."""
import ctypes as C
import random
import struct

import numpy as np
import pytest

from qwenny_b200 import _lib

DECAY = 20000
PUBLISH = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_uint32), C.c_int, C.POINTER(C.c_int), C.c_int)


def u32(v):
    v = list(v)
    return (C.c_uint32 * max(1, len(v)))(*v), len(v)


class Rows:
    """A handle on the library's bookkeeping."""

    def __init__(self, vocab, ids, score=None, cap=64):
        self.l, self.h = _lib.lib(), C.c_void_p()
        a, n = u32(ids)
        s = None if score is None else (C.c_float * max(1, n))(*score)
        rc = self.l.qb_draft_vocab_create(vocab, a, s, n, cap, C.byref(self.h))
        if rc:
            raise ValueError(rc)

    def __del__(self):
        if getattr(self, "h", None):
            self.l.qb_draft_vocab_destroy(self.h)

    def take(self, toks):
        return self.learn(toks)

    def learn(self, toks, fail=0):
        got = []

        def publish(_, ids, n_ids, tiles, n_tiles):
            got.append((n_ids, [tiles[i] for i in range(n_tiles)]))
            return fail

        a, n = u32(toks)
        changed = C.c_int(-1)
        rc = self.l.qb_draft_vocab_learn(self.h, a, n, PUBLISH(publish), None, C.byref(changed))
        assert len(got) <= 1
        if rc:
            assert rc == fail and changed.value == 0
            return None
        tiles = got[0][1] if got else []
        assert changed.value == len(tiles) and tiles == sorted(set(tiles))
        self.published = got[0] if got else None
        return tiles

    def may_change(self, toks):
        a, n = u32(toks)
        return bool(self.l.qb_draft_vocab_may_change(self.h, a, n))

    def state(self):
        n = self.l.qb_draft_vocab_rows(self.h)
        ids, score = (C.c_uint32 * max(1, n))(), (C.c_float * max(1, n))()
        assert self.l.qb_draft_vocab_get(self.h, ids, score, n) == 0
        return list(ids)[:n], list(score)[:n]

    def row_of(self, t):
        return self.l.qb_draft_vocab_row_of(self.h, t)

    def waiting(self, t):
        return bool(self.l.qb_draft_vocab_waiting(self.h, t))

    def pending(self):
        return self.l.qb_draft_vocab_pending(self.h)

    def dirty(self):
        return bool(self.l.qb_draft_vocab_dirty(self.h))


def rows(cap):
    return Rows(1000, range(32), [0.0] * 32, cap)


# ---- the reference's unit tests, case by case

def test_new_tokens_wait_for_a_tile_then_append():
    r = rows(64)
    assert r.take(range(100, 115)) == []
    assert r.take([100, 5, 115]) == [2]  # 100 again waits once; 115 is the 16th: a third tile
    ids, score = r.state()
    assert len(ids) == 48 and r.row_of(115) == 47 and score[5] == 1.0


def test_full_head_replaces_the_coldest_rows():
    r = rows(32)
    r.take(range(16))
    # tokens 16..31 (score 0) give way, tokens 0..15 (score 1) stay
    assert r.take(range(200, 216)) == [1]
    ids, _ = r.state()
    assert all(r.row_of(t) == t for t in range(16))
    assert all(r.row_of(t) == -1 for t in range(16, 32))
    assert all(r.row_of(t) != -1 and ids[r.row_of(t)] == t for t in range(200, 216))


def test_hot_rows_are_kept_and_decay():
    r = rows(32)
    r.take(range(32))
    assert r.take(range(200, 216)) == []  # every row in use: the new ones get none
    assert r.pending() == 0 and all(r.row_of(t) == -1 and not r.waiting(t) for t in range(200, 216))
    assert r.take([5000] * (DECAY - 1 - 48)) == []  # tokens beyond the vocabulary only count towards the halving
    r.take([0])  # the halving: rows 1..31 fall below 1
    ids, score = r.state()
    assert score[0] == 1.0 and all(s == 0.5 for s in score[1:])
    assert r.take(range(200, 216)) != []
    ids, _ = r.state()
    assert r.row_of(0) == 0
    assert sum(r.row_of(t) != -1 for t in range(32)) == 16
    assert all(ids[r.row_of(t)] == t for t in range(200, 216))


def test_may_change_exactly_when_take_can():
    # repeats count once; a token waiting already is no new one; tokens with rows and beyond the vocabulary are none
    r = rows(64)
    assert not r.may_change(list(range(100, 115)) * 2 + list(range(32)) + [5000])
    assert r.may_change(range(100, 116))
    assert r.take(range(100, 115)) == []
    assert not r.may_change(range(100, 115))
    assert r.may_change([115])
    assert r.take([115]) != []


def test_learn_publishes_changed_tiles_and_marks_only_them_dirty():
    a = rows(64)
    assert a.learn([1, 2, 3]) == [] and a.published is None  # counting alone publishes nothing, leaves nothing to save
    assert not a.dirty()
    assert a.learn(range(100, 116)) == [2] and a.published == (48, [2])
    assert a.dirty()
    assert a.state()[0][32:48] == list(range(100, 116))
    assert a.l.qb_draft_vocab_saved(a.h) == 0 and not a.dirty()


def test_a_failed_publish_rolls_the_rows_back():
    a = rows(64)
    a.learn([1])
    before = a.state()
    new = list(range(100, 116))
    assert a.learn(new, fail=1234) is None
    assert not a.dirty() and a.state() == before
    assert all(a.row_of(t) == -1 and not a.waiting(t) for t in new)
    assert a.learn(new) == [2] and len(a.state()[0]) == 48  # the same tokens again: nothing was lost


def pt_file(ids):
    """A zip archive as PyTorch writes one tensor: a stored entry archive/data/0 with the ids as int64."""
    name, data = b"archive/data/0", b"".join(struct.pack("<q", i) for i in ids)
    local = bytearray(30)
    local[:4] = b"PK\x03\x04"
    local[26:28] = struct.pack("<H", len(name))
    central = bytearray(46)
    central[:4] = b"PK\x01\x02"
    central[20:24] = struct.pack("<I", len(data))
    central[28:30] = struct.pack("<H", len(name))
    end = bytearray(22)
    end[:4] = b"PK\x05\x06"
    end[10:12] = struct.pack("<H", 1)
    end[16:20] = struct.pack("<I", len(local) + len(name) + len(data))
    return bytes(local) + name + data + bytes(central) + name + bytes(end)


def draft_ids(b, vocab, cap=64):
    ids, n = (C.c_uint32 * cap)(), C.c_int(0)
    buf = (C.c_uint8 * max(1, len(b))).from_buffer_copy(b if b else b"\0")
    rc = _lib.lib().qb_draft_ids_pt(buf, len(b), vocab, ids, cap, C.byref(n))
    return rc, list(ids)[:n.value]


def test_draft_ids_drop_repeats_and_tell_the_errors_apart():
    assert draft_ids(pt_file([7, 3, 7, 9, 3]), 100) == (0, [7, 3, 9])
    assert draft_ids(pt_file([7, 100]), 100)[0] == 4       # beyond the vocabulary
    assert draft_ids(pt_file([-1]), 100)[0] == 4
    assert draft_ids(b"not a zip" * 4, 100)[0] == 1        # not a zip archive
    assert draft_ids(b"PK", 100)[0] == 1
    good = pt_file([1, 2, 3])
    past = bytearray(good)
    past[-6:-2] = struct.pack("<I", len(good) + 100)       # a central directory beyond the end of the file
    assert draft_ids(bytes(past), 100)[0] == 1
    cd = len(good) - 22 - 14 - 46
    longer = bytearray(good)
    longer[cd + 20:cd + 24] = struct.pack("<I", 4096)      # an entry longer than the file: truncated
    assert draft_ids(bytes(longer), 100)[0] == 1
    packed = bytearray(good)
    packed[cd + 10:cd + 12] = struct.pack("<H", 8)         # a compressed entry
    assert draft_ids(bytes(packed), 100)[0] == 3
    other = pt_file([1, 2]).replace(b"archive/data/0", b"archive/data/1")
    assert draft_ids(other, 100)[0] == 2                   # no tensor data
    assert draft_ids(pt_file(range(20)), 100, cap=8)[0] == 1003


# ---- Adaptive::load and Rows::new

def load(vocab, saved, score, seed):
    l, h = _lib.lib(), C.c_void_p()
    a, n = u32(saved)
    s = (C.c_float * max(1, n))(*score)
    b, m = u32(seed)
    rc = l.qb_draft_vocab_load(vocab, a if n else None, s if n else None, n, b, m, C.byref(h))
    if rc:
        return rc, None, None
    k = l.qb_draft_vocab_rows(h)
    ids, sc = (C.c_uint32 * k)(), (C.c_float * k)()
    l.qb_draft_vocab_get(h, ids, sc, k)
    l.qb_draft_vocab_destroy(h)
    return 0, list(ids), list(sc)


def test_load_takes_the_saved_rows_then_the_seed_in_whole_tiles():
    saved, score = list(range(500, 516)), [float(i) for i in range(16)]
    seed = list(range(40)) + [505, 3]                      # repeats and saved tokens are no new ones
    rc, ids, sc = load(1000, saved, score, seed)
    assert rc == 0 and ids == saved + list(range(32)) and sc == score + [0.0] * 32  # 56 -> 48: whole tiles
    # saved rows that do not fit the vocabulary (or repeat) are dropped as a whole
    assert load(510, saved, score, seed) == (0, list(range(32)), [0.0] * 32)
    assert load(1000, saved[:15] + [500], score, seed)[1] == list(range(32))
    assert load(1000, [], [], list(range(15)))[0] == 1000  # less than one tile
    assert load(1000, [], [], list(range(15)) + [1000])[0] == 1000  # a seed token beyond the vocabulary


def test_rows_new_refusals():
    for ids, cap in ((range(15), 64), (range(32), 16), (range(16), 40), ([1] * 16, 64), (list(range(15)) + [1000], 64)):
        with pytest.raises(ValueError):
            Rows(1000, ids, None, cap)
    assert Rows(1000, range(16), None, 64).state()[1] == [0.0] * 16  # no scores: none yet


# ---- random streams against the rules written out in Python

class Model:
    def __init__(self, vocab, ids, cap):
        self.ids, self.score, self.row_of = list(ids), [0.0] * len(ids), {t: r for r, t in enumerate(ids)}
        self.vocab, self.cap, self.pending, self.since = vocab, cap, [], 0

    def take(self, toks):
        for t in toks:
            if t >= self.vocab:
                continue
            if t in self.row_of:
                self.score[self.row_of[t]] += 1.0
            elif t not in self.pending:
                self.pending.append(t)
        self.since += len(toks)
        if self.since >= DECAY:
            self.since = 0
            self.score = [float(np.float32(s) * np.float32(0.5)) for s in self.score]
        n = len(self.pending) // 16 * 16
        if n == 0:
            return []
        new, self.pending = self.pending[:n], self.pending[n:]
        room = min(self.cap - len(self.ids), n)
        tiles = list(range(len(self.ids) // 16, (len(self.ids) + room) // 16))
        for t in new[:room]:
            self.row_of[t] = len(self.ids)
            self.ids.append(t)
            self.score.append(1.0)
        rest = new[room:]
        cold = sorted((r for r in range(len(self.ids)) if self.score[r] < 1.0), key=lambda r: (self.score[r], r))
        for r, t in zip(cold, rest):
            del self.row_of[self.ids[r]]
            self.ids[r], self.score[r], self.row_of[t] = t, 1.0, r
            tiles.append(r // 16)
        return sorted(set(tiles))


@pytest.mark.parametrize("seed", range(4))
def test_random_streams(seed):
    rng = random.Random(seed)
    vocab, cap = 3000, 160
    r, m = Rows(vocab, range(64), None, cap), Model(vocab, range(64), cap)
    hot = rng.sample(range(vocab), 200)
    for step in range(400):
        k = rng.choice([1, 1, 5, 40, 700, 3000])
        toks = [rng.choice(hot) if rng.random() < 0.7 else rng.randrange(vocab + 50) for _ in range(k)]
        assert r.take(toks) == m.take(toks), step
        ids, score = r.state()
        assert ids == m.ids and score == m.score, step
        assert r.pending() == len(m.pending)
    assert len(m.ids) == cap and m.since != 0
