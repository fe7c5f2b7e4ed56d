"""Host-side mirror of the reference's loader functions for this path (src/cuda/core.rs): numpy in, numpy out, the
work done by the library's C++ packers."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib

QG = 128


def _np(a):
    return a.ctypes.data_as(C.c_void_p)


def row_order(rows: int, silu: bool) -> np.ndarray:
    out = np.empty(rows, dtype=np.int32)
    check(lib().qb_row_order(rows, int(silu), _np(out)), "qb_row_order")
    return out


def quant_words(codes: np.ndarray) -> np.ndarray:
    """uint8 codes [rows][cols] (q + 8) -> the stored form u32 [rows][cols/8], column c at bits (c % 8) * 4."""
    rows, cols = codes.shape
    c = codes.reshape(rows, cols // 8, 8).astype(np.uint32)
    w = np.zeros((rows, cols // 8), dtype=np.uint32)
    for i in range(8):
        w |= c[:, :, i] << np.uint32(4 * i)
    return w


def pack_marlin(codes: np.ndarray, scales: np.ndarray, silu: bool = False, order: np.ndarray | None = None,
                group: int = QG, zeros: np.ndarray | None = None):
    """codes uint8 [rows][cols] (q + 8), scales f32 [rows][cols/group] -> (words uint32 [cols/16][2n],
    scales float16 [cols/128][n]) as Mat::marlin does (src/cuda/core.rs:160-164). With zeros (uint8
    [rows][cols/group], w = (q - z) * scale) the scales are followed by the table (8 - z) * scale: [2 cols/128][n]."""
    rows, cols = codes.shape
    if order is None:
        order = row_order(rows, silu)
    order = np.ascontiguousarray(order, dtype=np.int32)
    n = len(order)
    q = np.ascontiguousarray(quant_words(codes))
    sc = np.ascontiguousarray(scales, dtype=np.float32)
    words = np.empty((cols // 16, 2 * n), dtype=np.uint32)
    if zeros is not None:
        z = np.ascontiguousarray(zeros, dtype=np.uint8)
        s16 = np.empty((2 * (cols // 128), n), dtype=np.uint16)
        check(lib().qb_pack_marlin_z(_np(q), _np(sc), _np(z), rows, cols, group, _np(order), n, _np(words), _np(s16)),
              "qb_pack_marlin_z")
        return words, s16.view(np.float16)
    s16 = np.empty((cols // 128, n), dtype=np.uint16)
    check(lib().qb_pack_marlin(_np(q), _np(sc), rows, cols, group, _np(order), n, _np(words), _np(s16)),
          "qb_pack_marlin")
    return words, s16.view(np.float16)


def marlin_block(codes: np.ndarray, scales: np.ndarray, rows16, zeros: np.ndarray | None = None, zero_points: bool = False,
                 group: int = QG):
    """The host half of Gemm::put_block (src/cuda/core.rs:614-656): the 16 stored rows `rows16` of a quantized matrix
    (codes uint8 [rows][cols] = q + 8, scales f32 [rows][cols/group], zeros uint8 or None) -> (words uint32
    [cols/16][32], scales float16 [tables * cols/128][16])."""
    rows, cols = codes.shape
    q = np.ascontiguousarray(quant_words(codes))
    sc = np.ascontiguousarray(scales, dtype=np.float32)
    r16 = np.ascontiguousarray(rows16, dtype=np.int32)
    assert r16.shape == (16,)
    z = None if zeros is None else np.ascontiguousarray(zeros, dtype=np.uint8)
    tables = 2 if zero_points else 1
    words = np.empty((cols // 16, 32), dtype=np.uint32)
    s16 = np.empty((tables * (cols // 128), 16), dtype=np.uint16)
    check(lib().qb_marlin_block(_np(q), _np(sc), C.c_void_p(0) if z is None else _np(z), int(zero_points), rows, cols,
                                group, _np(r16), _np(words), _np(s16)), "qb_marlin_block")
    return words, s16.view(np.float16)


def pack_f16(w: np.ndarray, order: np.ndarray | None = None) -> np.ndarray:
    """f32 [rows][cols] -> float16 [rows/16][cols/16][32][8] (mma A-fragment order)."""
    rows, cols = w.shape
    w = np.ascontiguousarray(w, dtype=np.float32)
    n = rows if order is None else len(order)
    out = np.empty((n // 16, cols // 16, 32, 8), dtype=np.uint16)
    o = None if order is None else np.ascontiguousarray(order, dtype=np.int32)
    check(lib().qb_pack_f16(_np(w), rows, cols, C.c_void_p(0) if o is None else _np(o), n, _np(out)), "qb_pack_f16")
    return out.view(np.float16)


def pack_i8(w: np.ndarray, order: np.ndarray | None = None) -> tuple[np.ndarray, np.ndarray]:
    """f32 [rows][cols] -> (uint8 [rows/16][16 * cols] codes in fragment order, f32 [rows/16][cols/128][16] scales)."""
    rows, cols = w.shape
    w = np.ascontiguousarray(w, dtype=np.float32)
    n = rows if order is None else len(order)
    out = np.empty((n // 16, 16 * cols), dtype=np.uint8)
    sc = np.empty((n // 16, cols // 128, 16), dtype=np.float32)
    o = None if order is None else np.ascontiguousarray(order, dtype=np.int32)
    check(lib().qb_pack_i8(_np(w), rows, cols, C.c_void_p(0) if o is None else _np(o), n, _np(out), _np(sc)),
          "qb_pack_i8")
    return out, sc


def split_for(tiles: int, cols: int, bits: int, kd: int) -> int:
    return lib().qb_split_for(tiles, cols, bits, kd)


def sample_row(logits: np.ndarray, seen_words, outs_words, step, row, q=None) -> tuple[int, bool]:
    """sample::sample_row / sample_row_q (src/sample.rs:141-200) as Step::sample_on_host calls them: the sampler rows
    the GPU kernel leaves to the host. seen_words / outs_words: the slot's bitsets (uint32 words) or None; step: the
    step's tokens of the row's sequence after its first; q: (ids ascending, probabilities) of a sampled draft."""
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    sw = None if seen_words is None else np.ascontiguousarray(seen_words, dtype=np.uint32)
    ow = None if outs_words is None else np.ascontiguousarray(outs_words, dtype=np.uint32)
    st = np.ascontiguousarray(step if step is not None else [], dtype=np.int32)
    r = np.ascontiguousarray(row, dtype=np.float32)
    qi = qp = None
    if q is not None:
        qi, qp = np.ascontiguousarray(q[0], dtype=np.int32), np.ascontiguousarray(q[1], dtype=np.float32)
    tok, acc = C.c_int(0), C.c_int(0)
    check(lib().qb_host_sample_row(_np(lg), len(lg), _np(sw) if sw is not None else None,
                                   _np(ow) if ow is not None else None, _np(st) if len(st) else None, len(st), _np(r),
                                   _np(qi) if qi is not None else None, _np(qp) if qp is not None else None,
                                   0 if qi is None else len(qi), C.byref(tok), C.byref(acc)), "qb_host_sample_row")
    return tok.value, bool(acc.value)


class DraftVocab:
    """Which token has which row of a draft head (Rows / Adaptive, src/draft_vocab.rs:22-201): a handle on the library's
    bookkeeping. ids: the token of each row (a multiple of 16), cap: the head's rows at most."""

    def __init__(self, vocab: int, ids, score=None, cap: int = 65536):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        sc = None if score is None else np.ascontiguousarray(score, dtype=np.float32)
        self.h = C.c_void_p()
        check(lib().qb_draft_vocab_create(int(vocab), _np(ids), C.c_void_p(0) if sc is None else _np(sc), len(ids), int(cap),
                                          C.byref(self.h)), "qb_draft_vocab_create")

    def close(self):
        if getattr(self, "h", None):
            lib().qb_draft_vocab_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def ids(self) -> np.ndarray:
        n = lib().qb_draft_vocab_rows(self.h)
        out = np.empty(max(1, n), dtype=np.uint32)
        check(lib().qb_draft_vocab_get(self.h, _np(out), C.c_void_p(0), n), "qb_draft_vocab_get")
        return out[:n]

    def scores(self) -> np.ndarray:
        n = lib().qb_draft_vocab_rows(self.h)
        out = np.empty(max(1, n), dtype=np.float32)
        check(lib().qb_draft_vocab_get(self.h, C.c_void_p(0), _np(out), n), "qb_draft_vocab_get")
        return out[:n]

    def row_of(self, token: int) -> int:
        return lib().qb_draft_vocab_row_of(self.h, int(token))
