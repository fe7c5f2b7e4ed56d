"""CPU tests of the weight layouts: the library's host packers against the oracle's numpy restatement, and the
layout algebra the kernels rely on."""
import numpy as np
import pytest
import torch

from oracle import ref_ops as R
from qwenny_b200 import host, synth


@pytest.mark.parametrize("silu", [False, True])
def test_row_order(silu):
    o = host.row_order(512, silu)
    assert np.array_equal(o, R.row_order(512, silu))
    assert sorted(o.tolist()) == list(range(512))
    if silu:  # block p holds gate rows 8p..8p+7 then up rows 256+8p..
        assert o[:16].tolist() == list(range(8)) + list(range(256, 264))


@pytest.mark.parametrize("rows,cols,silu", [(256, 256, False), (512, 384, True), (256, 1024, False)])
def test_pack_marlin_matches_oracle(rows, cols, silu):
    g = synth.gen(1)
    codes, sc = synth.int4_matrix(rows, cols, g)
    words, s16 = host.pack_marlin(codes, sc, silu=silu)
    ow, os_ = R.pack_marlin(codes, sc.astype(np.float16), R.row_order(rows, silu))
    assert np.array_equal(words, ow)
    assert np.array_equal(s16.view(np.uint16), os_.view(np.uint16))


def test_marlin_word_is_an_mma_a_fragment():
    """The property the GEMV kernel is built on: nibble x of lane (g, t)'s word is output g + 8*((x>>1)&1), column
    2t + 8*(x&1) + (x>>2) of its 16 x 16 block, i.e. registers a0..a3 of mma.m16n8k16's A operand are nibble pairs
    (0,4), (2,6), (1,5), (3,7)."""
    codes = (np.arange(64 * 128).reshape(64, 128) * 7 % 16).astype(np.uint8)
    sc = np.ones((64, 1), dtype=np.float32)
    words, _ = host.pack_marlin(codes, sc)
    rows, cols = R.frag_map()  # a0..a7 (row, col) per lane
    pairs = [(0, 4), (2, 6), (1, 5), (3, 7)]  # register r = elements (2r, 2r+1) of frag_map
    for k16 in range(8):
        for c64 in range(1):
            for lane in range(32):
                for blk in range(4):
                    w = int(words[k16, (c64 * 32 + lane) * 4 + blk])
                    for reg, (xa, xb) in enumerate(pairs):
                        for e, x in enumerate((xa, xb)):
                            r, c = rows[lane, 2 * reg + e], cols[lane, 2 * reg + e]
                            assert (w >> (4 * x)) & 15 == codes[16 * blk + r, 16 * k16 + c]


def test_unpack_roundtrip():
    g = synth.gen(2)
    codes, sc = synth.int4_matrix(128, 256, g)
    words, s16 = host.pack_marlin(codes, sc)
    q, s = R.unpack_marlin(words, s16)
    assert np.array_equal(q, codes)
    assert np.array_equal(s.astype(np.float32), sc)


def test_pack_f16_matches_oracle():
    g = synth.gen(3)
    w = synth.activations(96, 256, g).astype(np.float32)
    assert np.array_equal(host.pack_f16(w).view(np.uint16), R.pack_f16(w).view(np.uint16))


def test_split_for():
    # in_proj_b/a of the 27B build: 6 tiles x 5120 columns -> 40 splits of 128 (decode, 8-token tile)
    assert host.split_for(6, 5120, 16, 1024) == R.split_for(6, 5120, 16, 1024) == 40


def test_kv_slots_are_permutations():
    d = np.arange(R.HD)
    assert sorted(R.kslot(d).tolist()) == list(range(R.HD))
    pos = np.repeat(np.arange(32), R.HD)
    dd = np.tile(d, 32)
    assert sorted(R.vslot(pos, dd).tolist()) == list(range(32 * R.HD))


def test_pack_marlin_with_zero_points_matches_oracle():
    """The second scale table (8 - z) * scale of asymmetric int4 (pack_marlin with zeros, src/cuda/core.rs:262-285)."""
    g = synth.gen(9)
    rows, cols = 128, 512
    codes, sc = synth.int4_matrix(rows, cols, g)
    zeros = torch.randint(0, 16, (rows, cols // 128), generator=g, dtype=torch.uint8).numpy()
    words, s16 = host.pack_marlin(codes, sc, zeros=zeros)
    ow, os_ = R.pack_marlin(codes, sc.astype(np.float16), R.row_order(rows, False), zeros=zeros)
    assert np.array_equal(words, ow) and s16.shape == (2 * cols // 128, rows)
    assert np.array_equal(s16.view(np.uint16), os_.view(np.uint16))
    # the offsets are exact: |8 - z| <= 8 times a bf16 significand
    off = (8.0 - zeros.astype(np.float64)) * sc.astype(np.float64)
    o = np.arange(rows)
    at = (o // 64) * 64 + 8 * (o % 8) + (o % 64) // 8
    assert np.array_equal(s16[cols // 128:][:, at].T.astype(np.float64), off)


def test_pack_i8_matches_oracle():
    """The library's int8 packer against the oracle's restatement of the reference's (quantisation per row and 128
    columns, fragment order with two k16 steps per load, scales per tile and group), with a row order and an
    all-zero group."""
    g = np.random.default_rng(11)
    w = (g.standard_normal((64, 384)) * 0.05).astype(np.float32)
    w[5, 128:256] = 0
    w[7, 3] = 1.0  # an outlier sets its group's scale
    order = host.row_order(64, True)
    codes, sc = host.pack_i8(w, order)
    oc, os_ = R.pack_i8(w, order)
    assert np.array_equal(codes, oc) and np.array_equal(sc, os_)
    q, scale = R.quant_i8(w)
    assert np.abs(q).max() == 127 and scale[5, 1] == 1.0 and np.all(q[5, 128:256] == 0)
    assert np.abs(R.dequant_i8(w) - w).max() <= scale.max() * 0.5 + 1e-7
