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


def test_marlin_block_and_put_block_assemble_pack_marlin():
    """A matrix filled block by block (Gemm::put_block: the host's words and scales of 16 rows, then the scatter of
    marlin_put_block) is the matrix pack_marlin makes at once, with and without zero points; the library's host half
    equals the oracle's."""
    g = np.random.default_rng(5)
    rows, cols = 128, 256
    q = g.integers(0, 16, (rows, cols)).astype(np.uint8)
    sc = (np.abs(g.standard_normal((rows, cols // 128))) * 0.01 + 1e-4).astype(np.float16).astype(np.float32)  # f16 values
    zeros = g.integers(0, 16, (rows, cols // 128)).astype(np.uint8)
    order = g.permutation(rows)
    for z in (None, zeros):
        want_w, want_s = host.pack_marlin(q, sc, order=order, zeros=z)
        B = np.zeros_like(want_w)
        S = np.zeros_like(want_s)
        for block in range(rows // 16):
            r16 = order[16 * block:16 * block + 16]
            w, s16 = host.marlin_block(q, sc, r16, zeros=z, zero_points=z is not None)
            ow, os_ = R.marlin_block(q, sc.astype(np.float16), r16, z)
            assert np.array_equal(w, ow) and np.array_equal(s16.view(np.uint16), os_.view(np.uint16))
            R.put_block(B, S, w, s16, block)
        assert np.array_equal(B, want_w)
        assert np.array_equal(S.view(np.uint16), want_s.view(np.uint16))
    # rows with zero points cannot enter a symmetric matrix (put_block's ensure!, src/cuda/core.rs:630-634)
    with pytest.raises(Exception):
        host.marlin_block(q, sc, order[:16], zeros=zeros, zero_points=False)


def test_matrices_written_by_the_reference_kernel_pin_the_layout():
    """tests/golden/ref_marlin_blocks.npz holds matrices the reference's compiled marlin_put_block wrote block by block
    (make_golden_marlin.py): the positions of words and scales in pack_marlin's layout as executed reference code has
    them. The oracle's and the library's packers must produce the same buffers bit for bit, and the oracle's unpack
    must read the reference-written matrix back to the stored codes."""
    import importlib.util
    import os
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    spec = importlib.util.spec_from_file_location("make_golden_marlin", os.path.join(here, "make_golden_marlin.py"))
    # the generator's seeded inputs, without importing its GPU side
    src = open(spec.origin).read()
    ns = {"np": np, "R": R}
    exec(compile(src[src.index("ROWS, COLS ="):src.index("def write_with_reference")], spec.origin, "exec"), ns)
    q, sc, zeros, order = ns["inputs"]()
    gold = np.load(os.path.join(here, "ref_marlin_blocks.npz"))
    ow, os_ = R.pack_marlin(q, sc, order)
    assert np.array_equal(gold["words"], ow) and np.array_equal(gold["scales"], os_.view(np.uint16))
    owz, osz = R.pack_marlin(q, sc, order, zeros)
    assert np.array_equal(gold["words_z"], owz) and np.array_equal(gold["scales_z"], osz.view(np.uint16))
    lw, ls = host.pack_marlin(q, sc.astype(np.float32), order=order)
    assert np.array_equal(gold["words"], lw) and np.array_equal(gold["scales"], ls.view(np.uint16))
    lwz, lsz = host.pack_marlin(q, sc.astype(np.float32), order=order, zeros=zeros)
    assert np.array_equal(gold["words_z"], lwz) and np.array_equal(gold["scales_z"], lsz.view(np.uint16))
    uq, us = R.unpack_marlin(gold["words"], gold["scales"].view(np.float16))
    assert np.array_equal(uq, q[order]) and np.array_equal(us.view(np.uint16), sc[order].view(np.uint16))
    # the int8 embedding lookup of the reference's embed_q8, and its cleared argmax keys
    table, scales, ids = ns["embed_inputs"]()
    assert np.array_equal(gold["embed_q8"], R.embed_q8(table, scales, ids))
    assert gold["embed_keys"].tolist() == [0, 0, 1, 1]


def test_host_bookkeeping_selftests():
    """The step-graph cache policy (least recently used out when memory is short, three quarters kept after a capture
    without memory) and the per-device kernel-attribute cache, each run against fakes inside the library."""
    from qwenny_b200._lib import lib
    assert lib().qb_graph_cache_selftest() == 0
    assert lib().qb_attr_cache_selftest() == 0
