"""Generates tests/golden/ref_marlin_blocks.npz: Marlin matrices written block by block by the reference's OWN
marlin_put_block kernel (oracle/_ref; kernels/marlin.cuh:614-622), and an int8 embedding row looked up by its embed_q8
(kernels/qwen.cu:85-98), on seeded inputs, run on a GPU. marlin_put_block is the reference's one piece of device code
that places Marlin words and scales, so its output pins the layout of pack_marlin (src/cuda/core.rs:262-311) as far as
executed reference code can: where the word of (k16, 64-row group, lane, block) and the scale of a row sit. The nibble
order INSIDE a word (marlin_word, src/cuda/core.rs:244-253) is host code and stays pinned by reading.
tests/test_layouts_cpu.py regenerates the inputs and holds the oracle's and the library's packers to these buffers.

    python tests/golden/make_golden_marlin.py [out.npz]      (needs a CUDA device and oracle/_ref)
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_cuda  # noqa: E402
from oracle import ref_ops as R  # noqa: E402

ROWS, COLS = 256, 512


def inputs():
    """Seeded, regenerated identically by the CPU test: stored codes, f16 scales (not bf16-representable on purpose),
    zero points, and a packed-row order that is not the identity."""
    g = np.random.default_rng(20240)
    q = g.integers(0, 16, (ROWS, COLS)).astype(np.uint8)
    sc = (np.abs(g.standard_normal((ROWS, COLS // 128))) * 0.02 / 7 + 1e-4).astype(np.float16)
    zeros = g.integers(0, 16, (ROWS, COLS // 128)).astype(np.uint8)
    order = g.permutation(ROWS)
    return q, sc, zeros, order


def embed_inputs():
    g = np.random.default_rng(7)
    table = g.integers(0, 256, (40, R.H)).astype(np.uint8)
    scales = (np.abs(g.standard_normal((40, R.H // 128))) * 0.01 + 1e-3).astype(np.float32)
    ids = np.array([3, 39, 0, 17], dtype=np.int32)
    return table, scales, ids


def write_with_reference(m, q, sc, zeros, order):
    """Fill a zeroed matrix with the reference's marlin_put_block, one launch per 16-row block, as Gemm::put_block
    launches it (src/cuda/core.rs:656-668): grid k / 16 blocks of 32 threads."""
    n, k = len(order), q.shape[1]
    tables = 1 if zeros is None else 2
    B = torch.zeros(k // 16, 2 * n, dtype=torch.int32, device="cuda")
    S = torch.zeros(tables * (k // 128), n, dtype=torch.float16, device="cuda")
    for block in range(n // 16):
        words, s16 = R.marlin_block(q, sc, order[16 * block:16 * block + 16], zeros)
        wd = torch.from_numpy(words.view(np.int32)).cuda()
        sd = torch.from_numpy(s16.view(np.int16)).cuda()
        m.launch("marlin_put_block", (k // 16,), 32, 0, [
            C.c_void_p(B.data_ptr()), C.c_void_p(S.data_ptr()), C.c_void_p(wd.data_ptr()), C.c_void_p(sd.data_ptr()),
            C.c_int(n), C.c_int(block // 4), C.c_int(block % 4), C.c_int(k // 128), C.c_int(tables)])
    torch.cuda.synchronize()
    return B.cpu().numpy().view(np.uint32), S.cpu().numpy()


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_marlin_blocks.npz")
    m = ref_cuda.RefModule()
    q, sc, zeros, order = inputs()
    B, S = write_with_reference(m, q, sc, None, order)
    Bz, Sz = write_with_reference(m, q, sc, zeros, order)
    table, scales, ids = embed_inputs()
    o = torch.zeros(len(ids), R.H, device="cuda")
    keys = torch.ones(4, dtype=torch.int64, device="cuda")
    td, sd, idd = torch.from_numpy(table).cuda(), torch.from_numpy(scales).cuda(), torch.from_numpy(ids).cuda()
    m.launch("embed_q8", (len(ids),), 256, 0, [C.c_void_p(td.data_ptr()), C.c_void_p(sd.data_ptr()),
                                                C.c_void_p(idd.data_ptr()), C.c_void_p(o.data_ptr()),
                                                C.c_void_p(keys.data_ptr()), C.c_int(2)])
    torch.cuda.synchronize()
    np.savez_compressed(out, words=B, scales=S.view(np.uint16), words_z=Bz, scales_z=Sz.view(np.uint16),
                        embed_q8=o.cpu().numpy(), embed_keys=keys.cpu().numpy())
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
