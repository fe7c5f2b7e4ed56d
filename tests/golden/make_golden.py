"""Generates tests/golden/ref_kernels.npz: outputs of the reference's OWN kernels (oracle/_ref, compiled unmodified from
its sources) on small seeded inputs, run on a GPU. The CPU tests (tests/test_oracle_cpu.py) hold the numpy oracle to
these vectors, which pins it to the reference without a GPU at test time.

    python tests/golden/make_golden.py [out.npz]      (needs a CUDA device and oracle/_ref)
"""
import math
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_cuda  # noqa: E402
from oracle import ref_ops as R  # noqa: E402

QSCALE = math.log2(math.e) / 16.0
SST = (R.SLOT_FLOATS + 1023) // 1024 * 1024


def inputs():
    """Seeded inputs, regenerated identically by the CPU test."""
    g = torch.Generator().manual_seed(1234)
    d = {}
    n = 3
    d["n"] = n
    d["x"] = torch.randn(n, R.H, generator=g) * 2
    d["w"] = 1 + torch.randn(R.H, generator=g) * 0.02
    d["parts"] = torch.randn(2, n, R.H, generator=g)
    # attention
    d["apart"] = torch.randn(1, n, R.ATTN_IN, generator=g)
    d["qn"] = 1 + torch.randn(R.HD, generator=g) * 0.02
    d["kn"] = 1 + torch.randn(R.HD, generator=g) * 0.02
    d["cap"] = 128
    d["kc"] = torch.randint(1, 256, (R.NKV * 128 * R.HD,), generator=g, dtype=torch.uint8)
    d["vc"] = torch.randint(1, 256, (R.NKV * 128 * R.HD,), generator=g, dtype=torch.uint8)
    d["ks"] = (torch.randn(R.NKV * 128, generator=g) * 0.05).abs()
    d["vs"] = (torch.randn(R.NKV * 128, generator=g) * 0.05).abs()
    d["toks"] = [(0, 0, 70 + i) for i in range(n)]
    # DeltaNet
    d["dpart"] = torch.randn(1, n, R.DELTA_IN, generator=g)
    d["ba"] = torch.randn(1, n, 2 * R.LV_HEADS, generator=g)
    d["conv_w"] = torch.randn(R.LQKV, 4, generator=g) * 0.3
    d["a_log"] = torch.randn(R.LV_HEADS, generator=g) * 0.5
    d["dt_bias"] = torch.randn(R.LV_HEADS, generator=g) * 0.5
    d["norm_w"] = 1 + torch.randn(R.LVD, generator=g) * 0.02
    d["mem"] = torch.randn(SST, generator=g) * 0.01
    d["meta"] = torch.tensor([[70, 66, 1, 0]], dtype=torch.int32)
    # dense f16 product
    d["wd"] = torch.randn(32, 256, generator=g) * 0.05
    d["xd"] = torch.randn(n, 256, generator=g).half()
    return d


def main(out):
    ref = ref_cuda.RefModule()
    d = inputs()
    n = d["n"]
    st = R.build_step(d["toks"], [0])
    dv = ref_cuda.upload_step(st)
    res = {}
    c = lambda t: t.cuda()
    # rmsnorm / add_rmsnorm
    y = torch.zeros(n, R.H, dtype=torch.float16, device="cuda")
    ref.rmsnorm(c(d["x"]), c(d["w"]), y, n)
    res["rmsnorm"] = y.cpu().numpy()
    h = c(d["x"]).clone()
    ref.add_rmsnorm(h, c(d["parts"]), 2, n, c(d["w"]), y)
    res["add_h"], res["add_y"] = h.cpu().numpy(), y.cpu().numpy()
    # attention: prep writes the step's K/V into the cache, then decode over it
    q = torch.zeros(n, R.NH, R.HD, device="cuda")
    o = torch.zeros(n, R.MIX, device="cuda")
    kc, vc, ks, vs = c(d["kc"]), c(d["vc"]), c(d["ks"]), c(d["vs"])
    ref.attn_prep(c(d["apart"]), 1, n, c(d["qn"]), c(d["kn"]), c(torch.from_numpy(R.rope_inv_freq())), QSCALE, q, o, kc,
                  vc, ks, vs, dv["tok_slot"], dv["tok_pos"], d["cap"])
    res["q"], res["gate"] = q.cpu().numpy(), o.cpu().numpy()
    pos = st["tok_pos"]
    res["k_rows"] = np.stack([kc.cpu().numpy().reshape(R.NKV, d["cap"], R.HD)[:, p] for p in pos])
    res["ks_rows"] = np.stack([ks.cpu().numpy().reshape(R.NKV, d["cap"])[:, p] for p in pos])
    res["vs_rows"] = np.stack([vs.cpu().numpy().reshape(R.NKV, d["cap"])[:, p] for p in pos])
    res["vc_full"] = vc.cpu().numpy()
    ml = torch.zeros(64 * 128 * R.NH * 2, device="cuda")
    acc = torch.zeros(64 * 128 * R.NH * R.HD, device="cuda")
    ref.attn_decode(q, kc, vc, ks, vs, st, dv, d["cap"], ml, acc, o)
    res["attn_out"] = o.cpu().numpy()
    # DeltaNet
    mem, meta = c(d["mem"]), c(d["meta"])
    cv = torch.zeros(n, R.CVW, device="cuda")
    do = torch.zeros(n, R.MIX, device="cuda")
    mix = torch.zeros(n, R.MIX, dtype=torch.float16, device="cuda")
    ref.delta(c(d["dpart"]), 1, n, c(d["ba"]), 1, c(d["conv_w"]), c(d["a_log"]), c(d["dt_bias"]), c(d["norm_w"]), mem,
              SST, meta, cv, do, mix, st, dv)
    res["cv"], res["delta_out"], res["delta_mix"] = cv.cpu().numpy(), do.cpu().numpy(), mix.cpu().numpy()
    res["meta_after"] = meta.cpu().numpy()
    m = mem.cpu().numpy()
    # the end state of 4 heads (the whole state is 6 MB), the bank entries and ring rows of the step
    eb = int(res["meta_after"][0, 2])
    res["state_heads"] = m[eb * R.SLOT_STATE:(eb + 1) * R.SLOT_STATE].reshape(R.LV_HEADS, R.LVD, R.LKD)[[0, 17, 30, 47]]
    res["ring_rows"] = np.stack([m[R.SLOT_RING + ((p) & (R.CR - 1)) * R.LQKV:][:R.LQKV] for p in pos])
    # dense f16 product
    from qwenny_b200 import host
    wp = torch.from_numpy(host.pack_f16(d["wd"].numpy()).view(np.int16)).cuda().view(torch.float16)
    yd = torch.zeros(64, n, 32, device="cuda")
    split = ref.gemm_f16_plain(wp, c(d["xd"]), yd, n, 256, 2)
    res["gemm_f16"] = yd[:split].sum(0).cpu().numpy()
    torch.cuda.synchronize()
    np.savez_compressed(out, **res)
    print("wrote", out, {k: v.shape for k, v in res.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_kernels.npz"))
