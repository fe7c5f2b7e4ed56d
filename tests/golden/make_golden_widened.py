"""Generates tests/golden/ref_widened.npz: outputs of the reference's OWN kernels (oracle/_ref) for the rows built
around the hot path: the sampler (sample_rows, draft_sample), the unmerged LoRA kernels and the int8 dense product,
on seeded inputs, run on a GPU. tests/test_oracle_widened_cpu.py holds the CPU oracles to these vectors, which pins
them to the reference without a GPU at test time.

    python tests/golden/make_golden_widened.py [out.npz]      (needs a CUDA device and oracle/_ref)
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_cuda  # noqa: E402
from oracle import ref_sample as S  # noqa: E402

F = np.float32
V = 248320  # the reference module's compile-time vocabulary
IMAX = 2 ** 31 - 1
SAMPLER_SETS = [(0.0, 50, 1.0, 1.1, 0.0), (0.7, 20, 0.8, 1.0, 0.0), (1.0, 1024, 0.95, 1.1, 0.0), (0.9, 5, 0.5, 1.3, 0.0),
                (1.0, 20, 0.95, 1.0, 1.5), (0.7, 20, 0.8, 1.1, 2.0)]


def sampler_inputs():
    """Seeded inputs, regenerated identically by the CPU test: one logit row of the 27B vocabulary with a few likely
    tokens, a slot's seen and generated sets, and the sampling rows (plain, with an argmax draft)."""
    g = np.random.default_rng(4321)
    hist = [1000 + (i * 7) % 23 for i in range(60)]
    logits = (g.standard_normal(V) * 2.0).astype(F)
    hot = list(g.integers(0, V, 12)) + hist[:6]
    logits[hot] += g.uniform(4, 9, len(hot)).astype(F)
    seen = np.zeros(V, dtype=bool)
    seen[hist] = True
    gen = np.zeros(V, dtype=bool)
    gen[hist[-20:]] = True
    rng = S.Rng(11)
    top = np.argsort(-logits)[:3]
    rows = []
    for (temp, k, p, rep, pres) in SAMPLER_SETS:
        for it in range(4):
            draft = None if it < 2 else int(top[it - 2])
            rows.append(S.params_row(temp, k, p, rep, pres, rng, draft=draft))
    drows = []
    for (temp, k, p, rep, pres) in [(1.0, 20, 0.95, 1.0, 1.5), (0.7, 0, 0.8, 1.1, 0.0)]:
        r = S.draft_row(temp, k, p, rep, pres)
        r[4] = rng.next_f32()
        drows.append(r)
    return dict(logits=logits, seen=seen, gen=gen, rows=np.stack(rows), drows=np.stack(drows), last=hist[-1])


def lora_inputs():
    g = np.random.default_rng(99)
    rank, rows, n, split = 16, 512, 6, 3
    M = 48
    return dict(rank=rank, rows=rows, n=n, split=split, M=M,
                xa=(g.standard_normal((split, n, M)) * 0.3).astype(F),
                B=(g.standard_normal((rows, rank)) * 0.1).astype(np.float16),
                tab=[128, 256, IMAX, IMAX, 16, -1, 0, -1], tab_silu=[IMAX, IMAX, IMAX, IMAX, 16, 0, -1, -1],
                tok_slot=np.array([0, 1, 2, 0, 2, 1], dtype=np.int32), slot_scale=np.array([2.0, 0.0, 0.5], dtype=F),
                y=g.standard_normal((n, rows)).astype(F))


def i8_inputs():
    g = np.random.default_rng(7)
    return dict(w=(g.standard_normal((64, 512)) * 0.04).astype(F), x=(g.standard_normal((5, 512)) * 0.5).astype(np.float16))


def bits(mask):
    return np.packbits(mask, bitorder="little").view(np.uint32).copy()


def main(out):
    from qwenny_b200 import host
    ref = ref_cuda.RefModule()
    res = {}
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    # ---- sampler: every row as a step of its own (one sequence in slot 0, its last token alone)
    d = sampler_inputs()
    logits, seen, outs = dev(d["logits"][None]), dev(bits(d["seen"]).view(np.int32)), dev(bits(d["gen"]).view(np.int32))
    one = torch.zeros(1, dtype=torch.int32, device="cuda")
    ids = torch.tensor([d["last"]], dtype=torch.int32, device="cuda")
    q = [torch.full((16,), -1, dtype=torch.int32, device="cuda"), torch.zeros(16, dtype=torch.int32, device="cuda"),
         torch.zeros(16 * 1024, dtype=torch.int32, device="cuda"), torch.zeros(16 * 1024, device="cuda")]
    toks, accs = [], []
    for r in d["rows"]:
        tok = torch.zeros(1, dtype=torch.int32, device="cuda")
        acc = torch.zeros(1, dtype=torch.int32, device="cuda")
        ref.sample_rows(logits, one, one, ids, one, seen, outs, dev(r[None]), *q, tok, acc, 1)
        toks.append(int(tok.item()))
        accs.append(int(acc.item()))
    res["sample_tok"], res["sample_acc"] = np.array(toks), np.array(accs)
    dtok, dqn, dqid, dqp = [], [], [], []
    for r in d["drows"]:
        for t in q:
            t.zero_()
        q[0].fill_(-1)
        dr = torch.zeros(1, dtype=torch.int32, device="cuda")
        ref.draft_sample(logits, V, V, None, one, one, seen, outs, dev(r[None]), dr, *q, 1)
        n = int(q[1][0].item())
        dtok.append(int(dr.item()))
        dqn.append(n)
        dqid.append(np.pad(q[2][:n].cpu().numpy(), (0, 1024 - n)))
        dqp.append(np.pad(q[3][:n].cpu().numpy(), (0, 1024 - n)))
    res["draft_tok"], res["draft_qn"] = np.array(dtok), np.array(dqn)
    res["draft_qid"], res["draft_qp"] = np.stack(dqid), np.stack(dqp)
    # ---- LoRA
    L = lora_inputs()
    y = dev(L["y"]).clone()
    ref.lora_add(L["rank"], dev(L["xa"]), L["split"], L["M"], dev(L["B"]), L["rows"],
                 torch.tensor(L["tab"], dtype=torch.int32).cuda(), dev(L["tok_slot"]), dev(L["slot_scale"]), L["n"], y,
                 L["rows"])
    res["lora_add"] = y.cpu().numpy()
    mid = torch.zeros(L["n"], L["rows"] // 2, dtype=torch.float16, device="cuda")
    ref.lora_silu(L["rank"], dev(L["xa"]), L["split"], L["M"], dev(L["B"]), L["rows"],
                  torch.tensor(L["tab_silu"], dtype=torch.int32).cuda(), dev(L["tok_slot"]), dev(L["slot_scale"]), L["n"],
                  dev(L["y"]), L["rows"], mid)
    res["lora_silu"] = mid.cpu().numpy()
    # ---- int8 dense product
    I = i8_inputs()
    codes, sc = host.pack_i8(I["w"])
    yi = torch.zeros(1, 5, 64, device="cuda")
    ref.gemm_dec("i8", "plain", dev(codes), dev(sc), dev(I["x"]), yi, 5, 512, 4, 512, 64)
    res["gemm_i8"] = yi[0].cpu().numpy()
    torch.cuda.synchronize()
    np.savez_compressed(out, **res)
    print("wrote", out, {k: v.shape for k, v in res.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_widened.npz"))
