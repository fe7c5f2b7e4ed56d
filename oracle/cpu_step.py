"""CPU restatement of the whole decode / verify step (the oracle of the full path) and the CPU baseline's workload.

TEST INFRASTRUCTURE ONLY. `CpuModel` holds a model's tensors on the host in the library's own layouts (Marlin words,
cache bytes, slot memory) and runs a step with the per-op oracles of ref_ops in the reference's launch order
(launch_step, src/cuda/qwen/mod.rs:744-766; Stack::layer/mix/mlp :498-575; Attn::run, DeltaNet::run). The method of
the reference's own CPU check path (tools/make_reference.py:25-39: an fp32 forward of the same weights) is what the
timed baseline follows: weights dequantised once to f32, activations f32, torch CPU matmuls on all host threads.
"""
from __future__ import annotations

import math
import time

import numpy as np
import torch

from . import ref_ops as R

QSCALE = math.log2(math.e) / 16.0


def dequant_marlin(words: np.ndarray, scales: np.ndarray) -> torch.Tensor:
    """Marlin words + scales -> f32 [n][k] in packed row order (what the kernels multiply by): ref_ops.unpack_marlin
    followed by ref_ops.dequant (w = f16((q - 8) * f16 scale)), the same index arithmetic run through torch's threaded
    CPU kernels so that full-width layers unpack in seconds (tests/test_oracle_cpu.py holds the two forms equal)."""
    k16, n2 = words.shape
    n, k = n2 // 2, k16 * 16
    w = torch.from_numpy(np.ascontiguousarray(words).view(np.int32)).reshape(k16, n // 64, 32, 4)
    r, c = R._marlin_lane_maps()
    inv = np.zeros(256, dtype=np.int64)
    inv[(r * 16 + c).reshape(-1)] = np.arange(256)
    nib = torch.stack([((w >> (4 * x)) & 15).to(torch.uint8) for x in range(8)], dim=-1)   # [k16][c64][lane][blk][x]
    nib = nib.permute(0, 1, 3, 2, 4).reshape(k16, n // 64, 4, 256)[..., torch.from_numpy(inv)]
    q = nib.reshape(k16, n // 64, 4, 16, 16).permute(1, 2, 3, 0, 4).reshape(n, k)
    o = np.arange(n)
    at = (o // 64) * 64 + 8 * (o % 8) + (o % 64) // 8
    s = torch.from_numpy(np.ascontiguousarray(scales[:k // 128]).view(np.int16)).view(torch.float16)
    s = s[:, torch.from_numpy(at)].T.float()
    return ((q.reshape(n, k // 128, 128).float() - 8.0) * s[:, :, None]).half().float().reshape(n, k)


class CpuModel:
    """layers: list of dicts of numpy arrays with the names of qwenny_b200.model.synthetic()."""

    def __init__(self, layers, embed_f32, final_norm, lm_words, lm_scales, vocab_valid, slots):
        self.layers, self.embed, self.final_norm = layers, embed_f32, final_norm
        self.vocab_valid, self.slots = vocab_valid, slots
        for l in layers:
            for name in ("in_proj", "out", "gate_up", "down"):
                l[name + "_f32"] = dequant_marlin(l[name + "_words"], l[name + "_scales"])
            if l["kind"] == "delta":
                # in_ba arrives in fragment order: unpack to [96][5120]
                rows, cols = R.frag_map()
                a = np.zeros((l["in_ba"].shape[0], 16, l["in_ba"].shape[1], 16), dtype=np.float32)
                a[:, rows, :, cols] = np.transpose(l["in_ba"].astype(np.float32), (2, 3, 0, 1))
                l["in_ba_f32"] = torch.from_numpy(a.transpose(0, 1, 2, 3).reshape(-1, l["in_ba"].shape[1] * 16))
        self.lm = dequant_marlin(lm_words, lm_scales)

    @staticmethod
    def _host_layer(l):
        d = dict(kind=l["kind"])
        for name in ("in_proj", "out", "gate_up", "down"):
            d[name + "_words"] = l[name].words.cpu().numpy().view(np.uint32)
            d[name + "_scales"] = l[name].scales.cpu().numpy()
        for k, v in l.items():
            if isinstance(v, torch.Tensor):
                d[k] = v.cpu().numpy()
            elif k in ("sst", "cap"):
                d[k] = v
            elif k == "lora":  # the adapter's host copies (qwenny_b200.model.synthetic_adapter)
                d[k] = {name: {f: p[f] for f in ("A", "B", "tab_h", "B2", "tab2_h") if f in p}
                        for name, p in v.items() if isinstance(p, dict)}
        return d

    @staticmethod
    def from_device(model):
        """Host copy of a qwenny_b200.model.Model (small models only), its MTP layer included."""
        layers = [CpuModel._host_layer(l) for l in model.layers]
        mtp = getattr(model, "mtp", None)
        if mtp is not None:
            layers.append(CpuModel._host_layer(mtp["layer"]))
        cm = CpuModel(layers, model.embed.float().cpu().numpy(), model.final_norm.cpu().numpy(),
                      model.lm_head.words.cpu().numpy().view(np.uint32), model.lm_head.scales.cpu().numpy(),
                      model.vocab_valid, model.slots)
        cm.mtp = None
        if mtp is not None:
            cm.mtp_layer = cm.layers.pop()
            cm.mtp = dict(fc=dequant_marlin(mtp["fc"].words.cpu().numpy().view(np.uint32), mtp["fc"].scales.cpu().numpy()),
                          pre_e=mtp["pre_e"].cpu().numpy(), pre_h=mtp["pre_h"].cpu().numpy(),
                          norm=mtp["norm"].cpu().numpy(), head=None)
            if mtp.get("head") is not None:
                cm.mtp["head"] = dequant_marlin(mtp["head"].words.cpu().numpy().view(np.uint32),
                                                mtp["head"].scales.cpu().numpy())
                cm.mtp["head_valid"] = mtp["head_valid"]
                cm.mtp["head_ids"] = mtp["head_ids"].cpu().numpy()
        return cm

    @staticmethod
    def _mm(x_f16: np.ndarray, w: torch.Tensor) -> np.ndarray:
        return (torch.from_numpy(x_f16.astype(np.float32)) @ w.T).numpy()

    def step(self, toks, out_rows):
        """Returns (logits f32 [n_out][vocab_rows], greedy tokens). Updates the caches and states in place."""
        st = R.build_step(toks, out_rows)
        n = st["n"]
        if getattr(self, "slot_scale", None) is not None:
            st["lora_scale"] = np.asarray(self.slot_scale, dtype=np.float32)[st["tok_slot"]]
        h = R.embed(self.embed, st["ids"])
        xn = R.rmsnorm(h, self.layers[0]["input_norm"])
        for i, l in enumerate(self.layers):
            w_next = self.layers[i + 1]["input_norm"] if i + 1 < len(self.layers) else self.final_norm
            h, xn = self._layer(l, st, h, xn, w_next)
        self.h_last = h
        logits = self._mm(xn[st["out_rows"]], self.lm)
        keys = R.argmax_keys(logits, self.vocab_valid)
        return logits, R.key_token(keys), h, xn

    def draft(self, toks, rows, out, k):
        """Engine::draft with greedy rows (draft_chains, src/cuda/qwen/mod.rs:870-896) on the residual stream the last
        step() left. Returns (drafts [len(out)][k], logits of every MTP step)."""
        chains, all_logits = [[] for _ in out], []
        cur, at, outs, own = list(toks), list(rows), list(out), False
        for t in range(k):
            st = R.build_step(cur, outs)
            e = R.embed(self.embed, st["ids"])
            fw = self.mtp["norm"] if own else self.final_norm
            xin = R.mtp_in(e, self.h_last, np.asarray(at), fw, self.mtp["pre_e"], self.mtp["pre_h"])
            h = self._mm(xin, self.mtp["fc"])
            xn = R.rmsnorm(h, self.mtp_layer["input_norm"])
            h, xn = self._layer(self.mtp_layer, st, h, xn, self.mtp["norm"])
            self.h_last = h
            if self.mtp["head"] is not None:
                logits = self._mm(xn[st["out_rows"]], self.mtp["head"])
                idx = R.key_token(R.argmax_keys(logits, self.mtp["head_valid"]))
                picked = [int(self.mtp["head_ids"][i]) for i in idx]
            else:
                logits = self._mm(xn[st["out_rows"]], self.lm)
                picked = [int(i) for i in R.key_token(R.argmax_keys(logits, self.vocab_valid))]
            all_logits.append(logits)
            for i, p in enumerate(picked):
                chains[i].append(p)
            cur = [(picked[i], cur[o][1], cur[o][2] + 1) for i, o in enumerate(outs)]
            at, outs, own = list(range(len(cur))), list(range(len(cur))), True
        return chains, all_logits

    def _lora(self, l, st, prod, x, which="B", silu=False):
        """The delta of an adapted product (src/cuda/qwen/lora.rs:1-8): s * B (A x) for the tokens of adapter slots, A
        and B as the device holds them (f16 values), 0 when the step has no such token or the product no adapter."""
        lo = l.get("lora")
        sc = st.get("lora_scale")
        if lo is None or sc is None or not np.any(sc != 0) or lo.get(prod) is None or lo[prod].get(which) is None:
            return 0.0
        p = lo[prod]
        xa = (x.astype(np.float32) @ p["A"].T)[None]
        return R.lora_delta(xa, p[which], p["tab_h" if which == "B" else "tab2_h"], sc, silu)

    def _layer(self, l, st, h, xn, w_next):
        n = st["n"]
        part = (self._mm(xn, l["in_proj_f32"]) + self._lora(l, st, "inp", xn))[None]
        if l["kind"] == "delta":
            ba = (self._mm(xn, l["in_ba_f32"]) + self._lora(l, st, "inp", xn, "B2"))[None]
            cv = R.delta_conv(part, ba, l["conv_w"], l["a_log"], l["dt_bias"], l["mem"], l["sst"], st["tok_slot"],
                              st["tok_pos"])
            o = R.delta_rule(part, cv, l["mem"], l["sst"], l["meta"], st["seg_start"], st["seg_len"],
                             st["seg_slot"], st["seg_pos0"])
            mix = R.delta_norm(part, l["norm_w"], o, l["meta"], st["seg_len"], st["seg_slot"], st["seg_pos0"])
        else:
            q, gate, k, v = R.attn_prep(part, l["q_norm"], l["k_norm"], l["inv_freq"], QSCALE, st["tok_pos"])
            R.kv_store(l["kc"], l["vc"], l["ks"], l["vs"], k, v, st["tok_slot"], st["tok_pos"], l["cap"])
            o = R.attn_decode(q, gate, l["kc"], l["vc"], l["ks"], l["vs"], st["tok_slot"], st["tok_pos"], l["cap"])
            mix = o.astype(np.float16)
        h, xn = R.add_rmsnorm(h, (self._mm(mix, l["out_f32"]) + self._lora(l, st, "out", mix))[None], l["post_norm"])
        gu = self._mm(xn, l["gate_up_f32"]) + self._lora(l, st, "gate_up", xn, silu=True)
        b = gu.reshape(n, -1, 2, 8)
        mid = (R.silu(b[:, :, 0, :]) * b[:, :, 1, :]).reshape(n, -1).astype(np.float16)
        h, xn = R.add_rmsnorm(h, (self._mm(mid, l["down_f32"]) + self._lora(l, st, "down", mid))[None], w_next)
        return h, xn


def host_block_model(seed: int = 0, position: int = 32000, vocab: int = 151936, layers=("delta", "delta", "delta", "attn"),
                     max_ctx: int = 32768) -> CpuModel:
    """One [DeltaNet, DeltaNet, DeltaNet, attention] block of the 27B shape and the output layer, built on the host
    with the distributions of qwenny_b200.model.synthetic (random int4 words, bf16-valued scales |N(0, 0.02)| / 7 + 1e-4,
    norms 1 + N(0, 0.02)), its caches filled as if `position` tokens had been processed. No GPU is involved."""
    g = np.random.default_rng(seed)
    f32 = np.float32

    def marlin(n, k):
        words = g.integers(0, 2 ** 32, (k // 16, 2 * n), dtype=np.uint64).astype(np.uint32)
        sc = torch.from_numpy((np.abs(g.standard_normal((k // 128, n))) * (0.02 / 7) + 1e-4).astype(f32))
        return words, sc.to(torch.bfloat16).to(torch.float16).numpy()

    norm = lambda n: (1 + g.standard_normal(n) * 0.02).astype(f32)
    cap = (max_ctx + 63) // 64 * 64
    sst = (R.SLOT_FLOATS + 1023) // 1024 * 1024
    ls = []
    for kind in layers:
        l = dict(kind=kind, input_norm=norm(R.H), post_norm=norm(R.H))
        for name, (n, k) in dict(out=(R.H, R.MIX), gate_up=(2 * R.FF, R.H), down=(R.H, R.FF),
                                 in_proj=(R.DELTA_IN if kind == "delta" else R.ATTN_IN, R.H)).items():
            l[name + "_words"], l[name + "_scales"] = marlin(n, k)
        if kind == "delta":
            l["in_ba"] = (g.standard_normal((2 * R.LV_HEADS // 16, R.H // 16, 32, 8)) * 0.02).astype(np.float16)
            l["conv_w"] = (g.standard_normal((R.LQKV, 4)) * 0.3).astype(f32)
            l["a_log"] = (g.standard_normal(R.LV_HEADS) * 0.5).astype(f32)
            l["dt_bias"] = (g.standard_normal(R.LV_HEADS) * 0.5).astype(f32)
            l["norm_w"] = norm(R.LVD)
            l["mem"] = (g.standard_normal(sst) * 0.01).astype(f32)
            l["meta"] = np.array([[position, position, 0, 0]], dtype=np.int32)
            l["sst"] = sst
        else:
            l["q_norm"], l["k_norm"] = norm(R.HD), norm(R.HD)
            l["inv_freq"] = (1.0 / (R.THETA ** (np.arange(0, R.ROT, 2, dtype=np.float64) / R.ROT))).astype(f32)
            nb = R.NKV * cap
            l["kc"] = g.integers(1, 256, nb * R.HD, dtype=np.uint8)
            l["vc"] = g.integers(1, 256, nb * R.HD, dtype=np.uint8)
            l["ks"] = np.abs(g.standard_normal(nb) * 0.05).astype(f32)
            l["vs"] = np.abs(g.standard_normal(nb) * 0.05).astype(f32)
            l["cap"] = cap
        ls.append(l)
    rows = (vocab + 255) // 256 * 256
    lm_w, lm_s = marlin(rows, R.H)
    embed = (g.standard_normal((4096, R.H)) * 0.02).astype(f32)  # token ids below 4096 are enough for the timed rows
    return CpuModel(ls, embed, norm(R.H), lm_w, lm_s, vocab, 1)


def time_step_baseline(seconds: float = 15.0, threads: int | None = None, rows: int = 5, position: int = 32000,
                       vocab: int = 151936, model: "CpuModel | None" = None):
    """The CPU baseline of the benchmark: CpuModel.step, the oracle of the full path with the real op arithmetic
    (int4 weights dequantised once to f32 as the reference's fp32 check path does, tools/make_reference.py:25-39; conv,
    gated delta rule with its rollback plan, RoPE, int8 KV quantisation, attention over `position` int8 keys, norms),
    on a verify step of `rows` rows at `position`: one [DeltaNet x3, attention] block and the output layer are timed
    on `threads` host threads and the block is scaled by 16 (the 64-layer model in f32 does not fit a host).
    Returns dict(step_s, rows_per_s, cores, sample)."""
    if threads:
        torch.set_num_threads(threads)
    threads = torch.get_num_threads()
    m = model if model is not None else host_block_model(position=position, vocab=vocab)
    lm, full_valid = m.lm, m.vocab_valid
    m.lm, m.vocab_valid = lm[:256], 256   # the block alone first: a 256-row stand-in for the output layer
    pos = position
    toks = lambda p: [(1000 + i, 0, p + i) for i in range(rows)]
    m.step(toks(pos), list(range(rows)))   # warm-up
    t0, nb = time.time(), 0
    while True:
        m.step(toks(pos), list(range(rows)))   # the same positions again: the drafts were "rejected", state rolls back
        nb += 1
        if time.time() - t0 > seconds * 0.8:
            break
    tb = (time.time() - t0) / nb
    xn = np.random.default_rng(1).standard_normal((rows, R.H)).astype(np.float16)
    t1 = time.time()
    logits = CpuModel._mm(xn, lm)
    R.key_token(R.argmax_keys(logits, vocab))
    tl = time.time() - t1
    m.lm, m.vocab_valid = lm, full_valid
    step_s = 16 * tb + tl
    return dict(step_s=step_s, rows_per_s=rows / step_s, cores=threads,
                sample=f"{nb} verify steps of {rows} rows at position {position} through one [DeltaNet x3, attention] "
                       f"block of the CPU oracle (CpuModel.step: real op arithmetic, f32 weights), x16, + 1 output layer")
