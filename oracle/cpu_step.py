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


def time_baseline(seconds: float = 15.0, threads: int | None = None, rows: int = 5, vocab: int = 151936):
    """The CPU baseline of the benchmark: the fp32 forward of one [DeltaNet, DeltaNet, DeltaNet, attention] block of
    the 27B shape (the matrix products and the element-wise work of a 5-row verify step; attention over 32000 int8
    keys dequantised on the fly) plus the output layer, on `threads` host threads. The full 64-layer model does not
    fit the host in f32 (~100 GB), so the block is timed and scaled by 16; the output layer is timed once per step.
    Returns dict(step_s, rows_per_s, cores, sample)."""
    if threads:
        torch.set_num_threads(threads)
    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    H, FF = R.H, R.FF
    mk = lambda n, k: torch.randn(n, k, generator=g) * 0.01
    blocks = []
    for kind in ("delta", "delta", "delta", "attn"):
        blocks.append(dict(kind=kind, inp=mk(R.DELTA_IN if kind == "delta" else R.ATTN_IN, H), out=mk(H, R.MIX),
                           gu=mk(2 * FF, H), down=mk(H, FF)))
    lm = mk(vocab, H)
    ctx_keys = 32000
    kc = torch.randint(-127, 128, (R.NKV, ctx_keys, R.HD), generator=g, dtype=torch.int8)
    vc = torch.randint(-127, 128, (R.NKV, ctx_keys, R.HD), generator=g, dtype=torch.int8)
    ksc, vsc = torch.rand(R.NKV, ctx_keys, generator=g) * 0.05, torch.rand(R.NKV, ctx_keys, generator=g) * 0.05
    S = torch.randn(R.LV_HEADS, R.LVD, R.LKD, generator=g) * 0.01
    x = torch.randn(rows, H, generator=g)

    def norm(t):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + 1e-6)

    def block_pass():
        h = x
        for b in blocks:
            p = norm(h) @ b["inp"].T
            if b["kind"] == "delta":
                q = torch.nn.functional.normalize(p[:, :2048].view(rows, 16, 128), dim=-1).repeat_interleave(3, 1)
                k = torch.nn.functional.normalize(p[:, 2048:4096].view(rows, 16, 128), dim=-1).repeat_interleave(3, 1)
                v = p[:, 4096:10240].view(rows, 48, 128)
                St, o = S, []
                for t in range(rows):
                    dk = torch.einsum("hvk,hk->hv", St, k[t])
                    d = (v[t] - 0.9 * dk) * 0.5
                    o.append(0.9 * torch.einsum("hvk,hk->hv", St, q[t]) + d * (k[t] * q[t]).sum(-1, keepdim=True))
                    St = 0.9 * St + d[:, :, None] * k[t][:, None, :]
                mix = norm(torch.stack(o)).reshape(rows, -1) * torch.nn.functional.silu(p[:, 10240:])
            else:
                qh = p[:, :12288].view(rows, 24, 2, 256)[:, :, 0]
                o = []
                for gi in range(R.NKV):
                    K = kc[gi].float() * ksc[gi][:, None]
                    V = vc[gi].float() * vsc[gi][:, None]
                    sc = torch.einsum("rhd,kd->rhk", qh[:, gi * 6:(gi + 1) * 6], K) / 16
                    o.append(torch.softmax(sc, -1) @ V)
                mix = torch.cat(o, 1).reshape(rows, -1)
            h = h + mix @ b["out"].T
            gu = norm(h) @ b["gu"].T
            h = h + (torch.nn.functional.silu(gu[:, :FF]) * gu[:, FF:]) @ b["down"].T
        return h

    block_pass()  # warm-up
    t0, nb = time.time(), 0
    while True:
        hlast = block_pass()
        nb += 1
        if time.time() - t0 > seconds * 0.8:
            break
    tb = (time.time() - t0) / nb
    t1 = time.time()
    _ = (norm(hlast) @ lm.T).argmax(-1)
    tl = time.time() - t1
    step_s = 16 * tb + tl
    return dict(step_s=step_s, rows_per_s=rows / step_s, cores=threads,
                sample=f"{nb} passes of one [DeltaNet x3, attention] block x16 + 1 output layer, {rows} rows, f32 torch CPU")
