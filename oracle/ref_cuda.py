"""Runs the reference's own CUDA kernels (oracle/_ref/, compiled unmodified from its sources by build_ref.py).

TEST INFRASTRUCTURE ONLY: the parity tests and the benchmark's reference arm use this to put the reference's kernels
next to the library's on the same device buffers. It restates the launch geometry the reference's Rust host computes
(each function cites it) and launches by kernel name through the driver API, as the reference's host does
(src/cuda/core.rs:42-46). Needs a GPU; reads only oracle/_ref/ at run time.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

from . import ref_ops as R

HERE = os.path.dirname(os.path.abspath(__file__))
PTX = os.path.join(HERE, "_ref", "qwen27b.ptx")
CUBIN = os.path.join(HERE, "_ref", "qwen27b.cubin")

VOCAB = 248320  # the reference's compile-time vocabulary (kernels/qwen.cu:34): sizes mark_seen's bitsets
MARLIN_SLOT = 64 * 256
MARLIN_CFG = [(1, 8, 8), (1, 16, 4), (2, 16, 4), (3, 16, 4), (4, 16, 4)]  # src/cuda/core.rs:402


def available() -> bool:
    return os.path.exists(CUBIN) or os.path.exists(PTX)


def marlin_smem(cfg, zp=False):
    """src/cuda/core.rs:409-411."""
    mb, nb, kb = cfg
    return 4 * 16 * (32 * kb * mb + 8 * nb * kb + 2 * nb * (2 if zp else 1))


class _Arg:
    pass


def _ptr(t):
    return C.c_void_p(0 if t is None else (t.data_ptr() if hasattr(t, "data_ptr") else int(t)))


class RefModule:
    """The reference's kernel module on the current device, with the scratch its host allocates."""

    def __init__(self, prefer_ptx: bool = False):
        from cuda.bindings import driver as drv
        self.drv = drv
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # primary context current
        path = PTX if (prefer_ptx or not os.path.exists(CUBIN)) else CUBIN
        with open(path, "rb") as f:
            image = f.read()
        if path.endswith(".ptx"):
            image += b"\0"
        err, self.mod = drv.cuModuleLoadData(image)
        self._ck(err, f"cuModuleLoadData({os.path.basename(path)})")
        self.image = os.path.basename(path)
        self.fns = {}
        self.smem_set = {}
        dev = torch.cuda.current_device()
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        # Marlin's scratch (src/cuda/core.rs:455-464)
        self.red = torch.zeros(self.sms * MARLIN_SLOT, dtype=torch.float32, device="cuda")
        self.locks = torch.zeros(self.sms, dtype=torch.int32, device="cuda")

    def _ck(self, err, what):
        if int(err) != 0:
            raise RuntimeError(f"{what}: CUDA driver error {err}")

    def fn(self, name, smem=0):
        f = self.fns.get(name)
        if f is None:
            err, f = self.drv.cuModuleGetFunction(self.mod, name.encode())
            self._ck(err, f"cuModuleGetFunction({name})")
            self.fns[name] = f
        if smem > self.smem_set.get(name, 48 * 1024):
            (err,) = self.drv.cuFuncSetAttribute(
                f, self.drv.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, smem)
            self._ck(err, f"cuFuncSetAttribute({name})")
            self.smem_set[name] = smem
        return f

    def launch(self, name, grid, block, smem, args):
        """args: list of ctypes values (c_void_p, c_int, c_longlong, c_float) in the kernel's parameter order."""
        f = self.fn(name, smem)
        stream = torch.cuda.current_stream().cuda_stream
        vals = tuple(a.value if a.value is not None else 0 for a in args)
        types = tuple(type(a) for a in args)
        gx, gy, gz = (tuple(grid) + (1, 1))[:3]
        (err,) = self.drv.cuLaunchKernel(f, gx, gy, gz, block, 1, 1, smem, stream, (vals, types), 0)
        self._ck(err, f"cuLaunchKernel({name})")

    # ------------------------------------------------------------------------------------------ matrix products
    def marlin(self, n, words, scales, x, y, epi="plain", keys=None, valid=None):
        """Gemm::marlin (src/cuda/core.rs:569-612): one launch per run of 64-token problems and one for the rest;
        steps of up to 16 tokens use the 128 x 128 tile kernels (marlin_m1_n8_*).

        CLOSED: on B200 (driver 580.159) the reference's marlin_m1_n8_* kernels end with "an illegal instruction
        was encountered", both as the driver-JIT PTX and as the ptxas-built cubin, on 256 x 256 and 1024 x 1024
        problems, while its other kernels run through this same loader. The cause was not found by reading
        kernels/marlin.cuh, so these kernels are not launched; the restated launch below is kept for the record."""
        raise RuntimeError("the reference's Marlin kernels fault on B200 (illegal instruction); not launched")
        rows, cols = words.shape[1] // 2, words.shape[0] * 16
        blocks = -(-n // 16)
        pad = blocks * 16 - n
        i = 0
        while i < blocks:
            mb, m, par = blocks - i, n - 16 * i, 1
            if mb > 4:
                par = (16 * mb - pad) // 64
                m, mb = 64 * par, 4
            c = 0 if n <= 16 else mb
            cfg = MARLIN_CFG[c]
            name = f"marlin_m{cfg[0]}_n{cfg[1]}_{epi}"
            smem = marlin_smem(cfg)
            self.launch(name, (self.sms,), 256, smem, [
                _ptr(x), _ptr(words), _ptr(y), _ptr(scales), C.c_int(m), C.c_int(rows), C.c_int(cols),
                C.c_int(16 * i), _ptr(self.red), _ptr(self.locks), _ptr(keys),
                C.c_int(rows if valid is None else valid)])
            i += 4 * par

    def marlin_gather(self, x, rows_idx, out, k):
        """kernels/marlin.cuh:605-608, launched as src/cuda/core.rs:518-525."""
        self.launch("marlin_gather", (rows_idx.numel(),), 128, 0, [_ptr(x), _ptr(rows_idx), _ptr(out), C.c_int(k // 8)])

    def gemm_f16_plain(self, w_packed, x, y, n, K, tiles, xrows=None):
        """Gemm::run_split for a dense f16 matrix at a decode-sized step (src/cuda/core.rs:532-560): returns the
        split factor; y gets [split][n][tiles*16] partial products."""
        tile_i = next(i for i, t in enumerate((8, 16, 32)) if n <= t)
        split = R.split_for(tiles, K, 16, 1024 * 8 // (8, 16, 32)[tile_i])
        name = f"gemm_f16_t{(8, 16, 32)[tile_i]}_plain"
        self.launch(name, (-(-tiles // 4), split, 1), 128, 0, [
            _ptr(w_packed), _ptr(None), _ptr(x), _ptr(xrows), C.c_int(K), C.c_int(tiles), C.c_int(n),
            C.c_int(K // split), _ptr(y), C.c_int(tiles * 16), _ptr(None)])
        return split

    def gemm_dec(self, wt, epi, w_packed, scales, x, y, n, K, tiles, kper, ldy, keys=None, xrows=None):
        """Gemm::run_split at a decode-sized step (src/cuda/core.rs:532-560) for a 16-bit ("f16") or int8 ("i8") matrix:
        4 tiles per block, K / kper splits; epi "plain" | "silu" | "argmax"."""
        tt = next(t for t in (8, 16, 32) if n <= t)
        self.launch(f"gemm_{wt}_t{tt}_{epi}", (-(-tiles // 4), K // kper, 1), 128, 0, [
            _ptr(w_packed), _ptr(scales), _ptr(x), _ptr(xrows), C.c_int(K), C.c_int(tiles), C.c_int(n), C.c_int(kper),
            _ptr(y), C.c_int(ldy), _ptr(keys)])

    # ------------------------------------------------------------------------------------------ dense kernels
    def embed(self, table, ids, out, keys, nkeys, n):
        self.launch("embed", (n,), 256, 0, [_ptr(table), _ptr(ids), _ptr(out), _ptr(keys), C.c_int(nkeys)])

    def rmsnorm(self, x, w, y, n, eps=R.EPS):
        self.launch("rmsnorm", (n,), 256, 0, [_ptr(x), _ptr(w), _ptr(y), C.c_float(eps)])

    def add_rmsnorm(self, h, x, splits, n, w_next, y, eps=R.EPS):
        self.launch("add_rmsnorm", (n,), 512, 0, [_ptr(h), _ptr(x), C.c_int(splits), C.c_int(n), _ptr(w_next),
                                                    _ptr(y), C.c_float(eps)])

    def to_xin(self, x, y, length):
        self.launch("to_xin", (min(-(-length // 1024), 1024),), 256, 0, [_ptr(x), _ptr(y), C.c_int(length)])

    def mark_seen(self, seen, mark, mark_at, seg_slot, seg_pos0, segs):
        self.launch("mark_seen", (segs,), 256, 0, [_ptr(seen), _ptr(mark), _ptr(mark_at), _ptr(seg_slot), _ptr(seg_pos0)])

    # ------------------------------------------------------------------------------------------ LoRA
    def lora_add(self, rank, xa, split, M, B, rows, tab, tok_slot, slot_scale, n, y, ldy):
        """LoraA::launch without mid (src/cuda/qwen/lora.rs:163-196): a block per 256 rows and 8 tokens."""
        self.launch(f"lora_add_r{rank}", (-(-rows // 256), -(-n // 8)), 256, 0,
                    [_ptr(xa), C.c_int(split), C.c_int(M), _ptr(B), C.c_int(rows), _ptr(tab), _ptr(tok_slot),
                     _ptr(slot_scale), C.c_int(n), _ptr(y), C.c_int(ldy)])

    def lora_silu(self, rank, xa, split, M, B, rows, tab, tok_slot, slot_scale, n, y, ldy, mid):
        """LoraA::launch with mid: a block per 512 rows of y (256 of mid)."""
        self.launch(f"lora_silu_r{rank}", (-(-rows // 512), -(-n // 8)), 256, 0,
                    [_ptr(xa), C.c_int(split), C.c_int(M), _ptr(B), C.c_int(rows), _ptr(tab), _ptr(tok_slot),
                     _ptr(slot_scale), C.c_int(n), _ptr(y), C.c_int(ldy), _ptr(mid)])

    # ------------------------------------------------------------------------------------------ sampler
    def sample_rows(self, logits, out_rows, tok_slot, ids, row_first, seen, outs, params, qtok, qn, qid, qp, out_tok,
                    out_acc, n_out):
        """Step::sample's launch (src/cuda/core.rs:982-999): one block of 1024 threads per logit row; the vocabulary is
        the module's compile-time VOCAB."""
        self.launch("sample_rows", (n_out,), 1024, 0,
                    [_ptr(logits), _ptr(out_rows), _ptr(tok_slot), _ptr(ids), _ptr(row_first), _ptr(seen), _ptr(outs),
                     _ptr(params), _ptr(qtok), _ptr(qn), _ptr(qid), _ptr(qp), _ptr(out_tok), _ptr(out_acc)])

    def draft_sample(self, logits, width, ld, head_ids, out_rows, tok_slot, seen, outs, params, drafts, qtok, qn, qid,
                     qp, n_out):
        """Step::draft_sample's launch (src/cuda/core.rs:1052-1071)."""
        self.launch("draft_sample", (n_out,), 1024, 0,
                    [_ptr(logits), C.c_int(width), C.c_int(ld), _ptr(head_ids), _ptr(out_rows), _ptr(tok_slot),
                     _ptr(seen), _ptr(outs), _ptr(params), _ptr(drafts), _ptr(qtok), _ptr(qn), _ptr(qid), _ptr(qp)])

    # ------------------------------------------------------------------------------------------ attention
    def attn_prep(self, part, splits, n, q_norm, k_norm, inv_freq, qscale, q, out, kc, vc, ks, vs, tok_slot, tok_pos,
                  cap):
        """src/cuda/qwen/attn.rs:285-302."""
        self.launch("attn_prep", (n,), 32 * (R.NH + 2 * R.NKV), 0, [
            _ptr(part), C.c_int(splits), C.c_int(n), _ptr(q_norm), _ptr(k_norm), _ptr(inv_freq), C.c_float(qscale),
            _ptr(q), _ptr(out), _ptr(kc), _ptr(vc), _ptr(ks), _ptr(vs), _ptr(tok_slot), _ptr(tok_pos), C.c_int(cap)])

    @staticmethod
    def dec_splits(dec_max_pos):
        """Attn::splits (src/cuda/qwen/attn.rs:256-264)."""
        v = -(-(dec_max_pos + 1) // R.KPS)
        p = 1
        while p < v:
            p *= 2
        return min(p, R.DSPLITS)

    def attn_decode(self, q, kc, vc, ks, vs, st, dev, cap, part_ml, part_acc, out):
        """attn_mq{rt} + attn_combine as Attn::run launches them (src/cuda/qwen/attn.rs:303-336). st: the host
        counts of build_step; dev: its device arrays."""
        z = self.dec_splits(st["dec_max_pos"])
        rt = -(-(st["dmax"] * R.GROUP) // 16)
        smem = rt * 16 * (R.HD + 8) * 2
        self.launch(f"attn_mq{rt}", (st["ndseg"], R.NKV, z), 32 * rt, smem, [
            _ptr(q), _ptr(kc), _ptr(vc), _ptr(ks), _ptr(vs), _ptr(dev["dseg"]), _ptr(dev["dtok"]),
            _ptr(dev["tok_slot"]), _ptr(dev["tok_pos"]), C.c_int(cap), C.c_int(z), _ptr(part_ml), _ptr(part_acc),
            _ptr(out)])
        if z > 1:
            self.launch("attn_combine", (st["ndec"], R.NH, 1), R.HD, 0, [
                _ptr(part_ml), _ptr(part_acc), _ptr(dev["dtok"]), _ptr(dev["dkeys"]), C.c_int(z), _ptr(out)])

    def attn_prefill(self, q, kc, vc, ks, vs, st, dev, cap, part_ml, part_acc, out):
        """attn_prefill + attn_combine_tiles as Attn::run launches them (src/cuda/qwen/attn.rs:266-274,338-368)."""
        ntile = st["ntile"]
        most = 1 << (max(min(128, 256 // ntile), 1).bit_length() - 1)
        want = -(-(st["tile_max_pos"] + 1) // (64 * ntile))
        z = min(1 << (want - 1).bit_length(), most)
        smem = 64 * (R.HD + 8) * 2 + 2 * 2 * 64 * R.HD
        self.launch("attn_prefill", (ntile, R.NKV, z), 128, smem, [
            _ptr(q), _ptr(kc), _ptr(vc), _ptr(ks), _ptr(vs), _ptr(dev["ptile"]), _ptr(dev["tok_slot"]),
            _ptr(dev["tok_pos"]), C.c_int(cap), C.c_int(z), C.c_int(64 * ntile), _ptr(part_ml), _ptr(part_acc),
            _ptr(out)])
        if z > 1:
            self.launch("attn_combine_tiles", (ntile * (64 // R.GROUP), R.NH, 1), R.HD, 0, [
                _ptr(part_ml), _ptr(part_acc), _ptr(dev["ptile"]), _ptr(dev["tok_pos"]), C.c_int(z),
                C.c_int(64 * ntile), _ptr(out)])

    # ------------------------------------------------------------------------------------------ DeltaNet
    def delta(self, part, splits, n, ba, ba_splits, conv_w, a_log, dt_bias, norm_w, mem, sst, meta, cv, o, mix, st,
              dev, which=("conv", "rule", "norm")):
        """DeltaNet::run (src/cuda/qwen/deltanet.rs:109-160)."""
        if "conv" in which:
            self.launch("delta_conv", (R.LQKV // 128, -(-n // 4), 1), 128, 0, [
                _ptr(part), C.c_int(splits), C.c_int(n), _ptr(ba), C.c_int(ba_splits), _ptr(conv_w), _ptr(a_log),
                _ptr(dt_bias), _ptr(mem), C.c_longlong(sst), _ptr(cv), _ptr(dev["tok_slot"]), _ptr(dev["tok_pos"])])
        if "rule" in which:
            self.launch("delta_rule", (R.LVD // 16, R.LV_HEADS, st["segs"]), 64, 0, [
                _ptr(part), C.c_int(splits), C.c_int(n), _ptr(cv), _ptr(mem), C.c_longlong(sst), _ptr(meta), _ptr(o),
                _ptr(dev["seg_start"]), _ptr(dev["seg_len"]), _ptr(dev["seg_slot"]), _ptr(dev["seg_pos0"])])
        if "norm" in which:
            self.launch("delta_norm", (n, R.LV_HEADS // 16, 1), 512, 0, [
                _ptr(part), C.c_int(splits), C.c_int(n), _ptr(norm_w), _ptr(o), _ptr(mix), _ptr(meta),
                _ptr(dev["seg_len"]), _ptr(dev["seg_slot"]), _ptr(dev["seg_pos0"]), C.c_int(st["segs"])])


def upload_step(st: dict, device="cuda") -> dict:
    """The device arrays of a step (Step::upload, src/cuda/core.rs:897-913)."""
    dev = {}
    for k, v in st.items():
        if isinstance(v, np.ndarray):
            buf = torch.zeros(max(v.size, 1) + 8, dtype=torch.int32, device=device)
            if v.size:
                buf[:v.size] = torch.from_numpy(v).to(device)
            dev[k] = buf
    return dev
