"""Thin torch-tensor front end of the C ABI: each function takes CUDA tensors, passes their device pointers and the
current stream to the library, and returns/fills tensors. torch is plumbing here (device memory, streams); all the
arithmetic happens in the library's kernels."""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, lib

EPI = {"plain": 0, "silu": 1, "argmax": 2}


def _p(t):
    """A device tensor's address, a raw device address (int), or null."""
    if t is None:
        return C.c_void_p(0)
    return C.c_void_p(t) if isinstance(t, int) else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Context:
    """The library context of one device (scratch, tickets, error word): Gemm::load of the reference."""

    def __init__(self, device: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("qwenny_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.device = device
        h = C.c_void_p()
        check(lib().qb_create(device, C.byref(h)), "qb_create")
        self.h = h

    def close(self):
        if self.h:
            lib().qb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def sms(self) -> int:
        return lib().qb_sm_count(self.h)

    def device_error(self) -> int:
        return lib().qb_device_error(self.h)

    def wait_probe(self, limit: int = 1 << 12, stream=None):
        """Tests: a block waits `limit` polls on an mbarrier nothing arrives on and records error 99."""
        check(lib().qb_wait_probe(self.h, stream, limit), "qb_wait_probe")

    def set_pdl(self, on: bool):
        check(lib().qb_set_pdl(self.h, int(on)), "qb_set_pdl")

    def early(self, stages=1):
        """How many stages of weights the next skinny products request before they wait for the kernel before them."""
        check(lib().qb_marlin_early(self.h, stages), "qb_marlin_early")

    def tune(self, cg=0, kg=0, nstages=0, ctas=0):
        check(lib().qb_marlin_tune(self.h, cg, kg, nstages, ctas), "qb_marlin_tune")

    # ---- products
    def marlin_gemm(self, x, words, scales, epi="plain", y=None, row0=0, m=None, xrows=None, keys=None,
                    n_valid=None, zp=False):
        """x f16 [rows][k]; words int32 [k/16][2n]; scales f16 [k/128][n]. Returns y (f32 [m][n] or f16 [m][n/2])."""
        k = x.shape[1]
        n = words.shape[1] // 2
        if m is None:
            m = (xrows.numel() if xrows is not None else x.shape[0] - row0)
        if y is None:
            rows = m if xrows is not None else row0 + m
            y = torch.empty((rows, n // 2), dtype=torch.float16, device=x.device) if epi == "silu" else \
                torch.empty((rows, n), dtype=torch.float32, device=x.device)
        fn = lib().qb_marlin_gemm_z if zp else lib().qb_marlin_gemm  # zp: scales followed by the (8 - z) * scale table
        check(fn(self.h, _stream(), _p(x), _p(words), _p(y), _p(scales), m, n, k, row0, EPI[epi],
                 _p(xrows), _p(keys), n if n_valid is None else n_valid), "qb_marlin_gemm")
        return y

    def gemm_f16_plain(self, w_packed, x, n, K, ntiles, kper, y=None, xrows=None):
        """w_packed f16 [ntiles][K/16][32][8]; x f16 [.][K]. Returns y f32 [K/kper][n][ntiles*16] partial products."""
        split = -(-K // kper)
        if y is None:
            y = torch.zeros((split, n, ntiles * 16), dtype=torch.float32, device=x.device)
        check(lib().qb_gemm_f16_plain(self.h, _stream(), _p(w_packed), _p(x), _p(xrows), K, ntiles, n, kper, _p(y),
                                      ntiles * 16), "qb_gemm_f16_plain")
        return y

    # ---- per-token kernels
    def embed(self, table, ids, out, keys, nkeys, n):
        check(lib().qb_embed(self.h, _stream(), _p(table), _p(ids), _p(out), _p(keys), nkeys, n), "qb_embed")

    def embed_q8(self, table, scales, ids, out, keys, nkeys, n):
        check(lib().qb_embed_q8(self.h, _stream(), _p(table), _p(scales), _p(ids), _p(out), _p(keys), nkeys, n),
              "qb_embed_q8")

    def marlin_put_block(self, words, scales, blk_words, blk_scales, block, tables=1):
        """qb_marlin_put_block: the 16-row block `block` of the Marlin matrix (words int32 [k/16][2n], scales f16
        [tables * k/128][n]) from device staging buffers blk_words [k/16][32], blk_scales [tables * k/128][16]."""
        k16s, n = words.shape[0], words.shape[1] // 2
        check(lib().qb_marlin_put_block(self.h, _stream(), _p(words), _p(scales), _p(blk_words), _p(blk_scales), n,
                                        block // 4, block % 4, k16s // 8, tables, k16s), "qb_marlin_put_block")

    def mtp_in(self, emb, h, rows, fw, pre_e, pre_h, y, n, eps=1e-6):
        check(lib().qb_mtp_in(self.h, _stream(), _p(emb), _p(h), _p(rows), _p(fw), _p(pre_e), _p(pre_h), _p(y), eps, n),
              "qb_mtp_in")

    def draft_pick(self, keys, head_ids, n_out, next_ids, chain, chain_ld, t):
        check(lib().qb_draft_pick(self.h, _stream(), _p(keys), _p(head_ids), n_out, _p(next_ids), _p(chain), chain_ld, t),
              "qb_draft_pick")

    def gemm_dec(self, w, scales, wbits, x, K, ntiles, n, kper, epi, y, ldy, keys=None, xrows=None):
        """The dense 16-bit / int8 products (Gemm::run_split); epi: 0 plain, 1 SwiGLU, 2 argmax."""
        check(lib().qb_gemm_dec(self.h, _stream(), _p(w), _p(scales), wbits, _p(x), _p(xrows), K, ntiles, n, kper, epi,
                                _p(y), ldy, _p(keys)), "qb_gemm_dec")

    def lora_add(self, xa, split, M, B, rows, tab, tok_slot, slot_scale, n, y, ldy, rank):
        check(lib().qb_lora_add(self.h, _stream(), _p(xa), split, M, _p(B), rows, _p(tab), _p(tok_slot), _p(slot_scale),
                                n, _p(y), ldy, rank), "qb_lora_add")

    def lora_silu(self, xa, split, M, B, rows, tab, tok_slot, slot_scale, n, y, ldy, mid, rank):
        check(lib().qb_lora_silu(self.h, _stream(), _p(xa), split, M, _p(B), rows, _p(tab), _p(tok_slot),
                                 _p(slot_scale), n, _p(y), ldy, _p(mid), rank), "qb_lora_silu")

    def sample_rows(self, logits, vocab, n_out, out_rows, tok_slot, ids, row_first, seen, outs, params, qtok, qn, qid,
                    qp, out_tok, out_acc, width=None, ld=None):
        """Step::sample (src/cuda/core.rs:977-1005) without the host rows: out_acc -1 marks those."""
        check(lib().qb_sample_rows(self.h, _stream(), _p(logits), width or vocab, ld or vocab, vocab, n_out,
                                   _p(out_rows), _p(tok_slot), _p(ids),
                                   _p(row_first), _p(seen), _p(outs), _p(params), _p(qtok), _p(qn), _p(qid), _p(qp),
                                   _p(out_tok), _p(out_acc)), "qb_sample_rows")

    def draft_sample(self, logits, width, ld, head_ids, vocab, n_out, out_rows, tok_slot, seen, outs, params, drafts,
                     qtok, qn, qid, qp):
        """Step::draft_sample (src/cuda/core.rs:1036-1073)."""
        check(lib().qb_draft_sample(self.h, _stream(), _p(logits), width, ld, _p(head_ids), vocab, n_out, _p(out_rows),
                                    _p(tok_slot), _p(seen), _p(outs), _p(params), _p(drafts), _p(qtok), _p(qn),
                                    _p(qid), _p(qp)), "qb_draft_sample")

    def rmsnorm(self, x, w, y, n, eps=1e-6):
        check(lib().qb_rmsnorm(self.h, _stream(), _p(x), _p(w), _p(y), eps, n), "qb_rmsnorm")

    def add_rmsnorm(self, h, x, splits, n, w_next, y, eps=1e-6):
        check(lib().qb_add_rmsnorm(self.h, _stream(), _p(h), _p(x), splits, n, _p(w_next), _p(y), eps),
              "qb_add_rmsnorm")

    def to_xin(self, x, y, length):
        check(lib().qb_to_xin(self.h, _stream(), _p(x), _p(y), length), "qb_to_xin")

    def sum_parts(self, x, splits, n, ld, y):
        check(lib().qb_sum_parts(self.h, _stream(), _p(x), splits, n, ld, _p(y)), "qb_sum_parts")

    def mark_seen(self, seen, mark, mark_at, seg_slot, seg_pos0, segs, vocab):
        check(lib().qb_mark_seen(self.h, _stream(), _p(seen), _p(mark), _p(mark_at), _p(seg_slot), _p(seg_pos0), segs,
                                 vocab), "qb_mark_seen")

    def marlin_gather(self, x, rows, out, k, n):
        check(lib().qb_marlin_gather(self.h, _stream(), _p(x), _p(rows), _p(out), k // 8, n), "qb_marlin_gather")

    # ---- attention
    def attn_prep(self, part, splits, n, q_norm, k_norm, inv_freq, qscale, q, out, kc, vc, ks, vs, tok_slot, tok_pos,
                  cap):
        check(lib().qb_attn_prep(self.h, _stream(), _p(part), splits, n, _p(q_norm), _p(k_norm), _p(inv_freq), qscale,
                                 _p(q), _p(out), _p(kc), _p(vc), _p(ks), _p(vs), _p(tok_slot), _p(tok_pos), cap),
              "qb_attn_prep")

    def attn_decode(self, q, kc, vc, ks, vs, dev, st, cap, part_ml, part_acc, out, mix=None):
        """dev: the step's device arrays (dseg, dtok, dkeys, tok_slot, tok_pos); st: its host counts."""
        check(lib().qb_attn_decode(self.h, _stream(), _p(q), _p(kc), _p(vc), _p(ks), _p(vs), _p(dev["dseg"]),
                                   _p(dev["dtok"]), _p(dev["dkeys"]), _p(dev["tok_slot"]), _p(dev["tok_pos"]), cap,
                                   st["ndseg"], st["ndec"], st["dmax"], st["dec_max_pos"] + 1, _p(part_ml),
                                   _p(part_acc), _p(out), _p(mix)), "qb_attn_decode")

    def attn_prefill(self, q, kc, vc, ks, vs, dev, st, cap, part_ml, part_acc, out, mix=None):
        """The prompt tiles of a step (dev["ptile"], st["ntile"], st["tile_max_pos"])."""
        check(lib().qb_attn_prefill(self.h, _stream(), _p(q), _p(kc), _p(vc), _p(ks), _p(vs), _p(dev["ptile"]),
                                    _p(dev["tok_slot"]), _p(dev["tok_pos"]), cap, st["ntile"], st["tile_max_pos"] + 1,
                                    _p(part_ml), _p(part_acc), _p(out), _p(mix)), "qb_attn_prefill")

    # ---- DeltaNet
    def delta_conv(self, part, splits, n, ba, ba_splits, conv_w, a_log, dt_bias, mem, sst, cv, dev):
        check(lib().qb_delta_conv(self.h, _stream(), _p(part), splits, n, _p(ba), ba_splits, _p(conv_w), _p(a_log),
                                  _p(dt_bias), _p(mem), sst, _p(cv), _p(dev["tok_slot"]), _p(dev["tok_pos"])),
              "qb_delta_conv")

    def delta_rule(self, part, splits, n, cv, mem, sst, meta, out, dev, segs):
        check(lib().qb_delta_rule(self.h, _stream(), _p(part), splits, n, _p(cv), _p(mem), sst, _p(meta), _p(out),
                                  _p(dev["seg_start"]), _p(dev["seg_len"]), _p(dev["seg_slot"]), _p(dev["seg_pos0"]),
                                  segs), "qb_delta_rule")

    def delta_norm(self, part, splits, n, norm_w, out, y, meta, dev, segs):
        check(lib().qb_delta_norm(self.h, _stream(), _p(part), splits, n, _p(norm_w), _p(out), _p(y), _p(meta),
                                  _p(dev["seg_len"]), _p(dev["seg_slot"]), _p(dev["seg_pos0"]), segs), "qb_delta_norm")

    def delta_mixer(self, part, splits, n, ba, ba_splits, conv_w, a_log, dt_bias, norm_w, mem, sst, meta, out, y, dev,
                    segs):
        check(lib().qb_delta_mixer(self.h, _stream(), _p(part), splits, n, _p(ba), ba_splits, _p(conv_w), _p(a_log),
                                   _p(dt_bias), _p(norm_w), _p(mem), sst, _p(meta), _p(out), _p(y),
                                   _p(dev["seg_start"]), _p(dev["seg_len"]), _p(dev["seg_slot"]), _p(dev["seg_pos0"]),
                                   segs), "qb_delta_mixer")
