"""Host-side mirror of the reference's `Model` for the decode / verify path: holds the layer stack's device tensors,
hands their pointers to the library (qb_model_*), and exposes step / argmax with the reference's argument meaning
(`Engine::step(toks, out)` and `Engine::argmax`, src/engine.rs:106-239). torch only owns device memory here.

`synthetic()` builds the random-init 27B-shape model of the benchmark (there are no checkpoints in this environment):
every int4 matrix gets uniform codes and group scales |N(0, 0.02)| / 7 + 1e-4 rounded to bf16, norms 1 + N(0, 0.02),
embedding N(0, 0.02) bf16. Codes are drawn directly in Marlin's packed form (a uniform random word is a uniform random
tile of codes), so nothing the size of the model ever exists on the host.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import _lib
from ._lib import QbLoraLayer, QbMtp, QbLayer, QbTok, check, lib

H, NH, NKV, HD = 5120, 24, 4, 256
LK_HEADS, LV_HEADS, LKD, LVD = 16, 48, 128, 128
LQKV = 2 * LK_HEADS * LKD + LV_HEADS * LVD
DELTA_IN = LQKV + LV_HEADS * LVD
ATTN_IN = 2 * NH * HD + 2 * NKV * HD
MIX, FF = NH * HD, 17408
CR, KEEP = 32, 16
REP = LK_HEADS * LKD + LV_HEADS * LVD + 2 * LV_HEADS
SLOT_FLOATS = 2 * LV_HEADS * LVD * LKD + 2 * KEEP * REP + CR * LQKV
THETA = 1e7
ROT = 64
LAYER_PATTERN = ("delta", "delta", "delta", "attn")  # three of four layers Gated DeltaNet, every fourth attention


def _p(t):
    return C.c_void_p(t.data_ptr())


def inv_freq() -> torch.Tensor:
    i = torch.arange(ROT // 2, dtype=torch.float64)
    return (1.0 / (THETA ** (2 * i / ROT))).float()


class Marlin:
    """An int4 matrix in Marlin's layout on the device: words int32 [k/16][2n], scales f16 [k/128][n]."""

    def __init__(self, words: torch.Tensor, scales: torch.Tensor):
        self.words, self.scales = words, scales
        self.n, self.k = words.shape[1] // 2, words.shape[0] * 16

    @staticmethod
    def random(n: int, k: int, g: torch.Generator, device="cuda") -> "Marlin":
        words = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 16, 2 * n), generator=g, dtype=torch.int32, device=device)
        sc = (torch.randn(k // 128, n, generator=g, device=device).abs() * (0.02 / 7) + 1e-4)
        return Marlin(words, sc.to(torch.bfloat16).to(torch.float16))

    def bytes(self) -> int:
        return self.words.numel() * 4 + self.scales.numel() * 2


class Model:
    """The layer stack on one device. `layers`: list of dicts of device tensors (see synthetic())."""

    def __init__(self, ctx, layers, embed, final_norm, lm_head: Marlin, vocab_valid, slots, max_ctx):
        self.ctx, self.layers, self.embed, self.final_norm, self.lm_head = ctx, layers, embed, final_norm, lm_head
        self.slots, self.max_ctx, self.vocab_valid = slots, max_ctx, vocab_valid
        # the model's own stream: the legacy default stream cannot be captured into a graph (the reference opens one
        # the same way, src/cuda/core.rs:42-46)
        torch.cuda.synchronize()
        self.stream = torch.cuda.Stream()
        h = C.c_void_p()
        check(lib().qb_model_create(ctx.h, len(layers), slots, max_ctx, lm_head.n, vocab_valid, C.byref(h)),
              "qb_model_create")
        self.h = h
        for i, l in enumerate(layers):
            q = self._layer_struct(l)
            check(lib().qb_model_set_layer(self.h, i, C.byref(q)), f"qb_model_set_layer({i})")
        check(lib().qb_model_set_head(self.h, _p(embed), _p(final_norm), _p(lm_head.words), _p(lm_head.scales)),
              "qb_model_set_head")
        self.mtp = None

    @staticmethod
    def _layer_struct(l):
        q = QbLayer()
        q.kind = 0 if l["kind"] == "delta" else 1
        for name in ("in_proj", "out", "gate_up", "down"):
            setattr(q, name + "_w", l[name].words.data_ptr())
            setattr(q, name + "_s", l[name].scales.data_ptr())
        q.input_norm, q.post_norm = l["input_norm"].data_ptr(), l["post_norm"].data_ptr()
        if l["kind"] == "delta":
            q.in_ba = l["in_ba"].data_ptr()
            for name in ("conv_w", "a_log", "dt_bias", "norm_w", "mem", "meta"):
                setattr(q, name, l[name].data_ptr())
            q.sst = l["sst"]
        else:
            for name in ("q_norm", "k_norm", "inv_freq", "kc", "vc", "ks", "vs"):
                setattr(q, name, l[name].data_ptr())
            q.cap = l["cap"]
        return q

    def set_mtp(self, mtp: dict):
        """mtp: dict(layer=<layer dict>, fc=Marlin 5120 x 10240, pre_e, pre_h, norm, head=Marlin or None, head_valid,
        head_ids=int32 device tensor or None) (Mtp, src/cuda/qwen/mod.rs:648-661)."""
        q = QbMtp()
        q.layer = self._layer_struct(mtp["layer"])
        q.fc_w, q.fc_s = mtp["fc"].words.data_ptr(), mtp["fc"].scales.data_ptr()
        q.pre_e, q.pre_h, q.norm = mtp["pre_e"].data_ptr(), mtp["pre_h"].data_ptr(), mtp["norm"].data_ptr()
        if mtp.get("head") is not None:
            q.head_w, q.head_s = mtp["head"].words.data_ptr(), mtp["head"].scales.data_ptr()
            q.head_rows, q.head_valid = mtp["head"].n, mtp["head_valid"]
            q.head_ids = mtp["head_ids"].data_ptr()
            q.head_zero_points = int(bool(mtp.get("head_zero_points")))
        check(lib().qb_model_set_mtp(self.h, C.byref(q)), "qb_model_set_mtp")
        self.mtp = mtp

    def draft(self, toks, rows, out, k):
        """Engine::draft with greedy rows: k drafts per row of `out`; returns [len(out)][k] token ids (waits)."""
        arr = self._toks(toks)
        r = (C.c_int * len(rows))(*rows)
        o = (C.c_int * max(1, len(out)))(*out)
        res = (C.c_int * max(1, len(out) * k))()
        s = C.c_void_p(self.stream.cuda_stream)
        check(lib().qb_model_draft(self.h, s, arr, len(toks), r, o, len(out), k, res), "qb_model_draft")
        self._n, self._n_out = (len(out) if k > 1 else len(toks)), len(out)
        self._cols = self.mtp["head"].n if self.mtp.get("head") is not None else None
        return [list(res[i * k:(i + 1) * k]) for i in range(len(out))]

    def learn_block(self, block, words, scales16, ids16) -> bool:
        """DraftHead::learn for one 16-row block: host arrays from host.marlin_block and the block's 16 tokens. Returns
        whether the head's valid row count grew."""
        import numpy as np
        w = np.ascontiguousarray(words, dtype=np.uint32)
        sc = np.ascontiguousarray(scales16).view(np.uint16)
        ids = np.ascontiguousarray(ids16, dtype=np.int32)
        grew = C.c_int(0)
        s = C.c_void_p(self.stream.cuda_stream)
        check(lib().qb_model_learn_block(self.h, s, block, w.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p),
                                         ids.ctypes.data_as(C.c_void_p), C.byref(grew)), "qb_model_learn_block")
        return bool(grew.value)

    def learn(self, vocab, toks, stored_words, scales, zeros=None, zero_points=False, group=128) -> bool:
        """DraftHead::learn (src/cuda/qwen/draft.rs:55-68): the tokens a step commits go into the bookkeeping `vocab`
        (host.DraftVocab); every tile of 16 rows that changed is packed from the stored output layer (stored_words u32
        [rows][cols/8] as host.quant_words gives them, scales f32 [rows][cols/group], zeros u8 or None) and written
        into the draft head. Returns whether the head's valid row count grew."""
        import numpy as np
        q = np.ascontiguousarray(stored_words, dtype=np.uint32)
        sc = np.ascontiguousarray(scales, dtype=np.float32)
        z = None if zeros is None else np.ascontiguousarray(zeros, dtype=np.uint8)
        t = np.ascontiguousarray(toks, dtype=np.uint32)
        rows, cols = q.shape[0], q.shape[1] * 8
        grew = C.c_int(0)
        s = C.c_void_p(self.stream.cuda_stream)
        ptr = lambda a: a.ctypes.data_as(C.c_void_p)
        check(lib().qb_model_learn(self.h, s, vocab.h, ptr(t), len(t), ptr(q), ptr(sc), C.c_void_p(0) if z is None else ptr(z),
                                   int(zero_points), rows, cols, int(group), C.byref(grew)), "qb_model_learn")
        return bool(grew.value)

    def graph_stats(self):
        """(graphs held, cap or -1, steps that ran without a graph for want of memory)."""
        a, b, c = C.c_longlong(0), C.c_longlong(0), C.c_longlong(0)
        check(lib().qb_model_graph_stats(self.h, C.byref(a), C.byref(b), C.byref(c)), "qb_model_graph_stats")
        return a.value, b.value, c.value

    def fail_captures(self, n: int):
        check(lib().qb_model_fail_captures(self.h, n), "qb_model_fail_captures")

    def set_adapter(self, i, lora):
        """Layer i's LoRA (LayerLora, src/cuda/qwen/lora.rs:199-205): lora = dict(rank=r, inp=.., out=.., gate_up=..,
        down=..), each product None or dict(a=packed f16 device tensor, a_tiles=.., b=f16 [rows][r] device tensor in the
        product's row order, tab=int32[8] device tensor[, b2=.., tab2=..]); None removes it."""
        if lora is None:
            check(lib().qb_model_set_adapter(self.h, i, None), "qb_model_set_adapter")
            self.layers[i].pop("lora_dev", None)
            return
        q = QbLoraLayer()
        q.rank = lora["rank"]
        for name in ("inp", "out", "gate_up", "down"):
            p = lora.get(name)
            if p is None:
                continue
            f = getattr(q, name)
            f.a, f.a_tiles = p["a"].data_ptr(), p["a_tiles"]
            if p.get("b") is not None:
                f.b, f.tab = p["b"].data_ptr(), p["tab"].data_ptr()
            if p.get("b2") is not None:
                f.b2, f.tab2 = p["b2"].data_ptr(), p["tab2"].data_ptr()
        check(lib().qb_model_set_adapter(self.h, i, C.byref(q)), "qb_model_set_adapter")
        self.layers[i]["lora_dev"] = lora  # keeps the tensors alive

    def set_slot_scale(self, slot, scale):
        """Model::set_adapter for a slot: alpha / r when its request uses the adapter, else 0."""
        check(lib().qb_model_set_slot_scale(self.h, C.c_void_p(self.stream.cuda_stream), slot, float(scale)),
              "qb_model_set_slot_scale")

    def save_kv(self, slot, start, end, out=None) -> np.ndarray:
        """Model::save_kv: the attention layers' caches of positions [start, end) as the reference's byte image
        (into `out`, a uint8 array of that size, e.g. over pinned memory, when given)."""
        n = lib().qb_model_kv_bytes(self.h, start, end)
        out = np.zeros(n, dtype=np.uint8) if out is None else out
        assert out.dtype == np.uint8 and out.size == n and out.flags.c_contiguous
        check(lib().qb_model_save_kv(self.h, C.c_void_p(self.stream.cuda_stream), slot, start, end,
                                     out.ctypes.data_as(C.c_void_p), n), "qb_model_save_kv")
        return out

    def load_kv(self, slot, start, end, data: np.ndarray):
        d = np.ascontiguousarray(data, dtype=np.uint8)
        check(lib().qb_model_load_kv(self.h, C.c_void_p(self.stream.cuda_stream), slot, start, end,
                                     d.ctypes.data_as(C.c_void_p), len(d)), "qb_model_load_kv")

    def save_state(self, slot):
        """Model::save_state: (byte image, the position the DeltaNet states are at)."""
        n = lib().qb_model_state_bytes(self.h)
        out = np.zeros(n, dtype=np.uint8)
        pos = C.c_int(0)
        check(lib().qb_model_save_state(self.h, C.c_void_p(self.stream.cuda_stream), slot,
                                        out.ctypes.data_as(C.c_void_p), n, C.byref(pos)), "qb_model_save_state")
        return out, pos.value

    def load_state(self, slot, data: np.ndarray, pos: int):
        d = np.ascontiguousarray(data, dtype=np.uint8)
        check(lib().qb_model_load_state(self.h, C.c_void_p(self.stream.cuda_stream), slot,
                                        d.ctypes.data_as(C.c_void_p), len(d), pos), "qb_model_load_state")

    def set_outputs(self, slot, words):
        """Step::set_outputs: the set of tokens the slot's request generated (uint32 words over the padded vocabulary)."""
        w = np.ascontiguousarray(words, dtype=np.uint32)
        check(lib().qb_model_set_outputs(self.h, C.c_void_p(self.stream.cuda_stream), slot,
                                         w.ctypes.data_as(C.c_void_p)), "qb_model_set_outputs")

    def sample(self, params):
        """Step::sample: [(token, draft accepted)] per logit row of the last step; params [n_out][8]."""
        p = np.ascontiguousarray(params, dtype=np.float32)
        n = len(p)
        tok, acc = (C.c_int * n)(), (C.c_int * n)()
        check(lib().qb_model_sample(self.h, C.c_void_p(self.stream.cuda_stream), p.ctypes.data_as(C.c_void_p), n, tok,
                                    acc), "qb_model_sample")
        return [(tok[i], bool(acc[i])) for i in range(n)]

    def draft_sampled(self, toks, rows, out, k, sampling, u):
        """Engine::draft with sampled rows: sampling [len(out)][8] (Params::draft_row; temperature <= 0: the argmax),
        u [len(out)][k] draws; returns [len(out)][k] drafts (waits)."""
        arr = self._toks(toks)
        r = (C.c_int * len(rows))(*rows)
        o = (C.c_int * len(out))(*out)
        res = (C.c_int * (len(out) * k))()
        sp = np.ascontiguousarray(sampling, dtype=np.float32)
        uu = np.ascontiguousarray(u, dtype=np.float32)
        assert sp.shape == (len(out), 8) and uu.shape == (len(out), k)
        check(lib().qb_model_draft_sampled(self.h, C.c_void_p(self.stream.cuda_stream), arr, len(toks), r, o, len(out),
                                           k, sp.ctypes.data_as(C.c_void_p), uu.ctypes.data_as(C.c_void_p), res),
              "qb_model_draft_sampled")
        self._n, self._n_out = (len(out) if k > 1 else len(toks)), len(out)
        self._cols = self.mtp["head"].n if self.mtp.get("head") is not None else None
        return [list(res[i * k:(i + 1) * k]) for i in range(len(out))]

    def draft_q(self, slot, t):
        """Step::draft_q: (ids ascending, probabilities, token drawn) kept for the slot's draft at index t."""
        tok, n = C.c_int(0), C.c_int(0)
        ids = np.zeros(1024, dtype=np.int32)
        p = np.zeros(1024, dtype=np.float32)
        check(lib().qb_model_draft_q(self.h, C.c_void_p(self.stream.cuda_stream), slot, t, C.byref(tok), C.byref(n),
                                     ids.ctypes.data_as(C.c_void_p), p.ctypes.data_as(C.c_void_p)),
              "qb_model_draft_q")
        return ids[:n.value].copy(), p[:n.value].copy(), tok.value

    def close(self):
        if getattr(self, "h", None):
            lib().qb_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- Engine::step / Engine::argmax
    @staticmethod
    def _toks(toks):
        arr = (QbTok * len(toks))()
        for i, (tid, slot, pos) in enumerate(toks):
            arr[i].id, arr[i].slot, arr[i].pos = int(tid), int(slot), int(pos)
        return arr

    def step(self, toks, out, marks=None):
        """toks: [(id, slot, pos)], sequences contiguous and in order; out: indices whose logits are wanted; marks
        (optional): per segment the tokens to add to its slot's seen set instead of the segment's own."""
        arr = self._toks(toks)
        o = (C.c_int * max(1, len(out)))(*out)
        s = C.c_void_p(self.stream.cuda_stream)
        if marks is None:
            check(lib().qb_model_step(self.h, s, arr, len(toks), o, len(out)), "qb_model_step")
        else:
            nseg = 1 + sum(1 for i in range(1, len(toks)) if toks[i][1] != toks[i - 1][1])
            if len(marks) != nseg:
                raise ValueError(f"{len(marks)} mark lists for a step of {nseg} segments")
            flat = [int(t) for seg in marks for t in seg]
            at = [0]
            for seg in marks:
                at.append(at[-1] + len(seg))
            mk, ma = (C.c_uint32 * max(1, len(flat)))(*flat), (C.c_int * len(at))(*at)
            check(lib().qb_model_step_marks(self.h, s, arr, len(toks), o, len(out), mk, ma), "qb_model_step_marks")
        self._n, self._n_out, self._cols = len(toks), len(out), None

    def argmax(self, n_out=None):
        n_out = self._n_out if n_out is None else n_out
        res = (C.c_int * max(1, n_out))()
        s = C.c_void_p(self.stream.cuda_stream)
        check(lib().qb_model_argmax(self.h, s, res, n_out), "qb_model_argmax")
        return list(res)[:n_out]

    def use_fused(self, on: bool):
        check(lib().qb_model_use_fused(self.h, int(on)), "qb_model_use_fused")

    def use_fork(self, on: bool):
        check(lib().qb_model_use_fork(self.h, int(on)), "qb_model_use_fork")

    def use_graphs(self, on: bool):
        check(lib().qb_model_use_graphs(self.h, int(on)), "qb_model_use_graphs")

    def logits(self) -> torch.Tensor:
        """f32 [n_out][vocab_rows] of the last step (a copy)."""
        self.stream.synchronize()
        ptr = lib().qb_model_logits(self.h)
        cols = getattr(self, "_cols", None) or self.lm_head.n
        return _device_copy(ptr, (self._n_out, cols), torch.float32)

    def hidden(self) -> torch.Tensor:
        self.stream.synchronize()
        return _device_copy(lib().qb_model_hidden(self.h), (self._n, H), torch.float32)

    def seen(self, slot: int) -> np.ndarray:
        """The seen set of a slot (Step::seen, src/cuda/core.rs:928-931) as a bool per vocabulary row."""
        self.stream.synchronize()
        w = self.lm_head.n // 32
        ptr = lib().qb_model_seen(self.h) + 4 * w * int(slot)
        words = _device_copy(ptr, (w,), torch.int32).cpu().numpy().view(np.uint32)
        return ((words[:, None] >> np.arange(32, dtype=np.uint32)) & 1).astype(bool).reshape(-1)

    def xn(self) -> torch.Tensor:
        self.stream.synchronize()
        return _device_copy(lib().qb_model_xn(self.h), (self._n, H), torch.float16)

    def run(self):
        """Replays the uploaded step (Graphs::run) without a new upload: the device-resident timing path."""
        check(lib().qb_model_run(self.h, C.c_void_p(self.stream.cuda_stream)), "qb_model_run")

    @property
    def step_kernels(self) -> int:
        return lib().qb_model_step_kernels(self.h)

    @property
    def launches(self) -> int:
        return lib().qb_model_launches(self.h)

    # ---- bytes a step must move (the roofline's numerator)
    def step_bytes(self, positions: int) -> int:
        b = int(self.vocab_valid * H * 0.515625)  # the output layer's rows that count
        for l in self.layers:
            for name in ("in_proj", "out", "gate_up", "down"):
                b += int(l[name].n * l[name].k * 0.515625)
            if l["kind"] == "delta":
                b += 2 * LV_HEADS * H * 2          # in_proj_b / in_proj_a kept in f16
                b += 2 * LV_HEADS * LVD * LKD * 4  # the f32 state, read and written
            else:
                b += NKV * 520 * positions         # int8 keys and values + two f32 scales per position and head
        return b


def _device_copy(ptr: int, shape, dtype) -> torch.Tensor:
    """A torch copy of library-owned device memory."""
    n = int(np.prod(shape))
    out = torch.empty(shape, dtype=dtype, device="cuda")
    from cuda.bindings import runtime as rt
    (err,) = rt.cudaMemcpy(out.data_ptr(), ptr, n * out.element_size(), rt.cudaMemcpyKind.cudaMemcpyDeviceToDevice)
    if int(err) != 0:
        raise RuntimeError(f"cudaMemcpy failed: {err}")
    return out


def synthetic(ctx, nlayers=64, slots=1, max_ctx=32768, vocab=151936, seed=0, device="cuda", position=0,
              pattern=LAYER_PATTERN, mtp=False, draft_rows=0):
    """The random-init 27B-shape hybrid decoder. With position > 0 the caches are filled as if `position` tokens had
    been processed: random int8 keys / values with scales |N(0, 0.05)|, DeltaNet state N(0, 0.01), metadata
    {position, position, 0}."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    cap = (max_ctx + 63) // 64 * 64
    sst = (SLOT_FLOATS + 1023) // 1024 * 1024
    norm = lambda n: 1 + torch.randn(n, generator=g, device=device) * 0.02
    layers = []

    def make_layer(kind):
        l = dict(kind=kind, input_norm=norm(H), post_norm=norm(H),
                 out=Marlin.random(H, MIX, g, device), gate_up=Marlin.random(2 * FF, H, g, device),
                 down=Marlin.random(H, FF, g, device))
        if kind == "delta":
            l["in_proj"] = Marlin.random(DELTA_IN, H, g, device)
            # in_proj_b / in_proj_a stay 16-bit (96 x 5120, fragment order: any order of N(0, 0.02) values is one)
            l["in_ba"] = (torch.randn(2 * LV_HEADS // 16, H // 16, 32, 8, generator=g, device=device) * 0.02).half()
            l["conv_w"] = torch.randn(LQKV, 4, generator=g, device=device) * 0.3
            l["a_log"] = torch.randn(LV_HEADS, generator=g, device=device) * 0.5
            l["dt_bias"] = torch.randn(LV_HEADS, generator=g, device=device) * 0.5
            l["norm_w"] = norm(LVD)
            mem = torch.zeros(slots * sst, device=device)
            meta = torch.tensor([[-1, 0, 0, 0]] * slots, dtype=torch.int32, device=device)
            if position > 0:
                mem.normal_(0, 0.01, generator=g)
                meta = torch.tensor([[position, position, 0, 0]] * slots, dtype=torch.int32, device=device)
            l["mem"], l["meta"], l["sst"] = mem, meta, sst
        else:
            l["in_proj"] = Marlin.random(ATTN_IN, H, g, device)
            l["q_norm"], l["k_norm"] = norm(HD), norm(HD)
            l["inv_freq"] = inv_freq().to(device)
            nb = slots * NKV * cap
            if position > 0:
                l["kc"] = torch.randint(1, 256, (nb * HD,), generator=g, dtype=torch.uint8, device=device)
                l["vc"] = torch.randint(1, 256, (nb * HD,), generator=g, dtype=torch.uint8, device=device)
                l["ks"] = (torch.randn(nb, generator=g, device=device) * 0.05).abs()
                l["vs"] = (torch.randn(nb, generator=g, device=device) * 0.05).abs()
            else:
                l["kc"] = torch.zeros(nb * HD, dtype=torch.uint8, device=device)
                l["vc"] = torch.zeros(nb * HD, dtype=torch.uint8, device=device)
                l["ks"], l["vs"] = torch.zeros(nb, device=device), torch.zeros(nb, device=device)
            l["cap"] = cap
        return l

    for i in range(nlayers):
        layers.append(make_layer(pattern[i % len(pattern)]))
    vocab_rows = (vocab + 255) // 256 * 256
    embed = (torch.randn(vocab, H, generator=g, device=device) * 0.02).to(torch.bfloat16)
    lm_head = Marlin.random(vocab_rows, H, g, device)
    model = Model(ctx, layers, embed, norm(H), lm_head, vocab, slots, max_ctx)
    if mtp:
        # the MTP draft layer: an attention layer of its own, fc over [embedding; hidden], its norms, and (draft_rows > 0)
        # a draft head of that many rows over a random subset of the vocabulary
        d = dict(layer=make_layer("attn"), fc=Marlin.random(H, 2 * H, g, device), pre_e=norm(H), pre_h=norm(H),
                 norm=norm(H), head=None, head_valid=0, head_ids=None)
        if draft_rows:
            rows = (draft_rows + 255) // 256 * 256
            d["head"] = Marlin.random(rows, H, g, device)
            d["head_valid"] = draft_rows
            ids = torch.randperm(vocab, generator=g, device=device)[:rows].to(torch.int32)
            d["head_ids"] = ids
        model.set_mtp(d)
    return model


IMAX = 2 ** 31 - 1


def synthetic_adapter(model, rank=16, seed=5, std=0.05, device="cuda"):
    """A random LoRA over every layer of `model`, laid out as the reference's loader does (lora::load,
    src/cuda/qwen/lora.rs:58-141): the products that read one input share one stacked A (adapted modules in order,
    rows padded to 16), B per stacked product in the product's row order with its table. Adapted here: DeltaNet
    in_proj_qkv and in_proj_a (not in_proj_z, in_proj_b), attention q_proj and v_proj (not k_proj), out_proj,
    gate_proj / up_proj (even layers both, odd layers up_proj only), down_proj. Sets the adapter on the model and keeps
    host copies under layer["lora"] for the CPU oracle."""
    from . import host
    g = np.random.default_rng(seed)
    f16 = lambda a: a.astype(np.float16).astype(np.float32)

    def stack(cols, stacks):
        """stacks: list of (module rows, adapted flags, silu). Returns the shared A and each stack's B / tab."""
        a_rows, offs = [], []
        for rows, flags, _ in stacks:
            o = []
            for f in flags:
                if f:
                    o.append(len(a_rows) * rank)
                    a_rows.append(f16(g.standard_normal((rank, cols)) * std))
                else:
                    o.append(-1)
            offs.append(o)
        A = np.concatenate(a_rows, 0)
        M = (A.shape[0] + 15) // 16 * 16
        A = np.concatenate([A, np.zeros((M - A.shape[0], cols), dtype=np.float32)], 0)
        out = []
        for (rows, flags, silu), o in zip(stacks, offs):
            if all(x < 0 for x in o):
                out.append(None)
                continue
            total = sum(rows)
            B = np.zeros((total, rank), dtype=np.float32)
            at = 0
            for r_, f in zip(rows, flags):
                if f:
                    B[at:at + r_] = f16(g.standard_normal((r_, rank)) * std)
                at += r_
            B = B[host.row_order(total, silu)]
            tab = [IMAX] * 8
            end = 0
            for i, r_ in enumerate(rows):
                end += r_
                if not silu and i < 3:
                    tab[i] = end
            for i in range(4):
                tab[4 + i] = o[i] if i < len(o) else -1
            out.append((B, tab))
        return A, M, out

    def dev(A, M, b, b2=None):
        d = dict(a=torch.from_numpy(host.pack_f16(A)).to(device), a_tiles=M // 16, A=A)
        if b is not None:
            d.update(b=torch.from_numpy(b[0].astype(np.float16)).to(device),
                     tab=torch.tensor(b[1], dtype=torch.int32, device=device), B=b[0], tab_h=b[1])
        if b2 is not None:
            d.update(b2=torch.from_numpy(b2[0].astype(np.float16)).to(device),
                     tab2=torch.tensor(b2[1], dtype=torch.int32, device=device), B2=b2[0], tab2_h=b2[1])
        return d

    for i, l in enumerate(model.layers):
        lo = dict(rank=rank)
        if l["kind"] == "delta":
            A, M, (bi, bb) = stack(H, [([LQKV, DELTA_IN - LQKV], [True, False], False),
                                       ([LV_HEADS, LV_HEADS], [False, True], False)])
            lo["inp"] = dev(A, M, bi, bb)
        else:
            A, M, (bi,) = stack(H, [([NH * HD * 2, NKV * HD, NKV * HD], [True, False, True], False)])
            lo["inp"] = dev(A, M, bi)
        A, M, (bo,) = stack(MIX, [([H], [True], False)])
        lo["out"] = dev(A, M, bo)
        A, M, (bg,) = stack(H, [([FF, FF], [i % 2 == 0, True], True)])
        lo["gate_up"] = dev(A, M, bg)
        A, M, (bd,) = stack(FF, [([H], [True], False)])
        lo["down"] = dev(A, M, bd)
        model.set_adapter(i, lo)
        l["lora"] = lo
