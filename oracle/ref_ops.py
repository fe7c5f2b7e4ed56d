"""CPU oracle of the decode / verify hot path of hellerchr/qwenny (27B build).

TEST INFRASTRUCTURE ONLY: this module restates, in numpy, what the reference's CUDA kernels and host packers
compute, so that the CUDA library can be checked against it. Nothing in the product imports it; only tests/, the
smoke check and the benchmark's CPU-baseline leg do.

Pinning: the reference ships no golden vectors for any kernel on this path (its numeric checks need external
checkpoints), so this restatement is pinned the other way round: the reference's own kernels, compiled unmodified
from its sources (oracle/build_ref.py -> oracle/_ref/), are run on the GPU next to it on the same seeded inputs
(tests/test_gpu_reference_*.py), and the fixtures under tests/golden/ hold outputs of those runs.

Each function cites the reference file:line it follows (paths inside the reference project).
"""
from __future__ import annotations

import numpy as np

# ---------------------------------------------------------------------------------------------------------------
# Model constants of the 27B build: kernels/qwen.cu:8-35 (QWEN_27B), kernels/qwen_deltanet.cuh:21-34
H = 5120
NH, NKV, HD, ROT = 24, 4, 256, 64
GROUP = NH // NKV
QG_ROWS = 2 * NH * HD
ATTN_IN = QG_ROWS + 2 * NKV * HD
LK_HEADS, LV_HEADS, LKD, LVD = 16, 48, 128, 128
LQKV = 2 * LK_HEADS * LKD + LV_HEADS * LVD
DELTA_IN = LQKV + LV_HEADS * LVD
CONV_K = 4
MIX = NH * HD
FF = 17408
EPS = 1e-6
CR, KEEP, META = 32, 16, 4
REP = LK_HEADS * LKD + LV_HEADS * LVD + 2 * LV_HEADS
SLOT_STATE = LV_HEADS * LVD * LKD
SLOT_BANK = KEEP * REP
SLOT_RING = 2 * SLOT_STATE + 2 * SLOT_BANK
SLOT_FLOATS = SLOT_RING + CR * LQKV
CVW = LQKV + 2 * LV_HEADS
QG = 128  # quantization group (src/cuda/core.rs:29)
KV_OFF = 1152.0
KPS, DSPLITS = 32, 128
THETA = 1e7  # src/cuda/qwen/attn.rs:21


# ---------------------------------------------------------------------------------------------------------------
# Weight layouts (host packers of src/cuda/core.rs)

def row_order(rows: int, silu: bool) -> np.ndarray:
    """Packed row i holds checkpoint row order[i]; SwiGLU matrices interleave 8 gate rows with their 8 up rows per
    16-row block (src/cuda/core.rs:106-114)."""
    i = np.arange(rows)
    if not silu:
        return i
    return (i // 16) * 8 + i % 8 + np.where(i % 16 >= 8, rows // 2, 0)


def _marlin_lane_maps():
    lane = np.arange(32)
    g, t = lane // 4, lane % 4
    x = np.arange(8)
    r = g[:, None] + 8 * ((x[None, :] >> 1) & 1)                      # output row inside the 16-block
    c = 2 * t[:, None] + 8 * (x[None, :] & 1) + (x[None, :] >> 2)      # column inside the k16 step
    return r, c


def pack_marlin(q: np.ndarray, scales_f16: np.ndarray, order: np.ndarray, zeros: np.ndarray | None = None):
    """q: uint8 [rows][k] stored codes (signed value + 8, 0..15); scales_f16: float16 [rows][k/128]; order: packed
    row -> source row. Returns (words uint32 [k/16][2n], scales float16 [k/128][n]) in Marlin's layout:
    marlin_word src/cuda/core.rs:244-253, pack_marlin :262-311 (word of (k16, c64, lane, blk) at
    k16*2n + (c64*32+lane)*4 + blk; scale of packed row o at gi*n + (o//64)*64 + 8*(o%8) + (o%64)//8)."""
    n, k = len(order), q.shape[1]
    assert n % 64 == 0 and k % 128 == 0
    wp = q[order].astype(np.uint32)                       # [n][k]
    a = wp.reshape(n // 64, 4, 16, k // 16, 16).transpose(3, 0, 1, 2, 4)  # [k16][c64][blk][r][c]
    r, c = _marlin_lane_maps()
    gth = a[:, :, :, r, c]                                # [k16][c64][blk][lane][x]
    words = np.zeros(gth.shape[:-1], dtype=np.uint32)
    for x in range(8):
        words |= gth[..., x] << np.uint32(4 * x)
    words = words.transpose(0, 1, 3, 2).reshape(k // 16, 2 * n)  # [k16][c64][lane][blk]
    o = np.arange(n)
    at = (o // 64) * 64 + 8 * (o % 8) + (o % 64) // 8
    sc = np.zeros((k // QG, n), dtype=np.float16)
    sc[:, at] = scales_f16[order].T
    if zeros is not None:
        # the second table (8 - z) * scale, exact in f16 (marlin_scale, src/cuda/core.rs:255-260; pack_marlin :269-283)
        off = np.zeros((k // QG, n), dtype=np.float16)
        off[:, at] = ((8.0 - zeros[order].astype(np.float32)) * scales_f16[order].astype(np.float32)).astype(np.float16).T
        sc = np.concatenate([sc, off], axis=0)
    return np.ascontiguousarray(words), sc


def marlin_block(q: np.ndarray, scales_f16: np.ndarray, rows16, zeros: np.ndarray | None = None):
    """The host half of Gemm::put_block (src/cuda/core.rs:636-652): the words [k/16][32] (marlin_word, :244-253) and
    scales [tables * k/128][16] (marlin_scale, :255-260) of the 16 stored rows `rows16`."""
    rows16 = np.asarray(rows16)
    k = q.shape[1]
    r, c = _marlin_lane_maps()
    a = q[rows16].astype(np.uint32).reshape(16, k // 16, 16).transpose(1, 0, 2)   # [k16][r][c]
    gth = a[:, r, c]                                                                # [k16][lane][x]
    words = np.zeros(gth.shape[:-1], dtype=np.uint32)
    for x in range(8):
        words |= gth[..., x] << np.uint32(4 * x)
    sc = np.ascontiguousarray(scales_f16[rows16].T.astype(np.float16))             # [groups][16]
    if zeros is not None:
        off = ((8.0 - zeros[rows16].astype(np.float32)) * scales_f16[rows16].astype(np.float32)).astype(np.float16).T
        sc = np.concatenate([sc, off], axis=0)
    return words, sc


def put_block(B: np.ndarray, S: np.ndarray, words: np.ndarray, sc: np.ndarray, block: int):
    """marlin_put_block (kernels/marlin.cuh:614-622) on host arrays, in place: B uint32 [k/16][2n], S float16
    [tables * k/128][n]; the block's words [k/16][32] and scales [tables * groups][16]."""
    n = B.shape[1] // 2
    c64, blk = block // 4, block % 4
    lane = np.arange(32)
    B[:, (c64 * 32 + lane) * 4 + blk] = words
    c = blk * 16 + np.arange(16)
    S[:sc.shape[0], c64 * 64 + 8 * (c % 8) + c // 8] = sc


def unpack_marlin(words: np.ndarray, sc: np.ndarray):
    """Inverse of pack_marlin for the identity order: (codes uint8 [n][k], scales float16 [n][k/128])."""
    k16, n2 = words.shape
    n, k = n2 // 2, k16 * 16
    w = words.reshape(k16, n // 64, 32, 4).transpose(0, 1, 3, 2)     # [k16][c64][blk][lane]
    r, c = _marlin_lane_maps()
    # (lane, nibble) -> (row, col) of the 16 x 16 block is a bijection: gather through its inverse
    inv = np.zeros(256, dtype=np.int64)
    inv[(r * 16 + c).reshape(-1)] = np.arange(256)
    nib = np.stack([((w >> np.uint32(4 * x)) & 15).astype(np.uint8) for x in range(8)], axis=-1)  # [..][lane][x]
    a = nib.reshape(k16, n // 64, 4, 256)[..., inv].reshape(k16, n // 64, 4, 16, 16)
    q = a.transpose(1, 2, 3, 0, 4).reshape(n, k)
    o = np.arange(n)
    at = (o // 64) * 64 + 8 * (o % 8) + (o % 64) // 8
    return q, np.ascontiguousarray(sc[:, at].T)


def dequant_z(q: np.ndarray, scales_f16: np.ndarray, offsets_f16: np.ndarray) -> np.ndarray:
    """With zero points: w = f16((q - 8) * scale + (8 - z) * scale), the fused multiply-add rounded once (scale_z,
    kernels/marlin.cuh:126-133); offsets_f16 [rows][k/128] is the second table."""
    s = np.repeat(scales_f16.astype(np.float64), QG, axis=1)
    o = np.repeat(offsets_f16.astype(np.float64), QG, axis=1)
    return ((q.astype(np.float64) - 8.0) * s + o).astype(np.float16)


def dequant(q: np.ndarray, scales_f16: np.ndarray) -> np.ndarray:
    """w = f16((q - 8) * f16 scale), one rounding, as marlin::dequant + scale (kernels/marlin.cuh:100-124)."""
    s = np.repeat(scales_f16.astype(np.float32), QG, axis=1)
    return ((q.astype(np.float32) - 8.0) * s).astype(np.float16)


def frag_map():
    """(row, col) of a0..a7 of the mma A fragment per lane (src/cuda/core.rs:222-227)."""
    lane = np.arange(32)
    g, t = lane // 4, lane % 4
    rows = np.stack([g, g, g + 8, g + 8, g, g, g + 8, g + 8], 1)
    cols = np.stack([2 * t, 2 * t + 1, 2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9, 2 * t + 8, 2 * t + 9], 1)
    return rows, cols


def pack_f16(w: np.ndarray, order: np.ndarray | None = None) -> np.ndarray:
    """Dense f16 matrix [rows][cols] -> tiles of 16 rows in mma A-fragment order, float16 [tiles][cols/16][32][8]
    (pack, src/cuda/core.rs:337-391, f16 branch)."""
    rows, cols = w.shape
    if order is not None:
        w = w[order]
    a = w.astype(np.float16).reshape(rows // 16, 16, cols // 16, 16).transpose(0, 2, 1, 3)  # [tile][k16][r][c]
    r, c = frag_map()
    return np.ascontiguousarray(a[:, :, r, c])


def split_for(tiles: int, cols: int, bits: int, kd: int) -> int:
    """Split-K factor of the dense decode products (src/cuda/core.rs:393-398)."""
    units = 1024
    stage_cols = 2048 // bits
    chunks = cols // stage_cols
    want = max(-(-units // tiles), -(-cols // kd))
    for d in range(1, chunks + 1):
        if chunks % d == 0 and d >= want:
            return d
    return chunks


def embed_q8(table_u8: np.ndarray, scales: np.ndarray, ids) -> np.ndarray:
    """embed_q8 (kernels/qwen.cu:85-98): row ids[t] of an int8 table as stored, (E - 128) * the scale of its 128
    columns, in f32."""
    rows = table_u8[np.asarray(ids)].astype(np.int32) - 128
    return (rows.astype(np.float32) * np.repeat(scales[np.asarray(ids)].astype(np.float32), 128, axis=1)).astype(np.float32)


# ---------------------------------------------------------------------------------------------------------------
# Matrix products

def silu(x):
    return x / (1.0 + np.exp(-x))


def ordered_u32(v: np.ndarray) -> np.ndarray:
    """kernels/common.cuh:60-63."""
    u = v.astype(np.float32).view(np.uint32)
    return np.where(u & 0x80000000, ~u, u | 0x80000000).astype(np.uint32)


def argmax_keys(logits: np.ndarray, n_valid: int) -> np.ndarray:
    """Per row max of (ordered(v) << 32 | ~index) over the first n_valid outputs (kernels/gemm.cuh:71-74,
    kernels/marlin.cuh:499-517)."""
    v = logits[:, :n_valid]
    key = (ordered_u32(v).astype(np.uint64) << np.uint64(32)) | (np.uint64(0xFFFFFFFF) - np.arange(n_valid, dtype=np.uint64))
    return key.max(axis=1)


def key_token(keys: np.ndarray) -> np.ndarray:
    """Token of an argmax key (src/cuda/core.rs:1100-1103: !low word)."""
    return (np.uint64(0xFFFFFFFF) - (keys & np.uint64(0xFFFFFFFF))).astype(np.int64)


def marlin_gemm(x_f16: np.ndarray, w_f16: np.ndarray, epi: str = "plain", n_valid: int | None = None):
    """Y = X . W^T with W the dequantised matrix in PACKED row order, f32 accumulation (kernels/marlin.cuh:171-582).
    plain: f32 [m][n]; silu: f16 [m][n/2] = silu(gate) * up with gate = packed rows 16p..16p+7, up = 16p+8..16p+15
    (:472-498); argmax: (f32 [m][n], u64 keys)."""
    y = x_f16.astype(np.float64) @ w_f16.astype(np.float64).T
    y = y.astype(np.float32)
    if epi == "plain":
        return y
    if epi == "silu":
        m, n = y.shape
        b = y.reshape(m, n // 16, 2, 8)
        return (silu(b[:, :, 0, :]) * b[:, :, 1, :]).reshape(m, n // 2).astype(np.float16)
    if epi == "argmax":
        return y, argmax_keys(y, y.shape[1] if n_valid is None else n_valid)
    raise ValueError(epi)


def dense_gemm(x_f16: np.ndarray, w_f16: np.ndarray) -> np.ndarray:
    """gemm_dec<16,1,EPI_PLAIN> summed over its splits (kernels/gemm.cuh:222-304): Y [m][rows] f32."""
    return (x_f16.astype(np.float64) @ w_f16.astype(np.float64).T).astype(np.float32)


# ---------------------------------------------------------------------------------------------------------------
# Embedding and norms

def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16, returned as float32."""
    u = x.astype(np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def embed(table_bf16_as_f32: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """kernels/dense.cuh:6-11."""
    return table_bf16_as_f32[ids].astype(np.float32)


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float = EPS) -> np.ndarray:
    """y = w * x / rms(x) -> f16 (kernels/dense.cuh:14-26); w is the pre-biased 1 + weight."""
    x = x.astype(np.float32)
    r = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps)
    return (w * (x * r.astype(np.float32))).astype(np.float16)


def add_rmsnorm(h: np.ndarray, parts: np.ndarray, w_next: np.ndarray, eps: float = EPS):
    """h += sum of parts [split][n][H]; y = w_next * h / rms(h) (kernels/qwen.cu:57-80). Returns (h, y f16)."""
    h = h.astype(np.float32).copy()
    for s in range(parts.shape[0]):
        h = h + parts[s]
    return h, rmsnorm(h, w_next, eps)


def mtp_in(emb: np.ndarray, h: np.ndarray, rows: np.ndarray, fw: np.ndarray, pre_e: np.ndarray, pre_h: np.ndarray,
           eps: float = EPS) -> np.ndarray:
    """fc's input of an MTP step (mtp_in, kernels/qwen.cu:100-133): y[t] = [pre_e * e / rms(e); pre_h * g / rms(g)] f16,
    e = emb[t], g = fw * h[rows[t]] / rms(h[rows[t]])."""
    def unit(x):
        x = x.astype(np.float32)
        return x * (1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps)).astype(np.float32)
    e = emb.astype(np.float32)
    g = (fw * unit(h[rows])).astype(np.float32)
    return np.concatenate([pre_e * unit(e), pre_h * unit(g)], axis=-1).astype(np.float16)


# ---------------------------------------------------------------------------------------------------------------
# Attention: cache layout, prep, decode

def kslot(d: np.ndarray) -> np.ndarray:
    """Byte of dim d inside a 256-byte key row (kernels/attn.cuh:23-29)."""
    d = np.asarray(d)
    b, w = d >> 6, d & 15
    t4, e = (w & 7) >> 1, (w & 1) | ((w >> 3) << 1)
    return b * 64 + t4 * 16 + ((d & 63) >> 4) * 4 + e


def vslot(pos: np.ndarray, d: np.ndarray) -> np.ndarray:
    """Byte of (position, dim) inside a head's values (kernels/attn.cuh:30-37)."""
    pos, d = np.asarray(pos), np.asarray(d)
    j = pos & 15
    t4, e = (j & 7) >> 1, (j & 1) | ((j >> 3) << 1)
    return ((pos >> 4).astype(np.int64) * HD + d) * 16 + t4 * 4 + e


def kv_quant(v: np.ndarray):
    """One head vector [.., HD] f32 -> (codes uint8 = round(v * 127 / max) + 128, scale = max / 127)
    (kv_store, kernels/attn.cuh:50-64; __float2int_rn is round-half-even)."""
    v = v.astype(np.float32)
    mx = np.abs(v).max(-1, keepdims=True)
    inv = np.where(mx > 0, np.float32(127.0) / np.where(mx > 0, mx, 1), np.float32(0)).astype(np.float32)
    codes = (np.rint(v * inv).astype(np.int32) + 128).astype(np.uint8)
    return codes, (mx[..., 0] / np.float32(127.0)).astype(np.float32)


def rope_inv_freq() -> np.ndarray:
    """inv_freq[i] = theta^(-2i/ROT), i < ROT/2 (src/cuda/qwen/attn.rs:125)."""
    i = np.arange(ROT // 2, dtype=np.float64)
    return (1.0 / (THETA ** (2 * i / ROT))).astype(np.float32)


def attn_prep(part: np.ndarray, q_norm: np.ndarray, k_norm: np.ndarray, inv_freq: np.ndarray, qscale: float,
              tok_pos: np.ndarray):
    """part [split][n][ATTN_IN] -> q f32 [n][NH][HD] (normed, RoPE'd, scaled), gate f32 [n][MIX] (sigmoid),
    k, v f32 [n][NKV][HD] before quantisation (kernels/qwen.cu:156-202). RoPE pairs dims (d, d + 32), d < 32."""
    x = part.astype(np.float32).sum(0) if part.shape[0] > 1 else part[0].astype(np.float32)
    n = x.shape[0]
    qg = x[:, :QG_ROWS].reshape(n, NH, 2, HD)
    qv, gate = qg[:, :, 0], qg[:, :, 1]
    kv = x[:, QG_ROWS:QG_ROWS + NKV * HD].reshape(n, NKV, HD)
    vv = x[:, QG_ROWS + NKV * HD:].reshape(n, NKV, HD)

    def norm_rope(v, w):
        r = 1.0 / np.sqrt((v.astype(np.float64) ** 2).mean(-1, keepdims=True) + EPS)
        v = (w * (v * r.astype(np.float32))).astype(np.float32)
        ang = tok_pos.astype(np.float32)[:, None] * inv_freq[None, :]
        sn, cs = np.sin(ang)[:, None, :], np.cos(ang)[:, None, :]
        a, b = v[..., :32].copy(), v[..., 32:64].copy()
        v[..., :32] = a * cs - b * sn
        v[..., 32:64] = b * cs + a * sn
        return v

    q = norm_rope(qv.copy(), q_norm) * np.float32(qscale)
    k = norm_rope(kv.copy(), k_norm)
    g = (1.0 / (1.0 + np.exp(-gate.astype(np.float32)))).reshape(n, MIX)
    return q.astype(np.float32), g.astype(np.float32), k, vv.astype(np.float32)


def kv_store(kc, vc, ks, vs, k, v, tok_slot, tok_pos, cap):
    """Write the step's keys and values into the int8 cache in its layout (kv_store, kernels/attn.cuh:50-64).
    kc, vc: uint8 [slots*NKV*cap*HD] flat; ks, vs: f32 [slots*NKV*cap]."""
    d = np.arange(HD)
    kcodes, kscale = kv_quant(k)
    vcodes, vscale = kv_quant(v)
    for t in range(k.shape[0]):
        s, p = int(tok_slot[t]), int(tok_pos[t])
        for g in range(NKV):
            head = (s * NKV + g) * cap * HD
            kc[head + p * HD + kslot(d)] = kcodes[t, g]
            vc[head + vslot(np.full(HD, p), d)] = vcodes[t, g]
            ks[(s * NKV + g) * cap + p] = kscale[t, g]
            vs[(s * NKV + g) * cap + p] = vscale[t, g]


def cache_keys(kc, slot, g, cap, npos):
    """Key codes (signed, q) of a head as int [npos][HD] in dim order."""
    head = (slot * NKV + g) * cap * HD
    rows = kc[head:head + npos * HD].reshape(npos, HD)
    return rows[:, kslot(np.arange(HD))].astype(np.int32) - 128


def cache_values(vc, slot, g, cap, npos):
    head = (slot * NKV + g) * cap * HD
    nb = -(-npos // 16)
    blk = vc[head:head + nb * 16 * HD].reshape(nb, HD, 16)
    j = np.arange(16)
    t4, e = (j & 7) >> 1, (j & 1) | ((j >> 3) << 1)
    v = blk[:, :, t4 * 4 + e]                      # [blk][dim][key j]
    return v.transpose(0, 2, 1).reshape(nb * 16, HD)[:npos].astype(np.int32) - 128


def dchunk(keys: int) -> int:
    """kernels/attn.cuh:45."""
    return max(KPS, ((keys + DSPLITS - 1) // DSPLITS + 15) // 16 * 16)


def attn_decode(q, gate, kc, vc, ks, vs, tok_slot, tok_pos, cap, emulate_f16: bool = True):
    """Decode attention of every token over its slot's cache, base-2 softmax, times the gate
    (attn_mq_tc + attn_combine, kernels/attn.cuh:77-325). q f32 [n][NH][HD] already scaled by log2(e)/16.
    Returns f32 [n][MIX]. With emulate_f16, Q and P*vscale are rounded to f16 as the kernel feeds them to the
    tensor cores (:93-96, :198-216)."""
    n = q.shape[0]
    out = np.zeros((n, MIX), dtype=np.float32)
    # the cache of a (slot, kv head) is decoded once per call, for the longest prefix any of the slot's tokens sees
    longest = {}
    for t in range(n):
        s = int(tok_slot[t])
        longest[s] = max(longest.get(s, 0), int(tok_pos[t]) + 1)
    for s, most in longest.items():
        for g in range(NKV):
            K = cache_keys(kc, s, g, cap, most).astype(np.float64)
            V = cache_values(vc, s, g, cap, most).astype(np.float64)
            base = (s * NKV + g) * cap
            ksc, vsc = ks[base:base + most].astype(np.float64), vs[base:base + most].astype(np.float64)
            for t in range(n):
                if int(tok_slot[t]) != s:
                    continue
                keys = int(tok_pos[t]) + 1
                qh = q[t, g * GROUP:(g + 1) * GROUP]
                qv = qh.astype(np.float16).astype(np.float64) if emulate_f16 else qh.astype(np.float64)
                sc = (K[:keys] @ qv.T) * ksc[:keys, None]          # [keys][GROUP]
                p = np.exp2(sc - sc.max(axis=0, keepdims=True))
                l = p.sum(axis=0)
                pv = p * vsc[:keys, None]
                if emulate_f16:
                    pv = pv.astype(np.float16).astype(np.float64)
                o = pv.T @ V[:keys]                                   # [GROUP][HD]
                for hh in range(GROUP):
                    h = g * GROUP + hh
                    out[t, h * HD:(h + 1) * HD] = (gate[t, h * HD:(h + 1) * HD] * (o[hh] / l[hh])).astype(np.float32)
    return out


# ---------------------------------------------------------------------------------------------------------------
# Gated DeltaNet

def softplus(a):
    return np.where(a > 20.0, a, np.log1p(np.exp(np.minimum(a, 20.0))))


def plan(meta_slot, p0: int, length: int):
    """What a segment's step does with the slot's state (kernels/qwen_deltanet.cuh:62-82). meta_slot = [end, ck,
    ebuf, _]. Returns dict(in_, r, from_, ck, cbuf, ebuf, zero, wck)."""
    end, ck, eb = int(meta_slot[0]), int(meta_slot[1]), int(meta_slot[2])
    p = dict(ck=max(p0, p0 + length - KEEP), r=0, from_=0)
    p["zero"] = p0 == 0 or end < 0
    if p["zero"]:
        p["in_"] = 0
    elif p0 == end:
        p["in_"] = eb
    else:
        p["in_"] = 1 - eb
        p["from_"] = ck
        p["r"] = min(max(p0 - ck, 0), KEEP)
    p["wck"] = p["zero"] or p["r"] > 0 or p["ck"] > p0
    p["cbuf"] = 1 - p["in_"] if p["wck"] else p["in_"]
    p["ebuf"] = 1 - p["cbuf"]
    return p


def delta_conv(part, ba, conv_w, a_log, dt_bias, mem, sst, tok_slot, tok_pos):
    """part [split][n][DELTA_IN], ba [bsplit][n][2*LV_HEADS] -> cv f32 [n][CVW]: causal depthwise conv (k=4) over
    the step's tokens / the slot's ring, SiLU, L2 norm of q and k heads (q also / sqrt(LKD)), then exp(g) and beta
    (kernels/qwen_deltanet.cuh:84-131). mem: flat f32 slot memory, sst floats per slot."""
    x = part.astype(np.float32).sum(0) if part.shape[0] > 1 else part[0].astype(np.float32)
    b = ba.astype(np.float32).sum(0) if ba.shape[0] > 1 else ba[0].astype(np.float32)
    n = x.shape[0]
    cv = np.zeros((n, CVW), dtype=np.float32)
    for t in range(n):
        slot, pos = int(tok_slot[t]), int(tok_pos[t])
        y = np.zeros(LQKV, dtype=np.float32)
        for j in range(CONV_K):
            qpos, tt = pos - (CONV_K - 1) + j, t - (CONV_K - 1) + j
            if qpos < 0:
                continue
            if tt >= 0 and int(tok_slot[tt]) == slot:
                xin = x[tt, :LQKV]
            else:
                base = slot * sst + SLOT_RING + (qpos & (CR - 1)) * LQKV
                xin = mem[base:base + LQKV]
            y = y + conv_w[:, j] * xin
        y = silu(y.astype(np.float32)).astype(np.float32)
        heads = y[:2 * LK_HEADS * LKD].reshape(2 * LK_HEADS, LKD)
        sc = 1.0 / np.sqrt((heads.astype(np.float64) ** 2).sum(-1, keepdims=True) + 1e-6)
        sc[:LK_HEADS] *= 1.0 / np.sqrt(float(LKD))
        y[:2 * LK_HEADS * LKD] = (heads * sc.astype(np.float32)).reshape(-1)
        cv[t, :LQKV] = y
        a = b[t, LV_HEADS:] + dt_bias
        cv[t, LQKV:LQKV + LV_HEADS] = np.exp(-np.exp(a_log) * softplus(a))
        cv[t, LQKV + LV_HEADS:] = 1.0 / (1.0 + np.exp(-b[t, :LV_HEADS]))
    return cv


def _rule_token(S, k, v, e, beta, q=None):
    """One token of the gated delta rule on the state S [LV_HEADS][LVD (v)][LKD (k)]; k, q [LV_HEADS][LKD] (already
    expanded per value head), v [LV_HEADS][LVD], e, beta [LV_HEADS] (kernels/qwen_deltanet.cuh:260-276):
    delta = (v - e S^T k) beta; o = e S^T q + delta (k.q); S = e S + k delta^T."""
    dk = np.einsum("hvk,hk->hv", S, k)
    delta = (v - e[:, None] * dk) * beta[:, None]
    o = None
    if q is not None:
        dq = np.einsum("hvk,hk->hv", S, q)
        kq = (k * q).sum(-1)
        o = e[:, None] * dq + delta * kq[:, None]
    S = e[:, None, None] * S + delta[:, :, None] * k[:, None, :]
    return S, o


def delta_chunk(S, q, k, v, e, beta, dtype=np.float64):
    """One chunk of C tokens of the gated delta rule in the chunked (WY) form the reference states for its MLX backend
    (src/mlx/delta.rs:6-15,85-137), for one value head: S [LVD (v)][LKD (k)], q, k [C][LKD], v [C][LVD], e, beta [C].
    With G_i the cumulative log decay, A_ij = b_i (k_i . k_j) exp(G_i - G_j) (j < i), T = (I + A)^-1:
      R = b (V - gam K S^T);  D = T R;  O = gam Q S^T + P D, P_ij = (q_i . k_j) exp(G_i - G_j) (j <= i);
      S' = gam_C S + D^T (k_j exp(G_C - G_j)).
    Returns (S', O [C][LVD]). Algebraically the token recurrence of _rule_token; sums in another order."""
    S, q, k, v = S.astype(dtype), q.astype(dtype), k.astype(dtype), v.astype(dtype)
    g = np.cumsum(np.log(e.astype(dtype)))
    gam = np.exp(g)
    dec = np.exp(np.minimum(g[:, None] - g[None, :], 0.0))
    C = len(g)
    strict, lower = np.tril(np.ones((C, C), bool), -1), np.tril(np.ones((C, C), bool), 0)
    A = np.where(strict, beta.astype(dtype)[:, None] * (k @ k.T) * dec, 0.0)
    T = np.linalg.inv(np.eye(C) + A)
    R = beta.astype(dtype)[:, None] * (v - gam[:, None] * (k @ S.T))
    D = T @ R
    P = np.where(lower, (q @ k.T) * dec, 0.0)
    O = gam[:, None] * (q @ S.T) + P @ D
    S1 = gam[-1] * S + D.T @ (k * np.exp(g[-1] - g)[:, None])
    return S1, O


def delta_rule(part, cv, mem, sst, meta, seg_start, seg_len, seg_slot, seg_pos0, dtype=np.float64):
    """The gated delta rule over the step's segments with the reference's rollback plan; updates `mem` in place
    (state buffers, replay banks, conv ring) and returns out f32 [n][MIX] (kernels/qwen_deltanet.cuh:172-288).
    `meta` int32 [slots][4] is read, not written (delta_norm writes it)."""
    x = part.astype(np.float32).sum(0) if part.shape[0] > 1 else part[0].astype(np.float32)
    n = cv.shape[0]
    out = np.zeros((n, MIX), dtype=np.float32)
    rep = LV_HEADS // LK_HEADS
    for sg in range(len(seg_start)):
        t0, ln, slot, p0 = int(seg_start[sg]), int(seg_len[sg]), int(seg_slot[sg]), int(seg_pos0[sg])
        pl = plan(meta[slot], p0, ln)
        base = slot * sst

        def sbuf(b):
            return mem[base + b * SLOT_STATE: base + (b + 1) * SLOT_STATE].reshape(LV_HEADS, LVD, LKD)

        def entry(b, pos):
            o = base + 2 * SLOT_STATE + b * SLOT_BANK + (pos % KEEP) * REP
            return mem[o:o + REP]

        S = np.zeros((LV_HEADS, LVD, LKD), dtype=dtype) if pl["zero"] else sbuf(pl["in_"]).astype(dtype)
        for i in range(pl["r"]):
            e = entry(pl["in_"], pl["from_"] + i)
            k = np.repeat(e[:LK_HEADS * LKD].reshape(LK_HEADS, LKD), rep, axis=0).astype(dtype)
            v = e[LK_HEADS * LKD:LK_HEADS * LKD + LV_HEADS * LVD].reshape(LV_HEADS, LVD).astype(dtype)
            ex = e[LK_HEADS * LKD + LV_HEADS * LVD:][:LV_HEADS].astype(dtype)
            be = e[LK_HEADS * LKD + LV_HEADS * LVD + LV_HEADS:][:LV_HEADS].astype(dtype)
            S, _ = _rule_token(S, k, v, ex, be)
        for tk in range(ln):
            row = cv[t0 + tk]
            pos = p0 + tk
            if pl["wck"] and pos == pl["ck"]:
                sbuf(pl["cbuf"])[...] = S.astype(np.float32)
            qh = row[:LK_HEADS * LKD].reshape(LK_HEADS, LKD)
            kh = row[LK_HEADS * LKD:2 * LK_HEADS * LKD].reshape(LK_HEADS, LKD)
            v = row[2 * LK_HEADS * LKD:LQKV].reshape(LV_HEADS, LVD)
            ex, be = row[LQKV:LQKV + LV_HEADS], row[LQKV + LV_HEADS:]
            if pos >= pl["ck"]:
                e = entry(pl["cbuf"], pos)
                e[:LK_HEADS * LKD] = kh.reshape(-1)
                e[LK_HEADS * LKD:LK_HEADS * LKD + LV_HEADS * LVD] = v.reshape(-1)
                e[LK_HEADS * LKD + LV_HEADS * LVD:][:LV_HEADS] = ex
                e[LK_HEADS * LKD + LV_HEADS * LVD + LV_HEADS:][:LV_HEADS] = be
            S, o = _rule_token(S, np.repeat(kh, rep, 0).astype(dtype), v.astype(dtype), ex.astype(dtype),
                               be.astype(dtype), np.repeat(qh, rep, 0).astype(dtype))
            out[t0 + tk] = o.reshape(-1).astype(np.float32)
        sbuf(pl["ebuf"])[...] = S.astype(np.float32)
        m = min(ln, CR)
        for tk in range(ln - m, ln):
            o = base + SLOT_RING + ((p0 + tk) & (CR - 1)) * LQKV
            mem[o:o + LQKV] = x[t0 + tk, :LQKV]
    return out


def delta_norm(part, norm_w, out, meta, seg_len, seg_slot, seg_pos0):
    """y = norm_w * o / rms(o) * silu(z) per value head -> f16 [n][MIX]; then the slots' metadata
    (kernels/qwen_deltanet.cuh:295-315). Updates `meta` in place."""
    x = part.astype(np.float32).sum(0) if part.shape[0] > 1 else part[0].astype(np.float32)
    n = out.shape[0]
    o = out.reshape(n, LV_HEADS, LVD).astype(np.float32)
    z = x[:, LQKV:].reshape(n, LV_HEADS, LVD)
    r = 1.0 / np.sqrt((o.astype(np.float64) ** 2).mean(-1, keepdims=True) + EPS)
    y = norm_w * (o * r.astype(np.float32)) * silu(z)
    for sg in range(len(seg_len)):
        slot, p0, ln = int(seg_slot[sg]), int(seg_pos0[sg]), int(seg_len[sg])
        pl = plan(meta[slot], p0, ln)
        meta[slot, 0], meta[slot, 1], meta[slot, 2] = p0 + ln, pl["ck"], pl["ebuf"]
    return y.reshape(n, MIX).astype(np.float16)


# ---------------------------------------------------------------------------------------------------------------
# Step metadata (Step::upload, src/cuda/core.rs:835-926) for the decode-attention path

def build_step(toks, out_rows, short=8, max_dec=64, ptile=10, cut=16 * DSPLITS, marks=None):
    """toks: list of (id, slot, pos). Returns the dict of host arrays the kernels read (ids, tok_slot, tok_pos,
    seg_*, dtok, dseg, dkeys, ptile, out_rows, mark, mark_at, row_first) and the host-side counts. marks: per segment
    the tokens to add to its slot's seen set (None: the segment's own tokens), core.rs:872-880."""
    n = len(toks)
    seg = [[], [], [], []]
    for i, (_, slot, pos) in enumerate(toks):
        if i > 0 and toks[i - 1][1] == slot:
            assert toks[i - 1][2] + 1 == pos
            seg[1][-1] += 1
        else:
            assert slot not in seg[2]
            seg[0].append(i); seg[1].append(1); seg[2].append(slot); seg[3].append(pos)
    dtok, ptl, dseg, dkeys = [], [], [], []
    for st, ln in zip(seg[0], seg[1]):
        if ln <= short and len(dtok) + ln <= max_dec:
            a = st
            while a < st + ln:
                part = toks[a][2] // cut
                e = a + 1
                while e < st + ln and toks[e][2] // cut == part:
                    e += 1
                dseg += [len(dtok), e - a]
                dtok += list(range(a, e))
                dkeys += [toks[e - 1][2] + 1] * (e - a)
                a = e
        else:
            for o in range(0, ln, ptile):
                ptl += [st + o, min(ln - o, ptile)]
    i32 = lambda v: np.asarray(v, dtype=np.int32)
    pos = lambda t: toks[t][2]
    mark, mark_at = [], [0]
    assert marks is None or len(marks) == len(seg[0])
    for i, (st, ln) in enumerate(zip(seg[0], seg[1])):
        mark += [int(t) for t in marks[i]] if marks is not None else [toks[t][0] for t in range(st, st + ln)]
        mark_at.append(len(mark))
    assert len(mark) <= 2048 + 8 * 64
    row_first = [max(st for st in seg[0] if st <= o) for o in out_rows]  # core.rs:893-894
    return dict(
        mark=i32(mark), mark_at=i32(mark_at), row_first=i32(row_first),
        n=n, n_out=len(out_rows), segs=len(seg[0]), ndec=len(dtok), ntile=len(ptl) // 2, ndseg=len(dseg) // 2,
        dmax=max([dseg[i] for i in range(1, len(dseg), 2)], default=0), max_seg=max(seg[1], default=0),
        dec_max_pos=max([pos(t) for t in dtok], default=0),
        tile_max_pos=max([pos(ptl[i] + ptl[i + 1] - 1) for i in range(0, len(ptl), 2)], default=0),
        ids=i32([t[0] for t in toks]), tok_slot=i32([t[1] for t in toks]), tok_pos=i32([t[2] for t in toks]),
        seg_start=i32(seg[0]), seg_len=i32(seg[1]), seg_slot=i32(seg[2]), seg_pos0=i32(seg[3]),
        dtok=i32(dtok), dseg=i32(dseg), dkeys=i32(dkeys), ptile=i32(ptl), out_rows=i32(out_rows),
    )


# ------------------------------------------------------------------------------------------------- LoRA (unmerged)
def lora_delta(xa_parts, B, tab, scale, silu=False):
    """The delta kernels/lora.cuh adds: xa_parts f32 [split][n][M] summed over the splits in order, B f32 [rows][r]
    (the product's row order), tab as LoraB::tab (src/cuda/qwen/lora.rs:128-141), scale f32 [n] per token (0: none).
    Returns f32 [n][rows]: s_t * B[o] . xa[t][off(o) : off(o) + r], accumulated as one fused multiply-add chain per
    row (here in float64, rounded once: the kernels' f32 chain differs by rounding only)."""
    xa = np.zeros(xa_parts.shape[1:], dtype=np.float32)
    for s in range(xa_parts.shape[0]):
        xa = xa + xa_parts[s]
    rows, r = B.shape
    n = xa.shape[0]
    out = np.zeros((n, rows), dtype=np.float64)
    if silu:  # 16-row tile p: gate rows 8p .. 8p + 7 (module 0), then their up rows (module 1)
        mod = (np.arange(rows) % 16) // 8
    else:
        mod = sum((np.arange(rows) >= tab[i]).astype(np.int64) for i in range(3))
    for m in range(4):
        off = tab[4 + m]
        sel = np.nonzero(mod == m)[0]
        if off < 0 or len(sel) == 0:
            continue
        out[:, sel] = xa[:, off:off + r].astype(np.float64) @ B[sel].astype(np.float64).T
    return (out * np.asarray(scale, dtype=np.float64)[:, None]).astype(np.float32)


def lora_silu(y, delta):
    """lora_silu (kernels/lora.cuh:82-107): mid[t][8p + g] = f16(silu(gate) * up) of y + delta in the SwiGLU row order."""
    v = (y + delta).astype(np.float32)
    n, rows = v.shape
    v = v.reshape(n, rows // 16, 2, 8)
    g, u = v[:, :, 0, :], v[:, :, 1, :]
    return ((g / (1.0 + np.exp(-g.astype(np.float64)))) * u).reshape(n, rows // 2).astype(np.float16)


# ------------------------------------------------------------------------------------------------- int8 dense weights
def quant_i8(w: np.ndarray):
    """The int8 form of a 16-bit matrix (pack with int8, src/cuda/core.rs:349-363): per row and group of 128 columns
    scale = max |w| / 127 (1 for an all-zero group), codes round-half-away(w / scale) clamped to +-127.
    Returns (q int32 [rows][cols], scale f32 [rows][cols / 128])."""
    rows, cols = w.shape
    g = w.astype(np.float32).reshape(rows, cols // 128, 128)
    mx = np.abs(g).max(-1)
    scale = np.where(mx > 0, (mx / np.float32(127.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    v = (g / scale[..., None]).astype(np.float32)
    q = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -127, 127).astype(np.int32)
    return q.reshape(rows, cols), scale


def pack_i8(w: np.ndarray, order: np.ndarray | None = None):
    """Codes q + 128 in tiles of 16 rows, mma A-fragment order, two k16 steps per 16-byte load of a lane (frags_int8,
    src/cuda/core.rs:233-244): uint8 [tiles][cols/32][32 lanes][2][8]; scales f32 [tiles][cols/128][16 rows]."""
    if order is not None:
        w = w[order]
    rows, cols = w.shape
    q, scale = quant_i8(w)
    a = (q + 128).astype(np.uint8).reshape(rows // 16, 16, cols // 32, 2, 16).transpose(0, 2, 3, 1, 4)  # [tile][k32][ks][r][c]
    r, c = frag_map()
    codes = a[:, :, :, r, c]  # [tile][k32][ks][lane][8]
    codes = np.ascontiguousarray(codes.transpose(0, 1, 3, 2, 4))  # [tile][k32][lane][ks][8]
    sc = np.ascontiguousarray(scale.reshape(rows // 16, 16, cols // 128).transpose(0, 2, 1))
    return codes.reshape(rows // 16, 16 * cols), sc


def dequant_i8(w: np.ndarray) -> np.ndarray:
    """The values the int8 product multiplies with: q * scale in float32."""
    q, scale = quant_i8(w)
    rows, cols = w.shape
    return (q.reshape(rows, cols // 128, 128).astype(np.float32) * scale[..., None]).reshape(rows, cols)
