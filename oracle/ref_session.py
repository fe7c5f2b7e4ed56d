"""CPU restatement of the reference's saved-session byte images.

TEST INFRASTRUCTURE ONLY. The images are defined by the reference's host code (pure byte layout, no arithmetic):
Attn::layout / save (src/cuda/qwen/attn.rs:182-214), DeltaNet::saved_bytes / save / load
(src/cuda/qwen/deltanet.rs:181-226) and their concatenation over the layers, MTP layer last, in Model::save_kv /
save_state (src/cuda/qwen/mod.rs:993-1047). The reference holds no fixtures for them; the tests pin the library's images
to this restatement byte for byte and to the round trip save -> load -> identical logits.
Inputs are CPU copies (numpy) of the layer buffers as the reference's kernels lay them out.
"""
from __future__ import annotations

import numpy as np

from . import ref_ops as R

NKV, HD, CONV_K = R.NKV, R.HD, 4


def kv_layer_image(kc, vc, ks, vs, cap, slot, start, end) -> bytes:
    """Attn::layout: per kv head the keys of [start, end), the values in whole blocks of 16 positions, the two scale
    rows. kc / vc: uint8 [slots * 4 * cap * 256]; ks / vs: float32 [slots * 4 * cap]."""
    assert start % 16 == 0 and start <= end <= cap
    n, vl = end - start, (end + 15) // 16 * 16 - start
    out = []
    for g in range(NKV):
        p = (slot * NKV + g) * cap + start
        out += [kc[p * HD:(p + n) * HD].tobytes(), vc[p * HD:(p + vl) * HD].tobytes(), ks[p:p + n].tobytes(),
                vs[p:p + n].tobytes()]
    return b"".join(out)


def kv_image(attn_layers, slot, start, end) -> np.ndarray:
    """Model::save_kv: the attention layers' images in layer order (the MTP's layer last)."""
    return np.frombuffer(b"".join(kv_layer_image(l["kc"], l["vc"], l["ks"], l["vs"], l["cap"], slot, start, end)
                                  for l in attn_layers), dtype=np.uint8)


def delta_layer_image(mem, meta, sst, slot) -> tuple[bytes, int]:
    """DeltaNet::save: the end state's buffer (meta[2]) and the conv ring's rows of positions end - 3 .. end - 1
    (zeros before position 0); returns the image and `end`."""
    end, _, ebuf, _ = (int(v) for v in meta[slot])
    base = slot * sst
    out = [mem[base + ebuf * R.SLOT_STATE: base + (ebuf + 1) * R.SLOT_STATE].tobytes()]
    for j in range(CONV_K - 1):
        q = end - (CONV_K - 1) + j
        if q >= 0:
            o = base + R.SLOT_RING + (q & (R.CR - 1)) * R.LQKV
            out.append(mem[o:o + R.LQKV].tobytes())
        else:
            out.append(bytes(R.LQKV * 4))
    return b"".join(out), end


def state_image(delta_layers, seen_words, slot) -> tuple[np.ndarray, int]:
    """Model::save_state: the DeltaNet layers' images in layer order, then the slot's seen set (little-endian words)."""
    parts, at = [], None
    for l in delta_layers:
        img, end = delta_layer_image(l["mem"], l["meta"], l["sst"], slot)
        assert at is None or at == end
        at = end
        parts.append(img)
    parts.append(np.asarray(seen_words, dtype="<u4").tobytes())
    return np.frombuffer(b"".join(parts), dtype=np.uint8), (at or 0)
