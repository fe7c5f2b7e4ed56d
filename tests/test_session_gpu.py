"""A slot's saved images (qb_model_save_kv / load_kv / save_state / load_state) against the byte layout the
reference's host writes (oracle/ref_session.py), and the property the images exist for: a slot restored from them
continues exactly as the slot they were taken from."""
import numpy as np
import pytest
import torch

from oracle import ref_session as RS
from qwenny_b200 import model as M
from qwenny_b200._lib import QbError

pytestmark = pytest.mark.gpu


def cpu_layers(m, kind):
    ls = list(m.layers) + ([m.mtp["layer"]] if m.mtp else [])
    out = []
    for l in ls:
        if l["kind"] != kind:
            continue
        if kind == "attn":
            out.append(dict(kc=l["kc"].cpu().numpy(), vc=l["vc"].cpu().numpy(), ks=l["ks"].cpu().numpy(),
                            vs=l["vs"].cpu().numpy(), cap=l["cap"]))
        else:
            out.append(dict(mem=l["mem"].cpu().numpy(), meta=l["meta"].cpu().numpy(), sst=l["sst"]))
    return out


def seen_words(m, slot):
    from qwenny_b200._lib import lib
    m.stream.synchronize()
    w = m.lm_head.n // 32
    ptr = lib().qb_model_seen(m.h)
    return M._device_copy(ptr, (m.slots, w), torch.int32).cpu().numpy().view(np.uint32)[slot]


def test_images_and_round_trip(ctx):
    m = M.synthetic(ctx, nlayers=4, slots=2, max_ctx=256, vocab=2000, seed=91,
                    pattern=("delta", "delta", "delta", "attn"), mtp=True)
    seq = [(31 + 17 * i) % 2000 for i in range(80)]
    # a prompt of 37 tokens in one step, then three single-token steps: the slot is at position 40
    m.step([(seq[i], 0, i) for i in range(37)], [36])
    # the MTP layer's cache gets content too: a draft chain after the prompt writes its positions 37 and 38
    m.draft([(m.argmax()[0], 0, 37)], [36], [0], 2)
    for i in range(37, 40):
        m.step([(seq[i], 0, i)], [0])
    torch.cuda.synchronize()

    img = m.save_kv(0, 0, 40)
    want = RS.kv_image(cpu_layers(m, "attn"), 0, 0, 40)
    assert img.shape == want.shape and np.array_equal(img, want)
    part = m.save_kv(0, 16, 37)
    assert np.array_equal(part, RS.kv_image(cpu_layers(m, "attn"), 0, 16, 37))
    assert len(m.save_kv(0, 32, 32)) == 0
    st, pos = m.save_state(0)
    want_st, want_pos = RS.state_image(cpu_layers(m, "delta"), seen_words(m, 0), 0)
    assert pos == 40 == want_pos and np.array_equal(st, want_st)

    with pytest.raises(QbError):
        m.save_kv(0, 8, 40)  # `from` not a multiple of 16
    with pytest.raises(QbError):
        m.load_kv(1, 0, 40, img[:-4])
    with pytest.raises(QbError):
        m.load_state(1, st[:-1], 40)

    # restore into slot 1: in two parts, as a host that swaps a prefix and its tail would
    m.load_kv(1, 0, 32, m.save_kv(0, 0, 32))
    m.load_kv(1, 32, 40, m.save_kv(0, 32, 40))
    m.load_state(1, st, 40)
    assert np.array_equal(m.save_kv(1, 0, 40), img)
    st1, pos1 = m.save_state(1)
    assert pos1 == 40 and np.array_equal(st1, st)
    # both slots continue: one token, then a five-row verify step, then drafts: identical bits
    m.step([(seq[40], 0, 40), (seq[40], 1, 40)], [0, 1])
    lg = m.logits().cpu().numpy()
    assert np.array_equal(lg[0], lg[1])
    toks = [(seq[41 + i], 0, 41 + i) for i in range(5)] + [(seq[41 + i], 1, 41 + i) for i in range(5)]
    m.step(toks, list(range(10)))
    lg = m.logits().cpu().numpy()
    assert np.array_equal(lg[:5], lg[5:])
    got = m.argmax()
    d = m.draft([(got[4], 0, 46), (got[9], 1, 46)], [4, 9], [0, 1], 3)
    assert d[0] == d[1]
    m.close()


def test_state_before_position_three(ctx):
    """A slot at position 2: the ring rows of positions before 0 are zeros in the image and are skipped on loading."""
    m = M.synthetic(ctx, nlayers=2, slots=2, max_ctx=64, vocab=1000, seed=92, pattern=("delta", "attn"))
    m.step([(5, 0, 0), (6, 0, 1)], [1])
    torch.cuda.synchronize()
    st, pos = m.save_state(0)
    want, wp = RS.state_image(cpu_layers(m, "delta"), seen_words(m, 0), 0)
    assert pos == 2 == wp and np.array_equal(st, want)
    m.load_kv(1, 0, 2, m.save_kv(0, 0, 2))
    m.load_state(1, st, 2)
    m.step([(7, 0, 2), (7, 1, 2)], [0, 1])
    lg = m.logits().cpu().numpy()
    assert np.array_equal(lg[0], lg[1])
    m.close()
