"""The CPU oracles of the rows around the hot path (sampler, LoRA, int8 dense product) held to outputs of the reference's
own kernels on seeded inputs (tests/golden/ref_widened.npz, written on a GPU by tests/golden/make_golden_widened.py):
the pin of those oracles to the reference that needs no GPU at test time."""
import importlib.util
import os

import numpy as np
import pytest

from oracle import ref_ops as R
from oracle import ref_sample as S

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "ref_widened.npz")
F = np.float32


def _gen():
    """The generator's seeded input functions; importing them must not touch a GPU."""
    path = os.path.join(HERE, "golden", "make_golden_widened.py")
    src = open(path).read().split("def bits(mask):")[0].replace("from oracle import ref_cuda  # noqa: E402", "")
    ns = {"__file__": path, "__name__": "golden_widened_inputs"}
    exec(compile(src, path, "exec"), ns)
    return ns


@pytest.fixture(scope="module")
def gold():
    if not os.path.exists(GOLDEN):
        pytest.fail("tests/golden/ref_widened.npz is missing (python tests/golden/make_golden_widened.py on a GPU)")
    return np.load(GOLDEN), _gen()


def test_sampler_oracle_against_reference_kernel(gold):
    """The host definition (src/sample.rs restated) gives the tokens the reference's sample_rows kernel drew; a draw
    may differ only where its uniform number sits within rounding distance of a boundary (margin below 1e-5)."""
    g, ns = gold
    d = ns["sampler_inputs"]()
    near = accepted = 0
    for r, tok, acc in zip(d["rows"], g["sample_tok"], g["sample_acc"]):
        t, a, margin = S.sample_row(d["logits"], d["seen"], d["gen"], r, want_margin=True)
        if (t, a) != (int(tok), bool(acc)):
            assert margin < 1e-5, (r, (t, a), (int(tok), int(acc)), margin)
            near += 1
        accepted += int(acc)
    assert near <= 1 and 0 < accepted < len(d["rows"])


def test_draft_oracle_against_reference_kernel(gold):
    g, ns = gold
    d = ns["sampler_inputs"]()
    for i, r in enumerate(d["drows"]):
        tok, qi, qp, margin = S.draft_draw(d["logits"], d["seen"], d["gen"], r, None, want_margin=True)
        n = int(g["draft_qn"][i])
        assert n == len(qi) and np.array_equal(g["draft_qid"][i][:n], qi)
        np.testing.assert_allclose(g["draft_qp"][i][:n], qp, rtol=2e-5, atol=1e-9)
        assert tok == int(g["draft_tok"][i]) or margin < 1e-5


def test_lora_oracle_against_reference_kernels(gold):
    g, ns = gold
    L = ns["lora_inputs"]()
    sc = L["slot_scale"][L["tok_slot"]]
    B = L["B"].astype(F)
    want = L["y"] + R.lora_delta(L["xa"], B, L["tab"], sc)
    np.testing.assert_allclose(g["lora_add"], want, rtol=1e-5, atol=1e-5)
    idle = np.nonzero(sc == 0)[0]
    assert len(idle) and np.array_equal(g["lora_add"][idle], L["y"][idle])
    mid = R.lora_silu(L["y"], R.lora_delta(L["xa"], B, L["tab_silu"], sc, silu=True)).astype(F)
    got = g["lora_silu"].astype(F)
    assert np.abs(got - mid).max() <= 2 ** -9 * max(1.0, np.abs(mid).max())


def test_int8_oracle_against_reference_kernel(gold):
    g, ns = gold
    I = ns["i8_inputs"]()
    want = I["x"].astype(np.float64) @ R.dequant_i8(I["w"]).astype(np.float64).T
    assert np.abs(g["gemm_i8"] - want).max() < 1e-3 * np.abs(want).max()
