"""The CPU oracle held to (a) outputs of the reference's own kernels on seeded inputs (tests/golden/ref_kernels.npz,
made on a GPU by tests/golden/make_golden.py from oracle/_ref) and (b) independent formulations of the same math."""
import importlib.util
import math
import os

import numpy as np
import pytest
import torch

from oracle import ref_ops as R

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "ref_kernels.npz")
QSCALE = math.log2(math.e) / 16.0


def _inputs():
    spec = importlib.util.spec_from_file_location("make_golden_inputs", os.path.join(HERE, "golden", "make_golden.py"))
    # only the seeded input generator is needed; importing the module must not touch a GPU
    src = open(spec.origin).read()
    ns = {"__file__": spec.origin, "__name__": "golden_inputs"}
    exec(compile(src.split("def main(out):")[0].replace("from oracle import ref_cuda  # noqa: E402", ""), spec.origin, "exec"), ns)
    return ns["inputs"](), ns["SST"]


@pytest.fixture(scope="module")
def gold():
    if not os.path.exists(GOLDEN):
        pytest.fail("tests/golden/ref_kernels.npz is missing (python tests/golden/make_golden.py on a GPU)")
    return np.load(GOLDEN), _inputs()


def f16close(a, b, ulps=2):
    a, b = a.astype(np.float32), b.astype(np.float32)
    return np.abs(a - b) <= ulps * 2.0 ** -10 * np.maximum(np.abs(b), 2.0 ** -14)


def test_norms_against_reference_kernels(gold):
    g, (d, _) = gold
    x, w, parts = d["x"].numpy(), d["w"].numpy(), d["parts"].numpy()
    assert f16close(R.rmsnorm(x, w), g["rmsnorm"]).all()
    h, y = R.add_rmsnorm(x, parts, w)
    assert np.array_equal(h, g["add_h"])
    assert f16close(y, g["add_y"]).all()


def test_attention_against_reference_kernels(gold):
    g, (d, _) = gold
    n, cap = d["n"], d["cap"]
    st = R.build_step(d["toks"], [0])
    q, gate, k, v = R.attn_prep(d["apart"].numpy(), d["qn"].numpy(), d["kn"].numpy(), R.rope_inv_freq(), QSCALE,
                                st["tok_pos"])
    assert np.allclose(q, g["q"], rtol=1e-4, atol=1e-6) and np.allclose(gate, g["gate"], rtol=1e-5, atol=1e-7)
    kc, vc = d["kc"].numpy().copy(), d["vc"].numpy().copy()
    ks, vs = d["ks"].numpy().copy(), d["vs"].numpy().copy()
    R.kv_store(kc, vc, ks, vs, k, v, st["tok_slot"], st["tok_pos"], cap)
    krows = np.stack([kc.reshape(R.NKV, cap, R.HD)[:, p] for p in st["tok_pos"]])
    dk = np.abs(krows.astype(np.int32) - g["k_rows"].astype(np.int32))
    dv = np.abs(vc.astype(np.int32) - g["vc_full"].astype(np.int32))
    # codes: identical but for values on a rounding boundary (the oracle norms in f64)
    assert dk.max() <= 1 and (dk > 0).mean() < 2e-3 and dv.max() <= 1 and (dv > 0).mean() < 1e-4
    assert np.allclose(np.stack([ks.reshape(R.NKV, cap)[:, p] for p in st["tok_pos"]]), g["ks_rows"], rtol=1e-5)
    assert np.allclose(np.stack([vs.reshape(R.NKV, cap)[:, p] for p in st["tok_pos"]]), g["vs_rows"], rtol=1e-6)
    # decode over the reference's own cache bytes
    kc2 = d["kc"].numpy().copy(); vc2 = g["vc_full"].copy()
    ks2, vs2 = d["ks"].numpy().copy(), d["vs"].numpy().copy()
    for i, p in enumerate(st["tok_pos"]):
        kc2.reshape(R.NKV, cap, R.HD)[:, p] = g["k_rows"][i]
        ks2.reshape(R.NKV, cap)[:, p] = g["ks_rows"][i]
        vs2.reshape(R.NKV, cap)[:, p] = g["vs_rows"][i]
    out = R.attn_decode(g["q"], g["gate"], kc2, vc2, ks2, vs2, st["tok_slot"], st["tok_pos"], cap)
    assert np.allclose(out, g["attn_out"], rtol=1e-2, atol=2e-3)
    assert np.abs(out - g["attn_out"]).max() < 5e-3 * np.abs(g["attn_out"]).max()


def test_deltanet_against_reference_kernels(gold):
    g, (d, SST) = gold
    st = R.build_step(d["toks"], [0])
    mem, meta = d["mem"].numpy().copy(), d["meta"].numpy().copy()
    cv = R.delta_conv(d["dpart"].numpy(), d["ba"].numpy(), d["conv_w"].numpy(), d["a_log"].numpy(), d["dt_bias"].numpy(),
                      mem, SST, st["tok_slot"], st["tok_pos"])
    assert np.allclose(cv, g["cv"], rtol=2e-4, atol=1e-5)
    out = R.delta_rule(d["dpart"].numpy(), g["cv"], mem, SST, meta, st["seg_start"], st["seg_len"], st["seg_slot"],
                       st["seg_pos0"])
    assert np.allclose(out, g["delta_out"], rtol=1e-3, atol=1e-4)
    mix = R.delta_norm(d["dpart"].numpy(), d["norm_w"].numpy(), g["delta_out"], meta, st["seg_len"], st["seg_slot"],
                       st["seg_pos0"])
    assert np.array_equal(meta, g["meta_after"])
    assert f16close(mix, g["delta_mix"], ulps=4).all()
    eb = int(meta[0, 2])
    state = mem[eb * R.SLOT_STATE:(eb + 1) * R.SLOT_STATE].reshape(R.LV_HEADS, R.LVD, R.LKD)[[0, 17, 30, 47]]
    assert np.abs(state - g["state_heads"]).max() < 1e-4   # the benchmark's f32-state tolerance
    ring = np.stack([mem[R.SLOT_RING + (p & (R.CR - 1)) * R.LQKV:][:R.LQKV] for p in st["tok_pos"]])
    assert np.array_equal(ring, g["ring_rows"])


def test_dense_product_against_reference_kernel(gold):
    g, (d, _) = gold
    want = R.dense_gemm(d["xd"].numpy(), d["wd"].numpy().astype(np.float16))
    assert np.allclose(want, g["gemm_f16"], rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------------------- independent formulations

def test_delta_rule_matches_the_textbook_recurrence():
    """S <- e S; delta = (v - S^T k) beta; S += k delta^T; o = S^T q (the gated delta rule as published), against the
    one-pass form the kernels use."""
    g = torch.Generator().manual_seed(7)
    n = 6
    S0 = torch.randn(R.LV_HEADS, R.LVD, R.LKD, generator=g, dtype=torch.float64) * 0.01
    q = torch.nn.functional.normalize(torch.randn(n, R.LV_HEADS, R.LKD, generator=g, dtype=torch.float64), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(n, R.LV_HEADS, R.LKD, generator=g, dtype=torch.float64), dim=-1)
    v = torch.randn(n, R.LV_HEADS, R.LVD, generator=g, dtype=torch.float64)
    e = torch.rand(n, R.LV_HEADS, generator=g, dtype=torch.float64)
    b = torch.rand(n, R.LV_HEADS, generator=g, dtype=torch.float64)
    S, Sn = S0.clone(), S0.numpy().copy()
    for t in range(n):
        S = e[t][:, None, None] * S
        delta = (v[t] - torch.einsum("hvk,hk->hv", S, k[t])) * b[t][:, None]
        S = S + delta[:, :, None] * k[t][:, None, :]
        o = torch.einsum("hvk,hk->hv", S, q[t])
        Sn, on = R._rule_token(Sn, k[t].numpy(), v[t].numpy(), e[t].numpy(), b[t].numpy(), q[t].numpy())
        assert np.allclose(on, o.numpy(), rtol=1e-10, atol=1e-12)
    assert np.allclose(Sn, S.numpy(), rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("dims", [(2, 4, 16, 16), (1, 2, 128, 128)])
def test_chunked_delta_rule_matches_the_token_recurrence(dims):
    """The design of the reference's own unit test of its chunked form (chunked_matches_tokens, src/mlx/delta.rs:194-240):
    two chunks of 64 tokens, keys and queries of unit length shared by the value heads of a key head, log decays in
    (-0.5, 0), beta in (0, 1), a state in (-1, 1); the chunked (WY) form the prompt scan uses and the token recurrence
    must agree to 1e-4 in f32 arithmetic (the reference's bound) on every output, on the state after the first chunk
    and on the end state, and to rounding in f64."""
    lk, hv, dk, dv = dims
    CH, n = 64, 128
    state = [7]

    def values(shape, lo, hi):  # the test's generator: a 64-bit LCG, 24 bits per value
        out = np.empty(int(np.prod(shape)), dtype=np.float32)
        for i in range(out.size):
            state[0] = (state[0] * 6364136223846793005 + 1442695040888963407) % (1 << 64)
            out[i] = np.float32(lo) + np.float32(hi - lo) * np.float32((state[0] >> 40) / float(1 << 24))
        return out.reshape(shape)

    unit = lambda x: x / np.sqrt((x * x).sum(-1, keepdims=True))
    q1, k1 = unit(values((n, lk, dk), -1, 1)), unit(values((n, lk, dk), -1, 1))
    q, k = np.repeat(q1, hv // lk, axis=1), np.repeat(k1, hv // lk, axis=1)
    v = values((n, hv, dv), -1, 1)
    e = np.exp(values((n, hv), -0.5, 0.0))
    b = values((n, hv), 0.0, 1.0)
    s0 = values((hv, dv, dk), -1, 1)
    for dtype, tol in ((np.float32, 1e-4), (np.float64, 1e-10)):
        S_tok, outs = s0.astype(dtype), []
        at_ch = None
        for t in range(n):
            S_tok, o = R._rule_token(S_tok, k[t].astype(dtype), v[t].astype(dtype), e[t].astype(dtype), b[t].astype(dtype),
                                     q[t].astype(dtype))
            outs.append(o)
            if t + 1 == CH:
                at_ch = S_tok.copy()
        outs = np.stack(outs)
        worst = 0.0
        for h in range(hv):
            S = s0[h]
            for c in range(0, n, CH):
                S, O = R.delta_chunk(S, q[c:c + CH, h], k[c:c + CH, h], v[c:c + CH, h], e[c:c + CH, h], b[c:c + CH, h],
                                     dtype=dtype)
                worst = max(worst, float(np.abs(O - outs[c:c + CH, h]).max()))
                if c == 0:
                    assert np.abs(S - at_ch[h]).max() < tol, "state at CH"
            assert np.abs(S - S_tok[h]).max() < tol, "end states differ"
        assert worst < tol, f"outputs differ by {worst}"


def test_plan_worked_examples():
    """The rollback plan on the cases the reference's comments walk through (kernels/qwen_deltanet.cuh:12-19,62-82)."""
    p = R.plan([100, 95, 1, 0], 100, 5)           # a verify step continuing at `end`
    assert (p["in_"], p["r"], p["ck"], p["wck"], p["cbuf"], p["ebuf"]) == (1, 0, 100, False, 1, 0)
    p = R.plan([105, 100, 0, 0], 103, 5)          # restart after 2 of 4 drafts were accepted
    assert (p["in_"], p["from_"], p["r"], p["wck"], p["cbuf"], p["ebuf"]) == (1, 100, 3, True, 0, 1)
    p = R.plan([-1, 0, 0, 0], 0, 64)              # a new sequence: zeros, checkpoint KEEP before the end
    assert p["zero"] and p["ck"] == 48 and p["wck"]
    p = R.plan([50, 50, 0, 0], 50, 40)            # a long continuation writes its checkpoint
    assert p["ck"] == 74 and p["wck"] and p["cbuf"] == 1 and p["ebuf"] == 0


def test_build_step_verify_example():
    """Step metadata of one 5-row verify step at 32000 (Step::upload, src/cuda/core.rs:835-926)."""
    st = R.build_step([(7, 0, 32000 + i) for i in range(5)], list(range(5)))
    assert st["segs"] == 1 and st["ndec"] == 5 and st["ndseg"] == 1 and st["dmax"] == 5 and st["ntile"] == 0
    assert st["dseg"].tolist() == [0, 5] and st["dkeys"].tolist() == [32005] * 5
    # a segment that crosses a multiple of 2048 keys is cut in two
    st = R.build_step([(7, 0, 2046 + i) for i in range(4)], [0])
    assert st["ndseg"] == 2 and st["dseg"].tolist() == [0, 2, 2, 2] and st["dkeys"].tolist() == [2048, 2048, 2050, 2050]
    # long segments become prompt tiles
    st = R.build_step([(7, 0, i) for i in range(25)], [24])
    assert st["ndec"] == 0 and st["ntile"] == 3


def test_kv_quant_and_attention_against_float_math():
    g = torch.Generator().manual_seed(9)
    v = torch.randn(4, R.HD, generator=g).numpy()
    codes, scale = R.kv_quant(v)
    assert codes.min() >= 1 and codes.max() == 255 or codes.min() == 1
    assert np.abs((codes.astype(np.float32) - 128) * scale[:, None] - v).max() <= scale.max() * 0.5001
    # attention over a dequantised cache equals softmax(q k^T / 16) v
    cap, npos = 64, 40
    kc = torch.randint(1, 256, (R.NKV * cap * R.HD,), generator=g, dtype=torch.uint8).numpy()
    vc = torch.randint(1, 256, (R.NKV * cap * R.HD,), generator=g, dtype=torch.uint8).numpy()
    ks = (torch.rand(R.NKV * cap, generator=g) * 0.05).numpy()
    vs = (torch.rand(R.NKV * cap, generator=g) * 0.05).numpy()
    q = (torch.randn(1, R.NH, R.HD, generator=g)).numpy()
    gate = np.ones((1, R.MIX), dtype=np.float32)
    out = R.attn_decode(q * QSCALE, gate, kc, vc, ks, vs, np.array([0]), np.array([npos - 1]), cap, emulate_f16=False)
    for h in (0, 7, 23):
        gkv = h // R.GROUP
        K = R.cache_keys(kc, 0, gkv, cap, npos) * ks[gkv * cap:gkv * cap + npos, None]
        V = R.cache_values(vc, 0, gkv, cap, npos) * vs[gkv * cap:gkv * cap + npos, None]
        s = (K @ q[0, h]) / 16.0
        p = np.exp(s - s.max()); p /= p.sum()
        assert np.allclose(out[0, h * R.HD:(h + 1) * R.HD], p @ V, rtol=1e-5, atol=1e-6)


def test_threaded_dequant_equals_the_numpy_restatement():
    """cpu_step.dequant_marlin (torch, threaded) against ref_ops.unpack_marlin + ref_ops.dequant on the same buffers."""
    from oracle import cpu_step
    g = np.random.default_rng(8)
    words = g.integers(0, 2 ** 32, (512 // 16, 2 * 256), dtype=np.uint64).astype(np.uint32)
    scales = (np.abs(g.standard_normal((512 // 128, 256))) * 0.01 + 1e-4).astype(np.float16)
    q, s = R.unpack_marlin(words, scales)
    assert np.array_equal(cpu_step.dequant_marlin(words, scales).numpy(), R.dequant(q, s).astype(np.float32))
