"""Greedy tokens over 256 verify steps (the reference's speccheck, src/checks.rs:892-937, stretched to the benchmark's
256 steps): steps of 1 + 4 drafts, some drafts right, then a wrong one, restarting inside the step, must give exactly
the tokens of one token per step; and the CPU oracle of the full path, fed the same steps, must pick the same greedy
token in every row unless its own two best logits are within 1e-3 of each other. Also here: the step-graph cache's
behaviour when a capture finds no memory, and a LoRA adapter swapped at run time."""
import numpy as np
import pytest
import torch

from oracle import cpu_step
from qwenny_b200 import model as M

pytestmark = pytest.mark.gpu
VOCAB = 2000
STEPS = 256


def verify_run(m, slot, reference, first_tok, pos0, k=4, steps=STEPS, on_step=None):
    """speccheck's run: every step feeds the last token and k drafts, of which the first `step % (k + 1)` are the
    reference's tokens and the rest wrong ones; accepted tokens are appended, the first mismatch ends the step."""
    out = [first_tok]
    for step in range(steps):
        pos = pos0 + len(out) - 1
        good = step % (k + 1)
        d = [reference[len(out) + j] if j < good and len(out) + j < len(reference) else 7 + j for j in range(k)]
        toks = [(t, slot, pos + j) for j, t in enumerate([out[-1]] + d)]
        m.step(toks, list(range(len(toks))))
        am = m.argmax()
        if on_step:
            on_step(step, toks, am)
        for j, t in enumerate(am):
            out.append(t)
            if j >= len(d) or d[j] != t:
                break
    return out


def test_256_verify_steps_give_the_tokens_of_one_token_per_step(ctx):
    """Eight full-width layers [D, D, D, A] x 2, two slots with the same prompt: slot 0 decodes one token per step, slot 1
    runs 256 verify steps of 5 rows. Identical tokens, step by step (exact: a row's logits do not depend on the drafts
    after it, and a restart inside a step replays the DeltaNet state bit for bit)."""
    m = M.synthetic(ctx, nlayers=8, slots=2, max_ctx=1536, vocab=VOCAB, seed=41)
    prompt = [(1000 + 7919 * i) % VOCAB for i in range(40)]
    firsts = []
    for slot in (0, 1):
        m.step([(t, slot, i) for i, t in enumerate(prompt)], [len(prompt) - 1])
        firsts.append(m.argmax()[0])
    assert firsts[0] == firsts[1]
    # one token per step: enough tokens for 256 verify steps that accept 1..5 tokens each
    need = 1 + STEPS * 3 + 8
    reference = [firsts[0]]
    for i in range(need - 1):
        m.step([(reference[-1], 0, len(prompt) + i)], [0])
        reference.append(m.argmax()[0])
    got = verify_run(m, 1, reference, firsts[1], len(prompt))
    same = next((i for i, (a, b) in enumerate(zip(got, reference)) if a != b), min(len(got), len(reference)))
    assert len(got) >= STEPS and same == min(len(got), len(reference)), \
        f"first divergence at token {same} of {len(got)}: {got[same:same + 3]} vs {reference[same:same + 3]}"
    assert ctx.device_error() == 0
    m.close()


def test_256_verify_steps_against_the_cpu_oracle(ctx):
    """The same schedule on one [D, D, D, A] block at full width next to oracle/cpu_step.CpuModel, which is fed the
    GPU's steps (so both stay on one token stream): every row's greedy token equals the oracle's unless the oracle's top
    two logits are closer than 1e-3, and the logits of the last step agree within the step tolerance. Reports the first
    differing row and its margin."""
    m = M.synthetic(ctx, nlayers=4, slots=1, max_ctx=1536, vocab=VOCAB, seed=43)
    cpu = cpu_step.CpuModel.from_device(m)
    prompt = [(1000 + 7919 * i) % VOCAB for i in range(24)]
    toks = [(t, 0, i) for i, t in enumerate(prompt)]
    m.step(toks, [len(prompt) - 1])
    first = m.argmax()[0]
    lg, want, _, _ = cpu.step(toks, [len(prompt) - 1])
    assert first == int(want[0])
    # the drafts: the oracle cannot know the future tokens either, so the "right" drafts come from a one-token-per-step
    # run of a twin model on the GPU
    twin = M.synthetic(ctx, nlayers=4, slots=1, max_ctx=1536, vocab=VOCAB, seed=43)
    twin.step(toks, [len(prompt) - 1])
    reference = [twin.argmax()[0]]
    for i in range(STEPS * 3 + 8):
        twin.step([(reference[-1], 0, len(prompt) + i)], [0])
        reference.append(twin.argmax()[0])
    torch.cuda.synchronize()
    twin.close()
    near, rows, worst = [], 0, 0.0

    def check(step, toks, am):
        nonlocal rows, worst
        logits, want, _, _ = cpu.step(toks, list(range(len(toks))))
        srt = np.sort(logits[:, :VOCAB], axis=1)
        for r in range(len(toks)):
            rows += 1
            if am[r] != int(want[r]):
                margin = float(srt[r, -1] - srt[r, -2])
                near.append((step, r, margin))
                assert margin < 1e-3, f"step {step} row {r}: token {am[r]} vs the oracle's {int(want[r])}, margin {margin}"
        if step == STEPS - 1:
            a = m.logits().cpu().numpy().astype(np.float64)
            worst = float(np.linalg.norm(a - logits) / np.linalg.norm(logits))

    got = verify_run(m, 0, reference, first, len(prompt), on_step=check)
    assert got[:len(reference)] == reference[:len(got)]
    assert rows == STEPS * 5 and worst < 2e-3, (rows, worst)
    print(f"greedy 256: {rows} rows, {len(near)} near-ties {near[:3]}, last step relative L2 {worst:.2e}")
    m.close()


def test_a_capture_without_memory_costs_the_graph_not_the_step(ctx):
    """Graphs::run's out-of-memory branch (src/cuda/core.rs:1180-1192) with the failure made on the host: the next two
    captures report no memory. Those steps run directly (same logits as a model that never uses graphs), the cache's cap
    drops to three quarters of what it holds, and later steps capture and replay again."""
    kw = dict(nlayers=2, slots=1, max_ctx=256, vocab=VOCAB, seed=47, pattern=("delta", "attn"))
    m, plain = M.synthetic(ctx, **kw), M.synthetic(ctx, **kw)
    plain.use_graphs(False)
    seq = [(5 + 13 * i) % VOCAB for i in range(64)]
    pos = 0

    def both(n):
        nonlocal pos
        toks = [(seq[pos + i], 0, pos + i) for i in range(n)]
        m.step(toks, list(range(n)))
        a = m.logits()
        plain.step(toks, list(range(n)))
        assert torch.equal(a, plain.logits())
        pos += n
    for n in (1, 2, 3, 4):          # four shapes captured
        both(n)
        both(n)                     # and replayed
    assert m.graph_stats() == (4, -1, 0)
    m.fail_captures(2)
    both(5)                         # no memory: runs without a graph, the cap becomes 3
    held, cap, graphless = m.graph_stats()
    assert (held, cap, graphless) == (2, 3, 1)
    both(6)                         # still none
    assert m.graph_stats()[2] == 2
    both(5)                         # memory is back: captured (one of the old graphs makes room), then replayed
    both(5)
    held, cap, graphless = m.graph_stats()
    assert graphless == 2 and 1 <= held <= cap
    m.close()
    plain.close()


def test_an_adapter_swapped_at_run_time_drops_the_captured_steps(ctx):
    """Captured steps hold the adapter's pointers and each layer's adapted / plain choice: after qb_model_set_adapter
    (another adapter, or none) the next step of a shape already captured must run the new kernels. Compared with fresh
    models that had the new adapter (or none) from the start."""
    kw = dict(nlayers=2, slots=1, max_ctx=128, vocab=VOCAB, seed=53, pattern=("delta", "attn"))
    seq = [(3 + 31 * i) % VOCAB for i in range(32)]

    def run(model, start, n=2):
        outs = []
        for r in range(n):
            toks = [(seq[start + 3 * r + i], 0, start + 3 * r + i) for i in range(3)]
            model.step(toks, [0, 1, 2])
            outs.append(model.logits().clone())
        return outs
    m = M.synthetic(ctx, **kw)
    M.synthetic_adapter(m, rank=16, seed=7, std=0.12)
    m.set_slot_scale(0, 2.0)
    run(m, 0)                                    # captured and replayed with adapter A
    M.synthetic_adapter(m, rank=16, seed=8, std=0.12)   # adapter B takes its place
    got_b = run(m, 6)
    fresh = M.synthetic(ctx, **kw)
    M.synthetic_adapter(fresh, rank=16, seed=7, std=0.12)
    fresh.set_slot_scale(0, 2.0)
    run(fresh, 0)
    torch.cuda.synchronize()
    M.synthetic_adapter(fresh, rank=16, seed=8, std=0.12)
    fresh.use_graphs(False)                      # never replays anything
    want_b = run(fresh, 6)
    for a, b in zip(got_b, want_b):
        assert torch.equal(a, b)
    for i in range(2):                           # and none at all: the base model's kernels
        m.set_adapter(i, None)
        fresh.set_adapter(i, None)
    for a, b in zip(run(m, 12), run(fresh, 12)):
        assert torch.equal(a, b)
    m.close()
    fresh.close()
