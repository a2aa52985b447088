"""GPU parity of the selection kernels (argmax, fused lm_head + acceptance) against the oracle.

Greedy results must be identical (integer work). Stochastic acceptance is compared token for
token with the oracle's restatement on the same logits and the same Philox counters, and its
output distribution against softmax(logits / T) with the total-variation bound stated below.
"""
import numpy as np
import pytest
import torch

import ctox_llm_b200 as ctox
from ctox_llm_b200 import synthetic
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    b = ctox.B200Backend(0)
    yield b
    b.close()


def test_argmax_matches_total_cmp_last_index(be, orc):
    rng = np.random.default_rng(0)
    for n in (1, 3, 1000, 248320):
        logits = rng.standard_normal(n).astype(np.float32)
        if n > 10:
            logits[rng.integers(0, n, 5)] = logits.max()  # ties: the later index wins
        d = torch.from_numpy(logits).cuda()
        assert be.argmax(d.data_ptr(), n) == orc.greedy_token(logits)
    # sampler.rs:229-239 and the total order of signed zeros
    for vals in ([2.0, 2.0], [-0.0, 0.0], [0.0, -0.0], [-1.0, 3.0, 2.0], [-np.inf, -np.inf]):
        d = torch.tensor(vals, dtype=torch.float32).cuda()
        if np.all(np.isfinite(vals)):
            assert be.argmax(d.data_ptr(), len(vals)) == orc.greedy_token(vals)
    ids = torch.tensor([1, 4], dtype=torch.int32).cuda()
    d = torch.tensor([0.0, 3.0], dtype=torch.float32).cuda()
    assert be.argmax(d.data_ptr(), 2, ids.data_ptr()) == 4  # engine.rs:1346-1413
    bad = torch.tensor([1.0, float("nan"), 0.0], dtype=torch.float32).cuda()
    with pytest.raises(ctox.CtoxError) as e:
        be.argmax(bad.data_ptr(), 3)
    assert e.value.kind == "InvalidState"


def make_head(be, rows, columns, dtype=ctox.Q4B64, seed=5):
    w = synthetic.packed_weights(dtype, rows, columns, seed)
    s_in = synthetic.recovery_scales_f16(columns, seed, 3)
    s_out = synthetic.recovery_scales_f16(rows, seed, 4)
    op = ctox.FusedMatVec(dtype, w, rows, columns, None, s_in=s_in, s_out=s_out)
    return be.prepare_fused_matvec(op), op


def oracle_logits(orc, op, hidden):
    out = []
    for h in hidden:
        out.append(orc.fused_matvec(orc.FusedMatVec(op.dtype, op.weights, op.rows, op.columns, h,
                                                    s_in=op.s_in, s_out=op.s_out), threads=8))
    return np.stack(out)


def test_greedy_chain_matches_verify_greedy_mtp(be, orc):
    rows, columns, k = 8192, 512, 4
    mv, op = make_head(be, rows, columns)
    try:
        hidden = synthetic.activations(columns, 9, positions=k + 1) * 4.0
        exp_logits = oracle_logits(orc, op, hidden)
        targets = [orc.greedy_token(l) for l in exp_logits]
        dh = torch.from_numpy(hidden).cuda()
        logits = torch.empty(k + 1, rows, dtype=torch.float32, device="cuda")
        parent = [-1, 0, 1, 2, 3]
        for accepted in range(k + 1):
            drafts = [targets[i] if i < accepted else (targets[i] + 1) % rows for i in range(k)]
            rec = mv.lmhead_verify(dh.data_ptr(), ctox.F32, columns, parent, [0] + drafts, 0.0, 1, 0,
                                   logits_out_ptr=logits.data_ptr())
            nxt, verified, acc = orc.verify_greedy_mtp_tokens(drafts, targets[:k], targets[k])
            assert rec["emitted"] == acc + [nxt]
            assert rec["path"] == list(range(1, len(acc) + 1))
            assert rec["node_argmax"] == targets
            emitted, path = orc.spec_tree_accept(exp_logits, parent, [0] + drafts, 0.0, 1, 0)
            assert rec["emitted"] == emitted and rec["path"] == path
        assert rel_l2(logits.cpu().numpy(), exp_logits) <= 2e-5
        # bf16 hidden states, vocabulary limit, single node
        hb = dh.to(torch.bfloat16)
        lim = 5000
        rec = mv.lmhead_verify(hb.data_ptr(), ctox.BF16, columns, [-1], [0], 0.0, 1, 0, vocab=lim)
        l0 = oracle_logits(orc, op, hb[:1].float().cpu().numpy())[0]
        assert rec["emitted"] == [orc.greedy_token(l0[:lim])]
    finally:
        mv.destroy()


TREE_PARENT = [-1, 0, 0, 1, 1, 2, 3, 3, 4, 4, 5, 5, 6, 6, 2]  # depth 3, 8 leaves, 15 nodes


def test_tree_acceptance_matches_oracle_token_for_token(be, orc):
    rows, columns = 4096, 256
    mv, op = make_head(be, rows, columns, seed=6)
    try:
        n = len(TREE_PARENT)
        hidden = synthetic.activations(columns, 11, positions=n) * 6.0
        dh = torch.from_numpy(hidden).cuda()
        logits = torch.empty(n, rows, dtype=torch.float32, device="cuda")
        rng = np.random.default_rng(1)
        mv.lmhead_verify(dh.data_ptr(), ctox.F32, columns, [-1] + [0] * (n - 1), [0] + [1] * (n - 1), 0.0,
                         0, 0, logits_out_ptr=logits.data_ptr())
        gl = logits.cpu().numpy()
        lengths = []
        for step in range(60):
            # drafts: likely tokens of the parent's distribution so that acceptance happens
            token = [0] * n
            for c in range(1, n):
                top = np.argsort(gl[TREE_PARENT[c]])[::-1]
                sibs = [token[s] for s in range(1, c) if TREE_PARENT[s] == TREE_PARENT[c]]
                token[c] = int(next(t for t in top[rng.integers(0, 2):] if t not in sibs))
            for temperature in (0.7, 0.0):
                rec = mv.lmhead_verify(dh.data_ptr(), ctox.F32, columns, TREE_PARENT, token, temperature,
                                       1234, step)
                emitted, path = orc.spec_tree_accept(gl, TREE_PARENT, token, temperature, 1234, step)
                assert rec["emitted"] == emitted, (step, temperature)
                assert rec["path"] == path
            lengths.append(len(emitted))
        assert max(lengths) >= 2  # some drafts were accepted
    finally:
        mv.destroy()


def test_sampled_distribution_total_variation(be, orc):
    """The emitted token is distributed as softmax(logits/T) whatever the drafts are. N trials
    over a K-token support: E[TV] <= sqrt(K / (2 pi N)) * ... ; with K = 64 effective, N = 4000
    the bound 0.08 is > 5 sigma above the expected ~0.05."""
    rows, columns, trials = 64, 64, 4000
    mv, op = make_head(be, rows, columns, seed=8)
    try:
        hidden = synthetic.activations(columns, 13, positions=3) * 3.0
        dh = torch.from_numpy(hidden).cuda()
        logits = torch.empty(3, rows, dtype=torch.float32, device="cuda")
        parent, token = [-1, 0, 0], [0, 5, 9]
        counts = np.zeros(rows)
        for step in range(trials):
            rec = mv.lmhead_verify(dh.data_ptr(), ctox.F32, columns, parent, token, 0.7, 99, step,
                                   logits_out_ptr=logits.data_ptr() if step == 0 else 0)
            counts[rec["emitted"][0]] += 1
        z = logits.cpu().numpy()[0].astype(np.float64) / 0.7
        p = np.exp(z - z.max())
        p /= p.sum()
        tv = 0.5 * np.abs(counts / trials - p).sum()  # training/sampling_tv/measure.py:45-47
        assert tv <= 0.08, tv
    finally:
        mv.destroy()


def test_verify_argument_errors(be):
    mv, op = make_head(be, 128, 64)
    try:
        h = torch.zeros(2, 64, device="cuda")
        for parent, token, temp, kind in [([0, 0], [0, 1], 0.0, "Shape"), ([-1, 1], [0, 1], 0.0, "Shape"),
                                          ([-1, 0], [0, 500], 0.0, "Shape"),
                                          ([-1, 0], [0, 1], float("nan"), "InvalidArtifact"),
                                          ([-1] + [0] * 16, [0] * 17, 0.0, "Shape")]:
            with pytest.raises(ctox.CtoxError) as e:
                mv.lmhead_verify(h.data_ptr(), ctox.F32, 64, parent, token, temp, 0, 0)
            assert e.value.kind == kind
    finally:
        mv.destroy()
