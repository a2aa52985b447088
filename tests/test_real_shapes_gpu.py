"""GPU parity at the real shapes of BASELINE configs 1 and 3 (the other GPU tests use small shapes so
that the scalar oracle finishes in milliseconds).

Config 1: the projections of one full-attention layer and its FFN (q 12288 x 5120 with the
interleaved gate rows as the reference holds it, k/v 1024 x 5120, o 5120 x 6144 in Q4_B64;
gate/up 17408 x 5120 and down 5120 x 17408 in Q2_B64), bf16 activations, M = 1, 2, 4, 8, 16 verify
positions, every position against the oracle's fused_matvec of that row: rel-L2 <= 1e-3 (the
reference's device check has the same form, src/bin/cuda_bench.rs:53-56).
Config 3: the 248320 x 5120 Q4 lm_head over a depth-3 draft tree with 8 leaves (15 nodes), greedy
and at temperature 0.7: logits within rel-L2 1e-3 and the acceptance record equal to the oracle's
walk over the oracle's logits (same Philox counters).
The oracle runs its AVX2 arm over all host threads here (a few seconds per case).
"""
import os

import numpy as np
import pytest
import torch

import ctox_llm_b200 as ctox
from ctox_llm_b200 import synthetic
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu
THREADS = max(1, min(32, os.cpu_count() or 1))


@pytest.fixture(scope="module")
def be():
    b = ctox.B200Backend(0)
    yield b
    assert b.allocated_bytes() == 0
    b.close()


def fast_weights(dtype, rows, columns, seed):
    """Canonical blocks with uniform code bytes and f16 scales exp(N(-4, 0.5)), like
    synthetic.packed_weights but cheap for 20 million blocks: one random chunk of a million
    blocks is repeated with a block-dependent byte added to it, so that no two rows are equal."""
    bb = 34 if dtype == ctox.Q4B64 else 18
    blocks = rows * (columns // 64)
    rng = np.random.default_rng(seed)
    chunk = min(blocks, 1 << 20)
    base = np.frombuffer(rng.bytes(chunk * bb), dtype=np.uint8).reshape(chunk, bb)
    out = np.tile(base, (-(-blocks // chunk), 1))[:blocks].copy()
    out += ((np.arange(blocks, dtype=np.uint64) // chunk * 37) & 0xff).astype(np.uint8)[:, None]
    scales = np.exp(rng.standard_normal(blocks, dtype=np.float32) * 0.5 - 4.0).astype(np.float16)
    out.view(np.uint16).reshape(blocks, bb // 2)[:, 0] = scales.view(np.uint16)
    return out.reshape(-1)


def bf16_round(x):
    return torch.from_numpy(x).to(torch.bfloat16).float().numpy()


CONFIG1 = [("q_proj", ctox.Q4B64, 12288, 5120), ("k_proj", ctox.Q4B64, 1024, 5120),
           ("o_proj", ctox.Q4B64, 5120, 6144), ("gate_proj", ctox.Q2B64, 17408, 5120),
           ("down_proj", ctox.Q2B64, 5120, 17408)]


@pytest.mark.parametrize("name,dtype,rows,columns", CONFIG1, ids=[c[0] for c in CONFIG1])
def test_config1_projection_at_1_to_16_positions(be, orc, name, dtype, rows, columns):
    seed = 1000 + rows % 97
    op = ctox.FusedMatVec(dtype, fast_weights(dtype, rows, columns, seed), rows, columns, None,
                          s_in=synthetic.recovery_scales_f16(columns, seed, 3),
                          s_out=synthetic.recovery_scales_f16(rows, seed, 4))
    x = bf16_round(synthetic.activations(columns, seed, positions=16).reshape(16, columns))
    want = np.stack([orc.fused_matvec(orc.FusedMatVec(dtype, op.weights, rows, columns, x[m], s_in=op.s_in,
                                                      s_out=op.s_out), threads=THREADS, avx2=True)
                     for m in range(16)])
    # the AVX2 arm itself against the scalar verifier on one position (backend/cpu.rs:732-812: 2e-4 + 1e-5)
    scalar = orc.fused_matvec(orc.FusedMatVec(dtype, op.weights, rows, columns, x[0], s_in=op.s_in, s_out=op.s_out),
                              threads=THREADS)
    assert rel_l2(want[0], scalar) <= 1e-5
    mv = be.prepare_fused_matvec(op)
    try:
        xd = torch.from_numpy(x).cuda().to(torch.bfloat16)
        for m in (1, 2, 4, 8, 16):
            y = torch.full((m, rows), float("nan"), device="cuda")
            mv.dispatch_device(xd.data_ptr(), ctox.BF16, m, columns, y.data_ptr(), rows)
            be.synchronize()
            got = y.cpu().numpy()
            for pos in range(m):
                err = rel_l2(got[pos], want[pos])
                assert err <= 1e-3, (name, m, pos, err)
        assert be.device_error() == 0
    finally:
        mv.destroy()


TREE_PARENT = [-1, 0, 0, 1, 1, 2, 3, 3, 4, 4, 5, 5, 6, 6, 2]  # depth 3, 8 leaves, 15 nodes


def test_config3_lm_head_with_a_depth3_tree(be, orc):
    rows, columns, n = 248_320, 5_120, len(TREE_PARENT)
    op = ctox.FusedMatVec(ctox.Q4B64, fast_weights(ctox.Q4B64, rows, columns, 3), rows, columns, None,
                          s_in=synthetic.recovery_scales_f16(columns, 3, 3),
                          s_out=synthetic.recovery_scales_f16(rows, 3, 4))
    hidden = bf16_round(synthetic.activations(columns, 31, positions=n).reshape(n, columns)) * 2.0
    hidden = bf16_round(hidden)
    want = np.stack([orc.fused_matvec(orc.FusedMatVec(op.dtype, op.weights, rows, columns, hidden[i], s_in=op.s_in,
                                                      s_out=op.s_out), threads=THREADS, avx2=True)
                     for i in range(n)])
    mv = be.prepare_fused_matvec(op)
    try:
        dh = torch.from_numpy(hidden).cuda().to(torch.bfloat16)
        logits = torch.empty(n, rows, dtype=torch.float32, device="cuda")
        # draft tokens: the parent's most likely tokens in order (first child = its greedy token,
        # so a greedy walk accepts a full-depth path), siblings distinct
        token = [0] * n
        for c in range(1, n):
            top = np.argsort(want[TREE_PARENT[c]])[::-1]
            sibs = [token[s] for s in range(1, c) if TREE_PARENT[s] == TREE_PARENT[c]]
            token[c] = int(next(t for t in top if t not in sibs))
        rec = mv.lmhead_verify(dh.data_ptr(), ctox.BF16, columns, TREE_PARENT, token, 0.0, 7, 0,
                               logits_out_ptr=logits.data_ptr())
        got = logits.cpu().numpy()
        for i in range(n):
            assert rel_l2(got[i], want[i]) <= 1e-3, (i, rel_l2(got[i], want[i]))
        assert rec["node_argmax"] == [orc.greedy_token(w) for w in want]
        emitted, path = orc.spec_tree_accept(want, TREE_PARENT, token, 0.0, 7, 0)
        assert rec["emitted"] == emitted and rec["path"] == path
        assert len(path) >= 3 and len(emitted) == len(path) + 1  # a full-depth greedy path + the next token
        # temperature 0.7: the walk is decided by the same counters on both sides; run it on the device's own
        # logits so that the last bits of a logit cannot flip a draw
        for step in range(8):
            rec = mv.lmhead_verify(dh.data_ptr(), ctox.BF16, columns, TREE_PARENT, token, 0.7, 99, step)
            emitted, path = orc.spec_tree_accept(got, TREE_PARENT, token, 0.7, 99, step)
            assert rec["emitted"] == emitted and rec["path"] == path, step
        assert be.device_error() == 0
    finally:
        mv.destroy()


def test_config4_shapes_two_layer_model_logits_tokens_and_mtp(orc):
    """The layer shapes of BASELINE config 4 (hidden 5120, FFN 17408, 24 / 4 heads of 256, 16 / 48 linear
    heads of 128, vocabulary 248 320, Q4 attention / head and Q2 FFN weights, bf16 KV, 40 000-row draft
    head) on a model of one linear-attention and one full-attention layer plus the MTP layer, random
    packed weights as the benchmark's synthetic model holds them: target logits within rel-L2 1e-3
    and greedy tokens equal for a few steps, then speculative blocks checked like tests/test_mtp_gpu.py
    (MTP hidden of every pair, drafts, accepted prefix, committed hidden)."""
    from ctox_llm_b200 import native as N
    from oracle_model import DeviceChainOracle, OracleModel
    cfg = ctox.qwen38_27b_config(num_hidden_layers=2, full_attention_interval=2, max_context_tokens=256,
                                 max_draft_tokens=3, draft_vocab=40_000)
    model = OracleModel(orc, cfg, seed=11, packed_random=True, threads=THREADS, tied_head=True)
    ids = (np.arange(cfg.draft_vocab, dtype=np.int64) * (cfg.vocab_size // cfg.draft_vocab))
    be = ctox.B200Backend(0)
    ex = ctox.B200Executor(be, cfg)
    try:
        model.load_into(ex)
        ex.load_vector(N.LAYER_GLOBAL, N.T_DRAFT_IDS, ids.astype(np.uint32))
        ex.warmup()
        ex.keep_logits(True)
        prompt = [17, 40_123, 200_001, 5, 99_999, 248_000, 3]
        want_tokens, want_logits, _ = model.greedy(prompt, 3)
        ex.prefill(prompt)
        tok = prompt[-1]
        for i in range(3):
            blk = ex.decode(tok, mtp_enabled=False)
            err = rel_l2(ex.last_logits(0), want_logits[i])
            assert err <= 1e-3, (i, err)
            assert blk.token_id == want_tokens[i]
            tok = blk.token_id
        dev = DeviceChainOracle(model, cfg.max_draft_tokens, ids)
        ex.prefill(prompt)
        dev.prefill(prompt)
        tok = prompt[-1]
        for block, force in enumerate((-1, 2, -1)):
            blk = ex.decode(tok, mtp_enabled=True, force_accept=force)
            want = dev.decode(tok, force_accept=force, given_drafts=blk.draft_tokens)
            for j, (g, w) in enumerate(zip(ex.last_mtp_hidden(), want["mtp_hidden"])):
                assert rel_l2(g, w) <= 1e-3, ("mtp hidden", block, j, rel_l2(g, w))
            for i in range(cfg.max_draft_tokens):
                if blk.draft_tokens[i] != want["drafts"][i]:  # only where the oracle's top two are a near-tie
                    lg = want["draft_logits"][i]
                    a, b = int(np.searchsorted(ids, blk.draft_tokens[i])), int(np.searchsorted(ids, want["drafts"][i]))
                    assert abs(float(lg[a]) - float(lg[b])) <= 1e-4 * max(abs(float(lg[a])), abs(float(lg[b])))
            assert blk.accepted_draft_tokens == want["accepted"] and blk.token_id == want["next_token"], block
            assert rel_l2(ex.last_hidden(), want["final_hidden"]) <= 1e-3
            tok = blk.token_id
        assert be.device_error() == 0
    finally:
        ex.unload()
        be.close()
