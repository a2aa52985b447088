"""Pins of tests/oracle_model.py, the composition of the C oracle's operators in the order of the
reference's scalar executor (models/qwen38_27b/src/decoder.rs).

1. The reference's own decoder integration test (decoder.rs:1533-2014) restated as a known-answer
   test: same constant-valued Q2 matrices, same closed-form expectations and tolerances, same
   position / MTP-cache bookkeeping of the CPU executor through prefill, decode and
   commit_speculative.
2. The accelerator-style speculative block (DeviceChainOracle, the checker of the GPU executor's
   MTP path) against the restatement of the reference CPU executor: same first draft, same MTP
   cache after commit, same emitted tokens as plain greedy decoding.
"""
import numpy as np
import pytest

from oracle_model import (DeviceChainOracle, OracleModel, ReferenceCpuExecutor, reference_fixture_model,
                          tiny_config)


def test_reference_decoder_fixture_closed_forms(orc):
    full = reference_fixture_model(orc, full_layer=True)
    emb = full.embedding(0)
    assert emb.size == 64 and np.all(np.abs(emb - 0.5) < 1e-6)  # decoder.rs:1741-1743
    residual = np.ones(64, np.float32)
    st = {"k": [], "v": []}
    att = full.full_attention(full.layers[0], residual, 0, st)  # decoder.rs:1757-1766
    normalized = np.float32(1.0) / np.sqrt(np.float32(1.0 + 1e-6))
    expected = 1.0 + 2.0 * normalized / (1.0 + np.exp(-normalized))
    assert np.all(np.abs(att - expected) < 2e-4)
    assert len(st["k"]) == 1

    lin = reference_fixture_model(orc, full_layer=False)
    out1 = lin.linear_attention(lin.layers[0], residual, lin.state[0])  # decoder.rs:1787-1803
    assert out1.size == 64 and np.all(np.isfinite(out1))
    lin.reset()
    assert np.array_equal(out1, lin.linear_attention(lin.layers[0], residual, lin.state[0]))

    mlp = lin.mlp(lin.layers[0], residual)  # decoder.rs:1805-1811
    gate, up = normalized, 2.0 * normalized
    assert np.all(np.abs(mlp - (1.0 + gate / (1.0 + np.exp(-gate)) * up)) < 2e-4)

    fh = lin.norm(mlp, lin.final_norm)
    logits = lin.proj(lin.lm_head, fh)  # decoder.rs:1813-1816
    assert logits.size == 2 and np.all(np.isfinite(logits)) and abs(logits[0] - logits[1]) < 1e-6
    assert np.array_equal(lin.restricted_logits(fh, [1]), logits[1:2])  # decoder.rs:1817-1831
    with pytest.raises(AssertionError):
        lin.restricted_logits(fh, [1, 1])
    with pytest.raises(AssertionError):
        lin.restricted_logits(fh, [2])


def test_reference_decoder_fixture_target_and_mtp_steps(orc):
    lin = reference_fixture_model(orc, full_layer=False)
    _, logits = lin.decode_target_step(0)  # decoder.rs:1847-1860
    assert logits.size == 2 and lin.position == 1
    lin.reset()
    assert lin.position == 0
    assert np.array_equal(lin.decode_target_step(0)[1], logits)

    full = reference_fixture_model(orc, full_layer=True)
    fh, logits = full.decode_target_step(0)  # decoder.rs:1870-1876
    assert fh.size == 64 and logits.size == 2 and np.all(np.isfinite(logits)) and full.position == 1
    mst = full.new_mtp_state()
    dh, dl = full.mtp_draft(0, fh, 1, mst)  # decoder.rs:1878-1891
    assert dh.size == 64 and dl.size == 2 and np.all(np.isfinite(dl)) and len(mst["k"]) == 1
    with pytest.raises(AssertionError):  # absolute position 2 with one cached token is refused
        full.mtp_draft(0, fh, 3, mst)
    again = full.new_mtp_state()
    dh2, dl2 = full.mtp_draft(0, fh, 1, again)
    assert np.array_equal(dh, dh2) and np.array_equal(dl, dl2)


def test_reference_decoder_fixture_executor_bookkeeping(orc):
    """decoder.rs:1917-1996: positions and MTP cache lengths through prefill / decode / commit."""
    m = reference_fixture_model(orc, full_layer=False)
    ex = ReferenceCpuExecutor(m, draft_tokens=4, draft_ids=[0, 1])
    assert ex.prefill([0], False).size == 2
    assert ex.decode(0, False)["target_logits"].size == 2
    ex.prefill([0], True)
    step = ex.decode(0, True)
    assert step["target_logits"].size == 2 and len(step["draft_logits"]) == 4
    assert all(d.size == 2 for d in step["draft_logits"])
    assert len(step["target_verification_logits"]) == 4 and step["bonus_logits"].size == 2
    assert np.array_equal(step["target_verification_logits"][0], step["target_logits"])
    assert ex.pending is not None
    ex.commit_speculative(0)
    assert m.position == 2 and len(ex.mtp["k"]) == 1

    ex.prefill([0], True)
    acc = ex.decode(0, True)
    for draft, target in zip(acc["draft_logits"], acc["target_verification_logits"]):
        assert m.draft_token(draft, ex.ids) == orc.greedy_token(target)
    ex.commit_speculative(2)
    assert m.position == 4 and len(ex.mtp["k"]) == 3
    fallback = orc.greedy_token(acc["target_verification_logits"][2])
    aligned = ex.decode(fallback, True)
    assert len(aligned["target_verification_logits"]) == 4
    ex.commit_speculative(0)
    assert m.position == 5 and len(ex.mtp["k"]) == 4
    with pytest.raises(AssertionError):
        ex.commit_speculative(0)  # no pending branch


PROMPT = [5, 17, 900, 3, 3, 41, 512, 77, 1001, 64, 9]


@pytest.mark.parametrize("draft_ids", [None, "restricted"])
def test_device_chain_oracle_agrees_with_the_reference_executor(orc, draft_ids):
    cfg = tiny_config()
    ids = None
    if draft_ids:
        ids = np.sort(np.random.default_rng(11).choice(cfg.vocab_size, 256, replace=False))
        ids = np.union1d(ids, [3, 17])
    k = 3
    loud = (3, 17)
    ref_model = OracleModel(orc, cfg, seed=3, loud_tokens=loud)
    dev_model = OracleModel(orc, cfg, seed=3, loud_tokens=loud)
    plain = OracleModel(orc, cfg, seed=3, loud_tokens=loud)
    want, _, _ = plain.greedy(PROMPT, 14)

    ref = ReferenceCpuExecutor(ref_model, k, ids)
    dev = DeviceChainOracle(dev_model, k, ids)
    ref.prefill(PROMPT[:-1], True)
    dev.prefill(PROMPT)
    tok, emitted, accepted_total = PROMPT[-1], [], 0
    while len(emitted) < 14:
        r = ref.decode(tok, True)
        d = dev.decode(tok)
        # the first draft comes from the same pair in both (token, last target hidden)
        assert d["drafts"][0] == r["candidates"][0]
        assert np.array_equal(d["draft_logits"][0], r["draft_logits"][0])
        # verify the CPU executor's own candidates the way the engine does (engine.rs:939-962)
        n_ref = 0
        for cand, tl in zip(r["candidates"], r["target_verification_logits"]):
            if cand != orc.greedy_token(tl):
                break
            n_ref += 1
        nxt_ref = orc.greedy_token((r["target_verification_logits"] + [r["bonus_logits"]])[n_ref])
        ref.commit_speculative(n_ref)
        # the two drafters may propose different later drafts; emitted tokens cannot differ
        got = d["accepted"] + [d["next_token"]]
        ref_got = r["candidates"][:n_ref] + [nxt_ref]
        m = min(len(got), len(ref_got))
        assert got[:m] == ref_got[:m]
        emitted += got
        accepted_total += len(d["accepted"])
        # bring the reference executor to the device chain's position (it may have accepted less/more)
        if len(got) != len(ref_got):
            ref.prefill(PROMPT[:-1] + [PROMPT[-1]] + emitted[:-1], True)
        tok = emitted[-1]
        # committed MTP caches agree once the device chain has paid the pairs it owes
        assert dev_model.position == ref_model.position
    assert emitted[:14] == want
    assert accepted_total > 0, "the loud-token model should accept some drafts"
