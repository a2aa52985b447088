"""GPU parity of the decode executor against the CPU oracle composed as the reference's scalar
executor composes it (decoder.rs): logits within rel-L2 1e-3 and, for greedy decoding, the emitted
token sequence identical with MTP on and off (engine.rs:939-962: verification guards every draft,
so the emitted sequence does not depend on the drafter)."""
import numpy as np
import pytest

import ctox_llm_b200 as ctox
from gpu_util import rel_l2
from oracle_model import OracleModel, tiny_config

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup(orc):
    be = ctox.B200Backend(0)
    cfg = tiny_config()
    model = OracleModel(orc, cfg, seed=3)
    ex = ctox.B200Executor(be, cfg)
    model.load_into(ex)
    ex.warmup()
    yield be, ex, model
    ex.unload()
    assert be.allocated_bytes() == 0
    be.close()


PROMPT = [5, 17, 900, 3, 3, 41, 512, 77, 1001, 64, 9]


def test_plain_greedy_decode_matches_oracle(setup):
    be, ex, model = setup
    n_new = 12
    exp_tokens, exp_logits, _ = model.greedy(PROMPT, n_new)
    ex.keep_logits(True)
    ex.prefill(PROMPT)
    assert ex.position() == len(PROMPT) - 1
    tok, got = PROMPT[-1], []
    for i in range(n_new):
        blk = ex.decode(tok, mtp_enabled=False)
        assert blk.draft_tokens_proposed == 0 and blk.accepted_draft_tokens == []
        err = rel_l2(ex.last_logits(0), exp_logits[i])
        assert err <= 1e-3, (i, err)
        tok = blk.token_id
        got.append(tok)
    assert got == exp_tokens
    assert ex.position() == len(PROMPT) - 1 + n_new


def test_mtp_greedy_emits_the_same_sequence(setup):
    be, ex, model = setup
    n_new = 24
    exp_tokens, _, exp_hidden = model.greedy(PROMPT, n_new)
    ex.prefill(PROMPT)
    tok, got, proposed, accepted = PROMPT[-1], [], 0, 0
    while len(got) < n_new:
        blk = ex.decode(tok, mtp_enabled=True, commit=False)
        assert ex.session_state()["pending_accepted"] == len(blk.accepted_draft_tokens)
        ex.commit_speculative(len(blk.accepted_draft_tokens))
        assert blk.draft_tokens_proposed == 4
        # engine.rs:118-136
        k, a = blk.draft_tokens_proposed, len(blk.accepted_draft_tokens)
        assert blk.draft_tokens_verified == (k if a == k else a + 1)
        assert blk.accepted_draft_tokens == blk.draft_tokens[:a]
        got += blk.emitted
        tok = blk.token_id
        proposed += k
        accepted += a
    assert got[:n_new] == exp_tokens
    assert ex.position() == len(PROMPT) - 1 + len(got)


def test_forced_acceptance_commits_the_prefix_state(setup):
    """Accepting n drafts must leave exactly the state of having decoded those tokens one by one."""
    be, ex, model = setup
    for n_force in (0, 1, 2, 3, 4):
        ex.prefill(PROMPT)
        blk = ex.decode(PROMPT[-1], mtp_enabled=True, force_accept=n_force)
        assert len(blk.accepted_draft_tokens) == n_force
        seq = PROMPT + blk.accepted_draft_tokens
        model.reset()
        for t in seq[:-1]:
            model.decode_target_step(int(t))
        fh, logits = model.decode_target_step(int(seq[-1]))
        assert rel_l2(ex.last_hidden(), fh) <= 1e-3
        assert blk.token_id == model.orc.greedy_token(logits)
        # and decoding continues correctly from the committed state
        nxt = ex.decode(blk.token_id, mtp_enabled=False)
        _, logits2 = model.decode_target_step(blk.token_id)
        assert nxt.token_id == model.orc.greedy_token(logits2)


def test_sampled_decode_runs_and_is_reproducible(setup):
    be, ex, model = setup
    runs = []
    for _ in range(2):
        ex.prefill(PROMPT)
        tok, got = PROMPT[-1], []
        for _ in range(6):
            blk = ex.decode(tok, mtp_enabled=True, temperature=0.7, seed=11)
            got += blk.emitted
            tok = blk.token_id
        runs.append(got)
    assert runs[0] == runs[1]
    assert all(0 <= t < 1024 for t in runs[0])


def test_lifecycle_errors(setup):
    be, ex, model = setup
    with pytest.raises(ctox.CtoxError) as e:
        ex.decode(5000)
    assert e.value.kind == "Shape"
    with pytest.raises(ctox.CtoxError) as e:
        ex.prefill([])
    assert e.value.kind == "Shape"
    alloc = ex.allocations()
    assert alloc["model_bytes"] > 0 and alloc["session_bytes"] > 0


def test_bf16_cache_tensor_core_attention_matches_oracle(orc):
    """head_dim 256 with a bfloat16 KV cache runs the tensor-core attention kernel; the oracle
    stores the same bf16-rounded K and V, so the logits still agree within rel-L2 1e-3."""
    be = ctox.B200Backend(0)
    cfg = tiny_config(num_attention_heads=4, num_key_value_heads=1, head_dim=256, rotary_dim=64,
                      kv_dtype=ctox.BF16, max_context_tokens=512, full_attention_interval=2)
    model = OracleModel(orc, cfg, seed=5)
    ex = ctox.B200Executor(be, cfg)
    try:
        model.load_into(ex)
        ex.warmup()
        ex.keep_logits(True)
        rng = np.random.default_rng(7)
        prompt = [int(t) for t in rng.integers(0, 1024, 150)]  # > 2 tiles of 64 tokens
        n_new = 6
        exp_tokens, exp_logits, _ = model.greedy(prompt, n_new)
        ex.prefill(prompt)
        tok, got = prompt[-1], []
        for i in range(n_new):
            blk = ex.decode(tok, mtp_enabled=False)
            assert rel_l2(ex.last_logits(0), exp_logits[i]) <= 1e-3
            tok = blk.token_id
            got.append(tok)
        assert got == exp_tokens
        # verify rows (5 queries per head group) through the same kernel
        ex.prefill(prompt)
        blk = ex.decode(prompt[-1], mtp_enabled=True)
        assert blk.emitted[0] == exp_tokens[0] or blk.accepted_draft_tokens[:1] == exp_tokens[:1]
        assert (blk.accepted_draft_tokens + [blk.token_id]) == exp_tokens[:len(blk.emitted)]
    finally:
        ex.unload()
        be.close()

@pytest.mark.parametrize("drafts", [0, 4])
def test_attention_over_many_tiles_per_split_matches_oracle(orc, drafts, monkeypatch):
    """One context split per KV head (CTOX_ATTN_SPLITS_MAX=1), so that a CTA of the tensor-core kernel
    walks all 64-token tiles of a 330-token context itself: the tile ring wraps around (two buffers
    with one query group, three with two). Logits of plain decode steps and the first emitted tokens
    of speculative blocks against the oracle with the same bf16-rounded cache."""
    monkeypatch.setenv("CTOX_ATTN_SPLITS_MAX", "1")
    be = ctox.B200Backend(0)
    cfg = tiny_config(max_draft_tokens=max(drafts, 1), num_attention_heads=4, num_key_value_heads=1, head_dim=256,
                      rotary_dim=64, kv_dtype=ctox.BF16, max_context_tokens=512, full_attention_interval=2)
    model = OracleModel(orc, cfg, seed=9)
    ex = ctox.B200Executor(be, cfg)
    try:
        model.load_into(ex)
        ex.warmup()
        ex.keep_logits(True)
        rng = np.random.default_rng(13)
        prompt = [int(t) for t in rng.integers(0, 1024, 330)]  # 6 tiles of 64 tokens
        n_new = 4
        exp_tokens, exp_logits, _ = model.greedy(prompt, n_new)
        ex.prefill(prompt)
        if drafts == 0:
            tok = prompt[-1]
            for i in range(n_new):
                blk = ex.decode(tok, mtp_enabled=False)
                assert rel_l2(ex.last_logits(0), exp_logits[i]) <= 1e-3, i
                assert blk.token_id == exp_tokens[i]
                tok = blk.token_id
        else:  # five verify positions x four query heads: the two-group kernel
            blk = ex.decode(prompt[-1], mtp_enabled=True)
            assert rel_l2(ex.last_logits(0), exp_logits[0]) <= 1e-3
            assert (blk.accepted_draft_tokens + [blk.token_id]) == exp_tokens[:len(blk.emitted)]
            blk2 = ex.decode(blk.token_id, mtp_enabled=True, force_accept=0)
            assert blk2.token_id == exp_tokens[len(blk.emitted)]
    finally:
        ex.unload()
        be.close()


def test_select_target_token_samples_from_the_kept_logits(setup, orc):
    """ModelExecutor::select_target_token (engine.rs:322-362): the sampler runs on the logits the
    executor kept on the device; same token as Sampler::sample_with_draw on those logits."""
    be, ex, model = setup
    ex.keep_logits(True)
    ex.prefill(PROMPT)
    ex.decode(PROMPT[-1], mtp_enabled=False)
    logits = ex.last_logits(0)
    for draw in (0.0, 0.37, 0.93):
        got = ex.select_target_token(0.8, 40, 0.9, draw)
        assert got == orc.sample_with_draw(logits, 0.8, 40, 0.9, draw)
    assert ex.select_target_token(0.0, 40, 0.9, 0.5) == orc.greedy_token(logits)
    with pytest.raises(ctox.CtoxError) as e:
        ex.select_target_token(0.8, 0, 0.9, 0.5)
    assert e.value.kind == "UnsupportedOperation"


def test_speculative_transaction_and_cancellation(setup):
    """trait ModelExecutor (engine.rs:322-377): a pending block must be committed with the depth the
    device resolved before the next decode; a raised cancellation token fails the call with
    Cancelled and leaves a decode's session untouched."""
    be, ex, model = setup
    ex.prefill(PROMPT)
    with pytest.raises(ctox.CtoxError) as e:
        ex.commit_speculative(0)  # decoder.rs:1401-1403: nothing pending
    assert e.value.kind == "InvalidState"
    blk = ex.decode(PROMPT[-1], mtp_enabled=True, force_accept=2, commit=False)
    assert ex.session_state() == {"pending_accepted": 2, "poisoned": False}
    with pytest.raises(ctox.CtoxError) as e:
        ex.decode(blk.token_id, mtp_enabled=True)  # decoder.rs:1293-1297
    assert e.value.kind == "InvalidState" and "committed" in str(e.value)
    with pytest.raises(ctox.CtoxError) as e:
        ex.commit_speculative(1)  # not the prefix the device holds
    assert e.value.kind == "InvalidState"
    token = ctox.CancellationToken()
    token.cancel()
    with pytest.raises(ctox.CtoxError) as e:
        ex.commit_speculative(2, token)
    assert e.value.kind == "Cancelled"
    ex.commit_speculative(2)
    assert ex.session_state()["pending_accepted"] == -1
    # a cancelled decode changes nothing: the same call without the token gives the oracle's token
    position = ex.position()
    with pytest.raises(ctox.CtoxError) as e:
        ex.decode(blk.token_id, mtp_enabled=True, cancellation=token)
    assert e.value.kind == "Cancelled" and ex.position() == position
    seq = PROMPT + blk.accepted_draft_tokens + [blk.token_id]
    model.reset()
    for t in seq[:-1]:
        model.decode_target_step(int(t))
    _, logits = model.decode_target_step(int(seq[-1]))
    nxt = ex.decode(blk.token_id, mtp_enabled=True)
    assert nxt.emitted[0] == model.orc.greedy_token(logits)
    with pytest.raises(ctox.CtoxError) as e:
        ex.prefill(PROMPT, token)
    assert e.value.kind == "Cancelled"

def test_phase_timing_reports_device_time_of_every_phase_and_changes_no_result(setup):
    """The four phases of a speculative block (drafting, target pass, head + acceptance, commit) get a
    positive device time each, their sum stays below the call's wall time, and the blocks are the
    ones the executor resolves without the events."""
    import time
    be, ex, model = setup
    ex.prefill(PROMPT)
    plain = []
    tok = PROMPT[-1]
    for force in (-1, 1, 0):
        blk = ex.decode(tok, mtp_enabled=True, force_accept=force)
        plain.append((blk.emitted, blk.draft_tokens))
        tok = blk.token_id
    ex.reset_session()
    ex.prefill(PROMPT)
    ex.phase_timing(True)
    tok = PROMPT[-1]
    for i, force in enumerate((-1, 1, 0)):
        t0 = time.perf_counter()
        blk = ex.decode(tok, mtp_enabled=True, force_accept=force)
        ph = ex.last_phase_ms()
        wall_ms = (time.perf_counter() - t0) * 1e3
        assert (blk.emitted, blk.draft_tokens) == plain[i]
        assert set(ph) == {"drafts", "target_pass", "head_and_acceptance", "commit"}
        assert all(v > 0.0 for v in ph.values()), ph
        assert sum(ph.values()) < wall_ms, (ph, wall_ms)
        tok = blk.token_id
    ex.phase_timing(False)

def test_context_capacity_is_a_shape_error_and_leaves_the_session_usable(orc):
    """A prompt that does not fit and a decode past the capacity are refused with Shape before any
    work is enqueued (the reference refuses both, decoder.rs:1177-1181 and its state-capacity
    checks); the session is neither advanced nor poisoned, and reset_session starts over."""
    cfg = tiny_config(max_context_tokens=96)
    be = ctox.B200Backend(0)
    model = OracleModel(orc, cfg, seed=3)
    ex = ctox.B200Executor(be, cfg)
    try:
        model.load_into(ex)
        ex.warmup()
        with pytest.raises(ctox.CtoxError) as e:
            ex.prefill(list(range(1, 200)))
        assert e.value.kind == "Shape" and ex.position() == 0
        ex.prefill(PROMPT)
        tok, steps = PROMPT[-1], 0
        while True:
            position = ex.position()
            try:
                tok = ex.decode(tok, mtp_enabled=True).token_id
            except ctox.CtoxError as err:
                assert err.kind == "Shape" and "capacity" in str(err)
                break
            steps += 1
            assert steps < 200
        assert steps > 10 and ex.position() == position
        assert ex.session_state() == {"pending_accepted": -1, "poisoned": False}
        ex.reset_session()
        ex.prefill(PROMPT)
        assert ex.decode(PROMPT[-1], mtp_enabled=False).token_id == model.greedy(PROMPT, 1)[0][0]
    finally:
        ex.unload()
        assert be.allocated_bytes() == 0
        be.close()

def test_dependent_launch_overlap_changes_no_bit(tmp_path):
    """Every kernel may start before the one in front of it has finished and does part of its work
    ahead of its dependency wait (weights, constants, piece references, committed state). Whatever it
    reads there must not be written by anything still in flight: the blocks, logits and hidden
    states of a full-width 8-layer model are the same, bit for bit, with CTOX_PDL=0, which
    serialises every launch."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    outs = []
    for name, pdl in (("overlapped", None), ("serialised", "0")):
        env = dict(os.environ)
        env["PYTHONPATH"] = os.path.dirname(here) + os.pathsep + env.get("PYTHONPATH", "")
        env.pop("CTOX_PDL", None)
        if pdl is not None:
            env["CTOX_PDL"] = pdl
        path = str(tmp_path / (name + ".npz"))
        r = subprocess.run([sys.executable, os.path.join(here, "pdl_worker.py"), path], env=env, capture_output=True,
                           text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(np.load(path))
    a, b = outs
    assert np.array_equal(a["tokens"], b["tokens"])
    assert np.array_equal(a["logits"], b["logits"]) and np.array_equal(a["hidden"], b["hidden"])


def test_a_peer_that_never_answers_runs_out_the_bounded_wait_and_poisons_the_session(orc):
    """Failure detection without a fault: rank 0 of a two-rank group whose peer never pushes its
    partial sums (host-side set-up, one GPU, no NCCL). The group sum waits for at most the limit
    given here (~10 ms), sets the device error word and returns; the decode call reports
    InvalidState, the session is poisoned until reset_session (engine.rs:594-611), and the context
    stays usable."""
    import time
    be = ctox.B200Backend(0)
    be.tp_debug_silent_peers(2, wait_limit_cycles=20_000_000)
    cfg = tiny_config(num_attention_heads=8, linear_num_key_heads=2, linear_num_value_heads=4)
    model = OracleModel(orc, cfg, seed=3)
    ex = ctox.B200Executor(be, cfg)
    try:
        model.load_into(ex, rank=0, world=2)
        ex.warmup()
        assert be.tp_collective() == "p2p_push"
        t0 = time.time()
        with pytest.raises(ctox.CtoxError) as e:
            ex.prefill(PROMPT)
        assert e.value.kind == "InvalidState" and "wait" in str(e.value)
        assert time.time() - t0 < 5.0, "later waits of the same call must be skipped"
        assert ex.session_state()["poisoned"]
        with pytest.raises(ctox.CtoxError) as e:
            ex.decode(5, mtp_enabled=False)
        assert e.value.kind == "InvalidState" and "reset_session" in str(e.value)
        ex.reset_session()
        assert not ex.session_state()["poisoned"]
        assert be.device_error() == 0  # cleared: the context is usable again
    finally:
        ex.unload()
        be.close()


def test_model_loaded_from_a_ctoxq_container_decodes_like_the_oracle(orc, tmp_path):
    """ModelExecutor::load from a container file (format.rs / loader.rs): the tiny model written as
    CTOXQ, opened with checksums on, loaded by tensor name with the fan-out groups joined, must
    emit the oracle's greedy tokens with speculation on."""
    from ctox_llm_b200 import artifact as A
    cfg = tiny_config(max_draft_tokens=3)
    model = OracleModel(orc, cfg, seed=3)
    path = str(tmp_path / "tiny.ctoxq")
    A.write_ctoxq(path, model.packed_tensors())
    art = A.CtoxqArtifact.open(path)
    be = ctox.B200Backend(0)
    ex = ctox.B200Executor(be, cfg)
    try:
        A.load_into_executor(art, ex)
        ex.warmup()
        want, _, _ = model.greedy(PROMPT, 10)
        ex.prefill(PROMPT)
        tok, got = PROMPT[-1], []
        while len(got) < 10:
            blk = ex.decode(tok, mtp_enabled=True)
            got += blk.emitted
            tok = blk.token_id
        assert got[:10] == want
    finally:
        ex.unload()
        be.close()
        art.close()
