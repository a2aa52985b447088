"""GPU parity of the top-k / top-p sampler against the oracle's Sampler::sample_with_draw
(sampler.rs:65-144): same token for the same draw, including ties (later token id first), top_k
larger than the vocabulary, a nucleus of one candidate, and the fail-closed argument checks."""
import numpy as np
import pytest
import torch

import ctox_llm_b200 as ctox

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    b = ctox.B200Backend(0)
    yield b
    b.close()


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def test_sampled_token_matches_the_oracle(be, orc):
    rng = np.random.default_rng(17)
    checked = 0
    for case in range(60):
        n = int(rng.choice([37, 1000, 5000, 50_000]))
        logits = (rng.standard_normal(n) * rng.uniform(0.5, 6.0)).astype(np.float32)
        if case % 5 == 0:  # ties, also across the top_k boundary
            logits = np.round(logits).astype(np.float32)
        temperature = float(rng.choice([0.3, 0.7, 1.0, 1.5]))
        top_k = int(rng.choice([1, 2, 8, 50, 256, 1024]))
        top_p = float(rng.choice([0.1, 0.5, 0.9, 1.0]))
        draw = float(np.float32(rng.uniform(0.0, 1.0)))
        if draw >= 1.0:
            draw = 0.5
        d = _dev(logits)
        got = be.sample_topk_topp(d.data_ptr(), n, temperature, top_k, top_p, draw)
        exp = orc.sample_with_draw(logits, temperature, top_k, top_p, draw)
        assert got == exp, (case, n, temperature, top_k, top_p, draw, got, exp)
        checked += 1
    assert checked == 60


def test_temperature_zero_is_greedy_with_later_index_on_ties(be, orc):
    logits = np.zeros(4096, dtype=np.float32)
    logits[[7, 300, 4000]] = 3.0
    d = _dev(logits)
    assert be.sample_topk_topp(d.data_ptr(), logits.size, 0.0, 5, 0.9, 0.25) == 4000 == orc.greedy_token(logits)


def test_all_equal_logits_take_the_largest_ids(be, orc):
    logits = np.full(3000, 1.25, dtype=np.float32)
    d = _dev(logits)
    for draw in (0.0, 0.33, 0.999):
        got = be.sample_topk_topp(d.data_ptr(), logits.size, 1.0, 4, 1.0, draw)
        assert got == orc.sample_with_draw(logits, 1.0, 4, 1.0, draw)
        assert got >= 2996


def test_arguments_fail_closed(be):
    d = _dev(np.arange(100))
    for args in [(1.0, 0, 0.9, 0.5), (1.0, 2000, 0.9, 0.5)]:
        with pytest.raises(ctox.CtoxError) as e:
            be.sample_topk_topp(d.data_ptr(), 100, *args)
        assert e.value.kind == "UnsupportedOperation"
    for args in [(1.0, 5, 0.0, 0.5), (1.0, 5, 1.5, 0.5), (1.0, 5, 0.9, 1.0), (1.0, 5, 0.9, -0.1), (-1.0, 5, 0.9, 0.5),
                 (float("nan"), 5, 0.9, 0.5)]:
        with pytest.raises(ctox.CtoxError) as e:
            be.sample_topk_topp(d.data_ptr(), 100, *args)
        assert e.value.kind == "InvalidArtifact"
    bad = np.arange(100, dtype=np.float32)
    bad[3] = np.inf
    with pytest.raises(ctox.CtoxError) as e:
        be.sample_topk_topp(_dev(bad).data_ptr(), 100, 1.0, 5, 0.9, 0.5)
    assert e.value.kind == "InvalidArtifact"
