"""Pins the CPU oracle to the reference's own known-answer tests.

Each case restates one `#[test]` of the reference crate (models/qwen38_27b/src/),
with the same inputs, expected values and tolerance.
"""
import math

import numpy as np
import pytest


def close(a, b, tol):
    a, b = np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)
    assert a.shape == b.shape
    assert np.all(np.abs(a - b) <= tol), (a, b)


# reference.rs:531-553
def test_qwen_norm_swiglu_gated_norm(orc):
    values = [1.0, -2.0, 3.0, -4.0]
    norm = orc.rms_norm_1p_weight(values, 1, 4, [0.1, -0.2, 0.3, -0.4], 1e-6)
    close(norm, [0.4016632, -0.5842374, 1.4240787, -0.8763561], 2e-6)
    close(orc.swiglu([0.0, 1.0, -1.0], [2.0, 3.0, 4.0]), [0.0, 2.1931758, -1.0757657], 2e-6)
    gated = orc.rms_norm_gated(values, [0.1, -0.2, 0.3, -0.4], 1, 4, [0.5, 1.0, 1.5, 2.0], 1e-6)
    close(gated, [0.009584765, 0.06575096, 0.28317162, 0.4689234], 2e-6)


# reference.rs:555-572
def test_partial_rope(orc):
    q, k = orc.apply_partial_rope([1.0, 2.0, 3.0, 4.0, 9.0, 10.0], [-1.0, 0.5, 2.0, -3.0, 7.0, 8.0],
                                  1, 1, 6, 4, 3, 10_000.0)
    close(q, [-1.4133525, 1.8791181, -2.8288574, 4.0581913, 9.0, 10.0], 2e-6)
    close(k, [0.70775247, 0.5897615, -2.121105, -2.9836524, 7.0, 8.0], 2e-6)
    close(q[4:], [9.0, 10.0], 0.0)
    close(k[4:], [7.0, 8.0], 0.0)


# reference.rs:574-587
def test_conv_update(orc):
    out, state = orc.causal_conv_silu_update(
        [5.0, -5.0], [1.0, 2.0, 3.0, 4.0, -1.0, -2.0, -3.0, -4.0],
        [0.1, 0.2, 0.3, 0.4, 0.4, 0.3, 0.2, 0.1], 2, 4)
    close(state, [2.0, 3.0, 4.0, 5.0, -2.0, -3.0, -4.0, -5.0], 0.0)
    close(out, [3.928055, -0.14227761], 2e-6)


# reference.rs:589-627
def test_delta_step(orc):
    state = [v / 100.0 for v in range(1, 13)]
    out, st = orc.recurrent_gated_delta_step(
        [1.0, 2.0, -1.0, 0.5, 1.5, -0.5], [0.5, -1.0, 2.0, 1.0, -0.5, 0.25], [1.0, -2.0, 0.5, 1.5],
        [-0.2, -0.7], [0.6, 0.25], state, 2, 3, 2)
    close(out, [-0.20637584, 0.44671553, 0.0062854784, -0.0195187], 2e-6)
    close(st, [0.1356092, -0.24969745, -0.23028184, 0.56489336, 0.5506241, -1.0151644, 0.13890404,
               0.3613783, -0.00737885, -0.11116721, 0.08066015, 0.14000311], 2e-6)


# reference.rs:755-799
def test_delta_sequence(orc):
    state = [v / 100.0 for v in range(1, 9)]
    out, st = orc.recurrent_gated_delta_sequence(
        [1.0, 2.0, 0.5, -1.0, -1.0, 0.25, 2.0, 1.0], [0.5, -0.25, 1.0, 0.5, 0.75, 1.25, -0.5, 2.0],
        [1.0, -1.0, 0.5, 2.0, -2.0, 0.25, 1.5, -0.5], [-0.2, -0.4, -0.1, -0.3], [0.6, 0.25, 0.8, 0.4],
        state, 2, 2, 2, 2)
    close(out.reshape(-1), [0.018123373, 0.02589053, -0.019077633, -0.021197364, -0.0373289,
                            0.32707188, 0.17473069, 0.24809137], 2e-6)
    close(st, [-0.35503477, -0.36432835, -1.6378022, 0.44982785, -0.04187046, 0.41027403, 0.636288,
               -0.03601411], 2e-6)


# reference.rs:629-722
def test_fp16_state_drift_bounds(orc):
    heads, key_dim, value_dim = 2, 4, 3
    f32_state = np.zeros(heads * key_dim * value_dim, dtype=np.float32)
    f16_state = np.zeros(f32_state.size, dtype=np.uint16)
    sq_err = sq_sig = 0.0
    max_err = 0.0
    f = np.float32
    for token in range(512):
        q = [math.sin(float(f((token * 17 + i * 11 + 1)) * f(0.013))) for i in range(heads * key_dim)]
        k = [math.cos(float(f((token * 13 + i * 7 + 3)) * f(0.017))) for i in range(heads * key_dim)]
        v = [0.75 * math.sin(float(f((token * 19 + i * 5 + 2)) * f(0.011)))
             for i in range(heads * value_dim)]
        g = [-0.01 - 0.04 * ((token + h * 3) % 5) for h in range(heads)]
        b = [0.15 + 0.15 * ((token + h) % 5) for h in range(heads)]
        exp, f32_state = orc.recurrent_gated_delta_step(q, k, v, g, b, f32_state, heads, key_dim,
                                                        value_dim)
        act, f16_state = orc.recurrent_gated_delta_step_f16_state(q, k, v, g, b, f16_state, heads,
                                                                  key_dim, value_dim)
        err = np.abs(exp - act)
        max_err = max(max_err, float(err.max()))
        sq_err += float((err.astype(np.float64) ** 2).sum())
        sq_sig += float((exp.astype(np.float64) ** 2).sum())
    assert max_err < 0.01
    assert math.sqrt(sq_err / max(sq_sig, 1e-300)) < 0.005

    channels = kernel = 4
    weights = [math.cos(float(f(i + 1) * f(0.031))) * 0.25 for i in range(channels * kernel)]
    c32 = np.zeros(channels * kernel, dtype=np.float32)
    c16 = np.zeros(channels * kernel, dtype=np.uint16)
    for token in range(512):
        inp = [math.sin(float(f(token * 7 + c * 3) * f(0.019))) for c in range(channels)]
        exp, c32 = orc.causal_conv_silu_update(inp, c32, weights, channels, kernel)
        act, c16 = orc.causal_conv_silu_update_f16_state(inp, c16, weights, channels, kernel)
        close(exp, act, 5e-4)


# reference.rs:724-753
def test_gqa_and_sigmoid_gate(orc):
    query = [1.0, 0.0, -1.0, 0.5, 1.0, 0.0, 0.0, 1.0, 1.0, -1.0, 0.5, 2.0]
    key = [0.2, 0.4, -0.5, 1.0, -0.25, 0.75]
    value = [1.0, 2.0, 3.0, -1.0, 0.5, 2.0]
    out = orc.grouped_query_attention(query, key, value, 2, 1, 2, 2, 3, 0)
    close(out, [1.0, 2.0, 3.0, 1.0, 2.0, 3.0, 0.07204375, 1.3040327, 2.5360217, -0.37731764,
                0.9670118, 2.3113413], 2e-6)
    gated = orc.sigmoid_gate(out, [0.0] * 12)
    assert np.all(np.abs(gated - out * 0.5) <= 1e-7)


# quant.rs:211-264
def test_quant_roundtrip_bounds(orc):
    fixture = np.array([math.sin((i - 31.5) / 31.5) for i in range(64)], dtype=np.float32)
    fixture = np.sin(((np.arange(64, dtype=np.float32) - np.float32(31.5)) / np.float32(31.5)))
    for dtype, bound in ((orc.Q2B64, 0.34), (orc.Q4B64, 0.07)):
        packed = orc.quantize_matrix(dtype, fixture.reshape(1, 64))
        again = orc.quantize_matrix(dtype, fixture.reshape(1, 64))
        assert np.array_equal(packed, again)
        deq = orc.dequantize_blocks(dtype, packed)[0]
        assert np.all(np.abs(deq - fixture) <= bound)
    bad = fixture.copy()
    bad[3] = np.nan
    with pytest.raises(orc.OracleError) as e:
        orc.quantize_matrix(orc.Q2B64, bad.reshape(1, 64))
    assert e.value.kind == "InvalidArtifact"
    scale, codes = orc.a8_quantize_block(fixture)
    assert codes[0] == -127 and codes[63] == 127
    assert np.all(np.abs(codes.astype(np.float32) * np.float32(scale) - fixture) <= scale * 0.501)
    scale, codes = orc.a8_quantize_block(np.zeros(64, dtype=np.float32))
    assert scale == 0.0 and not codes.any()


def test_f16_all_bit_patterns(orc):
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    got = np.array([orc.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    finite = ~np.isnan(ref)
    assert np.array_equal(ref[finite].view(np.uint32), got[finite].view(np.uint32))
    assert np.all(np.isnan(got[~finite]))
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 4000),
        ref[np.isfinite(ref)][::37],
        np.array([65504.0, 65519.9, 65520.0, 1e9, 5.96e-8, 2.98e-8, 2.99e-8, 0.0, -0.0],
                 dtype=np.float32)]).astype(np.float32)
    with np.errstate(over="ignore"):
        expect = vals.astype(np.float16).view(np.uint16)
    got = np.array([orc.f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(expect, got)


# sampler.rs:180-252
def test_sampler_cases(orc):
    assert orc.sample_with_draw([-1.0, 3.0, 2.0], 0.0, 40, 0.95, 0.0) == 1
    logits = [-0.5, 0.25, 1.5, 0.75]
    assert orc.sample_with_draw(logits, 0.8, 4, 0.9, 0.625) == orc.sample_with_draw(
        logits, 0.8, 4, 0.9, 0.625)
    # tied candidates use the later token, like greedy argmax
    assert orc.sample_with_draw([2.0, 2.0], 1.0, 1, 1.0, 0.0) == 1
    assert orc.greedy_token([2.0, 2.0]) == 1
    # fail-closed draws and scaled logits
    tiny = float(np.array([1], dtype=np.uint32).view(np.float32)[0])
    with pytest.raises(orc.OracleError):
        orc.sample_with_draw([1.0, 0.0], tiny, 2, 1.0, 0.5)
    with pytest.raises(orc.OracleError):
        orc.sample_with_draw([1.0], 1.0, 2, 1.0, 1.0)
    # same seed, same sequence; draws lie in [0, 1)
    a, b = orc.Pcg32(42), orc.Pcg32(42)
    seq = [a.next_f32() for _ in range(32)]
    assert seq == [b.next_f32() for _ in range(32)]
    assert all(0.0 <= x < 1.0 for x in seq)
    # PCG-XSH-RR reference stream for seed 0 (state/increment from sampler.rs:153-169)
    state = (0 + 0x853C49E6748FEA9B) & (2**64 - 1)
    outs = []
    for _ in range(4):
        old = state
        state = (old * 6364136223846793005 + 1442695040888963407) & (2**64 - 1)
        xs = (((old >> 18) ^ old) >> 27) & 0xFFFFFFFF
        rot = old >> 59
        outs.append(((xs >> rot) | (xs << ((32 - rot) & 31))) & 0xFFFFFFFF)
    g = orc.Pcg32(0)
    assert [g.next_u32() for _ in range(3)] == outs[1:]


# engine.rs:1212-1246, 1248-1305, 1346-1413
def test_verify_greedy_mtp_cases(orc):
    target = [0.0, 1.0, 2.0]
    drafts = [[0.0, 1.0, 2.0], [0.0, 1.0, 2.0], [0.0, 2.0, 1.0], [0.0, 1.0, 2.0]]
    assert orc.verify_greedy_mtp_logits(drafts, [target] * 4, [0.0, 2.0, 1.0]) == (2, 3, [2, 2])
    assert orc.verify_greedy_mtp_logits([target] * 4, [target] * 4, [0.0, 2.0, 1.0]) == (
        1, 4, [2, 2, 2, 2])
    assert orc.verify_greedy_mtp_tokens([2, 2, 1, 2], [2, 2, 0, 2], 1) == (0, 3, [2, 2])
    assert orc.verify_greedy_mtp_tokens([2, 1], [2, 1], 0) == (0, 2, [2, 1])
    # restricted draft vocabulary maps the local argmax through the id table
    target6 = [0.0, 0.1, 0.2, 0.3, 2.0, 0.4]
    assert orc.verify_greedy_mtp_logits([[0.0, 3.0]], [target6], [0.0, 0.1, 0.2, 3.0, 0.4, 0.5],
                                        draft_token_ids=[[1, 4]]) == (3, 1, [4])
    miss = [0.0, 0.1, 0.2, 0.3, 0.4, 4.0]
    assert orc.verify_greedy_mtp_logits([[0.0, 3.0]], [miss], [0.0, 0.1, 0.2, 3.0, 0.4, 0.5],
                                        draft_token_ids=[[1, 4]]) == (5, 1, [])


def test_softplus_and_prepare(orc):
    assert orc.softplus(25.0) == 25.0
    assert abs(orc.softplus(0.0) - math.log(2.0)) < 1e-7
    g, beta = orc.gated_delta_prepare([0.5], [0.0], [0.0], [0.25])
    assert abs(beta[0] - 0.5) < 1e-7
    assert abs(g[0] + math.log1p(math.exp(0.75))) < 1e-6
    rep = orc.repeat_heads(np.arange(4, dtype=np.float32), 2, 6, 2)
    assert rep.tolist() == [0, 1, 0, 1, 0, 1, 2, 3, 2, 3, 2, 3]
