"""GPU parity of the gated-delta recurrence against the CPU oracle, through the C ABI.

Tolerance: relative L2 <= 1e-3 on outputs and on the final state (fp32 state), the bar the path's
north star states; the reference's device check uses out atol 3e-4 / rtol 2e-4 and state 5e-4
(src/bin/cuda_gated_delta_verify.rs:21-26). Measured errors are ~1e-6.
"""
import numpy as np
import pytest
import torch

import ctox_llm_b200 as ctox
from gpu_util import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-3
TIGHT = 2e-5


@pytest.fixture(scope="module")
def be():
    b = ctox.B200Backend(0)
    yield b
    b.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def run_scan(be, q, k, v, g, beta, state, tokens, heads, qk_heads, kd, vd, in_place=True):
    dq, dk, dv, dg, db, ds = (dev(x) for x in (q, k, v, g, beta, state))
    dso = ds if in_place else torch.full_like(ds, float("nan"))
    out = torch.empty(tokens * heads * vd, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    be.gated_delta_scan(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), db.data_ptr(),
                        ds.data_ptr(), dso.data_ptr(), out.data_ptr(), tokens, heads, qk_heads, kd, vd)
    be.synchronize()
    return out.cpu().numpy().reshape(tokens, heads * vd), dso.cpu().numpy(), ds.cpu().numpy()


def test_reference_golden_step_and_sequence(be):
    # reference.rs:589-627
    out, st, _ = run_scan(be, [1.0, 2.0, -1.0, 0.5, 1.5, -0.5], [0.5, -1.0, 2.0, 1.0, -0.5, 0.25],
                          [1.0, -2.0, 0.5, 1.5], [-0.2, -0.7], [0.6, 0.25],
                          [x / 100.0 for x in range(1, 13)], 1, 2, 2, 3, 2)
    assert np.all(np.abs(out.reshape(-1) - [-0.20637584, 0.44671553, 0.0062854784, -0.0195187]) <= 2e-6)
    assert np.all(np.abs(st - [0.1356092, -0.24969745, -0.23028184, 0.56489336, 0.5506241, -1.0151644,
                               0.13890404, 0.3613783, -0.00737885, -0.11116721, 0.08066015,
                               0.14000311]) <= 2e-6)
    # reference.rs:755-799
    out, st, _ = run_scan(be, [1.0, 2.0, 0.5, -1.0, -1.0, 0.25, 2.0, 1.0],
                          [0.5, -0.25, 1.0, 0.5, 0.75, 1.25, -0.5, 2.0],
                          [1.0, -1.0, 0.5, 2.0, -2.0, 0.25, 1.5, -0.5], [-0.2, -0.4, -0.1, -0.3],
                          [0.6, 0.25, 0.8, 0.4], [x / 100.0 for x in range(1, 9)], 2, 2, 2, 2, 2)
    assert np.all(np.abs(out.reshape(-1) - [0.018123373, 0.02589053, -0.019077633, -0.021197364,
                                            -0.0373289, 0.32707188, 0.17473069, 0.24809137]) <= 2e-6)
    assert np.all(np.abs(st - [-0.35503477, -0.36432835, -1.6378022, 0.44982785, -0.04187046,
                               0.41027403, 0.636288, -0.03601411]) <= 2e-6)


def config2_inputs(tokens, heads, qk_heads, seed):
    """BASELINE config 2: state ~N(0,0.02); q,k ~N(0,1) L2-normalised; v ~N(0,1);
    g = log(sigmoid(N(2,1))); beta = sigmoid(N(0,1))."""
    rng = np.random.Generator(np.random.Philox(key=[seed, 2]))
    q = rng.standard_normal((tokens, qk_heads, 128)).astype(np.float32)
    k = rng.standard_normal((tokens, qk_heads, 128)).astype(np.float32)
    q /= np.linalg.norm(q, axis=-1, keepdims=True)
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.standard_normal((tokens, heads, 128)).astype(np.float32)
    g = np.log(1.0 / (1.0 + np.exp(-rng.normal(2.0, 1.0, (tokens, heads))))).astype(np.float32)
    beta = (1.0 / (1.0 + np.exp(-rng.standard_normal((tokens, heads))))).astype(np.float32)
    state = (rng.standard_normal((heads, 128, 128)) * 0.02).astype(np.float32)
    return q, k, v, g, beta, state


@pytest.mark.parametrize("tokens", [1, 4, 5, 11])
@pytest.mark.parametrize("qk_heads", [16, 48])
def test_config2_shape_matches_oracle(be, orc, tokens, qk_heads):
    heads = 48
    q, k, v, g, beta, state = config2_inputs(tokens, heads, qk_heads, seed=tokens)
    rep = heads // qk_heads
    exp_out, exp_state = orc.recurrent_gated_delta_sequence(
        np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1), v, g, beta, state, tokens, heads, 128, 128)
    out, st, st_in = run_scan(be, q, k, v, g, beta, state, tokens, heads, qk_heads, 128, 128,
                              in_place=False)
    assert rel_l2(out, exp_out) <= TIGHT
    assert rel_l2(st, exp_state) <= TIGHT
    assert np.array_equal(st_in.reshape(-1), state.reshape(-1)), "state_in must stay untouched"
    out2, st2, _ = run_scan(be, q, k, v, g, beta, state, tokens, heads, qk_heads, 128, 128)
    assert np.array_equal(out, out2) and np.array_equal(st, st2)


def test_scan_equals_step_by_step_and_layers_back_to_back(be, orc):
    """Scan over T tokens equals T single-token calls bit for bit (the reference's device check,
    benchmarks/cuda/sm86-gated-delta-scan-20260826.json:16-21), over several layers' states."""
    heads, tokens, layers = 48, 4, 3
    for layer in range(layers):
        q, k, v, g, beta, state = config2_inputs(tokens + 1, heads, 16, seed=100 + layer)
        out, st, _ = run_scan(be, q[:tokens], k[:tokens], v[:tokens], g[:tokens], beta[:tokens], state,
                              tokens, heads, 16, 128, 128)
        cur = state
        outs = []
        for t in range(tokens):
            o, cur, _ = run_scan(be, q[t:t + 1], k[t:t + 1], v[t:t + 1], g[t:t + 1], beta[t:t + 1], cur,
                                 1, heads, 16, 128, 128)
            outs.append(o[0])
        assert np.array_equal(np.stack(outs), out) and np.array_equal(cur, st)
        # then the decode token (T = 1) on the verified state
        o1, st1, _ = run_scan(be, q[tokens:], k[tokens:], v[tokens:], g[tokens:], beta[tokens:], st, 1,
                              heads, 16, 128, 128)
        eo, es = orc.recurrent_gated_delta_sequence(
            np.repeat(q[tokens:], 3, axis=1), np.repeat(k[tokens:], 3, axis=1), v[tokens:], g[tokens:],
            beta[tokens:], st, 1, heads, 128, 128)
        assert rel_l2(o1, eo) <= TIGHT and rel_l2(st1, es) <= TIGHT

def test_layers_in_one_launch_equal_one_launch_per_layer(be):
    """ctox_gated_delta_scan_layers over 5 layers (the form of the executor's prefix re-scan) gives the
    bits of 5 single-layer calls, with and without the output array, and leaves state_in untouched."""
    heads, qk, tokens, layers = 48, 16, 3, 5
    ins = [config2_inputs(tokens, heads, qk, seed=300 + l) for l in range(layers)]
    want_out, want_state = [], []
    for q, k, v, g, beta, state in ins:
        o, st, _ = run_scan(be, q, k, v, g, beta, state, tokens, heads, qk, 128, 128, in_place=False)
        want_out.append(o)
        want_state.append(st)
    dq, dk, dv, dg, db, ds = (dev(np.stack([x[i] for x in ins])) for i in range(6))
    dso = torch.full_like(ds, float("nan"))
    out = torch.full((layers * tokens * heads * 128,), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    be.gated_delta_scan_layers(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), db.data_ptr(),
                               ds.data_ptr(), dso.data_ptr(), out.data_ptr(), layers, tokens, heads, qk)
    be.synchronize()
    assert np.array_equal(out.cpu().numpy().reshape(layers, tokens, heads * 128), np.stack(want_out))
    assert np.array_equal(dso.cpu().numpy().reshape(layers, -1), np.stack([s.reshape(-1) for s in want_state]))
    assert np.array_equal(ds.cpu().numpy().reshape(layers, -1), np.stack([x[5].reshape(-1) for x in ins]))
    dso2 = torch.full_like(ds, float("nan"))
    be.gated_delta_scan_layers(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), db.data_ptr(),
                               ds.data_ptr(), dso2.data_ptr(), 0, layers, tokens, heads, qk)
    be.synchronize()
    assert torch.equal(dso, dso2)
    with pytest.raises(ctox.CtoxError) as e:
        be.gated_delta_scan_layers(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), db.data_ptr(),
                                   ds.data_ptr(), dso2.data_ptr(), 0, 0, tokens, heads, qk)
    assert e.value.kind == "Shape"


def test_prepare_matches_oracle(be, orc):
    rng = np.random.default_rng(3)
    tokens, heads = 5, 48
    a = rng.standard_normal((tokens, heads)).astype(np.float32) * 3
    a[0, 0] = 25.0  # softplus switch-over (decoder.rs:29-35)
    b = rng.standard_normal((tokens, heads)).astype(np.float32)
    a_log = rng.standard_normal(heads).astype(np.float32) * 0.5
    dt_bias = rng.standard_normal(heads).astype(np.float32)
    da, db, dal, ddt = dev(a), dev(b), dev(a_log), dev(dt_bias)
    g = torch.empty(tokens * heads, device="cuda")
    beta = torch.empty(tokens * heads, device="cuda")
    torch.cuda.synchronize()
    be.gated_delta_prepare(da.data_ptr(), db.data_ptr(), dal.data_ptr(), ddt.data_ptr(), g.data_ptr(),
                           beta.data_ptr(), tokens, heads)
    be.synchronize()
    for t in range(tokens):
        eg, eb = orc.gated_delta_prepare(a[t], b[t], a_log, dt_bias)
        assert np.allclose(g.cpu().numpy().reshape(tokens, heads)[t], eg, rtol=2e-6, atol=1e-7)
        assert np.allclose(beta.cpu().numpy().reshape(tokens, heads)[t], eb, rtol=2e-6, atol=1e-7)


def test_bad_arguments_are_shape_errors(be):
    x = torch.zeros(16, device="cuda")
    with pytest.raises(ctox.CtoxError) as e:
        be.gated_delta_scan(*([x.data_ptr()] * 8), 0, 48, 16)
    assert e.value.kind == "Shape"
    with pytest.raises(ctox.CtoxError) as e:
        be.gated_delta_scan(*([x.data_ptr()] * 8), 1, 48, 5)
    assert e.value.kind == "Shape"
    with pytest.raises(ctox.CtoxError) as e:
        be.gated_delta_scan(0, *([x.data_ptr()] * 7), 1, 48, 16)
    assert e.value.kind == "Shape"


def test_f16_resident_state_matches_oracle(be, orc):
    """The FP16-resident state mode (reference.rs:299-373): outputs within 2e-5 of the oracle and the
    binary16 state equal to the oracle's except for values where an fp32 last-bit difference straddles a
    rounding boundary (a few binary16 steps at most, on well under 1 % of the elements: the device adds
    the 128 products of a column as four partial sums, the scalar code as one). The reference's
    own drift test for this mode (reference.rs:629-722) bounds the distance to the fp32 state."""
    heads, qk, tokens = 48, 16, 5
    q, k, v, g, beta, state = config2_inputs(tokens, heads, qk, seed=77)
    bits = state.astype(np.float16).view(np.uint16).reshape(-1)
    dq, dk, dv, dg, db = (dev(x) for x in (q, k, v, g, beta))
    ds = torch.from_numpy(bits.view(np.float16).copy()).cuda()
    dso = torch.zeros_like(ds)
    out = torch.empty(tokens * heads * 128, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    be.gated_delta_scan_f16_state(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), db.data_ptr(),
                                  ds.data_ptr(), dso.data_ptr(), out.data_ptr(), tokens, heads, qk)
    be.synchronize()
    st, exp_out = bits.copy(), []
    for t in range(tokens):
        o, st = orc.recurrent_gated_delta_step_f16_state(
            np.repeat(q[t], 3, axis=0), np.repeat(k[t], 3, axis=0), v[t], g[t], beta[t], st, heads, 128, 128)
        exp_out.append(o)
    got = out.cpu().numpy().reshape(tokens, -1)
    assert rel_l2(got, np.stack(exp_out)) <= 2e-5
    got_state = dso.cpu().numpy().view(np.uint16).reshape(-1)
    diff = got_state != st
    assert diff.mean() < 5e-3, diff.mean()  # measured 1.2e-3 after 5 tokens
    a = got_state.view(np.float16).astype(np.float32)
    b = st.view(np.float16).astype(np.float32)
    # a one-step difference at one token is carried (and rescaled by the decay) through the following
    # tokens: bound it by one binary16 step at the magnitude of the largest state element
    assert np.max(np.abs(a - b)) <= np.max(np.abs(b)) * 2.0 ** -10
    assert torch.equal(ds.cpu(), torch.from_numpy(bits.view(np.float16).copy())), "state_in must stay untouched"
    # fp32 state of the same inputs stays close (the drift the reference accepts for this mode)
    _, st32, _ = run_scan(be, q, k, v, g, beta, state, tokens, heads, qk, 128, 128)
    assert np.max(np.abs(st32.reshape(-1) - a)) <= 5e-3
    with pytest.raises(ctox.CtoxError) as e:
        be._check(be._lib.ctox_gated_delta_scan_f16_state(be._ctx, *[ctypes_ptr(out)] * 8, 1, 48, 16, 64, 64))
    assert e.value.kind == "UnsupportedOperation"


def ctypes_ptr(t):
    import ctypes
    return ctypes.c_void_p(t.data_ptr())
