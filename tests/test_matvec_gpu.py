"""GPU parity of the fused Q2/Q4 dequantize-matvec against the CPU oracle, through the C ABI.

Tolerance: relative L2 <= 1e-3 (fp32 accumulation), the bar the path's north star states; the
reference's own device-vs-oracle check uses atol 2e-2 + rtol 1e-3 (src/bin/cuda_bench.rs:53-56).
Measured errors are ~1e-6 (Q4) to ~2e-5 (Q2, whose partial sums cancel more and whose tensor-core
accumulation rounds toward zero), so most cases assert a much tighter 5e-5.
"""
import os

import numpy as np
import pytest

import ctox_llm_b200 as ctox
from ctox_llm_b200 import synthetic
from gpu_util import rel_l2, to_oracle_op

pytestmark = pytest.mark.gpu
TOL = 1e-3
TIGHT = 5e-5
f32 = np.float32


@pytest.fixture(scope="module")
def be():
    b = ctox.B200Backend(0)
    yield b
    assert b.allocated_bytes() == 0, "device memory leaked by the matvec tests"
    b.close()


def reference_fixture(orc, dtype, rows, columns, activation):
    # the reference's SIMD-vs-scalar fixture (backend/cpu.rs:751-812)
    phase = np.arange(rows * columns, dtype=np.float32)
    values = (np.sin((phase * f32(0.013579)).astype(np.float32)) * f32(0.75)).astype(np.float32)
    weights = orc.quantize_matrix(dtype, values.reshape(rows, columns))
    idx = np.arange(columns)
    r = np.arange(rows)
    return ctox.FusedMatVec(
        dtype=dtype, weights=weights, rows=rows, columns=columns,
        input=np.cos(idx.astype(np.float32) * f32(0.03125)).astype(np.float32),
        s_in=(f32(0.75) + f32(0.005) * (idx % 7).astype(np.float32)).astype(np.float32),
        s_out=(f32(1.25) - f32(0.05) * (r % 5).astype(np.float32)).astype(np.float32),
        bias=(np.sin(r.astype(np.float32) * f32(1.7)) * f32(0.1)).astype(np.float32),
        activation=activation)


@pytest.mark.parametrize("dtype,rows,blocks,act", [
    (ctox.Q2B64, 7, 3, ctox.ACT_SILU), (ctox.Q4B64, 7, 3, ctox.ACT_SILU),
    (ctox.Q2B64, 3, 1, ctox.ACT_IDENTITY), (ctox.Q4B64, 3, 1, ctox.ACT_IDENTITY),
    (ctox.Q2B64, 257, 8, ctox.ACT_IDENTITY), (ctox.Q4B64, 257, 8, ctox.ACT_SILU)])
def test_reference_fixture_cases(be, orc, dtype, rows, blocks, act):
    op = reference_fixture(orc, dtype, rows, blocks * 64, act)
    expect = orc.fused_matvec(to_oracle_op(orc, op))
    got = be.fused_matvec(op)
    assert np.all(np.abs(got - expect) <= 2e-4 + 1e-3 * np.abs(expect))
    assert rel_l2(got, expect) <= TIGHT


@pytest.mark.parametrize("tag", ["q2", "q4"])
def test_golden_fixture_from_reference_python(be, tag):
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_fixtures.npz"))
    dtype = ctox.Q2B64 if tag == "q2" else ctox.Q4B64
    rows, columns = gold[f"{tag}_values"].shape
    for act, key in ((ctox.ACT_IDENTITY, "y"), (ctox.ACT_SILU, "y_silu")):
        op = ctox.FusedMatVec(dtype, gold[f"{tag}_packed"], rows, columns, gold[f"{tag}_x"],
                              s_in=gold[f"{tag}_s_in_f16"], s_out=gold[f"{tag}_s_out_f16"],
                              bias=gold[f"{tag}_bias"], activation=act)
        assert rel_l2(be.fused_matvec(op), gold[f"{tag}_{key}"]) <= TIGHT


def synthetic_op(dtype, rows, columns, seed, scales=True, act=ctox.ACT_IDENTITY):
    return ctox.FusedMatVec(
        dtype=dtype, weights=synthetic.packed_weights(dtype, rows, columns, seed), rows=rows,
        columns=columns, input=synthetic.activations(columns, seed),
        s_in=synthetic.recovery_scales_f16(columns, seed, 3) if scales else None,
        s_out=synthetic.recovery_scales_f16(rows, seed, 4) if scales else None,
        bias=synthetic.bias(rows, seed) if scales else None, activation=act)


@pytest.mark.parametrize("dtype,rows,columns", [
    (ctox.Q4B64, 1024, 5120), (ctox.Q2B64, 5120, 1024), (ctox.Q4B64, 48, 5120),
    (ctox.Q2B64, 16, 17408), (ctox.Q4B64, 6144 + 5, 64), (ctox.Q2B64, 33, 192)])
@pytest.mark.parametrize("kernel", [ctox.KERNEL_STREAM, ctox.KERNEL_ROWWARP])
def test_both_kernels_match_oracle(be, orc, dtype, rows, columns, kernel):
    op = synthetic_op(dtype, rows, columns, seed=rows + columns, act=ctox.ACT_SILU)
    expect = orc.fused_matvec(to_oracle_op(orc, op), threads=8)
    mv = be.prepare_fused_matvec(op, keep_canonical=True)
    try:
        got = mv.dispatch_host(op.input, kernel=kernel)
        again = mv.dispatch_host(op.input, kernel=kernel)
    finally:
        mv.destroy()
    assert rel_l2(got, expect) <= TIGHT, rel_l2(got, expect)
    assert np.array_equal(got, again), "same input must give bit-identical output"


def test_config0_full_size_q4_and_q2(be, orc):
    """BASELINE config 0: Q4 17408x5120 and Q2 5120x17408, f32 activations ~N(0,1)."""
    for dtype, rows, columns in ((ctox.Q4B64, 17408, 5120), (ctox.Q2B64, 5120, 17408)):
        for scales in (False, True):
            op = synthetic_op(dtype, rows, columns, seed=0, scales=scales)
            expect = orc.fused_matvec(to_oracle_op(orc, op), threads=16)
            got = be.fused_matvec(op)
            err = rel_l2(got, expect)
            assert err <= TOL, err
            assert err <= TIGHT, err


def test_mixed_segments_match_pure_and_oracle(be, orc):
    columns = 256
    q2 = synthetic.packed_weights(ctox.Q2B64, 40, columns, 11)
    q4 = synthetic.packed_weights(ctox.Q4B64, 24, columns, 12)
    x = synthetic.activations(columns, 13)
    weights = np.concatenate([q2, q4])
    segs = [ctox.Segment(0, ctox.Q2B64, 0, 40, 0, q2.size),
            ctox.Segment(1, ctox.Q4B64, 40, 64, q2.size, q4.size)]
    s_out = synthetic.recovery_scales_f16(64, 14, 4)
    mixed = ctox.FusedMatVec(ctox.MIXED_Q2Q4B64, weights, 64, columns, x, segments=segs, s_out=s_out)
    got = be.fused_matvec(mixed)
    expect = orc.fused_matvec(to_oracle_op(orc, mixed))
    assert rel_l2(got, expect) <= TIGHT
    a = be.fused_matvec(ctox.FusedMatVec(ctox.Q2B64, q2, 40, columns, x, s_out=s_out[:80]))
    b = be.fused_matvec(ctox.FusedMatVec(ctox.Q4B64, q4, 24, columns, x, s_out=s_out[80:]))
    assert np.array_equal(got[:40], a) and np.array_equal(got[40:], b)


def test_fanout_equals_independent(be, orc):
    x = synthetic.activations(320, 21)
    s_in = synthetic.recovery_scales_f16(320, 21, 3)
    ops = [ctox.FusedMatVec(ctox.Q2B64, synthetic.packed_weights(ctox.Q2B64, 20, 320, 22), 20, 320, x,
                            s_in=s_in),
           ctox.FusedMatVec(ctox.Q4B64, synthetic.packed_weights(ctox.Q4B64, 50, 320, 23), 50, 320, x,
                            s_in=s_in)]
    outs = be.fused_matvec_fanout(ops)
    for o, op in zip(outs, ops):
        assert np.array_equal(o, be.fused_matvec(op))
        assert rel_l2(o, orc.fused_matvec(to_oracle_op(orc, op))) <= TIGHT
    with pytest.raises(ctox.CtoxError) as e:
        be.fused_matvec_fanout([])
    assert e.value.kind == "Shape"


@pytest.mark.parametrize("positions", [1, 2, 4, 5, 8, 16])
@pytest.mark.parametrize("dtype", [ctox.Q2B64, ctox.Q4B64])
def test_verify_positions_match_per_row_oracle(be, orc, dtype, positions):
    import torch
    rows, columns = 320, 1024
    op = synthetic_op(dtype, rows, columns, seed=31)
    xs = synthetic.activations(columns, 32, positions=positions).reshape(positions, columns)
    mv = be.prepare_fused_matvec(op)
    try:
        got = mv.dispatch_host(xs, positions=positions).reshape(positions, rows)
        # bf16 activations on the device path (the verify step's element type)
        xb = torch.from_numpy(xs).to(torch.bfloat16).cuda()
        y = torch.empty(positions, rows, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        mv.dispatch_device(xb.data_ptr(), ctox.BF16, positions, columns, y.data_ptr(), rows)
        be.synchronize()
        got_bf16 = y.cpu().numpy()
        xs_bf16 = xb.float().cpu().numpy()
    finally:
        mv.destroy()
    for m in range(positions):
        oop = to_oracle_op(orc, op)
        oop.input = xs[m]
        assert rel_l2(got[m], orc.fused_matvec(oop)) <= TIGHT
        oop.input = xs_bf16[m]
        assert rel_l2(got_bf16[m], orc.fused_matvec(oop)) <= TIGHT


def test_large_dynamic_range_activations(be, orc):
    op = synthetic_op(ctox.Q4B64, 64, 2048, seed=41, scales=False)
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(2048) * 10.0 ** rng.integers(-6, 5, 2048)).astype(np.float32)
    op.input = x
    assert rel_l2(be.fused_matvec(op), orc.fused_matvec(to_oracle_op(orc, op))) <= TIGHT


def test_error_kinds_match_the_cpu_backend(be, orc):
    w = synthetic.packed_weights(ctox.Q4B64, 2, 64, 1)
    x = np.ones(64, np.float32)
    cases = [
        (ctox.FusedMatVec(ctox.Q4B64, w, 2, 60, np.ones(60, np.float32)), "Shape"),
        (ctox.FusedMatVec(ctox.Q4B64, w, 0, 64, x), "Shape"),
        (ctox.FusedMatVec(ctox.Q4B64, w, 3, 64, x), "Shape"),
        (ctox.FusedMatVec(ctox.Q4B64, w, 2, 64, np.ones(63, np.float32)), "Shape"),
        (ctox.FusedMatVec(ctox.Q4B64, w, 2, 64, x, s_out=np.ones(3, np.float32)), "Shape"),
        (ctox.FusedMatVec(ctox.F16, w, 2, 64, x), "UnsupportedDType"),
        (ctox.FusedMatVec(ctox.Q4B64, w, 2, 64, x, segments=[ctox.Segment(0, 1, 0, 2, 0, w.size)]),
         "InvalidArtifact"),
        (ctox.FusedMatVec(ctox.MIXED_Q2Q4B64, w, 2, 64, x), "InvalidArtifact"),
        (ctox.FusedMatVec(ctox.MIXED_Q2Q4B64, w, 2, 64, x,
                          segments=[ctox.Segment(0, ctox.Q4B64, 1, 2, 0, w.size)]), "InvalidArtifact"),
        (ctox.FusedMatVec(ctox.Q4B64, w, 2, 64, x, s_in=np.full(64, np.nan, np.float32)),
         "InvalidArtifact"),
    ]
    bad = w.copy()
    bad[34:36] = np.array([np.inf], dtype=np.float16).view(np.uint8)
    cases.append((ctox.FusedMatVec(ctox.Q4B64, bad, 2, 64, x), "InvalidArtifact"))
    for op, kind in cases:
        with pytest.raises(ctox.CtoxError) as e:
            be.fused_matvec(op)
        assert e.value.kind == kind, (kind, str(e.value))
        with pytest.raises(orc.OracleError) as oe:
            orc.fused_matvec(to_oracle_op(orc, op))
        assert oe.value.kind == kind
    # a non-finite activation gives a non-finite output: InvalidState
    # (backend/cuda_runtime.rs:10626-10630)
    xi = x.copy()
    xi[5] = np.inf
    with pytest.raises(ctox.CtoxError) as e:
        be.fused_matvec(ctox.FusedMatVec(ctox.Q4B64, w, 2, 64, xi))
    assert e.value.kind == "InvalidState"


def test_recovered_row_and_row_matvec(be, orc):
    for dtype in (ctox.Q2B64, ctox.Q4B64):
        columns = 5120
        w = synthetic.packed_weights(dtype, 1, columns, 51)
        s_in = synthetic.recovery_scales_f16(columns, 52, 3)
        row = be.recovered_row(ctox.RecoveredRow(dtype, w, columns, s_in, 1.125))
        expect = orc.recovered_row(dtype, w, columns, s_in, 1.125)
        assert np.allclose(row, expect, rtol=3e-7, atol=0)
        x = synthetic.activations(columns, 53)
        dot = be.recovered_row_matvec(ctox.RecoveredRowMatVec(dtype, w, x, 0.875))
        ref = orc.recovered_row_matvec(dtype, w, x, 0.875)
        assert abs(dot - ref) <= 1e-5 * max(1.0, abs(ref))
    with pytest.raises(ctox.CtoxError) as e:
        be.recovered_row(ctox.RecoveredRow(ctox.Q4B64, w, 5120, s_in, float("nan")))
    assert e.value.kind == "Shape"
    with pytest.raises(ctox.CtoxError) as e:
        be.recovered_row_matvec(ctox.RecoveredRowMatVec(ctox.F32, w, x, 1.0))
    assert e.value.kind == "UnsupportedDType"


def test_device_fanout_matches_independent_dispatches(orc):
    """Backend::fused_matvec_fanout on prepared matrices (cpu.rs:444-472, fanout.rs:31-70): one set of
    activation fragments, every member bit-identical to its own dispatch; members with a different
    s_in are refused."""
    import torch
    be = ctox.B200Backend(0)
    rng = np.random.default_rng(21)
    cols, positions = 1024, 3
    s_in = synthetic.recovery_scales_f16(cols, 5, 1)
    mats = []
    for rows, seed in ((512, 1), (96, 2), (2048, 3)):
        mats.append(be.prepare_fused_matvec(ctox.FusedMatVec(
            ctox.Q4B64, synthetic.packed_weights(ctox.Q4B64, rows, cols, seed), rows, cols, None, s_in=s_in,
            s_out=synthetic.recovery_scales_f16(rows, seed, 2))))
    x = torch.from_numpy(rng.standard_normal((positions, cols)).astype(np.float32)).cuda()
    ys = [torch.zeros(positions, m.rows, device="cuda") for m in mats]
    be.fanout_dispatch_device(mats, x.data_ptr(), ctox.F32, positions, cols, [y.data_ptr() for y in ys],
                              [m.rows for m in mats])
    be.synchronize()
    for m, y in zip(mats, ys):
        single = torch.zeros(positions, m.rows, device="cuda")
        m.dispatch_device(x.data_ptr(), ctox.F32, positions, cols, single.data_ptr(), m.rows)
        be.synchronize()
        assert torch.equal(y, single)
    other = be.prepare_fused_matvec(ctox.FusedMatVec(
        ctox.Q4B64, synthetic.packed_weights(ctox.Q4B64, 64, cols, 9), 64, cols, None,
        s_in=synthetic.recovery_scales_f16(cols, 6, 1)))
    with pytest.raises(ctox.CtoxError) as e:
        be.fanout_dispatch_device([mats[0], other], x.data_ptr(), ctox.F32, 1, cols,
                                  [ys[0].data_ptr(), ys[1].data_ptr()], [mats[0].rows, 64])
    assert e.value.kind == "Shape"
    for m in mats + [other]:
        m.destroy()
    assert be.allocated_bytes() == 0
    be.close()


def test_device_recovered_rows_match_the_oracle(orc):
    import torch
    be = ctox.B200Backend(0)
    rows, cols = 300, 512
    w = synthetic.packed_weights(ctox.Q2B64, rows, cols, 4)
    s_in, s_out = synthetic.recovery_scales_f16(cols, 4, 1), synthetic.recovery_scales_f16(rows, 4, 2)
    mv = be.prepare_fused_matvec(ctox.FusedMatVec(ctox.Q2B64, w, rows, cols, None, s_in=s_in, s_out=s_out),
                                 keep_canonical=True)
    ids = np.array([0, 299, 17, 17, 128], dtype=np.uint32)
    out = torch.zeros(ids.size, cols, device="cuda")
    mv.recovered_rows_device(torch.from_numpy(ids.view(np.int32)).cuda().data_ptr(), ids.size, out.data_ptr())
    be.synchronize()
    rb = cols // 64 * 18
    so = np.frombuffer(s_out.tobytes(), dtype=np.float16).astype(np.float32)
    for i, r in enumerate(ids):
        exp = orc.recovered_row(orc.Q2B64, w[r * rb:(r + 1) * rb], cols, s_in, float(so[r]))
        assert np.array_equal(out[i].cpu().numpy(), exp), (i, r)
    mv.destroy()
    be.close()
