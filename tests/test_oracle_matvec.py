"""Restates the CPU-backend tests of the reference (backend/cpu.rs:732-1126) on the oracle."""
import numpy as np
import pytest

f32 = np.float32


def encode_fixture(orc, dtype, rows, columns):
    # backend/cpu.rs:751-769
    phase = np.arange(rows * columns, dtype=np.float32)
    values = (np.sin((phase * f32(0.013579)).astype(np.float32)) * f32(0.75)).astype(np.float32)
    return orc.quantize_matrix(dtype, values.reshape(rows, columns))


def fused_case(orc, dtype, rows, columns, activation):
    # backend/cpu.rs:774-812
    weights = encode_fixture(orc, dtype, rows, columns)
    idx = np.arange(columns)
    x = np.cos((idx.astype(np.float32) * f32(0.03125))).astype(np.float32)
    s_in = (f32(0.75) + f32(0.005) * (idx % 7).astype(np.float32)).astype(np.float32)
    r = np.arange(rows)
    s_out = (f32(1.25) - f32(0.05) * (r % 5).astype(np.float32)).astype(np.float32)
    bias = (np.sin(r.astype(np.float32) * f32(1.7)) * f32(0.1)).astype(np.float32)
    return orc.FusedMatVec(dtype=dtype, weights=weights, rows=rows, columns=columns, input=x,
                           s_in=s_in, s_out=s_out, bias=bias, activation=activation)


@pytest.mark.parametrize("dtype_name,rows,blocks,act", [
    ("Q2B64", 7, 3, 1), ("Q4B64", 7, 3, 1), ("Q2B64", 3, 1, 0), ("Q4B64", 3, 1, 0)])
def test_simd_arm_matches_scalar(orc, dtype_name, rows, blocks, act):
    op = fused_case(orc, getattr(orc, dtype_name), rows, blocks * 64, act)
    scalar = orc.fused_matvec(op)
    simd = orc.fused_matvec(op, avx2=True)
    assert np.all(np.abs(scalar - simd) <= 2e-4)
    # independent float64 evaluation of the same formula
    deq = orc.dequantize_blocks(op.dtype, op.weights).reshape(rows, -1).astype(np.float64)
    y = (deq @ (op.input.astype(np.float64) * op.s_in) + op.bias) * op.s_out
    if act:
        y = y / (1.0 + np.exp(-y))
    assert np.all(np.abs(scalar - y) <= 1e-5)


def test_f16_scales_match_f32_scales(orc):
    # backend/cpu.rs:834-875
    weights = encode_fixture(orc, orc.Q2B64, 2, 64)
    idx = np.arange(64)
    x = np.sin(idx.astype(np.float32) * f32(0.0625)).astype(np.float32)
    s_in16 = (f32(0.75) + (idx % 9).astype(np.float32) * f32(0.03125)).astype(np.float16)
    s_out16 = np.array([1.25, 0.875], dtype=np.float16)
    a = orc.FusedMatVec(orc.Q2B64, weights, 2, 64, x, s_in=s_in16.astype(np.float32),
                        s_out=s_out16.astype(np.float32))
    b = orc.FusedMatVec(orc.Q2B64, weights, 2, 64, x, s_in=s_in16.view(np.uint8),
                        s_out=s_out16.view(np.uint8))
    assert np.array_equal(orc.fused_matvec(a), orc.fused_matvec(b))


def test_mixed_rows_match_pure_kernels(orc):
    # backend/cpu.rs:877-952
    columns = 128
    q2 = encode_fixture(orc, orc.Q2B64, 2, columns)
    q4 = encode_fixture(orc, orc.Q4B64, 2, columns)
    weights = np.concatenate([q2, q4])
    segs = [orc.Segment(0, orc.Q2B64, 0, 2, 0, q2.size), orc.Segment(1, orc.Q4B64, 2, 4, q2.size, q4.size)]
    x = np.cos(np.arange(columns, dtype=np.float32) * f32(0.0234375)).astype(np.float32)
    mixed = orc.fused_matvec(orc.FusedMatVec(orc.MIXED_Q2Q4B64, weights, 4, columns, x, segments=segs))
    assert np.array_equal(mixed[:2], orc.fused_matvec(orc.FusedMatVec(orc.Q2B64, q2, 2, columns, x)))
    assert np.array_equal(mixed[2:], orc.fused_matvec(orc.FusedMatVec(orc.Q4B64, q4, 2, columns, x)))
    # backend/cpu.rs:1012-1042: non-contiguous manifest segments are rejected
    bad = [orc.Segment(0, orc.Q2B64, 1, 2, 0, q2.size)]
    with pytest.raises(orc.OracleError) as e:
        orc.fused_matvec(orc.FusedMatVec(orc.MIXED_Q2Q4B64, q2, 2, columns, x, segments=bad))
    assert e.value.kind == "InvalidArtifact"


def test_fanout_matches_independent(orc):
    # backend/cpu.rs:954-1010
    x = np.sin(np.arange(64, dtype=np.float32) * f32(0.0625)).astype(np.float32)
    q2 = encode_fixture(orc, orc.Q2B64, 2, 64)
    q4 = encode_fixture(orc, orc.Q4B64, 3, 64)
    shared = np.full(64, 1.125, dtype=np.float32)
    other = np.full(64, 0.875, dtype=np.float32)
    a = orc.FusedMatVec(orc.Q2B64, q2, 2, 64, x, s_in=shared)
    b = orc.FusedMatVec(orc.Q4B64, q4, 3, 64, x, s_in=shared)
    outs = orc.fused_matvec_fanout([a, b])
    assert np.array_equal(outs[0], orc.fused_matvec(a)) and np.array_equal(outs[1], orc.fused_matvec(b))
    c = orc.FusedMatVec(orc.Q4B64, q4, 3, 64, x, s_in=other)
    outs = orc.fused_matvec_fanout([a, c])
    assert np.array_equal(outs[1], orc.fused_matvec(c))
    with pytest.raises(orc.OracleError):
        orc.fused_matvec_fanout([])


def test_arbitrary_code_bytes(orc):
    # backend/cpu.rs:1046-1088
    i = np.arange(64, dtype=np.float32)
    codes2 = ((np.arange(16) * 0x45 + 0x1B) & 0xFF).astype(np.uint8)
    blk = np.concatenate([np.array([0.625], dtype=np.float16).view(np.uint8), codes2])
    x = (np.sin(i * f32(0.11)) + f32(0.25)).astype(np.float32)
    ref = float((orc.dequantize_blocks(orc.Q2B64, blk)[0] * x).sum(dtype=np.float32))
    got = orc.fused_matvec(orc.FusedMatVec(orc.Q2B64, blk, 1, 64, x))[0]
    assert abs(ref - got) <= 1e-5
    codes4 = ((np.arange(32) * 0x9E + 0x3D) & 0xFF).astype(np.uint8)
    blk = np.concatenate([np.array([0.375], dtype=np.float16).view(np.uint8), codes4])
    x = (np.cos(i * f32(0.07)) - f32(0.125)).astype(np.float32)
    ref = float((orc.dequantize_blocks(orc.Q4B64, blk)[0] * x).sum(dtype=np.float32))
    got = orc.fused_matvec(orc.FusedMatVec(orc.Q4B64, blk, 1, 64, x))[0]
    assert abs(ref - got) <= 1e-5


def test_bias_before_s_out(orc):
    # backend/cpu.rs:1090-1115 (rows=1, s_out=2, bias=1, input all ones)
    src = ((np.arange(64, dtype=np.float32) - f32(31.5)) / f32(31.5)).reshape(1, 64)
    for dtype in (orc.Q2B64, orc.Q4B64):
        w = orc.quantize_matrix(dtype, src)
        y = orc.fused_matvec(orc.FusedMatVec(dtype, w, 1, 64, np.ones(64, np.float32),
                                             s_out=np.array([2.0], np.float32),
                                             bias=np.array([1.0], np.float32)))[0]
        plain = orc.fused_matvec(orc.FusedMatVec(dtype, w, 1, 64, np.ones(64, np.float32)))[0]
        assert y == np.float32((plain + np.float32(1.0)) * np.float32(2.0))


def test_validation_errors(orc):
    w = encode_fixture(orc, orc.Q4B64, 2, 64)
    x = np.ones(64, np.float32)
    for kwargs, kind in [
        (dict(rows=2, columns=60), "Shape"), (dict(rows=0, columns=64), "Shape"),
        (dict(rows=3, columns=64), "Shape")]:
        with pytest.raises(orc.OracleError) as e:
            orc.fused_matvec(orc.FusedMatVec(orc.Q4B64, w, kwargs["rows"], kwargs["columns"],
                                             np.ones(kwargs["columns"], np.float32)))
        assert e.value.kind == kind
    with pytest.raises(orc.OracleError) as e:
        orc.fused_matvec(orc.FusedMatVec(orc.F16, w, 2, 64, x))
    assert e.value.kind == "UnsupportedDType"
    bad = w.copy()
    bad[0:2] = np.array([np.inf], dtype=np.float16).view(np.uint8)
    with pytest.raises(orc.OracleError) as e:
        orc.fused_matvec(orc.FusedMatVec(orc.Q4B64, bad, 2, 64, x))
    assert e.value.kind == "InvalidArtifact"
    # recovered row (backend/cpu.rs:312-370) equals dequant * s_in * s_out
    s_in = np.linspace(0.5, 1.5, 64).astype(np.float32)
    row = orc.recovered_row(orc.Q4B64, w[:34], 64, s_in, 1.5)
    deq = orc.dequantize_blocks(orc.Q4B64, w[:34])[0]
    assert np.allclose(row, deq * s_in * np.float32(1.5), rtol=1e-6, atol=0)
    dot = orc.recovered_row_matvec(orc.Q4B64, w[:34], x * s_in, 2.0)
    assert abs(dot - 2.0 * float((deq * s_in).sum())) < 1e-5
