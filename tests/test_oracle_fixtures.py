"""Oracle vs. golden vectors produced by the reference's own Python packer and decoder
(tests/golden/make_fixtures.py)."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden", "quant_fixtures.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


@pytest.mark.parametrize("tag", ["q2", "q4"])
def test_quantize_bytes_match_reference_packer(orc, gold, tag):
    dtype = orc.Q2B64 if tag == "q2" else orc.Q4B64
    packed = orc.quantize_matrix(dtype, gold[f"{tag}_values"])
    assert np.array_equal(packed, gold[f"{tag}_packed"])


@pytest.mark.parametrize("tag", ["q2", "q4"])
def test_decode_matches_reference_decoder(orc, gold, tag):
    dtype = orc.Q2B64 if tag == "q2" else orc.Q4B64
    deq = orc.dequantize_blocks(dtype, gold[f"{tag}_packed"]).reshape(gold[f"{tag}_decoded"].shape)
    ref = gold[f"{tag}_decoded"]
    # the Python decoder evaluates code/7.5 - 1, the Rust one (code - 7.5)/7.5: one ulp apart
    assert np.all(np.abs(deq - ref) <= 1.2e-7 * np.abs(ref).max(axis=1, keepdims=True) + 1e-12)


@pytest.mark.parametrize("tag", ["q2", "q4"])
@pytest.mark.parametrize("act", ["identity", "silu"])
def test_fused_matvec_matches_reference_formula(orc, gold, tag, act):
    dtype = orc.Q2B64 if tag == "q2" else orc.Q4B64
    rows, columns = gold[f"{tag}_values"].shape
    op = orc.FusedMatVec(dtype=dtype, weights=gold[f"{tag}_packed"], rows=rows, columns=columns,
                         input=gold[f"{tag}_x"], s_in=gold[f"{tag}_s_in_f16"],
                         s_out=gold[f"{tag}_s_out_f16"], bias=gold[f"{tag}_bias"],
                         activation=orc.ACT_SILU if act == "silu" else orc.ACT_IDENTITY)
    y = orc.fused_matvec(op)
    ref = gold[f"{tag}_y_silu" if act == "silu" else f"{tag}_y"]
    rel = np.linalg.norm(y - ref) / np.linalg.norm(ref)
    assert rel < 2e-6, rel
    assert np.array_equal(y, orc.fused_matvec(op, threads=3))
    simd = orc.fused_matvec(op, threads=2, avx2=True)
    assert np.all(np.abs(simd - y) <= 2e-4)  # backend/cpu.rs:745 SIMD_TOLERANCE
