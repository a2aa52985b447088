"""CTOXQ container (models/qwen38_27b/src/format.rs, loader.rs, fanout.rs): the reference's own
format tests restated against the host-side reader / writer, the frozen fan-out digest, and a
container written here that the reference's Python reader (training/ctox_artifact.py) accepted when
the fixture was made (tests/golden/make_container_fixture.py holds the script and what it checked).
"""
import json
import os
import struct

import numpy as np
import pytest

import ctox_llm_b200 as ctox
from ctox_llm_b200 import artifact as A
from oracle_model import OracleModel, tiny_config

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_header_round_trip_and_refusals(tmp_path):  # format.rs:579-589, 403-437
    raw = A.HEADER.pack(A.MAGIC, 1, A.ENDIAN_MARKER, 123, 512, 7, 256)
    assert len(raw) == 64 and A.HEADER.unpack(raw) == (A.MAGIC, 1, A.ENDIAN_MARKER, 123, 512, 7, 256)
    cases = {"short": raw[:40], "magic": b"CTOXQ3Q4" + raw[8:], "version": raw[:8] + struct.pack("<I", 3) + raw[12:],
             "endian": raw[:12] + struct.pack("<I", 0x04030201) + raw[16:]}
    for name, blob in cases.items():
        p = tmp_path / f"{name}.ctoxq"
        p.write_bytes(blob)
        with pytest.raises(ctox.CtoxError) as e:
            A.CtoxqArtifact.open(str(p))
        assert e.value.kind == "InvalidArtifact", name


def test_q3_is_not_a_manifest_dtype():  # format.rs:591-600
    with pytest.raises(ctox.CtoxError):
        A.expected_bytes("q3_b64", [64], [])


def mixed_segments():  # format.rs:602-638: 3 rows of 128 columns: row 0 in Q2, rows 1-2 in Q4
    return [{"group_index": 0, "row_start": 0, "row_end": 1, "dtype": "q2_b64", "offset": 0, "length": 36},
            {"group_index": 1, "row_start": 1, "row_end": 3, "dtype": "q4_b64", "offset": 36, "length": 136}]


def test_mixed_q2_q4_segments_validate_exact_coverage():  # format.rs:640-651
    segs = mixed_segments()
    assert A.expected_bytes("mixed_q2_q4_b64", [3, 128], segs) == 172
    gap = [dict(s) for s in segs]
    gap[1]["row_start"] = 2
    with pytest.raises(ctox.CtoxError):
        A.expected_bytes("mixed_q2_q4_b64", [3, 128], gap)
    short = [dict(s) for s in segs]
    short[1]["row_end"] = 2
    short[1]["length"] = 68
    with pytest.raises(ctox.CtoxError):
        A.expected_bytes("mixed_q2_q4_b64", [3, 128], short)
    manifest = {"format": "ctox.q2q4.v1", "model": "m", "revision": "0123456", "alignment": 256, "target": "t",
                "tensors": [{"name": "w", "dtype": "mixed_q2_q4_b64", "shape": [3, 128], "offset": 0, "length": 172,
                             "sha256": "0" * 64, "segments": segs}]}
    with pytest.raises(ctox.CtoxError):  # mixed tensors need manifest v2
        A.validate_manifest(manifest, 172)
    manifest["format"] = "ctox.q2q4.v2"
    A.validate_manifest(manifest, 172)
    manifest["alignment"] = 48
    with pytest.raises(ctox.CtoxError):
        A.validate_manifest(manifest, 172)


def test_artifact_builder_round_trips_and_checksums(tmp_path):  # format.rs:730-790
    rng = np.random.default_rng(0)
    q4 = rng.integers(0, 256, 2 * 34, dtype=np.uint8)
    q4[0::34], q4[1::34] = 0x00, 0x3C  # f16 scale 1.0
    tensors = [A.PackedTensor("a.weight", "q4_b64", [2, 64], q4.tobytes()),
               A.PackedTensor("a.weight.s_in", "f16", [64], np.ones(64, "<f2").tobytes()),
               A.PackedTensor("a.weight.s_out", "f16", [2], np.ones(2, "<f2").tobytes()),
               A.PackedTensor("norm", "f32", [3], np.array([0.5, -1.0, 2.0], "<f4").tobytes())]
    path = str(tmp_path / "m.ctoxq")
    manifest = A.write_ctoxq(path, tensors)
    assert [t["offset"] % 256 for t in manifest["tensors"]] == [0, 0, 0, 0]
    art = A.CtoxqArtifact.open(path)
    assert art.file_bytes() == os.path.getsize(path)
    op = art.recovered_matrix("a.weight")
    assert (op.rows, op.columns, op.dtype) == (2, 64, ctox.Q4B64) and np.array_equal(op.weights, q4)
    assert np.array_equal(art.float_tensor("norm"), np.array([0.5, -1.0, 2.0], np.float32))
    with pytest.raises(ctox.CtoxError) as e:
        art.recovery_scales("norm")  # F32 scales are refused (loader.rs:177-187)
    assert e.value.kind == "UnsupportedDType"
    art.close()
    with pytest.raises(FileExistsError):
        A.write_ctoxq(path, tensors)  # write_new never overwrites
    blob = bytearray(open(path, "rb").read())
    blob[-1] ^= 1  # flip one payload bit: the checksum policy must notice
    bad = str(tmp_path / "bad.ctoxq")
    open(bad, "wb").write(bytes(blob))
    with pytest.raises(ctox.CtoxError) as e:
        A.CtoxqArtifact.open(bad)
    assert "checksum" in str(e.value)
    A.CtoxqArtifact.open(bad, verify_checksums=False).close()


def test_frozen_fanout_groups_match_the_reference_digest():  # fanout.rs:78-95
    groups = A.fanout_groups()
    assert len(groups) == 130 and sum(len(g["scale_names"]) for g in groups) == 373
    assert A.fanout_group_sha256(groups) == "5cac430d5da6762c8a3525c658f310daebdff0197bb3ca28b3c5cb067d5d35f0"


def test_container_fixture_checked_by_the_reference_reader():
    """tests/golden/container_fixture.ctoxq was written by write_ctoxq and opened with the reference's
    reader (checksums on) when it was made; the JSON beside it holds what that reader returned."""
    art = A.CtoxqArtifact.open(os.path.join(GOLDEN, "container_fixture.ctoxq"))
    want = json.load(open(os.path.join(GOLDEN, "container_fixture.json")))
    assert sorted(art.tensors) == sorted(want["tensors"])
    for name, info in want["tensors"].items():
        assert art.tensors[name]["sha256"] == info["sha256"]
        assert int(np.sum(art.tensor_bytes(name), dtype=np.uint64)) == info["byte_sum"]
    op = art.recovered_matrix("w.mixed")
    assert op.dtype == ctox.MIXED_Q2Q4B64 and [(s.row_start, s.row_end) for s in op.segments] == [(0, 8), (8, 24)]
    art.close()


def test_model_container_round_trip_names(tmp_path, orc):
    """A whole tiny model written as a container and read back tensor by tensor."""
    cfg = tiny_config()
    model = OracleModel(orc, cfg, seed=3)
    path = str(tmp_path / "tiny.ctoxq")
    A.write_ctoxq(path, model.packed_tensors())
    art = A.CtoxqArtifact.open(path)
    q = art.recovered_matrix("model.language_model.layers.3.self_attn.q_proj.weight")
    assert np.array_equal(q.weights, model.layers[3]["q"].packed) and np.array_equal(q.s_in, model.layers[3]["q"].s_in)
    assert np.array_equal(art.float_tensor("model.language_model.layers.0.linear_attn.A_log"),
                          model.layers[0]["a_log"])
    art.close()
