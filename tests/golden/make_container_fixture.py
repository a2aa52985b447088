"""Writes tests/golden/container_fixture.ctoxq with this repository's writer and checks it with the
reference's own reader, unmodified (training/ctox_artifact.py::CtoxArtifact with checksums on, and
its `_decode_blocks` against the oracle's block decode). Stores what the reference reader returned.

    python tests/golden/make_container_fixture.py /path/to/reference
"""
import json
import os
import sys
from pathlib import Path

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def main(reference_root):
    sys.path.insert(0, f"{reference_root}/training")
    import ctox_artifact  # the reference's reader
    import oracle
    from ctox_llm_b200 import artifact as A

    oracle.build()
    rng = np.random.default_rng(20260826)
    q2 = oracle.quantize_matrix(oracle.Q2B64, rng.standard_normal((8, 128)).astype(np.float32))
    q4 = oracle.quantize_matrix(oracle.Q4B64, rng.standard_normal((16, 128)).astype(np.float32))
    segs = [{"group_index": 0, "row_start": 0, "row_end": 8, "dtype": "q2_b64", "offset": 0, "length": int(q2.size)},
            {"group_index": 1, "row_start": 8, "row_end": 24, "dtype": "q4_b64", "offset": int(q2.size),
             "length": int(q4.size)}]
    tensors = [
        A.PackedTensor("w.q2", "q2_b64", [8, 128], q2.tobytes()),
        A.PackedTensor("w.q4", "q4_b64", [16, 128], q4.tobytes()),
        A.PackedTensor("w.mixed", "mixed_q2_q4_b64", [24, 128], np.concatenate([q2, q4]).tobytes(), segs),
        A.PackedTensor("w.mixed.s_in", "f16", [128], rng.uniform(0.75, 1.25, 128).astype("<f2").tobytes()),
        A.PackedTensor("w.mixed.s_out", "f16", [24], rng.uniform(0.75, 1.25, 24).astype("<f2").tobytes()),
        A.PackedTensor("norm.weight", "f32", [5], rng.standard_normal(5).astype("<f4").tobytes()),
    ]
    path = os.path.join(HERE, "container_fixture.ctoxq")
    if os.path.exists(path):
        os.remove(path)
    A.write_ctoxq(path, tensors, model="fixture/ctoxq", revision="0123456789abcdef")
    ref = ctox_artifact.CtoxArtifact(Path(path), verify_tensors=True)  # raises on any contract violation
    out = {"tensors": {}}
    for name, t in ref.tensors.items():
        payload = bytes(ref.tensor_bytes(name))
        out["tensors"][name] = {"sha256": t["sha256"], "byte_sum": int(np.frombuffer(payload, np.uint8).sum())}
    # the reference's block decoder agrees with the oracle's on the fixture's matrices
    for name, dtype, code in (("w.q2", "q2_b64", oracle.Q2B64), ("w.q4", "q4_b64", oracle.Q4B64)):
        import torch
        got = ctox_artifact.CtoxArtifact._decode_blocks(torch, ref.tensor_bytes(name), dtype, "cpu").reshape(-1).numpy()
        want = oracle.dequantize_blocks(code, np.frombuffer(bytes(ref.tensor_bytes(name)), np.uint8)).reshape(-1)
        assert np.allclose(got, want, rtol=1e-6, atol=1e-6), name  # (code - 7.5) / 7.5 vs code / 7.5 - 1: last-bit differences
    ref.close()
    json.dump(out, open(os.path.join(HERE, "container_fixture.json"), "w"), indent=1, sort_keys=True)
    print("wrote", path)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_container_fixture.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
