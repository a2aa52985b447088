"""Generates tests/golden/quant_fixtures.npz by running the reference's own Python code.

Run in a container where the reference checkout is mounted:
    python tests/golden/make_fixtures.py /path/to/reference

It imports, unmodified, the reference's packer `training/pack_checkpoint.py::quantize_blocks`
(which calls `training/quantization.py::quantize_components`), its decoder
`training/ctox_artifact.py::CtoxArtifact._decode_blocks`, and restates the forward of
`training/packed_recovery_ops.py` (`linear(x * s_in, W, bias) * s_out`) with torch float64 on the
reference-decoded weights. The stored arrays are the golden vectors the oracle is pinned to for
the packed block format and the fused matvec semantics.
"""
import sys

import numpy as np


def main(reference_root: str) -> None:
    sys.path.insert(0, f"{reference_root}/training")
    import torch
    import ctox_artifact
    import pack_checkpoint

    gen = torch.Generator().manual_seed(20260826)
    out = {}
    for dtype, tag in (("q2_b64", "q2"), ("q4_b64", "q4")):
        rows, columns = 24, 320
        values = torch.randn(rows, columns, generator=gen) * torch.exp(
            torch.randn(rows, 1, generator=gen) - 3.0)
        values[3, 64:128] = 0.0  # an all-zero block
        packed = pack_checkpoint.quantize_blocks(values, dtype)
        decoded = ctox_artifact.CtoxArtifact._decode_blocks(torch, memoryview(packed), dtype, "cpu")
        decoded = decoded.reshape(rows, columns)
        x = torch.randn(columns, generator=gen)
        s_in = (0.75 + 0.5 * torch.rand(columns, generator=gen)).to(torch.float16)
        s_out = (0.75 + 0.5 * torch.rand(rows, generator=gen)).to(torch.float16)
        bias = torch.randn(rows, generator=gen) * 0.1
        corrected = x.double() * s_in.double()
        base = decoded.double() @ corrected + bias.double()
        y = base * s_out.double()
        out[f"{tag}_values"] = values.numpy()
        out[f"{tag}_packed"] = np.frombuffer(packed, dtype=np.uint8).copy()
        out[f"{tag}_decoded"] = decoded.numpy()
        out[f"{tag}_x"] = x.numpy()
        out[f"{tag}_s_in_f16"] = s_in.view(torch.uint8).numpy().copy()
        out[f"{tag}_s_out_f16"] = s_out.view(torch.uint8).numpy().copy()
        out[f"{tag}_bias"] = bias.numpy()
        out[f"{tag}_y"] = y.float().numpy()
        out[f"{tag}_y_silu"] = torch.nn.functional.silu(y).float().numpy()
    np.savez_compressed(f"{__file__.rsplit('/', 1)[0]}/quant_fixtures.npz", **out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_fixtures.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
