"""Helpers shared by the GPU parity tests."""
import numpy as np


def rel_l2(a, b) -> float:
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def to_oracle_op(orc, op):
    """ctox_llm_b200.FusedMatVec -> oracle.FusedMatVec (same fields)."""
    segs = [orc.Segment(s.group_index, s.dtype, s.row_start, s.row_end, s.offset, s.length)
            for s in op.segments]
    return orc.FusedMatVec(dtype=op.dtype, weights=op.weights, rows=op.rows, columns=op.columns,
                           input=op.input, segments=segs, s_in=op.s_in, s_out=op.s_out,
                           bias=op.bias, activation=op.activation)
