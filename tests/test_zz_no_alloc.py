"""The allocation-free dispatch (ctox_matvec_dispatch_static) against the ordinary one.

Some users of the library cannot allocate device memory around a dispatch (a serving loop whose
cache owns every free byte, a plug-in living in another framework's pool, code that cannot afford
an allocation's implicit synchronisation). Their entry point keeps the kernel's scratch in a fixed
array inside the library. It runs the same kernels as ctox_matvec_dispatch, so the outputs must
be identical; the check is repeated on a second call because the array keeps the first call's
contents. This file sorts last so that a stop-at-first-failure run has seen every other test.
"""
import numpy as np
import pytest
import torch

import ctox_llm_b200 as ctox
from ctox_llm_b200 import synthetic

pytestmark = pytest.mark.gpu


def test_static_scratch_dispatch_matches_ordinary_dispatch_twice():
    be = ctox.B200Backend(0)
    try:
        for dtype, rows, columns, positions in ((ctox.Q4B64, 1024, 5120, 1), (ctox.Q2B64, 5120, 1024, 5),
                                                (ctox.Q4B64, 257, 512, 3)):
            op = ctox.FusedMatVec(dtype, synthetic.packed_weights(dtype, rows, columns, 91), rows, columns,
                                  None, s_in=synthetic.recovery_scales_f16(columns, 91, 3),
                                  s_out=synthetic.recovery_scales_f16(rows, 91, 4),
                                  activation=ctox.ACT_SILU)
            mv = be.prepare_fused_matvec(op)
            try:
                before = be.allocated_bytes()
                for call in range(2):  # two calls in a row share the built-in array
                    x = torch.from_numpy(synthetic.activations(columns, 92 + call, positions=positions)
                                         .reshape(positions, columns)).cuda()
                    want = torch.empty(positions, rows, device="cuda")
                    got = torch.full((positions, rows), float("nan"), device="cuda")
                    torch.cuda.synchronize()
                    mv.dispatch_device(x.data_ptr(), ctox.F32, positions, columns, want.data_ptr(), rows)
                    mv.dispatch_static(x.data_ptr(), ctox.F32, positions, columns, got.data_ptr(), rows)
                    be.synchronize()
                    # same kernels, same order of additions: tolerance 0 (the suite's matvec bound is 5e-5)
                    assert torch.equal(got, want), (dtype, rows, columns, positions, call)
                assert be.allocated_bytes() == before, "the static dispatch must not allocate"
            finally:
                mv.destroy()
        # The places where the built-in array is shared more than once per call: every part of a
        # mixed Q2/Q4 matrix uses the same fragment and partial-sum regions; 16 positions run as
        # two passes through them; bf16 activations take the other input path; and two different
        # handles called back to back leave each other's contents behind.
        columns = 512
        q2 = synthetic.packed_weights(ctox.Q2B64, 96, columns, 94)
        q4 = synthetic.packed_weights(ctox.Q4B64, 160, columns, 95)
        segs = [ctox.Segment(0, ctox.Q2B64, 0, 96, 0, q2.size),
                ctox.Segment(1, ctox.Q4B64, 96, 256, q2.size, q4.size)]
        mixed = be.prepare_fused_matvec(ctox.FusedMatVec(
            ctox.MIXED_Q2Q4B64, np.concatenate([q2, q4]), 256, columns, None, segments=segs,
            s_in=synthetic.recovery_scales_f16(columns, 94, 3), s_out=synthetic.recovery_scales_f16(256, 94, 4)))
        pure = be.prepare_fused_matvec(ctox.FusedMatVec(
            ctox.Q4B64, synthetic.packed_weights(ctox.Q4B64, 320, columns, 96), 320, columns, None))
        try:
            before = be.allocated_bytes()
            for call, (positions, bf16) in enumerate(((16, False), (3, True), (16, True), (9, False))):
                x = torch.from_numpy(synthetic.activations(columns, 97 + call, positions=positions)
                                     .reshape(positions, columns)).cuda()
                xd, dt = (x.to(torch.bfloat16), ctox.BF16) if bf16 else (x, ctox.F32)
                for mv, rows in ((mixed, 256), (pure, 320), (mixed, 256)):  # handles interleaved
                    want = torch.empty(positions, rows, device="cuda")
                    got = torch.full((positions, rows), float("nan"), device="cuda")
                    torch.cuda.synchronize()
                    mv.dispatch_device(xd.data_ptr(), dt, positions, columns, want.data_ptr(), rows)
                    mv.dispatch_static(xd.data_ptr(), dt, positions, columns, got.data_ptr(), rows)
                    be.synchronize()
                    assert torch.equal(got, want), (positions, bf16, rows)
            assert be.allocated_bytes() == before, "the static dispatch must not allocate"
        finally:
            mixed.destroy()
            pure.destroy()
        # an operation whose scratch exceeds the built-in array is refused with a clear error
        rows, columns = 262144, 512
        big = be.prepare_fused_matvec(ctox.FusedMatVec(
            ctox.Q2B64, synthetic.packed_weights(ctox.Q2B64, rows, columns, 93), rows, columns, None))
        try:
            x = torch.zeros(columns, device="cuda")
            y = torch.zeros(rows, device="cuda")
            with pytest.raises(ctox.CtoxError) as e:
                big.dispatch_static(x.data_ptr(), ctox.F32, 1, columns, y.data_ptr(), rows)
            assert e.value.kind == "MemoryBudget" and "built-in array" in str(e.value)
        finally:
            big.destroy()
        assert be.device_error() == 0
    finally:
        be.close()
