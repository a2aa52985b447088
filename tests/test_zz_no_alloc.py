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
