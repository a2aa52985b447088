"""K/V rows as Q4_B64 / Q2_B64 blocks on the device against the oracle's restatement of quant.rs:
byte-exact for quantize (kv_cache.rs:22-45), requantize Q4 -> Q2 (:67-73) and dequantize (:55-65),
including all-zero blocks, a lone maximum, values on rounding ties and denormal scales."""
import numpy as np
import pytest
import torch

import ctox_llm_b200 as ctox

pytestmark = pytest.mark.gpu
Q2, Q4 = ctox.native.Q2B64, ctox.native.Q4B64


@pytest.fixture(scope="module")
def be():
    b = ctox.B200Backend(0)
    yield b
    b.close()


def blocks_under_test(seed, n):
    rng = np.random.default_rng(seed)
    v = rng.standard_normal((n, 64)).astype(np.float32)
    v[0] = 0.0                                   # scale 0: all codes 0 (quant.rs:150-155)
    v[1] = 0.0
    v[1, 17] = -3.5                              # a lone maximum
    v[2] = np.linspace(-1.0, 1.0, 64, dtype=np.float32)          # the 16 levels and points between
    v[3] = (np.arange(64, dtype=np.float32) - 31.5) / 31.5        # symmetric ramp
    v[4] = np.float32(1e-7) * rng.standard_normal(64).astype(np.float32)  # binary16-subnormal scale
    v[5] = np.float32(1e4) * rng.standard_normal(64).astype(np.float32)  # large scale (finite as binary16)
    # exact ties of the Q4 rounding: (n * 7.5 + 7.5) = k + 0.5 for n = (k - 7) / 7.5
    v[6] = np.array([(k % 15 - 7) / 7.5 for k in range(64)], dtype=np.float32)
    v[6, 0] = 1.0
    v[7] = rng.standard_normal(64).astype(np.float32) * np.float32(1e-3)
    return v


def test_pack_demote_unpack_equal_the_oracle_bytes(be, orc):
    n = 4096 + 8
    v = blocks_under_test(5, n)
    dv = torch.from_numpy(v).cuda()
    q4 = torch.zeros(n * 34, dtype=torch.uint8, device="cuda")
    q2 = torch.zeros(n * 18, dtype=torch.uint8, device="cuda")
    back4 = torch.empty(n * 64, dtype=torch.float32, device="cuda")
    back2 = torch.empty(n * 64, dtype=torch.float32, device="cuda")
    be.kv_pack_q4(dv.data_ptr(), n, q4.data_ptr())
    be.kv_demote_q4_to_q2(q4.data_ptr(), n, q2.data_ptr())
    be.kv_unpack(Q4, q4.data_ptr(), n, back4.data_ptr())
    be.kv_unpack(Q2, q2.data_ptr(), n, back2.data_ptr())
    be.synchronize()
    assert be.device_error() == 0
    want4 = orc.quantize_matrix(Q4, v)                        # [n][34]
    assert np.array_equal(q4.cpu().numpy().reshape(n, 34), want4.reshape(n, 34))
    deq4 = orc.dequantize_blocks(Q4, want4).reshape(n, 64)
    assert np.array_equal(back4.cpu().numpy().reshape(n, 64), deq4)
    want2 = orc.quantize_matrix(Q2, deq4)                     # requantize = quantize(dequantize(..))
    assert np.array_equal(q2.cpu().numpy().reshape(n, 18), want2.reshape(n, 18))
    assert np.array_equal(back2.cpu().numpy().reshape(n, 64), orc.dequantize_blocks(Q2, want2).reshape(n, 64))


def test_bad_arguments_and_non_finite_values(be):
    x = torch.zeros(64, device="cuda")
    out = torch.zeros(34, dtype=torch.uint8, device="cuda")
    with pytest.raises(ctox.CtoxError) as e:
        be.kv_pack_q4(x.data_ptr(), 0, out.data_ptr())
    assert e.value.kind == "Shape"
    with pytest.raises(ctox.CtoxError) as e:
        be.kv_unpack(ctox.native.F32, out.data_ptr(), 1, x.data_ptr())
    assert e.value.kind == "UnsupportedDType"
    x[3] = float("inf")  # quant.rs:37-41 refuses non-finite input: here the device error word is set
    be.kv_pack_q4(x.data_ptr(), 1, out.data_ptr())
    be.synchronize()
    assert be.device_error() != 0 and be.device_error() == 0
