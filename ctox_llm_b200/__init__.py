"""B200 (sm_100a) backend for the decode hot path of CTOX-LLM's Qwen3.8-27B integration.

The product is the C-ABI library ``libctox_b200.so`` (see ``include/ctox_b200.h``); this package
is the host-side mirror of the reference crate's ``Backend`` operator interface
(models/qwen38_27b/src/backend/mod.rs:153-169) over that ABI. Importing it never touches
``oracle/`` and there is no CPU fallback: operations raise if no CUDA device is usable.
"""
from ._native import (ACT_IDENTITY, ACT_SILU, BF16, F16, F32, KERNEL_AUTO, KERNEL_ROWWARP,
                      KERNEL_STREAM, MIXED_Q2Q4B64, PREPARE_KEEP_CANONICAL, Q2B64, Q4B64, CtoxError,
                      Segment, load)
from .backend import B200Backend, FusedMatVec, PreparedMatVec, RecoveredRow, RecoveredRowMatVec
from .executor import B200Executor, CancellationToken, GeneratedBlock, qwen38_27b_config
from . import _native as native

__all__ = [
    "B200Backend", "B200Executor", "CancellationToken", "GeneratedBlock", "qwen38_27b_config", "native", "FusedMatVec", "PreparedMatVec", "RecoveredRow", "RecoveredRowMatVec", "Segment",
    "CtoxError", "load", "Q2B64", "Q4B64", "MIXED_Q2Q4B64", "F16", "F32", "BF16", "ACT_IDENTITY",
    "ACT_SILU", "KERNEL_AUTO", "KERNEL_STREAM", "KERNEL_ROWWARP", "PREPARE_KEEP_CANONICAL",
]
