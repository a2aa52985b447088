"""Loads libctox_b200.so and declares the C ABI of include/ctox_b200.h for ctypes.

There is no Python or CPU fallback: if the library cannot be loaded this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

Q2B64, Q4B64, MIXED_Q2Q4B64, F16, F32, BF16 = 0, 1, 2, 3, 4, 5
ACT_IDENTITY, ACT_SILU = 0, 1
SCALE_NONE, SCALE_F32, SCALE_F16LE = 0, 1, 2
KERNEL_AUTO, KERNEL_STREAM, KERNEL_ROWWARP = 0, 1, 2
PREPARE_KEEP_CANONICAL = 1

ERROR_NAMES = {
    1: "Shape",
    2: "InvalidArtifact",
    3: "UnsupportedDType",
    4: "UnsupportedOperation",
    5: "MemoryBudget",
    6: "InvalidState",
    7: "Cancelled",
}


class CtoxError(RuntimeError):
    """Mirror of EngineError (models/qwen38_27b/src/error.rs:5-29)."""

    def __init__(self, code: int, message: str):
        self.code = code
        self.kind = ERROR_NAMES.get(code, f"code {code}")
        super().__init__(f"{self.kind}: {message}")


class Segment(C.Structure):
    """QuantSegment (models/qwen38_27b/src/format.rs:56-64)."""

    _fields_ = [
        ("group_index", C.c_uint32),
        ("dtype", C.c_uint32),
        ("row_start", C.c_uint64),
        ("row_end", C.c_uint64),
        ("offset", C.c_uint64),
        ("length", C.c_uint64),
    ]


MAX_VERIFY_NODES = 16


class SpecRecord(C.Structure):
    """ctox_spec_record (include/ctox_b200.h)."""

    _fields_ = [
        ("status", C.c_uint32),
        ("n_emitted", C.c_uint32),
        ("emitted", C.c_uint32 * (MAX_VERIFY_NODES + 1)),
        ("path", C.c_int32 * MAX_VERIFY_NODES),
        ("node_argmax", C.c_uint32 * MAX_VERIFY_NODES),
        ("node_token", C.c_uint32 * MAX_VERIFY_NODES),
    ]


class ModelConfig(C.Structure):
    """ctox_model_config (include/ctox_b200.h); Qwen38Config (config.rs:12-58) plus deployment."""

    _fields_ = [(n, C.c_uint32) for n in (
        "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
        "num_key_value_heads", "head_dim", "rotary_dim")] + [
        ("rope_theta", C.c_float), ("rms_norm_epsilon", C.c_float)] + [(n, C.c_uint32) for n in (
            "full_attention_interval", "linear_num_key_heads", "linear_num_value_heads",
            "linear_key_head_dim", "linear_value_head_dim", "linear_conv_kernel_dim",
            "mtp_num_hidden_layers", "max_context_tokens", "kv_page_tokens", "kv_dtype",
            "max_draft_tokens", "draft_vocab")]


class ExecStep(C.Structure):
    """ctox_exec_step (include/ctox_b200.h)."""

    _fields_ = [
        ("proposed_drafts", C.c_uint32),
        ("verified_drafts", C.c_uint32),
        ("n_accepted", C.c_uint32),
        ("accepted_draft_tokens", C.c_uint32 * MAX_VERIFY_NODES),
        ("next_token", C.c_uint32),
        ("draft_tokens", C.c_uint32 * MAX_VERIFY_NODES),
        ("target_tokens", C.c_uint32 * (MAX_VERIFY_NODES + 1)),
    ]


(T_EMBED, T_LM_HEAD, T_FINAL_NORM, T_INPUT_NORM, T_POST_NORM, T_ATTN_QKV, T_ATTN_O, T_Q_NORM, T_K_NORM,
 T_LIN_IN, T_LIN_OUT, T_CONV_W, T_A_LOG, T_DT_BIAS, T_LIN_NORM, T_MLP_GATE_UP, T_MLP_DOWN, T_MTP_FC,
 T_MTP_NORM_E, T_MTP_NORM_H, T_MTP_NORM, T_DRAFT_IDS) = range(22)
LAYER_GLOBAL = 0xFFFFFFFF


class FusedMatVecOp(C.Structure):
    _fields_ = [
        ("dtype", C.c_uint32),
        ("activation", C.c_uint32),
        ("weights", C.c_void_p),
        ("weights_len", C.c_uint64),
        ("segments", C.POINTER(Segment)),
        ("n_segments", C.c_uint64),
        ("rows", C.c_uint64),
        ("columns", C.c_uint64),
        ("input", C.c_void_p),
        ("input_len", C.c_uint64),
        ("s_in_kind", C.c_uint32),
        ("s_out_kind", C.c_uint32),
        ("s_in", C.c_void_p),
        ("s_in_len", C.c_uint64),
        ("s_out", C.c_void_p),
        ("s_out_len", C.c_uint64),
        ("bias", C.c_void_p),
        ("bias_len", C.c_uint64),
    ]


# name -> (restype, argtypes); every symbol of include/ctox_b200.h
SIGNATURES = {
    "ctox_abi_version": (C.c_uint32, []),
    "ctox_backend_profile": (C.c_char_p, []),
    "ctox_last_error_message": (C.c_char_p, [C.c_void_p]),
    "ctox_ctx_create": (C.c_int32, [C.c_int32, C.c_void_p, C.POINTER(C.c_void_p)]),
    "ctox_ctx_destroy": (C.c_int32, [C.c_void_p]),
    "ctox_ctx_synchronize": (C.c_int32, [C.c_void_p]),
    "ctox_tp_unique_id": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p]),
    "ctox_tp_init": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.c_int32, C.c_void_p]),
    "ctox_tp_destroy": (C.c_int32, [C.c_void_p]),
    "ctox_tp_all_reduce_f32": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64]),
    "ctox_tp_collective": (C.c_int32, [C.c_void_p, C.POINTER(C.c_char_p)]),
    "ctox_tp_debug_silent_peers": (C.c_int32, [C.c_void_p, C.c_int32, C.c_uint64]),
    "ctox_ctx_allocated_bytes": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "ctox_ctx_device_error": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32)]),
    "ctox_kernel_launches": (C.c_uint64, []),
    "ctox_ctx_kernel_timing": (C.c_int32, [C.c_void_p, C.c_int32]),
    "ctox_ctx_kernel_timing_read": (C.c_int32, [C.c_void_p, C.POINTER(C.c_double),
                                                C.POINTER(C.c_uint64)]),
    "ctox_fused_matvec": (C.c_int32, [C.c_void_p, C.POINTER(FusedMatVecOp), C.c_void_p]),
    "ctox_fused_matvec_fanout": (C.c_int32, [C.c_void_p, C.POINTER(FusedMatVecOp), C.c_uint64,
                                             C.POINTER(C.c_void_p)]),
    "ctox_recovered_row": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64, C.c_uint64,
                                       C.c_uint32, C.c_void_p, C.c_uint64, C.c_float, C.c_void_p]),
    "ctox_recovered_row_matvec": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64,
                                              C.c_void_p, C.c_uint64, C.c_float,
                                              C.POINTER(C.c_float)]),
    "ctox_matvec_prepare": (C.c_int32, [C.c_void_p, C.POINTER(FusedMatVecOp), C.c_uint32,
                                        C.POINTER(C.c_void_p)]),
    "ctox_matvec_destroy": (C.c_int32, [C.c_void_p]),
    "ctox_matvec_dispatch": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64,
                                         C.c_void_p, C.c_uint64, C.c_uint32]),
    "ctox_matvec_dispatch_static": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                                C.c_uint64, C.c_void_p, C.c_uint64]),
    "ctox_matvec_dispatch_host": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p,
                                              C.c_uint32]),
    "ctox_gated_delta_scan": (C.c_int32, [C.c_void_p] + [C.c_void_p] * 8 + [C.c_uint32] * 5),
    "ctox_kv_pack_q4": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]),
    "ctox_kv_demote_q4_to_q2": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]),
    "ctox_kv_unpack": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p]),
    "ctox_gated_delta_scan_layers": (C.c_int32, [C.c_void_p] + [C.c_void_p] * 8 + [C.c_uint32] * 4),
    "ctox_gated_delta_scan_f16_state": (C.c_int32, [C.c_void_p] + [C.c_void_p] * 8 + [C.c_uint32] * 5),
    "ctox_gated_delta_prepare": (C.c_int32, [C.c_void_p] + [C.c_void_p] * 6 + [C.c_uint32] * 2),
    "ctox_argmax_f32": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]),
    "ctox_argmax_f32_host": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p,
                                         C.POINTER(C.c_uint32)]),
    "ctox_matvec_fanout_dispatch": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint32, C.c_uint32,
                                                C.c_uint64, C.c_void_p, C.c_void_p]),
    "ctox_matvec_recovered_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    "ctox_sample_topk_topp": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_float, C.c_uint32, C.c_float,
                                          C.c_float, C.POINTER(C.c_uint32)]),
    "ctox_exec_select_target": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_float, C.c_uint32, C.c_float, C.c_float,
                                            C.POINTER(C.c_uint32)]),
    "ctox_lmhead_verify": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32,
                                       C.POINTER(C.c_int32), C.POINTER(C.c_uint32), C.c_float,
                                       C.c_uint64, C.c_uint64, C.c_uint32, C.c_void_p,
                                       C.POINTER(SpecRecord)]),
    "ctox_exec_create": (C.c_int32, [C.c_void_p, C.POINTER(ModelConfig), C.POINTER(C.c_void_p)]),
    "ctox_exec_destroy": (C.c_int32, [C.c_void_p]),
    "ctox_exec_load_matrix": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(FusedMatVecOp)]),
    "ctox_exec_load_vector": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64]),
    "ctox_exec_fill_synthetic": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_float, C.c_float]),
    "ctox_exec_warmup": (C.c_int32, [C.c_void_p]),
    "ctox_exec_reset_session": (C.c_int32, [C.c_void_p]),
    "ctox_exec_prefill": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]),
    "ctox_exec_prefill_synthetic": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint64]),
    "ctox_exec_decode": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_int32, C.c_float, C.c_uint64, C.c_int32,
                                     C.c_void_p, C.POINTER(ExecStep)]),
    "ctox_exec_commit_speculative": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p]),
    "ctox_exec_session_state": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "ctox_exec_phase_timing": (C.c_int32, [C.c_void_p, C.c_int32]),
    "ctox_exec_last_phase_ms": (C.c_int32, [C.c_void_p, C.POINTER(C.c_float)]),
    "ctox_exec_last_enqueue_us": (C.c_int32, [C.c_void_p, C.POINTER(C.c_double)]),
    "ctox_exec_last_mtp_hidden": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p, C.POINTER(C.c_uint32)]),
    "ctox_exec_last_draft_logits": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p, C.POINTER(C.c_uint32),
                                                C.POINTER(C.c_uint32)]),
    "ctox_exec_position": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "ctox_exec_last_hidden": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "ctox_exec_keep_logits": (C.c_int32, [C.c_void_p, C.c_int32]),
    "ctox_exec_last_logits": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p]),
    "ctox_exec_allocated_bytes": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "ctox_matvec_info": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                                     C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
}

_lib = None


def lib_path() -> str:
    return _build.LIB_PATH


def load() -> C.CDLL:
    """Loads the shared library (building it first only if nvcc is present and it is stale)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_build.LIB_PATH) or (_build.is_stale() and os.path.exists(
            os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc"))):
        _build.build()
    lib = C.CDLL(_build.LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # raises AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
