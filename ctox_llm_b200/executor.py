"""Host-side mirror of ``trait ModelExecutor`` (models/qwen38_27b/src/engine.rs:322-362) over the
C ABI: load / warmup / prefill / decode / commit_speculative / reset_session / unload / allocations.

``decode`` returns the device-resolved form of a speculative block (engine.rs:110-116,
``ResolvedGreedyMtpVerification``): proposed and verified draft counts, the accepted draft tokens
and the next token. The state is committed on the device for exactly that prefix and the block
stays pending until ``commit_speculative`` names the same depth (the library refuses any other).
Every call that the trait gives a ``CancellationToken`` takes one here (engine.rs:364-377).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import _native as N
from .backend import B200Backend, FusedMatVec, _marshal


class CancellationToken:
    """engine.rs:364-377: a flag another thread may raise; the library reads it between passes."""

    def __init__(self):
        self._word = C.c_int32(0)

    def cancel(self) -> None:
        self._word.value = 1

    def is_cancelled(self) -> bool:
        return self._word.value != 0

    def _ptr(self):
        return C.cast(C.byref(self._word), C.c_void_p)


def _cancel_ptr(token: Optional["CancellationToken"]):
    return token._ptr() if token is not None else None


def qwen38_27b_config(**overrides) -> N.ModelConfig:
    """Qwen38Config::default() (config.rs:35-58) with the benchmark's deployment choices."""
    cfg = N.ModelConfig(
        vocab_size=248_320, hidden_size=5_120, intermediate_size=17_408, num_hidden_layers=64,
        num_attention_heads=24, num_key_value_heads=4, head_dim=256, rotary_dim=64,
        rope_theta=10_000_000.0, rms_norm_epsilon=1e-6, full_attention_interval=4,
        linear_num_key_heads=16, linear_num_value_heads=48, linear_key_head_dim=128,
        linear_value_head_dim=128, linear_conv_kernel_dim=4, mtp_num_hidden_layers=1,
        max_context_tokens=32_768 + 1_024, kv_page_tokens=16, kv_dtype=N.BF16, max_draft_tokens=4,
        draft_vocab=40_000)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


@dataclass
class GeneratedBlock:
    """One decode call: engine.rs GeneratedStep / ResolvedGreedyMtpVerification."""

    token_id: int
    draft_tokens_proposed: int
    draft_tokens_verified: int
    accepted_draft_tokens: List[int]
    draft_tokens: List[int]
    target_tokens: List[int]

    @property
    def emitted(self) -> List[int]:
        return self.accepted_draft_tokens + [self.token_id]


class B200Executor:
    def __init__(self, backend: B200Backend, config: N.ModelConfig):
        self._b = backend
        self._lib = backend._lib
        self.config = config
        handle = C.c_void_p()
        backend._check(self._lib.ctox_exec_create(backend._ctx, C.byref(config), C.byref(handle)))
        self._h = handle

    # -- load ------------------------------------------------------------------------------
    def load_matrix(self, layer: int, tensor: int, op: FusedMatVec) -> None:
        c, keep = _marshal(op)
        self._b._check(self._lib.ctox_exec_load_matrix(self._h, layer, tensor, C.byref(c)))

    def load_vector(self, layer: int, tensor: int, values) -> None:
        v = np.ascontiguousarray(values, dtype=np.uint32 if tensor == N.T_DRAFT_IDS else np.float32)
        self._b._check(self._lib.ctox_exec_load_vector(self._h, layer, tensor,
                                                       v.ctypes.data_as(C.c_void_p), v.size))

    def fill_synthetic(self, seed: int, scale_mu: float = -4.0, scale_sigma: float = 0.5) -> None:
        self._b._check(self._lib.ctox_exec_fill_synthetic(self._h, seed, C.c_float(scale_mu),
                                                          C.c_float(scale_sigma)))

    # -- trait ModelExecutor -----------------------------------------------------------------
    def warmup(self) -> None:
        self._b._check(self._lib.ctox_exec_warmup(self._h))

    def prefill(self, tokens: Sequence[int], cancellation: Optional[CancellationToken] = None) -> None:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        self._b._check(self._lib.ctox_exec_prefill(self._h, t.ctypes.data_as(C.c_void_p), t.size,
                                                   _cancel_ptr(cancellation)))

    def prefill_synthetic(self, n: int, seed: int = 0) -> None:
        self._b._check(self._lib.ctox_exec_prefill_synthetic(self._h, n, seed))

    def decode(self, token: int, mtp_enabled: bool = True, temperature: float = 0.0, seed: int = 0,
               force_accept: int = -1, cancellation: Optional[CancellationToken] = None,
               commit: bool = True) -> GeneratedBlock:
        """One decode call. ``commit=True`` (the default) confirms the device-resolved prefix
        right away, which is what ``Engine::decode`` does with a resolved block (engine.rs:583-640);
        ``commit=False`` leaves the block pending for an explicit ``commit_speculative``."""
        step = N.ExecStep()
        self._b._check(self._lib.ctox_exec_decode(self._h, token, int(mtp_enabled),
                                                  C.c_float(temperature), seed, force_accept,
                                                  _cancel_ptr(cancellation), C.byref(step)))
        k = step.proposed_drafts
        if commit and k > 0:
            self.commit_speculative(step.n_accepted, cancellation)
        return GeneratedBlock(
            token_id=step.next_token, draft_tokens_proposed=k,
            draft_tokens_verified=step.verified_drafts,
            accepted_draft_tokens=[int(x) for x in step.accepted_draft_tokens[:step.n_accepted]],
            draft_tokens=[int(x) for x in step.draft_tokens[:k]],
            target_tokens=[int(x) for x in step.target_tokens[:k + 1]])

    def commit_speculative(self, accepted_drafts: int,
                           cancellation: Optional[CancellationToken] = None) -> None:
        self._b._check(self._lib.ctox_exec_commit_speculative(self._h, accepted_drafts,
                                                              _cancel_ptr(cancellation)))

    def phase_timing(self, enable: bool = True) -> None:
        """Device events at the phase boundaries of every decode call (off by default)."""
        self._b._check(self._lib.ctox_exec_phase_timing(self._h, int(enable)))

    def last_phase_ms(self) -> dict:
        """Device milliseconds of the last decode call's phases (after phase_timing(True))."""
        v = (C.c_float * 4)()
        self._b._check(self._lib.ctox_exec_last_phase_ms(self._h, v))
        return {"drafts": v[0], "target_pass": v[1], "head_and_acceptance": v[2], "commit": v[3]}

    def last_enqueue_us(self) -> float:
        """Host microseconds the last decode spent enqueuing kernels before waiting for the device."""
        v = C.c_double()
        self._b._check(self._lib.ctox_exec_last_enqueue_us(self._h, C.byref(v)))
        return v.value

    def session_state(self) -> dict:
        pending, poisoned = C.c_int32(), C.c_int32()
        self._b._check(self._lib.ctox_exec_session_state(self._h, C.byref(pending), C.byref(poisoned)))
        return {"pending_accepted": pending.value, "poisoned": bool(poisoned.value)}

    def reset_session(self) -> None:
        self._b._check(self._lib.ctox_exec_reset_session(self._h))

    def position(self) -> int:
        v = C.c_uint64()
        self._b._check(self._lib.ctox_exec_position(self._h, C.byref(v)))
        return v.value

    def allocations(self) -> dict:
        m, s = C.c_uint64(), C.c_uint64()
        self._b._check(self._lib.ctox_exec_allocated_bytes(self._h, C.byref(m), C.byref(s)))
        return {"model_bytes": m.value, "session_bytes": s.value}

    # -- evidence paths ----------------------------------------------------------------------
    def last_hidden(self) -> np.ndarray:
        out = np.zeros(self.config.hidden_size, dtype=np.float32)
        self._b._check(self._lib.ctox_exec_last_hidden(self._h, out.ctypes.data_as(C.c_void_p)))
        return out

    def keep_logits(self, enable: bool = True) -> None:
        self._b._check(self._lib.ctox_exec_keep_logits(self._h, int(enable)))

    def last_logits(self, position: int = 0) -> np.ndarray:
        # in a tensor-parallel group: this rank's vocabulary rows [rank * n, (rank + 1) * n)
        out = np.zeros(self.config.vocab_size // self._b.tp_world, dtype=np.float32)
        self._b._check(self._lib.ctox_exec_last_logits(self._h, position,
                                                       out.ctypes.data_as(C.c_void_p)))
        return out

    def last_mtp_hidden(self) -> np.ndarray:
        """[pairs][hidden]: the MTP layer's final hidden of every pair the last decode ran."""
        n = C.c_uint32()
        self._b._check(self._lib.ctox_exec_last_mtp_hidden(self._h, 0, None, C.byref(n)))
        out = np.zeros((n.value, self.config.hidden_size), dtype=np.float32)
        for i in range(n.value):
            self._b._check(self._lib.ctox_exec_last_mtp_hidden(self._h, i, out[i].ctypes.data_as(C.c_void_p), None))
        return out

    def last_draft_logits(self) -> np.ndarray:
        """[drafts][rows of the draft head]: the logits every draft of the last decode was taken from."""
        rows, n = C.c_uint32(), C.c_uint32()
        self._b._check(self._lib.ctox_exec_last_draft_logits(self._h, 0, None, C.byref(rows), C.byref(n)))
        out = np.zeros((n.value, rows.value), dtype=np.float32)
        for i in range(n.value):
            self._b._check(self._lib.ctox_exec_last_draft_logits(self._h, i, out[i].ctypes.data_as(C.c_void_p),
                                                                 None, None))
        return out

    def select_target_token(self, temperature: float, top_k: int, top_p: float, draw: float,
                            position: int = 0) -> int:
        """ModelExecutor::select_target_token over the logits kept by the last decode call."""
        tok = C.c_uint32()
        self._b._check(self._lib.ctox_exec_select_target(self._h, position, C.c_float(temperature), top_k,
                                                         C.c_float(top_p), C.c_float(draw), C.byref(tok)))
        return tok.value

    def unload(self) -> None:
        if self._h:
            self._lib.ctox_exec_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            if self._b._ctx:
                self.unload()
        except Exception:
            pass
