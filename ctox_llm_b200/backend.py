"""Host-side mirror of the reference's per-op API over the C ABI.

``B200Backend`` has the methods of ``trait Backend`` (models/qwen38_27b/src/backend/mod.rs:153-169)
with the same argument meaning and error kinds as ``CpuBackend`` (backend/cpu.rs). Inputs and
outputs are numpy arrays in host memory, exactly like the borrowed slices / owned ``Vec``s of the
trait. ``PreparedMatVec`` is the resident form (``CudaCandidateRuntime::prepare_fused_matvec`` /
``dispatch_prepared``, backend/cuda_runtime.rs:8341-8382,10560): weights uploaded once, dispatch
on device pointers or host arrays.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import _native as N


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


@dataclass
class FusedMatVec:
    """FusedMatVec<'a> (backend/mod.rs:115-128). A scale given as a ``uint8`` array is
    ``ScaleSlice::F16Le`` (little-endian f16 bytes); a float array is ``ScaleSlice::F32``."""

    dtype: int
    weights: np.ndarray
    rows: int
    columns: int
    input: Optional[np.ndarray]
    segments: Sequence[N.Segment] = field(default_factory=list)
    s_in: Optional[np.ndarray] = None
    s_out: Optional[np.ndarray] = None
    bias: Optional[np.ndarray] = None
    activation: int = N.ACT_IDENTITY


@dataclass
class RecoveredRow:
    """RecoveredRow<'a> (backend/mod.rs:131-141)."""

    dtype: int
    weights: np.ndarray
    columns: int
    s_in: np.ndarray
    s_out: float


@dataclass
class RecoveredRowMatVec:
    """RecoveredRowMatVec<'a> (backend/mod.rs:143-151)."""

    dtype: int
    weights: np.ndarray
    corrected_input: np.ndarray
    s_out: float


def _scale_args(s):
    if s is None:
        return N.SCALE_NONE, None, 0, None
    s = np.asarray(s)
    if s.dtype == np.uint8:
        s = np.ascontiguousarray(s)
        return N.SCALE_F16LE, _ptr(s), s.size // 2, s
    s = _f32(s)
    return N.SCALE_F32, _ptr(s), s.size, s


def _marshal(op: FusedMatVec):
    keep = []
    w = np.ascontiguousarray(op.weights, dtype=np.uint8)
    x = None if op.input is None else _f32(op.input)
    seg = None
    if op.segments:
        seg = (N.Segment * len(op.segments))(*op.segments)
    sik, sip, sil, si = _scale_args(op.s_in)
    sok, sop, sol, so = _scale_args(op.s_out)
    bias = None if op.bias is None else _f32(op.bias)
    keep += [w, x, seg, si, so, bias]
    c = N.FusedMatVecOp(
        op.dtype, op.activation, _ptr(w), w.size,
        C.cast(seg, C.POINTER(N.Segment)) if seg is not None else None, len(op.segments),
        op.rows, op.columns, _ptr(x), 0 if x is None else x.size, sik, sok, sip, sil, sop, sol,
        _ptr(bias), 0 if bias is None else bias.size)
    return c, keep


class B200Backend:
    """``impl Backend`` for the B200 library: kind() == Cuda, no CPU fallback."""

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        self._lib = N.load()
        handle = C.c_void_p()
        rc = self._lib.ctox_ctx_create(device, C.c_void_p(stream) if stream else None,
                                       C.byref(handle))
        if rc:
            raise N.CtoxError(rc, self._lib.ctox_last_error_message(None).decode())
        self._ctx = handle
        self.device = device

    # -- trait Backend ---------------------------------------------------------------------
    def kind(self) -> str:
        return "cuda"

    def promotion_state(self) -> str:
        return "experimental"

    def profile(self) -> str:
        return self._lib.ctox_backend_profile().decode()

    def fused_matvec(self, operation: FusedMatVec) -> np.ndarray:
        c, keep = _marshal(operation)
        out = np.zeros(max(int(operation.rows), 1), dtype=np.float32)
        self._check(self._lib.ctox_fused_matvec(self._ctx, C.byref(c), _ptr(out)))
        return out[: operation.rows]

    def fused_matvec_fanout(self, operations: Sequence[FusedMatVec]) -> list:
        n = len(operations)
        arr = (N.FusedMatVecOp * max(n, 1))()
        keep = []
        for i, op in enumerate(operations):
            arr[i], k = _marshal(op)
            keep.append(k)
        outs = [np.zeros(int(op.rows), dtype=np.float32) for op in operations]
        ptrs = (C.c_void_p * max(n, 1))(*[o.ctypes.data for o in outs])
        self._check(self._lib.ctox_fused_matvec_fanout(self._ctx, arr, n, ptrs))
        return outs

    def recovered_row(self, operation: RecoveredRow) -> np.ndarray:
        w = np.ascontiguousarray(operation.weights, dtype=np.uint8)
        kind, p, n, keep = _scale_args(operation.s_in)
        out = np.zeros(max(int(operation.columns), 1), dtype=np.float32)
        self._check(self._lib.ctox_recovered_row(self._ctx, operation.dtype, _ptr(w), w.size,
                                                 operation.columns, kind, p, n,
                                                 C.c_float(operation.s_out), _ptr(out)))
        return out[: operation.columns]

    def recovered_row_matvec(self, operation: RecoveredRowMatVec) -> float:
        w = np.ascontiguousarray(operation.weights, dtype=np.uint8)
        x = _f32(operation.corrected_input)
        out = C.c_float()
        self._check(self._lib.ctox_recovered_row_matvec(self._ctx, operation.dtype, _ptr(w), w.size,
                                                        _ptr(x), x.size, C.c_float(operation.s_out),
                                                        C.byref(out)))
        return out.value

    # -- resident form ---------------------------------------------------------------------
    def prepare_fused_matvec(self, operation: FusedMatVec, keep_canonical: bool = False
                             ) -> "PreparedMatVec":
        c, keep = _marshal(operation)
        handle = C.c_void_p()
        flags = N.PREPARE_KEEP_CANONICAL if keep_canonical else 0
        self._check(self._lib.ctox_matvec_prepare(self._ctx, C.byref(c), flags, C.byref(handle)))
        return PreparedMatVec(self, handle, int(operation.rows), int(operation.columns))

    # -- gated-delta recurrence (device pointers) -------------------------------------------
    def gated_delta_scan(self, q: int, k: int, v: int, log_decay: int, beta: int, state_in: int,
                         state_out: int, out: int, tokens: int, heads: int, qk_heads: int,
                         key_dim: int = 128, value_dim: int = 128) -> None:
        """recurrent_gated_delta_sequence (reference.rs:377-415) on raw device addresses."""
        self._check(self._lib.ctox_gated_delta_scan(
            self._ctx, *(C.c_void_p(a) for a in (q, k, v, log_decay, beta, state_in, state_out, out)),
            tokens, heads, qk_heads, key_dim, value_dim))

    def gated_delta_scan_layers(self, q: int, k: int, v: int, log_decay: int, beta: int, state_in: int,
                                state_out: int, out: int, layers: int, tokens: int, heads: int, qk_heads: int) -> None:
        """`layers` independent scans in one launch (arrays hold the layers back to back; out may be 0)."""
        self._check(self._lib.ctox_gated_delta_scan_layers(
            self._ctx, *(C.c_void_p(a) if a else None for a in (q, k, v, log_decay, beta, state_in, state_out, out)),
            layers, tokens, heads, qk_heads))

    def gated_delta_scan_f16_state(self, q: int, k: int, v: int, log_decay: int, beta: int, state_in: int,
                                   state_out: int, out: int, tokens: int, heads: int, qk_heads: int) -> None:
        """recurrent_gated_delta_step_f16_state (reference.rs:299-373) over `tokens` tokens: the state
        buffers hold binary16 values, everything else is fp32."""
        self._check(self._lib.ctox_gated_delta_scan_f16_state(
            self._ctx, *(C.c_void_p(a) for a in (q, k, v, log_decay, beta, state_in, state_out, out)),
            tokens, heads, qk_heads, 128, 128))

    # -- K/V rows as packed blocks (kv_cache.rs:22-73) ----------------------------------------
    def kv_pack_q4(self, values: int, n_blocks: int, q4_bytes: int) -> None:
        """QuantizedKvToken::quantize(.., Q4) over n_blocks blocks of 64 floats (device addresses)."""
        self._check(self._lib.ctox_kv_pack_q4(self._ctx, C.c_void_p(values), n_blocks, C.c_void_p(q4_bytes)))

    def kv_demote_q4_to_q2(self, q4_bytes: int, n_blocks: int, q2_bytes: int) -> None:
        """QuantizedKvToken::requantize(Q2) of Q4 blocks (a page leaving the recent window)."""
        self._check(self._lib.ctox_kv_demote_q4_to_q2(self._ctx, C.c_void_p(q4_bytes), n_blocks,
                                                      C.c_void_p(q2_bytes)))

    def kv_unpack(self, dtype: int, packed: int, n_blocks: int, values: int) -> None:
        """QuantizedKvToken::dequantize."""
        self._check(self._lib.ctox_kv_unpack(self._ctx, dtype, C.c_void_p(packed), n_blocks, C.c_void_p(values)))

    def gated_delta_prepare(self, a: int, b: int, a_log: int, dt_bias: int, log_decay: int,
                            beta: int, tokens: int, heads: int) -> None:
        self._check(self._lib.ctox_gated_delta_prepare(
            self._ctx, *(C.c_void_p(x) for x in (a, b, a_log, dt_bias, log_decay, beta)), tokens,
            heads))

    # -- selection ------------------------------------------------------------------------
    def argmax(self, logits_ptr: int, n: int, row_ids_ptr: int = 0) -> int:
        """Greedy token over device logits: last maximal index under f32::total_cmp
        (sampler.rs:76-82); row_ids maps restricted-vocabulary rows to token ids."""
        tok = C.c_uint32()
        self._check(self._lib.ctox_argmax_f32_host(self._ctx, C.c_void_p(logits_ptr), n,
                                                   C.c_void_p(row_ids_ptr) if row_ids_ptr else None,
                                                   C.byref(tok)))
        return tok.value

    # -- housekeeping ----------------------------------------------------------------------
    def sample_topk_topp(self, logits_ptr: int, n: int, temperature: float, top_k: int, top_p: float,
                         draw: float) -> int:
        """Sampler::sample_with_draw (sampler.rs:65-144) over device logits."""
        tok = C.c_uint32()
        self._check(self._lib.ctox_sample_topk_topp(self._ctx, C.c_void_p(logits_ptr), n, C.c_float(temperature),
                                                    top_k, C.c_float(top_p), C.c_float(draw), C.byref(tok)))
        return tok.value

    def fanout_dispatch_device(self, prepared, x_ptr: int, x_dtype: int, positions: int, x_stride: int,
                               y_ptrs, y_strides) -> None:
        """Backend::fused_matvec_fanout over prepared matrices: one set of activation fragments."""
        n = len(prepared)
        handles = (C.c_void_p * n)(*[p._h for p in prepared])
        ys = (C.c_void_p * n)(*[C.c_void_p(int(y)) for y in y_ptrs])
        strides = (C.c_uint64 * n)(*[int(v) for v in y_strides])
        self._check(self._lib.ctox_matvec_fanout_dispatch(handles, n, C.c_void_p(x_ptr), x_dtype, positions,
                                                          x_stride, ys, strides))

    def synchronize(self) -> None:
        self._check(self._lib.ctox_ctx_synchronize(self._ctx))

    def allocated_bytes(self) -> int:
        v = C.c_uint64()
        self._check(self._lib.ctox_ctx_allocated_bytes(self._ctx, C.byref(v)))
        return v.value

    def device_error(self) -> int:
        v = C.c_int32()
        self._check(self._lib.ctox_ctx_device_error(self._ctx, C.byref(v)))
        return v.value

    def kernel_launches(self) -> int:
        """Kernels this library has enqueued in this process so far."""
        return int(self._lib.ctox_kernel_launches())

    def kernel_timing(self, enable: bool) -> None:
        self._check(self._lib.ctox_ctx_kernel_timing(self._ctx, int(enable)))

    def kernel_timing_read(self):
        """(total milliseconds, launches) of the dominant kernel since the last read."""
        ms, n = C.c_double(), C.c_uint64()
        self._check(self._lib.ctox_ctx_kernel_timing_read(self._ctx, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    # -- tensor-parallel group (one process per GPU; no counterpart in the reference) --------
    tp_rank, tp_world = 0, 1

    @staticmethod
    def nccl_library() -> str:
        """The NCCL that torch itself uses, so that one copy of the library serves both."""
        try:
            import nvidia.nccl as pkg
            path = os.path.join(list(pkg.__path__)[0], "lib", "libnccl.so.2")
            if os.path.exists(path):
                return path
        except ImportError:
            pass
        return "libnccl.so.2"

    def tp_unique_id(self) -> bytes:
        buf = (C.c_uint8 * 128)()
        self._check(self._lib.ctox_tp_unique_id(self._ctx, self.nccl_library().encode(), buf))
        return bytes(buf)

    def tp_init(self, rank: int, world: int, unique_id: bytes) -> None:
        if len(unique_id) != 128:
            raise ValueError("a group id is 128 bytes")
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        self._check(self._lib.ctox_tp_init(self._ctx, self.nccl_library().encode(), rank, world, buf))
        self.tp_rank, self.tp_world = rank, world

    def tp_init_from_torch(self) -> None:
        """Joins a group that mirrors the default torch.distributed group (rank 0 draws the id)."""
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        box = [self.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        self.tp_init(rank, world, box[0])

    def tp_collective(self) -> str:
        """"none", "p2p_push" (peer-memory one-shot all-reduce) or "nccl": what sums the group."""
        name = C.c_char_p()
        self._check(self._lib.ctox_tp_collective(self._ctx, C.byref(name)))
        return name.value.decode()

    def tp_debug_silent_peers(self, world: int, wait_limit_cycles: int = 0) -> None:
        """Failure-detection tests: rank 0 of a group whose other ranks never answer."""
        self._check(self._lib.ctox_tp_debug_silent_peers(self._ctx, world, wait_limit_cycles))
        self.tp_rank, self.tp_world = 0, world

    def tp_all_reduce(self, buf_ptr: int, n: int) -> None:
        self._check(self._lib.ctox_tp_all_reduce_f32(self._ctx, C.c_void_p(buf_ptr), n))

    def close(self) -> None:
        if getattr(self, "_ctx", None):
            self._lib.ctox_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int) -> None:
        if rc:
            raise N.CtoxError(rc, self._lib.ctox_last_error_message(self._ctx).decode())


class PreparedMatVec:
    """PreparedCudaMatVec (backend/cuda_runtime.rs:8341-8382): device-resident weights."""

    def __init__(self, backend: B200Backend, handle, rows: int, columns: int):
        self._b = backend
        self._h = handle
        self.rows = rows
        self.columns = columns

    def recovered_rows_device(self, row_ids_ptr: int, n: int, out_ptr: int) -> None:
        """Rows of the matrix times both recovery scales, for row ids in device memory."""
        self._b._check(self._b._lib.ctox_matvec_recovered_rows(self._h, C.c_void_p(row_ids_ptr), n,
                                                               C.c_void_p(out_ptr)))

    def dispatch_host(self, x, positions: int = 1, kernel: int = N.KERNEL_AUTO) -> np.ndarray:
        x = _f32(x)
        if x.size != positions * self.columns:
            raise N.CtoxError(1, f"input has {x.size}, expected {positions * self.columns} values")
        y = np.zeros(positions * self.rows, dtype=np.float32)
        self._b._check(self._b._lib.ctox_matvec_dispatch_host(self._h, _ptr(x), positions, _ptr(y),
                                                              kernel))
        return y.reshape(positions, self.rows) if positions > 1 else y

    def dispatch_device(self, x_ptr: int, x_dtype: int, positions: int, x_stride: int, y_ptr: int,
                        y_stride: int, kernel: int = N.KERNEL_AUTO) -> None:
        """Enqueue on the context's stream; pointers are raw device addresses."""
        self._b._check(self._b._lib.ctox_matvec_dispatch(self._h, C.c_void_p(x_ptr), x_dtype,
                                                         positions, x_stride, C.c_void_p(y_ptr),
                                                         y_stride, kernel))

    def lmhead_verify(self, hidden_ptr: int, hidden_dtype: int, hidden_stride: int, parent, token,
                      temperature: float, seed: int, step: int, vocab: int = 0,
                      logits_out_ptr: int = 0) -> dict:
        """Fused lm_head + softmax statistics + acceptance over a draft tree (this object is the
        lm_head). Returns the emitted tokens (accepted drafts, then the next token), the accepted
        node path and the per-node greedy tokens."""
        n = len(parent)
        par = (C.c_int32 * n)(*[int(x) for x in parent])
        tok = (C.c_uint32 * n)(*[int(x) for x in token])
        rec = N.SpecRecord()
        self._b._check(self._b._lib.ctox_lmhead_verify(
            self._h, C.c_void_p(hidden_ptr), hidden_dtype, hidden_stride, n, par, tok,
            C.c_float(temperature), seed, step, vocab,
            C.c_void_p(logits_out_ptr) if logits_out_ptr else None, C.byref(rec)))
        k = rec.n_emitted
        return {"emitted": [int(x) for x in rec.emitted[:k]],
                "path": [int(x) for x in rec.path[:max(k - 1, 0)]],
                "node_argmax": [int(x) for x in rec.node_argmax[:n]]}

    def dispatch_static(self, x_ptr: int, x_dtype: int, positions: int, x_stride: int, y_ptr: int,
                        y_stride: int) -> None:
        """Same as dispatch_device, but the kernel's scratch is the fixed 8 MiB array inside the
        library, so nothing is allocated: for callers that must not touch the device allocator
        (see ctox_matvec_dispatch_static in include/ctox_b200.h for the limits)."""
        self._b._check(self._b._lib.ctox_matvec_dispatch_static(
            self._h, C.c_void_p(x_ptr), x_dtype, positions, x_stride, C.c_void_p(y_ptr), y_stride))

    def info(self) -> dict:
        r, c, p, d = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
        self._b._check(self._b._lib.ctox_matvec_info(self._h, C.byref(r), C.byref(c), C.byref(p),
                                                     C.byref(d)))
        return {"rows": r.value, "columns": c.value, "packed_bytes": p.value,
                "device_bytes": d.value}

    def destroy(self) -> None:
        if self._h:
            self._b._lib.ctox_matvec_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            if self._b._ctx:
                self.destroy()
        except Exception:
            pass
