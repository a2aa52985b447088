"""ctypes binding of the CPU oracle (``ctox_oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA library and the timed CPU
baseline. Only the test-suite, the smoke check and the benchmark's CPU-baseline
leg may import this package; the product package never does.

Every wrapper takes and returns numpy arrays and raises :class:`OracleError`
with the reference's error kind (models/qwen38_27b/src/error.rs:5-29).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_DIR, "libctox_oracle.so")

Q2B64, Q4B64, MIXED_Q2Q4B64, F16, F32 = 0, 1, 2, 3, 4
ACT_IDENTITY, ACT_SILU = 0, 1
SCALE_NONE, SCALE_F32, SCALE_F16LE = 0, 1, 2
BLOCK_LEN = 64
BLOCK_BYTES = {Q2B64: 18, Q4B64: 34}

ERROR_NAMES = {
    1: "Shape",
    2: "InvalidArtifact",
    3: "UnsupportedDType",
    4: "UnsupportedOperation",
    5: "MemoryBudget",
    6: "InvalidState",
    7: "Cancelled",
}


class OracleError(RuntimeError):
    def __init__(self, code: int):
        self.code = code
        self.kind = ERROR_NAMES.get(code, f"code {code}")
        super().__init__(f"oracle error: {self.kind}")


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (idempotent)."""
    src = os.path.join(_DIR, "ctox_oracle.c")
    hdr = os.path.join(_DIR, "ctox_oracle.h")
    stale = (
        force
        or not os.path.exists(_LIB_PATH)
        or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(hdr))
    )
    if stale:
        subprocess.check_call(["make", "-s", "-B", "-C", _DIR, "libctox_oracle.so"])
    return _LIB_PATH


class Segment(C.Structure):
    _fields_ = [
        ("group_index", C.c_uint32),
        ("dtype", C.c_uint32),
        ("row_start", C.c_uint64),
        ("row_end", C.c_uint64),
        ("offset", C.c_uint64),
        ("length", C.c_uint64),
    ]


class _FusedMatVec(C.Structure):
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


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_silu.restype = C.c_float
        _lib.orc_silu.argtypes = [C.c_float]
        _lib.orc_softplus.restype = C.c_float
        _lib.orc_softplus.argtypes = [C.c_float]
        _lib.orc_pcg32_next_u32.restype = C.c_uint32
        _lib.orc_pcg32_next_f32.restype = C.c_float
        _lib.orc_u32_to_unit_f32.restype = C.c_float
        _lib.orc_u32_to_unit_f32.argtypes = [C.c_uint32]
        _lib.orc_gumbel_from_bits.restype = C.c_float
        _lib.orc_gumbel_from_bits.argtypes = [C.c_uint32]
        _lib.orc_accept_draw.restype = C.c_float
        _lib.orc_accept_draw.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32]
        _lib.orc_gumbel_noise.restype = C.c_float
        _lib.orc_gumbel_noise.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32]
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise OracleError(rc)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# --------------------------------------------------------------------------- formats
def f16_to_f32(bits: int) -> float:
    return float(lib().orc_f16_to_f32(bits))


def f32_to_f16(value: float) -> int:
    return int(lib().orc_f32_to_f16(C.c_float(value)))


def quantize_matrix(dtype: int, values: np.ndarray) -> np.ndarray:
    """quant.rs Q2Block64/Q4Block64::quantize + encode over a row-major matrix."""
    values = _f32(values)
    rows, columns = values.shape
    out = np.zeros(rows * (columns // BLOCK_LEN) * BLOCK_BYTES[dtype], dtype=np.uint8)
    _check(lib().orc_quantize_matrix(dtype, _ptr(values), C.c_uint64(rows), C.c_uint64(columns),
                                     _ptr(out)))
    return out


def dequantize_blocks(dtype: int, packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    bb = BLOCK_BYTES[dtype]
    n = packed.size // bb
    out = np.zeros((n, BLOCK_LEN), dtype=np.float32)
    fn = lib().orc_q2_dequantize_block if dtype == Q2B64 else lib().orc_q4_dequantize_block
    base = packed.ctypes.data
    for b in range(n):
        _check(fn(C.c_void_p(base + b * bb), C.c_void_p(out.ctypes.data + b * 256)))
    return out


def a8_quantize_block(values: np.ndarray):
    values = _f32(values)
    scale = C.c_float()
    codes = np.zeros(64, dtype=np.int8)
    _check(lib().orc_a8_quantize_block(_ptr(values), C.byref(scale), _ptr(codes)))
    return scale.value, codes


# --------------------------------------------------------------------------- matvec
@dataclass
class FusedMatVec:
    """Mirror of backend/mod.rs:115-128. Scales may be float32 arrays (ScaleSlice::F32)
    or uint8 arrays holding little-endian f16 (ScaleSlice::F16Le)."""

    dtype: int
    weights: np.ndarray
    rows: int
    columns: int
    input: np.ndarray
    segments: Sequence[Segment] = field(default_factory=list)
    s_in: Optional[np.ndarray] = None
    s_out: Optional[np.ndarray] = None
    bias: Optional[np.ndarray] = None
    activation: int = ACT_IDENTITY


def _scale_args(s):
    if s is None:
        return SCALE_NONE, None, 0, None
    if s.dtype == np.uint8:
        s = np.ascontiguousarray(s)
        return SCALE_F16LE, _ptr(s), s.size // 2, s
    s = _f32(s)
    return SCALE_F32, _ptr(s), s.size, s


def _marshal(op: FusedMatVec):
    keep = []
    w = np.ascontiguousarray(op.weights, dtype=np.uint8)
    x = _f32(op.input)
    keep += [w, x]
    seg_arr = None
    if op.segments:
        seg_arr = (Segment * len(op.segments))(*op.segments)
        keep.append(seg_arr)
    sik, sip, sil, si = _scale_args(op.s_in)
    sok, sop, sol, so = _scale_args(op.s_out)
    keep += [si, so]
    bias = None if op.bias is None else _f32(op.bias)
    keep.append(bias)
    c = _FusedMatVec(
        op.dtype, op.activation, _ptr(w), w.size,
        C.cast(seg_arr, C.POINTER(Segment)) if seg_arr is not None else None,
        len(op.segments), op.rows, op.columns, _ptr(x), x.size, sik, sok, sip, sil, sop, sol,
        _ptr(bias), 0 if bias is None else bias.size,
    )
    return c, keep


def fused_matvec(op: FusedMatVec, threads: int = 1, avx2: bool = False) -> np.ndarray:
    """CpuBackend::fused_matvec, ScalarVerifier arm (backend/cpu.rs:432-442)."""
    c, keep = _marshal(op)
    out = np.zeros(max(op.rows, 1), dtype=np.float32)
    if avx2:
        rc = lib().orc_fused_matvec_run_avx2(C.byref(c), _ptr(out), threads)
    elif threads > 1:
        rc = lib().orc_fused_matvec_run_mt(C.byref(c), _ptr(out), threads)
    else:
        rc = lib().orc_fused_matvec_run(C.byref(c), _ptr(out))
    _check(rc)
    return out[: op.rows]


def fused_matvec_fanout(ops: Sequence[FusedMatVec]) -> list:
    """CpuBackend::fused_matvec_fanout (backend/cpu.rs:444-472). Operations that
    pass the *same* numpy array object as input share one corrected input."""
    if not ops:
        raise OracleError(1)
    keep = []
    arr = (_FusedMatVec * len(ops))()
    shared = {}
    for i, op in enumerate(ops):
        c, k = _marshal(op)
        key = id(op.input)
        if key in shared:
            c.input = shared[key]
        else:
            shared[key] = c.input
        arr[i] = c
        keep.append(k)
    outs = [np.zeros(op.rows, dtype=np.float32) for op in ops]
    ptrs = (C.c_void_p * len(ops))(*[o.ctypes.data for o in outs])
    _check(lib().orc_fused_matvec_fanout(arr, C.c_uint64(len(ops)), ptrs))
    return outs


def recovered_row(dtype, weights, columns, s_in, s_out: float) -> np.ndarray:
    w = np.ascontiguousarray(weights, dtype=np.uint8)
    kind, p, n, keep = _scale_args(s_in)
    out = np.zeros(columns, dtype=np.float32)
    _check(lib().orc_recovered_row(dtype, _ptr(w), C.c_uint64(w.size), C.c_uint64(columns), kind, p,
                                   C.c_uint64(n), C.c_float(s_out), _ptr(out)))
    return out


def recovered_row_matvec(dtype, weights, corrected_input, s_out: float) -> float:
    w = np.ascontiguousarray(weights, dtype=np.uint8)
    x = _f32(corrected_input)
    out = C.c_float()
    _check(lib().orc_recovered_row_matvec(dtype, _ptr(w), C.c_uint64(w.size), _ptr(x),
                                          C.c_uint64(x.size), C.c_float(s_out), C.byref(out)))
    return out.value


# --------------------------------------------------------------------------- reference.rs ops
def silu(v: float) -> float:
    return float(lib().orc_silu(C.c_float(v)))


def softplus(v: float) -> float:
    return float(lib().orc_softplus(C.c_float(v)))


def rms_norm_1p_weight(values, rows, columns, weight, epsilon=1e-6):
    values, weight = _f32(values), _f32(weight)
    if weight.size != columns or values.size != rows * columns:
        raise OracleError(1)
    out = np.zeros(rows * columns, dtype=np.float32)
    _check(lib().orc_rms_norm_1p_weight(_ptr(values), C.c_uint64(rows), C.c_uint64(columns),
                                        _ptr(weight), C.c_float(epsilon), _ptr(out)))
    return out


def rms_norm_gated(values, gate, rows, columns, weight, epsilon=1e-6):
    values, gate, weight = _f32(values), _f32(gate), _f32(weight)
    if weight.size != columns or values.size != rows * columns or gate.size != values.size:
        raise OracleError(1)
    out = np.zeros(rows * columns, dtype=np.float32)
    _check(lib().orc_rms_norm_gated(_ptr(values), _ptr(gate), C.c_uint64(rows), C.c_uint64(columns),
                                    _ptr(weight), C.c_float(epsilon), _ptr(out)))
    return out


def swiglu(gate, up):
    gate, up = _f32(gate), _f32(up)
    if gate.size != up.size:
        raise OracleError(1)
    out = np.zeros(gate.size, dtype=np.float32)
    _check(lib().orc_swiglu(_ptr(gate), _ptr(up), C.c_uint64(gate.size), _ptr(out)))
    return out


def apply_partial_rope(query, key, query_heads, key_heads, head_dim, rotary_dim, position, theta):
    q, k = _f32(query).copy(), _f32(key).copy()
    if q.size != query_heads * head_dim or k.size != key_heads * head_dim:
        raise OracleError(1)
    _check(lib().orc_apply_partial_rope(_ptr(q), _ptr(k), C.c_uint64(query_heads),
                                        C.c_uint64(key_heads), C.c_uint64(head_dim),
                                        C.c_uint64(rotary_dim), C.c_uint64(position),
                                        C.c_float(theta)))
    return q, k


def causal_conv_silu_update(inp, state, weight, channels, kernel):
    """Returns (output, new_state); `state` is not modified."""
    inp, st, weight = _f32(inp), _f32(state).copy(), _f32(weight)
    if inp.size != channels or st.size != channels * kernel or weight.size != channels * kernel:
        raise OracleError(1)
    out = np.zeros(channels, dtype=np.float32)
    _check(lib().orc_causal_conv_silu_update(_ptr(inp), _ptr(st), _ptr(weight), C.c_uint64(channels),
                                             C.c_uint64(kernel), _ptr(out)))
    return out, st


def causal_conv_silu_update_f16_state(inp, state_bits, weight, channels, kernel):
    inp, weight = _f32(inp), _f32(weight)
    st = np.ascontiguousarray(state_bits, dtype=np.uint16).copy()
    out = np.zeros(channels, dtype=np.float32)
    _check(lib().orc_causal_conv_silu_update_f16_state(_ptr(inp), _ptr(st), _ptr(weight),
                                                       C.c_uint64(channels), C.c_uint64(kernel),
                                                       _ptr(out)))
    return out, st


def recurrent_gated_delta_step(query, key, value, log_decay, beta, state, heads, key_dim, value_dim):
    """Returns (output, new_state) (reference.rs:230-297)."""
    q, k, v = _f32(query), _f32(key), _f32(value)
    g, b, st = _f32(log_decay), _f32(beta), _f32(state).copy()
    if (q.size != heads * key_dim or k.size != q.size or v.size != heads * value_dim
            or g.size != heads or b.size != heads or st.size != heads * key_dim * value_dim):
        raise OracleError(1)
    out = np.zeros(heads * value_dim, dtype=np.float32)
    _check(lib().orc_recurrent_gated_delta_step(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(b), _ptr(st),
                                                C.c_uint64(heads), C.c_uint64(key_dim),
                                                C.c_uint64(value_dim), _ptr(out)))
    return out, st


def recurrent_gated_delta_step_f16_state(query, key, value, log_decay, beta, state_bits, heads,
                                         key_dim, value_dim):
    q, k, v = _f32(query), _f32(key), _f32(value)
    g, b = _f32(log_decay), _f32(beta)
    st = np.ascontiguousarray(state_bits, dtype=np.uint16).copy()
    out = np.zeros(heads * value_dim, dtype=np.float32)
    _check(lib().orc_recurrent_gated_delta_step_f16_state(
        _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(b), _ptr(st), C.c_uint64(heads),
        C.c_uint64(key_dim), C.c_uint64(value_dim), _ptr(out)))
    return out, st


def recurrent_gated_delta_sequence(query, key, value, log_decay, beta, state, tokens, heads,
                                   key_dim, value_dim):
    """Returns (output [tokens, heads*value_dim], new_state) (reference.rs:377-415)."""
    q, k, v = _f32(query), _f32(key), _f32(value)
    g, b, st = _f32(log_decay), _f32(beta), _f32(state).copy()
    if (q.size != tokens * heads * key_dim or k.size != q.size
            or v.size != tokens * heads * value_dim or g.size != tokens * heads
            or b.size != tokens * heads or st.size != heads * key_dim * value_dim):
        raise OracleError(1)
    out = np.zeros(tokens * heads * value_dim, dtype=np.float32)
    _check(lib().orc_recurrent_gated_delta_sequence(
        _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(b), _ptr(st), C.c_uint64(tokens), C.c_uint64(heads),
        C.c_uint64(key_dim), C.c_uint64(value_dim), _ptr(out)))
    return out.reshape(tokens, heads * value_dim), st


def grouped_query_attention(query, key, value, query_heads, kv_heads, query_tokens, kv_tokens,
                            head_dim, query_start_position):
    q, k, v = _f32(query), _f32(key), _f32(value)
    if (q.size != query_heads * query_tokens * head_dim or k.size != kv_heads * kv_tokens * head_dim
            or v.size != k.size):
        raise OracleError(1)
    out = np.zeros(query_tokens * query_heads * head_dim, dtype=np.float32)
    _check(lib().orc_grouped_query_attention(
        _ptr(q), _ptr(k), _ptr(v), C.c_uint64(query_heads), C.c_uint64(kv_heads),
        C.c_uint64(query_tokens), C.c_uint64(kv_tokens), C.c_uint64(head_dim),
        C.c_uint64(query_start_position), _ptr(out)))
    return out


def sigmoid_gate(values, gate):
    v, g = _f32(values).copy(), _f32(gate)
    if v.size != g.size:
        raise OracleError(1)
    _check(lib().orc_sigmoid_gate(_ptr(v), _ptr(g), C.c_uint64(v.size)))
    return v


def repeat_heads(x, source_heads, target_heads, head_dim):
    x = _f32(x)
    out = np.zeros(target_heads * head_dim, dtype=np.float32)
    _check(lib().orc_repeat_heads(_ptr(x), C.c_uint64(source_heads), C.c_uint64(target_heads),
                                  C.c_uint64(head_dim), _ptr(out)))
    return out


def gated_delta_prepare(a, b, a_log, dt_bias):
    a, b, a_log, dt_bias = _f32(a), _f32(b), _f32(a_log), _f32(dt_bias)
    heads = a.size
    g = np.zeros(heads, dtype=np.float32)
    beta = np.zeros(heads, dtype=np.float32)
    _check(lib().orc_gated_delta_prepare(_ptr(a), _ptr(b), _ptr(a_log), _ptr(dt_bias),
                                         C.c_uint64(heads), _ptr(g), _ptr(beta)))
    return g, beta


# --------------------------------------------------------------------------- selection
def greedy_token(logits) -> int:
    l = _f32(logits)
    tok = C.c_uint32()
    _check(lib().orc_greedy_token(_ptr(l), C.c_uint64(l.size), C.byref(tok)))
    return tok.value


def sample_with_draw(logits, temperature, top_k, top_p, draw) -> int:
    l = _f32(logits)
    tok = C.c_uint32()
    _check(lib().orc_sample_with_draw(_ptr(l), C.c_uint64(l.size), C.c_float(temperature),
                                      C.c_uint64(top_k), C.c_float(top_p), C.c_float(draw),
                                      C.byref(tok)))
    return tok.value


class Pcg32:
    """sampler.rs:149-174."""

    def __init__(self, seed: int):
        self._state = C.c_uint64()
        lib().orc_pcg32_new(C.c_uint64(seed), C.byref(self._state))

    def next_u32(self) -> int:
        return int(lib().orc_pcg32_next_u32(C.byref(self._state)))

    def next_f32(self) -> float:
        return float(lib().orc_pcg32_next_f32(C.byref(self._state)))


def verify_greedy_mtp_tokens(draft_tokens, target_tokens, bonus_token):
    """engine.rs:923-938. Returns (next_token, verified, accepted list)."""
    d = np.ascontiguousarray(draft_tokens, dtype=np.uint32)
    t = np.ascontiguousarray(target_tokens, dtype=np.uint32)
    acc = np.zeros(max(d.size, 1), dtype=np.uint32)
    nxt, ver, na = C.c_uint32(), C.c_uint32(), C.c_uint32()
    _check(lib().orc_verify_greedy_mtp_tokens(_ptr(d), _ptr(t), C.c_uint64(d.size),
                                              C.c_uint32(bonus_token), C.byref(nxt), C.byref(ver),
                                              _ptr(acc), C.byref(na)))
    return nxt.value, ver.value, [int(x) for x in acc[: na.value]]


def verify_greedy_mtp_logits(draft_logits, target_logits, bonus_logits, draft_token_ids=None):
    """engine.rs:939-962. draft_token_ids[i] (or None) gives a Restricted distribution."""
    k = len(draft_logits)
    dl = [_f32(x) for x in draft_logits]
    tl = [_f32(x) for x in target_logits]
    vocab = tl[0].size if tl else 0
    ids = [None] * k if draft_token_ids is None else [
        None if x is None else np.ascontiguousarray(x, dtype=np.uint32) for x in draft_token_ids]
    dlp = (C.c_void_p * k)(*[x.ctypes.data for x in dl])
    dlen = (C.c_uint64 * k)(*[x.size for x in dl])
    idp = (C.c_void_p * k)(*[None if x is None else x.ctypes.data for x in ids])
    tlp = (C.c_void_p * k)(*[x.ctypes.data for x in tl])
    bonus = None if bonus_logits is None else _f32(bonus_logits)
    acc = np.zeros(max(k, 1), dtype=np.uint32)
    nxt, ver, na = C.c_uint32(), C.c_uint32(), C.c_uint32()
    _check(lib().orc_verify_greedy_mtp_logits(dlp, dlen, idp, tlp, C.c_uint64(vocab), C.c_uint64(k),
                                              _ptr(bonus), C.byref(nxt), C.byref(ver), _ptr(acc),
                                              C.byref(na)))
    return nxt.value, ver.value, [int(x) for x in acc[: na.value]]


# --------------------------------------------------------------------------- RNG + tree acceptance
def philox4x32_10(counter, key):
    ctr = (C.c_uint32 * 4)(*counter)
    k = (C.c_uint32 * 2)(*key)
    out = (C.c_uint32 * 4)()
    lib().orc_philox4x32_10(ctr, k, out)
    return [int(x) for x in out]


def accept_draw(seed, step, node) -> float:
    return float(lib().orc_accept_draw(seed, step, node))


def gumbel_noise(seed, step, node, token) -> float:
    return float(lib().orc_gumbel_noise(seed, step, node, token))


def gumbel_from_bits(bits) -> float:
    return float(lib().orc_gumbel_from_bits(bits))


def softmax_stats(logits, inv_temperature):
    l = _f32(logits)
    m, s = C.c_float(), C.c_float()
    _check(lib().orc_softmax_stats(_ptr(l), C.c_uint64(l.size), C.c_float(inv_temperature),
                                   C.byref(m), C.byref(s)))
    return m.value, s.value


def spec_tree_accept(target_logits, parent, node_token, temperature, seed, step):
    """Returns (emitted tokens, accepted node path)."""
    tl = _f32(target_logits)
    n_nodes, vocab = tl.shape
    par = np.ascontiguousarray(parent, dtype=np.int32)
    tok = np.ascontiguousarray(node_token, dtype=np.uint32)
    emitted = np.zeros(n_nodes + 1, dtype=np.uint32)
    path = np.full(n_nodes + 1, -1, dtype=np.int32)
    n = C.c_uint32()
    _check(lib().orc_spec_tree_accept(_ptr(tl), C.c_uint64(vocab), _ptr(par), _ptr(tok),
                                      C.c_uint64(n_nodes), C.c_float(temperature), C.c_uint64(seed),
                                      C.c_uint64(step), _ptr(emitted), C.byref(n), _ptr(path)))
    return [int(x) for x in emitted[: n.value]], [int(x) for x in path[: n.value - 1]]
