"""CTOXQ container: reader, writer and the executor loader (host side, no device work).

The container of the reference (models/qwen38_27b/src/format.rs): a 64-byte header
(`FileHeader`, format.rs:394-450: magic "CTOXQ2Q4", version 1..2, endian marker 0x01020304,
manifest length, data offset, tensor count, alignment), a JSON manifest (`ModelManifest`,
format.rs:293-391) and an aligned tensor-data region; every tensor carries its SHA-256. Quantised
matrices are Q2_B64 / Q4_B64 blocks, or contiguous row groups of either (`QuantSegment`,
format.rs:56-64, manifest v2); a matrix `name` has FP16 recovery scales `name.s_in` [columns] and
`name.s_out` [rows] (loader.rs:192-230 `RecoveredMatrixView`).

`CtoxqArtifact.open` applies the reference's validation (header, manifest, alignment, ranges,
lengths, optional checksums) and hands out zero-copy views; `load_into_executor` builds the
fan-out matrices of the executor ([q|k|v], [in_proj_qkv|z|a|b], [gate|up]) from the tensor names of
the reference (tensor_contract.rs:70-249) and checks that the members of a fan-out group share
one s_in (fanout.rs:31-70). `fanout_groups` / `fanout_group_sha256` restate the frozen group list
and its digest. `write_ctoxq` is `ArtifactBuilder::write_new` (format.rs:472-560).
"""
from __future__ import annotations

import hashlib
import json
import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _native as N
from ._native import CtoxError
from .backend import FusedMatVec

MAGIC = b"CTOXQ2Q4"
ENDIAN_MARKER = 0x01020304
HEADER = struct.Struct("<8sIIQQII24x")
HEADER_BYTES = 64
DEFAULT_ALIGNMENT = 256
BLOCK_LEN = 64
BLOCK_BYTES = {"q2_b64": 18, "q4_b64": 34}
DTYPE_CODE = {"q2_b64": N.Q2B64, "q4_b64": N.Q4B64, "mixed_q2_q4_b64": N.MIXED_Q2Q4B64}
INVALID_ARTIFACT, SHAPE, UNSUPPORTED_DTYPE = 2, 1, 3


def _bad(msg: str) -> CtoxError:
    return CtoxError(INVALID_ARTIFACT, msg)


def align_up(value: int, alignment: int) -> int:  # format.rs:452-462
    if alignment <= 0 or alignment & (alignment - 1):
        raise _bad(f"invalid alignment {alignment}")
    return (value + alignment - 1) & ~(alignment - 1)


def expected_bytes(dtype: str, shape: Sequence[int], segments: Sequence[dict]) -> int:
    """TensorEntry::expected_bytes (format.rs:209-290)."""
    if not shape or any(int(d) <= 0 for d in shape):
        raise _bad("tensor shape is empty or has a zero dimension")
    elements = 1
    for d in shape:
        elements *= int(d)
    if dtype in BLOCK_BYTES:
        if segments:
            raise _bad("non-mixed tensor declares row segments")
        return -(-elements // BLOCK_LEN) * BLOCK_BYTES[dtype]
    if dtype == "mixed_q2_q4_b64":
        if len(shape) != 2 or int(shape[1]) % BLOCK_LEN or not segments:
            raise _bad("mixed Q2/Q4 tensor must be a block-aligned matrix with row segments")
        row = offset = 0
        for index, seg in enumerate(segments):
            if (int(seg["group_index"]) != index or int(seg["row_start"]) != row or int(seg["row_end"]) <= row
                    or int(seg["row_end"]) > int(shape[0]) or int(seg["offset"]) != offset
                    or seg["dtype"] not in BLOCK_BYTES):
                raise _bad(f"mixed Q2/Q4 segment {index} is not contiguous")
            length = (int(seg["row_end"]) - row) * (int(shape[1]) // BLOCK_LEN) * BLOCK_BYTES[seg["dtype"]]
            if int(seg["length"]) != length:
                raise _bad(f"mixed Q2/Q4 segment {index} has {seg['length']} bytes, expected {length}")
            row, offset = int(seg["row_end"]), offset + length
        if row != int(shape[0]):
            raise _bad("mixed Q2/Q4 segments do not cover all rows")
        return offset
    if dtype == "f16":
        return elements * 2
    if dtype == "f32":
        return elements * 4
    raise _bad(f"unsupported tensor dtype {dtype}")  # e.g. a Q3 dtype is not a manifest dtype (format.rs:591-600)


def validate_manifest(manifest: dict, data_len: int) -> None:
    """ModelManifest::validate (format.rs:306-391), without the recovery-provenance hashes."""
    fmt = manifest.get("format")
    if fmt not in ("ctox.q2q4.v1", "ctox.q2q4.v2"):
        raise _bad(f"unsupported manifest format {fmt}")
    if not manifest.get("model") or len(str(manifest.get("revision", ""))) < 7:
        raise _bad("model and immutable revision are required")
    alignment = int(manifest.get("alignment", 0))
    if alignment < 64 or alignment & (alignment - 1):
        raise _bad(f"alignment {alignment} must be a power of two >= 64")
    tensors = manifest.get("tensors", [])
    if fmt == "ctox.q2q4.v1" and any(t["dtype"] == "mixed_q2_q4_b64" for t in tensors):
        raise _bad("mixed Q2/Q4 tensors require manifest v2")
    names, ranges = set(), []
    for t in tensors:
        name = str(t.get("name", ""))
        if not name or name in names:
            raise _bad(f"tensor name is empty or duplicated: {name}")
        names.add(name)
        offset, length = int(t["offset"]), int(t["length"])
        if offset % alignment:
            raise _bad(f"tensor {name} offset {offset} is not {alignment}-byte aligned")
        digest = str(t.get("sha256", ""))
        if len(digest) != 64 or any(c not in "0123456789abcdefABCDEF" for c in digest):
            raise _bad(f"tensor {name} has an invalid SHA-256")
        want = expected_bytes(str(t["dtype"]), t["shape"], t.get("segments", []))
        if length != want:
            raise _bad(f"tensor {name} has {length} bytes, {t['dtype']} shape requires {want}")
        if offset + length > data_len:
            raise _bad(f"tensor {name} ends at {offset + length}, data region has {data_len} bytes")
        ranges.append((offset, offset + length, name))
    ranges.sort()
    for left, right in zip(ranges, ranges[1:]):
        if left[1] > right[0]:
            raise _bad(f"tensor ranges {left[2]} and {right[2]} overlap")


@dataclass
class PackedTensor:  # format.rs:464-470
    name: str
    dtype: str
    shape: Sequence[int]
    data: bytes
    segments: Sequence[dict] = ()


def write_ctoxq(path: str, tensors: Sequence[PackedTensor], model: str = "test/qwen", revision: str = "0123456789abcdef",
                target: str = "cuda-sm100a-b200", alignment: int = DEFAULT_ALIGNMENT) -> dict:
    """ArtifactBuilder::write_new (format.rs:472-560): header, manifest, zero padding, aligned payloads."""
    version = 2 if any(t.dtype == "mixed_q2_q4_b64" for t in tensors) else 1
    entries, offset = [], 0
    for t in tensors:
        data = bytes(t.data)
        entry = {"name": t.name, "dtype": t.dtype, "shape": [int(d) for d in t.shape], "offset": offset,
                 "length": len(data), "sha256": hashlib.sha256(data).hexdigest()}
        if t.segments:
            entry["segments"] = [dict(s) for s in t.segments]
        entries.append(entry)
        offset = align_up(offset + len(data), alignment)
    manifest = {"format": f"ctox.q2q4.v{version}", "model": model, "revision": revision, "alignment": alignment,
                "target": target, "tensors": entries}
    data_len = max((e["offset"] + e["length"] for e in entries), default=0)
    validate_manifest(manifest, data_len)
    blob = json.dumps(manifest, separators=(",", ":")).encode()
    data_offset = align_up(HEADER_BYTES + len(blob), alignment)
    with open(path, "xb") as f:
        f.write(HEADER.pack(MAGIC, version, ENDIAN_MARKER, len(blob), data_offset, len(entries), alignment))
        f.write(blob)
        f.write(b"\0" * (data_offset - HEADER_BYTES - len(blob)))
        pos = 0
        for t, e in zip(tensors, entries):
            f.write(b"\0" * (e["offset"] - pos))
            f.write(bytes(t.data))
            pos = e["offset"] + e["length"]
    return manifest


class CtoxqArtifact:
    """ModelArtifact (loader.rs:232-330): an immutable mapping of a container file."""

    def __init__(self, path: str, verify_checksums: bool = True):
        self.path = path
        self._file = open(path, "rb")
        try:
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError:
            self._file.close()
            raise _bad("header is 0 bytes, expected at least 64")
        try:
            if len(self._map) < HEADER_BYTES:
                raise _bad(f"header is {len(self._map)} bytes, expected at least {HEADER_BYTES}")
            magic, version, endian, manifest_len, data_offset, tensor_count, alignment = HEADER.unpack_from(self._map)
            if magic != MAGIC:
                raise _bad("bad CTOX Q2/Q4 magic")
            if version not in (1, 2):
                raise _bad(f"format version {version} is unsupported")
            if endian != ENDIAN_MARKER:
                raise _bad("endianness marker mismatch")
            manifest_end = HEADER_BYTES + manifest_len
            if manifest_end > len(self._map) or data_offset > len(self._map):
                raise _bad("manifest or data offset lies beyond file")
            if data_offset < manifest_end:
                raise _bad("tensor data overlaps manifest")
            blob = self._map[HEADER_BYTES:manifest_end]
            self.manifest_sha256 = hashlib.sha256(blob).hexdigest()
            try:
                self.manifest = json.loads(blob)
            except ValueError as e:
                raise _bad(f"manifest is not JSON: {e}")
            if self.manifest.get("format") != f"ctox.q2q4.v{version}":
                raise _bad(f"header version {version} requires manifest ctox.q2q4.v{version}, got "
                           f"{self.manifest.get('format')}")
            if int(self.manifest.get("alignment", 0)) != alignment or len(self.manifest.get("tensors", [])) != tensor_count:
                raise _bad("header and manifest disagree on alignment or tensor count")
            self.data_offset = int(data_offset)
            validate_manifest(self.manifest, len(self._map) - self.data_offset)
            self.tensors: Dict[str, dict] = {t["name"]: t for t in self.manifest["tensors"]}
            if verify_checksums:  # ChecksumPolicy::AllTensors
                for name in self.tensors:
                    self.verify_tensor(name)
        except Exception:
            self.close()
            raise

    @classmethod
    def open(cls, path: str, verify_checksums: bool = True) -> "CtoxqArtifact":
        return cls(path, verify_checksums)

    def close(self) -> None:
        for h in ("_map", "_file"):
            obj = getattr(self, h, None)
            if obj is not None:
                try:
                    obj.close()
                except (BufferError, ValueError):
                    pass  # views handed out are still alive; the mapping goes with them
                setattr(self, h, None)

    def file_bytes(self) -> int:
        return len(self._map)

    def tensor_bytes(self, name: str) -> np.ndarray:
        """Zero-copy uint8 view of a tensor's payload."""
        t = self._entry(name)
        start = self.data_offset + int(t["offset"])
        return np.frombuffer(self._map, dtype=np.uint8, count=int(t["length"]), offset=start)

    def verify_tensor(self, name: str) -> None:
        if hashlib.sha256(self.tensor_bytes(name)).hexdigest() != str(self._entry(name)["sha256"]).lower():
            raise _bad(f"tensor {name} checksum differs")

    def _entry(self, name: str) -> dict:
        if name not in self.tensors:
            raise _bad(f"tensor {name} is not in the artifact")
        return self.tensors[name]

    def float_tensor(self, name: str) -> np.ndarray:
        """FloatTensorView::to_f32_vec (loader.rs:120-175): F16 or F32, non-finite values refused."""
        t = self._entry(name)
        raw = self.tensor_bytes(name)
        if t["dtype"] == "f16":
            v = raw.view("<f2").astype(np.float32)
        elif t["dtype"] == "f32":
            v = raw.view("<f4").astype(np.float32)
        else:
            raise CtoxError(UNSUPPORTED_DTYPE, f"tensor {name} is {t['dtype']}, not a float tensor")
        if not np.all(np.isfinite(v)):
            raise _bad(f"float tensor {name} holds a non-finite value")
        return v

    def recovery_scales(self, name: str) -> np.ndarray:
        """FloatTensorView::as_recovery_scales: the on-disk FP16 bytes; F32 is refused (loader.rs:177-187)."""
        if self._entry(name)["dtype"] != "f16":
            raise CtoxError(UNSUPPORTED_DTYPE, "recovery scales must be packed FP16")
        return self.tensor_bytes(name)

    def recovered_matrix(self, name: str) -> FusedMatVec:
        """RecoveredMatrixView::operation without an input (loader.rs:192-230)."""
        t = self._entry(name)
        if t["dtype"] not in DTYPE_CODE or len(t["shape"]) != 2:
            raise CtoxError(UNSUPPORTED_DTYPE, f"tensor {name} is not a packed Q2/Q4 matrix")
        rows, cols = int(t["shape"][0]), int(t["shape"][1])
        segs = [N.Segment(int(s["group_index"]), DTYPE_CODE[s["dtype"]], int(s["row_start"]), int(s["row_end"]),
                          int(s["offset"]), int(s["length"])) for s in t.get("segments", [])]
        s_in, s_out = self.recovery_scales(f"{name}.s_in"), self.recovery_scales(f"{name}.s_out")
        if s_in.size != 2 * cols or s_out.size != 2 * rows:
            raise CtoxError(SHAPE, f"recovery scales of {name} do not match its {rows}x{cols} shape")
        return FusedMatVec(DTYPE_CODE[t["dtype"]], self.tensor_bytes(name), rows, cols, None, segments=segs,
                           s_in=s_in, s_out=s_out)


# ---- fan-out groups (fanout.rs:31-70; training/fanout_recovery.py writes the same list)
def fanout_groups(num_hidden_layers: int = 64, full_attention_interval: int = 4) -> List[dict]:
    def group(kind, prefix, projections):
        return {"kind": kind, "prefix": prefix,
                "scale_names": [f"{prefix}.{p}.weight.s_in" for p in projections]}

    groups = []
    for layer in range(num_hidden_layers):
        prefix = f"model.language_model.layers.{layer}"
        groups.append(group("mlp_gate_up", f"{prefix}.mlp", ["gate_proj", "up_proj"]))
        if (layer + 1) % full_attention_interval == 0:
            groups.append(group("full_attention_qkv", f"{prefix}.self_attn", ["q_proj", "k_proj", "v_proj"]))
        else:
            groups.append(group("linear_attention_inputs", f"{prefix}.linear_attn",
                                ["in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b"]))
    groups.append(group("mlp_gate_up", "mtp.layers.0.mlp", ["gate_proj", "up_proj"]))
    groups.append(group("full_attention_qkv", "mtp.layers.0.self_attn", ["q_proj", "k_proj", "v_proj"]))
    groups.sort(key=lambda g: (g["kind"], g["prefix"]))
    return groups


def fanout_group_sha256(groups: List[dict]) -> str:
    """serde_json::to_vec of the group list (field order kind, prefix, scale_names; no spaces)."""
    return hashlib.sha256(json.dumps(groups, separators=(",", ":")).encode()).hexdigest()


# ---- executor loading
def _concat_rows(ops: List[FusedMatVec], group_name: str) -> FusedMatVec:
    """Rows of a fan-out group as one matrix; the members must be pure, of one code format and share
    one s_in (fanout.rs: one logical s_in per group)."""
    first = ops[0]
    for op in ops[1:]:
        if op.dtype != first.dtype or op.segments or first.segments or op.columns != first.columns:
            raise CtoxError(4, f"fan-out group {group_name}: members must be pure matrices of one code format and width")
        if not np.array_equal(op.s_in, first.s_in):
            raise _bad(f"fan-out group {group_name}: members do not share one s_in")
    return FusedMatVec(first.dtype, np.concatenate([op.weights for op in ops]), sum(op.rows for op in ops),
                       first.columns, None, s_in=first.s_in, s_out=np.concatenate([op.s_out for op in ops]))


def load_into_executor(art: CtoxqArtifact, ex, draft_token_ids: Optional[Sequence[int]] = None) -> None:
    """ModelExecutor::load for a one-GPU executor: every tensor of the model by its name in the
    reference's tensor contract (tensor_contract.rs:70-249), fan-out groups as single matrices."""
    c, G = ex.config, N.LAYER_GLOBAL
    ex.load_matrix(G, N.T_EMBED, art.recovered_matrix("model.language_model.embed_tokens.weight"))
    ex.load_matrix(G, N.T_LM_HEAD, art.recovered_matrix("lm_head.weight"))
    ex.load_vector(G, N.T_FINAL_NORM, art.float_tensor("model.language_model.norm.weight"))
    for l in range(c.num_hidden_layers + c.mtp_num_hidden_layers):
        mtp = l >= c.num_hidden_layers
        prefix = "mtp.layers.0" if mtp else f"model.language_model.layers.{l}"
        full = mtp or (l + 1) % c.full_attention_interval == 0
        ex.load_vector(l, N.T_INPUT_NORM, art.float_tensor(f"{prefix}.input_layernorm.weight"))
        ex.load_vector(l, N.T_POST_NORM, art.float_tensor(f"{prefix}.post_attention_layernorm.weight"))
        if full:
            a = f"{prefix}.self_attn"
            ex.load_matrix(l, N.T_ATTN_QKV, _concat_rows(
                [art.recovered_matrix(f"{a}.{p}.weight") for p in ("q_proj", "k_proj", "v_proj")], a))
            ex.load_matrix(l, N.T_ATTN_O, art.recovered_matrix(f"{a}.o_proj.weight"))
            ex.load_vector(l, N.T_Q_NORM, art.float_tensor(f"{a}.q_norm.weight"))
            ex.load_vector(l, N.T_K_NORM, art.float_tensor(f"{a}.k_norm.weight"))
        else:
            a = f"{prefix}.linear_attn"
            ex.load_matrix(l, N.T_LIN_IN, _concat_rows(
                [art.recovered_matrix(f"{a}.{p}.weight") for p in ("in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b")],
                a))
            ex.load_matrix(l, N.T_LIN_OUT, art.recovered_matrix(f"{a}.out_proj.weight"))
            ex.load_vector(l, N.T_CONV_W, art.float_tensor(f"{a}.conv1d.weight"))
            ex.load_vector(l, N.T_A_LOG, art.float_tensor(f"{a}.A_log"))
            ex.load_vector(l, N.T_DT_BIAS, art.float_tensor(f"{a}.dt_bias"))
            ex.load_vector(l, N.T_LIN_NORM, art.float_tensor(f"{a}.norm.weight"))
        m = f"{prefix}.mlp"
        ex.load_matrix(l, N.T_MLP_GATE_UP, _concat_rows(
            [art.recovered_matrix(f"{m}.{p}.weight") for p in ("gate_proj", "up_proj")], m))
        ex.load_matrix(l, N.T_MLP_DOWN, art.recovered_matrix(f"{m}.down_proj.weight"))
    if c.mtp_num_hidden_layers:
        ex.load_matrix(G, N.T_MTP_FC, art.recovered_matrix("mtp.fc.weight"))
        ex.load_vector(G, N.T_MTP_NORM_E, art.float_tensor("mtp.pre_fc_norm_embedding.weight"))
        ex.load_vector(G, N.T_MTP_NORM_H, art.float_tensor("mtp.pre_fc_norm_hidden.weight"))
        ex.load_vector(G, N.T_MTP_NORM, art.float_tensor("mtp.norm.weight"))
    if c.draft_vocab:
        if draft_token_ids is None or len(draft_token_ids) != c.draft_vocab:
            raise _bad("the executor's draft vocabulary needs its canonical token id table")
        ex.load_vector(G, N.T_DRAFT_IDS, np.asarray(draft_token_ids, dtype=np.uint32))
