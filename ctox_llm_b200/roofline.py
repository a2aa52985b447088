"""Roofline gate record of the reference (models/qwen38_27b/src/roofline.rs:8-9,40-142), host side.

``RooflineMeasurement.evaluate()`` restates the reference's accounting: the practical floor is the
largest of (bytes / sustainable bandwidth, flops / sustainable compute, dispatch floor), practical
efficiency = floor / elapsed; a backend counts as optimized at >= 0.85, and an efficiency above
1.05 means the byte or flop accounting is incomplete. ``bench.py`` attaches the report to its lines.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

ROOFLINE_FORMAT = "ctox.qwen38.roofline-measurement.v1"
REPORT_FORMAT = "ctox.qwen38.roofline-report.v1"
MIN_OPTIMIZED_PRACTICAL_EFFICIENCY = 0.85
MAX_ACCOUNTING_OVERSHOOT = 1.05
PHASES = ("prefill", "decode", "batched_decode", "speculative_verify", "kv_attention", "recurrent_state",
          "fused_kernel")
TRAFFIC_SOURCES = ("hardware_counter", "exact_tensor_schedule")


class InvalidArtifact(ValueError):
    """EngineError::InvalidArtifact (error.rs:5-29) for a malformed measurement."""


@dataclass
class RooflineMeasurement:
    hardware_profile: str
    phase: str
    traffic_source: str
    elapsed_seconds: float
    accepted_tokens: float
    bytes_read: int
    bytes_written: int
    floating_point_operations: float
    sustainable_bandwidth_bytes_per_second: float
    sustainable_compute_flops_per_second: float
    dispatch_floor_seconds: float = 0.0
    theoretical_bandwidth_bytes_per_second: Optional[float] = None
    theoretical_compute_flops_per_second: Optional[float] = None
    format: str = ROOFLINE_FORMAT
    # roofline.rs requires a positive flop count; a pure streaming path passes 0 here and the
    # compute floor is then 0 (the record says so in `floating_point_operations`).
    allow_zero_flops: bool = True

    def validate(self) -> None:  # roofline.rs:144-209
        if self.format != ROOFLINE_FORMAT:
            raise InvalidArtifact("unsupported roofline measurement format")
        if not self.hardware_profile.strip():
            raise InvalidArtifact("roofline hardware profile is empty")
        if self.phase not in PHASES or self.traffic_source not in TRAFFIC_SOURCES:
            raise InvalidArtifact("unknown roofline phase or traffic source")
        if self.accepted_tokens <= 0 or self.bytes_read <= 0:
            raise InvalidArtifact("roofline measurement requires accepted tokens and byte traffic")
        for name, value, allow_zero in (
                ("elapsed_seconds", self.elapsed_seconds, False),
                ("floating_point_operations", self.floating_point_operations, self.allow_zero_flops),
                ("sustainable_bandwidth_bytes_per_second", self.sustainable_bandwidth_bytes_per_second, False),
                ("sustainable_compute_flops_per_second", self.sustainable_compute_flops_per_second, False),
                ("dispatch_floor_seconds", self.dispatch_floor_seconds, True)):
            if not math.isfinite(value) or value < 0.0 or (not allow_zero and value == 0.0):
                raise InvalidArtifact(f"roofline {name} is not finite and positive")
        for name, value in (("theoretical_bandwidth_bytes_per_second", self.theoretical_bandwidth_bytes_per_second),
                            ("theoretical_compute_flops_per_second", self.theoretical_compute_flops_per_second)):
            if value is not None and (not math.isfinite(value) or value <= 0.0):
                raise InvalidArtifact(f"roofline {name} is not finite and positive")
        if (self.theoretical_bandwidth_bytes_per_second is None) != (self.theoretical_compute_flops_per_second is None):
            raise InvalidArtifact("roofline theoretical bandwidth and compute ceilings must be paired")

    def evaluate(self) -> dict:  # roofline.rs:82-142
        self.validate()
        total_bytes = self.bytes_read + self.bytes_written
        memory_floor = total_bytes / self.sustainable_bandwidth_bytes_per_second
        compute_floor = self.floating_point_operations / self.sustainable_compute_flops_per_second
        practical_floor = max(memory_floor, compute_floor, self.dispatch_floor_seconds)
        if practical_floor == memory_floor:
            dominant = "memory_bandwidth"
        elif practical_floor == compute_floor:
            dominant = "compute"
        else:
            dominant = "dispatch"
        efficiency = practical_floor / self.elapsed_seconds
        theoretical = None
        if self.theoretical_bandwidth_bytes_per_second is not None:
            floor = max(total_bytes / self.theoretical_bandwidth_bytes_per_second,
                        self.floating_point_operations / self.theoretical_compute_flops_per_second,
                        self.dispatch_floor_seconds)
            theoretical = floor / self.elapsed_seconds
        overshoot = efficiency > MAX_ACCOUNTING_OVERSHOOT
        return {
            "format": REPORT_FORMAT, "hardware_profile": self.hardware_profile, "phase": self.phase,
            "traffic_source": self.traffic_source, "accepted_tokens": self.accepted_tokens,
            "measured_tokens_per_second": self.accepted_tokens / self.elapsed_seconds,
            "practical_roofline_tokens_per_second": self.accepted_tokens / practical_floor,
            "practical_efficiency": efficiency, "theoretical_efficiency": theoretical,
            "operational_intensity_flops_per_byte": self.floating_point_operations / total_bytes,
            "achieved_bandwidth_bytes_per_second": total_bytes / self.elapsed_seconds,
            "achieved_compute_flops_per_second": self.floating_point_operations / self.elapsed_seconds,
            "memory_floor_seconds": memory_floor, "compute_floor_seconds": compute_floor,
            "dispatch_floor_seconds": self.dispatch_floor_seconds, "practical_floor_seconds": practical_floor,
            "dominant_ceiling": dominant, "accounting_overshoot": overshoot,
            "optimized_gate_passed": (not overshoot) and efficiency >= MIN_OPTIMIZED_PRACTICAL_EFFICIENCY,
            "minimum_practical_efficiency": MIN_OPTIMIZED_PRACTICAL_EFFICIENCY,
        }
