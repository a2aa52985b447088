"""The reference's own tests of its roofline gate (models/qwen38_27b/src/roofline.rs:213-281), same
inputs and expectations, against the host-side restatement the benchmark uses for its gate record."""
import pytest

from ctox_llm_b200.roofline import InvalidArtifact, RooflineMeasurement


def measurement(elapsed_seconds, **kw):
    fields = dict(hardware_profile="sm86-test", phase="decode", traffic_source="hardware_counter",
                  elapsed_seconds=elapsed_seconds, accepted_tokens=10, bytes_read=900_000_000,
                  bytes_written=100_000_000, floating_point_operations=100_000_000_000.0,
                  sustainable_bandwidth_bytes_per_second=100_000_000_000.0,
                  sustainable_compute_flops_per_second=100_000_000_000_000.0, dispatch_floor_seconds=0.001,
                  theoretical_bandwidth_bytes_per_second=125_000_000_000.0,
                  theoretical_compute_flops_per_second=125_000_000_000_000.0)
    fields.update(kw)
    return RooflineMeasurement(**fields)


def test_memory_bound_measurement_passes_at_eighty_five_percent():
    report = measurement(0.01 / 0.85).evaluate()
    assert report["dominant_ceiling"] == "memory_bandwidth"
    assert abs(report["practical_efficiency"] - 0.85) < 1e-12
    assert report["optimized_gate_passed"] and not report["accounting_overshoot"]


def test_unexplained_gap_cannot_be_promoted():
    report = measurement(0.02).evaluate()
    assert abs(report["practical_efficiency"] - 0.5) < 1e-12
    assert not report["optimized_gate_passed"]


def test_impossible_result_exposes_incomplete_accounting():
    report = measurement(0.005).evaluate()
    assert report["accounting_overshoot"] and not report["optimized_gate_passed"]


def test_theoretical_ceilings_must_be_a_pair():
    with pytest.raises(InvalidArtifact):
        measurement(0.01, theoretical_compute_flops_per_second=None).evaluate()


def test_malformed_measurements_are_refused():
    for bad in (dict(format="other"), dict(hardware_profile=" "), dict(accepted_tokens=0), dict(bytes_read=0),
                dict(elapsed_seconds=0.0), dict(sustainable_bandwidth_bytes_per_second=float("inf")),
                dict(floating_point_operations=0.0, allow_zero_flops=False), dict(phase="training")):
        with pytest.raises(InvalidArtifact):
            measurement(bad.pop("elapsed_seconds", 0.01), **bad).evaluate()
    report = measurement(0.02, dispatch_floor_seconds=0.015).evaluate()
    assert report["dominant_ceiling"] == "dispatch" and abs(report["practical_efficiency"] - 0.75) < 1e-12
