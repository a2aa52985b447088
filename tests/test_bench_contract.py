"""The reference arm of bench.py needs no GPU: its JSON line must carry the contract's keys with the
same metric, unit and workload name as the library's own arm."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    assert line["metric"] == "decode_tokens_per_s_mtp" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1
    assert line["steps"] == 2 and line["warmup"] == 1 and line["value"] > 0 and line["ms_per_step"] > 0
    assert "BASELINE config 4" in line["config"]["workload"]
    cpu = line["cpu_baseline"]
    assert cpu["kind"] in ("port", "reference") and cpu["cores"] >= 1 and cpu["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}


def test_decode_workload_name_is_shared_by_both_arms():
    sys.path.insert(0, ROOT)
    import bench
    name = bench.decode_workload_name(32768, 64, 3)
    assert "context 32768" in name and "64 layers" in name and "MTP k=3" in name
