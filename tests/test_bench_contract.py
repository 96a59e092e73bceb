"""The benchmark's reference arm runs on the CPU: its one JSON line must carry the keys the driver reads,
with a step time that is the time a step really took (the bounded sample) beside the extrapolated one."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "1", "--scale", "0.0005", "--rows", "8"], capture_output=True, text=True,
                         timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "jl_projected_examples_per_s" and d["unit"] == "examples/s"
    assert d["higher_is_better"] is True and d["steps"] == 2 and d["warmup"] == 1 and d["vs_baseline"] is None
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"] == d["e2e"]["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"] and "model" not in d["config"]
    # the sample: 1 of the 41 column blocks per step; value is computed from the extrapolated time
    assert d["sampled"] == "1/41" and d["ms_per_step"] == d["measured_ms_per_step"]
    assert abs(d["extrapolated_ms_per_step"] - 41 * d["ms_per_step"]) <= 1e-6 * d["extrapolated_ms_per_step"]
    assert abs(d["value"] - 8 / (d["extrapolated_ms_per_step"] * 1e-3)) <= 1e-6 * d["value"]


def test_other_ranks_of_the_reference_arm_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0", "--scale", "0.0005"], capture_output=True, text=True,
                         timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""
