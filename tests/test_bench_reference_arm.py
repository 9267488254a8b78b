"""The benchmark's CPU arm (`bench.py --impl reference`) on a one-layer case: exactly one line
on stdout, valid JSON, with the keys and meanings the measurement contract gives that arm —
the metric, unit and direction of the CUDA arm, a `cpu_baseline` describing this very run and
an `e2e` that repeats the value with no host-device bytes.  Needs no GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "1", "--layers", "1"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, lines
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    assert line["metric"] == "decode_matmul_tok_per_s" and line["unit"] == "tok/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert abs(line["value"] * line["ms_per_step"] / 1e3 - 1.0) < 1e-6  # batch 1: tokens per second = 1 / step time
    assert line["data"] == "synthetic" and "workload" in line["config"]
    base = line["cpu_baseline"]
    assert base["kind"] in ("port", "reference") and base["cores"] >= 1 and base["sample"]
    assert base["value"] == line["value"] and base["unit"] == line["unit"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_reference_arm_on_another_rank_does_no_work_and_prints_nothing():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29533")
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                           "--warmup", "1", "--layers", "1"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=120)
    assert done.returncode == 0, done.stderr[-2000:]
    assert done.stdout.strip() == ""
