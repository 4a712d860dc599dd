"""The reference arm of bench.py runs on host cores only: its JSON line can be checked without a GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, lines   # exactly one JSON line on stdout
    return json.loads(lines[0])


def test_reference_arm_prints_one_line_with_the_contract_keys():
    line = _run("--impl", "reference", "--workload", "c1", "--steps", "2", "--warmup", "1")
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "extrapolated", "sample_rows",
                "sample_seconds_per_pass"):
        assert key in line, key
    assert line["impl"] == "reference" and line["higher_is_better"] is True and line["value"] > 0
    assert line["steps"] == 2 and line["warmup"] == 2            # what was really timed (warm-up: at least 3 asked, at most 2 run)
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["config"]["rows"] == 10_000 and line["extrapolated"] is False   # c1 is small enough to be scored whole


def test_reference_arm_caps_its_steps_and_says_so():
    line = _run("--impl", "reference", "--workload", "c1", "--steps", "50", "--warmup", "5")
    assert line["steps"] == 10 and line["warmup"] == 2
    assert line["steps_requested"] == 50 and line["warmup_requested"] == 5


def test_other_ranks_of_a_reference_run_print_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1", "--gpus", "2"],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""
