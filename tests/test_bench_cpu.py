"""Host-side contract of bench.py: the reference arm always answers with one JSON line and exit code 0 (a result, or an
``unavailable`` line that says why), the clock sampler's summary, and the command line both arms share."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_json_line_and_exits_zero():
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    # without a GPU (or without the built harness) the arm says why; with one it reports the metric
    assert ("unavailable" in d and isinstance(d["unavailable"], str) and d["unavailable"]) or d["value"] > 0


def test_reference_arm_runs_on_local_rank_zero_only():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and r.stdout.strip() == "", (r.stdout, r.stderr[-500:])


def test_clock_sampler_summary_reports_median_and_active_reasons():
    b = _bench_module()
    s = b.ClockSampler(0)
    s.samples = [["1410", "1965", "990.1", "Not Active", "Not Active", "Not Active", "Active"],
                 ["1395", "1965", "985.0", "Not Active", "Not Active", "Not Active", "Active"],
                 ["1965", "1965", "300.0", "Not Active", "Not Active", "Not Active", "Not Active"]]
    out = s.summary()
    assert out == {"sm_mhz": 1410, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"], "samples": 3}
    s.samples = []
    assert s.summary()["sm_mhz"] is None and s.summary()["samples"] == 0


def test_command_line_has_the_driver_flags():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--model", "--batch", "--seq-len", "--matmul-dtype"):
        assert flag in r.stdout, flag
