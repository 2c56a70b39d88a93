"""CPU tests of the benchmark's command line: what it answers without a GPU."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def run_bench(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300, env=e, cwd=ROOT)


def test_reference_arm_says_unavailable_for_workloads_the_reference_has_no_cpu_code_for():
    for workload in ("dp_step", "adamw_step"):
        r = run_bench("--impl", "reference", "--workload", workload, "--steps", "2", "--warmup", "1")
        assert r.returncode == 0, r.stderr
        line = json.loads(r.stdout.strip().splitlines()[-1])
        assert line["impl"] == "reference" and workload in line["unavailable"]
    # under a launcher only rank 0 prints
    r = run_bench("--impl", "reference", "--workload", "dp_step", env={"RANK": "1", "WORLD_SIZE": "2"})
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_unknown_workload_is_refused_by_the_parser():
    r = run_bench("--workload", "no_such_workload")
    assert r.returncode == 2 and "invalid choice" in r.stderr
