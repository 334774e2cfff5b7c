"""CPU suite: the reference arm of bench.py (the CPU restatement timed on the host cores) prints one
JSON line with the contract's keys, also when a launcher has pinned OMP_NUM_THREADS to 1."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", *args], capture_output=True, text=True, env=e, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0])


def test_reference_arm_line_has_the_contract_keys():
    d = run("--workload", "c1", "--steps", "3", "--warmup", "1", env={"OMP_NUM_THREADS": "1"})
    assert d["impl"] == "reference" and d["metric"] == "SpMV GFLOP/s" and d["unit"] == "GFLOP/s" and d["higher_is_better"] is True
    assert d["steps"] == 3 and d["warmup"] == 1 and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] == d["value"]
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))  # not the launcher's single thread
    assert d["e2e"] == {"value": d["value"], "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["config"]["workload"] == "c1" and d["config"]["nnz"] > 60000


def test_other_ranks_of_the_reference_arm_do_nothing():
    e = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1", "--gpus", "2"], capture_output=True, text=True, env=e, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_reference_arm_of_the_sharded_workload_times_one_pass_per_step():
    d = run("--workload", "c5", "--scale", "12", "--steps", "2", "--warmup", "1")
    assert d["impl"] == "reference" and d["config"]["workload"] == "c5" and d["scaling"] == "strong"
    assert d["config"]["rows"] == 4096 and "ONE SpMV pass" in d["cpu_baseline"]["sample"]
    assert d["steps"] == 2 and d["value"] > 0
