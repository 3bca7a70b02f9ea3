"""The CPU-only parts of bench.py: the reference arm's JSON line and the argument rules."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def _run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, env=e, timeout=600)


def test_reference_arm_prints_one_contract_line():
    r = _run("--impl", "reference", "--steps", "3", "--warmup", "3")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "pooled_lookups_per_sec" and d["unit"] == "lookups/s"
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] == 3 and d["higher_is_better"] is True
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["vs_baseline"] is None and d["data"] == "synthetic"
    assert d["config"]["workload"].startswith("c2:") and "model" not in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "lookups/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}


def test_other_ranks_of_the_reference_arm_do_no_work():
    r = _run("--impl", "reference", "--gpus", "2", "--steps", "3", "--warmup", "3",
             env={"WORLD_SIZE": "2", "RANK": "1", "LOCAL_RANK": "1"})
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_argument_rules():
    r = _run("--workload", "c2", "--exchange", "stage")
    assert r.returncode != 0 and "row-sharded" in (r.stderr + r.stdout)
    r = _run("--gpus", "2")                       # more than one GPU needs the launcher
    assert r.returncode != 0 and "torch.distributed.run" in (r.stderr + r.stdout)
