"""The reference arm of bench.py runs on the host cores: it must print exactly one JSON line with the agreed keys."""
from __future__ import annotations

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "1", "--m", "64", "--k", "256", "--n", "64"], capture_output=True, text=True,
                         timeout=300, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["value"] > 0 and line["unit"] == "TOPS"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"]
    assert line["steps"] == 2 and line["warmup"] == 1  # --steps / --warmup are honoured
    # both arms of one command line carry the same `config` object
    sys.path.insert(0, ROOT)
    import argparse
    import bench
    args = argparse.Namespace(workload="linear", m=64, k=256, n=64, block=128, exchange="push")
    assert line["config"] == bench.workload_config(args, 1)


def test_other_ranks_of_the_reference_arm_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0", "--m", "64", "--k", "256", "--n", "64"],
                         capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_operand_set_counts_keep_launches_cold_and_graphs_small():
    """sets_for(): enough operand sets that consecutive launches cannot find their inputs in L2 (2.5 x L2 in total), two
    for a set that is larger than L2 by itself, never more than 256 launches per graph or 6 GB of copies."""
    sys.path.insert(0, ROOT)
    import bench
    l2 = bench.L2_BYTES
    assert bench.sets_for(2 * l2) == 2
    n = bench.sets_for(29.4e6)                      # the headline GEMM's operands
    assert n * 29.4e6 >= 2.5 * l2 and n <= 16
    assert bench.sets_for(10e3) == 256              # tiny sets: capped (they stay L2-resident, and say so)
    assert bench.sets_for(1.5e9) * 1.5e9 <= 6e9 + 1.5e9
