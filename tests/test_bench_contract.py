"""The bench's output contract, as far as it can be checked without a GPU: standard output carries
exactly one JSON line whatever else the process prints, the reference arm answers on a box without
CUDA, and every workload's line is named after its own shape."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a CUDA device is present: the arm would build the 10M index")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "1",
                        "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and "unavailable" in d


def test_other_ranks_of_the_reference_arm_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_result_line_survives_library_banners_on_stdout():
    code = ("import os, sys; sys.path.insert(0, %r); import bench; bench.claim_stdout(); "
            "os.write(1, b'NCCL version 0.0\\n'); print('a library banner'); bench.emit({'value': 1})" % ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    assert r.stdout == '{"value": 1}\n'
    assert "NCCL version 0.0" in r.stderr and "a library banner" in r.stderr


def test_metric_names():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.metric_name("c3", bench.WORKLOADS["c3"]) == bench.METRIC == "QPS @ recall@10>=0.95, 10Mx512 IP"
    assert bench.metric_name("c5", bench.WORKLOADS["c5"]) == bench.METRIC
    assert bench.metric_name("c1", bench.WORKLOADS["c1"]) == "QPS @ recall@10>=0.95, 1Mx200 L2"
    assert "sharded" in bench.metric_name("c4", bench.WORKLOADS["c4"]) and "recall@100" in bench.metric_name("c4", bench.WORKLOADS["c4"])
