"""The reference arm of bench.py (`--impl reference`) needs no GPU: it times the CPU oracle port
on the host cores. This test runs it on a tiny configuration and checks the one JSON line it has
to print: the keys of the measurement contract, the metric and unit of the headline line, and
that nothing on that path loads the CUDA library or counts a kernel launch."""

import json
import os
import socket
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent


def run_reference_arm(*extra):
    command = [sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1",
               "--layers", "1", "--context", "128", "--cpu-sample-batch", "2", *extra]
    done = subprocess.run(command, cwd=REPO, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1, done.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_prints_the_contract_line():
    line = run_reference_arm()
    assert line["impl"] == "reference"
    assert line["metric"] == "qwen2_0.5b_bf16_decode_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["scaling"] == "weak" and line["vs_baseline"] is None
    assert line["n_gpus"] == 1 and line["steps"] == 2 and line["warmup"] == 1
    assert line["dtype"] == "bf16" and line["data"] == "synthetic"
    assert "workload" in line["config"] and "model" not in line["config"]
    assert line["value"] > 0 and line["ms_per_step"] > 0
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["cores"] >= 1 and baseline["value"] == line["value"]
    assert "2 of the 64 sequences" in baseline["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_reference_arm_value_is_sample_tokens_over_step_time():
    line = run_reference_arm()
    # 2 sequences per step of ms_per_step milliseconds
    assert abs(line["value"] - 2 / (line["ms_per_step"] * 1e-3)) <= 1e-6 * line["value"]


def test_reference_arm_under_a_two_rank_launch_prints_one_line_from_rank_0():
    """Launched the way the multi-GPU arm is (torch.distributed.run, one process per rank), rank 0
    alone measures, with all host cores although the launcher sets OMP_NUM_THREADS=1; the other
    rank leaves with exit code 0 and prints nothing."""
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
               "--master-addr", "127.0.0.1", "--master-port", str(port), str(REPO / "bench.py"),
               "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1", "--layers", "1",
               "--context", "128", "--cpu-sample-batch", "2"]
    done = subprocess.run(command, cwd=REPO, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1, done.stdout[-2000:]
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["gpu_launches"] == 0
    assert line["config"]["global_batch"] == 128
    assert line["cpu_baseline"]["cores"] > 1 or (os.cpu_count() or 1) == 1  # not the launcher's one thread
