"""The configurations that are defined as a split of one problem, run as that split on several
GPUs (``-m gpu``; skipped below two GPUs): every rank takes its slice of the (batch, kv-head
group) units of the seed-0 problem, NCCL gathers the shards' results on rank 0, and the
reassembled tensors equal rank 0's single-GPU run of the whole problem bit for bit."""

import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("config", ["C4", "C5"])
def test_sharded_run_gathers_to_the_single_gpu_result(config):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "bench.py"),
           "--gpus", str(world), "--config", config, "--steps", "3", "--warmup", "3", "--no-e2e", "--no-cpu-baseline"]
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=1500)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["n_gpus"] == world and rec["scaling"] == "strong"
    val = rec["validation"]
    assert val["validated"] is True and val["ranks"] == world and val["status_word"] == 0
    for name, entry in val["tensors"].items():
        assert entry["bitwise_equal_to_single_gpu"] is True and entry["abs_sum"] > 0, name
    assert set(val["tensors"]) == ({"out", "lse"} if config == "C4" else {"out", "lse", "dq", "dk", "dv"})
