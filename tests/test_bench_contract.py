"""The bench's reference arm runs on host cores only, so its output contract is checked here:
one JSON line with the keys the bench contract names, rank 0 alone working under N > 1."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(env_extra=None, *args):
    env = dict(os.environ)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "C2",
                           "--steps", "1", "--warmup", "0", *args],
                          capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)


def test_reference_arm_prints_one_contract_line():
    proc = _run()
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in rec, key
    assert rec["unit"] == "TFLOP/s" and rec["higher_is_better"] is True and rec["vs_baseline"] is None
    assert rec["value"] > 0 and rec["cpu_baseline"]["value"] == rec["value"]
    assert rec["cpu_baseline"]["kind"] in ("port", "reference") and rec["cpu_baseline"]["cores"] >= 1
    assert rec["e2e"] == {"value": rec["value"], "unit": rec["unit"], "h2d_bytes_per_step": 0,
                          "d2h_bytes_per_step": 0}
    assert "workload" in rec["config"]
    # the metric names the configuration's own dtype and mask
    assert rec["metric"] == "flash-attn fwd+bwd TFLOP/s (bf16, causal)"


def test_metric_label_follows_the_configuration():
    sys.path.insert(0, ROOT)
    import bench
    from oracle import sdpa_oracle as O

    assert bench.metric_name(O.CONFIGS["C1"]) == "flash-attn fwd TFLOP/s (fp32, causal)"
    assert bench.metric_name(O.CONFIGS["C3"]) == "flash-attn fwd+bwd TFLOP/s (bf16, causal)"
    assert bench.metric_name(O.CONFIGS["C4"]) == "flash-attn fwd TFLOP/s (bf16, causal)"
    assert bench.metric_name(O.CONFIGS["C5"]) == "flash-attn fwd+bwd TFLOP/s (fp16, non-causal)"


def test_reference_arm_other_ranks_exit_without_work():
    proc = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}, "--gpus", "2")
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert not [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
