"""The benchmark script's reference arm (the CPU oracle timed on the host cores) and its line format.  The product arm
needs a GPU and is run by the GPU tiers; here: the JSON line of `--impl reference`, ranks other than 0 leaving without
work, and the product arm refusing to run without a device instead of falling back to anything."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, env=None, timeout=600):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, "bench.py"] + args, cwd=ROOT, env=e, capture_output=True, text=True, timeout=timeout)


def test_reference_arm_prints_one_line_with_the_contract_keys():
    p = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"])
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "decoder_block_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 0 and line["higher_is_better"] is True
    assert line["vs_baseline"] is None and line["data"] == "synthetic" and line["dtype"] == "bf16"
    assert "workload" in line["config"] and "model" not in line["config"]
    assert line["value"] > 0 and abs(line["value"] - line["config"]["sample_tokens"] / (line["ms_per_step"] * 1e-3)) < 1e-6 * line["value"]
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"] and base["unit"] == line["unit"] and base["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_runs_on_rank_zero_only():
    p = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
             env={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29533"}, timeout=120)
    assert p.returncode == 0 and p.stdout.strip() == ""


def test_product_arm_needs_a_device():
    """No CPU path stands in for the kernels: without a GPU the run ends with an error and prints no result line."""
    import torch
    if torch.cuda.is_available():
        return
    p = _run(["--steps", "1", "--warmup", "3"], timeout=300)
    assert p.returncode != 0
    assert not [l for l in p.stdout.splitlines() if l.startswith("{")]
