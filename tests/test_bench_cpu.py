"""bench.py on a machine without a GPU: the reference arm (the reference's CPU path on the host cores)
prints the contract's JSON line; the other ranks of a multi-rank launch stay silent; the library arm
refuses to run without a CUDA device instead of falling back to the CPU."""
import json
import os
import subprocess
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent


def _run(args, **env):
    e = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        e.pop(k, None)
    e.update({k: str(v) for k, v in env.items()})
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, cwd=ROOT, env=e,
                          timeout=600)


def test_reference_arm_prints_one_contract_line():
    r = _run(["--impl", "reference", "--steps", "2", "--warmup", "1"])
    assert r.returncode == 0, r.stderr[-500:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    assert d["metric"] == "RMSNorm fwd+bwd GB/s" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 1 and d["dtype"] == "bf16" and d["data"] == "synthetic"
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["vs_baseline"] is None
    assert "workload" in d["config"] and "model" not in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_do_no_work():
    r = _run(["--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"], RANK=1, WORLD_SIZE=2, LOCAL_RANK=1)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_library_arm_has_no_cpu_fallback():
    if torch.cuda.is_available():
        return   # on a GPU machine the arm simply runs; the GPU tests cover it
    r = _run(["--steps", "1"])
    assert r.returncode != 0 and r.stdout.strip() == ""
    assert "no CPU fallback" in r.stderr
