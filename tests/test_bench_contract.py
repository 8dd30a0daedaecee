"""The benchmark script's command-line contract, as far as it can run without a GPU: the reference arm
(`bench.py --impl reference`) times the CPU restatement of the reference's loop nest and prints one JSON line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "1"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["unit"] == "TFLOP/s" and line["higher_is_better"] is True and line["value"] > 0
    assert line["metric"].startswith("TFLOP/s batched GEMM bf16")
    assert "workload" in line["config"] and "model" not in line["config"]
    base = line["cpu_baseline"]
    assert base["kind"] in ("port", "reference") and base["cores"] >= 1 and base["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["vs_baseline"] is None


def test_without_a_gpu_the_product_arm_fails_loudly():
    import torch
    if torch.cuda.is_available():
        return  # covered by the GPU runs themselves
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "1"], cwd=ROOT,
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0   # no CPU fallback
    assert not [l for l in proc.stdout.splitlines() if l.startswith("{") and '"value"' in l]
