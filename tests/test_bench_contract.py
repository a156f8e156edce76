"""The benchmark driver's reference arm (the CPU implementation of the path) keeps the one-JSON-line contract."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_contract_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1",
                           "--ctx", "2048"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "decode_attn_kv_stream_bandwidth" and line["unit"] == "GB/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"]
    assert "workload" in line["config"]
    assert line["steps"] == 1 and line["warmup"] == 1


def test_reference_arm_uses_all_cores_under_a_multi_process_launcher_and_shares_the_config():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its ranks; the CPU arm must not be timed on one thread.
    Rank 0 alone prints; the workload description equals the one the GPU arm prints for the same N."""
    import importlib.util
    import os
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="2", LOCAL_RANK="0")
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "0",
           "--ctx", "1024"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads([l for l in proc.stdout.splitlines() if l.startswith("{")][0])
    assert line["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
    assert line["n_gpus"] == 2 and line["steps"] == 2 and line["warmup"] == 0
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert line["config"] == bench.workload_config(1024, 32, 2)
    # the other ranks print nothing and exit 0
    env["RANK"] = "1"
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert proc.returncode == 0 and not [l for l in proc.stdout.splitlines() if l.startswith("{")]
