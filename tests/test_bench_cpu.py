"""bench.py's reference arm runs without a GPU (it times the CPU oracle): the line must parse
and carry the keys the harness around it reads."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    env = dict(os.environ, OMP_NUM_THREADS="1")   # what torchrun exports to its workers
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", *args],
                         capture_output=True, text=True, env=env, timeout=900, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    return json.loads(out.stdout.strip().splitlines()[-1])


def test_reference_arm_op_workload():
    d = _run("--steps", "1", "--warmup", "1")
    assert d["impl"] == "reference" and d["metric"] == "ddf_forward_hbm_gbs" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port"
    # all the cores the process may use, not the launcher's OMP_NUM_THREADS=1
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0


def test_reference_arm_model_workload():
    d = _run("--workload", "model", "--steps", "1", "--warmup", "1")
    assert d["impl"] == "reference" and d["metric"] == "ddf_mul_resnet50_images_per_s" and d["value"] > 0
