"""Host-side behaviour of bench.py that needs no GPU."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, env_extra, timeout=120):
    env = dict(os.environ)
    env.update(env_extra)
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, cwd=ROOT, env=env, capture_output=True,
                          text=True, timeout=timeout)


def test_reference_arm_runs_on_rank_zero_only():
    """Under a multi-rank launch only rank 0 times the CPU path; the other ranks leave at once
    with exit code 0 and print nothing."""
    r = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"], {"RANK": "1", "WORLD_SIZE": "2"})
    assert r.returncode == 0
    assert r.stdout.strip() == ""


def test_product_arm_refuses_to_run_without_a_gpu():
    """No CPU fallback: without a CUDA device the product arm stops with a message."""
    import torch

    if torch.cuda.is_available():
        return
    r = _run(["--steps", "1", "--warmup", "0"], {})
    assert r.returncode != 0
    assert "CUDA" in (r.stderr + r.stdout)
