"""Tensor parallelism on two GPUs: one process per GPU, the all-reduce after o and down
fused into the GEMV epilogues over peer memory, the argmax winners exchanged the same
way. Needs two B200s; skipped on a one-GPU box."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def free_port() -> int:
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="tensor parallelism needs two GPUs")
def test_two_rank_decode_matches_tensor_parallel_oracle(tmp_path, plan_dir):
    out = tmp_path / "result.json"
    plans = plan_dir / "two-ranks"    # inside the package tree; rank r writes its plan into plans/rank<r>
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
               str(ROOT / "tests" / "tp_worker.py"), "--plan-dir", str(plans), "--out", str(out)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TILEMEGA_WATCHDOG_MS="4000")
    try:
        done = subprocess.run(command, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    finally:
        from tilemega_b200.planbuild import remove_plans
        for rank in range(2):
            remove_plans(plans / f"rank{rank}")
        if plans.is_dir() and not any(plans.iterdir()):
            plans.rmdir()
    assert done.returncode == 0, done.stdout[-4000:] + done.stderr[-4000:]
    assert out.exists()
