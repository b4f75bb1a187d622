"""Tensor-parallel kernels and engine on 2, 4 and 8 GPUs (each case is skipped when the machine has fewer)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_worker(world: int, nvls: str, port: int):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, TAH_B200_NVLS=nvls, NCCL_NVLS_ENABLE=nvls)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    sys.stdout.write(res.stdout[-6000:])
    sys.stderr.write(res.stderr[-4000:])
    assert res.returncode == 0 and "TP_WORKER_PASS" in res.stdout


@pytest.mark.parametrize("nvls", ["1", "0"])
def test_tp_two_ranks(nvls):
    _run_worker(2, nvls, 29617)


@pytest.mark.parametrize("world", [4, 8])
def test_tp_wider_groups(world):
    _run_worker(world, "1", 29617 + world)
