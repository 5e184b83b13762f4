"""GPU, two or more devices: the expert-parallel layer across real ranks (one process per GPU over NCCL / NVLink peer
memory).  Skipped on a single-GPU box; the same exchange logic runs on the CPU with gloo in tests/test_ep_cpu.py."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4])
def test_peer_and_nccl_exchange_equal_the_single_device_layer(cuda, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this box has {torch.cuda.device_count()}")
    worker = Path(__file__).with_name("ep_rank_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(worker)]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if done.returncode != 0:
        lines = (done.stdout + done.stderr).splitlines()
        first = next((n for n, line in enumerate(lines) if "Traceback" in line), max(0, len(lines) - 40))
        pytest.fail("\n".join(lines[first:first + 40]))
    for rank in range(world):
        assert f"rank {rank}: OK" in done.stdout, done.stdout[-2000:]
