"""Multi-GPU parity: one process per GPU, both transports, against the
oracle.  Runs when the box has at least two GPUs."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", (2, 4, 8))
def test_all_reduce_across_processes(cuda, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this box has {torch.cuda.device_count()}")
    worker = os.path.join(os.path.dirname(__file__), "multi_gpu_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    done = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(free_port()), worker],
        capture_output=True, text=True, timeout=600, env=env)
    # keep the ranks' output when a log directory is given
    log_dir = os.environ.get("NNTRAIN_TEST_LOG_DIR", "")
    if log_dir and os.path.isdir(log_dir):
        with open(os.path.join(log_dir, f"multi_gpu_worker_{world}.log"), "w") as log:
            log.write(done.stdout + "\n--- stderr ---\n" + done.stderr)
    relevant = "\n".join(line for line in (done.stdout + done.stderr).splitlines()
                         if "OMP_NUM_THREADS" not in line and not line.startswith("*****"))
    assert done.returncode == 0, relevant[-6000:]
    assert "multi-gpu parity ok" in done.stdout
