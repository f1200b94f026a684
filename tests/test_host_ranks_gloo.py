"""The N > 1 host logic on CPU: world_size-2 (and 4) gloo ranks, no GPU."""
import os
import socket
import subprocess
import sys

import pytest


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", (2, 4))
def test_ranks_agree_on_layout_order_shards_and_failures(lib, world):
    worker = os.path.join(os.path.dirname(__file__), "gloo_worker.py")
    done = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(free_port()), worker],
        capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    assert f"host logic ok on {world} ranks" in done.stdout
