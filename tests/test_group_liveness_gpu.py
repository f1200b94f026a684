"""Host-side liveness and teardown of a group (`nntrain_gradient_group_poll`,
`_abort`): what a survivor does after the host declared a peer lost.  No GPU is
faulted or hung: the lost rank leaves between steps, with nothing in flight,
and the survivor learns of it on the host."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from nntrain_b200 import reducers

pytestmark = pytest.mark.gpu


def test_poll_and_abort_on_a_group_without_a_communicator(cuda):
    group = reducers.GradientGroup(1, 0, 0)
    assert group.poll() == 0
    group.abort()                 # nothing to abandon: returns at once
    assert group.poll() == 0
    group.close()


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_survivor_polls_aborts_and_destroys_after_a_peer_left(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = os.path.join(os.path.dirname(__file__), "liveness_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    done = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", str(free_port()), worker],
        capture_output=True, text=True, timeout=300, env=env)
    log_dir = os.environ.get("NNTRAIN_TEST_LOG_DIR", "")
    if log_dir and os.path.isdir(log_dir):
        with open(os.path.join(log_dir, "liveness_worker.log"), "w") as log:
            log.write(done.stdout + "\n--- stderr ---\n" + done.stderr)
    assert done.returncode == 0, (done.stdout + done.stderr)[-4000:]
    assert "survivor ok" in done.stdout
