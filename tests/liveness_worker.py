"""Two ranks; after one completed step rank 1 closes its buffers and leaves,
cleanly, with nothing in flight.  Rank 0 learns of it on the host (a flag in
a file on the node), enqueues nothing more, and must get through poll, abort
and destroy within a host deadline."""
import os
import sys
import tempfile
import time

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from nntrain_b200 import reducers  # noqa: E402
from nntrain_b200.library import load  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    # how the survivor hears of the loss: a file both ranks of this node can see
    notice = os.path.join(tempfile.gettempdir(), f"nntrain_liveness_{os.environ.get('MASTER_PORT', '0')}.left")
    if rank == 0 and os.path.exists(notice):
        os.remove(notice)
    group = reducers.GradientGroup(world, rank, local)
    n = 1 << 18
    step = reducers.Bfp8ArenaAllReduce(group, n, 32, reducers.PEER, reduction_scale=0.5)
    gradients = [oracle.generate_gradient(n, 21, r) for r in range(world)]
    arena = torch.from_numpy(gradients[rank]).cuda()
    step.enqueue(arena, max_norm=1.0)
    step.complete(max_norm=1.0)
    payload, _, _, _ = oracle.allreduce_bfp8(gradients, 32, 0.5)
    assert np.array_equal(step.payload.cpu().numpy(), payload)
    assert group.poll() == 0
    # both ranks unmap each other's buffers together (nothing is in flight)
    step.close()
    dist.barrier()
    if rank == 1:
        # the leaver: gives up its communicator without a collective and exits
        group.abort()
        load().nntrain_gradient_group_destroy(group.handle)
        with open(notice, "w") as f:
            f.write("1")
        dist.destroy_process_group()
        return
    # the survivor: learns of the loss on the host, launches nothing more
    deadline = time.time() + 120.0
    while not os.path.exists(notice):
        assert time.time() < deadline, "the leaving rank never reported"
        time.sleep(0.05)
    os.remove(notice)
    begin = time.time()
    status = group.poll()            # must return at once, whatever it reports
    group.abort()
    assert group.poll() == 0         # no communicator left to ask
    group.close()
    elapsed = time.time() - begin
    assert elapsed < 30.0, f"teardown took {elapsed:.1f} s"
    print(f"survivor ok: poll returned {status}, teardown {elapsed:.2f} s")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
