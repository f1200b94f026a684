"""One CPU rank of the host-logic run (launched by test_host_ranks_gloo.py).
No GPU: the ranks exercise everything of the N-rank path that is host logic -
identical bucket layout, a cross-rank agreed enqueue order although leaves
arrive in different orders, disjoint covering shards, the id / handle exchange
plumbing over the process group, and a host-side failure (a rank whose step is
non-finite) that every rank must learn of before it completes."""
import os
import random
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from nntrain_b200 import reducers  # noqa: E402
from nntrain_b200.host_plan import GradientStepPlan, InvalidOperationError  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    failures = []
    layer = [512 * 1536, 1536, 512 * 512, 512, 512, 512, 512 * 2048, 2048, 2048 * 512, 512, 512, 512]
    numels = [32000 * 512] + layer * 8 + [512, 512]
    plan = GradientStepPlan(numels, devices=list(range(world)))

    # every rank derives the same layout from the same tensor list
    layouts = [None] * world
    dist.all_gather_object(layouts, (plan.bucket_element_counts, [plan.locate(t) for t in range(len(numels))]))
    if any(l != layouts[0] for l in layouts):
        failures.append("bucket layouts differ between ranks")

    # leaves become ready in a different order on every rank; the enqueue
    # order must still be identical (collectives are matched by order)
    for _ in range(3):
        step = plan.begin_step()
        plan.begin_device_step(step)
        order = list(range(len(numels)))
        random.Random(1000 * rank + step).shuffle(order)
        enqueued = []
        for tensor in order:
            plan.notify_gradient_ready(tensor, step)
            while (bucket := plan.next_enqueueable(step)) >= 0:
                enqueued.append(bucket)
        sequences = [None] * world
        dist.all_gather_object(sequences, enqueued)
        if any(s != sequences[0] for s in sequences) or sorted(enqueued) != list(range(plan.bucket_count)):
            failures.append(f"enqueue order differs between ranks in step {step}: {sequences}")
        # the finite flag is job-wide: rank world-1 saw a NaN in step 2
        flag = torch.tensor([1.0 if (step == 2 and rank == world - 1) else 0.0])
        dist.all_reduce(flag)
        try:
            plan.complete(step, non_finite=bool(flag.item()))
            if step == 2:
                failures.append("a non-finite step completed")
        except InvalidOperationError:
            if step != 2:
                failures.append(f"step {step} failed to complete")
            plan.abort(step)
    if plan.completed_steps != 2:
        failures.append(f"completed steps {plan.completed_steps}")
    plan.optimizer_validate_and_consume()

    # shards: contiguous, 512-aligned, disjoint, covering, identical on every rank
    for length in (1, 515, 70001, 41_604_096, 1_543_714_304):
        mine = reducers.shard_range(length, world, rank)
        shards = [None] * world
        dist.all_gather_object(shards, mine)
        cursor = 0
        for first, end in shards:
            if end > first and (first != cursor or first % 512):
                failures.append(f"shards of {length} do not tile: {shards}")
            cursor = max(cursor, end)
        if cursor != length:
            failures.append(f"shards of {length} do not cover it: {shards}")

    # the 128-byte id travels from rank 0 to everyone (as GradientGroup does it)
    holder = [bytes(range(128)) if rank == 0 else None]
    dist.broadcast_object_list(holder, src=0)
    if holder[0] != bytes(range(128)):
        failures.append("id broadcast")
    # and the 64-byte memory handles are all-gathered (as PeerBuffer does it)
    handles = [None] * world
    dist.all_gather_object(handles, bytes([rank]) * 64)
    if [h[0] for h in handles] != list(range(world)):
        failures.append("handle all-gather")

    gathered = [None] * world
    dist.all_gather_object(gathered, failures)
    dist.destroy_process_group()
    if any(gathered):
        print("FAILURES:", gathered)
        sys.exit(1)
    if rank == 0:
        print(f"host logic ok on {world} ranks")


if __name__ == "__main__":
    main()
