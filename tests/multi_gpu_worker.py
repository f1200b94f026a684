"""One rank of the multi-GPU parity run (launched by test_multi_gpu.py with
torch.distributed.run).  Every rank regenerates all ranks' gradients from the
seed, computes the oracle's all-reduce on the CPU and compares its own
device's result bit for bit."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from nntrain_b200 import reducers  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    group = reducers.GradientGroup(world, rank, local)
    failures = []
    cases = [(515, 32, None), (70001, 32, None), ((1 << 20) + 4096, 32, 1 << 18), (1 << 20, 128, None)]
    for mode in (reducers.PEER, reducers.COPY_ENGINE, reducers.NCCL):
        for n, block, chunk in cases:
            gradients = [oracle.generate_gradient(n, 0xB2000000 + n, r) for r in range(world)]
            scale = 1.0 / world
            step = reducers.Bfp8ArenaAllReduce(group, n, block, mode, chunk_elements=chunk,
                                               reduction_scale=scale)
            arena = torch.from_numpy(gradients[rank]).cuda()
            for _ in range(2):          # two steps in a row: buffers are reused
                arena.copy_(torch.from_numpy(gradients[rank]))
                step.enqueue(arena, max_norm=1.0)
                result = step.complete(max_norm=1.0)
            payload, scales, final, sq = oracle.allreduce_bfp8(gradients, block, scale)
            norm, c = oracle.clip_coefficient(sq, 1.0)
            tag = f"mode={mode} n={n} block={block} chunk={chunk}"
            if not np.array_equal(step.payload.cpu().numpy(), payload):
                failures.append(f"{tag}: payload differs")
            got_scales = step.scales.cpu().numpy()
            want_scales = oracle.scale_bfp8_scales(scales, result.coefficient)
            if not np.array_equal(got_scales.view(np.uint32), want_scales.view(np.uint32)):
                failures.append(f"{tag}: scales differ")
            if not np.array_equal(arena.cpu().numpy().view(np.uint32), final.view(np.uint32)):
                failures.append(f"{tag}: fp32 arena differs from decode(encode(sum))")
            if abs(result.squared_sum - sq) > 1e-9 * sq:
                failures.append(f"{tag}: squared sum {result.squared_sum} vs {sq}")
            if abs(result.norm - norm) > max(1e-5, 2e-6 * norm) or abs(result.coefficient - c) > 2e-6 * c:
                failures.append(f"{tag}: norm/coefficient {result.norm}/{result.coefficient} vs {norm}/{c}")
            expected_bytes = 2 * (world - 1) * (n + 4 * ((n + block - 1) // block)) // world
            if step.transport_bytes_per_step != expected_bytes:
                failures.append(f"{tag}: transport bytes")
            step.close()
    # bf16 arena reducer: fp32 accumulate in rank order, bf16 result, clip
    for mode in (reducers.PEER, reducers.NCCL):
        for n, chunk in ((515, None), ((1 << 20) + 1024, None), (1 << 20, 1 << 18)):
            inputs = [oracle.bf16_encode(oracle.generate_gradient(n, 0xB2000002 + n, r, sigma_lo=1e-3, sigma_hi=1e-3,
                                                                  outlier_fraction=0.0, zero_fraction=0.0,
                                                                  subnormals=0), 1) for r in range(world)]
            step = reducers.Bf16ArenaAllReduce(group, n, mode, reduction_scale=1.0, chunk_elements=chunk)
            for _ in range(2):
                step.values.copy_(torch.from_numpy(inputs[rank].view(np.int16)))
                step.enqueue()
                result = step.complete(max_norm=0.05)
            _, expect_bf16, expect_sq = oracle.bf16_reduce(inputs, 1.0, want_bf16=True, square_of_bf16=True)
            norm, c = oracle.clip_coefficient(expect_sq, 0.05)
            expect = oracle.scale_bf16(expect_bf16, c) if c != 1.0 else expect_bf16
            tag = f"bf16 mode={mode} n={n} chunk={chunk}"
            if not np.array_equal(step.values.cpu().numpy().view(np.uint16), expect):
                failures.append(f"{tag}: arena differs")
            if abs(result.squared_sum - expect_sq) > 1e-9 * expect_sq or abs(result.coefficient - c) > 2e-6 * c:
                failures.append(f"{tag}: sum of squares / coefficient")
            if step.transport_bytes_per_step != 2 * (world - 1) * 2 * n // world:
                failures.append(f"{tag}: transport bytes")
            step.close()
    # a NaN on one rank fails the step on every rank
    n = 1 << 16
    g = oracle.generate_gradient(n, 7, rank)
    if rank == world - 1:
        g[5] = np.nan
    step = reducers.Bfp8ArenaAllReduce(group, n, 32, reducers.PEER)
    step.enqueue(torch.from_numpy(g).cuda())
    try:
        step.complete()
        failures.append("non-finite gradient on one rank did not fail the step here")
    except FloatingPointError:
        pass
    step.close()
    gathered = [None] * world
    dist.all_gather_object(gathered, failures)
    group.close()
    dist.destroy_process_group()
    if any(gathered):
        if rank == 0:
            print("FAILURES:", gathered)
        sys.exit(1)
    if rank == 0:
        print(f"multi-gpu parity ok on {world} ranks")


if __name__ == "__main__":
    main()
