"""The N-rank reducers with all ranks in ONE process (the reference engine's
host model: one worker thread per device, the last arriver enqueues the
cross-device work; NNtrain.Core/Training/CudaBfp8GradientAllReduce.cs:352-363).

Ranks are ordered by events only, so they may share a device: on a one-GPU box
every case runs with all ranks on device 0, which executes exactly the host
flow and kernels of a multi-GPU run minus NVLink; with two or more GPUs the
same cases also run across real devices."""
import threading

import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, host
from nntrain_b200 import reducers

pytestmark = pytest.mark.gpu


def device_lists(world: int):
    lists = [[0] * world]
    if torch.cuda.device_count() >= world and world > 1:
        lists.append(list(range(world)))
    return lists


def to(device: int, array):
    return torch.from_numpy(np.ascontiguousarray(array)).to(f"cuda:{device}")


@pytest.mark.parametrize("world", (2, 3, 4, 8))
@pytest.mark.parametrize("n,block,chunk", ((515, 32, None), (70001, 32, None), ((1 << 20) + 4096, 32, 1 << 18),
                                           (1 << 20, 128, None)))
def test_in_process_all_reduce_matches_the_oracle(cuda, oracle, world, n, block, chunk):
    gradients = [vectors.config0_gradient(oracle, r, n) for r in range(world)]
    scale = 1.0 / world
    payload, scales, final, sq = oracle.allreduce_bfp8(gradients, block, scale)
    norm, c = oracle.clip_coefficient(sq, 1.0)
    want_scales = oracle.scale_bfp8_scales(scales, c)
    for devices in device_lists(world):
        group = reducers.LocalGradientGroup(devices)
        step = reducers.InProcessBfp8AllReduce(group, n, block, chunk_elements=chunk, reduction_scale=scale)
        arenas = [to(d, g) for d, g in zip(devices, gradients)]
        for _ in range(2):                       # buffers and events are reused
            for arena, g in zip(arenas, gradients):
                arena.copy_(torch.from_numpy(g))
            step.enqueue(arenas, max_norm=1.0)
            results = step.complete(max_norm=1.0)
        for rank, state in enumerate(step.ranks):     # replica identity: the same bits on every rank
            assert_bits_equal(host(state.payload), payload, f"payload on rank {rank} ({devices})")
            assert_bits_equal(host(state.scales), want_scales, f"clipped scales on rank {rank}")
            assert_bits_equal(host(arenas[rank]), final, f"fp32 arena on rank {rank}")
            result = results[rank]
            assert result.squared_sum == pytest.approx(sq, rel=1e-12)
            assert abs(result.norm - norm) <= max(1e-5, 2e-6 * norm)
            assert abs(result.coefficient - c) <= 2e-6 * c
            assert result.squared_sum == results[0].squared_sum      # fixed rank order: identical everywhere
        assert step.transport_bytes_per_step == 2 * (world - 1) * (n + 4 * ((n + block - 1) // block)) // world
        step.close()
        group.close()


def test_last_arriving_worker_thread_enqueues_the_collective(cuda, oracle):
    """One thread per rank, as the reference's replica executor runs them; the
    result does not depend on who arrives last."""
    world, n, block = 4, 300137, 32
    gradients = [vectors.config0_gradient(oracle, r, n) for r in range(world)]
    payload, scales, final, sq = oracle.allreduce_bfp8(gradients, block, 0.25)
    for devices in device_lists(world):
        group = reducers.LocalGradientGroup(devices)
        step = reducers.InProcessBfp8AllReduce(group, n, block, chunk_elements=1 << 16, reduction_scale=0.25)
        arenas = [to(d, g) for d, g in zip(devices, gradients)]
        for round_index in range(3):
            for arena, g in zip(arenas, gradients):
                arena.copy_(torch.from_numpy(g))
            torch.cuda.synchronize()
            enqueued = [False] * world
            gate = threading.Barrier(world)

            def worker(rank):
                torch.cuda.set_device(devices[rank])
                gate.wait()
                enqueued[rank] = step.publish(rank, arenas[rank])

            threads = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
            assert sum(enqueued) == 1, "exactly one worker enqueues the cross-device part"
            results = step.complete()
            for rank, state in enumerate(step.ranks):
                assert_bits_equal(host(state.payload), payload, f"payload on rank {rank}, round {round_index}")
                assert_bits_equal(host(state.scales), scales, f"scales on rank {rank}")
                assert_bits_equal(host(arenas[rank]), final, f"fp32 on rank {rank}")
                assert results[rank].squared_sum == pytest.approx(sq, rel=1e-12)
                assert results[rank].coefficient == 1.0
        step.close()
        group.close()


def test_non_finite_gradient_on_one_rank_fails_every_rank(cuda, oracle):
    world, n = 3, 1 << 16
    gradients = [vectors.config0_gradient(oracle, r, n) for r in range(world)]
    gradients[2][5] = np.nan
    group = reducers.LocalGradientGroup([0] * world)
    step = reducers.InProcessBfp8AllReduce(group, n, 32)
    step.enqueue([to(0, g) for g in gradients])
    with pytest.raises(FloatingPointError):
        step.complete()
    flags = [int(state.result.finite_status.item()) for state in step.ranks]
    assert flags == [1] * world
    # the next step starts clean
    gradients[2][5] = 0.0
    step.enqueue([to(0, g) for g in gradients])
    assert all(r.finite for r in step.complete())
    step.close()
    group.close()


@pytest.mark.parametrize("world", (2, 5, 8))
@pytest.mark.parametrize("n,chunk", ((515, None), ((1 << 20) + 1024, None), (1 << 20, 1 << 18)))
def test_in_process_bf16_arena_reducer(cuda, oracle, world, n, chunk):
    inputs = [oracle.bf16_encode(oracle.generate_gradient(n, 0xB2000002 + n, r, sigma_lo=1e-3, sigma_hi=1e-3,
                                                          outlier_fraction=0.0, zero_fraction=0.0, subnormals=0), 1)
              for r in range(world)]
    _, expect_bf16, expect_sq = oracle.bf16_reduce(inputs, 1.0, want_bf16=True, square_of_bf16=True)
    norm, c = oracle.clip_coefficient(expect_sq, 0.05)
    expect = oracle.scale_bf16(expect_bf16, c) if c != 1.0 else expect_bf16
    for devices in device_lists(world):
        group = reducers.LocalGradientGroup(devices)
        step = reducers.InProcessBf16AllReduce(group, n, 1.0, chunk_elements=chunk)
        for _ in range(2):
            for rank in range(world):
                step.values[rank].copy_(torch.from_numpy(inputs[rank].view(np.int16)))
            step.enqueue()
            results = step.complete(max_norm=0.05)
        for rank in range(world):
            assert_bits_equal(host(step.values[rank]).view(np.uint16), expect, f"bf16 arena on rank {rank}")
            assert results[rank].squared_sum == pytest.approx(expect_sq, rel=1e-12)
            assert abs(results[rank].coefficient - c) <= 2e-6 * c
        assert step.transport_bytes_per_step == 2 * (world - 1) * 2 * n // world
        step.close()
        group.close()


def test_two_groups_keep_their_own_launch_shape(cuda, oracle):
    """The launch shape belongs to a group: configuring one reducer must not
    retune another one in the same process."""
    n = 1 << 18
    gradients = [vectors.config0_gradient(oracle, r, n) for r in range(2)]
    payload, scales, _, _ = oracle.allreduce_bfp8(gradients, 32, 0.5)
    first, second = reducers.LocalGradientGroup([0, 0]), reducers.LocalGradientGroup([0, 0])
    first.configure(collective_ctas=3, asynchronous_copies=0)
    second.configure(collective_ctas=2, asynchronous_copies=1, exclusive_sms=True)
    for group in (first, second, first):
        step = reducers.InProcessBfp8AllReduce(group, n, 32, reduction_scale=0.5, write_fp32=False)
        step.enqueue([to(0, g) for g in gradients])
        step.complete()
        for state in step.ranks:
            assert_bits_equal(host(state.payload), payload, "payload")
            assert_bits_equal(host(state.scales), scales, "scales")
        step.close()
    first.close()
    second.close()


@pytest.mark.parametrize("world", (2, 3, 8))
@pytest.mark.parametrize("n,block", ((515, 32), (70001, 32), ((1 << 20) + 4096 + 13, 32), (1 << 18, 128)))
def test_parameter_publication_after_a_sharded_step(cuda, oracle, world, n, block):
    """Rank r owns shard r of the fp32 master parameters; after the fused
    encode + all-gather every rank holds the encoding of the assembled vector."""
    masters = [vectors.config0_gradient(oracle, r, n, seed=0xB2000031) for r in range(world)]
    assembled = np.empty(n, np.float32)
    for rank in range(world):
        first, end = reducers.shard_range(n, world, rank)
        assembled[first:end] = masters[rank][first:end]
    expect_payload, expect_scales = oracle.encode(assembled, block, strict=False)
    for devices in device_lists(world):
        group = reducers.LocalGradientGroup(devices)
        sources = [to(d, m) for d, m in zip(devices, masters)]
        payloads = [torch.zeros(n, dtype=torch.int8, device=f"cuda:{d}") for d in devices]
        scales = [torch.zeros((n + block - 1) // block, dtype=torch.float32, device=f"cuda:{d}") for d in devices]
        flags = [torch.zeros(1, dtype=torch.int32, device=f"cuda:{d}") for d in devices]
        streams = [torch.cuda.Stream(d) for d in devices]
        for _ in range(2):
            group.publish_shards_bfp8([s.data_ptr() for s in sources], [p.data_ptr() for p in payloads],
                                      [s.data_ptr() for s in scales], n, block, [f.data_ptr() for f in flags],
                                      [s.cuda_stream for s in streams])
        for d in set(devices):
            torch.cuda.synchronize(d)
        for rank in range(world):
            assert_bits_equal(host(payloads[rank]), expect_payload, f"payload on rank {rank}")
            assert_bits_equal(host(scales[rank]), expect_scales, f"scales on rank {rank}")
            assert int(flags[rank].item()) == 0
        group.close()
