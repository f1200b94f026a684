"""The bucketed, notification-driven BFP8 reducer (the host flow of
NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:449-537,912-1029 over
buckets laid out as in :1572-1601,1647-1678) against the oracle, with all
ranks in one process.  On a one-GPU box the ranks share device 0; with more
GPUs the same cases also run across real devices."""
import numpy as np
import pytest
import torch

from gpu_helpers import assert_bits_equal, host
from nntrain_b200 import bucketed, reducers
from nntrain_b200.host_plan import InvalidOperationError

pytestmark = pytest.mark.gpu


def device_lists(world: int):
    lists = [[0] * world]
    if torch.cuda.device_count() >= world and world > 1:
        lists.append(list(range(world)))
    return lists


def fill(reducer, oracle, numels, seed):
    """Per-tensor seeded gradients written through the arena views; returns
    the per-rank flat copies."""
    world = len(reducer.ranks)
    total = sum(numels)
    flats = [oracle.generate_gradient(total, seed, r) for r in range(world)]
    offsets = np.concatenate([[0], np.cumsum(numels)])
    for rank in range(world):
        for tensor in range(len(numels)):
            view = reducer.gradient_view(rank, tensor)
            view.copy_(torch.from_numpy(flats[rank][offsets[tensor]:offsets[tensor + 1]]))
    return flats, offsets


def expected_buckets(reducer, oracle, numels, flats, offsets, block, scale):
    world = len(flats)
    out, squared = [], 0.0
    for bucket in range(reducer.bucket_count):
        tensors = [t for t in range(len(numels)) if reducer.ranks[0].location[t][0] == bucket]
        inputs = [np.concatenate([flats[r][offsets[t]:offsets[t + 1]] for t in tensors]) for r in range(world)]
        payload, scales, fp32, sq = oracle.allreduce_bfp8(inputs, block, scale)
        squared += sq
        out.append((payload, scales, fp32))
    return out, squared


def run_step(reducer, numels, order=None, max_norm=1.0):
    world = len(reducer.ranks)
    reducer.begin_step()
    for rank in range(world):
        reducer.begin_device_step(rank)
    completed = []
    for tensor in (order if order is not None else reversed(range(len(numels)))):
        for rank in range(world):
            completed.append(reducer.notify_gradient_ready(rank, tensor))
    return reducer.complete(max_norm), completed


@pytest.mark.parametrize("world", (2, 4))
def test_small_list_with_unaligned_tensors(cuda, oracle, world):
    # odd sizes: tensors start at arbitrary element offsets, 32-value blocks straddle tensors
    numels = [4099, 33, 1, 20000, 517, 16384, 7, 9001, 12345, 31, 65, 40000]
    for devices in device_lists(world):
        group = reducers.LocalGradientGroup(devices)
        reducer = bucketed.BucketedBfp8Reducer(group, numels, 32, 1 << 14, 1.0 / world)
        assert sum(reducer.bucket_elements) == sum(numels) and reducer.bucket_count > 3
        for step in range(2):
            flats, offsets = fill(reducer, oracle, numels, 0xB2000001 + step)
            results, _ = run_step(reducer, numels)
            expect, squared = expected_buckets(reducer, oracle, numels, flats, offsets, 32, 1.0 / world)
            norm, c = oracle.clip_coefficient(squared, 1.0)
            for bucket, (payload, scales, fp32) in enumerate(expect):
                want = oracle.scale_bfp8_scales(scales, c)
                for rank in range(world):
                    arena, got_payload, got_scales = reducer.bucket_views(rank, bucket)
                    assert_bits_equal(host(got_payload), payload, f"payload, bucket {bucket}, rank {rank}")
                    assert_bits_equal(host(got_scales), want, f"clipped scales, bucket {bucket}, rank {rank}")
                    assert_bits_equal(host(arena), fp32, f"fp32 arena, bucket {bucket}, rank {rank}")
            for result in results:
                assert result.squared_sum == pytest.approx(squared, rel=1e-12)
                assert abs(result.norm - norm) <= max(1e-5, 2e-6 * norm)
                assert abs(result.coefficient - c) <= 2e-6 * c
            assert all(s.plan.completed_steps == step + 1 for s in reducer.ranks)
        reducer.close()
        group.close()


def test_small_transformer_list_two_ranks(cuda, oracle):
    """Benchmark configuration 1 (a small decoder Transformer): 41,604,096 values, nine buckets of at most
    4 Mi values (the embedding alone is oversize), two replicas, clip 1.0."""
    numels = bucketed.small_transformer_numels()
    assert sum(numels) == 41_604_096
    for devices in device_lists(2):
        group = reducers.LocalGradientGroup(devices)
        reducer = bucketed.BucketedBfp8Reducer(group, numels, 32, 4 << 20, 0.5)
        assert reducer.bucket_elements == [16_384_000, 3_940_352, 3_416_064] + [3_152_384] * 5 + [2_101_760]
        flats, offsets = fill(reducer, oracle, numels, 0xB2000001)
        results, completed = run_step(reducer, numels)
        assert sorted(b for b in completed if b >= 0) == sorted(list(range(9)) * 2)
        expect, squared = expected_buckets(reducer, oracle, numels, flats, offsets, 32, 0.5)
        norm, c = oracle.clip_coefficient(squared, 1.0)
        for bucket, (payload, scales, fp32) in enumerate(expect):
            want = oracle.scale_bfp8_scales(scales, c)
            for rank in range(2):
                arena, got_payload, got_scales = reducer.bucket_views(rank, bucket)
                assert_bits_equal(host(got_payload), payload, f"payload, bucket {bucket}, rank {rank}")
                assert_bits_equal(host(got_scales), want, f"clipped scales, bucket {bucket}, rank {rank}")
                assert_bits_equal(host(arena), fp32, f"fp32 arena, bucket {bucket}, rank {rank}")
        assert results[0].squared_sum == pytest.approx(squared, rel=1e-12)
        assert abs(results[0].coefficient - c) <= 2e-6 * c
        assert reducer.transport_bytes_per_step == sum(e + 4 * ((e + 31) // 32) for e in reducer.bucket_elements)
        reducer.close()
        group.close()


def test_duplicate_notification_abort_and_recovery(cuda, oracle):
    """A tensor notified twice fails the step closed; abort, and the next step
    is clean (NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:59-93)."""
    numels = [5000, 3000, 9000, 100]
    group = reducers.LocalGradientGroup([0, 0])
    reducer = bucketed.BucketedBfp8Reducer(group, numels, 32, 1 << 13, 0.5)
    flats, offsets = fill(reducer, oracle, numels, 11)
    reducer.begin_step()
    for rank in range(2):
        reducer.begin_device_step(rank)
    reducer.notify_gradient_ready(0, 3)
    with pytest.raises(InvalidOperationError):
        reducer.notify_gradient_ready(0, 3)
    with pytest.raises(InvalidOperationError):
        reducer.complete(1.0)                       # buckets are missing
    reducer.abort()
    assert all(s.plan.completed_steps == 0 for s in reducer.ranks)
    with pytest.raises(InvalidOperationError):
        reducer.notify_gradient_ready(0, 2)         # no step is active
    flats, offsets = fill(reducer, oracle, numels, 12)
    results, _ = run_step(reducer, numels, order=[1, 0, 3, 2])     # any notification order
    expect, squared = expected_buckets(reducer, oracle, numels, flats, offsets, 32, 0.5)
    _, c = oracle.clip_coefficient(squared, 1.0)
    for bucket, (payload, scales, fp32) in enumerate(expect):
        for rank in range(2):
            arena, got_payload, got_scales = reducer.bucket_views(rank, bucket)
            assert_bits_equal(host(got_payload), payload, "payload after recovery")
            assert_bits_equal(host(got_scales), oracle.scale_bfp8_scales(scales, c), "scales after recovery")
            assert_bits_equal(host(arena), fp32, "fp32 after recovery")
    assert all(s.plan.completed_steps == 1 for s in reducer.ranks)
    # a NaN gradient: the step fails on complete and nothing becomes Reduced
    fill(reducer, oracle, numels, 13)
    reducer.gradient_view(1, 2)[17] = float("nan")
    with pytest.raises(InvalidOperationError):
        run_step(reducer, numels)
    reducer.abort()
    assert all(s.plan.completed_steps == 1 for s in reducer.ranks)
    reducer.close()
    group.close()
