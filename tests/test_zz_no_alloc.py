"""The allocation-free owner reduce against the regular entry points.

Some hosts cannot allocate device memory where they reduce gradients (a pool
owner that forbids foreign allocations, a step being recorded for replay, a
loop that must stay off the allocator).  For them the library carries its
scratch inside its own image.  This file is collected last on purpose: it
must pass both on its own in a fresh process and after every other test has
used the GPU, and a failure here must not hide any other test's result."""
import ctypes

import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, dev, host
from nntrain_b200 import reducers
from nntrain_b200.library import load
from nntrain_b200.native import CudaBfp8Native, scale_count

pytestmark = pytest.mark.gpu


def encoded_replicas(oracle, world, n, block, seed_shift=0):
    payloads, scales = [], []
    for r in range(world):
        g = oracle.generate_gradient(n, 0xB2000010 + seed_shift, r)
        p = torch.empty(n, dtype=torch.int8, device="cuda")
        s = torch.empty(scale_count(n, block), dtype=torch.float32, device="cuda")
        CudaBfp8Native.block_encode(0, dev(g), p, s, block)
        payloads.append(p)
        scales.append(s)
    return payloads, scales


def run_both(payloads, scales, n, block, scale):
    """(regular outputs, allocation-free outputs), each (payload, scales, sum, flag)."""
    results = []
    for entry in (reducers.reduce_shards_bfp8, reducers.reduce_shards_bfp8_no_alloc):
        out_p = torch.zeros(n, dtype=torch.int8, device="cuda")
        out_s = torch.zeros(scale_count(n, block), dtype=torch.float32, device="cuda")
        sq = torch.zeros(1, dtype=torch.float64, device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        entry(0, payloads, scales, [out_p], [out_s], 0, n, block, scale, sq, flag)
        torch.cuda.synchronize()
        results.append((host(out_p), host(out_s), float(sq.item()), int(flag.item())))
    return results


@pytest.mark.parametrize("block", (32, 128))
def test_two_calls_in_a_row_match_the_regular_entry_point(cuda, oracle, block):
    world = 3
    # first call: one input scale is invalid, so the flag word gets raised in
    # the shared scratch; the ragged length exercises the scalar tail
    n1 = 3 * 65536 + 777
    payloads, scales = encoded_replicas(oracle, world, n1, block)
    scales[1][5] = float("nan")
    regular, static = run_both(payloads, scales, n1, block, 1.0 / world)
    assert regular[3] == 1 and static[3] == 1
    # second call, straight after, on clean data of another length: nothing of
    # the first call may leak through the scratch (flag cleared, stale partial
    # slots beyond this call's span count ignored)
    n2 = 65536 + 4096
    payloads, scales = encoded_replicas(oracle, world, n2, block, seed_shift=1)
    regular, static = run_both(payloads, scales, n2, block, 1.0 / world)
    assert_bits_equal(static[0], regular[0], "payload")
    assert_bits_equal(static[1], regular[1], "scales")
    assert static[3] == regular[3] == 0
    assert static[2] == pytest.approx(regular[2], rel=1e-12)
    # and both equal the oracle's rank-ordered reduce
    gradients = [oracle.generate_gradient(n2, 0xB2000011, r) for r in range(world)]
    expect_payload, expect_scales, _, expect_sq = oracle.allreduce_bfp8(gradients, block, 1.0 / world)
    assert_bits_equal(static[0], expect_payload, "payload vs oracle")
    assert_bits_equal(static[1], expect_scales, "scales vs oracle")
    assert static[2] == pytest.approx(expect_sq, rel=1e-12)


def test_matches_the_single_rank_all_reduce_that_uses_allocated_scratch(cuda, oracle):
    # the regular all-reduce keeps its shard sum of squares and flag in scratch
    # allocated by the group; with one rank it is the same owner arithmetic
    n, block = 2 * 65536 + 512, 32
    payloads, scales = encoded_replicas(oracle, 1, n, block, seed_shift=2)
    expect_p, expect_s = payloads[0].clone(), scales[0].clone()
    group = reducers.GradientGroup(1, 0, 0)
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    table_p = (ctypes.c_void_p * 1)(expect_p.data_ptr())
    table_s = (ctypes.c_void_p * 1)(expect_s.data_ptr())
    assert load().nntrain_gradient_allreduce_bfp8(group.handle, table_p, table_s, n, block, 1.0, sq.data_ptr(),
                                                 flag.data_ptr(), 0, 3, None, None, None,
                                                 torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    sq2 = torch.zeros(1, dtype=torch.float64, device="cuda")
    flag2 = torch.zeros(1, dtype=torch.int32, device="cuda")
    reducers.reduce_shards_bfp8_no_alloc(0, payloads, scales, payloads, scales, 0, n, block, 1.0, sq2, flag2)
    torch.cuda.synchronize()
    assert torch.equal(payloads[0], expect_p) and torch.equal(scales[0], expect_s)
    assert int(flag2.item()) == int(flag.item()) == 0
    assert sq2.item() == pytest.approx(sq.item(), rel=1e-12)
    group.close()


def test_the_sum_of_squares_is_reproducible_and_accumulates(cuda, oracle):
    n, block = 5 * 65536 + 100, 32
    payloads, scales = encoded_replicas(oracle, 2, n, block, seed_shift=3)
    sums = []
    for _ in range(3):
        out_p = torch.zeros(n, dtype=torch.int8, device="cuda")
        out_s = torch.zeros(scale_count(n, block), dtype=torch.float32, device="cuda")
        sq = torch.zeros(1, dtype=torch.float64, device="cuda")
        reducers.reduce_shards_bfp8_no_alloc(0, payloads, scales, [out_p], [out_s], 0, n, block, 0.5, sq, None)
        torch.cuda.synchronize()
        sums.append(sq.item())
    assert sums[0] == sums[1] == sums[2]          # fixed summation order: identical bits
    sq = torch.full((1,), 10.0, dtype=torch.float64, device="cuda")
    reducers.reduce_shards_bfp8_no_alloc(0, payloads, scales, [out_p], [out_s], 0, n, block, 0.5, sq, None)
    torch.cuda.synchronize()
    assert sq.item() == pytest.approx(10.0 + sums[0], rel=1e-14)


def test_ranges_beyond_the_fixed_scratch_are_refused(cuda, lib):
    # 2^30 values is the most the built-in scratch covers; nothing is launched
    dummy = torch.zeros(64, dtype=torch.int8, device="cuda")
    table = (ctypes.c_void_p * 1)(dummy.data_ptr())
    status = lib.nntrain_gradient_reduce_shards_bfp8_no_alloc(
        0, 1, table, table, 1, table, table, 0, (1 << 30) + 65536, 32, 1.0, None, None, None)
    assert status == 1
    from nntrain_b200.library import last_error
    info = last_error()
    assert info.status == 1 and info.operation == 200


def both_entries_on(payloads, scales, first, end, block, scale, outputs=1, offset_bytes=0):
    """Runs both entry points over [first, end) with `outputs` destinations
    each; returns per entry (list of payload arrays, list of scale arrays, sum,
    flag).  offset_bytes shifts every payload pointer off its 16-byte alignment."""
    n = payloads[0].numel()
    results = []
    for entry in (reducers.reduce_shards_bfp8, reducers.reduce_shards_bfp8_no_alloc):
        holders = [torch.zeros(n + 64, dtype=torch.int8, device="cuda") for _ in range(outputs)]
        out_p = [h[offset_bytes:offset_bytes + n] for h in holders]
        out_s = [torch.zeros(scale_count(n, block), dtype=torch.float32, device="cuda") for _ in range(outputs)]
        sq = torch.zeros(1, dtype=torch.float64, device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        entry(0, payloads, scales, out_p, out_s, first, end, block, scale, sq, flag)
        torch.cuda.synchronize()
        results.append(([host(p) for p in out_p], [host(s) for s in out_s], float(sq.item()), int(flag.item())))
    return results


def check_against_oracle(oracle, results, gradients, first, end, block, scale):
    regular, static = results
    expect_payload, expect_scales, _, _ = oracle.allreduce_bfp8(gradients, block, scale)
    sa, sb = first // block, (end + block - 1) // block
    expect_sq = oracle.squared_sum_bfp8(expect_payload[first:end], expect_scales[sa:sb], block)
    for d in range(len(static[0])):
        assert_bits_equal(static[0][d][first:end], regular[0][d][first:end], f"payload, output {d}")
        assert_bits_equal(static[1][d][sa:sb], regular[1][d][sa:sb], f"scales, output {d}")
        assert_bits_equal(static[0][d][first:end], expect_payload[first:end], f"payload vs oracle, output {d}")
        assert_bits_equal(static[1][d][sa:sb], expect_scales[sa:sb], f"scales vs oracle, output {d}")
        # nothing outside the range is written
        assert not static[0][d][:first].any() and not static[0][d][end:].any()
    assert static[3] == regular[3] == 0
    assert static[2] == pytest.approx(regular[2], rel=1e-12)
    assert static[2] == pytest.approx(expect_sq, rel=1e-12)


def test_a_shard_in_the_middle_of_the_arena_with_a_ragged_end(cuda, oracle):
    # what the owner of the last shard passes: a 512-aligned first value and the
    # arena's ragged end (its last block is a partial one)
    world, block, n = 3, 32, 7 * 65536 + 300
    gradients = [oracle.generate_gradient(n, 0xB2000014, r) for r in range(world)]
    payloads, scales = encoded_replicas(oracle, world, n, block, seed_shift=4)
    first, end = 512 * 259, n
    for _ in range(2):        # two calls in a row share the scratch
        results = both_entries_on(payloads, scales, first, end, block, 1.0 / world)
        check_against_oracle(oracle, results, gradients, first, end, block, 1.0 / world)


def test_payload_pointers_off_their_16_byte_alignment(cuda, oracle):
    # pointers offset by 4 bytes force the scalar path of the kernel
    world, block, n = 2, 32, 65536 + 96
    gradients = [oracle.generate_gradient(n, 0xB2000015, r) for r in range(world)]
    aligned_p, scales = encoded_replicas(oracle, world, n, block, seed_shift=5)
    payloads = []
    for p in aligned_p:
        holder = torch.zeros(n + 64, dtype=torch.int8, device="cuda")
        holder[4:4 + n].copy_(p)
        payloads.append(holder[4:4 + n])
        assert payloads[-1].data_ptr() % 16 == 4
    results = both_entries_on(payloads, scales, 0, n, block, 0.5, offset_bytes=4)
    check_against_oracle(oracle, results, gradients, 0, n, block, 0.5)


def test_block_64_with_two_outputs(cuda, oracle):
    world, block, n = 4, 64, 3 * 65536 + 64 * 5
    gradients = [oracle.generate_gradient(n, 0xB2000016, r) for r in range(world)]
    payloads, scales = encoded_replicas(oracle, world, n, block, seed_shift=6)
    results = both_entries_on(payloads, scales, 1024, n, block, 0.25, outputs=2)
    check_against_oracle(oracle, results, gradients, 1024, n, block, 0.25)
