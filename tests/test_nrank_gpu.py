"""The N-rank owner kernels and the single-rank step on one GPU.  Ranks are
emulated as N arenas on the same device: the kernel only sees pointer tables,
so this exercises exactly the code a multi-GPU run executes, minus NVLink."""
import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, bf16_dev, bf16_host, dev, host
from nntrain_b200 import reducers
from nntrain_b200.native import CudaBfp8Native, scale_count

pytestmark = pytest.mark.gpu


def encode_on_device(gradients, block):
    payloads, scales = [], []
    for g in gradients:
        n = g.size
        p = torch.empty(n, dtype=torch.int8, device="cuda")
        s = torch.empty(scale_count(n, block), dtype=torch.float32, device="cuda")
        CudaBfp8Native.block_encode(0, dev(g), p, s, block)
        payloads.append(p)
        scales.append(s)
    return payloads, scales


@pytest.mark.parametrize("world", (1, 2, 3, 4, 8))
@pytest.mark.parametrize("block", (32, 128))
@pytest.mark.parametrize("n", (1, 515, 70001, 1 << 20))
def test_emulated_ranks_match_rank_ordered_oracle(cuda, oracle, world, block, n):
    gradients = [vectors.config0_gradient(oracle, r, n) for r in range(world)]
    scale = 1.0 / world
    payloads, scales = encode_on_device(gradients, block)
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    covered = 0
    for rank in range(world):
        first, end = reducers.shard_range(n, world, rank)
        assert first <= end <= n and (end == first or first % 512 == 0)
        covered += end - first
        if end > first:
            # in place: every "rank's" arena receives the owner's shard
            reducers.reduce_shards_bfp8(0, payloads, scales, payloads, scales, first, end, block, scale, sq, flag)
    assert covered == n
    torch.cuda.synchronize()
    expect_payload, expect_scales, _, expect_sq = oracle.allreduce_bfp8(gradients, block, scale)
    for rank in range(world):     # replica identity: bit-identical on every rank
        assert_bits_equal(host(payloads[rank]), expect_payload, f"payload on rank {rank}")
        assert_bits_equal(host(scales[rank]), expect_scales, f"scales on rank {rank}")
    assert int(flag.item()) == 0
    assert sq.item() == pytest.approx(expect_sq, rel=1e-12)


def test_two_rank_sum_is_the_reference_tests_formula(cuda, oracle):
    # Encode(Decode(Encode a) + Decode(Encode b)), n in {1, 257, 515}
    # (NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:8-57), at block 32
    for n in (1, 257, 515):
        a = vectors.reducer_vector(n, 0.0, 0.25, 2.75)
        b = vectors.reducer_vector(n, 11.0, 0.5, 3.25)
        payloads, scales = encode_on_device([a, b], 32)
        out_p = [torch.zeros(n, dtype=torch.int8, device="cuda")]
        out_s = [torch.zeros(scale_count(n, 32), dtype=torch.float32, device="cuda")]
        reducers.reduce_shards_bfp8(0, payloads, scales, out_p, out_s, 0, n, 32, 1.0)
        torch.cuda.synchronize()
        ea, eb = oracle.encode(a, 32), oracle.encode(b, 32)
        total = oracle.decode(*ea, 32) + oracle.decode(*eb, 32)
        expect_payload, expect_scales = oracle.encode(total, 32)
        assert_bits_equal(host(out_p[0]), expect_payload, "payload")
        assert_bits_equal(host(out_s[0]), expect_scales, "scales")


def test_invalid_scale_or_overflow_raises_the_flag(cuda, oracle):
    n = 4096
    g = vectors.config0_gradient(oracle, 0, n)
    payloads, scales = encode_on_device([g, g], 32)
    scales[1][3] = float("nan")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    reducers.reduce_shards_bfp8(0, payloads, scales, payloads[:1], scales[:1], 0, n, 32, 1.0, None, flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    payloads, scales = encode_on_device([g, g], 32)
    scales[0][5] = 3e38
    scales[1][5] = 3e38
    flag.zero_()
    reducers.reduce_shards_bfp8(0, payloads, scales, payloads[:1], scales[:1], 0, n, 32, 1.0, None, flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 1          # 127*3e38 overflows to Inf


def test_unaligned_arenas_take_the_scalar_path(cuda, oracle):
    n, block, world = 5000, 32, 3
    gradients = [vectors.config0_gradient(oracle, r, n) for r in range(world)]
    payloads, scales = encode_on_device(gradients, block)
    shifted = []
    for p in payloads:
        base = torch.zeros(n + 64, dtype=torch.int8, device="cuda")
        base[3:3 + n].copy_(p)
        shifted.append(base[3:3 + n])
    reducers.reduce_shards_bfp8(0, shifted, scales, shifted, scales, 0, n, block, 1.0)
    torch.cuda.synchronize()
    expect_payload, expect_scales, _, _ = oracle.allreduce_bfp8(gradients, block, 1.0)
    assert_bits_equal(host(shifted[0]), expect_payload, "payload")
    assert_bits_equal(host(scales[2]), expect_scales, "scales")


@pytest.mark.parametrize("world", (2, 8))
@pytest.mark.parametrize("n", (1, 515, 70001, 1 << 20))
def test_bf16_emulated_ranks(cuda, oracle, world, n):
    # fp32 accumulate in rank order, bf16 result, sum of squares of the bf16
    # result (NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:1413-1459)
    inputs = [oracle.bf16_encode(vectors.config0_gradient(oracle, r, n), 1) for r in range(world)]
    arenas = [bf16_dev(b) for b in inputs]
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    reduced = torch.zeros(n, dtype=torch.float32, device="cuda")
    for rank in range(world):
        first, end = reducers.shard_range(n, world, rank)
        if end > first:
            reducers.reduce_shards_bf16(0, arenas, arenas, reduced, first, end, 1.0, sq, True)
    torch.cuda.synchronize()
    expect_f32, expect_bf16, expect_sq = oracle.bf16_reduce(inputs, 1.0, want_bf16=True, square_of_bf16=True)
    assert_bits_equal(host(reduced), expect_f32, "fp32 sum")
    for rank in range(world):
        assert_bits_equal(bf16_host(arenas[rank]), expect_bf16, f"bf16 arena on rank {rank}")
    assert sq.item() == pytest.approx(expect_sq, rel=1e-12)


@pytest.mark.parametrize("chunk", (None, 1 << 16))
@pytest.mark.parametrize("max_norm", (1.0, None))
def test_single_rank_step_is_the_one_gpu_publication(cuda, oracle, chunk, max_norm):
    # world 1: encode + decode write-back + sum of squares + finite flag, then
    # the scale-only clip (NNtrain.Core/Tensors/CudaBfp8GradientPublicationScope.cs:12-521;
    # NNtrain.Core.Tests/CudaBfp8GradientClipNormTests.cs:275-302)
    n = (1 << 18) + 1000
    g = vectors.config0_gradient(oracle, 0, n)
    group = reducers.GradientGroup(1, 0, 0)
    step = reducers.Bfp8ArenaAllReduce(group, n, 32, reducers.PEER, chunk_elements=chunk)
    arena = dev(g)
    step.enqueue(arena, max_norm)
    result = step.complete(max_norm)
    expect_g, expect_payload, expect_scales, _, expect_sq = oracle.gradient_publish(g, 32)
    assert_bits_equal(host(step.payload), expect_payload, "payload")
    assert_bits_equal(host(arena), expect_g, "fp32 arena holds decode(encode(g))")
    assert result.squared_sum == pytest.approx(expect_sq, rel=1e-12)
    norm, c = oracle.clip_coefficient(expect_sq, max_norm if max_norm else 1e30)
    assert abs(result.norm - norm) <= max(1e-5, 2e-6 * abs(norm))
    if max_norm is not None:
        assert result.coefficient == pytest.approx(c, rel=2e-6)
        assert_bits_equal(host(step.scales), oracle.scale_bfp8_scales(expect_scales, result.coefficient),
                          "clipped scales")
    else:
        assert_bits_equal(host(step.scales), expect_scales, "scales")
    assert step.transport_bytes_per_step == 0
    step.close()
    group.close()


def test_non_finite_gradient_fails_complete(cuda, oracle):
    # NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:95-130
    n = 1 << 16
    g = vectors.config0_gradient(oracle, 0, n)
    g[777] = np.inf
    group = reducers.GradientGroup(1, 0, 0)
    step = reducers.Bfp8ArenaAllReduce(group, n, 32)
    step.enqueue(dev(g))
    with pytest.raises(FloatingPointError):
        step.complete()
    step.close()
    group.close()


@pytest.mark.parametrize("mode", (0, 1, 2, 3, 4))
@pytest.mark.parametrize("world", (2, 4, 8))
@pytest.mark.parametrize("block", (32, 128))
def test_every_way_of_fetching_the_shards_gives_the_same_bits(cuda, oracle, lib, mode, world, block):
    """The owner kernel's forms -- register prefetch, cp.async rings, rings in
    CTAs that own their SM, bulk asynchronous copies in big and in small CTAs
    -- on emulated ranks,
    with a ragged end and a shard that starts in the middle of the arena."""
    n = 6 * 65536 + 1024 + 333
    gradients = [vectors.config0_gradient(oracle, r, n) for r in range(world)]
    scale = 1.0 / world
    expect_payload, expect_scales, _, expect_sq = oracle.allreduce_bfp8(gradients, block, scale)
    assert lib.nntrain_gradient_configure_collective(mode) == 0
    assert lib.nntrain_gradient_configure(2, 5) == 0          # few CTAs: every warp loops over several tiles
    try:
        for _ in range(2):
            payloads, scales = encode_on_device(gradients, block)
            sq = torch.zeros(1, dtype=torch.float64, device="cuda")
            flag = torch.zeros(1, dtype=torch.int32, device="cuda")
            for rank in range(world):
                first, end = reducers.shard_range(n, world, rank)
                reducers.reduce_shards_bfp8(0, payloads, scales, payloads, scales, first, end, block, scale, sq, flag)
            torch.cuda.synchronize()
            for rank in range(world):
                assert_bits_equal(host(payloads[rank]), expect_payload, f"payload on rank {rank}, mode {mode}")
                assert_bits_equal(host(scales[rank]), expect_scales, f"scales on rank {rank}, mode {mode}")
            assert int(flag.item()) == 0
            assert sq.item() == pytest.approx(expect_sq, rel=1e-12)
    finally:
        assert lib.nntrain_gradient_configure_collective(1) == 0
        assert lib.nntrain_gradient_configure(2, 0) == 0
