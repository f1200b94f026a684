"""Local kernels recorded into a CUDA graph and replayed: what the reference's
captured-backward path relies on (publication scope with stable slot
addresses, NNtrain.Core/Tensors/CudaBfp8GradientPublicationScope.cs:12-521;
replay == eager, NNtrain.Core.Tests/CudaCapturedGradientReducerTests.cs:550-574).
Cross-device work is never captured, there as here."""
import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, dev, host
from nntrain_b200.native import CudaBfp8GradientNative, CudaBfp8Native, GradientNorm, scale_count

pytestmark = pytest.mark.gpu


def test_block_publication_and_clip_replay_equals_eager(cuda, oracle):
    n, block = 300137, 32
    gradients = [vectors.config0_gradient(oracle, r, n) for r in range(3)]
    arena = torch.zeros(n, dtype=torch.float32, device="cuda")
    payload = torch.zeros(n, dtype=torch.int8, device="cuda")
    scales = torch.zeros(scale_count(n, block), dtype=torch.float32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    coefficient = torch.zeros(2, dtype=torch.float32, device="cuda")

    def step():
        sq.zero_()
        flag.zero_()
        CudaBfp8Native.block_encode(0, arena, payload, scales, block, roundtrip=arena, squared_sum=sq,
                                    finite_status=flag)
        GradientNorm.clip_coefficient(0, sq, 1.0, coefficient)
        GradientNorm.clip_apply(0, GradientNorm.BFP8, scales, coefficient=coefficient)

    arena.copy_(torch.from_numpy(gradients[0]))
    step()                                   # eager warm-up (also loads every kernel before capture)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    arena.copy_(torch.from_numpy(gradients[0]))
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        step()
    for g in gradients:                      # the same recorded step on new data in the same slots
        arena.copy_(torch.from_numpy(g))
        graph.replay()
        torch.cuda.synchronize()
        replayed = (host(payload).copy(), host(scales).copy(), host(arena).copy(), sq.item(), int(flag.item()))
        arena.copy_(torch.from_numpy(g))
        step()
        torch.cuda.synchronize()
        assert_bits_equal(replayed[0], host(payload), "payload: replay vs eager")
        assert_bits_equal(replayed[1], host(scales), "clipped scales: replay vs eager")
        assert_bits_equal(replayed[2], host(arena), "write-back: replay vs eager")
        assert replayed[3] == pytest.approx(sq.item(), rel=1e-12) and replayed[4] == 0
        fp32, expect_payload, expect_scales, _, expect_sq = oracle.gradient_publish(g, block)
        _, c = oracle.clip_coefficient(expect_sq, 1.0)
        assert_bits_equal(replayed[0], expect_payload, "payload vs oracle")
        assert_bits_equal(replayed[2], fp32, "write-back vs oracle")
        assert replayed[3] == pytest.approx(expect_sq, rel=1e-12)
        assert np.array_equal(replayed[1], oracle.scale_bfp8_scales(expect_scales, float(coefficient[1].item())))
        assert abs(float(coefficient[1].item()) - c) <= 2e-6 * c


def test_whole_bucket_publication_replays(cuda, oracle):
    numels = [4099, 33, 1, 20000, 517, 16384, 7, 9001]
    offsets = np.concatenate([[0], np.cumsum(numels)]).astype(np.int64)
    total = int(offsets[-1])
    arena = torch.zeros(total, dtype=torch.float32, device="cuda")
    payload = torch.zeros(total, dtype=torch.int8, device="cuda")
    scales = torch.zeros(len(numels), dtype=torch.float32, device="cuda")
    scratch = torch.zeros(len(numels), dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    table = dev(offsets)

    def step():
        sq.zero_()
        CudaBfp8GradientNative.publish_tensors(0, arena, payload, scales, table, scratch, flag, sq)

    flat = oracle.generate_gradient(total, 31, 0)
    arena.copy_(torch.from_numpy(flat))
    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        step()
    for seed in (32, 33):
        flat = oracle.generate_gradient(total, seed, 0)
        arena.copy_(torch.from_numpy(flat))
        graph.replay()
        torch.cuda.synchronize()
        expect_total = 0.0
        for t in range(len(numels)):
            a, b = offsets[t], offsets[t + 1]
            g, p, s, bad, squares = oracle.gradient_publish(flat[a:b], 0)
            assert_bits_equal(host(payload)[a:b], p, f"payload of tensor {t}")
            assert_bits_equal(host(scales)[t:t + 1], s, f"scale of tensor {t}")
            assert_bits_equal(host(arena)[a:b], g, f"write-back of tensor {t}")
            expect_total += squares
        assert sq.item() == pytest.approx(expect_total, rel=1e-12) and int(flag.item()) == 0
