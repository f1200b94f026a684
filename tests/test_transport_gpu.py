"""Bucket transport entry points (pack, exchange, unpack) against the oracle.
The exchange runs with source and destination on device 0: the peer copy is
then a device-local copy, the arithmetic and the stream / event protocol are
the same as across two devices."""
import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, bf16_dev, bf16_host, dev, host
from nntrain_b200.native import CudaGradientBuckets

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,offset", ((515, 0), (515, 3), (1 << 18, 128), (70001, 1)))
def test_pack_bf16_rounds_to_nearest_even_at_an_offset(cuda, oracle, n, offset):
    g = vectors.config0_gradient(oracle, 0, n)
    bucket = torch.zeros(n + offset + 8, dtype=torch.int16, device="cuda")
    CudaGradientBuckets.pack(0, dev(g), bucket, offset)
    torch.cuda.synchronize()
    out = bf16_host(bucket)
    assert_bits_equal(out[offset:offset + n], oracle.bf16_encode(g, 1), "packed bf16")
    assert not out[:offset].any() and not out[offset + n:].any()


@pytest.mark.parametrize("n", (1, 100, 128, 515, 1 << 18, 300137))
def test_pack_bfp8_block_matches_oracle_including_poisoned_blocks(cuda, oracle, n):
    g = vectors.config0_gradient(oracle, 1, n)
    if n > 300:
        g[130] = np.nan
        g[n - 1] = np.inf
    expect_payload, expect_scales = oracle.pack_bfp8_block(g, 128)
    payload = torch.full((n,), 9, dtype=torch.int8, device="cuda")
    scales = torch.zeros((n + 127) // 128, dtype=torch.float32, device="cuda")
    CudaGradientBuckets.pack_bfp8_block(0, dev(g), payload, scales)
    torch.cuda.synchronize()
    assert_bits_equal(host(payload), expect_payload, "payload")
    assert_bits_equal(host(scales), expect_scales, "scales")


def _events_and_stream():
    stream = CudaGradientBuckets.create_communication_stream(0)
    a = CudaGradientBuckets.create_ready_event(0)
    b = CudaGradientBuckets.create_ready_event(0)
    return stream, a, b


def _release(stream, a, b):
    CudaGradientBuckets.destroy_event(0, a)
    CudaGradientBuckets.destroy_event(0, b)
    CudaGradientBuckets.destroy_communication_stream(0, stream)


@pytest.mark.parametrize("n", (1, 257, 515, 1 << 18))
def test_exchange_bf16_sums_in_fp32(cuda, oracle, n):
    # NNtrain.Core.Tests/CudaMix8GradientTransportTests.cs:83-88
    a = oracle.bf16_encode(vectors.config0_gradient(oracle, 0, n), 1)
    b = oracle.bf16_encode(vectors.config0_gradient(oracle, 1, n), 1)
    local, remote = bf16_dev(a), bf16_dev(b)
    staging = torch.zeros(n, dtype=torch.int16, device="cuda")
    reduced = torch.zeros(n, dtype=torch.float32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    stream, ready_a, ready_b = _events_and_stream()
    CudaGradientBuckets.record_ready(0, ready_a)
    CudaGradientBuckets.record_ready(0, ready_b)
    CudaGradientBuckets.exchange(0, 0, local, remote, staging, reduced, sq, stream, ready_a, ready_b)
    CudaGradientBuckets.synchronize(0, stream)
    expect, _, expect_sq = oracle.bf16_reduce([a, b])
    assert_bits_equal(host(reduced), expect, "reduced")
    assert_bits_equal(bf16_host(staging), b, "staging holds the peer's bucket")
    assert sq.item() == pytest.approx(expect_sq, rel=1e-12)
    _release(stream, ready_a, ready_b)


@pytest.mark.parametrize("n", (1, 257, 515, 1 << 18))
def test_exchange_bfp8_block_keeps_the_raw_fp32_sum(cuda, oracle, n):
    # NNtrain.Cuda/native/gradient_collectives.cu:92-129: no re-encode, both
    # replicas get fl(fl(q0*s0) + fl(q1*s1))
    ga, gb = vectors.config0_gradient(oracle, 0, n), vectors.config0_gradient(oracle, 1, n)
    pa, sa = oracle.pack_bfp8_block(ga, 128)
    pb, sb = oracle.pack_bfp8_block(gb, 128)
    staging = torch.zeros(n, dtype=torch.int8, device="cuda")
    staging_scales = torch.zeros_like(dev(sb))
    reduced = torch.zeros(n, dtype=torch.float32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    stream, ready_a, ready_b = _events_and_stream()
    CudaGradientBuckets.record_ready(0, ready_a)
    CudaGradientBuckets.record_ready(0, ready_b, external=False)
    CudaGradientBuckets.exchange_bfp8_block(0, 0, dev(pa), dev(sa), dev(pb), dev(sb), staging, staging_scales,
                                            reduced, sq, stream, ready_a, ready_b)
    CudaGradientBuckets.synchronize(0, stream)
    expect, expect_sq = oracle.block_transport_sum([pa, pb], [sa, sb], 128)
    assert_bits_equal(host(reduced), expect, "reduced")
    assert sq.item() == pytest.approx(expect_sq, rel=1e-12)
    # transport bytes per step, 2 devices: 2 * (n + 4 * ceil(n / 128))
    # (NNtrain.Core.Tests/CudaMix8GradientTransportTests.cs:267-270)
    assert 2 * (staging.numel() + 4 * staging_scales.numel()) == 2 * (n + 4 * ((n + 127) // 128))
    _release(stream, ready_a, ready_b)


def test_unpack_copies_a_slice(cuda):
    source = torch.arange(5000, dtype=torch.float32, device="cuda")
    destination = torch.zeros(1237, dtype=torch.float32, device="cuda")
    stream, a, b = _events_and_stream()
    CudaGradientBuckets.unpack(0, source, 1001, destination, stream)
    CudaGradientBuckets.synchronize(0, stream)
    assert torch.equal(destination, source[1001:1001 + 1237])
    _release(stream, a, b)


def test_external_ready_event_records_inside_stream_capture(cuda, oracle):
    """Pack + external ready record are capturable; the exchange stays outside
    the graph (NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:562-583).
    Replay must equal eager bit for bit."""
    n = 1 << 16
    g = vectors.config0_gradient(oracle, 0, n)
    src = dev(g)
    payload = torch.zeros(n, dtype=torch.int8, device="cuda")
    scales = torch.zeros(n // 128, dtype=torch.float32, device="cuda")
    event = CudaGradientBuckets.create_ready_event(0)
    capture_stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=capture_stream, capture_error_mode="thread_local"):
        CudaGradientBuckets.pack_bfp8_block(0, src, payload, scales)
        CudaGradientBuckets.record_ready(0, event, external=True)
    payload.zero_()
    scales.zero_()
    graph.replay()
    torch.cuda.synchronize()
    expect_payload, expect_scales = oracle.pack_bfp8_block(g, 128)
    assert_bits_equal(host(payload), expect_payload, "payload after replay")
    assert_bits_equal(host(scales), expect_scales, "scales after replay")
    CudaGradientBuckets.destroy_event(0, event)
