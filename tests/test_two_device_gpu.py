"""The reference's own two-device entry points, one process driving two GPUs:
the tensor-wide BFP8 reduce / broadcast and the bucket exchanges across real
peer copies.  Runs when the box has at least two GPUs."""
import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, host
from nntrain_b200.native import CudaBfp8GradientNative, CudaGradientBuckets

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def two_devices(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    return cuda


def on(device: int, array, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(array))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(f"cuda:{device}")


@pytest.mark.parametrize("n", (1, 257, 515, 300137))
@pytest.mark.parametrize("reduction_scale", (1.0, 0.5))
def test_tensor_wide_reduce_and_broadcast(two_devices, oracle, n, reduction_scale):
    # result == Encode(Decode(Encode a) + Decode(Encode b)): payload exact,
    # scale exact, both replicas bit-identical, fp32 = decode of the result
    # (NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:8-57)
    a = vectors.reducer_vector(n, 0.0, 0.25, 2.75)
    b = vectors.reducer_vector(n, 11.0, 0.5, 3.25)
    grads = [on(0, a), on(1, b)]
    payload = [torch.zeros(n, dtype=torch.int8, device=f"cuda:{d}") for d in (0, 1)]
    scale = [torch.zeros(1, dtype=torch.float32, device=f"cuda:{d}") for d in (0, 1)]
    flag = [torch.zeros(1, dtype=torch.int32, device=f"cuda:{d}") for d in (0, 1)]
    streams, ready = [], []
    for d in (0, 1):
        with torch.cuda.device(d):
            CudaBfp8GradientNative.quantize(d, grads[d], payload[d], scale[d], flag[d])
            event = CudaGradientBuckets.create_ready_event(d)
            CudaGradientBuckets.record_ready(d, event)
            ready.append(event)
            streams.append(CudaGradientBuckets.create_communication_stream(d))
    with torch.cuda.device(0):
        staging_payload = torch.zeros(n, dtype=torch.int8, device="cuda:0")
        staging_scale = torch.zeros(1, dtype=torch.float32, device="cuda:0")
        staging_status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        out_payload = torch.zeros(n, dtype=torch.int8, device="cuda:0")
        out_scale = torch.zeros(1, dtype=torch.float32, device="cuda:0")
        sq = torch.zeros(1, dtype=torch.float64, device="cuda:0")
        reduced_ready = CudaGradientBuckets.create_ready_event(0)
        CudaBfp8GradientNative.reduce(0, 1, payload[0], scale[0], payload[1], scale[1], staging_payload, staging_scale,
                                      grads[0], out_payload, out_scale, reduction_scale, flag[0], flag[1],
                                      staging_status, sq, streams[0], ready[0], ready[1], reduced_ready)
    with torch.cuda.device(1):
        CudaBfp8GradientNative.broadcast(1, 0, out_payload, out_scale, payload[1], scale[1], grads[1], flag[1],
                                         streams[1], reduced_ready)
    for d in (0, 1):
        CudaGradientBuckets.synchronize(d, streams[d])
    ea, eb = oracle.encode(a, 0), oracle.encode(b, 0)
    total, _ = oracle.reduce_bfp8([ea[0], eb[0]], [ea[1], eb[1]], 0, reduction_scale)
    expect_payload, expect_scale = oracle.encode(total, 0)
    expect_fp32 = oracle.decode(expect_payload, expect_scale, 0)
    assert_bits_equal(host(out_payload), expect_payload, "reduced payload on the primary")
    assert_bits_equal(host(out_scale), expect_scale, "reduced scale on the primary")
    assert_bits_equal(host(payload[1]), expect_payload, "payload on the secondary")
    assert_bits_equal(host(scale[1]), expect_scale, "scale on the secondary")
    assert_bits_equal(host(grads[0]), expect_fp32, "fp32 on the primary")
    assert_bits_equal(host(grads[1]), expect_fp32, "fp32 on the secondary")
    assert int(flag[0].item()) == 0 and int(flag[1].item()) == 0
    assert sq.item() == pytest.approx(oracle.squared_sum_bfp8(expect_payload, expect_scale, 0), rel=1e-12)
    for d in (0, 1):
        CudaGradientBuckets.destroy_event(d, ready[d])
        CudaGradientBuckets.destroy_communication_stream(d, streams[d])
    CudaGradientBuckets.destroy_event(0, reduced_ready)


def test_non_finite_on_the_secondary_raises_the_primary_flag(two_devices, oracle):
    # NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:95-130
    n = 4096
    a = vectors.codec_vector(n)
    b = vectors.codec_vector(n)
    b[17] = np.nan
    grads = [on(0, a), on(1, b)]
    payload = [torch.zeros(n, dtype=torch.int8, device=f"cuda:{d}") for d in (0, 1)]
    scale = [torch.zeros(1, dtype=torch.float32, device=f"cuda:{d}") for d in (0, 1)]
    flag = [torch.zeros(1, dtype=torch.int32, device=f"cuda:{d}") for d in (0, 1)]
    ready, streams = [], []
    for d in (0, 1):
        with torch.cuda.device(d):
            CudaBfp8GradientNative.quantize(d, grads[d], payload[d], scale[d], flag[d])
            event = CudaGradientBuckets.create_ready_event(d)
            CudaGradientBuckets.record_ready(d, event)
            ready.append(event)
            streams.append(CudaGradientBuckets.create_communication_stream(d))
    with torch.cuda.device(0):
        stage_p = torch.zeros(n, dtype=torch.int8, device="cuda:0")
        stage_s = torch.zeros(1, dtype=torch.float32, device="cuda:0")
        stage_f = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        out_p = torch.zeros(n, dtype=torch.int8, device="cuda:0")
        out_s = torch.zeros(1, dtype=torch.float32, device="cuda:0")
        sq = torch.zeros(1, dtype=torch.float64, device="cuda:0")
        done = CudaGradientBuckets.create_ready_event(0)
        CudaBfp8GradientNative.reduce(0, 1, payload[0], scale[0], payload[1], scale[1], stage_p, stage_s, grads[0],
                                      out_p, out_s, 1.0, flag[0], flag[1], stage_f, sq, streams[0], ready[0],
                                      ready[1], done)
        CudaGradientBuckets.synchronize(0, streams[0])
    assert int(flag[1].item()) == 1 and int(flag[0].item()) == 1


@pytest.mark.parametrize("n", (515, 1 << 20))
def test_bucket_exchanges_across_two_devices(two_devices, oracle, n):
    # symmetric pull: each device pulls the other's bucket and sums; both end
    # with bit-identical fp32 (NNtrain.Cuda/native/gradient_collectives.cu:272-357)
    g = [vectors.config0_gradient(oracle, r, n) for r in (0, 1)]
    packed = [oracle.pack_bfp8_block(x, 128) for x in g]
    bf16 = [oracle.bf16_encode(x, 1) for x in g]
    expect_block, expect_block_sq = oracle.block_transport_sum([p[0] for p in packed], [p[1] for p in packed], 128)
    expect_bf16, _, expect_bf16_sq = oracle.bf16_reduce(bf16)
    local_p = [on(d, packed[d][0]) for d in (0, 1)]
    local_s = [on(d, packed[d][1]) for d in (0, 1)]
    local_16 = [on(d, bf16[d].view(np.int16)) for d in (0, 1)]
    events, streams = [], []
    for d in (0, 1):
        with torch.cuda.device(d):
            torch.cuda.synchronize(d)
            event = CudaGradientBuckets.create_ready_event(d)
            CudaGradientBuckets.record_ready(d, event)
            events.append(event)
            streams.append(CudaGradientBuckets.create_communication_stream(d))
    for d in (0, 1):
        peer = 1 - d
        with torch.cuda.device(d):
            stage_p = torch.zeros(n, dtype=torch.int8, device=f"cuda:{d}")
            stage_s = torch.zeros_like(local_s[d])
            stage_16 = torch.zeros(n, dtype=torch.int16, device=f"cuda:{d}")
            reduced = torch.zeros(n, dtype=torch.float32, device=f"cuda:{d}")
            reduced16 = torch.zeros(n, dtype=torch.float32, device=f"cuda:{d}")
            sq = torch.zeros(2, dtype=torch.float64, device=f"cuda:{d}")
            CudaGradientBuckets.exchange_bfp8_block(d, peer, local_p[d], local_s[d], local_p[peer], local_s[peer],
                                                    stage_p, stage_s, reduced, sq[0:1], streams[d], events[d],
                                                    events[peer])
            CudaGradientBuckets.exchange(d, peer, local_16[d], local_16[peer], stage_16, reduced16, sq[1:2],
                                         streams[d], events[d], events[peer])
            CudaGradientBuckets.synchronize(d, streams[d])
            # the sum is commutative in fp32, so both devices hold the same bits
            assert_bits_equal(host(reduced), expect_block, f"block transport sum on device {d}")
            assert_bits_equal(host(reduced16), expect_bf16, f"bf16 transport sum on device {d}")
            assert sq[0].item() == pytest.approx(expect_block_sq, rel=1e-12)
            assert sq[1].item() == pytest.approx(expect_bf16_sq, rel=1e-12)
    for d in (0, 1):
        CudaGradientBuckets.destroy_event(d, events[d])
        CudaGradientBuckets.destroy_communication_stream(d, streams[d])


def test_pinned_host_pipeline_gives_the_same_sums(two_devices, oracle):
    # the no-peer-access fallback: chunks bounce through pinned host memory,
    # double-buffered; results must equal the peer-copy exchange
    # (NNtrain.Cuda/native/gradient_collectives.cu:359-709;
    #  NNtrain.Core.Tests/CudaMix8GradientTransportTests.cs:108-219)
    chunk = 4096
    n = 3 * chunk + 515                       # three full chunks and a ragged one
    g = [vectors.config0_gradient(oracle, r, n) for r in (0, 1)]
    packed = [oracle.pack_bfp8_block(x, 128) for x in g]
    bf16 = [oracle.bf16_encode(x, 1) for x in g]
    expect_block, expect_block_sq = oracle.block_transport_sum([p[0] for p in packed], [p[1] for p in packed], 128)
    expect_bf16, _, expect_bf16_sq = oracle.bf16_reduce(bf16)
    local_p, local_s, local_16 = on(0, packed[0][0]), on(0, packed[0][1]), on(0, bf16[0].view(np.int16))
    remote_p, remote_s, remote_16 = on(1, packed[1][0]), on(1, packed[1][1]), on(1, bf16[1].view(np.int16))
    events = []
    for d in (0, 1):
        with torch.cuda.device(d):
            torch.cuda.synchronize(d)
            event = CudaGradientBuckets.create_ready_event(d)
            CudaGradientBuckets.record_ready(d, event)
            events.append(event)
    reduced = torch.zeros(n, dtype=torch.float32, device="cuda:0")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda:0")
    pipeline = CudaGradientBuckets.create_host_pipeline(1, 0, chunk, bfp8_block=True)
    CudaGradientBuckets.host_pipeline_exchange_bfp8_block(pipeline, local_p, local_s, remote_p, remote_s, reduced, sq,
                                                          events[0], events[1])
    CudaGradientBuckets.destroy_host_pipeline(pipeline)
    assert_bits_equal(host(reduced), expect_block, "block transport through the host pipeline")
    assert sq.item() == pytest.approx(expect_block_sq, rel=1e-12)
    reduced.zero_()
    sq.zero_()
    torch.cuda.synchronize(0)
    pipeline = CudaGradientBuckets.create_host_pipeline(1, 0, chunk)
    CudaGradientBuckets.host_pipeline_exchange(pipeline, local_16, remote_16, reduced, sq, events[0], events[1])
    CudaGradientBuckets.destroy_host_pipeline(pipeline)
    assert_bits_equal(host(reduced), expect_bf16, "bf16 transport through the host pipeline")
    assert sq.item() == pytest.approx(expect_bf16_sq, rel=1e-12)
    for d in (0, 1):
        CudaGradientBuckets.destroy_event(d, events[d])
