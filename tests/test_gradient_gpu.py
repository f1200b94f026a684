"""Tensor-wide BFP8 gradient publication, sum of squares, scale-only clip and
the norm / clip entry points, against the CPU oracle through the C ABI."""
import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, bf16_dev, bf16_host, dev, host
from nntrain_b200.native import CudaBfp8GradientNative, GradientNorm

pytestmark = pytest.mark.gpu


def norm_tolerance(norm: float) -> float:
    # NNtrain.Core.Tests/CudaBfp8GradientClipNormTests.cs:275-279
    return max(1e-5, 2e-6 * abs(norm))


@pytest.mark.parametrize("n", (1, 257, 515, 300137, 1 << 20))
def test_publish_matches_cpu_codec(cuda, oracle, n):
    source = vectors.reducer_vector(n, 3.0, 0.25, 2.75) if n < 1000 else vectors.config0_gradient(oracle, 0, n)
    gradient = dev(source)
    payload = torch.zeros(n, dtype=torch.int8, device="cuda")
    scale = torch.zeros(1, dtype=torch.float32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    CudaBfp8GradientNative.quantize(0, gradient, payload, scale, flag, sq)
    torch.cuda.synchronize()
    expect_g, expect_payload, expect_scale, expect_flag, expect_sq = oracle.gradient_publish(source, 0)
    assert int(flag.item()) == expect_flag == 0
    assert_bits_equal(host(payload), expect_payload, "payload")
    assert_bits_equal(host(scale), expect_scale, "scale")
    assert_bits_equal(host(gradient), expect_g, "gradient after publish (decode cache)")
    assert sq.item() == pytest.approx(expect_sq, rel=1e-12)
    # the stand-alone sum of squares agrees
    sq2 = torch.zeros(1, dtype=torch.float64, device="cuda")
    CudaBfp8GradientNative.accumulate_squared_sum(0, payload, scale, sq2, flag)
    torch.cuda.synchronize()
    assert sq2.item() == pytest.approx(expect_sq, rel=1e-12)
    # the no-accumulate entry point gives the same payload
    gradient2 = dev(source)
    payload2 = torch.zeros_like(payload)
    scale2 = torch.zeros_like(scale)
    CudaBfp8GradientNative.quantize(0, gradient2, payload2, scale2, flag)
    torch.cuda.synchronize()
    assert torch.equal(payload, payload2) and torch.equal(scale, scale2) and torch.equal(gradient, gradient2)


@pytest.mark.parametrize("poison", (float("nan"), float("inf"), float("-inf")))
def test_non_finite_gradient_publishes_nothing(cuda, oracle, poison):
    # NNtrain.Core.Tests/CudaBfp8KernelTests.cs:293-414;
    # NNtrain.Cuda/native/tensor_kernels.cu:1011-1042
    n = 70000
    source = vectors.config0_gradient(oracle, 0, n)
    source[n // 2] = poison
    gradient = dev(source)
    payload = torch.full((n,), 5, dtype=torch.int8, device="cuda")
    scale = torch.zeros(1, dtype=torch.float32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    CudaBfp8GradientNative.quantize(0, gradient, payload, scale, flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    assert scale.item() == 1.0
    assert bool((payload == 5).all())
    assert_bits_equal(host(gradient), source, "gradient must be untouched")
    # the flag is sticky: a later clean tensor of the same step is skipped too
    clean = dev(vectors.codec_vector(515))
    payload2 = torch.full((515,), 5, dtype=torch.int8, device="cuda")
    CudaBfp8GradientNative.quantize(0, clean, payload2, scale, flag)
    torch.cuda.synchronize()
    assert bool((payload2 == 5).all()) and scale.item() == 1.0


def test_scale_only_clip_leaves_payload_untouched(cuda, oracle):
    # NNtrain.Core.Tests/CudaBfp8GradientClipNormTests.cs:281-302
    scale = dev(np.array([0.0375], np.float32))
    CudaBfp8GradientNative.scale(0, scale, 0.25)
    torch.cuda.synchronize()
    assert_bits_equal(host(scale), oracle.scale_bfp8_scales(np.array([0.0375], np.float32), 0.25), "scale")
    tiny = dev(np.array([1e-37], np.float32))
    CudaBfp8GradientNative.scale(0, tiny, 1e-5)
    torch.cuda.synchronize()
    assert tiny.item() == np.finfo(np.float32).tiny


@pytest.mark.parametrize("n", (1, 1023, 1 << 20, (1 << 20) + 3))
def test_squared_sums_of_all_three_kinds(cuda, oracle, n):
    g = vectors.config0_gradient(oracle, 1, n)
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    GradientNorm.squared_sum(0, GradientNorm.FP32, dev(g), sq)
    torch.cuda.synchronize()
    expect = oracle.squared_sum_f32(g)
    assert sq.item() == pytest.approx(expect, rel=1e-12)

    bits = oracle.bf16_encode(g, 1)
    sq.zero_()
    GradientNorm.squared_sum(0, GradientNorm.BF16, bf16_dev(bits), sq)
    torch.cuda.synchronize()
    assert sq.item() == pytest.approx(oracle.squared_sum_bf16(bits), rel=1e-12)

    for block in (32, 128, 0):
        payload, scales = oracle.encode(g, block, strict=False)
        sq.zero_()
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        GradientNorm.squared_sum(0, GradientNorm.BFP8, dev(payload), sq, dev(scales), block, flag)
        torch.cuda.synchronize()
        assert int(flag.item()) == 0
        assert sq.item() == pytest.approx(oracle.squared_sum_bfp8(payload, scales, block), rel=1e-12)


def test_invalid_scale_raises_the_flag_and_contributes_nothing(cuda, oracle):
    # NNtrain.Cuda/native/tensor_kernels.cu:1051-1054
    payload = dev(np.full(256, 3, np.int8))
    scales = dev(np.array([0.5, -1.0, np.nan, 0.25, 0.0, 1.0, 1.0, 1.0], np.float32))
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    GradientNorm.squared_sum(0, GradientNorm.BFP8, payload, sq, scales, 32, flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    assert sq.item() == pytest.approx(32 * (1.5 ** 2 + 0.75 ** 2 + 3 * 9.0), rel=1e-12)


@pytest.mark.parametrize("max_norm", (1.0, 1e6))
def test_device_side_clip_matches_cpu_clip(cuda, oracle, max_norm):
    # NNtrain.Core/Torch/nn.cs:62-81; all three storage kinds
    n = (1 << 18) + 5
    g = vectors.config0_gradient(oracle, 0, n)
    expect_sq = oracle.squared_sum_f32(g)
    expect_norm, expect_c = oracle.clip_coefficient(expect_sq, max_norm)
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    out = torch.zeros(2, dtype=torch.float32, device="cuda")
    values = dev(g)
    GradientNorm.squared_sum(0, GradientNorm.FP32, values, sq)
    GradientNorm.clip_coefficient(0, sq, max_norm, out)
    torch.cuda.synchronize()
    norm, c = float(out[0].item()), float(out[1].item())
    assert abs(norm - expect_norm) <= norm_tolerance(expect_norm)          # <= 1e-5 relative
    assert c == pytest.approx(expect_c, rel=2e-6)
    if max_norm > expect_norm:
        assert c == 1.0
    GradientNorm.clip_apply(0, GradientNorm.FP32, values, multiplier=expect_c)
    torch.cuda.synchronize()
    assert_bits_equal(host(values), oracle.scale_f32(g, expect_c), "fp32 clip")

    bits = oracle.bf16_encode(g, 1)
    values16 = bf16_dev(bits)
    GradientNorm.clip_apply(0, GradientNorm.BF16, values16, multiplier=expect_c)
    torch.cuda.synchronize()
    assert_bits_equal(bf16_host(values16), oracle.scale_bf16(bits, expect_c), "bf16 clip")

    payload, scales = oracle.encode(g, 32, strict=False)
    scales_dev = dev(scales)
    coefficient = dev(np.array([expect_norm, expect_c], np.float32))
    GradientNorm.clip_apply(0, GradientNorm.BFP8, scales_dev, coefficient=coefficient)
    torch.cuda.synchronize()
    assert_bits_equal(host(scales_dev), oracle.scale_bfp8_scales(scales, expect_c), "BFP8 scale-only clip")


def test_implicit_stream_entry_points(cuda, oracle, lib):
    # the four exports without a stream argument run on the stream set by
    # nntrain_cuda_use_external_stream (tensor_kernels.cu:2888-2891)
    n = 4099
    g = vectors.codec_vector(n)
    stream = torch.cuda.Stream()
    assert lib.nntrain_cuda_use_external_stream(stream.cuda_stream) == 0
    values = dev(g)
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    bits = torch.zeros(n, dtype=torch.int16, device="cuda")
    back = torch.zeros(n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    assert lib.nntrain_tensor_squared_sum(values.data_ptr(), n, sq.data_ptr()) == 0
    assert lib.nntrain_tensor_encode_bf16(values.data_ptr(), bits.data_ptr(), n) == 0
    assert lib.nntrain_tensor_decode_bf16(bits.data_ptr(), back.data_ptr(), n) == 0
    assert lib.nntrain_tensor_scale(values.data_ptr(), n, 0.5) == 0
    stream.synchronize()
    assert lib.nntrain_cuda_use_external_stream(None) == 0
    assert sq.item() == pytest.approx(oracle.squared_sum_f32(g), rel=1e-12)
    expect_bits = oracle.bf16_encode(g, 1)
    assert_bits_equal(bf16_host(bits), expect_bits, "bf16 encode")
    assert_bits_equal(host(back), oracle.bf16_decode(expect_bits), "bf16 decode")
    assert_bits_equal(host(values), oracle.scale_f32(g, 0.5), "scale")
