"""CUDA block codec against the CPU oracle, through the C ABI: bit-exact
payload, scales and decode on the reference's own test vectors and sizes, on
the benchmark's distribution (outlier blocks, zero blocks, subnormals), on
ragged lengths and on unaligned pointers."""
import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, dev, host, misaligned
from nntrain_b200.native import CudaBfp8Native, scale_count

pytestmark = pytest.mark.gpu


def run_codec(source: np.ndarray, block: int, src_tensor=None):
    n = source.size
    src = dev(source) if src_tensor is None else src_tensor
    payload = torch.full((n,), 99, dtype=torch.int8, device="cuda")
    scales = torch.full((scale_count(n, block),), -1.0, dtype=torch.float32, device="cuda")
    decoded = torch.full((n,), -7.0, dtype=torch.float32, device="cuda")
    CudaBfp8Native.quantize_float32(0, src, payload, scales, block)
    CudaBfp8Native.dequantize_float32(0, payload, scales, decoded, block)
    torch.cuda.synchronize()
    return host(payload), host(scales), host(decoded)


@pytest.mark.parametrize("block", vectors.REFERENCE_BLOCKS)
def test_quantize_and_dequantize_match_cpu_reference(cuda, oracle, block):
    # NNtrain.Core.Tests/CudaBfp8KernelTests.cs:8-58 (payload exact; scales are
    # compared exactly here, the reference test allows 1e-6)
    source = vectors.codec_vector(515)
    expect_payload, expect_scales = oracle.encode(source, block)
    payload, scales, decoded = run_codec(source, block)
    assert_bits_equal(payload, expect_payload, f"payload block={block}")
    assert_bits_equal(scales, expect_scales, f"scales block={block}")
    assert_bits_equal(decoded, oracle.decode(expect_payload, expect_scales, block), "decoded")


@pytest.mark.parametrize("n", vectors.REFERENCE_LENGTHS)
@pytest.mark.parametrize("block", (0, 32, 64, 96, 128, 1000, 20000))
def test_all_reference_lengths_and_block_sizes(cuda, oracle, n, block):
    source = vectors.tail_max_vector(n) if n > 1000 else vectors.codec_vector(n)
    expect_payload, expect_scales = oracle.encode(source, block)
    payload, scales, decoded = run_codec(source, block)
    assert_bits_equal(payload, expect_payload, f"payload n={n} block={block}")
    assert_bits_equal(scales, expect_scales, f"scales n={n} block={block}")
    assert_bits_equal(decoded, oracle.decode(expect_payload, expect_scales, block), "decoded")


@pytest.mark.parametrize("block", (32, 96, 128))
def test_roundtrip_publishes_encoded_state_in_one_pass(cuda, oracle, block):
    # NNtrain.Core.Tests/CudaBfp8KernelTests.cs:60-111 (all three exact)
    source = vectors.roundtrip_vector(515)
    expect_payload, expect_scales = oracle.encode(source, block)
    state = dev(source)
    payload = torch.zeros(515, dtype=torch.int8, device="cuda")
    scales = torch.zeros(scale_count(515, block), dtype=torch.float32, device="cuda")
    CudaBfp8Native.quantize_float32_roundtrip(0, state, payload, scales, block)
    torch.cuda.synchronize()
    assert_bits_equal(host(payload), expect_payload, "payload")
    assert_bits_equal(host(scales), expect_scales, "scales")
    assert_bits_equal(host(state), oracle.decode(expect_payload, expect_scales, block), "state")


def test_tensor_wide_maximum_at_the_tail(cuda, oracle):
    # NNtrain.Core.Tests/CudaBfp8KernelTests.cs:204-266
    source = vectors.tail_max_vector(300137)
    expect_payload, expect_scales = oracle.encode(source, 0)
    payload, scales, _ = run_codec(source, 0)
    assert scales[0] == np.float32(7.5) / np.float32(127)
    assert_bits_equal(payload, expect_payload, "payload")
    assert_bits_equal(scales, expect_scales, "scale")


@pytest.mark.parametrize("block", (32, 128))
@pytest.mark.parametrize("replica", (0, 1))
def test_benchmark_distribution_with_subnormals_is_bit_exact(cuda, oracle, block, replica):
    # outlier blocks x100, all-zero blocks, subnormal values: nothing may be
    # flushed to zero or rounded differently from the CPU codec
    source = vectors.config0_gradient(oracle, replica, 1 << 20)
    tiny = np.abs(source) < np.finfo(np.float32).tiny
    assert (tiny & (source != 0)).sum() >= 1
    expect_payload, expect_scales = oracle.encode(source, block)
    payload, scales, decoded = run_codec(source, block)
    assert_bits_equal(payload, expect_payload, "payload")
    assert_bits_equal(scales, expect_scales, "scales")
    assert_bits_equal(decoded, oracle.decode(expect_payload, expect_scales, block), "decoded")


def test_all_subnormal_block_keeps_a_subnormal_scale(cuda, oracle):
    source = np.zeros(256, np.float32)
    source[32:64] = np.linspace(1e-40, 9e-40, 32).astype(np.float32)
    source[64] = 1.0
    expect_payload, expect_scales = oracle.encode(source, 32, strict=False)
    assert 0 < expect_scales[1] < np.finfo(np.float32).tiny
    payload, scales, decoded = run_codec(source, 32)
    assert_bits_equal(payload, expect_payload, "payload")
    assert_bits_equal(scales, expect_scales, "scales")
    assert_bits_equal(decoded, oracle.decode(expect_payload, expect_scales, 32, strict=False), "decoded")


@pytest.mark.parametrize("n", (31, 33, 511, 513, 4097, 65537))
def test_ragged_lengths_use_the_same_arithmetic(cuda, oracle, n):
    source = vectors.config0_gradient(oracle, 0, n)
    for block in (32, 64, 128):
        expect_payload, expect_scales = oracle.encode(source, block, strict=False)
        payload, scales, _ = run_codec(source, block)
        assert_bits_equal(payload, expect_payload, f"payload n={n} block={block}")
        assert_bits_equal(scales, expect_scales, f"scales n={n} block={block}")


@pytest.mark.parametrize("offset", (1, 2, 3))
def test_unaligned_pointers_take_the_scalar_path(cuda, oracle, offset):
    # gradient slices of an arena start at arbitrary element offsets
    n = 5000
    source = vectors.config0_gradient(oracle, 0, n)
    src = misaligned(n, torch.float32, offset)
    src.copy_(dev(source))
    payload = misaligned(n, torch.int8, offset)
    scales = torch.zeros(scale_count(n, 32), dtype=torch.float32, device="cuda")
    decoded = misaligned(n, torch.float32, offset)
    CudaBfp8Native.quantize_float32(0, src, payload, scales, 32)
    CudaBfp8Native.dequantize_float32(0, payload, scales, decoded, 32)
    torch.cuda.synchronize()
    expect_payload, expect_scales = oracle.encode(source, 32, strict=False)
    assert_bits_equal(host(payload), expect_payload, "payload")
    assert_bits_equal(host(scales), expect_scales, "scales")
    assert_bits_equal(host(decoded), oracle.decode(expect_payload, expect_scales, 32, strict=False), "decoded")


def test_non_finite_values_follow_device_semantics(cuda, oracle):
    # the generic codec ignores NaN in the maximum and encodes it as 0
    # (NNtrain.Cuda/native/cuda_runtime_bridge.cu:138-192)
    source = vectors.codec_vector(4096)
    source[7] = np.nan
    source[100] = np.inf
    source[2000] = -np.inf
    for block in (32, 128, 96):
        expect_payload, expect_scales = oracle.encode(source, block, strict=False)
        payload, scales, _ = run_codec(source, block)
        assert_bits_equal(payload, expect_payload, f"payload block={block}")
        assert_bits_equal(scales, expect_scales, f"scales block={block}")


@pytest.mark.parametrize("block", (32, 64, 128, 96, 0))
def test_block_encode_fused_outputs(cuda, oracle, block):
    """64-bit-length encode with write-back, sum of squares and finite flag."""
    n = 70001
    source = vectors.config0_gradient(oracle, 1, n)
    expect_payload, expect_scales = oracle.encode(source, block, strict=False)
    expect_decoded = oracle.decode(expect_payload, expect_scales, block, strict=False)
    src = dev(source)
    payload = torch.zeros(n, dtype=torch.int8, device="cuda")
    scales = torch.zeros(scale_count(n, block), dtype=torch.float32, device="cuda")
    roundtrip = torch.zeros(n, dtype=torch.float32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    CudaBfp8Native.block_encode(0, src, payload, scales, block, roundtrip, sq, flag)
    torch.cuda.synchronize()
    assert_bits_equal(host(payload), expect_payload, "payload")
    assert_bits_equal(host(scales), expect_scales, "scales")
    assert_bits_equal(host(roundtrip), expect_decoded, "roundtrip")
    assert int(flag.item()) == 0
    expect_sq = oracle.squared_sum_bfp8(expect_payload, expect_scales, block)
    assert sq.item() == pytest.approx(expect_sq, rel=1e-12)
    # a NaN raises the flag
    source[123] = np.nan
    CudaBfp8Native.block_encode(0, dev(source), payload, scales, block, None, None, flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 1


def test_encode_decode_encode_is_idempotent_at_full_bucket_size(cuda):
    """Size-independent property at a 64 Mi-element bucket: re-encoding the
    decode reproduces the payload, and the scales up to the one rounding the
    format allows."""
    n = 64 << 20
    torch.manual_seed(7)
    src = torch.randn(n, device="cuda") * 1e-3
    payload = torch.empty(n, dtype=torch.int8, device="cuda")
    scales = torch.empty(n // 32, dtype=torch.float32, device="cuda")
    decoded = torch.empty(n, dtype=torch.float32, device="cuda")
    CudaBfp8Native.block_encode(0, src, payload, scales, 32)
    CudaBfp8Native.block_decode(0, payload, scales, decoded, 32)
    payload2 = torch.empty_like(payload)
    scales2 = torch.empty_like(scales)
    CudaBfp8Native.block_encode(0, decoded, payload2, scales2, 32)
    torch.cuda.synchronize()
    top0 = payload.view(-1, 32).to(torch.int16).abs().amax(dim=1)
    assert torch.equal(payload, payload2)
    # The second scale is the IEEE quotient of the decoded maximum, 127 * scale
    # (one binary32 multiply), by 127: equal to the first for most significands,
    # one unit in the last place away for the rest; all-zero blocks keep 1.
    # (computed with numpy: a tensor library may turn a division by a constant
    # into a multiplication by its reciprocal)
    first, top = host(scales), host(top0)
    expect2 = np.where(top == 0, np.float32(1.0), (first * np.float32(127.0)).astype(np.float32) / np.float32(127.0))
    assert_bits_equal(host(scales2), expect2.astype(np.float32), "second scales")
    assert bool(((scales2.view(torch.int32) - scales.view(torch.int32)).abs() <= 1).all())
    # |x - decode| <= scale/2 per block, scale = max/127
    err = (src - decoded).abs().view(-1, 32).amax(dim=1)
    assert bool((err <= scales * 0.50002).all())
    # a block's largest code is +-127 unless the block is all zero
    top = payload.view(-1, 32).to(torch.int16).abs().amax(dim=1)
    assert bool(((top == 127) | (scales == 1.0)).all())


@pytest.mark.parametrize("exponent_bits", (0x3F800000, 0x12800000, 0x71000000, 0x00800000, 0x7E800000))
def test_scale_is_the_ieee_quotient_for_every_significand(cuda, exponent_bits):
    """One block per binary32 significand (2^23 blocks), the block's only
    non-zero value being that significand at the given exponent: the stored
    scale must be the correctly rounded max / 127 for all of them, in the fast
    range and outside it."""
    count = 1 << 23
    bits = torch.arange(count, dtype=torch.int32, device="cuda") + exponent_bits
    maxima = bits.view(torch.float32)
    source = torch.zeros(count * 32, dtype=torch.float32, device="cuda")
    source[7::32] = -maxima
    payload = torch.empty(count * 32, dtype=torch.int8, device="cuda")
    scales = torch.empty(count, dtype=torch.float32, device="cuda")
    CudaBfp8Native.block_encode(0, source, payload, scales, 32)
    torch.cuda.synchronize()
    expect = host(maxima) / np.float32(127.0)
    assert_bits_equal(host(scales), expect, "scales")
    codes = host(payload[7::32])
    assert (codes == -127).all()


@pytest.mark.parametrize("n", (1, 33, 515, 4099, 300137))
@pytest.mark.parametrize("block", (0, 32, 64, 96, 128))
def test_bf16_source_codec_matches_the_fp32_rules_on_the_widened_value(cuda, oracle, n, block):
    # NNtrain.Cuda/native/cuda_runtime_bridge.cu:868-935 (encode), 769-806 (decode to bf16)
    bits = oracle.bf16_encode(vectors.codec_vector(n) if n <= 515 else vectors.config0_gradient(oracle, 0, n), 1)
    widened = oracle.bf16_decode(bits)
    expect_payload, expect_scales = oracle.encode(widened, block, strict=False)
    source = torch.from_numpy(bits.view(np.int16)).cuda()
    payload = torch.zeros(n, dtype=torch.int8, device="cuda")
    scales = torch.zeros(scale_count(n, block), dtype=torch.float32, device="cuda")
    CudaBfp8Native.quantize_bfloat16(0, source, payload, scales, block)
    back = torch.zeros(n, dtype=torch.int16, device="cuda")
    CudaBfp8Native.dequantize_bfloat16(0, payload, scales, back, block)
    torch.cuda.synchronize()
    assert_bits_equal(host(payload), expect_payload, "payload")
    assert_bits_equal(host(scales), expect_scales, "scales")
    expect_back = oracle.bf16_encode(oracle.decode(expect_payload, expect_scales, block, strict=False), 1)
    assert_bits_equal(host(back).view(np.uint16), expect_back, "bf16 decode")


def test_bf16_source_codec_on_misaligned_buffers(cuda, oracle):
    n, block = 70001, 32
    bits = oracle.bf16_encode(vectors.config0_gradient(oracle, 1, n), 1)
    source = misaligned(n, torch.int16, 1)
    source.copy_(torch.from_numpy(bits.view(np.int16)))
    payload = misaligned(n, torch.int8, 3)
    scales = torch.zeros(scale_count(n, block), dtype=torch.float32, device="cuda")
    CudaBfp8Native.quantize_bfloat16(0, source, payload, scales, block)
    back = misaligned(n, torch.int16, 1)
    CudaBfp8Native.dequantize_bfloat16(0, payload, scales, back, block)
    torch.cuda.synchronize()
    expect_payload, expect_scales = oracle.encode(oracle.bf16_decode(bits), block, strict=False)
    assert_bits_equal(host(payload), expect_payload, "payload")
    assert_bits_equal(host(scales), expect_scales, "scales")
    assert_bits_equal(host(back).view(np.uint16),
                      oracle.bf16_encode(oracle.decode(expect_payload, expect_scales, block, strict=False), 1), "bf16")
