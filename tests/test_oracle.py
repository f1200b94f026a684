"""The CPU oracle against the reference's own known-answer assertions and the
committed golden fixtures (outputs of the reference's CUDA kernels)."""
import glob
import os

import numpy as np
import pytest

import vectors

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_tensor_wide_uses_one_scale(oracle):
    # NNtrain.Core.Tests/Bfp8QuantizationTests.cs:26-51
    source = np.array([-4, -1, 0, 0.75, 3], np.float32)
    payload, scales = oracle.encode(source, 0)
    assert scales.shape == (1,)
    assert scales[0] == np.float32(4) / np.float32(127)
    assert payload.tolist() == [-127, -32, 0, 24, 95]
    decoded = oracle.decode(payload, scales, 0)
    assert np.all(np.abs(decoded - source) <= scales[0] * np.float32(0.501))
    assert (payload < 0).any() and (payload > 0).any()


def test_mix8_uses_block_128(oracle):
    # NNtrain.Core.Tests/Bfp8QuantizationTests.cs:53-67: 300 values -> 3 scales
    payload, scales = oracle.encode(vectors.mix8_vector(300), 128)
    assert scales.shape == (3,) and payload.shape == (300,)
    assert oracle.scale_count(300, 128) == 3
    assert oracle.scale_count(5, 0) == 1


def test_zero_blocks_have_unit_scale(oracle):
    # NNtrain.Core.Tests/Bfp8QuantizationTests.cs:91-101
    payload, scales = oracle.encode(np.zeros(257, np.float32), 128)
    assert scales.tolist() == [1.0, 1.0, 1.0]
    assert not payload.any()


def test_encode_rejects_non_finite_like_the_cpu_codec(oracle):
    # NNtrain.Core/Tensors/Bfp8Quantization.cs:206-211
    bad = vectors.codec_vector(64)
    bad[5] = np.nan
    with pytest.raises(oracle.OracleError):
        oracle.encode(bad, 32)
    payload, _ = oracle.encode(bad, 32, strict=False)   # device semantics: NaN -> code 0
    assert payload[5] == 0


def test_round_half_even_and_clamp(oracle):
    # scale = 127/127 = 1: quotients equal the values
    source = np.array([127, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, -126.5], np.float32)
    payload, scales = oracle.encode(source, 0)
    assert scales[0] == 1.0
    assert payload.tolist() == [127, 0, 2, 2, 0, -2, -2, 126, -126]


def test_decode_is_one_multiply(oracle):
    source = vectors.codec_vector(515)
    for block in vectors.REFERENCE_BLOCKS:
        payload, scales = oracle.encode(source, block)
        eb = 515 if block == 0 else block
        expect = payload.astype(np.float32) * np.repeat(scales, eb)[:515]
        assert np.array_equal(oracle.decode(payload, scales, block), expect)


def test_two_replica_reduce_matches_the_reference_tests_formula(oracle):
    # Encode(Decode(Encode a) + Decode(Encode b))
    # NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:44-51
    for n in (1, 257, 515):
        a = vectors.reducer_vector(n, 0.0, 0.25, 2.75)
        b = vectors.reducer_vector(n, 11.0, 0.5, 3.25)
        pa, sa = oracle.encode(a, 0)
        pb, sb = oracle.encode(b, 0)
        expect_sum = oracle.decode(pa, sa, 0) + oracle.decode(pb, sb, 0)
        expect_payload, expect_scales = oracle.encode(expect_sum, 0)
        payload, scales, final, sq = oracle.allreduce_bfp8([a, b], 0, 1.0)
        assert np.array_equal(payload, expect_payload) and np.array_equal(scales, expect_scales)
        assert np.array_equal(final, oracle.decode(expect_payload, expect_scales, 0))
        assert sq == pytest.approx(float(np.sum(final.astype(np.float64) ** 2)), rel=1e-12)


def test_reduction_scale_applies_to_the_finished_sum(oracle):
    a = vectors.config0_gradient(oracle, 0, 4096)
    b = vectors.config0_gradient(oracle, 1, 4096)
    ea, eb = oracle.encode(a, 32, strict=False), oracle.encode(b, 32, strict=False)
    r, flag = oracle.reduce_bfp8([ea[0], eb[0]], [ea[1], eb[1]], 32, 0.5)
    expect = np.float32(0.5) * (oracle.decode(*ea, 32, strict=False) + oracle.decode(*eb, 32, strict=False))
    assert flag == 0 and np.array_equal(r, expect)


def test_bf16_round_to_nearest_even(oracle):
    # NNtrain.Core/Tensors/TensorStorage.cs:758-767
    values = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, np.inf, 1e-40], np.float32)
    bits = values.view(np.uint32)
    expect = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(oracle.bf16_encode(values, 0), expect)
    assert np.array_equal(oracle.bf16_encode(values, 1), expect)
    nan = np.array([np.nan], np.float32)
    assert oracle.bf16_encode(nan, 0)[0] == ((nan.view(np.uint32)[0] >> 16) | 0x40)
    assert oracle.bf16_encode(nan, 1)[0] == 0x7FFF
    assert np.array_equal(oracle.bf16_decode(expect).view(np.uint32), expect.astype(np.uint32) << 16)


def test_clip_matches_the_cpu_reference(oracle):
    # NNtrain.Core/Torch/nn.cs:62-81
    g = vectors.config0_gradient(oracle, 0, 1 << 16)
    sq = oracle.squared_sum_f32(g)
    assert sq == pytest.approx(float(np.sum(g.astype(np.float64) ** 2)), rel=1e-12)
    norm, c = oracle.clip_coefficient(sq, 1.0)
    assert norm == np.float32(np.sqrt(sq))
    if norm > 1.0:
        assert c == np.float32(1.0) / (np.float32(norm) + np.float32(1e-6))
    norm2, c2 = oracle.clip_coefficient(1e-6, 1.0)
    assert c2 == 1.0 and norm2 == np.float32(1e-3)
    scales = np.array([1e-3, 1e-38, 5.0], np.float32)
    clipped = oracle.scale_bfp8_scales(scales, 1e-3)
    assert clipped[1] == np.finfo(np.float32).tiny            # fmaxf(scale*c, FLT_MIN)
    assert clipped[0] == np.float32(1e-3) * np.float32(1e-3)


def test_pack_bfp8_block_poisons_non_finite_blocks(oracle):
    # NNtrain.Cuda/native/gradient_collectives.cu:49-58
    g = vectors.codec_vector(515)
    g[130] = np.inf
    payload, scales = oracle.pack_bfp8_block(g, 128)
    assert scales.view(np.uint32)[1] == 0x7FFFFFFF and not payload[128:256].any()
    clean, clean_scales = oracle.encode(vectors.codec_vector(515), 128)
    assert np.array_equal(payload[:128], clean[:128]) and scales[0] == clean_scales[0]
    assert np.array_equal(payload[256:], clean[256:])


def test_generator_is_counter_based(oracle):
    whole = oracle.generate_gradient(1 << 16, 0xB2000000, 1, total_length=1 << 16)
    part = oracle.generate_gradient(1 << 12, 0xB2000000, 1, offset=3 << 12, total_length=1 << 16)
    assert np.array_equal(whole[3 << 12:4 << 12], part)
    assert not np.array_equal(whole, oracle.generate_gradient(1 << 16, 0xB2000000, 0, total_length=1 << 16))


def test_threads_do_not_change_results(oracle):
    g = vectors.config0_gradient(oracle, 0, 1 << 16)
    oracle.set_threads(1)
    one = oracle.encode(g, 32, strict=False)
    oracle.set_threads(oracle.max_threads())
    many = oracle.encode(g, 32, strict=False)
    oracle.set_threads(1)
    assert np.array_equal(one[0], many[0]) and np.array_equal(one[1], many[1])


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "*.npz"))) or [None])
def test_oracle_matches_reference_kernel_outputs(oracle, path):
    """Fixtures recorded from the reference's own CUDA kernels (compiled
    unmodified) by tests/golden/make_golden.py."""
    if path is None:
        pytest.skip("no golden fixtures committed yet")
    data = np.load(path)
    kind = str(data["kind"])
    if kind == "codec":
        payload, scales = oracle.encode(data["source"], int(data["block"]), strict=False)
        assert np.array_equal(payload, data["payload"])
        assert np.array_equal(scales.view(np.uint32), data["scales"].view(np.uint32))
        decoded = oracle.decode(payload, scales, int(data["block"]), strict=False)
        assert np.array_equal(decoded.view(np.uint32), data["decoded"].view(np.uint32))
    elif kind == "pack_bfp8_block":
        payload, scales = oracle.pack_bfp8_block(data["source"], 128)
        assert np.array_equal(payload, data["payload"])
        assert np.array_equal(scales.view(np.uint32), data["scales"].view(np.uint32))
    elif kind == "block_transport_sum":
        reduced, sq = oracle.block_transport_sum([data["payload0"], data["payload1"]],
                                                 [data["scales0"], data["scales1"]], 128)
        assert np.array_equal(reduced.view(np.uint32), data["reduced"].view(np.uint32))
        assert sq == pytest.approx(float(data["squared_sum"]), rel=1e-12)
    elif kind == "bf16_transport_sum":
        reduced, _, sq = oracle.bf16_reduce([data["a"], data["b"]])
        assert np.array_equal(reduced.view(np.uint32), data["reduced"].view(np.uint32))
        assert sq == pytest.approx(float(data["squared_sum"]), rel=1e-12)
    elif kind == "pack_bf16":
        assert np.array_equal(oracle.bf16_encode(data["source"], 1), data["packed"])
    elif kind == "gradient_publish":
        g, payload, scales, flag, sq = oracle.gradient_publish(data["source"], 0)
        assert np.array_equal(payload, data["payload"])
        assert np.array_equal(scales.view(np.uint32), data["scale"].view(np.uint32))
        assert np.array_equal(g.view(np.uint32), data["gradient_after"].view(np.uint32))
        assert flag == int(data["finite_status"])
        assert sq == pytest.approx(float(data["squared_sum"]), rel=1e-12)
    else:
        pytest.fail(f"unknown fixture kind {kind}")
