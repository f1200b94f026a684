"""Live three-way comparison on the GPU: this library, the CPU oracle and the
reference project's own CUDA kernels (compiled unmodified).  Pins the oracle
to the reference where the reference's C# codec cannot run.  Inputs carry no
subnormals (the reference library flushes them under --use_fast_math)."""
import numpy as np
import pytest

import reference_kernels as rk
import vectors
from gpu_helpers import assert_bits_equal
from test_codec_gpu import run_codec

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def reference(cuda):
    if not rk.available():
        pytest.skip("oracle/_ref/libref_grad.so was not built (reference tree absent at build time)")
    return rk


@pytest.mark.parametrize("block", (0, 32, 96, 128))
@pytest.mark.parametrize("n", (515, 300137))
def test_codec_three_way(reference, oracle, block, n):
    source = vectors.codec_vector(n) if n < 1000 else vectors.tail_max_vector(n)
    ref_payload, ref_scales, ref_decoded = reference.codec(source, block)
    cpu_payload, cpu_scales = oracle.encode(source, block)
    assert_bits_equal(cpu_payload, ref_payload, "oracle payload vs reference kernel")
    assert_bits_equal(cpu_scales, ref_scales, "oracle scales vs reference kernel")
    assert_bits_equal(oracle.decode(cpu_payload, cpu_scales, block), ref_decoded, "oracle decode vs reference")
    payload, scales, decoded = run_codec(source, block)
    assert_bits_equal(payload, ref_payload, "library payload vs reference kernel")
    assert_bits_equal(scales, ref_scales, "library scales vs reference kernel")
    assert_bits_equal(decoded, ref_decoded, "library decode vs reference kernel")


def test_seeded_distribution_three_way(reference, oracle):
    source = oracle.generate_gradient(1 << 18, 0xB2000000, 0, subnormals=0)
    for block in (32, 128):
        ref_payload, ref_scales, _ = reference.codec(source, block)
        cpu_payload, cpu_scales = oracle.encode(source, block)
        assert_bits_equal(cpu_payload, ref_payload, f"oracle payload block={block}")
        assert_bits_equal(cpu_scales, ref_scales, f"oracle scales block={block}")


def test_transport_three_way(reference, oracle):
    a = oracle.generate_gradient(1 << 16, 0xB2000000, 0, subnormals=0)
    b = oracle.generate_gradient(1 << 16, 0xB2000000, 1, subnormals=0)
    a[777] = np.nan
    pa, sa = reference.pack_bfp8_block(a)
    pb, sb = reference.pack_bfp8_block(b)
    cpu_pa, cpu_sa = oracle.pack_bfp8_block(a, 128)
    assert_bits_equal(cpu_pa, pa, "pack payload")
    assert_bits_equal(cpu_sa, sa, "pack scales")
    reduced, sq = reference.block_transport_sum(pa, sa, pb, sb)
    cpu_reduced, cpu_sq = oracle.block_transport_sum([pa, pb], [sa, sb], 128)
    assert_bits_equal(cpu_reduced, reduced, "block transport sum")
    bits_a, bits_b = reference.pack_bf16(a), reference.pack_bf16(b)
    assert_bits_equal(oracle.bf16_encode(a, 1), bits_a, "bf16 pack")
    reduced16, _ = reference.bf16_transport_sum(bits_a, bits_b)
    assert_bits_equal(oracle.bf16_reduce([bits_a, bits_b])[0], reduced16, "bf16 transport sum")


@pytest.mark.parametrize("n", (1, 257, 515))
def test_gradient_publish_three_way(reference, oracle, n):
    source = vectors.reducer_vector(n, 0.0, 0.25, 2.75)
    g, payload, scale, flag, sq = reference.gradient_publish(source)
    cpu_g, cpu_payload, cpu_scale, cpu_flag, cpu_sq = oracle.gradient_publish(source, 0)
    assert flag == cpu_flag == 0
    assert_bits_equal(cpu_payload, payload, "payload")
    assert_bits_equal(cpu_scale, scale, "scale")
    assert_bits_equal(cpu_g, g, "decode cache")
    assert cpu_sq == pytest.approx(sq, rel=1e-12)
