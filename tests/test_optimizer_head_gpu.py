"""AdamW reading the reduced BFP8 gradient directly, against the reference's
adamw_kernel arithmetic (NNtrain.Cuda/native/tensor_kernels.cu:1148-1174) run
on the decoded gradient: bit-exact, every operation rounded separately."""
import numpy as np
import pytest
import torch

import vectors
from gpu_helpers import assert_bits_equal, dev, host, misaligned
from nntrain_b200.native import Bfp8GradientOptimizers

pytestmark = pytest.mark.gpu

HYPER = dict(beta1=0.9, beta2=0.95, learning_rate=3e-4, weight_decay=0.1, update_scale=2.9e-4,
             scaled_epsilon=1.1e-8)


@pytest.mark.parametrize("n", (1, 515, 70001, 1 << 20))
@pytest.mark.parametrize("block", (0, 32, 96, 128))
@pytest.mark.parametrize("decay", (True, False))
def test_adamw_head_equals_decode_then_adamw(cuda, oracle, n, block, decay):
    gradient = vectors.config0_gradient(oracle, 0, n)
    payload, scales = oracle.encode(gradient, block, strict=False)
    scales = oracle.scale_bfp8_scales(scales, 0.73)               # as left by the scale-only clip
    decoded = oracle.decode(payload, scales, block, strict=False)
    rng = np.random.default_rng(n + block)
    data = rng.standard_normal(n).astype(np.float32)
    first = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    second = (rng.random(n) * 1e-6).astype(np.float32)
    d_data, d_first, d_second = dev(data), dev(first), dev(second)
    compute = torch.zeros(n, dtype=torch.int16, device="cuda")
    for _ in range(2):                                              # two steps: the state carries over
        Bfp8GradientOptimizers.adamw(0, d_data, dev(payload), dev(scales), block, d_first, d_second,
                                     apply_weight_decay=decay, compute_bf16=compute, **HYPER)
        data, first, second = oracle.adamw_step(data, decoded, first, second, apply_weight_decay=decay, **HYPER)
    torch.cuda.synchronize()
    assert_bits_equal(host(d_first), first, "first moment")
    assert_bits_equal(host(d_second), second, "second moment")
    assert_bits_equal(host(d_data), data, "parameters")
    assert_bits_equal(host(compute).view(np.uint16), oracle.bf16_encode(data, 1), "bf16 working copy")


def test_adamw_head_on_misaligned_buffers(cuda, oracle):
    n, block = 4099, 32
    gradient = vectors.config0_gradient(oracle, 1, n)
    payload, scales = oracle.encode(gradient, block, strict=False)
    decoded = oracle.decode(payload, scales, block, strict=False)
    data = np.linspace(-1, 1, n).astype(np.float32)
    zeros = np.zeros(n, np.float32)
    d_data, d_first, d_second = misaligned(n, torch.float32, 1), misaligned(n, torch.float32, 3), misaligned(n, torch.float32, 2)
    d_data.copy_(torch.from_numpy(data))
    d_payload = misaligned(n, torch.int8, 1)
    d_payload.copy_(torch.from_numpy(payload))
    Bfp8GradientOptimizers.adamw(0, d_data, d_payload, dev(scales), block, d_first, d_second, **HYPER)
    torch.cuda.synchronize()
    want, first, second = oracle.adamw_step(data, decoded, zeros, zeros, **HYPER)
    assert_bits_equal(host(d_data), want, "parameters")
    assert_bits_equal(host(d_first), first, "first moment")
    assert_bits_equal(host(d_second), second, "second moment")
