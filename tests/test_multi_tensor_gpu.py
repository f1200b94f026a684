"""Whole-bucket launches of the tensor-wide reducer: every tensor of a bucket
published / reduced / decoded by one launch train, against per-tensor oracle
results (what one `nntrain_bfp8_gradient_quantize_accumulate` per tensor gives;
NNtrain.Cuda/native/tensor_kernels.cu:1114-1146,3935-4038)."""
import numpy as np
import pytest
import torch

from gpu_helpers import assert_bits_equal, dev, host
from nntrain_b200.native import CudaBfp8GradientNative

pytestmark = pytest.mark.gpu


def qwen2_1p5b_numels(hidden=1536, layers=28, kv=256, intermediate=8960, vocab=151936):
    numels = [vocab * hidden]
    for _ in range(layers):
        numels += [hidden * hidden, hidden, hidden * kv, kv, hidden * kv, kv, hidden * hidden,
                   hidden * intermediate, hidden * intermediate, intermediate * hidden, hidden, hidden]
    return numels + [hidden]


def publish(numels, flat, squared=True):
    offsets = np.concatenate([[0], np.cumsum(numels)]).astype(np.int64)
    arena = dev(flat)
    payload = torch.zeros(arena.numel(), dtype=torch.int8, device="cuda")
    scales = torch.zeros(len(numels), dtype=torch.float32, device="cuda")
    scratch = torch.full((len(numels),), -1, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda") if squared else None
    CudaBfp8GradientNative.publish_tensors(0, arena, payload, scales, dev(offsets), scratch, flag, sq)
    torch.cuda.synchronize()
    return arena, payload, scales, flag, sq, offsets


def check_against_per_tensor_oracle(oracle, numels, flat, arena, payload, scales, sq, offsets):
    got_arena, got_payload, got_scales = host(arena), host(payload), host(scales)
    total = 0.0
    for t in range(len(numels)):
        a, b = offsets[t], offsets[t + 1]
        g, p, s, flag, squares = oracle.gradient_publish(flat[a:b], 0)
        assert flag == 0
        assert_bits_equal(got_payload[a:b], p, f"payload of tensor {t}")
        assert_bits_equal(got_scales[t:t + 1], s, f"scale of tensor {t}")
        assert_bits_equal(got_arena[a:b], g, f"write-back of tensor {t}")
        total += squares
    if sq is not None:
        assert sq.item() == pytest.approx(total, rel=1e-12)


@pytest.mark.parametrize("numels", (
    [1], [515], [127, 1, 128, 129, 3, 4096, 4097, 31, 100000, 2, 2, 2, 5000],
    [4096] * 7, [300137, 17, 33, 257]))
def test_publish_tensors_matches_one_publication_per_tensor(cuda, oracle, numels):
    flat = oracle.generate_gradient(sum(numels), 0xB2000021, 0)
    flat[:1] = 0.0
    arena, payload, scales, flag, sq, offsets = publish(numels, flat)
    assert int(flag.item()) == 0
    check_against_per_tensor_oracle(oracle, numels, flat, arena, payload, scales, sq, offsets)


def test_an_all_zero_tensor_keeps_scale_one(cuda, oracle):
    numels = [1000, 640, 77]
    flat = oracle.generate_gradient(sum(numels), 5, 0)
    flat[1000:1640] = 0.0
    arena, payload, scales, flag, sq, offsets = publish(numels, flat)
    assert host(scales)[1] == 1.0 and not host(payload)[1000:1640].any()
    check_against_per_tensor_oracle(oracle, numels, flat, arena, payload, scales, sq, offsets)


def test_a_non_finite_value_publishes_nothing(cuda, oracle):
    numels = [5000, 300, 9000]
    flat = oracle.generate_gradient(sum(numels), 6, 0)
    flat[5100] = np.inf
    arena, payload, scales, flag, sq, offsets = publish(numels, flat)
    assert int(flag.item()) == 1
    assert (host(scales) == 1.0).all() and not host(payload).any()
    assert_bits_equal(host(arena), flat, "gradient left as it was")
    assert sq.item() == 0.0


def test_qwen2_1p5b_tensor_list(cuda, oracle):
    """The full 1,543,714,304-value tensor list (338 tensors) in one launch
    train, every tensor compared with its own oracle publication."""
    numels = qwen2_1p5b_numels()
    assert sum(numels) == 1_543_714_304 and len(numels) == 338
    flat = oracle.generate_gradient(sum(numels), 0xB2000004, 0)
    arena, payload, scales, flag, sq, offsets = publish(numels, flat)
    assert int(flag.item()) == 0
    check_against_per_tensor_oracle(oracle, numels, flat, arena, payload, scales, sq, offsets)


@pytest.mark.parametrize("inputs", (2, 3))
def test_reduce_tensors_and_decode_tensors(cuda, oracle, inputs):
    numels = [4099, 33, 1, 20000, 517, 16384, 7, 9001]
    total = sum(numels)
    offsets = np.concatenate([[0], np.cumsum(numels)]).astype(np.int64)
    flats = [oracle.generate_gradient(total, 0xB2000022, r) for r in range(inputs)]
    published = [publish(numels, f, squared=False) for f in flats]
    scale = 1.0 / inputs
    reduced = torch.zeros(total, dtype=torch.float32, device="cuda")
    out_payload = torch.zeros(total, dtype=torch.int8, device="cuda")
    out_scales = torch.zeros(len(numels), dtype=torch.float32, device="cuda")
    scratch = torch.zeros(len(numels), dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    device_offsets = dev(offsets)
    CudaBfp8GradientNative.reduce_tensors(0, [p[1] for p in published], [p[2] for p in published], reduced,
                                          out_payload, out_scales, device_offsets, scratch, flag, scale, sq)
    replica = torch.zeros(total, dtype=torch.float32, device="cuda")
    CudaBfp8GradientNative.decode_tensors(0, out_payload, out_scales, replica, device_offsets, flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    expect_sq = 0.0
    for t in range(len(numels)):
        a, b = offsets[t], offsets[t + 1]
        encoded = [oracle.encode(f[a:b], 0) for f in flats]
        r, bad = oracle.reduce_bfp8([e[0] for e in encoded], [e[1] for e in encoded], 0, scale)
        assert bad == 0
        p, s = oracle.encode(r, 0)
        final = oracle.decode(p, s, 0)
        assert_bits_equal(host(out_payload)[a:b], p, f"reduced payload of tensor {t}")
        assert_bits_equal(host(out_scales)[t:t + 1], s, f"reduced scale of tensor {t}")
        assert_bits_equal(host(reduced)[a:b], final, f"fp32 on the primary, tensor {t}")
        assert_bits_equal(host(replica)[a:b], final, f"fp32 on the receiving side, tensor {t}")
        expect_sq += oracle.squared_sum_bfp8(p, s, 0)
    assert sq.item() == pytest.approx(expect_sq, rel=1e-12)
    # an invalid input scale fails the bucket closed
    published[1][2][3] = float("nan")
    flag.zero_()
    CudaBfp8GradientNative.reduce_tensors(0, [p[1] for p in published], [p[2] for p in published], reduced,
                                          out_payload, out_scales, device_offsets, scratch, flag, scale, sq)
    torch.cuda.synchronize()
    assert int(flag.item()) == 1 and (host(out_scales) == 1.0).all()
