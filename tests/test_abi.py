"""The C-ABI library: it loads, exports every symbol the header declares, and
rejects bad arguments before touching a device."""
import ctypes
import os
import subprocess

from nntrain_b200 import build as builder
from nntrain_b200.library import ErrorInfo, declared_functions

# Hot-path exports the reference's managed gateway requires
# (NNtrain.Core.Tests/CudaNativeAbiGatewayTests.cs:127-156,244-294).
REQUIRED = """
nntrain_abi_version nntrain_last_error nntrain_error_snapshot nntrain_capability_bitmap
nntrain_cuda_set_device nntrain_cuda_use_external_stream
nntrain_cuda_bfp8_quantize_f32 nntrain_cuda_bfp8_dequantize_f32 nntrain_cuda_bfp8_quantize_f32_roundtrip
nntrain_bfp8_gradient_quantize nntrain_bfp8_gradient_quantize_accumulate nntrain_bfp8_gradient_squared_sum
nntrain_bfp8_gradient_scale nntrain_bfp8_gradient_reduce nntrain_bfp8_gradient_broadcast
nntrain_gradient_comm_create nntrain_gradient_event_create nntrain_gradient_pack_bf16
nntrain_gradient_pack_bfp8_block nntrain_gradient_record_ready nntrain_gradient_record_ready_external
nntrain_gradient_exchange_bf16 nntrain_gradient_exchange_bfp8_block nntrain_gradient_host_pipeline_create
nntrain_gradient_host_pipeline_create_bfp8_block nntrain_gradient_host_pipeline_exchange_bf16
nntrain_gradient_host_pipeline_exchange_bfp8_block nntrain_gradient_host_pipeline_destroy
nntrain_gradient_unpack_float nntrain_gradient_comm_synchronize nntrain_gradient_event_destroy
nntrain_gradient_comm_destroy nntrain_tensor_squared_sum nntrain_tensor_scale nntrain_tensor_encode_bf16
nntrain_tensor_decode_bf16 nntrain_tensor_bf16_gradient_squared_sum nntrain_tensor_bf16_gradient_scale
""".split()


def test_library_exports_every_declared_symbol(lib):
    declared = declared_functions()
    assert set(REQUIRED) <= set(declared)
    for name in declared:
        assert getattr(lib, name) is not None
    listing = subprocess.run(["nm", "-D", "--defined-only", builder.LIBRARY],
                             capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in listing.splitlines() if " T nntrain_" in line}
    assert exported == set(declared), (sorted(exported - set(declared)), sorted(set(declared) - exported))


def test_abi_version_is_major_1_minor_36(lib):
    version = lib.nntrain_abi_version()
    assert version >> 16 == 1 and version & 0xFFFF == 36


def test_invalid_arguments_return_invalid_value_without_a_device(lib):
    invalid = 1  # cudaErrorInvalidValue
    assert lib.nntrain_cuda_bfp8_quantize_f32(0, None, None, None, 16, 32, None) == invalid
    assert lib.nntrain_cuda_bfp8_quantize_f32(0, 8, 8, 8, 0, 32, None) == invalid
    assert lib.nntrain_cuda_bfp8_dequantize_f32(0, 8, 8, 8, 16, 0, None) == invalid
    # the roundtrip export rejects the tensor-wide case (block >= length)
    assert lib.nntrain_cuda_bfp8_quantize_f32_roundtrip(0, 8, 8, 8, 32, 32, None) == invalid
    assert lib.nntrain_bfp8_gradient_quantize(-1, 8, 8, 8, 4, 8, None) == invalid
    assert lib.nntrain_bfp8_gradient_scale(0, 8, float("nan"), None) == invalid
    assert lib.nntrain_bfp8_gradient_scale(0, 8, 0.0, None) == invalid
    assert lib.nntrain_gradient_pack_bf16(0, 8, 8, -1, 4, None) == invalid
    assert lib.nntrain_gradient_host_pipeline_create(0, 0, 1024, None) == invalid
    assert lib.nntrain_gradient_host_pipeline_create_bfp8_block(0, 1, 100, 8) == invalid
    assert lib.nntrain_tensor_squared_sum(None, 4, None) == invalid
    assert lib.nntrain_gradient_clip_coefficient(0, 8, -1.0, 8, None) == invalid
    assert lib.nntrain_bfp8_gradient_reduce(0, 0, *([8] * 9), 4, 1.0, *([8] * 8)) == invalid


def test_failed_calls_land_in_the_error_ring(lib):
    lib.nntrain_cuda_bfp8_quantize_f32(3, None, None, None, 16, 32, None)
    info = ErrorInfo()
    assert lib.nntrain_last_error(ctypes.addressof(info), ctypes.sizeof(info)) == 0
    assert info.struct_size == ctypes.sizeof(ErrorInfo) == 32
    assert info.status == 1 and info.device == 3 and info.operation == 26
    found = ErrorInfo()
    assert lib.nntrain_error_snapshot(1, 3, 26, ctypes.addressof(found), ctypes.sizeof(found)) == 0
    assert found.sequence == info.sequence
    assert lib.nntrain_error_snapshot(77, 3, 26, ctypes.addressof(found), ctypes.sizeof(found)) == 1
    assert lib.nntrain_last_error(None, 0) == 1


def test_every_declaration_carries_a_comment_and_the_header_cites_the_reference():
    import re
    include = os.path.join(os.path.dirname(builder.__file__), "..", "include")
    text = open(os.path.join(include, "nntrain_grad_abi.h")).read() + open(os.path.join(include, "nntrain_host_plan.h")).read()
    for name in declared_functions():
        before = text[:text.index(name + "(")]
        last_statement = max(before.rfind(";"), before.rfind("{"))
        assert "*/" in before[last_statement:], f"{name} has no comment of its own"
    assert len(re.findall(r"\.(?:cu|cs):\d+", text)) >= 45
