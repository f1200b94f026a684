"""Checked wrappers over the C ABI, one per managed wrapper class of the
reference.  They validate device / dtype / length the way the managed wrappers
do, pass raw device pointers across the boundary, and turn a non-zero status
into NativeCudaError.  Tensors are torch CUDA tensors used purely as device
buffers.

  CudaBfp8Native          NNtrain.Core/Tensors/CudaBfp8Native.cs (QuantizeFloat32, ...)
  CudaBfp8GradientNative  NNtrain.Core/Tensors/CudaBfp8GradientNative.cs:10-237
  CudaGradientBuckets     NNtrain.Core/Tensors/CudaGradientBuckets.cs:6-349
  GradientNorm            the norm / clip kernels behind
                          NNtrain.Core/Tensors/Tensor.CudaKernels.cs:119-854
"""
from __future__ import annotations

import torch

from .library import check, load


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _require(t: torch.Tensor, dtype, name: str, device: int | None = None) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if device is not None and t.device.index != device:
        raise ValueError(f"{name} is on device {t.device.index}, expected {device}")


def scale_count(length: int, block_size: int) -> int:
    """Bfp8QuantizationDescriptor.GetScaleCount
    (NNtrain.Core/Tensors/Bfp8Quantization.cs:64-78); block_size 0 = tensor-wide."""
    block = max(1, length) if block_size <= 0 or block_size >= length else block_size
    return (length + block - 1) // block


class CudaBfp8Native:
    """Block / tensor-wide codec.  block_size 0 means tensor-wide."""

    @staticmethod
    def quantize_float32(device: int, source, payload, scales, block_size: int, stream=None) -> None:
        _require(source, torch.float32, "source", device)
        _require(payload, torch.int8, "payload", device)
        _require(scales, torch.float32, "scales", device)
        n = source.numel()
        if payload.numel() != n or scales.numel() != scale_count(n, block_size):
            raise ValueError("BFP8 payload / scale lengths do not match the descriptor")
        block = n if block_size <= 0 else block_size
        check("bfp8_quantize_f32", load().nntrain_cuda_bfp8_quantize_f32(
            device, _ptr(source), _ptr(payload), _ptr(scales), n, block, _stream(stream)))

    @staticmethod
    def dequantize_float32(device: int, payload, scales, destination, block_size: int, stream=None) -> None:
        _require(payload, torch.int8, "payload", device)
        _require(scales, torch.float32, "scales", device)
        _require(destination, torch.float32, "destination", device)
        n = payload.numel()
        if destination.numel() != n or scales.numel() != scale_count(n, block_size):
            raise ValueError("BFP8 payload / scale lengths do not match the descriptor")
        block = n if block_size <= 0 else block_size
        check("bfp8_dequantize_f32", load().nntrain_cuda_bfp8_dequantize_f32(
            device, _ptr(payload), _ptr(scales), _ptr(destination), n, block, _stream(stream)))

    @staticmethod
    def quantize_bfloat16(device: int, source_bits, payload, scales, block_size: int, stream=None) -> None:
        """`source_bits`: bf16 bit patterns (int16 tensor)."""
        _require(source_bits, torch.int16, "source", device)
        _require(payload, torch.int8, "payload", device)
        n = source_bits.numel()
        if payload.numel() != n or scales.numel() != scale_count(n, block_size):
            raise ValueError("BFP8 payload / scale lengths do not match the descriptor")
        check("cuda_bfp8_quantize_bf16", load().nntrain_cuda_bfp8_quantize_bf16(
            device, _ptr(source_bits), _ptr(payload), _ptr(scales), n, n if block_size <= 0 else block_size,
            _stream(stream)))

    @staticmethod
    def dequantize_bfloat16(device: int, payload, scales, destination_bits, block_size: int, stream=None) -> None:
        _require(destination_bits, torch.int16, "destination", device)
        n = payload.numel()
        if destination_bits.numel() != n or scales.numel() != scale_count(n, block_size):
            raise ValueError("BFP8 payload / scale lengths do not match the descriptor")
        check("cuda_bfp8_dequantize_bf16", load().nntrain_cuda_bfp8_dequantize_bf16(
            device, _ptr(payload), _ptr(scales), _ptr(destination_bits), n, n if block_size <= 0 else block_size,
            _stream(stream)))

    @staticmethod
    def quantize_float32_roundtrip(device: int, state, payload, scales, block_size: int, stream=None) -> None:
        _require(state, torch.float32, "state", device)
        _require(payload, torch.int8, "payload", device)
        _require(scales, torch.float32, "scales", device)
        n = state.numel()
        check("bfp8_quantize_f32_roundtrip", load().nntrain_cuda_bfp8_quantize_f32_roundtrip(
            device, _ptr(state), _ptr(payload), _ptr(scales), n, block_size, _stream(stream)))

    @staticmethod
    def block_encode(device: int, source, payload, scales, block_size: int, roundtrip=None,
                     squared_sum=None, finite_status=None, stream=None) -> None:
        """64-bit-length encode with optional fused write-back / sum of squares / finite flag."""
        _require(source, torch.float32, "source", device)
        _require(payload, torch.int8, "payload", device)
        _require(scales, torch.float32, "scales", device)
        n = source.numel()
        if payload.numel() < n or scales.numel() < scale_count(n, block_size):
            raise ValueError("BFP8 payload / scale buffers are too small")
        check("bfp8_block_encode", load().nntrain_bfp8_block_encode(
            device, _ptr(source), _ptr(payload), _ptr(scales), n, block_size, _ptr(roundtrip),
            _ptr(squared_sum), _ptr(finite_status), _stream(stream)))

    @staticmethod
    def block_decode(device: int, payload, scales, destination, block_size: int, stream=None) -> None:
        _require(payload, torch.int8, "payload", device)
        _require(destination, torch.float32, "destination", device)
        n = destination.numel()
        check("bfp8_block_decode", load().nntrain_bfp8_block_decode(
            device, _ptr(payload), _ptr(scales), _ptr(destination), n, block_size, _stream(stream)))


class CudaBfp8GradientNative:
    """Tensor-wide gradient publication and the 2-device reduce / broadcast."""

    @staticmethod
    def quantize(device: int, gradient, payload, scale, finite_status, squared_sum=None, stream=None) -> None:
        _require(gradient, torch.float32, "gradient", device)
        _require(payload, torch.int8, "payload", device)
        _require(scale, torch.float32, "scale", device)
        _require(finite_status, torch.int32, "finite_status", device)
        n = gradient.numel()
        if payload.numel() != n or scale.numel() != 1:
            raise ValueError("tensor-wide BFP8 gradient needs numel payload bytes and one scale")
        lib = load()
        if squared_sum is None:
            check("bfp8_gradient_quantize", lib.nntrain_bfp8_gradient_quantize(
                device, _ptr(gradient), _ptr(payload), _ptr(scale), n, _ptr(finite_status), _stream(stream)))
        else:
            _require(squared_sum, torch.float64, "squared_sum", device)
            check("bfp8_gradient_quantize_accumulate", lib.nntrain_bfp8_gradient_quantize_accumulate(
                device, _ptr(gradient), _ptr(payload), _ptr(scale), n, _ptr(finite_status),
                _ptr(squared_sum), _stream(stream)))

    @staticmethod
    def publish_tensors(device: int, arena, payload, scales, tensor_offsets, maxima_scratch, finite_status,
                        squared_sum=None, stream=None) -> None:
        """Every tensor of a bucket arena in three stream operations:
        `tensor_offsets` is a device int64 tensor of tensors + 1 ascending
        element offsets, `scales` / `maxima_scratch` have one entry per tensor."""
        _require(arena, torch.float32, "arena", device)
        _require(payload, torch.int8, "payload", device)
        _require(scales, torch.float32, "scales", device)
        _require(tensor_offsets, torch.int64, "tensor_offsets", device)
        _require(maxima_scratch, torch.int32, "maxima_scratch", device)
        tensors = tensor_offsets.numel() - 1
        if payload.numel() != arena.numel() or scales.numel() != tensors or maxima_scratch.numel() < tensors:
            raise ValueError("payload / scales / scratch sizes do not match the arena and the offset table")
        check("bfp8_gradient_publish_tensors", load().nntrain_bfp8_gradient_publish_tensors(
            device, _ptr(arena), _ptr(payload), _ptr(scales), _ptr(tensor_offsets), tensors, arena.numel(),
            _ptr(maxima_scratch), _ptr(finite_status), _ptr(squared_sum), _stream(stream)))

    @staticmethod
    def reduce_tensors(device: int, payloads, scales, reduced, out_payload, out_scales, tensor_offsets,
                       maxima_scratch, finite_status, reduction_scale: float = 1.0, squared_sum=None,
                       stream=None) -> None:
        import ctypes
        tensors = tensor_offsets.numel() - 1
        table_p = (ctypes.c_void_p * len(payloads))(*[_ptr(p) for p in payloads])
        table_s = (ctypes.c_void_p * len(scales))(*[_ptr(s) for s in scales])
        check("bfp8_gradient_reduce_tensors", load().nntrain_bfp8_gradient_reduce_tensors(
            device, len(payloads), table_p, table_s, _ptr(reduced), _ptr(out_payload), _ptr(out_scales),
            _ptr(tensor_offsets), tensors, reduced.numel(), reduction_scale, _ptr(maxima_scratch),
            _ptr(finite_status), _ptr(squared_sum), _stream(stream)))

    @staticmethod
    def decode_tensors(device: int, payload, scales, destination, tensor_offsets, skip_flag=None,
                       stream=None) -> None:
        check("bfp8_gradient_decode_tensors", load().nntrain_bfp8_gradient_decode_tensors(
            device, _ptr(payload), _ptr(scales), _ptr(destination), _ptr(tensor_offsets),
            tensor_offsets.numel() - 1, destination.numel(), _ptr(skip_flag), _stream(stream)))

    @staticmethod
    def accumulate_squared_sum(device: int, payload, scale, squared_sum, finite_status, stream=None) -> None:
        check("bfp8_gradient_squared_sum", load().nntrain_bfp8_gradient_squared_sum(
            device, _ptr(payload), _ptr(scale), payload.numel(), _ptr(squared_sum), _ptr(finite_status),
            _stream(stream)))

    @staticmethod
    def scale(device: int, scale, multiplier: float, stream=None) -> None:
        check("bfp8_gradient_scale", load().nntrain_bfp8_gradient_scale(
            device, _ptr(scale), multiplier, _stream(stream)))

    @staticmethod
    def reduce(primary: int, secondary: int, local_payload, local_scale, remote_payload, remote_scale,
               remote_payload_staging, remote_scale_staging, reduced, output_payload, output_scale,
               reduction_scale: float, finite_status, remote_finite_status, remote_status_staging,
               squared_sum, communication_stream: int, local_ready: int, remote_ready: int,
               reduced_ready: int) -> None:
        check("bfp8_gradient_reduce", load().nntrain_bfp8_gradient_reduce(
            primary, secondary, _ptr(local_payload), _ptr(local_scale), _ptr(remote_payload),
            _ptr(remote_scale), _ptr(remote_payload_staging), _ptr(remote_scale_staging), _ptr(reduced),
            _ptr(output_payload), _ptr(output_scale), reduced.numel(), reduction_scale,
            _ptr(finite_status), _ptr(remote_finite_status), _ptr(remote_status_staging),
            _ptr(squared_sum), communication_stream, local_ready, remote_ready, reduced_ready))

    @staticmethod
    def broadcast(destination: int, source: int, source_payload, source_scale, destination_payload,
                  destination_scale, destination_float, destination_finite_status,
                  destination_stream: int, source_ready: int) -> None:
        check("bfp8_gradient_broadcast", load().nntrain_bfp8_gradient_broadcast(
            destination, source, _ptr(source_payload), _ptr(source_scale), _ptr(destination_payload),
            _ptr(destination_scale), _ptr(destination_float), destination_float.numel(),
            _ptr(destination_finite_status), destination_stream, source_ready))


class CudaGradientBuckets:
    """Bucket transport between two devices of one process."""

    @staticmethod
    def create_communication_stream(device: int) -> int:
        import ctypes
        handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            check("gradient_comm_create", load().nntrain_gradient_comm_create(device, ctypes.addressof(handle)))
        return handle.value

    @staticmethod
    def create_ready_event(device: int) -> int:
        import ctypes
        handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            check("gradient_event_create", load().nntrain_gradient_event_create(device, ctypes.addressof(handle)))
        return handle.value

    @staticmethod
    def pack(device: int, source, destination_bf16, destination_offset: int, stream=None) -> None:
        _require(source, torch.float32, "source", device)
        check("gradient_pack_bf16", load().nntrain_gradient_pack_bf16(
            device, _ptr(source), _ptr(destination_bf16), destination_offset, source.numel(), _stream(stream)))

    @staticmethod
    def pack_bfp8_block(device: int, source, destination, scales, stream=None) -> None:
        _require(source, torch.float32, "source", device)
        _require(destination, torch.int8, "destination", device)
        check("gradient_pack_bfp8_block", load().nntrain_gradient_pack_bfp8_block(
            device, _ptr(source), _ptr(destination), _ptr(scales), source.numel(), _stream(stream)))

    @staticmethod
    def record_ready(device: int, event: int, stream=None, external: bool = False) -> None:
        fn = load().nntrain_gradient_record_ready_external if external else load().nntrain_gradient_record_ready
        check("gradient_record_ready", fn(device, event, _stream(stream)))

    @staticmethod
    def exchange(destination_device: int, source_device: int, local, remote_source, remote_staging, reduced,
                 squared_sum, communication_stream: int, local_ready: int, remote_ready: int) -> None:
        check("gradient_exchange_bf16", load().nntrain_gradient_exchange_bf16(
            destination_device, source_device, _ptr(local), _ptr(remote_source), _ptr(remote_staging),
            _ptr(reduced), reduced.numel(), _ptr(squared_sum), communication_stream, local_ready, remote_ready))

    @staticmethod
    def exchange_bfp8_block(destination_device: int, source_device: int, local, local_scales, remote_source,
                            remote_source_scales, remote_staging, remote_staging_scales, reduced, squared_sum,
                            communication_stream: int, local_ready: int, remote_ready: int) -> None:
        check("gradient_exchange_bfp8_block", load().nntrain_gradient_exchange_bfp8_block(
            destination_device, source_device, _ptr(local), _ptr(local_scales), _ptr(remote_source),
            _ptr(remote_source_scales), _ptr(remote_staging), _ptr(remote_staging_scales), _ptr(reduced),
            reduced.numel(), _ptr(squared_sum), communication_stream, local_ready, remote_ready))

    @staticmethod
    def create_host_pipeline(source_device: int, destination_device: int, chunk_elements: int,
                             bfp8_block: bool = False) -> int:
        """The pinned-host fallback for a device pair without peer access."""
        import ctypes
        handle = ctypes.c_void_p()
        fn = (load().nntrain_gradient_host_pipeline_create_bfp8_block if bfp8_block
              else load().nntrain_gradient_host_pipeline_create)
        check("gradient_host_pipeline_create", fn(source_device, destination_device, chunk_elements,
                                                  ctypes.addressof(handle)))
        return handle.value

    @staticmethod
    def host_pipeline_exchange(pipeline: int, local, remote_source, reduced, squared_sum, local_ready: int,
                               remote_ready: int) -> None:
        check("gradient_host_pipeline_exchange_bf16", load().nntrain_gradient_host_pipeline_exchange_bf16(
            pipeline, _ptr(local), _ptr(remote_source), _ptr(reduced), reduced.numel(), _ptr(squared_sum),
            local_ready, remote_ready))

    @staticmethod
    def host_pipeline_exchange_bfp8_block(pipeline: int, local, local_scales, remote_source, remote_source_scales,
                                          reduced, squared_sum, local_ready: int, remote_ready: int) -> None:
        check("gradient_host_pipeline_exchange_bfp8_block",
              load().nntrain_gradient_host_pipeline_exchange_bfp8_block(
                  pipeline, _ptr(local), _ptr(local_scales), _ptr(remote_source), _ptr(remote_source_scales),
                  _ptr(reduced), reduced.numel(), _ptr(squared_sum), local_ready, remote_ready))

    @staticmethod
    def destroy_host_pipeline(pipeline: int) -> None:
        check("gradient_host_pipeline_destroy", load().nntrain_gradient_host_pipeline_destroy(pipeline))

    @staticmethod
    def unpack(device: int, source, source_offset: int, destination, communication_stream: int) -> None:
        check("gradient_unpack_float", load().nntrain_gradient_unpack_float(
            device, _ptr(source), source_offset, _ptr(destination), destination.numel(), communication_stream))

    @staticmethod
    def synchronize(device: int, communication_stream: int) -> None:
        check("gradient_comm_synchronize", load().nntrain_gradient_comm_synchronize(device, communication_stream))

    @staticmethod
    def destroy_event(device: int, event: int) -> None:
        check("gradient_event_destroy", load().nntrain_gradient_event_destroy(device, event))

    @staticmethod
    def destroy_communication_stream(device: int, stream: int) -> None:
        check("gradient_comm_destroy", load().nntrain_gradient_comm_destroy(device, stream))


class GradientNorm:
    """Sum of squares and clip kernels (kinds: 0 fp32, 1 bf16, 2 BFP8)."""

    FP32, BF16, BFP8 = 0, 1, 2

    @staticmethod
    def squared_sum(device: int, kind: int, values, squared_sum, scales=None, block_size: int = 0,
                    finite_status=None, stream=None) -> None:
        _require(squared_sum, torch.float64, "squared_sum", device)
        check("gradient_squared_sum", load().nntrain_gradient_squared_sum(
            device, kind, _ptr(values), _ptr(scales), values.numel(), block_size, _ptr(squared_sum),
            _ptr(finite_status), _stream(stream)))

    @staticmethod
    def clip_coefficient(device: int, squared_sum, max_norm: float, norm_and_coefficient, stream=None) -> None:
        check("gradient_clip_coefficient", load().nntrain_gradient_clip_coefficient(
            device, _ptr(squared_sum), max_norm, _ptr(norm_and_coefficient), _stream(stream)))

    @staticmethod
    def clip_apply(device: int, kind: int, values, multiplier: float = 1.0, coefficient=None, stream=None) -> None:
        check("gradient_clip_apply", load().nntrain_gradient_clip_apply(
            device, kind, _ptr(values), values.numel(), multiplier, _ptr(coefficient), _stream(stream)))


class Bfp8GradientOptimizers:
    """Optimizer heads that read the reduced BFP8 gradient without a decode pass."""

    @staticmethod
    def adamw(device: int, data, gradient_payload, gradient_scales, block_size: int, first_moment, second_moment,
              beta1: float, beta2: float, learning_rate: float, weight_decay: float, update_scale: float,
              scaled_epsilon: float, apply_weight_decay: bool = True, compute_bf16=None, stream=None) -> None:
        for name, t in (("data", data), ("first_moment", first_moment), ("second_moment", second_moment)):
            _require(t, torch.float32, name, device)
        _require(gradient_payload, torch.int8, "gradient_payload", device)
        n = data.numel()
        if (gradient_payload.numel() != n or first_moment.numel() != n or second_moment.numel() != n
                or gradient_scales.numel() != scale_count(n, block_size)):
            raise ValueError("parameter, moment and gradient sizes do not match")
        check("optimizer_adamw_bfp8_gradient", load().nntrain_optimizer_adamw_bfp8_gradient(
            device, _ptr(data), _ptr(gradient_payload), _ptr(gradient_scales), block_size, _ptr(first_moment),
            _ptr(second_moment), _ptr(compute_bf16), n, beta1, beta2, learning_rate, weight_decay, update_scale,
            scaled_epsilon, int(apply_weight_decay), _stream(stream)))
