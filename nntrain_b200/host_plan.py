"""Python face of the host-side reducer bookkeeping in the library
(include/nntrain_host_plan.h): bucket layout, the exactly-once publication
state machine and the per-rank step plan with reduction stamps and the
optimizer guard.  Names follow the reference's managed classes
(NNtrain.Core/Training/CudaCapturedGradientPublicationState.cs,
CudaGradientCoherence.cs, CudaBFloat16GradientAllReduce.cs)."""
from __future__ import annotations

import ctypes

from .library import load

INVALID_OPERATION = 3000


class InvalidOperationError(RuntimeError):
    """The managed code's InvalidOperationException."""


class ArgumentError(ValueError):
    """The managed code's ArgumentException family."""


def _message() -> str:
    buffer = ctypes.create_string_buffer(512)
    load().nntrain_host_last_message(buffer, 512)
    return buffer.value.decode()


def _check(status: int) -> None:
    if status == 0:
        return
    if status == INVALID_OPERATION:
        raise InvalidOperationError(_message())
    raise ArgumentError(_message())


def build_buckets(numels, target_elements: int):
    """[(bucket, offset)] per tensor and the bucket count."""
    count = len(numels)
    lengths = (ctypes.c_longlong * count)(*numels)
    bucket_of = (ctypes.c_int * count)()
    offset_of = (ctypes.c_longlong * count)()
    buckets = ctypes.c_int()
    _check(load().nntrain_plan_build_buckets(lengths, count, target_elements, bucket_of, offset_of,
                                             ctypes.addressof(buckets)))
    return list(zip(bucket_of, offset_of)), buckets.value


class CapturedGradientPublicationState:
    def __init__(self, device_count: int):
        handle = ctypes.c_void_p()
        _check(load().nntrain_publication_state_create(device_count, ctypes.addressof(handle)))
        self._handle = handle.value

    def __del__(self):
        if getattr(self, "_handle", None):
            load().nntrain_publication_state_destroy(self._handle)
            self._handle = None

    def begin_step(self, step): _check(load().nntrain_publication_begin_step(self._handle, step))
    def mark_device_begun(self, step, slot, device): _check(load().nntrain_publication_mark_device_begun(self._handle, step, slot, device))
    def enter_notification_path(self, step, slot, device): _check(load().nntrain_publication_enter_notification_path(self._handle, step, slot, device))
    def begin_capture_recording(self, step, slot, device): _check(load().nntrain_publication_begin_capture_recording(self._handle, step, slot, device))

    def is_capture_recording(self, step, slot) -> bool:
        flag = ctypes.c_int()
        _check(load().nntrain_publication_is_capture_recording(self._handle, step, slot, ctypes.addressof(flag)))
        return bool(flag.value)

    def enter_capture_notification_path(self, step, slot, device): _check(load().nntrain_publication_enter_capture_notification_path(self._handle, step, slot, device))
    def end_capture_recording(self, step, slot, device): _check(load().nntrain_publication_end_capture_recording(self._handle, step, slot, device))
    def validate_capture_discard(self, step): _check(load().nntrain_publication_validate_capture_discard(self._handle, step))
    def begin_captured_publication(self, step, slot, device): _check(load().nntrain_publication_begin_captured_publication(self._handle, step, slot, device))
    def complete_captured_publication(self, step, slot, device): _check(load().nntrain_publication_complete_captured_publication(self._handle, step, slot, device))
    def fail_captured_publication(self, step, slot): _check(load().nntrain_publication_fail_captured_publication(self._handle, step, slot))
    def validate_complete(self, step): _check(load().nntrain_publication_validate_complete(self._handle, step))
    def end_step(self, step): _check(load().nntrain_publication_end_step(self._handle, step))


HOST, LOCAL, REDUCED = 0, 1, 2


class GradientStepPlan:
    """One rank's reducer bookkeeping over a list of tensor lengths."""

    def __init__(self, numels, devices, target_bucket_elements: int = 4 << 20, block_size: int = 32):
        count = len(numels)
        handle = ctypes.c_void_p()
        _check(load().nntrain_plan_create((ctypes.c_longlong * count)(*numels), count, target_bucket_elements,
                                          (ctypes.c_int * len(devices))(*devices), len(devices), block_size,
                                          ctypes.addressof(handle)))
        self._handle = handle.value
        self.devices = list(devices)

    def close(self):
        if getattr(self, "_handle", None):
            load().nntrain_plan_destroy(self._handle)
            self._handle = None

    __del__ = close

    @property
    def bucket_count(self) -> int:
        value = ctypes.c_int()
        _check(load().nntrain_plan_bucket_count(self._handle, ctypes.addressof(value)))
        return value.value

    @property
    def bucket_element_counts(self) -> list[int]:
        out = []
        for bucket in range(self.bucket_count):
            value = ctypes.c_longlong()
            _check(load().nntrain_plan_bucket_elements(self._handle, bucket, ctypes.addressof(value)))
            out.append(value.value)
        return out

    def locate(self, tensor: int) -> tuple[int, int]:
        bucket, offset = ctypes.c_int(), ctypes.c_longlong()
        _check(load().nntrain_plan_locate(self._handle, tensor, ctypes.addressof(bucket), ctypes.addressof(offset)))
        return bucket.value, offset.value

    @property
    def transport_bytes_per_step(self) -> int:
        value = ctypes.c_longlong()
        _check(load().nntrain_plan_transport_bytes_per_step(self._handle, ctypes.addressof(value)))
        return value.value

    @property
    def completed_steps(self) -> int:
        value = ctypes.c_longlong()
        _check(load().nntrain_plan_completed_steps(self._handle, ctypes.addressof(value)))
        return value.value

    def begin_step(self) -> int:
        step = ctypes.c_longlong()
        _check(load().nntrain_plan_begin_step(self._handle, ctypes.addressof(step)))
        return step.value

    def begin_device_step(self, step: int) -> None:
        _check(load().nntrain_plan_begin_device_step(self._handle, step))

    def notify_gradient_ready(self, tensor: int, step: int) -> int:
        ready = ctypes.c_int()
        _check(load().nntrain_plan_notify_gradient_ready(self._handle, step, tensor, ctypes.addressof(ready)))
        return ready.value

    def next_enqueueable(self, step: int) -> int:
        bucket = ctypes.c_int()
        _check(load().nntrain_plan_next_enqueueable(self._handle, step, ctypes.addressof(bucket)))
        return bucket.value

    def complete(self, step: int, non_finite: bool = False) -> None:
        _check(load().nntrain_plan_complete(self._handle, step, int(non_finite)))

    def abort(self, step: int) -> None:
        _check(load().nntrain_plan_abort(self._handle, step))

    def coherence_snapshot(self, tensor: int) -> dict:
        out = (ctypes.c_longlong * 6)()
        _check(load().nntrain_plan_coherence_snapshot(self._handle, tensor, out))
        return {"kind": out[0], "stamp": (out[1], out[2]), "pending_step": out[3], "version": out[4],
                "consumed_version": out[5]}

    def optimizer_validate_and_consume(self, devices=None) -> None:
        devices = self.devices if devices is None else list(devices)
        _check(load().nntrain_plan_optimizer_validate_and_consume(
            self._handle, (ctypes.c_int * max(1, len(devices)))(*devices), len(devices)))

    def publish_squared_sum(self, squared_sum: float, devices=None) -> None:
        devices = self.devices if devices is None else list(devices)
        _check(load().nntrain_plan_publish_squared_sum(
            self._handle, (ctypes.c_int * len(devices))(*devices), len(devices), squared_sum))

    def try_consume_squared_sum(self, devices=None):
        """The cached fused sum of squares, or None on a miss (one shot)."""
        devices = self.devices if devices is None else list(devices)
        value, hit = ctypes.c_double(), ctypes.c_int()
        _check(load().nntrain_plan_try_consume_squared_sum(
            self._handle, (ctypes.c_int * len(devices))(*devices), len(devices), ctypes.addressof(value),
            ctypes.addressof(hit)))
        return value.value if hit.value else None


def clip_decision(squared_sum: float, max_norm: float) -> tuple[float, float]:
    """(pre-clip norm, coefficient) of clip_grad_norm_ (NNtrain.Core/Torch/nn.cs:32-81)."""
    norm, coefficient = ctypes.c_float(), ctypes.c_float()
    _check(load().nntrain_gradient_clip_decision(squared_sum, max_norm, ctypes.addressof(norm),
                                                 ctypes.addressof(coefficient)))
    return norm.value, coefficient.value
