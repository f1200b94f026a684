"""The bucketed BFP8 gradient reducer, driven by per-tensor notifications.

This is the host flow of the reference's bucketed plan
(`CudaBFloat16GradientAllReducePlan` in its block-BFP8 mode,
NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs): tensors are packed
into buckets of at most `target_bucket_elements` values, never split
(`BuildBuckets`, :1647-1678); every parameter's gradient lives at its
running-sum offset inside its bucket's contiguous fp32 arena, with no padding
or alignment between tensors (`BindGradientArenas`, :1572-1601), so autograd
accumulates straight into the arena; the encoded sidecars (int8 payload, one
fp32 scale per block) have the same element layout and their blocks run over
the bucket, not per tensor.  Each device's worker thread calls
`notify_gradient_ready(rank, tensor)` as backward produces gradients
(:449-537); the notification that completes a bucket on a rank encodes that
bucket there, and once every rank has a bucket encoded, the thread that
arrived last enqueues its cross-device all-reduce -- buckets always in the
same descending order on all ranks -- followed by the decodes.  `complete`
(:912-1029) applies the fused global clip-norm and reads 16 bytes per rank.

The legality of every transition (step active, device step begun, a tensor
notified once, every bucket enqueued before completion) is decided by the
library's host-side step plan, one per rank (`GradientStepPlan`); the device
work rides on the in-process N-rank group (`LocalGradientGroup`).
"""
from __future__ import annotations

import threading

import torch

from .host_plan import GradientStepPlan, InvalidOperationError
from .native import CudaBfp8Native, CudaGradientBuckets, GradientNorm
from .reducers import LocalGradientGroup, StepResult, _ResultBlock, _wait

_ALIGN = 512          # values between bucket bases inside a rank's allocation


def small_transformer_numels(d_model: int = 512, layers: int = 8, ffn: int = 2048, vocab: int = 32000) -> list[int]:
    """Parameter sizes, in `parameters()` order, of a small decoder Transformer
    with an untied token embedding: 41,604,096 values at the defaults."""
    numels = [vocab * d_model]
    for _ in range(layers):
        numels += [d_model * 3 * d_model, 3 * d_model,      # fused qkv projection
                   d_model * d_model, d_model,              # attention output
                   d_model, d_model,                        # layer norm
                   d_model * ffn, ffn, ffn * d_model, d_model,
                   d_model, d_model]                        # layer norm
    numels += [d_model, d_model]                            # final layer norm
    return numels


class _Rank:
    def __init__(self, device: int, numels, devices, target: int, block: int):
        self.device = device
        # the plan wants distinct device ids: ranks that share a physical device
        # (single-GPU runs) are told apart by their rank
        self.plan = GradientStepPlan(numels, list(range(len(devices))), target, block)
        self.bucket_elements = self.plan.bucket_element_counts
        self.location = [self.plan.locate(t) for t in range(len(numels))]
        # one allocation per kind; bucket b starts at a 512-value boundary
        self.base = []
        total = 0
        for elements in self.bucket_elements:
            self.base.append(total)
            total += (elements + _ALIGN - 1) // _ALIGN * _ALIGN
        self.total = total
        name = f"cuda:{device}"
        with torch.cuda.device(device):
            self.arena = torch.zeros(total, dtype=torch.float32, device=name)
            self.payload = torch.zeros(total, dtype=torch.int8, device=name)
            self.scales = torch.ones(total // block, dtype=torch.float32, device=name)
            self.result = _ResultBlock(device)
            self.compute_stream = torch.cuda.Stream(device)
            self.communication_stream = torch.cuda.Stream(device, priority=-1)
            self.decode_stream = torch.cuda.Stream(device)
        buckets = len(self.bucket_elements)
        self.begun = CudaGradientBuckets.create_ready_event(device)
        self.written = [CudaGradientBuckets.create_ready_event(device) for _ in range(buckets)]
        self.encoded = [CudaGradientBuckets.create_ready_event(device) for _ in range(buckets)]
        self.reduced = [CudaGradientBuckets.create_ready_event(device) for _ in range(buckets)]
        self.decoded = CudaGradientBuckets.create_ready_event(device)
        self.done = CudaGradientBuckets.create_ready_event(device)
        self.ready_queue: list[int] = []     # buckets this rank has encoded, in enqueue order

    def events(self):
        return [self.begun, self.decoded, self.done, *self.written, *self.encoded, *self.reduced]


class BucketedBfp8Reducer:
    def __init__(self, group: LocalGradientGroup, numels, block_size: int = 32,
                 target_bucket_elements: int = 4 << 20, reduction_scale: float = 1.0):
        if block_size not in (32, 64, 128):
            raise ValueError("block size must be 32, 64 or 128")
        self.group, self.block, self.reduction_scale = group, block_size, reduction_scale
        self.numels = list(numels)
        self.ranks = [_Rank(d, self.numels, group.devices, target_bucket_elements, block_size)
                      for d in group.devices]
        self.bucket_elements = self.ranks[0].bucket_elements
        self.bucket_count = len(self.bucket_elements)
        self._lock = threading.Lock()
        self.step = 0
        self._enqueued = 0
        self.kernel_launches = 0

    # ---- layout --------------------------------------------------------------------
    def gradient_view(self, rank: int, tensor: int) -> torch.Tensor:
        """The slice of the bucket arena that IS tensor `tensor`'s gradient on
        rank `rank`: [offset, offset + numel) from the bucket's base, offsets
        being running sums of the earlier tensors' sizes (unaligned)."""
        state = self.ranks[rank]
        bucket, offset = state.location[tensor]
        start = state.base[bucket] + offset
        return state.arena[start:start + self.numels[tensor]]

    def bucket_views(self, rank: int, bucket: int):
        """(fp32 arena, payload, scales) of one bucket on one rank."""
        state = self.ranks[rank]
        a, n = state.base[bucket], self.bucket_elements[bucket]
        return (state.arena[a:a + n], state.payload[a:a + n],
                state.scales[a // self.block:a // self.block + (n + self.block - 1) // self.block])

    @property
    def transport_bytes_per_step(self) -> int:
        return self.ranks[0].plan.transport_bytes_per_step

    # ---- lifecycle -------------------------------------------------------------------
    def begin_step(self) -> int:
        """Coordinator: opens a step on every rank's plan (the step ids agree
        because every plan has completed or aborted the same steps)."""
        steps = [state.plan.begin_step() for state in self.ranks]
        if len(set(steps)) != 1:
            raise InvalidOperationError(f"rank plans disagree on the step id: {steps}")
        self.step = steps[0]
        self._enqueued = 0
        self.kernel_launches = 0
        for state in self.ranks:
            state.ready_queue = []
        return self.step

    def begin_device_step(self, rank: int) -> None:
        """Rank `rank`'s worker: the device part of opening a step, behind the
        work already on the rank's current stream."""
        state = self.ranks[rank]
        state.plan.begin_device_step(self.step)
        device = state.device
        with torch.cuda.device(device):
            CudaGradientBuckets.record_ready(device, state.begun, torch.cuda.current_stream(device))
            for stream in (state.compute_stream, state.communication_stream, state.decode_stream):
                _wait(stream, state.begun)
            _wait(state.compute_stream, state.done)      # the previous step's last accesses
            with torch.cuda.stream(state.compute_stream):
                state.result.raw.zero_()

    def notify_gradient_ready(self, rank: int, tensor: int) -> int:
        """Rank `rank`'s worker: tensor `tensor`'s gradient is final in stream
        order on the rank's current stream.  Returns the bucket this
        notification completed on the rank, or -1.  A second notification of
        the same tensor in a step raises InvalidOperationError."""
        state = self.ranks[rank]
        bucket = state.plan.notify_gradient_ready(tensor, self.step)
        if bucket < 0:
            return -1
        device = state.device
        with torch.cuda.device(device):
            CudaGradientBuckets.record_ready(device, state.written[bucket], torch.cuda.current_stream(device))
            _wait(state.compute_stream, state.written[bucket])
            arena, payload, scales = self.bucket_views(rank, bucket)
            CudaBfp8Native.block_encode(device, arena, payload, scales, self.block,
                                        finite_status=state.result.finite_status, stream=state.compute_stream)
            CudaGradientBuckets.record_ready(device, state.encoded[bucket], state.compute_stream)
        with self._lock:
            self.kernel_launches += 1
            while True:
                handed = state.plan.next_enqueueable(self.step)
                if handed < 0:
                    break
                state.ready_queue.append(handed)
            self._drain()
        return bucket

    def _drain(self) -> None:
        """Enqueues the all-reduce of every bucket that is now encoded on all
        ranks; called with the lock held, by whichever worker arrived last."""
        while all(s.ready_queue for s in self.ranks):
            heads = {s.ready_queue[0] for s in self.ranks}
            if len(heads) != 1:
                raise InvalidOperationError(f"ranks disagree on the bucket order: {sorted(heads)}")
            bucket = heads.pop()
            for s in self.ranks:
                s.ready_queue.pop(0)
            self._enqueue_bucket(bucket)

    def _enqueue_bucket(self, bucket: int) -> None:
        first = self._enqueued == 0
        last = self._enqueued == self.bucket_count - 1
        self._enqueued += 1
        phase = (1 if first else 0) | (2 if last else 0)
        elements = self.bucket_elements[bucket]
        for s in self.ranks:
            _wait(s.communication_stream, s.encoded[bucket])
        self.group.allreduce_bfp8(
            [s.payload.data_ptr() + s.base[bucket] for s in self.ranks],
            [s.scales.data_ptr() + 4 * (s.base[bucket] // self.block) for s in self.ranks],
            elements, self.block, self.reduction_scale,
            [s.result.squared_sum.data_ptr() for s in self.ranks],
            [s.result.finite_status.data_ptr() for s in self.ranks], phase,
            [s.communication_stream.cuda_stream for s in self.ranks])
        world = len(self.ranks)
        self.kernel_launches += world * (1 + (1 if first else 0) + (2 if last else 0))
        for rank, s in enumerate(self.ranks):
            # the entry points select the rank's device for the calling thread;
            # the guard puts the caller's own device back afterwards
            with torch.cuda.device(s.device):
                CudaGradientBuckets.record_ready(s.device, s.reduced[bucket], s.communication_stream)
                _wait(s.decode_stream, s.reduced[bucket])
                arena, payload, scales = self.bucket_views(rank, bucket)
                CudaBfp8Native.block_decode(s.device, payload, scales, arena, self.block, stream=s.decode_stream)
            self.kernel_launches += 1

    def complete(self, max_norm: float | None = None) -> list[StepResult]:
        """Coordinator: the fused global clip-norm on every rank (device-side
        coefficient from the all-reduced sum of squares, scale-only clip over
        every bucket's scales in one launch), one 16-byte read per rank, and
        the step's end on every plan.  Fails when a bucket was never enqueued
        or a gradient was not finite; the step then stays active (abort it)."""
        if self._enqueued != self.bucket_count:
            # let the plan phrase it
            self.ranks[0].plan.complete(self.step, False)
        for s in self.ranks:
            device = s.device
            with torch.cuda.device(device):
                CudaGradientBuckets.record_ready(device, s.decoded, s.decode_stream)
                _wait(s.communication_stream, s.decoded)
                if max_norm is not None:
                    GradientNorm.clip_coefficient(device, s.result.squared_sum, max_norm,
                                                  s.result.norm_and_coefficient, stream=s.communication_stream)
                    GradientNorm.clip_apply(device, GradientNorm.BFP8, s.scales,
                                            coefficient=s.result.norm_and_coefficient,
                                            stream=s.communication_stream)
                    with torch.cuda.stream(s.communication_stream):
                        s.result.coefficient.copy_(s.result.norm_and_coefficient[1:2])
                    self.kernel_launches += 2
                CudaGradientBuckets.record_ready(device, s.done, s.communication_stream)
        results, bad = [], False
        for s in self.ranks:
            with torch.cuda.device(s.device):
                s.communication_stream.synchronize()
                squared_sum, finite, norm, coefficient = s.result.read(max_norm is not None)
            bad = bad or not finite
            results.append(StepResult(norm, coefficient, squared_sum, finite, fp32_clipped=coefficient == 1.0))
        for s in self.ranks:
            s.plan.complete(self.step, bad)      # raises on a non-finite step: nothing becomes Reduced
        return results

    def wait(self, rank: int) -> None:
        """Makes rank `rank`'s current stream wait for the enqueued step."""
        s = self.ranks[rank]
        with torch.cuda.device(s.device):
            _wait(torch.cuda.current_stream(s.device), s.done)

    def abort(self) -> None:
        """Fail-closed end of the active step on every rank: whatever was
        enqueued drains, nothing becomes Reduced, the next step starts clean."""
        for s in self.ranks:
            with torch.cuda.device(s.device):
                torch.cuda.synchronize(s.device)
            try:
                s.plan.abort(self.step)
            except InvalidOperationError:
                pass                      # that rank's plan had already left the step
            s.ready_queue = []
        self._enqueued = 0

    def close(self) -> None:
        for s in self.ranks:
            with torch.cuda.device(s.device):
                torch.cuda.synchronize(s.device)
            for event in s.events():
                CudaGradientBuckets.destroy_event(s.device, event)
            s.plan.close()
        self.ranks = []
