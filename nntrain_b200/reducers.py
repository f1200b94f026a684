"""N-rank gradient-arena reducers: the host side of the all-reduce, one
process per GPU.

The reference's reducers (`CudaBfp8GradientAllReducePlan`,
NNtrain.Core/Training/CudaBfp8GradientAllReduce.cs:9-841, and
`CudaBFloat16GradientAllReducePlan`, CudaBFloat16GradientAllReduce.cs:47-1866)
live in one process, drive two devices from two threads and move whole
buckets with peer copies.  Here every rank is a process; the encoded arena of
each rank sits in peer-visible memory, and one call of the C ABI performs the
reduce-scatter, the owner's fp32 accumulate + re-encode and the all-gather.
`torch.distributed` is used only to hand out the NCCL id and the IPC handles.

Arena layout is the reference's (CudaBFloat16GradientAllReduce.cs:1515-1601):
one contiguous fp32 gradient arena per bucket with parameters at running-sum
offsets, an int8 payload sidecar of the same element layout and one fp32
scale per block, blocks running over the bucket (not per tensor).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .library import check, load
from .native import CudaBfp8Native, CudaGradientBuckets, GradientNorm, _stream

PEER, NCCL, COPY_ENGINE = 0, 1, 2


def shard_range(length: int, world: int, rank: int) -> tuple[int, int]:
    first, end = ctypes.c_longlong(), ctypes.c_longlong()
    check("gradient_shard_range", load().nntrain_gradient_shard_range(
        length, world, rank, ctypes.addressof(first), ctypes.addressof(end)))
    return first.value, end.value


def _pointer_table(pointers):
    return (ctypes.c_void_p * len(pointers))(*pointers)


def reduce_shards_bfp8(device: int, payloads, scales, out_payloads, out_scales, first: int, end: int,
                       block_size: int, reduction_scale: float = 1.0, squared_sum=None, finite_status=None,
                       stream=None) -> None:
    """Owner arithmetic on explicit tensors (each list entry one rank's arena)."""
    check("gradient_reduce_shards_bfp8", load().nntrain_gradient_reduce_shards_bfp8(
        device, len(payloads), _pointer_table([t.data_ptr() for t in payloads]),
        _pointer_table([t.data_ptr() for t in scales]), len(out_payloads),
        _pointer_table([t.data_ptr() for t in out_payloads]),
        _pointer_table([t.data_ptr() for t in out_scales]), first, end, block_size, reduction_scale,
        0 if squared_sum is None else squared_sum.data_ptr(),
        0 if finite_status is None else finite_status.data_ptr(), _stream(stream)))


def reduce_shards_bfp8_no_alloc(device: int, payloads, scales, out_payloads, out_scales, first: int, end: int,
                                block_size: int, reduction_scale: float = 1.0, squared_sum=None,
                                finite_status=None, stream=None) -> None:
    """`reduce_shards_bfp8` for a host that may not allocate device memory at
    this point: its scratch is a fixed array inside the library (at most 2^30
    values per call; calls that overlap on one GPU race on that array)."""
    check("gradient_reduce_shards_bfp8_no_alloc", load().nntrain_gradient_reduce_shards_bfp8_no_alloc(
        device, len(payloads), _pointer_table([t.data_ptr() for t in payloads]),
        _pointer_table([t.data_ptr() for t in scales]), len(out_payloads),
        _pointer_table([t.data_ptr() for t in out_payloads]),
        _pointer_table([t.data_ptr() for t in out_scales]), first, end, block_size, reduction_scale,
        0 if squared_sum is None else squared_sum.data_ptr(),
        0 if finite_status is None else finite_status.data_ptr(), _stream(stream)))


def reduce_shards_bf16(device: int, values, out_values, reduced, first: int, end: int,
                       reduction_scale: float = 1.0, squared_sum=None, square_of_bf16: bool = True,
                       stream=None) -> None:
    check("gradient_reduce_shards_bf16", load().nntrain_gradient_reduce_shards_bf16(
        device, len(values), _pointer_table([t.data_ptr() for t in values]), len(out_values),
        _pointer_table([t.data_ptr() for t in out_values]) if out_values else None,
        0 if reduced is None else reduced.data_ptr(), first, end, reduction_scale,
        0 if squared_sum is None else squared_sum.data_ptr(), int(square_of_bf16), _stream(stream)))


class GradientGroup:
    """This rank's membership of the job (world, rank, device, communicator)."""

    def __init__(self, world: int = 1, rank: int = 0, device: int = 0, process_group=None):
        self.world, self.rank, self.device = world, rank, device
        self.process_group = process_group
        lib = load()
        identifier = None
        if world > 1:
            import torch.distributed as dist
            holder = [None]
            if rank == 0:
                buffer = ctypes.create_string_buffer(128)
                check("gradient_group_unique_id", lib.nntrain_gradient_group_unique_id(buffer))
                holder[0] = buffer.raw
            dist.broadcast_object_list(holder, src=0, group=process_group)
            identifier = ctypes.create_string_buffer(holder[0], 128)
        handle = ctypes.c_void_p()
        check("gradient_group_create", lib.nntrain_gradient_group_create(
            identifier, world, rank, device, ctypes.addressof(handle)))
        self.handle = handle.value

    def configure(self, collective_ctas: int = 0, asynchronous_copies: int = 1, exclusive_sms: bool = False):
        """Launch shape of THIS group's all-reduce kernels (other groups in the
        process keep theirs).  asynchronous_copies: 0 register prefetch, 1
        cp.async rings, 2 bulk asynchronous copies of whole tiles."""
        check("gradient_group_configure", load().nntrain_gradient_group_configure(
            self.handle, collective_ctas, int(asynchronous_copies), int(exclusive_sms)))

    def poll(self) -> int:
        """0 while the communicator is healthy; never blocks."""
        return load().nntrain_gradient_group_poll(self.handle)

    def abort(self) -> None:
        """Gives the communicator up without waiting (a peer was declared lost)."""
        check("gradient_group_abort", load().nntrain_gradient_group_abort(self.handle))

    def publish_shards_bfp8(self, source: torch.Tensor, payload_pointers, scales_pointers, length: int,
                            block_size: int, finite_status=None, stream=None) -> None:
        """This rank encodes its shard of `source` (fp32) into every rank's
        encoded arena; collective."""
        check("gradient_publish_shards_bfp8", load().nntrain_gradient_publish_shards_bfp8(
            self.handle, source.data_ptr(), _pointer_table(payload_pointers), _pointer_table(scales_pointers),
            length, block_size, 0 if finite_status is None else finite_status.data_ptr(), _stream(stream)))

    def sum(self, values: torch.Tensor, stream=None) -> None:
        check("gradient_group_sum", load().nntrain_gradient_group_sum(
            self.handle, values.data_ptr(), values.numel(), _stream(stream)))

    def barrier(self, stream=None) -> None:
        check("gradient_group_sum", load().nntrain_gradient_group_sum(self.handle, None, 0, _stream(stream)))

    def close(self) -> None:
        if self.handle:
            check("gradient_group_destroy", load().nntrain_gradient_group_destroy(self.handle))
            self.handle = None


class PeerBuffer:
    """`nbytes` of device memory every rank of the group can address.

    `pointers[k]` is rank k's buffer as mapped in this process; `tensor(dtype)`
    views this rank's own buffer as a torch tensor (no copy)."""

    def __init__(self, group: GradientGroup, nbytes: int):
        self.group, self.nbytes = group, nbytes
        lib = load()
        pointer = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        check("gradient_peer_alloc", lib.nntrain_gradient_peer_alloc(
            group.device, nbytes, ctypes.addressof(pointer), handle))
        self.local = pointer.value
        self.pointers = [None] * group.world
        self.pointers[group.rank] = self.local
        self._opened = []
        if group.world > 1:
            import torch.distributed as dist
            handles = [None] * group.world
            dist.all_gather_object(handles, handle.raw, group=group.process_group)
            for k, raw in enumerate(handles):
                if k == group.rank:
                    continue
                mapped = ctypes.c_void_p()
                check("gradient_peer_open", lib.nntrain_gradient_peer_open(
                    group.device, ctypes.create_string_buffer(raw, 64), ctypes.addressof(mapped)))
                self.pointers[k] = mapped.value
                self._opened.append(mapped.value)

    def tensor(self, dtype: torch.dtype, count: int | None = None) -> torch.Tensor:
        itemsize = torch.empty((), dtype=dtype).element_size()
        count = self.nbytes // itemsize if count is None else count
        return _device_view(self.local, count, dtype, self.group.device)

    def close(self) -> None:
        lib = load()
        if self.group.world > 1:
            import torch.distributed as dist
            torch.cuda.synchronize(self.group.device)
            dist.barrier(group=self.group.process_group)
        for mapped in self._opened:
            lib.nntrain_gradient_peer_close(self.group.device, mapped)
        self._opened = []
        if self.group.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group.process_group)
        if self.local:
            lib.nntrain_gradient_peer_free(self.group.device, self.local)
            self.local = None


class _CudaArrayInterface:
    def __init__(self, pointer: int, count: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (pointer, False),
                                         "version": 3, "strides": None}


_TYPESTR = {torch.int8: "|i1", torch.float32: "<f4", torch.int16: "<i2", torch.float64: "<f8",
            torch.int32: "<i4", torch.uint8: "|u1"}


def _device_view(pointer: int, count: int, dtype: torch.dtype, device: int) -> torch.Tensor:
    """A torch tensor over memory the library allocated (zero-copy)."""
    with torch.cuda.device(device):
        return torch.as_tensor(_CudaArrayInterface(pointer, count, _TYPESTR[dtype]), device=f"cuda:{device}")


@dataclass
class StepResult:
    norm: float            # global L2 norm before clipping
    coefficient: float     # clip multiplier that was applied (1.0 = none)
    squared_sum: float
    finite: bool
    # True when the fp32 arena holds the clipped gradient too.  The clip is
    # scale-only: payload x clipped scales is the authoritative gradient after a
    # step (the reference marks the BFP8 buffers synchronized and drops the fp32
    # copy, NNtrain.Core/Tensors/Tensor.CudaKernels.cs:321-437); the fp32 arena
    # keeps the decode of the UNCLIPPED result unless the reducer was built with
    # clip_fp32=True or the coefficient is 1.
    fp32_clipped: bool = True


class _ResultBlock:
    """The 16 bytes a step leaves for the host: sum of squares (double), finite
    flag (int32), applied clip coefficient (float32).  One device buffer, read
    back with ONE copy (the reference's transfer budget per step is the finite
    flags plus one double, NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:39-41)."""

    def __init__(self, device: int):
        with torch.cuda.device(device):
            self.raw = torch.zeros(16, dtype=torch.uint8, device=f"cuda:{device}")
            self.norm_and_coefficient = torch.zeros(2, dtype=torch.float32, device=f"cuda:{device}")
        self.squared_sum = self.raw[0:8].view(torch.float64)
        self.finite_status = self.raw[8:12].view(torch.int32)
        self.coefficient = self.raw[12:16].view(torch.float32)

    def read(self, clipped: bool) -> tuple[float, bool, float, float]:
        """(squared_sum, finite, norm, coefficient) from one 16-byte read."""
        import numpy as np
        host = self.raw.cpu().numpy()
        squared_sum = float(host[0:8].view(np.float64)[0])
        finite = int(host[8:12].view(np.int32)[0]) == 0
        coefficient = float(host[12:16].view(np.float32)[0]) if clipped else 1.0
        norm = float(np.float32(np.sqrt(np.float64(squared_sum))))   # what the device computed: (float)sqrt(double)
        return squared_sum, finite, norm, coefficient


def chunk_spans(elements: int, world: int, chunk_elements: int | None = None,
                chunk_plan: list[int] | None = None) -> tuple[list[tuple[int, int]], int]:
    """The [start, stop) pieces a step cuts an arena of `elements` values into,
    and the longest piece.  Every boundary is a multiple of 512 * world, so each
    piece splits into `world` shards on 512-value boundaries (whole 32-, 64- and
    128-value blocks, 16-byte aligned payload).  `chunk_elements`: equal pieces
    of about that length.  `chunk_plan`: explicit lengths, the rest of the arena
    becoming a last piece.  Neither, for an arena of 64 Mi values or more on
    more than one rank: a short first piece (the wire starts early), long middle
    ones (few barriers) and short last ones (little decode left at the end)."""
    align = 512 * world
    if chunk_elements is None or chunk_elements >= elements:
        chunk_elements = elements
    else:
        chunk_elements = max(align, chunk_elements // align * align)
    if chunk_plan is None and chunk_elements == elements and world > 1 and elements >= (64 << 20):
        chunk_plan = [int(elements * f) for f in (0.03, 0.10, 0.26, 0.26, 0.20, 0.09)]
    if chunk_plan:
        plan = [max(align, int(c) // align * align) for c in chunk_plan]
        spans, start = [], 0
        for length in plan:
            if start >= elements:
                break
            spans.append((start, min(start + length, elements)))
            start += length
        if start < elements:
            spans.append((start, elements))
    else:
        spans = [(a, min(a + chunk_elements, elements)) for a in range(0, elements, chunk_elements)]
    return spans, max(b - a for a, b in spans)


class Bfp8ArenaAllReduce:
    """BFP8 all-reduce of one fp32 gradient arena across the group, with the
    fused global clip-norm.

    Per step (everything enqueued on streams, one host read at the end):
      encode     fp32 arena -> payload + scales           (compute stream)
      all-reduce in place over the encoded arena          (communication stream)
      decode     reduced payload -> fp32 arena            (optional; the fp32
                 arena then holds decode(encode(sum)), the reference's decode
                 cache, NNtrain.Cuda/native/tensor_kernels.cu:3988-3997,4034-4036)
      clip       scale-only, coefficient computed on the device from the fused
                 sum of squares (NNtrain.Core/Tensors/Tensor.CudaKernels.cs:321-437)
    The arena is processed in `chunk_elements` pieces so that the encode of
    chunk k+1 and the decode of chunk k-1 overlap the wire time of chunk k.
    With world == 1 the all-reduce degenerates to the single-GPU publication
    (NNtrain.Core/Tensors/CudaBfp8GradientPublicationScope.cs:12-521): encode
    with fused write-back, sum of squares and finite flag.
    """

    def __init__(self, group: GradientGroup, elements: int, block_size: int = 32, mode: int = PEER,
                 chunk_elements: int | None = None, reduction_scale: float = 1.0,
                 write_fp32: bool = True, codec_iterations_per_cta: int | None = None,
                 collective_ctas: int | None = None, chunk_plan: list[int] | None = None,
                 collective_async: int | None = None, collective_exclusive: bool | None = None,
                 clip_fp32: bool = False):
        if block_size not in (32, 64, 128):
            raise ValueError("block size must be 32, 64 or 128")
        self.group, self.elements, self.block, self.mode = group, elements, block_size, mode
        self.reduction_scale, self.write_fp32, self.clip_fp32 = reduction_scale, write_fp32, clip_fp32
        world = group.world
        spans, chunk_elements = chunk_spans(elements, world, chunk_elements, chunk_plan)
        self.spans = spans
        self.chunk = chunk_elements
        device = group.device
        self.scale_count = (elements + block_size - 1) // block_size
        with torch.cuda.device(device):
            self.payload_buffer = PeerBuffer(group, elements)
            self.scales_buffer = PeerBuffer(group, self.scale_count * 4)
            self.payload = self.payload_buffer.tensor(torch.int8, elements)
            self.scales = self.scales_buffer.tensor(torch.float32, self.scale_count)
            self.result = _ResultBlock(device)
            self.squared_sum, self.finite_status = self.result.squared_sum, self.result.finite_status
            self.norm_and_coefficient = self.result.norm_and_coefficient
            self.staging_payload = self.staging_scales = None
            if mode != PEER and world > 1:
                first, end = shard_range(min(self.chunk, elements), world, 0)
                shard = end - first
                shard = (shard + 511) // 512 * 512
                self.staging_payload = torch.empty(world * shard, dtype=torch.int8, device=f"cuda:{device}")
                self.staging_scales = torch.empty(world * shard // block_size + world, dtype=torch.float32,
                                                  device=f"cuda:{device}")
            # Overlap shape: with more than one chunk in flight the all-reduce
            # kernel runs on a high-priority stream beside the encode / decode
            # kernels of the neighbouring chunks.  Measured on 2 and 8 B200s: a
            # kernel whose CTAs share their SMs with codec CTAs loses 25-30 % of
            # its speed while those run; CTAs that own their SM do not, so the
            # overlapped step gives the collective cp.async rings on SMs of its
            # own (56 of 148 at 2-3 ranks, 64 from 4 ranks on) and leaves the
            # rest to the codec kernels.  The shape belongs to the group, not to
            # the process, so another reducer keeps its own.
            overlapped = world > 1 and len(self.spans) > 1
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            if collective_async is None:
                collective_async = 1
            if collective_exclusive is None:
                collective_exclusive = overlapped and mode == PEER and collective_async != 0
            if collective_ctas is None:
                if collective_exclusive:
                    collective_ctas = max(1, sms * (64 if world >= 4 else 56) // 148)
                else:
                    collective_ctas = sms if (overlapped and mode == PEER) else 0
            self.collective_ctas, self.collective_async = collective_ctas, collective_async
            self.collective_exclusive = bool(collective_exclusive)
            if world > 1:
                group.configure(collective_ctas, int(collective_async), bool(collective_exclusive))
            self.codec_iterations_per_cta = codec_iterations_per_cta
            if codec_iterations_per_cta is not None:
                # the encode / decode grids have no group: this one is process-wide
                check("gradient_configure", load().nntrain_gradient_configure(codec_iterations_per_cta, 0))
            self.compute_stream = torch.cuda.Stream(device)
            self.communication_stream = torch.cuda.Stream(device, priority=-1)
            self.decode_stream = torch.cuda.Stream(device)
            self.h2d_stream = torch.cuda.Stream(device)
            self.d2h_stream = torch.cuda.Stream(device)
            chunks = len(self.spans)
            # native events: recorded by the all-reduce entry point behind its
            # leading barrier ("every earlier chunk is final here")
            self.final_events = [CudaGradientBuckets.create_ready_event(device) for _ in range(chunks)]
            self.encoded = [torch.cuda.Event() for _ in range(chunks)]
            self.reduced = [torch.cuda.Event() for _ in range(chunks)]
            self.uploaded = [torch.cuda.Event() for _ in range(chunks)]
        self.kernel_launches = 0
        self._clipped = False
        # optional: the span of the communication stream's collective work inside
        # one step (first leading barrier .. last fence), for reporting
        self.collective_begin = torch.cuda.Event(enable_timing=True)
        self.collective_end = torch.cuda.Event(enable_timing=True)

    @property
    def transport_bytes_per_step(self) -> int:
        """Bytes this rank sends per step: 2 (N-1)/N (E + 4 ceil(E/block))
        (the N = 2, block = 128 case is the reference's
        2 (E + 4 ceil(E/128)), NNtrain.Core.Tests/CudaMix8GradientTransportTests.cs:267-270)."""
        world = self.group.world
        return 2 * (world - 1) * (self.elements + 4 * self.scale_count) // world

    def enqueue(self, gradient: torch.Tensor, max_norm: float | None = None, host_gradient=None,
                host_payload=None, host_scales=None) -> None:
        """Enqueues one whole step for `gradient` (the fp32 arena) behind the
        work already on the current stream.

        With `host_gradient` (pinned fp32) each chunk is first copied host ->
        device on its own stream, overlapping the previous chunk's kernels;
        with `host_payload` / `host_scales` (pinned) the reduced payload is
        copied back chunk by chunk as it becomes final and the (clipped) scale
        sidecar at the end."""
        group, device, lib = self.group, self.group.device, load()
        world = group.world
        current = torch.cuda.current_stream(device)
        self.result.raw.zero_()
        ready = current.record_event()
        for stream in (self.compute_stream, self.communication_stream, self.decode_stream, self.h2d_stream,
                       self.d2h_stream):
            stream.wait_event(ready)
        launches = 0      # the library's own kernels (torch's 16-byte fill and copy are not counted)
        spans = self.spans
        first_stream = self.communication_stream if world == 1 else self.compute_stream
        for index, (start, stop) in enumerate(spans):
            src = gradient[start:stop]
            payload = self.payload[start:stop]
            scales = self.scales[start // self.block:(stop + self.block - 1) // self.block]
            if host_gradient is not None:
                with torch.cuda.stream(self.h2d_stream):
                    src.copy_(host_gradient[start:stop], non_blocking=True)
                    self.uploaded[index].record(self.h2d_stream)
                first_stream.wait_event(self.uploaded[index])
            if world == 1:
                # single-GPU publication: encode + write-back + sum of squares + flag in one kernel
                CudaBfp8Native.block_encode(device, src, payload, scales, self.block,
                                            roundtrip=src if self.write_fp32 else None,
                                            squared_sum=self.squared_sum, finite_status=self.finite_status,
                                            stream=self.communication_stream)
                launches += 1
                self._result_final(index, gradient, host_payload, decode=False)
                continue
            CudaBfp8Native.block_encode(device, src, payload, scales, self.block,
                                        finite_status=self.finite_status, stream=self.compute_stream)
            self.encoded[index].record(self.compute_stream)
            self.communication_stream.wait_event(self.encoded[index])
            payload_table = _pointer_table([p + start for p in self.payload_buffer.pointers])
            scales_table = _pointer_table([p + 4 * (start // self.block) for p in self.scales_buffer.pointers])
            last = index == len(spans) - 1
            phase = (1 if index == 0 else 0) | (2 if last else 0)
            if index == 0:
                self.collective_begin.record(self.communication_stream)
            # A chunk's result is complete on every rank only after the NEXT
            # collective on the group: this call records final_events[index - 1]
            # right behind its leading barrier.
            check("gradient_allreduce_bfp8", lib.nntrain_gradient_allreduce_bfp8(
                group.handle, payload_table, scales_table, stop - start, self.block, self.reduction_scale,
                self.squared_sum.data_ptr(), self.finite_status.data_ptr(), self.mode, phase,
                0 if self.staging_payload is None else self.staging_payload.data_ptr(),
                0 if self.staging_scales is None else self.staging_scales.data_ptr(),
                self.final_events[index - 1] if index > 0 else None,
                self.communication_stream.cuda_stream))
            launches += 2 + (1 if phase & 1 else 0) + (2 if phase & 2 else 0)
            if last:
                self.collective_end.record(self.communication_stream)
            if index > 0:
                launches += self._result_final(index - 1, gradient, host_payload, self.write_fp32,
                                               self.final_events[index - 1])
            if last:
                launches += self._result_final(index, gradient, host_payload, self.write_fp32)
        # The decodes read the scale sidecar as reduced; the clip rewrites it in
        # place, so it must not start before the last decode has finished.
        self.communication_stream.wait_stream(self.decode_stream)
        self._clipped = max_norm is not None
        with torch.cuda.stream(self.communication_stream):
            if max_norm is not None:
                GradientNorm.clip_coefficient(device, self.squared_sum, max_norm, self.norm_and_coefficient,
                                              stream=self.communication_stream)
                GradientNorm.clip_apply(device, GradientNorm.BFP8, self.scales,
                                        coefficient=self.norm_and_coefficient, stream=self.communication_stream)
                launches += 2
                if self.clip_fp32 and self.write_fp32:
                    # an extra pass over the fp32 arena (8 B/value, skipped on
                    # the device when the coefficient is 1)
                    GradientNorm.clip_apply(device, GradientNorm.FP32, gradient,
                                            coefficient=self.norm_and_coefficient, stream=self.communication_stream)
                    launches += 1
                self.result.coefficient.copy_(self.norm_and_coefficient[1:2])
            if host_scales is not None:
                host_scales.copy_(self.scales, non_blocking=True)
        # every stream that was forked from the caller's joins it again (which
        # also makes the whole step recordable into a CUDA graph)
        for stream in (self.decode_stream, self.compute_stream, self.d2h_stream, self.h2d_stream):
            self.communication_stream.wait_stream(stream)
        current.wait_stream(self.communication_stream)
        self.kernel_launches = launches

    def record(self, gradient: torch.Tensor, max_norm: float | None = None):
        """Records one whole step for `gradient` into a CUDA graph and returns
        it: `graph.replay()` then costs the host one launch instead of some forty
        calls, and the device none of the gaps between them.  The arena's
        address is part of the recording (the reference's captured mode also
        relies on stable slot addresses, NNtrain.Core/Tensors/
        CudaBfp8GradientPublicationScope.cs:12-521); every rank must record,
        and later replay, in step with the others.  Run at least one eager step
        first: kernels must be loaded and NCCL's channels set up before a
        capture starts."""
        device = self.group.device
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self.enqueue(gradient, max_norm)
        torch.cuda.synchronize(device)
        return graph

    def _result_final(self, index: int, gradient, host_payload, decode: bool, native_event=None) -> int:
        """Chunk `index` is final: behind `native_event` when given, else in
        stream order on the communication stream.  Starts its decode and its
        copy back to the host."""
        start, stop = self.spans[index]
        if not decode and host_payload is None:
            return 0
        lib = load()
        waiters = ([self.d2h_stream] if host_payload is not None else []) + ([self.decode_stream] if decode else [])
        if native_event is None:
            self.reduced[index].record(self.communication_stream)
            for stream in waiters:
                stream.wait_event(self.reduced[index])
        else:
            for stream in waiters:
                check("gradient_stream_wait_event",
                      lib.nntrain_gradient_stream_wait_event(stream.cuda_stream, native_event))
        if host_payload is not None:
            with torch.cuda.stream(self.d2h_stream):
                host_payload[start:stop].copy_(self.payload[start:stop], non_blocking=True)
        if not decode:
            return 0
        CudaBfp8Native.block_decode(self.group.device, self.payload[start:stop],
                                    self.scales[start // self.block:(stop + self.block - 1) // self.block],
                                    gradient[start:stop], self.block, stream=self.decode_stream)
        return 1

    def complete(self, max_norm: float | None = None) -> StepResult:
        """The step's only device-to-host read: 16 bytes (sum of squares,
        finite flag, applied clip coefficient) in one copy."""
        device = self.group.device
        torch.cuda.current_stream(device).synchronize()
        squared_sum, finite, norm, coefficient = self.result.read(self._clipped and max_norm is not None)
        if not finite:
            raise FloatingPointError("BFP8 gradient reduction saw a non-finite gradient")
        return StepResult(norm, coefficient, squared_sum, finite,
                          fp32_clipped=(coefficient == 1.0 or (self.clip_fp32 and self.write_fp32)))

    def close(self) -> None:
        torch.cuda.synchronize(self.group.device)
        for event in self.final_events:
            CudaGradientBuckets.destroy_event(self.group.device, event)
        self.final_events = []
        self.payload = self.scales = None
        self.payload_buffer.close()
        self.scales_buffer.close()


class Bf16ArenaAllReduce:
    """All-reduce of a bf16 gradient arena across the group: fp32 accumulate in
    rank order, bf16 (round to nearest even) result in place on every rank, sum
    of squares of the bf16 result, then the clip `g = bf16(f32(g) * c)`.

    The arena-mode reducer of the reference
    (`CudaBFloat16GradientAllReducePlan` with bf16 gradient storage,
    NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:538-541,1413-1459;
    clip: NNtrain.Core/Tensors/Tensor.CudaKernels.cs:176-319) for N ranks.
    `values` is this rank's arena (bf16 bit patterns as int16) in peer-visible
    memory: backward accumulates straight into it, nothing is packed."""

    def __init__(self, group: GradientGroup, elements: int, mode: int = PEER, reduction_scale: float = 1.0,
                 chunk_elements: int | None = None):
        self.group, self.elements, self.mode, self.reduction_scale = group, elements, mode, reduction_scale
        world, device = group.world, group.device
        align = 512 * world
        if chunk_elements is None or chunk_elements >= elements:
            chunk_elements = elements
        else:
            chunk_elements = max(align, chunk_elements // align * align)
        self.spans = [(a, min(a + chunk_elements, elements)) for a in range(0, elements, chunk_elements)]
        with torch.cuda.device(device):
            self.buffer = PeerBuffer(group, elements * 2)
            self.values = self.buffer.tensor(torch.int16, elements)
            self.squared_sum = torch.zeros(1, dtype=torch.float64, device=f"cuda:{device}")
            self.staging = None
            if mode != PEER and world > 1:
                first, end = shard_range(chunk_elements, world, 0)
                shard = (end - first + 511) // 512 * 512
                self.staging = torch.empty(world * shard, dtype=torch.int16, device=f"cuda:{device}")

    @property
    def transport_bytes_per_step(self) -> int:
        """2 (N-1)/N * 2 E; for N = 2 the reference's 2 * 2 * E per pair
        (NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:292-297)."""
        world = self.group.world
        return 2 * (world - 1) * 2 * self.elements // world

    def enqueue(self) -> None:
        device, lib = self.group.device, load()
        stream = torch.cuda.current_stream(device)
        self.squared_sum.zero_()
        for index, (start, stop) in enumerate(self.spans):
            table = _pointer_table([p + 2 * start for p in self.buffer.pointers])
            phase = (1 if index == 0 else 0) | (2 if index == len(self.spans) - 1 else 0)
            check("gradient_allreduce_bf16", lib.nntrain_gradient_allreduce_bf16(
                self.group.handle, table, stop - start, self.reduction_scale, self.squared_sum.data_ptr(),
                self.mode, phase, 0 if self.staging is None else self.staging.data_ptr(), stream.cuda_stream))

    def complete(self, max_norm: float | None = None) -> StepResult:
        """Reads the sum of squares (8 bytes) and applies the clip."""
        from .host_plan import clip_decision
        device = self.group.device
        torch.cuda.current_stream(device).synchronize()
        squared_sum = float(self.squared_sum.item())
        finite = squared_sum == squared_sum and squared_sum != float("inf")
        if not finite:
            raise FloatingPointError("BF16 gradient reduction saw a non-finite gradient")
        norm, coefficient = clip_decision(squared_sum, max_norm if max_norm is not None else 3.0e38)
        if max_norm is not None and coefficient != 1.0:
            GradientNorm.clip_apply(device, GradientNorm.BF16, self.values, multiplier=coefficient)
            torch.cuda.current_stream(device).synchronize()
        return StepResult(norm, coefficient, squared_sum, finite)

    def close(self) -> None:
        torch.cuda.synchronize(self.group.device)
        self.values = None
        self.buffer.close()


# ---- one process, all devices -------------------------------------------------------
class LocalGradientGroup:
    """The ranks of a job that ONE process drives (the reference engine's host
    model: one worker thread per device, NNtrain.Core/Training/
    CudaReplicaExecutor.cs:29-116,339-369).  `devices[r]` is rank r's device; a
    device may repeat, in which case those ranks share it (the way the N-rank
    path is exercised on a single GPU)."""

    def __init__(self, devices):
        self.devices = list(devices)
        self.world = len(self.devices)
        handle = ctypes.c_void_p()
        check("gradient_local_group_create", load().nntrain_gradient_local_group_create(
            self.world, (ctypes.c_int * self.world)(*self.devices), ctypes.addressof(handle)))
        self.handle = handle.value

    def configure(self, collective_ctas: int = 0, asynchronous_copies: int = 1, exclusive_sms: bool = False):
        check("gradient_group_configure", load().nntrain_gradient_group_configure(
            self.handle, collective_ctas, int(asynchronous_copies), int(exclusive_sms)))

    def allreduce_bfp8(self, payload_pointers, scales_pointers, length: int, block_size: int,
                       reduction_scale: float, squared_sum_pointers, finite_status_pointers, phase: int,
                       streams) -> None:
        check("gradient_local_allreduce_bfp8", load().nntrain_gradient_local_allreduce_bfp8(
            self.handle, _pointer_table(payload_pointers), _pointer_table(scales_pointers), length, block_size,
            reduction_scale, _pointer_table(squared_sum_pointers) if squared_sum_pointers else None,
            _pointer_table(finite_status_pointers) if finite_status_pointers else None, phase,
            _pointer_table(streams)))

    def allreduce_bf16(self, value_pointers, length: int, reduction_scale: float, squared_sum_pointers,
                       phase: int, streams) -> None:
        check("gradient_local_allreduce_bf16", load().nntrain_gradient_local_allreduce_bf16(
            self.handle, _pointer_table(value_pointers), length, reduction_scale,
            _pointer_table(squared_sum_pointers) if squared_sum_pointers else None, phase,
            _pointer_table(streams)))

    def publish_shards_bfp8(self, source_pointers, payload_pointers, scales_pointers, length: int,
                            block_size: int, finite_status_pointers, streams) -> None:
        """Rank r encodes shard r of its fp32 arena into every rank's encoded
        arena (parameter publication after a sharded optimizer step)."""
        check("gradient_local_publish_shards_bfp8", load().nntrain_gradient_local_publish_shards_bfp8(
            self.handle, _pointer_table(source_pointers), _pointer_table(payload_pointers),
            _pointer_table(scales_pointers), length, block_size,
            _pointer_table(finite_status_pointers) if finite_status_pointers else None, _pointer_table(streams)))

    def close(self) -> None:
        if self.handle:
            check("gradient_local_group_destroy", load().nntrain_gradient_local_group_destroy(self.handle))
            self.handle = None


class _RankState:
    """What one rank of an in-process reducer owns on its device."""

    def __init__(self, device: int, elements: int, scale_count: int, chunks: int):
        self.device = device
        with torch.cuda.device(device):
            name = f"cuda:{device}"
            self.payload = torch.empty(elements, dtype=torch.int8, device=name)
            self.scales = torch.empty(scale_count, dtype=torch.float32, device=name)
            self.result = _ResultBlock(device)
            self.compute_stream = torch.cuda.Stream(device)
            self.communication_stream = torch.cuda.Stream(device, priority=-1)
            self.decode_stream = torch.cuda.Stream(device)
        self.begun = CudaGradientBuckets.create_ready_event(device)
        self.encoded = [CudaGradientBuckets.create_ready_event(device) for _ in range(chunks)]
        self.reduced = [CudaGradientBuckets.create_ready_event(device) for _ in range(chunks)]
        self.decoded = CudaGradientBuckets.create_ready_event(device)
        self.done = CudaGradientBuckets.create_ready_event(device)
        self.gradient = None

    def events(self):
        return [self.begun, self.decoded, self.done, *self.encoded, *self.reduced]


def _wait(stream, event) -> None:
    check("gradient_stream_wait_event", load().nntrain_gradient_stream_wait_event(_stream(stream), event))


class InProcessBfp8AllReduce:
    """`Bfp8ArenaAllReduce` for ranks that live in one process.

    The flow is the reference plan's (NNtrain.Core/Training/
    CudaBfp8GradientAllReduce.cs:225-364): every device's worker thread calls
    `publish(rank, gradient)` once its backward is enqueued -- that encodes the
    rank's arena on the rank's own streams -- and the worker that arrives LAST
    enqueues the cross-device all-reduce, the decodes and the clip for all ranks
    (`publish` returns True for it).  `complete()` then reads 16 bytes per rank.
    Ranks are ordered by events only, so a single thread may drive every rank
    (`enqueue`)."""

    def __init__(self, group: LocalGradientGroup, elements: int, block_size: int = 32,
                 chunk_elements: int | None = None, reduction_scale: float = 1.0, write_fp32: bool = True):
        import threading
        if block_size not in (32, 64, 128):
            raise ValueError("block size must be 32, 64 or 128")
        self.group, self.elements, self.block = group, elements, block_size
        self.reduction_scale, self.write_fp32 = reduction_scale, write_fp32
        world = group.world
        align = 512 * world
        if chunk_elements is None or chunk_elements >= elements:
            chunk_elements = elements
        else:
            chunk_elements = max(align, chunk_elements // align * align)
        self.spans = [(a, min(a + chunk_elements, elements)) for a in range(0, elements, chunk_elements)]
        self.scale_count = (elements + block_size - 1) // block_size
        self.ranks = [_RankState(d, elements, self.scale_count, len(self.spans)) for d in group.devices]
        self._lock = threading.Lock()
        self._arrived = 0
        self._max_norm = None
        self._clipped = False
        self.kernel_launches = 0

    @property
    def transport_bytes_per_step(self) -> int:
        world = self.group.world
        return 2 * (world - 1) * (self.elements + 4 * self.scale_count) // world

    def _slices(self, state: _RankState, start: int, stop: int):
        return (state.payload[start:stop],
                state.scales[start // self.block:(stop + self.block - 1) // self.block])

    def publish(self, rank: int, gradient: torch.Tensor, max_norm: float | None = None) -> bool:
        """Rank `rank`'s part of a step, called on that rank's worker thread (or
        by a single driver): encode the arena behind the work already on the
        rank's current stream.  Returns True when this call was the last
        arrival and therefore enqueued the cross-device part."""
        state = self.ranks[rank]
        device = state.device
        with torch.cuda.device(device):
            current = torch.cuda.current_stream(device)
            CudaGradientBuckets.record_ready(device, state.begun, current)
            for stream in (state.compute_stream, state.communication_stream):
                _wait(stream, state.begun)
            # the previous step's last writers of the result block and readers of
            # the arena (never recorded yet on the first step: no wait then)
            _wait(state.compute_stream, state.done)
            with torch.cuda.stream(state.compute_stream):
                state.result.raw.zero_()
            state.gradient = gradient
            for index, (start, stop) in enumerate(self.spans):
                payload, scales = self._slices(state, start, stop)
                CudaBfp8Native.block_encode(device, gradient[start:stop], payload, scales, self.block,
                                            finite_status=state.result.finite_status, stream=state.compute_stream)
                CudaGradientBuckets.record_ready(device, state.encoded[index], state.compute_stream)
        with self._lock:
            self._arrived += 1
            if max_norm is not None:
                self._max_norm = max_norm
            last = self._arrived == self.group.world
            if last:
                self._arrived = 0
                max_norm, self._max_norm = self._max_norm, None
        if last:
            self._enqueue_collective(max_norm)
        return last

    def _enqueue_collective(self, max_norm) -> None:
        world = self.group.world
        launches = world * len(self.spans)           # the encodes
        streams = [s.communication_stream.cuda_stream for s in self.ranks]
        for index, (start, stop) in enumerate(self.spans):
            for state in self.ranks:
                _wait(state.communication_stream, state.encoded[index])
            phase = (1 if index == 0 else 0) | (2 if index == len(self.spans) - 1 else 0)
            self.group.allreduce_bfp8(
                [s.payload.data_ptr() + start for s in self.ranks],
                [s.scales.data_ptr() + 4 * (start // self.block) for s in self.ranks],
                stop - start, self.block, self.reduction_scale,
                [s.result.squared_sum.data_ptr() for s in self.ranks],
                [s.result.finite_status.data_ptr() for s in self.ranks], phase, streams)
            launches += world * (1 + (1 if phase & 1 else 0) + (2 if phase & 2 else 0))
            if self.write_fp32:
                for state in self.ranks:
                    # (the entry points select the rank's device for this thread; the
                    # guard puts the caller's own device back)
                    with torch.cuda.device(state.device):
                        CudaGradientBuckets.record_ready(state.device, state.reduced[index],
                                                         state.communication_stream)
                        _wait(state.decode_stream, state.reduced[index])
                        payload, scales = self._slices(state, start, stop)
                        CudaBfp8Native.block_decode(state.device, payload, scales, state.gradient[start:stop],
                                                    self.block, stream=state.decode_stream)
                    launches += 1
        self._clipped = max_norm is not None
        for state in self.ranks:
            device = state.device
            with torch.cuda.device(device):
                # the clip rewrites the scales the decodes read
                CudaGradientBuckets.record_ready(device, state.decoded, state.decode_stream)
                _wait(state.communication_stream, state.decoded)
                if max_norm is not None:
                    block = state.result
                    GradientNorm.clip_coefficient(device, block.squared_sum, max_norm, block.norm_and_coefficient,
                                                  stream=state.communication_stream)
                    GradientNorm.clip_apply(device, GradientNorm.BFP8, state.scales,
                                            coefficient=block.norm_and_coefficient,
                                            stream=state.communication_stream)
                    with torch.cuda.stream(state.communication_stream):
                        block.coefficient.copy_(block.norm_and_coefficient[1:2])
                    launches += 2
                CudaGradientBuckets.record_ready(device, state.done, state.communication_stream)
        self.kernel_launches = launches

    def enqueue(self, gradients, max_norm: float | None = None) -> None:
        """Single-threaded driver: every rank's publish in turn."""
        for rank, gradient in enumerate(gradients):
            self.publish(rank, gradient, max_norm)

    def wait(self, rank: int) -> None:
        """Makes rank `rank`'s current stream wait for the step's result."""
        state = self.ranks[rank]
        with torch.cuda.device(state.device):
            _wait(torch.cuda.current_stream(state.device), state.done)

    def complete(self, max_norm: float | None = None) -> list[StepResult]:
        """One 16-byte read per rank; the results are identical on all ranks."""
        results, bad = [], False
        for state in self.ranks:
            with torch.cuda.device(state.device):
                state.communication_stream.synchronize()
                squared_sum, finite, norm, coefficient = state.result.read(self._clipped and max_norm is not None)
            bad = bad or not finite
            results.append(StepResult(norm, coefficient, squared_sum, finite, fp32_clipped=coefficient == 1.0))
        if bad:
            raise FloatingPointError("BFP8 gradient reduction saw a non-finite gradient")
        return results

    def close(self) -> None:
        for state in self.ranks:
            with torch.cuda.device(state.device):
                torch.cuda.synchronize(state.device)
            for event in state.events():
                CudaGradientBuckets.destroy_event(state.device, event)
        self.ranks = []


class InProcessBf16AllReduce:
    """The bf16 arena reducer for ranks that live in one process (see
    `Bf16ArenaAllReduce` for the arithmetic and the reference lines)."""

    def __init__(self, group: LocalGradientGroup, elements: int, reduction_scale: float = 1.0,
                 chunk_elements: int | None = None):
        self.group, self.elements, self.reduction_scale = group, elements, reduction_scale
        world = group.world
        align = 512 * world
        if chunk_elements is None or chunk_elements >= elements:
            chunk_elements = elements
        else:
            chunk_elements = max(align, chunk_elements // align * align)
        self.spans = [(a, min(a + chunk_elements, elements)) for a in range(0, elements, chunk_elements)]
        self.values, self.squared_sums, self.streams = [], [], []
        for device in group.devices:
            with torch.cuda.device(device):
                self.values.append(torch.zeros(elements, dtype=torch.int16, device=f"cuda:{device}"))
                self.squared_sums.append(torch.zeros(1, dtype=torch.float64, device=f"cuda:{device}"))
                self.streams.append(torch.cuda.Stream(device, priority=-1))
        self.begun = [CudaGradientBuckets.create_ready_event(d) for d in group.devices]

    @property
    def transport_bytes_per_step(self) -> int:
        world = self.group.world
        return 2 * (world - 1) * 2 * self.elements // world

    def enqueue(self) -> None:
        for rank, device in enumerate(self.group.devices):
            with torch.cuda.device(device):
                CudaGradientBuckets.record_ready(device, self.begun[rank], torch.cuda.current_stream(device))
                _wait(self.streams[rank], self.begun[rank])
                with torch.cuda.stream(self.streams[rank]):
                    self.squared_sums[rank].zero_()
        streams = [s.cuda_stream for s in self.streams]
        for index, (start, stop) in enumerate(self.spans):
            phase = (1 if index == 0 else 0) | (2 if index == len(self.spans) - 1 else 0)
            self.group.allreduce_bf16([v.data_ptr() + 2 * start for v in self.values], stop - start,
                                      self.reduction_scale, [q.data_ptr() for q in self.squared_sums], phase,
                                      streams)

    def complete(self, max_norm: float | None = None) -> list[StepResult]:
        from .host_plan import clip_decision
        results = []
        for rank, device in enumerate(self.group.devices):
            with torch.cuda.device(device):
                self.streams[rank].synchronize()
                squared_sum = float(self.squared_sums[rank].item())
                if squared_sum != squared_sum or squared_sum == float("inf"):
                    raise FloatingPointError("BF16 gradient reduction saw a non-finite gradient")
                norm, coefficient = clip_decision(squared_sum, max_norm if max_norm is not None else 3.0e38)
                if max_norm is not None and coefficient != 1.0:
                    GradientNorm.clip_apply(device, GradientNorm.BF16, self.values[rank], multiplier=coefficient,
                                            stream=self.streams[rank])
                    self.streams[rank].synchronize()
            results.append(StepResult(norm, coefficient, squared_sum, True))
        return results

    def close(self) -> None:
        for rank, device in enumerate(self.group.devices):
            torch.cuda.synchronize(device)
            CudaGradientBuckets.destroy_event(device, self.begun[rank])
        self.values = []
