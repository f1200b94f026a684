#!/usr/bin/env python
"""Benchmark of the compressed data-parallel gradient path.

    python bench.py --gpus N --steps K --warmup W          (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N \\
        --master-addr 127.0.0.1 --master-port P bench.py --gpus N --steps K --warmup W

One step = one BFP8 (block 32) all-reduce of the whole fp32 gradient arena of
the workload on every rank: encode, reduce-scatter + fp32 accumulate in rank
order + re-encode + all-gather, decode back into the fp32 arena, fused global
L2 clip-norm (max_norm 1.0, scale-only).  At N = 1 the collective is absent
and the step is the single-GPU publication: encode with fused decode
write-back, sum of squares and finite flag, then the clip.

Workload (default, `--config 4`): the gradient arena of a Qwen2-1.5B-shaped
model (1,543,714,304 fp32 values per rank, weak scaling: every rank holds a
full replica's gradient), synthetic N(0, sigma) with sigma log-uniform in
[1e-5, 1e-2] per 65,536-value slice, 1 % of 32-value blocks x100, 0.5 %
all-zero blocks.  Every timed step starts from the same un-quantised gradient:
a pristine copy is restored into the arena between steps, outside the timed
event pairs.

Rank 0 prints one JSON line.  `value` = N * 4 * E / t: fp32-equivalent
gradient bytes reduced per second summed over the ranks (the per-rank
all-reduce "algorithm bandwidth" 4E/t is `algbw_gbs`; wire bytes per rank per
direction over time is `busbw_gbs`).  After the timed region one more step is
checked against the CPU oracle in block-aligned windows of the arena
(`parity`); a mismatch makes the run exit non-zero.  `--impl reference` times
the CPU restatement of the reference's codec and reducer on the host cores
instead.

Other lines (each one JSON line, same conventions): `--config 2` the bf16
arena reducer on a GPT-2-small-sized arena, `--config 3` the bucket-size sweep,
`--config 1` the bucketed reducer of a small Transformer's tensor list (all
ranks in this process, no launcher), `--kernels` every kernel alone (with the
reference project's own kernels on the same buffers where they are built),
`--phases` / `--interference` what the overlapped step is made of, `--graph` the
step recorded once into a CUDA graph and replayed.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QWEN2_1P5B_ELEMENTS = 1_543_714_304
GPT2_SMALL_ELEMENTS = 124_439_808
BLOCK = 32
MAX_NORM = 1.0
METRIC = "bfp8_grad_allreduce_fp32_equiv_gbs"
UNIT = "GB/s"
NVLINK_PER_DIRECTION_GBS = 900.0          # nominal, per GPU per direction
NVLINK_MEASURED_PEER_COPY_GBS = 770.0     # measured peer copy on this pool
# DRAM bytes per value of the single-GPU publication kernel (encode +
# write-back + sum of squares), from an ncu capture of a 64 Mi-value launch
# scaled by the value count (about 0.7 B/value of its writes were still in L2
# when the captured kernel ended).
ENCODE_PUBLISH_DRAM_BYTES_PER_VALUE = 8.43
PARITY_WINDOW = 1 << 20


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", choices=("b200", "reference"), default="b200")
    p.add_argument("--config", type=int, default=4, choices=(1, 2, 3, 4))
    p.add_argument("--elements", type=int, default=0, help="0 = the configuration's own size")
    p.add_argument("--mode", choices=("peer", "nccl", "copy"), default="peer")
    p.add_argument("--chunk-elements", type=int, default=0, help="0 = pick by world size")
    p.add_argument("--chunk-plan", default="", help="comma-separated chunk lengths in Mi values (overrides --chunk-elements)")
    p.add_argument("--codec-iterations", type=int, default=-1, help="-1 = library default")
    p.add_argument("--collective-ctas", type=int, default=-1, help="-1 = library default for the run")
    p.add_argument("--collective-async", type=int, default=-1,
                   help="all-reduce kernel: 0 = register prefetch, 1 = cp.async rings, 2 = bulk copies, -1 = default")
    p.add_argument("--collective-exclusive", type=int, default=-1,
                   help="1 = the all-reduce kernel's CTAs take whole SMs, 0 = shared, -1 = default for the run")
    p.add_argument("--codec-ctas", type=int, default=0, help="cap on persistent codec grids (0 = none)")
    p.add_argument("--clip-fp32", action="store_true", help="also apply the clip to the fp32 arena (extra pass)")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-parity", action="store_true")
    p.add_argument("--no-phases", action="store_true")
    p.add_argument("--cpu-sample-elements", type=int, default=64 << 20)
    p.add_argument("--kernels", action="store_true",
                   help="time every kernel of the path alone (one JSON line each) instead of the step")
    p.add_argument("--phases", action="store_true",
                   help="only time encode, all-reduce and decode of the step separately (one JSON line)")
    p.add_argument("--interference", action="store_true",
                   help="N > 1: time the all-reduce kernel alone and beside memory traffic on this / the other ranks")
    p.add_argument("--only", default="", help="with --kernels: run only the cases whose name contains this")
    p.add_argument("--graph", action="store_true",
                   help="record the step into a CUDA graph once and time its replays: each bucket's step with "
                        "--config 3; the whole-arena step otherwise (then nothing runs eagerly on the group "
                        "afterwards: no phases, no end-to-end leg)")
    return p.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---- clocks -------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi while the timed region runs (reading only)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.rows = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, begin: float, end: float):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        rows = [r for t, r in self.rows if begin <= t <= end] or [r for _, r in self.rows]
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            if len(r) < 9:
                continue
            try:
                clocks.append(float(r[1]))
                maxima.append(float(r[2]))
            except ValueError:
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons),
                "samples": len(clocks)}


# ---- synthetic gradient on the device -------------------------------------------------
def fill_gradient(arena, seed: int, rank: int, sigma_range=(-5.0, -2.0), outliers: float = 0.01,
                  zeros: float = 0.005):
    """Configuration 0's distribution, generated on the device in slices."""
    import torch
    n = arena.numel()
    generator = torch.Generator(device=arena.device)
    generator.manual_seed(seed * 1000003 + rank)
    slice_elements = 65536
    piece = 1 << 26
    for start in range(0, n, piece):
        stop = min(start + piece, n)
        view = arena[start:stop]
        view.normal_(generator=generator)
        slices = (stop - start + slice_elements - 1) // slice_elements
        lo, hi = sigma_range
        exponents = torch.rand(slices, device=arena.device, generator=generator) * (hi - lo) + lo
        sigma = torch.pow(10.0, exponents).repeat_interleave(slice_elements)[:stop - start]
        view.mul_(sigma)
        blocks = (stop - start) // 32
        if blocks and (outliers or zeros):
            kind = torch.rand(blocks, device=arena.device, generator=generator)
            factor = torch.ones(blocks, device=arena.device)
            factor[kind < zeros] = 0.0
            factor[(kind >= zeros) & (kind < zeros + outliers)] = 100.0
            view[:blocks * 32].view(blocks, 32).mul_(factor.unsqueeze(1))
        del sigma, exponents


# ---- CPU baseline (the oracle port, checker code timed as the baseline) ---------------
def cpu_baseline(world: int, sample_elements: int, budget_seconds: float = 12.0):
    import oracle
    oracle.build()
    threads = oracle.max_threads()
    oracle.set_threads(threads)
    replicas = [oracle.generate_gradient(sample_elements, 0xB2000004, r) for r in range(world)]

    def one_pass():
        if world == 1:
            oracle.gradient_publish(replicas[0], BLOCK)
        else:
            oracle.allreduce_bfp8(replicas, BLOCK, 1.0 / world)

    one_pass()                      # warm-up
    times = []
    begin = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - begin < budget_seconds and len(times) < 50):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": world * 4.0 * sample_elements / best / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{sample_elements} fp32 values per replica x {world} replica(s), best of {len(times)} "
                      f"passes of encode(block 32)" + (" + decode write-back + sum of squares"
                                                       if world == 1 else
                                                       " x N + rank-ordered fp32 sum + re-encode + decode + sum of squares"),
            "seconds_per_pass": best}


def run_reference_arm(args, rank: int, world: int):
    """The reference's CPU implementation of the path (restated in C, see
    oracle/), all host threads, on a bounded sample of the same workload."""
    if rank != 0:
        return
    import oracle
    oracle.build()
    threads = oracle.max_threads()
    oracle.set_threads(threads)
    elements = args.elements or QWEN2_1P5B_ELEMENTS
    sample = min(args.cpu_sample_elements, elements)
    replicas = [oracle.generate_gradient(sample, 0xB2000004, r) for r in range(world)]

    def one_step():
        if world == 1:
            _, _, scales, _, sq = oracle.gradient_publish(replicas[0], BLOCK)
        else:
            _, scales, _, sq = oracle.allreduce_bfp8(replicas, BLOCK, 1.0 / world)
        _, c = oracle.clip_coefficient(sq, MAX_NORM)
        oracle.scale_bfp8_scales(scales, c)

    for _ in range(args.warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_step()
    elapsed = time.perf_counter() - t0
    ms = elapsed / args.steps * 1e3
    value = world * 4.0 * sample / (elapsed / args.steps) / 1e9
    sample_text = (f"{sample} of {elements} fp32 values per replica x {world} replica(s) per step "
                   f"(CPU restatement of the reference codec/reducer, OpenMP over blocks)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "qwen2-1.5b gradient arena, BFP8 block-32 all-reduce + clip-norm (CPU sample)",
                   "elements_per_rank": elements, "block": BLOCK, "max_norm": MAX_NORM,
                   "sample_elements": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample_text},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def qwen2_shaped_numels(total: int):
    """A 338-tensor list with the proportions of a Qwen2-1.5B parameter list
    (embedding, 28 x {q, k, v, o, gate, up, down, biases, norms}, final norm),
    scaled to `total` values; every tensor at least one value, sizes odd on
    purpose so tensors start at unaligned offsets."""
    hidden, layers, kv, inter, vocab = 1536, 28, 256, 8960, 151936
    numels = [vocab * hidden]
    for _ in range(layers):
        numels += [hidden * hidden, hidden, hidden * kv, kv, hidden * kv, kv, hidden * hidden,
                   hidden * inter, hidden * inter, inter * hidden, hidden, hidden]
    numels += [hidden]
    full = sum(numels)
    if total == full:
        return numels
    scaled = [max(1, n * total // full) for n in numels]
    scaled[0] += total - sum(scaled)
    return scaled


# ---- every kernel alone ---------------------------------------------------------------
def reference_kernel_cases(torch, E, arena, scratch, payload, scales, scales128, bf16):
    """The reference project's own kernels (compiled unmodified for sm_100a
    into oracle/_ref/libref_grad.so), launched on the same device buffers: the
    same-box bar for each operation.  Checker code, timed here only to be
    reported beside the library's kernels; never on the product path."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libref_grad.so")
    if not os.path.exists(path) or E >= (1 << 31):
        return []
    ref = ctypes.CDLL(path)

    def p(t):
        return ctypes.c_void_p(t.data_ptr())

    scale1 = torch.zeros(1, dtype=torch.float32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")

    def run(name, fn):
        def call():
            status = fn()
            if status != 0:
                raise RuntimeError(f"reference {name} returned {status}")
        return call

    n = int(E)
    import numpy as np
    numels = qwen2_shaped_numels(n)
    bounds = np.concatenate([[0], np.cumsum(numels)]).astype(np.int64)
    tensor_scales = torch.zeros(len(numels), dtype=torch.float32, device="cuda")

    def publish_per_tensor():
        status = 0
        for t in range(len(numels)):
            a, b = int(bounds[t]), int(bounds[t + 1])
            status |= ref.nntrain_bfp8_gradient_quantize_accumulate(
                0, ctypes.c_void_p(scratch.data_ptr() + 4 * a), ctypes.c_void_p(payload.data_ptr() + a),
                ctypes.c_void_p(tensor_scales.data_ptr() + 4 * t), b - a, p(flag), p(sq), None)
        return status

    extra = [("publish 338 tensors, one launch train (3 stream operations)", run("publish per tensor", publish_per_tensor), 13.0 * E)]
    return extra + [
        ("encode block32", run("quantize", lambda: ref.nntrain_cuda_bfp8_quantize_f32(0, p(arena), p(payload), p(scales), n, 32, None)), 5.125 * E),
        ("encode block128", run("quantize", lambda: ref.nntrain_cuda_bfp8_quantize_f32(0, p(arena), p(payload), p(scales128), n, 128, None)), (5 + 4 / 128) * E),
        ("encode tensor-wide (3 passes)", run("quantize", lambda: ref.nntrain_cuda_bfp8_quantize_f32(0, p(arena), p(payload), p(scale1), n, n, None)), 9.0 * E),
        ("decode block32", run("dequantize", lambda: ref.nntrain_cuda_bfp8_dequantize_f32(0, p(payload), p(scales), p(scratch), n, 32, None)), 5.125 * E),
        ("publish tensor-wide (quantize + write-back + squares)",
         run("quantize_accumulate", lambda: ref.nntrain_bfp8_gradient_quantize_accumulate(0, p(scratch), p(payload), p(scale1), n, p(flag), p(sq), None)), 13.0 * E),
        ("pack bf16", run("pack_bf16", lambda: ref.nntrain_gradient_pack_bf16(0, p(arena), p(bf16), 0, n, None)), 6.0 * E),
        ("pack bfp8 block128 (transport)", run("pack_bfp8_block", lambda: ref.nntrain_gradient_pack_bfp8_block(0, p(arena), p(payload), p(scales128), n, None)), (5 + 4 / 128) * E),
    ]


def time_kernels(args):
    """Every kernel of the path timed alone with CUDA events on its stream:
    algorithmic bytes / duration against the measured HBM peak."""
    import torch
    from nntrain_b200 import reducers
    from nntrain_b200.native import CudaBfp8GradientNative, CudaBfp8Native, CudaGradientBuckets, GradientNorm

    torch.cuda.set_device(0)
    from nntrain_b200.library import load
    if args.collective_async >= 0:
        load().nntrain_gradient_configure_collective(args.collective_async)
    E = min(args.elements or (256 << 20), 256 << 20)
    peak, kind = measured_peaks()
    arena = torch.empty(E, dtype=torch.float32, device="cuda")
    fill_gradient(arena, 0xB2000004, 0)
    scratch = torch.empty_like(arena)
    payload = torch.empty(E, dtype=torch.int8, device="cuda")
    scales = torch.empty(E // 32, dtype=torch.float32, device="cuda")
    scales128 = torch.empty(E // 128, dtype=torch.float32, device="cuda")
    bf16 = torch.empty(E, dtype=torch.int16, device="cuda")
    sq = torch.zeros(1, dtype=torch.float64, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale1 = torch.zeros(1, dtype=torch.float32, device="cuda")
    CudaBfp8Native.block_encode(0, arena, payload, scales, 32)
    replicas = [(payload.clone(), scales.clone()) for _ in range(7)]

    def reduce_n(n):
        ins = [(payload, scales)] + replicas[:n - 1]
        first, end = 0, E // n // 512 * 512      # one rank's shard, as in the all-reduce
        return (lambda: reducers.reduce_shards_bfp8(0, [p for p, _ in ins], [s for _, s in ins], [payload], [scales],
                                                    first, end, 32, 1.0 / n, sq, flag),
                (1.125 * n + 1.125) * (end - first))

    def reduce_bf16_n(n):
        CudaGradientBuckets.pack(0, arena, bf16, 0)
        ins = [bf16] + [bf16.clone() for _ in range(n - 1)]
        first, end = 0, E // n // 512 * 512
        return (lambda: reducers.reduce_shards_bf16(0, ins, [bf16], None, first, end, 1.0 / n, sq, True),
                (2.0 * n + 2.0) * (end - first))

    cases = [
        ("encode block32", lambda: CudaBfp8Native.block_encode(0, arena, payload, scales, 32), 5.125 * E),
        ("encode block32 + finite flag", lambda: CudaBfp8Native.block_encode(0, arena, payload, scales, 32, finite_status=flag), 5.125 * E),
        ("encode block32 publish (write-back + squares + flag)",
         lambda: CudaBfp8Native.block_encode(0, arena, payload, scales, 32, roundtrip=scratch, squared_sum=sq, finite_status=flag), 9.125 * E),
        ("encode block128", lambda: CudaBfp8Native.block_encode(0, arena, payload, scales128, 128), (5 + 4 / 128) * E),
        ("pack bfp8 block128 (transport)", lambda: CudaGradientBuckets.pack_bfp8_block(0, arena, payload, scales128), (5 + 4 / 128) * E),
        ("encode tensor-wide (3 passes)", lambda: CudaBfp8Native.block_encode(0, arena, payload, scales, 0), 9.0 * E),
        ("publish tensor-wide (quantize + write-back + squares)",
         lambda: CudaBfp8GradientNative.quantize(0, scratch, payload, scale1, flag, sq), 13.0 * E),
        ("decode block32", lambda: CudaBfp8Native.block_decode(0, payload, scales, scratch, 32), 5.125 * E),
        ("pack bf16", lambda: CudaGradientBuckets.pack(0, arena, bf16, 0), 6.0 * E),
        ("squared sum fp32", lambda: GradientNorm.squared_sum(0, GradientNorm.FP32, arena, sq), 4.0 * E),
        ("squared sum bf16", lambda: GradientNorm.squared_sum(0, GradientNorm.BF16, bf16, sq), 2.0 * E),
        ("squared sum bfp8", lambda: GradientNorm.squared_sum(0, GradientNorm.BFP8, payload, sq, scales, 32, flag), 1.125 * E),
        ("clip bfp8 scales", lambda: GradientNorm.clip_apply(0, GradientNorm.BFP8, scales, multiplier=0.999), 0.25 * E),
        ("clip fp32", lambda: GradientNorm.clip_apply(0, GradientNorm.FP32, scratch, multiplier=0.999), 8.0 * E),
    ]
    # the tensor-wide reducer over a 338-tensor bucket: one launch train for all
    # tensors against one publication per tensor
    import numpy as np
    numels = qwen2_shaped_numels(E)
    offsets_host = np.concatenate([[0], np.cumsum(numels)]).astype(np.int64)
    offsets = torch.from_numpy(offsets_host).cuda()
    tensor_scales = torch.zeros(len(numels), dtype=torch.float32, device="cuda")
    maxima = torch.zeros(len(numels), dtype=torch.int32, device="cuda")

    def publish_per_tensor():
        for t in range(len(numels)):
            a, b = int(offsets_host[t]), int(offsets_host[t + 1])
            CudaBfp8GradientNative.quantize(0, scratch[a:b], payload[a:b], tensor_scales[t:t + 1], flag, sq)

    cases += [
        ("publish 338 tensors, one launch train (3 stream operations)",
         lambda: CudaBfp8GradientNative.publish_tensors(0, scratch, payload, tensor_scales, offsets, maxima, flag, sq),
         13.0 * E),
        ("publish 338 tensors, one publication per tensor (338 x 4 stream operations)", publish_per_tensor, 13.0 * E),
    ]
    for n in (2, 4, 8):
        fn, nbytes = reduce_n(n)
        cases.append((f"owner reduce + re-encode, {n} local shards", fn, nbytes))
    for n in (2, 8):
        cases.append((f"bf16 owner reduce, {n} local shards", None, n))
    reference = reference_kernel_cases(torch, E, arena, scratch, payload, scales, scales128, bf16)
    ours = {}

    def time_case(fn, runs=10):
        for _ in range(3):
            fn()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(runs):
            fn()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / runs

    for name, fn, nbytes in cases:
        if args.only and args.only not in name:
            continue
        if fn is None:                      # bf16 owner reduce: built lazily (it overwrites `bf16`)
            fn, nbytes = reduce_bf16_n(nbytes)
        scratch.copy_(arena)
        ms = time_case(fn)
        achieved = nbytes / (ms * 1e-3) / 1e9
        ours[name] = ms
        emit({"kernel": name, "impl": "b200", "elements": E, "ms": round(ms, 4), "algorithmic_bytes": nbytes,
              "achieved_gbs": round(achieved, 1), "peak_gbs": peak, "peak_kind": kind,
              "frac": round(achieved / peak, 4)})
    for name, fn, nbytes in reference:
        if args.only and args.only not in name:
            continue
        scratch.copy_(arena)
        ms = time_case(fn, runs=5)
        achieved = nbytes / (ms * 1e-3) / 1e9
        emit({"kernel": name, "impl": "reference-kernel", "elements": E, "ms": round(ms, 4),
              "algorithmic_bytes": nbytes, "achieved_gbs": round(achieved, 1), "peak_gbs": peak, "peak_kind": kind,
              "frac": round(achieved / peak, 4),
              "b200_ms": round(ours[name], 4) if name in ours else None,
              "speedup_over_reference_kernel": round(ms / ours[name], 2) if name in ours else None})


# ---- pieces of the step ---------------------------------------------------------------
def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_phases(step, pristine, arena, world, local_rank, barrier, runs: int):
    """Encode, all-reduce and decode of one whole-arena step, each timed alone
    (CUDA events, max over ranks): what the overlapped step is made of."""
    import ctypes

    import torch
    from nntrain_b200.library import check, load
    from nntrain_b200.native import CudaBfp8Native

    lib, E = load(), step.elements
    stream = torch.cuda.current_stream()

    def encode():
        if world == 1:
            CudaBfp8Native.block_encode(local_rank, pristine, step.payload, step.scales, BLOCK, roundtrip=arena,
                                        squared_sum=step.squared_sum, finite_status=step.finite_status)
        else:
            CudaBfp8Native.block_encode(local_rank, pristine, step.payload, step.scales, BLOCK,
                                        finite_status=step.finite_status)

    def allreduce():
        table_p = (ctypes.c_void_p * world)(*step.payload_buffer.pointers)
        table_s = (ctypes.c_void_p * world)(*step.scales_buffer.pointers)
        check("allreduce", lib.nntrain_gradient_allreduce_bfp8(
            step.group.handle, table_p, table_s, E, BLOCK, 1.0 / world, step.squared_sum.data_ptr(),
            step.finite_status.data_ptr(), step.mode, 3,
            0 if step.staging_payload is None else step.staging_payload.data_ptr(),
            0 if step.staging_scales is None else step.staging_scales.data_ptr(), None, stream.cuda_stream))

    def allreduce_chunked():
        # the step's own chunk plan, collective calls only: what the barriers,
        # launches and kernel tails of the chunking cost without any codec kernel
        for index, (start, stop) in enumerate(step.spans):
            table_p = (ctypes.c_void_p * world)(*[p + start for p in step.payload_buffer.pointers])
            table_s = (ctypes.c_void_p * world)(*[p + 4 * (start // BLOCK) for p in step.scales_buffer.pointers])
            phase = (1 if index == 0 else 0) | (2 if index == len(step.spans) - 1 else 0)
            check("allreduce", lib.nntrain_gradient_allreduce_bfp8(
                step.group.handle, table_p, table_s, stop - start, BLOCK, 1.0 / world,
                step.squared_sum.data_ptr(), step.finite_status.data_ptr(), step.mode, phase,
                0 if step.staging_payload is None else step.staging_payload.data_ptr(),
                0 if step.staging_scales is None else step.staging_scales.data_ptr(), None, stream.cuda_stream))

    def decode():
        CudaBfp8Native.block_decode(local_rank, step.payload, step.scales, arena, BLOCK)

    out = {}
    todo = [("encode", encode)] + ([("allreduce", allreduce), ("allreduce_chunked", allreduce_chunked),
                                    ("decode", decode)] if world > 1 else [])
    for name, fn in todo:
        for _ in range(2):
            fn()
        barrier()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(runs):
            fn()
        end.record()
        torch.cuda.synchronize()
        barrier()
        out[name + "_ms"] = round(max_over_ranks(begin.elapsed_time(end) / runs, world), 4)
    if world > 1:
        wire = 2 * (world - 1) / world * (E + 4 * step.scale_count)
        out["allreduce_busbw_gbs"] = round(wire / (out["allreduce_ms"] * 1e-3) / 1e9, 1)
        out["serial_sum_ms"] = round(out["encode_ms"] + out["allreduce_ms"] + out["decode_ms"], 4)
    return out


def parity_windows(elements: int, spans, world: int, block: int, window: int = PARITY_WINDOW):
    """Block-aligned [a, b) windows of the arena to check against the oracle:
    the start, one straddling every chunk boundary of the plan, one straddling
    a shard boundary inside the largest chunk, two interior ones, the ragged
    tail.  Blocks are independent, so the oracle's result on a window is exact."""
    half = max(block, (window // 2) // block * block)
    picks = [(0, min(elements, 2 * half))]
    for start, _ in spans[1:]:
        picks.append((max(0, start - half), min(elements, start + half)))
    largest = max(spans, key=lambda s: s[1] - s[0])
    if world > 1:
        length = largest[1] - largest[0]
        shard = ((length + world - 1) // world + 511) // 512 * 512
        for k in (1, world - 1):
            edge = largest[0] + shard * k
            if largest[0] < edge < largest[1]:
                picks.append((max(0, edge - half), min(elements, edge + half)))
    for fraction in (0.37, 0.71):
        a = int(elements * fraction) // block * block
        picks.append((a, min(elements, a + 2 * half)))
    a = max(0, (elements - 2 * half) // block * block)
    picks.append((a, elements))
    out, seen = [], set()
    for a, b in picks:
        a = a // block * block
        if b > a and (a, b) not in seen:
            seen.add((a, b))
            out.append((a, b))
    return out


def check_parity(step, pristine, arena, result, world: int, rank: int, block: int):
    """One finished step against the CPU oracle, in windows; the sum of squares
    against an fp64 recomputation on the device; replica identity by checksums
    of the whole encoded arena.  Returns the `parity` block."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import oracle
    oracle.build()
    windows = parity_windows(step.elements, step.spans, world, block)
    mine = [pristine[a:b].cpu().numpy() for a, b in windows]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
    else:
        gathered = [mine]
    problems = []
    checked = 0
    for index, (a, b) in enumerate(windows):
        inputs = [gathered[r][index] for r in range(world)]
        if world == 1:
            fp32, payload, scales, flag, _ = oracle.gradient_publish(inputs[0], block)
        else:
            payload, scales, fp32, _ = oracle.allreduce_bfp8(inputs, block, step.reduction_scale)
        want_scales = oracle.scale_bfp8_scales(scales, result.coefficient) if result.coefficient != 1.0 else scales
        got_payload = step.payload[a:b].cpu().numpy()
        got_scales = step.scales[a // block:(b + block - 1) // block].cpu().numpy()
        got_fp32 = arena[a:b].cpu().numpy()
        if not np.array_equal(got_payload, payload):
            problems.append(f"payload differs in [{a},{b})")
        if not np.array_equal(got_scales.view(np.uint32), want_scales.view(np.uint32)):
            problems.append(f"scales differ in [{a},{b})")
        if not np.array_equal(got_fp32.view(np.uint32), fp32.view(np.uint32)):
            problems.append(f"fp32 arena differs in [{a},{b})")
        checked += b - a
    # sum of squares: the arena holds the decode of the (unclipped) result
    total = torch.zeros((), dtype=torch.float64, device=arena.device)
    piece = 1 << 26
    for start in range(0, step.elements, piece):
        total += arena[start:start + piece].double().square().sum()
    recomputed = float(total.item())
    norm_error = abs(result.squared_sum - recomputed) / max(recomputed, 1e-300)
    if norm_error > 1e-9:
        problems.append(f"sum of squares {result.squared_sum} vs fp64 recomputation {recomputed}")
    want_norm, want_c = oracle.clip_coefficient(result.squared_sum, MAX_NORM)
    if abs(result.norm - want_norm) > max(1e-5, 2e-6 * want_norm) or abs(result.coefficient - want_c) > 2e-6 * want_c:
        problems.append(f"norm / coefficient {result.norm} / {result.coefficient} vs {want_norm} / {want_c}")
    # replica identity over the WHOLE arena: every rank holds the same bytes
    checksum = [int(step.payload.view(torch.uint8).sum(dtype=torch.int64).item()),
                int(step.scales.view(torch.int32).sum(dtype=torch.int64).item()),
                int(arena.view(torch.int32).sum(dtype=torch.int64).item())]
    bad = {kind: any(kind in text for text in problems) for kind in ("payload", "scales", "fp32")}
    bad["other"] = any(not any(kind in text for kind in ("payload", "scales", "fp32")) for text in problems)
    agree = True
    if world > 1:
        everyone = [None] * world
        dist.all_gather_object(everyone, (checksum, bad))
        agree = all(entry[0] == everyone[0][0] for entry in everyone)
        bad = {kind: any(entry[1][kind] for entry in everyone) for kind in bad}
    for text in problems:
        print(f"rank {rank}: PARITY: {text}", file=sys.stderr)
    if not agree:
        print(f"rank {rank}: PARITY: ranks hold different results (whole-arena checksums)", file=sys.stderr)
    ok = agree and not any(bad.values())
    return {"ok": ok, "checked_values": checked, "windows": len(windows), "window_values": PARITY_WINDOW,
            "payload": "MISMATCH" if bad["payload"] else "exact", "scales": "MISMATCH" if bad["scales"] else "exact",
            "fp32": "MISMATCH" if bad["fp32"] else "exact", "norm_rel_err": norm_error,
            "norm_and_coefficient": "MISMATCH" if bad["other"] else "within 1e-9 / 2e-6 relative",
            "ranks_agree": agree,
            "oracle": "oracle.gradient_publish" if world == 1 else "oracle.allreduce_bfp8 (rank-ordered fp32 sum)",
            "problems_on_rank_0": problems[:4]}


def copy_floor_ms(arena, payload, scales, host_gradient, host_payload, host_scales, world, barrier, runs=2):
    """Bare pinned host <-> device copies of the end-to-end step's byte counts,
    all ranks copying at once: the floor under `e2e`."""
    import torch
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    best = None
    for _ in range(runs + 1):
        barrier()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        up.wait_event(begin)
        down.wait_event(begin)
        with torch.cuda.stream(up):
            arena.copy_(host_gradient, non_blocking=True)
        with torch.cuda.stream(down):
            host_payload.copy_(payload, non_blocking=True)
            host_scales.copy_(scales, non_blocking=True)
        torch.cuda.current_stream().wait_stream(up)
        torch.cuda.current_stream().wait_stream(down)
        end.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(begin.elapsed_time(end), world)
        best = ms if best is None else min(best, ms)
    return best


_REAL_STDOUT = None
_EXIT_WATCHDOG = None


def arm_exit_watchdog(status: int, seconds: float = 60.0) -> None:
    """The measurements are out; what is left is closing buffers, the group and
    the process group.  Should one of those calls not return (a communicator
    waiting for a peer that is already gone), leave with the status the run
    earned instead of hanging the launcher."""
    global _EXIT_WATCHDOG
    if _EXIT_WATCHDOG is not None:
        return

    def leave():
        print(f"teardown did not finish within {seconds:.0f} s; exiting without it", file=sys.stderr)
        sys.stderr.flush()
        os._exit(status)

    _EXIT_WATCHDOG = threading.Timer(seconds, leave)
    _EXIT_WATCHDOG.daemon = True
    _EXIT_WATCHDOG.start()


def disarm_exit_watchdog() -> None:
    global _EXIT_WATCHDOG
    if _EXIT_WATCHDOG is not None:
        _EXIT_WATCHDOG.cancel()
        _EXIT_WATCHDOG = None


def protect_stdout():
    """Libraries loaded below (NCCL prints its version) may write to fd 1; the
    contract is ONE JSON line on stdout, so everything else goes to stderr and
    the line is written to the saved descriptor."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    text = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, text)


def step_options(args):
    return dict(codec_iterations_per_cta=None if args.codec_iterations < 0 else args.codec_iterations,
                collective_ctas=None if args.collective_ctas < 0 else args.collective_ctas,
                chunk_plan=[int(float(c) * (1 << 20)) for c in args.chunk_plan.split(",")] if args.chunk_plan else None,
                collective_async=None if args.collective_async < 0 else args.collective_async,
                collective_exclusive=None if args.collective_exclusive < 0 else bool(args.collective_exclusive),
                clip_fp32=args.clip_fp32)


def run_step_bench(args, world, rank, local_rank, barrier):
    import torch
    import torch.distributed as dist
    from nntrain_b200 import reducers
    from nntrain_b200.library import load
    from nntrain_b200.native import CudaBfp8Native

    device = torch.device("cuda", local_rank)
    E = args.elements or QWEN2_1P5B_ELEMENTS
    mode = {"peer": reducers.PEER, "nccl": reducers.NCCL, "copy": reducers.COPY_ENGINE}[args.mode]
    group = reducers.GradientGroup(world, rank, local_rank)
    shape = step_options(args)
    step = reducers.Bfp8ArenaAllReduce(group, E, BLOCK, mode, chunk_elements=args.chunk_elements or None,
                                       reduction_scale=1.0 / world, write_fp32=True, **shape)
    if args.codec_ctas:
        load().nntrain_gradient_configure_codec_cap(args.codec_ctas)
    device_chunks = [b - a for a, b in step.spans]
    described = {"chunk_elements": step.chunk, "chunks": device_chunks,
                 "codec_iterations_per_cta": step.codec_iterations_per_cta if step.codec_iterations_per_cta is not None else 2,
                 "collective_ctas": step.collective_ctas, "collective_async": step.collective_async,
                 "collective_exclusive_sms": step.collective_exclusive}
    pristine = torch.empty(E, dtype=torch.float32, device=device)
    fill_gradient(pristine, 0xB2000004, rank)
    arena = torch.empty_like(pristine)
    torch.cuda.synchronize()

    if args.phases:
        phases = time_phases(step, pristine, arena, world, local_rank, barrier, max(3, min(args.steps, 10)))
        if rank == 0:
            emit({"phases": phases, "n_gpus": world, "elements_per_rank": E, "transport": args.mode, **described})
        step.close()
        group.close()
        return

    # -- device-resident timing: every step starts from the un-quantised gradient -----------
    graph = None

    def one_step(timed_pair=None):
        arena.copy_(pristine)
        torch.cuda.synchronize()
        barrier()
        if timed_pair is not None:
            timed_pair[0].record()
        if graph is not None:
            graph.replay()
        else:
            step.enqueue(arena, MAX_NORM)
        if timed_pair is not None:
            timed_pair[1].record()

    for _ in range(args.warmup):
        one_step()
    result = step.complete(MAX_NORM)
    recorded = args.graph
    if recorded:
        # the step as the reference's captured mode runs it: recorded once into a
        # CUDA graph (local kernels, the collective's barrier / kernel / fence,
        # clip), one replay per step afterwards
        barrier()
        graph = step.record(arena, MAX_NORM)
        barrier()
        one_step()
        step.complete(MAX_NORM)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    torch.cuda.synchronize()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    collective_ms = []
    wall_begin = time.time()
    for pair in pairs:
        one_step(pair)
        if world > 1 and graph is None:
            torch.cuda.synchronize()
            collective_ms.append(step.collective_begin.elapsed_time(step.collective_end))
    torch.cuda.synchronize()
    barrier()
    wall_end = time.time()
    result = step.complete(MAX_NORM)
    elapsed_ms = sum(a.elapsed_time(b) for a, b in pairs)
    clocks = sampler.stop(wall_begin, wall_end) if rank == 0 else None
    launches = step.kernel_launches * args.steps
    elapsed_ms = max_over_ranks(elapsed_ms, world)
    ms_per_step = elapsed_ms / args.steps
    seconds = ms_per_step * 1e-3
    algbw = 4.0 * E / seconds / 1e9
    wire_bytes = 2 * (world - 1) / world * (E + 4 * step.scale_count)
    busbw = wire_bytes / seconds / 1e9

    # -- parity: this very step (fresh input, the timed configuration) against the oracle ------
    parity = None
    if not args.no_parity:
        parity = check_parity(step, pristine, arena, result, world, rank, BLOCK)

    # a recording holds on to the collective's resources: let it go before any buffer or
    # group is closed
    graph = None

    # -- what the step is made of ----------------------------------------------------------------
    phases = None
    if not args.no_phases and not recorded:
        phases = time_phases(step, pristine, arena, world, local_rank, barrier, max(3, min(args.steps, 5)))
        phases["step_ms"] = round(ms_per_step, 4)
        if world > 1 and collective_ms:
            phases["allreduce_in_step_ms"] = round(max_over_ranks(sum(collective_ms) / len(collective_ms), world), 4)

    # -- roofline of the dominant kernel ---------------------------------------------------------
    hbm_peak, peak_kind = measured_peaks()
    if world == 1:
        # the publication kernel alone: fresh source, separate write-back buffer
        kernel_begin, kernel_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sq = torch.zeros(1, dtype=torch.float64, device=device)
        flag = torch.zeros(1, dtype=torch.int32, device=device)
        kernel_runs = max(3, min(args.steps, 10))
        for timed in (False, True):
            if timed:
                kernel_begin.record()
            for _ in range(kernel_runs if timed else 2):
                CudaBfp8Native.block_encode(local_rank, pristine, step.payload, step.scales, BLOCK, roundtrip=arena,
                                            squared_sum=sq, finite_status=flag)
            if timed:
                kernel_end.record()
        torch.cuda.synchronize()
        kernel_ms = kernel_begin.elapsed_time(kernel_end) / kernel_runs
        achieved = 9.125 * E / (kernel_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "bfp8_encode_blocks_kernel<32> publish (encode + write-back + squares + flag)",
                    "achieved": achieved, "peak": hbm_peak, "peak_kind": peak_kind, "unit": "GB/s",
                    "frac": achieved / hbm_peak, "traffic": ENCODE_PUBLISH_DRAM_BYTES_PER_VALUE * E,
                    "algorithmic_bytes": 9.125 * E, "ms_per_launch": kernel_ms,
                    "input": "un-quantised gradient, write-back into a second buffer",
                    "note": "frac may exceed 1: the denominator is a plain copy and part of the write-back is still in L2 when the kernel ends"}
    else:
        in_step = phases["allreduce_in_step_ms"] if (phases and "allreduce_in_step_ms" in phases) else ms_per_step
        achieved = wire_bytes / (in_step * 1e-3) / 1e9
        roofline = {"bound": "nvlink", "kernel": "bfp8_reduce_reencode (fused reduce-scatter + accumulate + re-encode + all-gather), in the step",
                    "achieved": achieved, "peak": NVLINK_PER_DIRECTION_GBS, "peak_kind": "nominal per direction per GPU",
                    "unit": "GB/s", "frac": achieved / NVLINK_PER_DIRECTION_GBS,
                    "peak_measured_peer_copy": NVLINK_MEASURED_PEER_COPY_GBS,
                    "frac_of_measured_peer_copy": achieved / NVLINK_MEASURED_PEER_COPY_GBS,
                    "traffic": None, "algorithmic_bytes": wire_bytes, "ms_per_launch": in_step,
                    "alone_ms": phases["allreduce_ms"] if phases else None,
                    "note": "algorithmic bytes = wire bytes per rank per direction; time = first leading barrier to last fence of the step's collective calls"}

    # -- end to end: pinned host buffers in, encoded result out -----------------------------
    e2e = None
    run_e2e = not args.no_e2e and not recorded
    if run_e2e:
        # Every rank must enter the collective part or none: agree first on
        # whether the pinned host buffers could be had everywhere.
        try:
            host_gradient = torch.empty(E, dtype=torch.float32, pin_memory=True)
            host_payload = torch.empty(E, dtype=torch.int8, pin_memory=True)
            host_scales = torch.empty(step.scale_count, dtype=torch.float32, pin_memory=True)
            have_buffers = 1.0
        except RuntimeError as error:
            print(f"rank {rank}: no pinned host buffers for the end-to-end leg: {error}", file=sys.stderr)
            host_gradient = host_payload = host_scales = None
            have_buffers = 0.0
        if world > 1:
            agreed = torch.tensor([have_buffers], dtype=torch.float64)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            have_buffers = float(agreed.item())
        if have_buffers == 0.0:
            run_e2e = False
            e2e = {"unavailable": "pinned host buffers could not be allocated on every rank"}
            host_gradient = host_payload = host_scales = None
    if run_e2e:
        host_gradient.copy_(pristine)
        floor = copy_floor_ms(arena, step.payload, step.scales, host_gradient, host_payload, host_scales, world, barrier)
        e2e_chunk = 64 << 20
        e2e_step = step if (step.chunk <= e2e_chunk) else None
        if e2e_step is None:
            step.close()
            e2e_step = reducers.Bfp8ArenaAllReduce(group, E, BLOCK, mode, chunk_elements=e2e_chunk,
                                                   reduction_scale=1.0 / world, write_fp32=True,
                                                   **{**shape, "chunk_plan": None})
        e2e_steps = max(1, min(args.steps, 5))
        for _ in range(min(args.warmup, 2)):
            e2e_step.enqueue(arena, MAX_NORM, host_gradient, host_payload, host_scales)
        barrier()
        torch.cuda.synchronize()
        b2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b2.record()
        for _ in range(e2e_steps):
            e2e_step.enqueue(arena, MAX_NORM, host_gradient, host_payload, host_scales)
            e2e_step.complete(MAX_NORM)       # the host reads the step's result
        e2.record()
        torch.cuda.synchronize()
        barrier()
        e2e_ms = max_over_ranks(b2.elapsed_time(e2) / e2e_steps, world)
        e2e = {"value": world * 4.0 * E / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": 4 * E, "d2h_bytes_per_step": E + 4 * step.scale_count + 16,
               "ms_per_step": e2e_ms, "steps": e2e_steps, "copy_floor_ms": floor,
               "over_copy_floor": e2e_ms / floor if floor else None,
               "bound": "pinned host <-> device copies of the same bytes, all ranks at once (copy_floor_ms)",
               "path": "Bfp8ArenaAllReduce.enqueue(host buffers) + complete(), per step"}
        step = e2e_step
        del host_gradient, host_payload, host_scales

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(world, min(args.cpu_sample_elements, E))

    if rank == 0:
        line = {
            "metric": METRIC, "value": world * algbw, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "qwen2-1.5b gradient arena, BFP8 block-32 all-reduce + decode + clip-norm"
                                   if E == QWEN2_1P5B_ELEMENTS else
                                   f"{E}-value gradient arena, BFP8 block-32 all-reduce + decode + clip-norm",
                       "elements_per_rank": E, "block": BLOCK, "max_norm": MAX_NORM,
                       "transport": args.mode if world > 1 else "none (single-GPU publication)",
                       **described,
                       "reduction": "mean (reduction_scale 1/N)",
                       "launch": ("one CUDA graph replay per step (the step recorded once after the warm-up; the "
                                  "parity block checks a replayed step)") if recorded else "eager: about forty host calls per step",
                       "l2": "inputs (6.2 GB per rank) exceed the 126 MB L2; no flush needed",
                       "input": "every timed step starts from the un-quantised gradient (pristine copy restored "
                                "between steps, outside the per-step event pairs); ms_per_step = sum of the "
                                "per-step device times / steps, max over ranks",
                       "fp32_arena": "decode cache of the reduced payload before the clip"
                                     + (" with the clip applied by an extra pass" if args.clip_fp32 else
                                        "; the clipped gradient is payload x clipped scales")},
            "algbw_gbs": algbw, "busbw_gbs": busbw,
            "nvlink": None if world == 1 else {
                "wire_bytes_per_rank_per_direction": wire_bytes, "achieved": busbw,
                "peak_nominal": NVLINK_PER_DIRECTION_GBS, "frac_nominal": busbw / NVLINK_PER_DIRECTION_GBS,
                "peak_measured_peer_copy": NVLINK_MEASURED_PEER_COPY_GBS,
                "frac_measured": busbw / NVLINK_MEASURED_PEER_COPY_GBS, "unit": "GB/s"},
            "roofline": roofline, "phases": phases, "parity": parity, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches, "clocks": clocks,
            "result": {"norm": result.norm, "clip_coefficient": result.coefficient, "finite": result.finite,
                       "fp32_clipped": result.fp32_clipped},
        }
        emit(line)
    status = 0 if (parity is None or parity["ok"]) else 3
    arm_exit_watchdog(status)
    step.close()
    group.close()
    return status


def run_bf16_bench(args, world, rank, local_rank, barrier):
    """Configuration 2: the bf16 arena reducer (fp32 accumulate in rank order,
    bf16 result, sum of squares of the bf16 result, clip) on a GPT-2-small-sized
    arena; values N(0, 1e-3) rounded to bf16."""
    import numpy as np
    import torch
    from nntrain_b200 import reducers

    device = torch.device("cuda", local_rank)
    E = args.elements or GPT2_SMALL_ELEMENTS
    group = reducers.GradientGroup(world, rank, local_rank)
    step = reducers.Bf16ArenaAllReduce(group, E, reducers.PEER, reduction_scale=1.0 / world,
                                       chunk_elements=args.chunk_elements or None)
    if world > 1 and (args.collective_ctas >= 0 or args.collective_async >= 0):
        group.configure(max(0, args.collective_ctas), 1 if args.collective_async != 0 else 0, False)
    generator = torch.Generator(device=device)
    generator.manual_seed(0xB2000002 * 1000003 + rank)
    pristine = (torch.randn(E, device=device, generator=generator) * 1e-3).to(torch.bfloat16).view(torch.int16)

    def one_step(pair=None):
        step.values.copy_(pristine)
        torch.cuda.synchronize()
        barrier()
        if pair is not None:
            pair[0].record()
        step.enqueue()
        result = step.complete(MAX_NORM * 0.05)
        if pair is not None:
            pair[1].record()
        return result

    for _ in range(args.warmup):
        one_step()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for pair in pairs:
        result = one_step(pair)
    torch.cuda.synchronize()
    ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in pairs) / args.steps, world)
    # parity on windows against the oracle's rank-ordered bf16 reduce
    import oracle
    oracle.build()
    import torch.distributed as dist
    windows = parity_windows(E, step.spans, world, 8)
    mine = [pristine[a:b].cpu().numpy().view(np.uint16) for a, b in windows]
    gathered = [mine]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
    problems = 0
    for index, (a, b) in enumerate(windows):
        _, expect, _ = oracle.bf16_reduce([gathered[r][index] for r in range(world)], 1.0 / world, want_bf16=True,
                                          square_of_bf16=True)
        if result.coefficient != 1.0:
            expect = oracle.scale_bf16(expect, result.coefficient)
        if not np.array_equal(step.values[a:b].cpu().numpy().view(np.uint16), expect):
            problems += 1
            print(f"rank {rank}: PARITY: bf16 arena differs in [{a},{b})", file=sys.stderr)
    if world > 1:
        counts = [None] * world
        dist.all_gather_object(counts, problems)
        problems = sum(counts)
    wire = 2 * (world - 1) / world * 2 * E
    hbm_peak, peak_kind = measured_peaks()
    if rank == 0:
        emit({"metric": "bf16_grad_allreduce_fp32_equiv_gbs", "value": world * 4.0 * E / (ms * 1e-3) / 1e9, "unit": UNIT,
              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
              "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
              "data": "synthetic",
              "config": {"workload": "gpt2-small-sized bf16 gradient arena, in-place all-reduce + sum of squares + clip",
                         "elements_per_rank": E, "chunks": [b - a for a, b in step.spans],
                         "timed": "enqueue() + complete(max_norm): includes the 8-byte host read and the clip pass"},
              "busbw_gbs": wire / (ms * 1e-3) / 1e9 if world > 1 else 0.0,
              "roofline": ({"bound": "nvlink", "achieved": wire / (ms * 1e-3) / 1e9, "peak": NVLINK_PER_DIRECTION_GBS,
                            "unit": "GB/s", "frac": wire / (ms * 1e-3) / 1e9 / NVLINK_PER_DIRECTION_GBS, "traffic": None}
                           if world > 1 else
                           {"bound": "hbm", "achieved": 8.0 * E / (ms * 1e-3) / 1e9, "peak": hbm_peak,
                            "peak_kind": peak_kind, "unit": "GB/s", "frac": 8.0 * E / (ms * 1e-3) / 1e9 / hbm_peak,
                            "traffic": None, "note": "N = 1: one rank's reduce (2+2 B/value) + clip (4 B/value)"}),
              "parity": {"ok": problems == 0, "windows": len(windows), "bf16": "exact" if problems == 0 else "MISMATCH"},
              "result": {"norm": result.norm, "clip_coefficient": result.coefficient}})
    status = 0 if problems == 0 else 3
    arm_exit_watchdog(status)
    step.close()
    group.close()
    return status


def run_sweep(args, world, rank, local_rank, barrier):
    """Configuration 3: one BFP8 all-reduce step (encode + all-reduce + decode +
    clip) of a single bucket, over bucket sizes; N(0, 1e-3) + 1 % outlier blocks."""
    import torch
    from nntrain_b200 import reducers

    device = torch.device("cuda", local_rank)
    group = reducers.GradientGroup(world, rank, local_rank)
    rows = []
    for E in (16 << 10, 256 << 10, 4 << 20, 64 << 20, 256 << 20):
        step = reducers.Bfp8ArenaAllReduce(group, E, BLOCK, reducers.PEER, reduction_scale=1.0 / world,
                                           write_fp32=True, **step_options(args))
        pristine = torch.empty(E, dtype=torch.float32, device=device)
        fill_gradient(pristine, 0xB2000003, rank, sigma_range=(-3.0, -3.0), outliers=0.01, zeros=0.0)
        arena = torch.empty_like(pristine)
        steps = args.steps if E >= (4 << 20) else args.steps * 5
        for _ in range(args.warmup):
            arena.copy_(pristine)
            step.enqueue(arena, MAX_NORM)
        step.complete(MAX_NORM)
        graph = None
        if args.graph:
            # the whole step (local kernels, the collective's barrier / kernel /
            # fence, clip) recorded once; a replay is one launch from the host
            torch.cuda.synchronize()
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                step.enqueue(arena, MAX_NORM)
            torch.cuda.synchronize()
            barrier()
        total = 0.0
        for _ in range(steps):
            arena.copy_(pristine)
            torch.cuda.synchronize()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if graph is not None:
                graph.replay()
            else:
                step.enqueue(arena, MAX_NORM)
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        if graph is not None:
            step.complete(MAX_NORM)
            del graph
        ms = max_over_ranks(total / steps, world)
        wire = 2 * (world - 1) / world * (E + 4 * step.scale_count)
        hbm_bytes = (5.125 + 5.125) * E + 2 * 1.125 * E
        rows.append({"elements": E, "fp32_bytes": 4 * E, "us_per_call": round(ms * 1e3, 2),
                     "algbw_gbs": round(4.0 * E / (ms * 1e-3) / 1e9, 2),
                     "busbw_gbs": round(wire / (ms * 1e-3) / 1e9, 2) if world > 1 else 0.0,
                     "frac_nvlink_nominal": round(wire / (ms * 1e-3) / 1e9 / NVLINK_PER_DIRECTION_GBS, 4) if world > 1 else None,
                     "hbm_gbs": round(hbm_bytes / (ms * 1e-3) / 1e9, 1),
                     "frac_hbm_measured": round(hbm_bytes / (ms * 1e-3) / 1e9 / measured_peaks()[0], 4),
                     "chunks": len(step.spans)})
        step.close()
        del pristine, arena
    if rank == 0:
        emit({"metric": "bfp8_grad_allreduce_bucket_sweep", "unit": "us per call / GB/s", "n_gpus": world,
              "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
              "dtype": "f32", "data": "synthetic",
              "config": {"workload": "single-bucket BFP8 block-32 all-reduce step (encode + all-reduce + decode + clip)",
                         "input": "un-quantised bucket restored before every timed call",
                         "launch": "one CUDA graph replay per step" if args.graph else "eager (about twenty host calls per step)"},
              "rows": rows})
    arm_exit_watchdog(0)
    group.close()
    return 0


def run_interference(args, world, rank, local_rank, barrier):
    """Why the all-reduce kernel slows down inside the step.  The fused kernel
    (this rank's shard, peer loads + peer stores, no collective call inside the
    timed region) is timed per rank: alone; while copy engines move memory on
    every rank (HBM load, no SM shared); while an encode loop runs on the OTHER
    ranks only (their HBM and SMs are busy, mine are not); on THIS rank only;
    on every rank.  Rank 0 is "this" rank."""
    import torch
    import torch.distributed as dist
    from nntrain_b200 import reducers
    from nntrain_b200.native import CudaBfp8Native

    device = torch.device("cuda", local_rank)
    E = args.elements or QWEN2_1P5B_ELEMENTS
    group = reducers.GradientGroup(world, rank, local_rank)
    step = reducers.Bfp8ArenaAllReduce(group, E, BLOCK, reducers.PEER, chunk_elements=E, reduction_scale=1.0 / world,
                                       **step_options(args))
    source = torch.empty(256 << 20, dtype=torch.float32, device=device)
    fill_gradient(source, 0xB2000004, rank)
    side_payload = torch.empty(source.numel(), dtype=torch.int8, device=device)
    side_scales = torch.empty(source.numel() // BLOCK, dtype=torch.float32, device=device)
    side_copy = torch.empty_like(source)
    for start in range(0, E, source.numel()):
        stop = min(E, start + source.numel())
        CudaBfp8Native.block_encode(local_rank, source[:stop - start], step.payload[start:stop],
                                    step.scales[start // BLOCK:(stop + BLOCK - 1) // BLOCK], BLOCK)
    torch.cuda.synchronize()
    barrier()
    # the bare owner-kernel export launches with the process-wide shape
    from nntrain_b200.library import check, load
    check("configure", load().nntrain_gradient_configure(2, step.collective_ctas))
    check("configure", load().nntrain_gradient_configure_collective(
        (3 if step.collective_exclusive else 4) if step.collective_async == 2
        else (2 if step.collective_exclusive else int(bool(step.collective_async)))))
    first, end = reducers.shard_range(E, world, rank)
    payloads = step.payload_buffer.pointers
    scales = step.scales_buffer.pointers
    side = torch.cuda.Stream(device)
    main = torch.cuda.Stream(device, priority=-1)

    class Raw:
        def __init__(self, pointer):
            self.pointer = pointer

        def data_ptr(self):
            return self.pointer

    def kernel():
        reducers.reduce_shards_bfp8(local_rank, [Raw(p) for p in payloads], [Raw(p) for p in scales],
                                    [Raw(p) for p in payloads], [Raw(p) for p in scales], first, end, BLOCK,
                                    1.0 / world, step.squared_sum, step.finite_status, stream=main)

    def load_codec(iterations):
        for _ in range(iterations):
            CudaBfp8Native.block_encode(local_rank, source, side_payload, side_scales, BLOCK, stream=side)

    def load_copy(iterations):
        with torch.cuda.stream(side):
            for _ in range(iterations):
                side_copy.copy_(source, non_blocking=True)

    rows = {}
    conditions = [("alone", None, ()), ("copy engines busy on every rank", load_copy, tuple(range(world))),
                  ("encode loop on the other ranks", load_codec, tuple(range(1, world))),
                  ("encode loop on this rank only", load_codec, (0,)),
                  ("encode loop on every rank", load_codec, tuple(range(world)))]
    for name, load, where in conditions:
        times = []
        for repeat in range(4):
            torch.cuda.synchronize()
            barrier()
            if load is not None and rank in where:
                load(40)                      # ~8-10 ms of side traffic, longer than the kernel
            begin, stop_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(main):
                begin.record(main)
                kernel()
                stop_event.record(main)
            torch.cuda.synchronize()
            barrier()
            if repeat:
                times.append(begin.elapsed_time(stop_event))
        mine = sum(times) / len(times)
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        rows[name] = {"this_rank_ms": round(everyone[0], 4),
                      "other_ranks_ms": [round(v, 4) for v in everyone[1:]]}
    wire = 2 * (world - 1) / world * (E + 4 * step.scale_count)
    if rank == 0:
        for row in rows.values():
            row["this_rank_busbw_gbs"] = round(wire / (row["this_rank_ms"] * 1e-3) / 1e9, 1)
        emit({"interference": rows, "n_gpus": world, "elements_per_rank": E,
              "collective_ctas": step.collective_ctas, "collective_async": step.collective_async,
              "collective_exclusive_sms": step.collective_exclusive,
              "note": "fused all-reduce kernel on the whole arena, per-rank CUDA-event time; side traffic started just before it"})
    arm_exit_watchdog(0)
    step.close()
    group.close()
    return 0


def run_bucketed(args):
    """Configuration 1: the bucketed BFP8 reducer of a small decoder
    Transformer's tensor list (41,604,096 values, buckets of at most 4 Mi
    values, tensors at running-sum offsets), all ranks driven from this process
    the way the reference's engine drives its devices.  A step: begin, one
    notification per tensor in backward (reverse) order on every rank -- each
    completed bucket is encoded and, once encoded everywhere, all-reduced and
    decoded -- then the fused clip-norm and the 16-byte read."""
    import numpy as np
    import torch

    import oracle
    from nntrain_b200 import bucketed, reducers

    world = max(1, args.gpus)
    visible = torch.cuda.device_count()
    devices = list(range(world)) if visible >= world else [0] * world
    numels = bucketed.small_transformer_numels()
    group = reducers.LocalGradientGroup(devices)
    reducer = bucketed.BucketedBfp8Reducer(group, numels, BLOCK, 4 << 20, 1.0 / world)
    oracle.build()
    total = sum(numels)
    pristine = []
    for rank, device in enumerate(devices):
        flat = torch.empty(total, dtype=torch.float32, device=f"cuda:{device}")
        with torch.cuda.device(device):
            fill_gradient(flat, 0xB2000001, rank)
        pristine.append(flat)
    offsets = np.concatenate([[0], np.cumsum(numels)])

    def restore():
        for rank in range(world):
            for tensor in range(len(numels)):
                reducer.gradient_view(rank, tensor).copy_(pristine[rank][offsets[tensor]:offsets[tensor + 1]])

    def one_step(pairs=None):
        restore()
        for device in set(devices):
            torch.cuda.synchronize(device)
        reducer.begin_step()
        for rank, device in enumerate(devices):
            with torch.cuda.device(device):
                if pairs is not None:
                    pairs[rank][0].record(torch.cuda.current_stream(device))
                reducer.begin_device_step(rank)
        for tensor in reversed(range(len(numels))):
            for rank, device in enumerate(devices):
                with torch.cuda.device(device):
                    reducer.notify_gradient_ready(rank, tensor)
        results = reducer.complete(MAX_NORM)
        for rank, device in enumerate(devices):
            with torch.cuda.device(device):
                reducer.wait(rank)
                if pairs is not None:
                    pairs[rank][1].record(torch.cuda.current_stream(device))
        return results

    for _ in range(args.warmup):
        one_step()
    elapsed = []
    for _ in range(args.steps):
        pairs = []
        for device in devices:
            with torch.cuda.device(device):
                pairs.append((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
        results = one_step(pairs)
        for device in set(devices):
            torch.cuda.synchronize(device)
        elapsed.append(max(a.elapsed_time(b) for a, b in pairs))
    ms = sum(elapsed) / len(elapsed)
    # parity: every bucket against the oracle (blocks run over the bucket)
    problems, squared = [], 0.0
    expected = []
    for bucket in range(reducer.bucket_count):
        tensors = [t for t in range(len(numels)) if reducer.ranks[0].location[t][0] == bucket]
        inputs = [np.concatenate([pristine[r][offsets[t]:offsets[t + 1]].cpu().numpy() for t in tensors])
                  for r in range(world)]
        if world == 1:
            fp32, payload, scales, _, sq = oracle.gradient_publish(inputs[0], BLOCK)
        else:
            payload, scales, fp32, sq = oracle.allreduce_bfp8(inputs, BLOCK, 1.0 / world)
        squared += sq
        expected.append((payload, scales, fp32))
    norm, c = oracle.clip_coefficient(squared, MAX_NORM)
    for bucket, (payload, scales, fp32) in enumerate(expected):
        want_scales = oracle.scale_bfp8_scales(scales, results[0].coefficient) if results[0].coefficient != 1.0 else scales
        for rank in range(world):
            arena, got_payload, got_scales = reducer.bucket_views(rank, bucket)
            if not np.array_equal(got_payload.cpu().numpy(), payload):
                problems.append(f"bucket {bucket} rank {rank}: payload")
            if not np.array_equal(got_scales.cpu().numpy().view(np.uint32), want_scales.view(np.uint32)):
                problems.append(f"bucket {bucket} rank {rank}: scales")
            if not np.array_equal(arena.cpu().numpy().view(np.uint32), fp32.view(np.uint32)):
                problems.append(f"bucket {bucket} rank {rank}: fp32")
    norm_error = abs(results[0].squared_sum - squared) / squared
    if norm_error > 1e-9 or abs(results[0].coefficient - c) > 2e-6 * c:
        problems.append(f"sum of squares {results[0].squared_sum} vs {squared}, coefficient {results[0].coefficient} vs {c}")
    for text in problems[:8]:
        print(f"PARITY: {text}", file=sys.stderr)
    wire = reducer.transport_bytes_per_step
    emit({"metric": "bfp8_bucketed_grad_allreduce_fp32_equiv_gbs", "value": world * 4.0 * total / (ms * 1e-3) / 1e9,
          "unit": UNIT, "n_gpus": len(set(devices)), "ranks": world, "steps": args.steps, "warmup": args.warmup,
          "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
          "data": "synthetic",
          "config": {"workload": "small decoder Transformer gradient (41.6 M values), bucketed BFP8 block-32 "
                                 "all-reduce + decode + clip-norm, one process driving all ranks",
                     "tensors": len(numels), "buckets": reducer.bucket_elements, "devices": devices,
                     "notifications": "one per tensor per rank, reverse order",
                     "timed": "begin_device_step .. complete() + wait(), device time per rank, max over ranks"},
          "busbw_gbs": wire / (ms * 1e-3) / 1e9, "transport_bytes_per_step": wire,
          "gpu_launches": reducer.kernel_launches * args.steps,
          "parity": {"ok": not problems, "buckets": reducer.bucket_count, "payload_scales_fp32": "exact" if not problems else "MISMATCH",
                     "norm_rel_err": norm_error, "problems": problems[:4]},
          "result": {"norm": results[0].norm, "clip_coefficient": results[0].coefficient}})
    reducer.close()
    group.close()
    return 0 if not problems else 3


def main():
    args = parse_args()
    protect_stdout()
    if args.kernels:
        time_kernels(args)
        return 0
    if args.config == 1 and args.impl != "reference":
        return run_bucketed(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        print(f"--gpus {args.gpus} needs torch.distributed.run with --nproc-per-node {args.gpus}", file=sys.stderr)
        return 2
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return 0

    import torch
    import torch.distributed as dist
    from nntrain_b200.library import load
    load()      # fails loudly when the CUDA library is missing

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()

    if args.interference:
        status = run_interference(args, world, rank, local_rank, barrier) if world > 1 else 2
    elif args.config == 2:
        status = run_bf16_bench(args, world, rank, local_rank, barrier)
    elif args.config == 3:
        status = run_sweep(args, world, rank, local_rank, barrier)
    else:
        status = run_step_bench(args, world, rank, local_rank, barrier)
    if world > 1:
        arm_exit_watchdog(status if status is not None else 0)
        dist.destroy_process_group()
        disarm_exit_watchdog()
        # everything is torn down in order; skip the interpreter's own shutdown of
        # the CUDA / NCCL libraries, which has nothing left to do for this job
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(status if status is not None else 0)
    disarm_exit_watchdog()
    return status


if __name__ == "__main__":
    sys.exit(main())
