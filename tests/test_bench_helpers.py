"""Host-side helpers of the benchmark that need no GPU: the windows its parity
check compares with the oracle, and the tensor list of the whole-bucket cases."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.mark.parametrize("world", (1, 2, 4, 8))
def test_parity_windows_are_block_aligned_and_straddle_every_boundary(bench, world):
    elements = bench.QWEN2_1P5B_ELEMENTS
    align = 512 * world
    fractions = (0.03, 0.10, 0.26, 0.26, 0.20, 0.09)
    spans, start = [], 0
    for f in fractions:
        length = int(elements * f) // align * align
        spans.append((start, start + length))
        start += length
    spans.append((start, elements))
    if world == 1:
        spans = [(0, elements)]
    windows = bench.parity_windows(elements, spans, world, 32)
    assert len(set(windows)) == len(windows)
    for a, b in windows:
        assert 0 <= a < b <= elements and a % 32 == 0
        assert b - a <= bench.PARITY_WINDOW + 32
    assert windows[0][0] == 0 and any(b == elements for _, b in windows)       # start and ragged tail
    for boundary, _ in spans[1:]:                                               # every chunk boundary is inside a window
        assert any(a < boundary < b for a, b in windows)
    if world > 1:
        largest = max(spans, key=lambda s: s[1] - s[0])
        shard = ((largest[1] - largest[0] + world - 1) // world + 511) // 512 * 512
        assert any(a < largest[0] + shard < b for a, b in windows)              # a shard boundary inside a chunk


def test_small_arena_windows(bench):
    windows = bench.parity_windows(70001, [(0, 70001)], 2, 32)
    assert all(0 <= a < b <= 70001 and a % 32 == 0 for a, b in windows)
    assert any(b == 70001 for _, b in windows)


def test_scaled_tensor_list_keeps_count_and_total(bench):
    for total in (1 << 20, 64 << 20, bench.QWEN2_1P5B_ELEMENTS):
        numels = bench.qwen2_shaped_numels(total)
        assert len(numels) == 338 and sum(numels) == total and min(numels) >= 1


def test_reference_arm_under_the_launcher_prints_one_line_from_rank_zero():
    """`bench.py --impl reference` launched as N ranks: rank 0 alone times the
    CPU restatement and prints the line, the other ranks leave with status 0."""
    import json
    import socket
    import subprocess
    import sys
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    done = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", str(port), os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
         "--steps", "1", "--warmup", "1", "--cpu-sample-elements", "65536"],
        capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["unit"] == "GB/s"
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] == "port"
    assert line["gpu_launches"] == 0 and line["value"] > 0
