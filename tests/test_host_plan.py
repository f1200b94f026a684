"""Host-side reducer bookkeeping (no GPU): bucket layout, the exactly-once
publication state machine, step lifecycle, reduction stamps and the optimizer
guard, following the reference's own host-logic tests."""
import pytest

from nntrain_b200.host_plan import (REDUCED, ArgumentError, CapturedGradientPublicationState, GradientStepPlan,
                                    InvalidOperationError, build_buckets, clip_decision)


def decoder_tensor_list():
    # the 41.6 M-value decoder of benchmark configuration 1: token embedding,
    # 8 layers of {qkv, out, ln, ffn in, ffn out, ln}, final ln
    layer = [512 * 1536, 1536, 512 * 512, 512, 512, 512, 512 * 2048, 2048, 2048 * 512, 512, 512, 512]
    return [32000 * 512] + layer * 8 + [512, 512]


def test_bucket_layout_never_splits_a_tensor():
    # NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:1647-1678
    numels = decoder_tensor_list()
    assert sum(numels) == 41_604_096
    placement, count = build_buckets(numels, 4 << 20)
    sizes = [0] * count
    for n, (bucket, offset) in zip(numels, placement):
        assert offset == sizes[bucket]          # running sum, no padding
        sizes[bucket] += n
    assert sizes == [16_384_000, 3_940_352, 3_416_064, 3_152_384, 3_152_384, 3_152_384, 3_152_384, 3_152_384,
                     2_101_760]
    assert [b for b, _ in placement] == sorted(b for b, _ in placement)
    placement, count = build_buckets([10, 20, 30], 25)       # 10+20 > 25: [10], [20], [30]
    assert count == 3 and [p[0] for p in placement] == [0, 1, 2]
    placement, count = build_buckets([10, 15, 1, 1], 25)      # closes exactly at the target
    assert count == 2 and placement == [(0, 0), (0, 10), (1, 0), (1, 1)]
    with pytest.raises(ArgumentError):
        build_buckets([4, 0], 8)


def test_captured_publication_requires_begun_current_step_and_is_exactly_once():
    # NNtrain.Core.Tests/CudaCapturedGradientPublicationStateTests.cs:6-36
    state = CapturedGradientPublicationState(2)
    state.begin_step(17)
    with pytest.raises(InvalidOperationError):
        state.begin_captured_publication(17, 0, 3)
    state.mark_device_begun(17, 0, 3)
    state.mark_device_begun(17, 1, 7)
    with pytest.raises(InvalidOperationError):
        state.begin_captured_publication(16, 0, 3)
    with pytest.raises(InvalidOperationError):
        state.begin_captured_publication(18, 0, 3)
    state.begin_captured_publication(17, 0, 3)
    state.complete_captured_publication(17, 0, 3)
    with pytest.raises(InvalidOperationError, match="twice"):
        state.begin_captured_publication(17, 0, 3)
    with pytest.raises(InvalidOperationError, match="mix"):
        state.enter_notification_path(17, 1, 7)
    state.begin_captured_publication(17, 1, 7)
    state.complete_captured_publication(17, 1, 7)
    state.validate_complete(17)
    state.end_step(17)


def test_capture_recording_suppresses_other_paths_and_must_be_discarded():
    # NNtrain.Core.Tests/CudaCapturedGradientPublicationStateTests.cs:38-67
    state = CapturedGradientPublicationState(2)
    state.begin_step(23)
    state.mark_device_begun(23, 0, 0)
    state.mark_device_begun(23, 1, 1)
    state.begin_capture_recording(23, 0, 0)
    assert state.is_capture_recording(23, 0)
    state.enter_capture_notification_path(23, 0, 0)
    for forbidden in (lambda: state.enter_notification_path(23, 1, 1),
                      lambda: state.begin_captured_publication(23, 1, 1),
                      lambda: state.validate_complete(23),
                      lambda: state.validate_capture_discard(23)):
        with pytest.raises(InvalidOperationError):
            forbidden()
    state.end_capture_recording(23, 0, 0)
    state.validate_capture_discard(23)
    state.end_step(23)
    state.begin_step(24)
    state.mark_device_begun(24, 0, 0)
    state.enter_notification_path(24, 0, 0)
    state.validate_complete(24)
    state.end_step(24)


def test_mid_publication_failure_requires_abort_generation_before_reuse():
    # NNtrain.Core.Tests/CudaCapturedGradientPublicationStateTests.cs:69-95
    state = CapturedGradientPublicationState(2)
    state.begin_step(31)
    state.mark_device_begun(31, 0, 0)
    state.mark_device_begun(31, 1, 1)
    state.begin_captured_publication(31, 0, 0)
    state.fail_captured_publication(31, 0)
    with pytest.raises(InvalidOperationError):
        state.begin_captured_publication(31, 1, 1)
    with pytest.raises(InvalidOperationError):
        state.validate_complete(31)
    state.end_step(31)
    state.begin_step(32)
    for slot in (0, 1):
        state.mark_device_begun(32, slot, slot)
    for slot in (0, 1):
        state.begin_captured_publication(32, slot, slot)
        state.complete_captured_publication(32, slot, slot)
    state.validate_complete(32)
    state.end_step(32)
    with pytest.raises(InvalidOperationError):
        state.begin_step(33) or state.begin_step(34)      # a second begin while active


def reduce_once(plan: GradientStepPlan, order=None) -> list[int]:
    """Runs one whole step; returns the order buckets were enqueued in."""
    step = plan.begin_step()
    plan.begin_device_step(step)
    tensors = list(range(len(decoder_tensor_list()))) if order is None else order
    enqueued = []
    for tensor in tensors:
        plan.notify_gradient_ready(tensor, step)
        while (bucket := plan.next_enqueueable(step)) >= 0:
            enqueued.append(bucket)
    plan.complete(step)
    return enqueued


def test_step_lifecycle_duplicate_notification_abort_and_recover():
    # NNtrain.Core.Tests/CudaGradientCoherenceTests.cs:74-113,
    # CudaBfp8GradientReducerTests.cs:59-93
    plan = GradientStepPlan(decoder_tensor_list(), devices=[0, 1])
    assert plan.bucket_count == 9
    failed = plan.begin_step()
    with pytest.raises(InvalidOperationError, match="still active"):
        plan.begin_step()
    with pytest.raises(InvalidOperationError, match="not begun"):
        plan.notify_gradient_ready(0, failed)
    plan.begin_device_step(failed)
    with pytest.raises(InvalidOperationError, match="twice"):
        plan.begin_device_step(failed)
    plan.notify_gradient_ready(5, failed)
    with pytest.raises(InvalidOperationError, match="notified twice"):
        plan.notify_gradient_ready(5, failed)
    with pytest.raises(InvalidOperationError, match="not completed"):
        plan.complete(failed)                       # buckets still outstanding
    assert plan.coherence_snapshot(5)["pending_step"] == failed
    plan.abort(failed)
    assert plan.coherence_snapshot(5)["pending_step"] == 0
    with pytest.raises(InvalidOperationError, match="not active"):
        plan.notify_gradient_ready(6, failed)
    order = reduce_once(plan)
    assert order == list(range(8, -1, -1))          # fixed order, descending bucket index
    snapshot = plan.coherence_snapshot(5)
    assert snapshot["kind"] == REDUCED and snapshot["stamp"][1] == 2 and plan.completed_steps == 1
    plan.close()


def test_non_finite_step_fails_complete_and_stays_abortable():
    # NNtrain.Core.Tests/CudaBfp8GradientReducerTests.cs:95-130
    plan = GradientStepPlan([100, 200], devices=[0, 1], target_bucket_elements=1000)
    step = plan.begin_step()
    plan.begin_device_step(step)
    for tensor in (1, 0):
        plan.notify_gradient_ready(tensor, step)
    assert plan.next_enqueueable(step) == 0
    with pytest.raises(InvalidOperationError, match="non-finite"):
        plan.complete(step, non_finite=True)
    plan.abort(step)
    with pytest.raises(InvalidOperationError, match="has not been reduced"):
        plan.optimizer_validate_and_consume()
    plan.close()


def test_optimizer_guard_is_fail_closed():
    # NNtrain.Core.Tests/CudaGradientCoherenceTests.cs:6-72,115-150;
    # NNtrain.Core/Training/CudaGradientCoherence.cs:61-173
    plan = GradientStepPlan([64, 64, 64], devices=[0, 1], target_bucket_elements=100)
    with pytest.raises(InvalidOperationError, match="already consumed|has not been reduced"):
        plan.optimizer_validate_and_consume()               # nothing was ever produced
    step = plan.begin_step()
    with pytest.raises(InvalidOperationError, match="incomplete reduction step"):
        plan.optimizer_validate_and_consume()
    plan.abort(step)
    reduce_once(plan, order=[2, 1, 0])
    with pytest.raises(InvalidOperationError, match="has not been reduced"):
        plan.optimizer_validate_and_consume([0, 2])          # another device set
    with pytest.raises(InvalidOperationError, match="unique"):
        plan.optimizer_validate_and_consume([0, 0])
    plan.optimizer_validate_and_consume()
    with pytest.raises(InvalidOperationError, match="already consumed"):
        plan.optimizer_validate_and_consume()                # the same gradients twice
    reduce_once(plan, order=[0, 1, 2])
    plan.optimizer_validate_and_consume()
    # a rebuilt reducer invalidates the old, unconsumed stamp
    reduce_once(plan, order=[0, 1, 2])
    rebuilt = GradientStepPlan([64, 64, 64], devices=[0, 1], target_bucket_elements=100)
    with pytest.raises(InvalidOperationError, match="has not been reduced"):
        plan.optimizer_validate_and_consume()
    rebuilt.close()
    plan.close()


def test_transport_bytes_formula():
    # 2 devices, block 128: 2 * (E + 4 * ceil(E / 128)) per pair, i.e. half per
    # rank (NNtrain.Core.Tests/CudaMix8GradientTransportTests.cs:267-270)
    numels = [515, 300, 1000]
    plan = GradientStepPlan(numels, devices=[0, 1], target_bucket_elements=1 << 20, block_size=128)
    e = sum(numels)
    assert plan.transport_bytes_per_step == (e + 4 * ((e + 127) // 128))
    plan.close()
    plan = GradientStepPlan(numels, devices=list(range(8)), target_bucket_elements=1 << 20, block_size=32)
    assert plan.transport_bytes_per_step == 2 * 7 * (e + 4 * ((e + 31) // 32)) // 8
    plan.close()


def test_fused_squared_sum_cache_is_one_shot_and_version_checked(oracle):
    # NNtrain.Core/Tensors/Tensor.CudaKernels.cs:768-854;
    # NNtrain.Core.Tests/CudaBfp8GradientClipNormTests.cs:192-200 (a hit costs no kernel)
    plan = GradientStepPlan([64, 64], devices=[0, 1], target_bucket_elements=1000)
    assert plan.try_consume_squared_sum() is None
    reduce_once(plan, order=[1, 0])
    plan.publish_squared_sum(12.5)
    assert plan.try_consume_squared_sum([0, 2]) is None      # other device set: miss, and the entry is gone
    assert plan.try_consume_squared_sum() is None
    plan.publish_squared_sum(12.5)
    assert plan.try_consume_squared_sum() == 12.5
    assert plan.try_consume_squared_sum() is None            # one shot
    plan.publish_squared_sum(float("nan"))                    # never cached
    assert plan.try_consume_squared_sum() is None
    plan.publish_squared_sum(3.0)
    reduce_once(plan, order=[0, 1])                           # gradients changed since
    assert plan.try_consume_squared_sum() is None
    plan.close()
    # the clip decision itself, against the oracle's restatement of nn.cs:62-81
    for squared_sum, max_norm in ((1e-6, 1.0), (4.0, 1.0), (1066.2 ** 2, 1.0), (0.0, 0.5)):
        norm, c = clip_decision(squared_sum, max_norm)
        expect_norm, expect_c = oracle.clip_coefficient(squared_sum, max_norm)
        assert norm == expect_norm and c == expect_c
    with pytest.raises(ArgumentError):
        clip_decision(1.0, 0.0)


def test_hundred_lifecycles_with_injected_host_faults_leave_no_state_behind():
    # after NNtrain.Core.Tests/CudaGradientHostPipelineStressTests.cs:9-171: step
    # lifecycles with faults injected on the host (early abort, abort after some
    # buckets, duplicate notification, non-finite completion); the plan must
    # reopen cleanly every time and count only the completed steps
    import random
    numels = decoder_tensor_list()
    plan = GradientStepPlan(numels, devices=[0, 1, 2, 3])
    rng = random.Random(20240917)
    completed = 0
    for lifecycle in range(100):
        fault = rng.choice(("none", "early_abort", "mid_abort", "duplicate", "non_finite"))
        step = plan.begin_step()
        if fault == "early_abort":
            plan.abort(step)
            continue
        plan.begin_device_step(step)
        order = list(range(len(numels)))
        rng.shuffle(order)
        stop_after = rng.randrange(1, len(order)) if fault in ("mid_abort", "duplicate") else len(order)
        enqueued = []
        for tensor in order[:stop_after]:
            plan.notify_gradient_ready(tensor, step)
            while (bucket := plan.next_enqueueable(step)) >= 0:
                enqueued.append(bucket)
        assert enqueued == sorted(enqueued, reverse=True)
        if fault == "duplicate":
            with pytest.raises(InvalidOperationError, match="notified twice"):
                plan.notify_gradient_ready(order[0], step)
        if fault in ("mid_abort", "duplicate"):
            with pytest.raises(InvalidOperationError):
                plan.complete(step)
            plan.abort(step)
            assert plan.coherence_snapshot(0)["pending_step"] == 0
            continue
        if fault == "non_finite":
            with pytest.raises(InvalidOperationError, match="non-finite"):
                plan.complete(step, non_finite=True)
            plan.abort(step)
            continue
        plan.complete(step)
        completed += 1
        plan.optimizer_validate_and_consume()
    assert plan.completed_steps == completed > 10
    plan.close()


def test_concurrent_notifications_are_exactly_once():
    # leaves are notified from several host threads (the reference has one
    # worker thread per device plus the autograd thread); every tensor must be
    # accepted exactly once and every bucket become ready exactly once
    import threading
    numels = [1000] * 400
    plan = GradientStepPlan(numels, devices=[0, 1], target_bucket_elements=10_000)
    step = plan.begin_step()
    plan.begin_device_step(step)
    accepted, rejected, ready = [], [], []
    lock = threading.Lock()

    def worker(seed: int) -> None:
        import random
        order = list(range(len(numels)))
        random.Random(seed).shuffle(order)
        for tensor in order:
            try:
                bucket = plan.notify_gradient_ready(tensor, step)
                with lock:
                    accepted.append(tensor)
                    if bucket >= 0:
                        ready.append(bucket)
            except InvalidOperationError:
                with lock:
                    rejected.append(tensor)

    threads = [threading.Thread(target=worker, args=(seed,)) for seed in range(4)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    assert sorted(accepted) == list(range(len(numels)))          # each tensor once
    assert len(rejected) == 3 * len(numels)                      # every other attempt refused
    assert sorted(ready) == list(range(plan.bucket_count))       # each bucket ready once
    enqueued = []
    while (bucket := plan.next_enqueueable(step)) >= 0:
        enqueued.append(bucket)
    assert enqueued == list(range(plan.bucket_count - 1, -1, -1))
    plan.complete(step)
    plan.close()


def test_bucket_layouts_of_the_benchmark_tensor_lists():
    """BuildBuckets (NNtrain.Core/Training/CudaBFloat16GradientAllReduce.cs:1647-1678: target 4 Mi elements,
    tensors never split, in parameter order) on the three model-shaped lists of the benchmark configurations."""
    from nntrain_b200.bucketed import small_transformer_numels
    from nntrain_b200.host_plan import build_buckets

    def sizes(numels):
        located, count = build_buckets(numels, 4 << 20)
        out = [0] * count
        for (bucket, offset), n in zip(located, numels):
            assert offset == out[bucket]              # running-sum offsets inside the bucket, no padding
            out[bucket] += n
        return out

    small = sizes(small_transformer_numels())
    assert small == [16_384_000, 3_940_352, 3_416_064] + [3_152_384] * 5 + [2_101_760]
    hidden, layers, kv, inter, vocab = 1536, 28, 256, 8960, 151936
    qwen = [vocab * hidden]
    for _ in range(layers):
        qwen += [hidden * hidden, hidden, hidden * kv, kv, hidden * kv, kv, hidden * hidden,
                 hidden * inter, hidden * inter, inter * hidden, hidden, hidden]
    qwen += [hidden]
    q = sizes(qwen)
    assert sum(q) == 1_543_714_304 and len(q) == 142 and max(q) == 233_373_696 and min(q) == 4_608
    gpt2 = [50257 * 768, 1024 * 768]
    for _ in range(12):
        gpt2 += [768 * 2304, 2304, 768 * 768, 768, 768, 768, 768 * 3072, 3072, 3072 * 768, 768, 768, 768]
    gpt2 += [768, 768]
    g = sizes(gpt2)
    assert sum(g) == 124_439_808 and len(g) == 26 and max(g) == 38_597_376
