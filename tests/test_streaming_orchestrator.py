"""Streaming scheduler on CPU with hand-written actors: ordering, backpressure, atomic ingress,
faults, cancellation, resource groups, stale/duplicate/orphan results, clean-up."""
import threading
import time
from concurrent.futures import Future

import pytest

from telefuser_b200.orchestrator import (
    LocalStageActor,
    StreamingActorBusyError,
    StreamingActorFailedError,
    StreamingActorHealth,
    StreamingActorState,
    StreamingEdgeSpec,
    StreamingPipelineOrchestrator,
    StreamingPipelineSpec,
    StreamingResourceGroupSpec,
    StreamingSessionStatus,
    StreamingStageSpec,
)


def three_stage_spec(capacity=2, out_capacity=2, groups=(), group_of=None):
    group_of = group_of or {}
    stages = (
        StreamingStageSpec("encode", {"request", "control"}, {"cond"}, resource_group=group_of.get("encode")),
        StreamingStageSpec("denoise", {"cond"}, {"latent"}, resource_group=group_of.get("denoise")),
        StreamingStageSpec("decode", {"latent"}, {"frames"}, resource_group=group_of.get("decode")),
    )
    edges = (
        StreamingEdgeSpec("request", "encode", None, capacity),
        StreamingEdgeSpec("control", "encode", None, capacity),
        StreamingEdgeSpec("cond", "denoise", "encode", capacity),
        StreamingEdgeSpec("latent", "decode", "denoise", capacity),
    )
    return StreamingPipelineSpec(stages, edges, frozenset({"frames"}), out_capacity, tuple(groups))


def make_actors(log=None, gates=None, fail_at=None, closes=None, mailbox=1):
    gates = gates or {}
    log = log if log is not None else []
    closes = closes if closes is not None else []

    def handler(stage, out):
        def run(inv):
            if stage in gates:
                gates[stage].wait(5)
            if fail_at == (stage, inv.key.sequence_id):
                raise RuntimeError(f"boom in {stage} at {inv.key.sequence_id}")
            log.append((stage, inv.key.session_id, inv.key.sequence_id))
            val = "+".join(str(inv.inputs[k]) for k in sorted(inv.inputs))
            return {out: f"{stage}({val})"}

        return run

    def on_close(stage):
        return lambda ctx, reason: closes.append((stage, ctx.session_id, reason.value))

    return {
        "encode": LocalStageActor("encode", handler("encode", "cond"), mailbox, on_close("encode")),
        "denoise": LocalStageActor("denoise", handler("denoise", "latent"), mailbox, on_close("denoise")),
        "decode": LocalStageActor("decode", handler("decode", "frames"), mailbox, on_close("decode")),
    }


def drain(orch, sid, n, timeout=5.0):
    out, t0 = [], time.monotonic()
    while len(out) < n and time.monotonic() - t0 < timeout:
        out.extend(orch.poll_outputs(sid))
        time.sleep(0.005)
    return out


def push_all(orch, sid, seq, timeout=5.0):
    t0 = time.monotonic()
    while not orch.try_push_inputs(sid, seq, {"request": f"r{seq}", "control": f"c{seq}"}):
        assert time.monotonic() - t0 < timeout
        time.sleep(0.002)


def test_outputs_arrive_in_order_with_values():
    log = []
    orch = StreamingPipelineOrchestrator(three_stage_spec(), make_actors(log))
    orch.create_session("s", final_sequence_id=5)
    got = []
    for i in range(6):
        push_all(orch, "s", i)
        got.extend(orch.poll_outputs("s"))
    got.extend(drain(orch, "s", 6 - len(got)))
    assert [g[0] for g in got] == list(range(6))
    assert got[3] == (3, "frames", "decode(denoise(encode(c3+r3)))")
    for stage in ("encode", "denoise", "decode"):
        assert [s for st, _, s in log if st == stage] == list(range(6))
    m = orch.session_metrics("s")
    assert m.first_output_latency_seconds is not None and m.chunk_period.count == 5
    assert m.control_to_output_latency.count == 6 and m.control_to_output_latency.p95_seconds >= 0
    assert len(orch.stage_timings("s", "denoise")) == 6
    assert orch.wait_until_idle("s")
    orch.close_session("s")
    assert orch.status("s") == StreamingSessionStatus.CLOSED and orch.diagnostics().slot_leaks == 0
    orch.close()


def test_ingress_is_atomic_and_bounded():
    gate = threading.Event()
    orch = StreamingPipelineOrchestrator(three_stage_spec(capacity=1), make_actors(gates={"encode": gate}))
    orch.create_session("s")
    assert orch.try_push_inputs("s", 0, {"request": "r0", "control": "c0"})  # taken by encode (blocked on gate)
    assert orch.try_push_inputs("s", 1, {"request": "r1", "control": "c1"})  # fills the capacity-1 edges
    assert not orch.can_push_inputs("s", ["request", "control"])
    assert not orch.try_push_inputs("s", 2, {"request": "r2", "control": "c2"})
    stats = orch.artifact_stats("s")
    assert stats.slot_count == 2 and stats.reference_count == 2  # nothing of sequence 2 was kept
    with pytest.raises(ValueError):
        orch.try_push_inputs("s", 1, {"request": "again"})
    gate.set()
    assert [g[0] for g in drain(orch, "s", 2)] == [0, 1]
    orch.close()


def test_output_backpressure_blocks_upstream_until_polled():
    orch = StreamingPipelineOrchestrator(three_stage_spec(capacity=1, out_capacity=1), make_actors())
    orch.create_session("s")
    push_all(orch, "s", 0)
    assert orch.wait_until_idle("s")
    pushed = 1
    while pushed < 8 and orch.try_push_inputs("s", pushed, {"request": "r", "control": "c"}):
        pushed += 1
        orch.wait_until_idle("s", 1.0)
    assert pushed < 8  # the pipeline filled up because nobody polled
    assert orch.wait_until_idle("s")
    first = orch.poll_outputs("s")
    assert [f[0] for f in first] == [0]
    rest = drain(orch, "s", pushed - 1)
    assert [r[0] for r in rest] == list(range(1, pushed))
    idle = orch.stage_idle_intervals("s", "decode")
    assert any(i.reason in ("output_backpressure", "waiting_for_inputs", "scheduler") for i in idle)
    orch.close()


@pytest.mark.parametrize("stage", ["encode", "denoise", "decode"])
def test_stage_fault_fails_session_and_cleans_up(stage):
    closes = []
    orch = StreamingPipelineOrchestrator(three_stage_spec(), make_actors(fail_at=(stage, 1), closes=closes))
    orch.create_session("s")
    push_all(orch, "s", 0)
    push_all(orch, "s", 1)
    t0 = time.monotonic()
    while orch.status("s") == StreamingSessionStatus.RUNNING and time.monotonic() - t0 < 5:
        time.sleep(0.01)
    assert orch.status("s") == StreamingSessionStatus.FAILED
    assert "boom" in repr(orch.error("s")) or "boom" in repr(orch.error("s").__cause__)
    with pytest.raises(RuntimeError):
        orch.try_push_inputs("s", 2, {"request": "r", "control": "c"})
    assert orch.actor_health(stage).state == StreamingActorState.FAILED
    t0 = time.monotonic()
    while len(closes) < 3 and time.monotonic() - t0 < 5:
        time.sleep(0.01)
    assert [c[0] for c in closes] == ["decode", "denoise", "encode"] and all(c[2] == "failed" for c in closes)
    orch.close()


def test_cancel_drains_in_flight_work_and_late_result_is_ignored():
    gate = threading.Event()
    closes = []
    orch = StreamingPipelineOrchestrator(three_stage_spec(), make_actors(gates={"denoise": gate}, closes=closes))
    orch.create_session("s")
    push_all(orch, "s", 0)
    time.sleep(0.05)
    threading.Timer(0.2, gate.set).start()
    orch.cancel_session("s", timeout=5.0)
    assert orch.status("s") == StreamingSessionStatus.CANCELLED
    assert orch.poll_outputs("s") == [] and orch.artifact_stats("s").slot_count == 0
    assert [c[0] for c in closes] == ["decode", "denoise", "encode"] and closes[0][2] == "cancelled"
    epoch2 = orch.create_session("s")
    assert epoch2 == 2
    push_all(orch, "s", 0)
    assert [g[0] for g in drain(orch, "s", 1)] == [0]
    orch.close()


class ManualActor:
    """Actor whose futures the test resolves by hand."""

    def __init__(self):
        self.calls = []
        self.closed_sessions = []

    def submit(self, invocation):
        f = Future()
        self.calls.append((invocation, f))
        return f

    def health(self):
        return StreamingActorHealth(StreamingActorState.RUNNING, 0)

    def barrier(self, timeout=5.0):
        return None

    def close_session(self, context, reason, timeout=5.0):
        self.closed_sessions.append((context.session_id, context.session_epoch, reason.value))

    def close(self):
        return None


def single_stage():
    spec = StreamingPipelineSpec((StreamingStageSpec("work", {"x"}, {"y"}),), (StreamingEdgeSpec("x", "work", None, 2),),
                                 frozenset({"y"}), 2)
    actor = ManualActor()
    return StreamingPipelineOrchestrator(spec, {"work": actor}), actor


def test_stale_duplicate_and_orphan_results_are_counted_not_applied():
    orch, actor = single_stage()
    orch.create_session("s")
    orch.push_input("s", 0, "x", 1)
    inv0, fut0 = actor.calls[0]
    orch.cancel_session("s", timeout=0.05)  # result still outstanding: epoch is bumped
    orch.create_session("s")
    orch.push_input("s", 0, "x", 2)
    fut0.set_result({"y": "old"})
    assert orch.diagnostics().stale_epoch_results == 1 and orch.poll_outputs("s") == []
    inv1, fut1 = actor.calls[1]
    fut1.set_result({"y": "new"})
    assert orch.poll_outputs("s") == [(0, "y", "new")]
    orch._complete("s", inv1.key, fut1)
    assert orch.diagnostics().duplicate_results == 1
    orch._complete("ghost", inv1.key, fut1)
    assert orch.diagnostics().orphaned_results == 1
    orch.close()


def test_wrong_output_names_fail_the_session():
    orch, actor = single_stage()
    orch.create_session("s")
    orch.push_input("s", 0, "x", 1)
    actor.calls[0][1].set_result({"z": 1})
    assert orch.status("s") == StreamingSessionStatus.FAILED and "expected exactly" in str(orch.error("s"))
    orch.close()


def test_resource_group_serialises_stages_that_share_a_device():
    running, peak, lock = [0], [0], threading.Lock()

    def handler(out):
        def run(inv):
            with lock:
                running[0] += 1
                peak[0] = max(peak[0], running[0])
            time.sleep(0.02)
            with lock:
                running[0] -= 1
            return {out: 1}

        return run

    spec = three_stage_spec(groups=(StreamingResourceGroupSpec("gpu0", 1),),
                            group_of={"encode": "gpu0", "denoise": "gpu0", "decode": "gpu0"})
    actors = {"encode": LocalStageActor("encode", handler("cond")), "denoise": LocalStageActor("denoise", handler("latent")),
              "decode": LocalStageActor("decode", handler("frames"))}
    orch = StreamingPipelineOrchestrator(spec, actors)
    orch.create_session("a")
    orch.create_session("b")
    for i in range(3):
        push_all(orch, "a", i)
        push_all(orch, "b", i)
        drain(orch, "a", 1, 0.2)
        drain(orch, "b", 1, 0.2)
    orch.barrier(5.0)
    assert peak[0] == 1 and orch.resource_group_usage("gpu0") == 0
    orch.close()


def test_cleanup_failure_is_retried_in_background():
    attempts = []

    def flaky_close(ctx, reason):
        attempts.append(reason.value)
        if len(attempts) < 3:
            raise RuntimeError("cannot free yet")

    spec = StreamingPipelineSpec((StreamingStageSpec("work", {"x"}, {"y"}),), (StreamingEdgeSpec("x", "work", None, 2),),
                                 frozenset({"y"}), 2)
    actor = LocalStageActor("work", lambda inv: {"y": inv.inputs["x"]}, 1, flaky_close)
    orch = StreamingPipelineOrchestrator(spec, {"work": actor})
    orch.create_session("s")
    orch.push_input("s", 0, "x", 7)
    assert drain(orch, "s", 1) == [(0, "y", 7)]
    orch.close_session("s")
    assert orch.cleanup_error("s") is not None
    t0 = time.monotonic()
    while orch.cleanup_error("s") is not None and time.monotonic() - t0 < 5:
        time.sleep(0.02)
    assert orch.cleanup_error("s") is None and len(attempts) == 3
    assert orch.diagnostics().cleanup_failures >= 1
    orch.close()


def test_spec_validation():
    a = {"work": ManualActor(), "b": ManualActor()}
    with pytest.raises(ValueError, match="no edge delivers"):
        StreamingPipelineOrchestrator(StreamingPipelineSpec((StreamingStageSpec("work", {"x"}, {"y"}),), (), {"y"}), a)
    with pytest.raises(ValueError, match="more than one producer"):
        StreamingPipelineOrchestrator(StreamingPipelineSpec(
            (StreamingStageSpec("work", {"x"}, {"y"}), StreamingStageSpec("b", {"x"}, {"y"})),
            (StreamingEdgeSpec("x", "work"), StreamingEdgeSpec("x", "b")), {"y"}), a)
    with pytest.raises(ValueError, match="cycle"):
        StreamingPipelineOrchestrator(StreamingPipelineSpec(
            (StreamingStageSpec("work", {"p"}, {"q"}), StreamingStageSpec("b", {"q"}, {"p"})),
            (StreamingEdgeSpec("q", "b", "work"), StreamingEdgeSpec("p", "work", "b")), set()), a)
    with pytest.raises(ValueError, match="neither consumed nor an output"):
        StreamingPipelineOrchestrator(StreamingPipelineSpec((StreamingStageSpec("work", {"x"}, {"y"}),),
                                                            (StreamingEdgeSpec("x", "work"),), set()), a)
    with pytest.raises(ValueError, match="no actor"):
        StreamingPipelineOrchestrator(StreamingPipelineSpec((StreamingStageSpec("zzz", {"x"}, {"y"}),),
                                                            (StreamingEdgeSpec("x", "zzz"),), {"y"}), a)
    with pytest.raises(ValueError):
        StreamingStageSpec("s", {"x"}, {"y"}, max_in_flight_per_session=2)


def test_local_actor_mailbox_and_failure():
    gate = threading.Event()
    actor = LocalStageActor("a", lambda inv: gate.wait(5) and {"y": 1}, mailbox_size=1)
    from telefuser_b200.orchestrator import StreamingStageInvocation, StreamingTaskKey

    inv = StreamingStageInvocation(StreamingTaskKey("s", 1, 0, "a", "r"), {}, True, False)
    f = actor.submit(inv)
    with pytest.raises(StreamingActorBusyError):
        actor.submit(inv)
    assert actor.health().pending_invocations == 1
    gate.set()
    assert f.result(2) == {"y": 1}
    actor.barrier()
    actor.close()
    with pytest.raises(StreamingActorFailedError):
        actor.submit(inv)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_sessions_with_jitter_cancellations_and_shared_devices_leave_nothing_behind(seed):
    """Several sessions at once through actors with random delays, stages sharing a resource group, some sessions
    cancelled mid-flight and re-created: every surviving session gets every chunk exactly once and in order with the
    right value, and the scheduler ends with no slot, no reference, no leak and no unexplained result."""
    import random

    rng = random.Random(seed)
    groups = (StreamingResourceGroupSpec("gpu0", 1),)
    spec = three_stage_spec(capacity=rng.choice([1, 2, 3]), out_capacity=rng.choice([1, 2]), groups=groups,
                            group_of={"encode": "gpu0", "decode": "gpu0"})  # fmt: skip
    delays = {st: rng.uniform(0.0, 0.004) for st in ("encode", "denoise", "decode")}
    running = {"gpu0": 0, "max": 0}
    lock = threading.Lock()

    def handler(stage, out):
        def run(inv):
            shared = stage in ("encode", "decode")
            if shared:
                with lock:
                    running["gpu0"] += 1
                    running["max"] = max(running["max"], running["gpu0"])
            time.sleep(delays[stage] * rng.random())
            if shared:
                with lock:
                    running["gpu0"] -= 1
            val = "+".join(str(inv.inputs[k]) for k in sorted(inv.inputs))
            return {out: f"{stage}({val})"}

        return run

    actors = {"encode": LocalStageActor("encode", handler("encode", "cond"), 2),
              "denoise": LocalStageActor("denoise", handler("denoise", "latent"), 2),
              "decode": LocalStageActor("decode", handler("decode", "frames"), 2)}  # fmt: skip
    orch = StreamingPipelineOrchestrator(spec, actors)
    n_chunks = 12
    sessions = [f"s{i}" for i in range(4)]
    cancel_at = {"s1": rng.randrange(2, 8), "s3": rng.randrange(2, 8)}  # pushed chunks after which the session is cancelled once
    got = {s: [] for s in sessions}
    nxt = {s: 0 for s in sessions}
    cancelled_once = set()
    for s in sessions:
        orch.create_session(s, final_sequence_id=n_chunks - 1)
    deadline = time.monotonic() + 60
    while any(len(got[s]) < n_chunks for s in sessions):
        assert time.monotonic() < deadline, {s: len(v) for s, v in got.items()}
        for s in rng.sample(sessions, len(sessions)):
            if s in cancel_at and s not in cancelled_once and nxt[s] >= cancel_at[s]:
                orch.cancel_session(s, timeout=10.0)
                assert orch.status(s) == StreamingSessionStatus.CANCELLED and orch.artifact_stats(s).slot_count == 0
                cancelled_once.add(s)
                assert orch.create_session(s, final_sequence_id=n_chunks - 1) == 2  # a new epoch of the same id
                got[s], nxt[s] = [], 0
                continue
            if nxt[s] < n_chunks and orch.try_push_inputs(s, nxt[s], {"request": f"{s}r{nxt[s]}", "control": f"c{nxt[s]}"}):
                nxt[s] += 1
            if rng.random() < 0.7:
                got[s].extend(orch.poll_outputs(s))
        time.sleep(0.0005)
    for s in sessions:
        assert [g[0] for g in got[s]] == list(range(n_chunks)), s
        assert all(g == (i, "frames", f"decode(denoise(encode(c{i}+{s}r{i})))") for i, g in enumerate(got[s])), s
        assert orch.wait_until_idle(s)
        orch.close_session(s)
        assert orch.status(s) == StreamingSessionStatus.CLOSED
        st = orch.artifact_stats(s)
        assert st.slot_count == 0 and st.reference_count == 0
    d = orch.diagnostics()
    assert d.slot_leaks == 0 and d.cleanup_failures == 0 and d.duplicate_results == 0 and d.orphaned_results == 0
    assert running["max"] == 1  # the two stages that share a device never ran at the same time
    assert orch.resource_group_usage("gpu0") == 0
    orch.close()
