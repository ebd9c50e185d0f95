"""OCS plan, controller, wire protocol, barrier state machine, runners.
Failures are injected on the host only: fake connectors, corrupted bytes,
missing / duplicate / mismatching READY records."""

import struct
from dataclasses import replace

import pytest
import torch

from pccl_b200 import ocs
from pccl_b200.dsl import Stream, build_graph
from pccl_b200.ocs import (OCSBarrierTimeout, OCSControlMessage, OCSControlMessageType,
                           OCSControlStatus, OCSLinkNotReady, OCSLinkState, OCSPlan,
                           OCSPlanMismatchError, OCSProtocolError, OCSRuntime, OCSSwitchResult,
                           OcsCollectivePlanRunner, OcsPhaseRunner, OcsTorchPlanRunner,
                           StaticPlanController, TorchDistributedSwitchConnector, ack_target,
                           build_ack, build_ready, build_release,
                           build_ring_allreduce_alltoall_plan,
                           build_torch_allreduce_alltoall_plan, plan_digest)

PLAN = OCSPlan(job_id="job", group_id=2, barrier_id=7, epoch_id=3, next_epoch_id=4,
               participant_ranks=(0, 1), topology_id=9, route_plan_id=11, algorithm="ring",
               backend="pccl", payload=b"route")


class FakeConnector:
    """Returns canned READY sets and switch results."""

    def __init__(self, records=None, result=None):
        self.records, self.result = records, result

    def exchange_ready(self, ready_record, group=None, timeout=None):
        return self.records(ready_record) if callable(self.records) else [ready_record]

    def commit_switch(self, plan, ready_records, group=None, timeout=None):
        return self.result or OCSSwitchResult(OCSLinkState.LINK_ALIGNED, 10, 20, 30)


def test_plan_validation_and_ready_record():
    assert PLAN.participant_bitmap == 3
    assert OCSPlan().with_default_participants(4).participant_ranks == (0, 1, 2, 3)
    for bad in (dict(algorithm="x"), dict(backend="x"), dict(route_mode="x"),
                dict(participant_ranks=(0, 0)), dict(participant_ranks=(-1,))):
        with pytest.raises(ValueError):
            OCSPlan(**bad)
    with pytest.raises(TypeError):
        OCSPlan(payload="text")
    rec = PLAN.ready_record(1, 2, arrive_seq=5, arrival_time_us=99)
    assert rec["msg_type"] == "OCS_BARRIER_READY" and rec["src_rank"] == 1
    assert rec["payload_len"] == 5 and rec["arrival_time_us"] == 99 and rec["topology_id"] == 9


def test_static_controller_cycles_and_synthesizes():
    ctl = StaticPlanController({"all_reduce": [PLAN, replace(PLAN, barrier_id=8)]})
    assert [ctl.next_plan("all_reduce", 0, 2).barrier_id for _ in range(3)] == [7, 8, 7]
    auto = [ctl.next_plan("other", 0, 4) for _ in range(2)]
    assert [p.barrier_id for p in auto] == [0, 1] and auto[0].participant_ranks == (0, 1, 2, 3)
    with pytest.raises(TypeError):
        StaticPlanController(["not a plan"])


def test_wire_format_is_fixed_128_byte_header_plus_payload_plus_crc():
    msg = build_ready(PLAN, src_rank=1, sequence=4)
    wire = msg.encode()
    assert len(wire) == 128 + len(PLAN.payload) + 4
    assert wire[:4] == b"OCSB" and wire[4:8] == bytes([1, 1, 0, 1])
    assert struct.unpack_from("!I", wire, 16)[0] == 2            # group_id after the job hash
    assert struct.unpack_from("!QQQ", wire, 20) == (7, 3, 4)      # barrier, epoch, next epoch
    assert wire[92:124] == plan_digest(PLAN) and struct.unpack_from("!I", wire, 124)[0] == 5
    back = OCSControlMessage.decode(wire)
    assert back == msg and back.matches_plan(PLAN) and back.key == msg.key
    assert not back.matches_plan(replace(PLAN, topology_id=1))
    assert plan_digest(PLAN) != plan_digest(replace(PLAN, payload=b"other"))


@pytest.mark.parametrize("mutate, message", [
    (lambda w: b"XXXX" + w[4:], "magic"),
    (lambda w: w[:4] + b"\x09" + w[5:], "version"),
    (lambda w: w[:-1], "length"),
    (lambda w: w[:60] + bytes([w[60] ^ 1]) + w[61:], "CRC32"),
    (lambda w: w[:10], "shorter"),
])
def test_corrupted_wire_messages_are_rejected(mutate, message):
    with pytest.raises(OCSProtocolError, match=message):
        OCSControlMessage.decode(mutate(build_ready(PLAN, 0).encode()))


def test_release_abort_ack():
    assert build_release(PLAN).message_type is OCSControlMessageType.RELEASE
    abort = build_release(PLAN, status=OCSControlStatus.LINK_NOT_READY)
    assert abort.message_type is OCSControlMessageType.ABORT and abort.payload == b""
    ready = build_ready(PLAN, 1, sequence=6)
    ack = OCSControlMessage.decode(build_ack(ready, src_rank=0).encode())
    assert ack_target(ack) == (OCSControlMessageType.READY, 1, 6)
    with pytest.raises(ValueError, match="ACK"):
        ack_target(ready)


def test_barrier_release_record_and_trace():
    rt = OCSRuntime(connector=FakeConnector())
    out = rt.barrier_switch(replace(PLAN, participant_ranks=(0,)))
    assert out["msg_type"] == "OCS_BARRIER_RELEASE" and out["status"] == "OK"
    assert [e["state"] for e in out["state_trace"]] == [
        "READY", "ALL_ARRIVED", "SWITCHING", "WAIT_LINK_ALIGN", "RELEASED"]
    assert set(out["timing"]) == {"ready_exchange_us", "ready_validation_us", "controller_commit_us",
                                  "release_local_us", "total_us", "controller_switch_us",
                                  "controller_link_align_us"}
    assert out["timing"]["controller_switch_us"] == 10 and rt.history == [out]


def test_injected_link_failure_aborts():
    failed = OCSSwitchResult(OCSLinkState.LINK_NOT_READY, 1, 2, None, 1, "no light")
    rt = OCSRuntime(connector=FakeConnector(result=failed))
    with pytest.raises(OCSLinkNotReady, match="LINK_NOT_READY"):
        rt.barrier_switch(replace(PLAN, participant_ranks=(0,)))
    assert rt.history[-1]["msg_type"] == "OCS_BARRIER_ABORT"
    assert rt.history[-1]["state_trace"][-1]["state"] == "FAILED"
    with pytest.raises(OCSLinkNotReady):
        OCSRuntime(connector=TorchDistributedSwitchConnector(link_ready=False)).barrier_switch(
            replace(PLAN, participant_ranks=(0,)))


@pytest.mark.parametrize("tamper, error, message", [
    (lambda me: [me, dict(me, src_rank=1, topology_id=0)], OCSPlanMismatchError, "topology_id"),
    (lambda me: [me, dict(me, src_rank=1, participant_bitmap=1)], OCSPlanMismatchError, "participant_bitmap"),
    (lambda me: [me, dict(me), dict(me, src_rank=1)], OCSPlanMismatchError, "duplicate READY"),
    (lambda me: [me], OCSBarrierTimeout, "missing READY from ranks \\[1\\]"),
    (lambda me: [me, dict(me, src_rank=1, msg_type="HELLO")], OCSPlanMismatchError, "unexpected"),
])
def test_ready_validation(tamper, error, message):
    with pytest.raises(error, match=message):
        OCSRuntime(connector=FakeConnector(records=tamper)).barrier_switch(PLAN)


def test_non_participant_and_reserved_modes():
    with pytest.raises(OCSPlanMismatchError, match="not listed"):
        OCSRuntime(connector=FakeConnector()).barrier_switch(replace(PLAN, participant_ranks=(1,)))
    with pytest.raises(NotImplementedError, match="STATIC_PLAN"):
        OCSRuntime().barrier_switch(replace(PLAN, route_mode="ID_ROUTE"))
    with pytest.raises(ValueError, match="delay_mode"):
        TorchDistributedSwitchConnector(delay_mode="nap")


class RecordingEngine:
    def __init__(self, log):
        self.log = log

    def register_operation(self, name, path):
        self.log.append(("register", name)); return True

    def execute_operation(self, name, x, out):
        self.log.append(("execute", name)); out.copy_(x + 1)

    def reset_signals(self, name):
        self.log.append(("reset", name))


class RecordingRuntime:
    def __init__(self, log):
        self.log = log

    def barrier_switch(self, plan, group=None, timeout=None):
        self.log.append(("barrier", plan.barrier_id))


def test_phase_runner_event_order(tmp_path):
    def build(op):
        op.tensor("float32", (8,))
        op.sm_copy(1, 0, 0, 4)
        op.ocs_barrier(barrier_id=5, epoch_id=0, next_epoch_id=1, participant_ranks=(0, 1),
                       topology_id=1, route_plan_id=1)
        with Stream("s"):
            op.sm_copy(1, 4, 4, 4)
    log = []
    runner = OcsPhaseRunner(RecordingEngine(log), RecordingRuntime(log), json_dir=str(tmp_path))
    prepared = runner.prepare(build_graph("g", build), "op")
    assert prepared.operation_names == ("op_phase_0", "op_phase_1")
    assert all(p.exists() for p in prepared.phase_files)
    out = runner.execute(prepared, torch.zeros(8))
    assert out.tolist() == [2.0] * 8
    assert log == [("register", "op_phase_0"), ("execute", "op_phase_0"), ("barrier", 5),
                   ("reset", "op_phase_0"), ("register", "op_phase_1"), ("execute", "op_phase_1")]
    with pytest.raises(NotImplementedError, match="blocking"):
        runner.execute(prepared, torch.zeros(8), async_op=True)
    prepared.close()
    assert all(p.exists() for p in prepared.phase_files), "caller-owned directory is kept"
    with pytest.raises(ValueError, match="OCS barrier"):
        runner.prepare(build_graph("plain", lambda op: (op.tensor("float32", (8,)), op.sm_copy(1, 0, 0, 4))))


def test_collective_plan_runner_and_builders():
    plan = build_ring_allreduce_alltoall_plan(0, 2, 64)
    assert [p.graph.collective_type for p in plan.phases] == ["allreduce", "alltoall", "allreduce"]
    assert [p.barrier_after.topology_id if p.barrier_after else None for p in plan.phases] == [1, 2, None]
    log = []
    runner = OcsCollectivePlanRunner(RecordingEngine(log), RecordingRuntime(log))
    prepared = runner.prepare(plan)
    runner.execute(prepared, torch.zeros(64))
    assert [e[0] for e in log] == ["register", "execute", "barrier", "reset"] * 2 + ["register", "execute"]
    # a second execution of the same prepared plan reuses the registrations ...
    del log[:]
    runner.execute(prepared, torch.zeros(64))
    # (and resets before the barrier: no host barrier follows that could order a later reset)
    assert [e[0] for e in log] == ["execute", "reset", "barrier"] * 2 + ["execute"]
    # ... unless the runner is told to register every time
    del log[:]
    runner.reuse_registrations = False
    runner.execute(prepared, torch.zeros(64))
    assert [e[0] for e in log] == ["register", "execute", "barrier", "reset"] * 2 + ["register", "execute"]
    switched = ocs.build_switched_allreduce_alltoall_plan(1, 4, 64)
    assert [p.graph.collective_type for p in switched.phases] == ["allreduce", "alltoall", "allreduce"]
    assert [p.barrier_after.algorithm if p.barrier_after else None for p in switched.phases] == ["auto", "auto", None]
    prepared.close()
    assert not prepared.json_dir.exists()
    with pytest.raises(RuntimeError, match="closed"):
        runner.execute(prepared, torch.zeros(64))
    with pytest.raises(ValueError, match="non-final"):
        ocs.OCSCollectivePlan(phases=(replace(plan.phases[0], barrier_after=None), plan.phases[2]))
    with pytest.raises(ValueError):
        build_ring_allreduce_alltoall_plan(0, 2, 63)
    tplan = build_torch_allreduce_alltoall_plan(2)
    assert [p.collective for p in tplan.phases] == ["all_reduce", "all_to_all_single", "all_reduce"]
    with pytest.raises(ValueError, match="unsupported torch collective"):
        ocs.TorchCollectivePhase("broadcast")
    assert isinstance(OcsTorchPlanRunner().runtime, OCSRuntime)
