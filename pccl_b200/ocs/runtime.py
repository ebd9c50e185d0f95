"""The OCS barrier: READY exchange -> validation -> switch commit -> release.

One barrier walks the states ``READY -> ALL_ARRIVED -> SWITCHING ->
WAIT_LINK_ALIGN -> RELEASED`` (or ``FAILED``).  Transport is behind the
``SwitchConnector`` protocol: ``exchange_ready`` gathers every participant's
READY record, ``commit_switch`` asks the switch to apply the plan and reports
whether the links came up aligned (reference: pccl/ocs/runtime.py:55-117 states
and protocol, :120-214 torch mock connector, :217-458 runtime, :461-498 helpers).

Connectors here:

* ``TorchDistributedSwitchConnector`` — object collectives of the process
  group; the lowest participant plays the switch (optionally with injected
  delays or an injected link failure).
* ``TensorSwitchConnector`` — same contract on a fixed-size tensor
  ``all_gather`` of the READY digests instead of pickled dictionaries; about an
  order of magnitude less host work per barrier, for back-to-back barriers.
"""

from __future__ import annotations

import hashlib
import json
import operator
import time
from dataclasses import dataclass
from enum import Enum
from typing import Any, Dict, List, Optional, Protocol, Sequence, Tuple, runtime_checkable

import torch
import torch.distributed as dist

from .controller import OCSPlanController, StaticPlanController
from .exceptions import OCSBarrierTimeout, OCSLinkNotReady, OCSPlanMismatchError
from .plan import OCSPlan

#: fields compared one by one between a READY record and the local plan
CONSISTENCY_FIELDS = ("job_id", "group_id", "barrier_id", "epoch_id", "next_epoch_id",
                      "topology_id", "route_mode", "route_plan_id", "algorithm", "backend")


_COMPARED_FIELDS = (*CONSISTENCY_FIELDS, "participant_bitmap")
_compared_values = operator.itemgetter(*_COMPARED_FIELDS)


def _time_us() -> int:
    return time.time_ns() // 1000


def _monotonic_ns() -> int:
    return time.perf_counter_ns()


def _duration_us(start_ns: int, end_ns: int) -> float:
    return max(0.0, (int(end_ns) - int(start_ns)) / 1_000.0)


def _dist_ready() -> bool:
    return dist.is_available() and dist.is_initialized()


def _rank_world_size(group: Optional[dist.ProcessGroup] = None) -> Tuple[int, int]:
    if not _dist_ready():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


class OCSBarrierState(str, Enum):
    READY = "READY"
    ALL_ARRIVED = "ALL_ARRIVED"
    SWITCHING = "SWITCHING"
    WAIT_LINK_ALIGN = "WAIT_LINK_ALIGN"
    RELEASED = "RELEASED"
    FAILED = "FAILED"


class OCSLinkState(str, Enum):
    OCS_CONFIG_ACCEPTED = "OCS_CONFIG_ACCEPTED"
    OCS_SWITCH_DONE = "OCS_SWITCH_DONE"
    LINK_ALIGNED = "LINK_ALIGNED"
    LINK_NOT_READY = "LINK_NOT_READY"


@dataclass(frozen=True)
class OCSSwitchResult:
    """What the switch reports after a commit.  ``*_time_us`` are wall-clock,
    ``*_mono_ns`` are the leader's monotonic clock (used only for durations)."""

    link_state: OCSLinkState
    switch_start_time_us: int
    switch_done_time_us: int
    link_ready_time_us: Optional[int]
    error_code: int = 0
    error_message: str = ""
    switch_start_mono_ns: Optional[int] = None
    switch_done_mono_ns: Optional[int] = None
    link_ready_mono_ns: Optional[int] = None

    @property
    def is_link_ready(self) -> bool:
        return self.link_state is OCSLinkState.LINK_ALIGNED


def _state_event(state: OCSBarrierState, timestamp_us: int) -> Dict[str, Any]:
    return {"state": state.value, "time_us": int(timestamp_us)}


@runtime_checkable
class SwitchConnector(Protocol):
    def exchange_ready(self, ready_record: Dict[str, Any],
                       group: Optional[dist.ProcessGroup] = None,
                       timeout: Optional[float] = None) -> List[Dict[str, Any]]:
        """Contribute this rank's READY and return all READY records seen."""

    def commit_switch(self, plan: OCSPlan, ready_records: Sequence[Dict[str, Any]],
                      group: Optional[dist.ProcessGroup] = None,
                      timeout: Optional[float] = None) -> OCSSwitchResult:
        """Apply the plan on the switch; report link alignment."""


class TorchDistributedSwitchConnector:
    """Mock switch on top of ``torch.distributed`` object collectives."""

    def __init__(self, switch_delay_s: float = 0.0, link_ready_delay_s: float = 0.0,
                 link_ready: bool = True, delay_mode: str = "sleep") -> None:
        if switch_delay_s < 0 or link_ready_delay_s < 0:
            raise ValueError("mock switch and link-ready delays must be non-negative")
        if delay_mode not in ("sleep", "spin"):
            raise ValueError("delay_mode must be 'sleep' or 'spin'")
        self.switch_delay_s = float(switch_delay_s)
        self.link_ready_delay_s = float(link_ready_delay_s)
        self.link_ready = bool(link_ready)
        self.delay_mode = delay_mode

    def exchange_ready(self, ready_record, group=None, timeout=None):
        if not _dist_ready():
            return [ready_record]
        slots: List[Optional[Dict[str, Any]]] = [None] * dist.get_world_size(group)
        dist.all_gather_object(slots, ready_record, group=group)
        return [record for record in slots if record is not None]

    def _wait_delay(self, delay_s: float) -> None:
        if delay_s <= 0:
            return
        if self.delay_mode == "sleep":
            time.sleep(delay_s)
            return
        deadline = _monotonic_ns() + int(delay_s * 1e9)
        while _monotonic_ns() < deadline:
            pass

    def _simulate_commit(self) -> OCSSwitchResult:
        start_mono, start_us = _monotonic_ns(), _time_us()
        self._wait_delay(self.switch_delay_s)
        done_mono, done_us = _monotonic_ns(), _time_us()
        self._wait_delay(self.link_ready_delay_s)
        common = dict(switch_start_time_us=start_us, switch_done_time_us=done_us,
                      switch_start_mono_ns=start_mono, switch_done_mono_ns=done_mono)
        if self.link_ready:
            return OCSSwitchResult(link_state=OCSLinkState.LINK_ALIGNED,
                                   link_ready_time_us=_time_us(),
                                   link_ready_mono_ns=_monotonic_ns(), **common)
        return OCSSwitchResult(link_state=OCSLinkState.LINK_NOT_READY, link_ready_time_us=None,
                               error_code=1, error_message="mock link did not reach alignment",
                               **common)

    def commit_switch(self, plan, ready_records, group=None, timeout=None):
        if not _dist_ready():
            return self._simulate_commit()
        rank, _ = _rank_world_size(group)
        leader = min(plan.participant_ranks)
        box: List[Optional[OCSSwitchResult]] = [
            self._simulate_commit() if rank == leader else None]
        dist.broadcast_object_list(box, src=leader, group=group)
        if not isinstance(box[0], OCSSwitchResult):
            raise RuntimeError("switch connector did not broadcast an OCSSwitchResult")
        return box[0]


class TensorSwitchConnector(TorchDistributedSwitchConnector):
    """READY exchange as one fixed-size tensor all-gather.

    Each rank contributes 5 int64 words: rank, arrive_seq, arrival time and a
    128-bit digest of the record's consistency fields.  Peers' full records are
    reconstructed from the local plan when the digest matches; a mismatching
    digest yields a record whose ``topology_id`` is poisoned so that validation
    raises ``OCSPlanMismatchError`` exactly as it would on the slow path.  The
    commit result travels as a 4-word tensor broadcast.
    """

    _WORDS = 5

    @staticmethod
    def _digest_words(record: Dict[str, Any]) -> Tuple[int, int]:
        # Canonical text of the agreed fields in a fixed order (field names never vary, so only
        # the values are hashed; "\x1f" cannot occur in any of them).
        text = "\x1f".join([str(record.get(k)) for k in CONSISTENCY_FIELDS] + [str(record.get("participant_bitmap"))])
        raw = hashlib.blake2b(text.encode(), digest_size=16).digest()
        # int64 tensors are signed: fold into the non-negative range.
        return (int.from_bytes(raw[:8], "big") >> 1, int.from_bytes(raw[8:], "big") >> 1)

    def _device(self, group) -> torch.device:
        backend = str(dist.get_backend(group)).lower()
        return torch.device("cuda", torch.cuda.current_device()) if "nccl" in backend \
            else torch.device("cpu")

    def exchange_ready(self, ready_record, group=None, timeout=None):
        if not _dist_ready():
            return [ready_record]
        world = dist.get_world_size(group)
        d0, d1 = self._digest_words(ready_record)
        mine = torch.tensor([ready_record["src_rank"], ready_record["arrive_seq"],
                             ready_record["arrival_time_us"], d0, d1],
                            dtype=torch.int64, device=self._device(group))
        gathered = torch.empty(world * self._WORDS, dtype=torch.int64, device=mine.device)
        dist.all_gather_into_tensor(gathered, mine, group=group)
        records = []
        for row in gathered.view(world, self._WORDS).tolist():
            peer = dict(ready_record, src_rank=row[0], src_gpu_id=row[0], arrive_seq=row[1],
                        arrival_time_us=row[2])
            if (row[3], row[4]) != (d0, d1):
                peer["topology_id"] = -1 - int(peer.get("topology_id", 0))
            records.append(peer)
        return records

    def commit_switch(self, plan, ready_records, group=None, timeout=None):
        if not _dist_ready():
            return self._simulate_commit()
        rank, _ = _rank_world_size(group)
        leader = min(plan.participant_ranks)
        words = torch.zeros(4, dtype=torch.int64, device=self._device(group))
        if rank == leader:
            r = self._simulate_commit()
            words = torch.tensor([int(r.is_link_ready), r.switch_start_time_us,
                                  r.switch_done_time_us, r.link_ready_time_us or 0],
                                 dtype=torch.int64, device=words.device)
        dist.broadcast(words, src=dist.get_global_rank(group, leader) if group is not None
                       else leader, group=group)
        ok, start_us, done_us, ready_us = words.tolist()
        if ok:
            return OCSSwitchResult(OCSLinkState.LINK_ALIGNED, start_us, done_us, ready_us)
        return OCSSwitchResult(OCSLinkState.LINK_NOT_READY, start_us, done_us, None, error_code=1,
                               error_message="mock link did not reach alignment")


class NvlinkSwitchConnector(TensorSwitchConnector):
    """READY exchange and RELEASE delivery as signals between the GPUs, without a host collective.

    Both rounds of a barrier run on the engine's *signal board* (native ``OcsSignalBoard``): one
    single-CTA kernel per round stores this rank's words straight into every peer's symmetric
    memory over NVLink, waits (bounded) for the peers' words, and hands all of them to the host
    through mapped pinned memory, so the host neither launches a collective nor synchronises a
    stream.  Each rank contributes its rank, arrival sequence number, arrival time and the
    128-bit digest of its plan's consistency fields; the host compares the digests out of the
    mapped memory and rebuilds the peers' records from the local plan, exactly like
    ``TensorSwitchConnector`` (a mismatching digest poisons ``topology_id`` so that validation
    raises ``OCSPlanMismatchError``).  A source whose words do not arrive within ``timeout``
    simply stays absent from the returned records, which the runtime reports as
    ``OCSBarrierTimeout`` naming the missing ranks.

    The board spans the engine's whole world; barriers over other groups, and processes
    without a connected native engine, use the tensor path of the parent class.  Construction
    is collective (the board's slots come from the symmetric arena).  The reference's
    connector is two pickled-object collectives (pccl/ocs/runtime.py:139-203).
    """

    def __init__(self, board: Any = None, default_timeout_s: float = 1.0, **mock_switch) -> None:
        super().__init__(**mock_switch)
        self.default_timeout_s = float(default_timeout_s)
        self.host_us: List[float] = []           # per round, launch to completion on the host
        if board is None:
            from .. import engine as _engine
            _engine.get_engine()                  # the native engine must be up (and connected) first
            board = _engine.load_native().OcsSignalBoard()
            if _dist_ready():
                dist.barrier()                    # nobody signals a rank whose slots are not zeroed yet
        self.board = board

    def _usable(self, group) -> bool:
        return self.board is not None and (not _dist_ready() or
                                           dist.get_world_size(group) == self.board.world())

    def _timeout_us(self, timeout: Optional[float]) -> int:
        return max(1, int((self.default_timeout_s if timeout is None else timeout) * 1e6))

    @staticmethod
    def _split64(value: int) -> Tuple[int, int]:
        return value & 0xffffffff, (value >> 32) & 0xffffffff

    def _leader_of(self, ready_record) -> int:
        bitmap = int(ready_record.get("participant_bitmap", 1)) or 1
        return (bitmap & -bitmap).bit_length() - 1

    def exchange_ready(self, ready_record, group=None, timeout=None):
        if not self._usable(group):
            return super().exchange_ready(ready_record, group=group, timeout=timeout)
        d0, d1 = self._digest_words(ready_record)
        split = self._split64
        words = [int(ready_record["src_rank"]) & 0xffffffff, int(ready_record["arrive_seq"]) & 0xffffffff,
                 *split(int(ready_record["arrival_time_us"])), *split(d0), *split(d1)]
        self._released = None
        if self.switch_delay_s == 0 and self.link_ready_delay_s == 0:
            # A leader with nothing to wait for on the host between the rounds: READY gather and
            # RELEASE delivery in one launch.  The leader's release carries its clock at launch and
            # is cleared on the device if some rank's digest differs from the leader's.
            now = _time_us()
            release = [int(self.link_ready), *split(now), *split(now), *split(now)]
            ok, missing, host_us, rows, got = self.board.gather_release(
                self._leader_of(ready_record), words, release, 4, 8, self._timeout_us(timeout))
            if ok:
                self._released = got
        else:
            ok, missing, host_us, rows = self.board.all_gather(words, self._timeout_us(timeout))
        self.host_us.append(host_us)
        if not ok:
            # Out of step with at least one peer: report the barrier as incomplete (the sender is
            # the only record known to be good).  The board needs reset() before the next barrier.
            return [ready_record]
        records = []
        mine = (d0, d1)
        for row in rows:
            peer = dict(ready_record)
            peer["src_rank"] = peer["src_gpu_id"] = row[0]
            peer["arrive_seq"] = row[1]
            peer["arrival_time_us"] = row[2] | (row[3] << 32)
            if (row[4] | (row[5] << 32), row[6] | (row[7] << 32)) != mine:
                peer["topology_id"] = -1 - int(peer.get("topology_id", 0))
            records.append(peer)
        return records

    def commit_switch(self, plan, ready_records, group=None, timeout=None):
        if not self._usable(group):
            return super().commit_switch(plan, ready_records, group=group, timeout=timeout)
        got = getattr(self, "_released", None)
        self._released = None
        if got is None:
            rank, _ = _rank_world_size(group)
            leader = min(plan.participant_ranks)
            words = [0] * 7
            if rank == leader:
                r = self._simulate_commit()
                words = [int(r.is_link_ready), *self._split64(r.switch_start_time_us),
                         *self._split64(r.switch_done_time_us), *self._split64(r.link_ready_time_us or 0)]
            ok, _, host_us, got = self.board.broadcast(leader, words, self._timeout_us(timeout))
            self.host_us.append(host_us)
            if not ok:
                raise OCSBarrierTimeout(f"barrier {plan.barrier_id}: no RELEASE from leader rank {leader}")
        start_us, done_us, ready_us = (got[1] | (got[2] << 32), got[3] | (got[4] << 32), got[5] | (got[6] << 32))
        if got[0]:
            return OCSSwitchResult(OCSLinkState.LINK_ALIGNED, start_us, done_us, ready_us)
        return OCSSwitchResult(OCSLinkState.LINK_NOT_READY, start_us, done_us, None, error_code=1,
                               error_message="mock link did not reach alignment")


class OCSRuntime:
    """Runs the barrier state machine and keeps a history of its outcomes."""

    def __init__(self, controller: Optional[OCSPlanController] = None,
                 connector: Optional[SwitchConnector] = None) -> None:
        self.controller = controller if controller is not None else StaticPlanController()
        self.connector = connector if connector is not None else TorchDistributedSwitchConnector()
        self.history: List[Dict[str, Any]] = []
        self._arrive_seq = 0

    def next_plan(self, event_key: str, group: Optional[dist.ProcessGroup] = None) -> OCSPlan:
        rank, world_size = _rank_world_size(group)
        return self.controller.next_plan(event_key, rank=rank, world_size=world_size)

    def barrier_switch(self, plan: OCSPlan, group: Optional[dist.ProcessGroup] = None,
                       timeout: Optional[float] = None) -> Dict[str, Any]:
        if plan.route_mode != "STATIC_PLAN":
            raise NotImplementedError(
                f"route_mode={plan.route_mode!r} is reserved; v0 only executes STATIC_PLAN")
        rank, world_size = _rank_world_size(group)
        plan = plan.with_default_participants(world_size)
        if rank not in plan.participant_ranks:
            raise OCSPlanMismatchError(
                f"rank {rank} is not listed in participant_ranks={plan.participant_ranks}")

        seq, self._arrive_seq = self._arrive_seq, self._arrive_seq + 1
        marks = {"arrival": _monotonic_ns()}
        arrival_us = _time_us()
        trace = [_state_event(OCSBarrierState.READY, arrival_us)]

        ready = plan.ready_record(src_rank=rank, world_size=world_size, arrive_seq=seq,
                                  arrival_time_us=arrival_us)
        records = self.connector.exchange_ready(ready, group=group, timeout=timeout)
        marks["exchanged"] = _monotonic_ns()
        self._validate_ready_records(plan, records)
        marks["validated"] = _monotonic_ns()
        trace.append(_state_event(OCSBarrierState.ALL_ARRIVED, _time_us()))

        marks["commit_start"] = _monotonic_ns()
        result = self.connector.commit_switch(plan, records, group=group, timeout=timeout)
        marks["commit_done"] = _monotonic_ns()
        trace.append(_state_event(OCSBarrierState.SWITCHING, result.switch_start_time_us))
        trace.append(_state_event(OCSBarrierState.WAIT_LINK_ALIGN, result.switch_done_time_us))

        final_state = OCSBarrierState.RELEASED if result.is_link_ready else OCSBarrierState.FAILED
        end_us = _time_us()
        marks["end"] = _monotonic_ns()
        trace.append(_state_event(final_state, end_us))
        timing = self._latency_breakdown(marks["arrival"], marks["exchanged"], marks["validated"],
                                         marks["commit_start"], marks["commit_done"],
                                         marks["end"], result)

        identity = {"version": 1, "job_id": plan.job_id, "group_id": plan.group_id,
                    "barrier_id": plan.barrier_id, "epoch_id": plan.epoch_id,
                    "next_epoch_id": plan.next_epoch_id}
        tail = {"timing": timing, "state_trace": trace, "ready_records": records}

        if not result.is_link_ready:
            self.history.append({
                "msg_type": "OCS_BARRIER_ABORT", **identity,
                "status": "LINK_NOT_READY", "error_code": result.error_code,
                "error_message": result.error_message, "link_state": result.link_state.value,
                "arrival_time_us": arrival_us,
                "switch_start_time_us": result.switch_start_time_us,
                "switch_done_time_us": result.switch_done_time_us, **tail})
            raise OCSLinkNotReady(
                f"barrier {plan.barrier_id} link state is {result.link_state.value}: "
                f"{result.error_message}")

        release = {
            "msg_type": "OCS_BARRIER_RELEASE", **identity,
            "status": "OK", "error_code": 0,
            "participant_bitmap": plan.participant_bitmap, "topology_id": plan.topology_id,
            "route_plan_id": plan.route_plan_id, "algorithm": plan.algorithm,
            "backend": plan.backend, "arrival_time_us": arrival_us,
            "switch_start_time_us": result.switch_start_time_us,
            "switch_done_time_us": result.switch_done_time_us,
            "link_ready_time_us": result.link_ready_time_us,
            "link_state": result.link_state.value, "release_time_us": end_us,
            "latency_us": int(round(timing["total_us"])), **tail}
        self.history.append(release)
        return release

    @staticmethod
    def _latency_breakdown(arrival_mono_ns: int, ready_exchange_done_mono_ns: int,
                           ready_validation_done_mono_ns: int, commit_start_mono_ns: int,
                           commit_done_mono_ns: int, completion_mono_ns: int,
                           switch_result: OCSSwitchResult) -> Dict[str, float]:
        """Local control-path durations, plus the two controller-internal
        durations (taken on the leader's clock, so reported separately and never
        added to local ones)."""
        r = switch_result
        if r.switch_start_mono_ns is not None and r.switch_done_mono_ns is not None:
            switching = _duration_us(r.switch_start_mono_ns, r.switch_done_mono_ns)
        else:
            switching = max(0.0, float(r.switch_done_time_us - r.switch_start_time_us))
        if r.switch_done_mono_ns is not None and r.link_ready_mono_ns is not None:
            aligning = _duration_us(r.switch_done_mono_ns, r.link_ready_mono_ns)
        elif r.link_ready_time_us is not None:
            aligning = max(0.0, float(r.link_ready_time_us - r.switch_done_time_us))
        else:
            aligning = 0.0
        return {
            "ready_exchange_us": _duration_us(arrival_mono_ns, ready_exchange_done_mono_ns),
            "ready_validation_us": _duration_us(ready_exchange_done_mono_ns,
                                                ready_validation_done_mono_ns),
            "controller_commit_us": _duration_us(commit_start_mono_ns, commit_done_mono_ns),
            "release_local_us": _duration_us(commit_done_mono_ns, completion_mono_ns),
            "total_us": _duration_us(arrival_mono_ns, completion_mono_ns),
            "controller_switch_us": switching,
            "controller_link_align_us": aligning,
        }

    def _validate_ready_records(self, plan: OCSPlan, records: Sequence[Dict[str, Any]]) -> None:
        expected = plan.consistency_fields()
        wanted = set(plan.participant_ranks)
        seen = set()
        names = _COMPARED_FIELDS
        expected_row = tuple(expected[name] for name in names)
        for record in records:
            if record.get("msg_type") != "OCS_BARRIER_READY":
                raise OCSPlanMismatchError(f"unexpected OCS message: {record!r}")
            src = int(record.get("src_rank", -1))
            if src not in wanted:
                continue                      # bystander of a sub-group barrier
            if src in seen:
                raise OCSPlanMismatchError(
                    f"duplicate READY from rank {src} for barrier {plan.barrier_id}")
            seen.add(src)
            try:
                same = _compared_values(record) == expected_row      # one C-level tuple comparison
            except KeyError:
                same = False
            if not same:
                for name in names:
                    if record.get(name) != expected[name]:
                        raise OCSPlanMismatchError(
                            f"rank {src} has inconsistent {name}: "
                            f"{record.get(name)!r} != {expected[name]!r}")
        missing = sorted(wanted - seen)
        if missing:
            raise OCSBarrierTimeout(
                f"barrier {plan.barrier_id} missing READY from ranks {missing}")


_default_runtime: Optional[OCSRuntime] = None


def get_default_runtime() -> OCSRuntime:
    global _default_runtime
    if _default_runtime is None:
        _default_runtime = OCSRuntime()
    return _default_runtime


def ocs_barrier_switch(group: Optional[dist.ProcessGroup], plan: OCSPlan,
                       timeout: Optional[float] = None) -> Dict[str, Any]:
    return get_default_runtime().barrier_switch(plan, group=group, timeout=timeout)


def ocs_all_reduce(tensor: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                   runtime: Optional[OCSRuntime] = None, op: dist.ReduceOp = dist.ReduceOp.SUM,
                   async_op: bool = False, timeout: Optional[float] = None) -> torch.Tensor:
    """Barrier-switch to the controller's next plan, then all-reduce."""
    if async_op:
        raise NotImplementedError("OCS all_reduce is blocking in v0; async_op is reserved")
    rt = runtime if runtime is not None else get_default_runtime()
    plan = rt.next_plan("all_reduce", group=group)
    if plan.backend != "torch":
        raise NotImplementedError(
            f"backend={plan.backend!r} is reserved; v0 only executes the torch backend")
    rt.barrier_switch(plan, group=group, timeout=timeout)
    dist.all_reduce(tensor, op=op, group=group)
    return tensor
