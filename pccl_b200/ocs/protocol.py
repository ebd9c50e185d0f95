"""Wire format of OCS control messages (READY / RELEASE / ABORT / ACK).

Layout (network byte order): a fixed 128-byte header, ``payload_len`` opaque
bytes, a CRC32 of everything before it.  The fixed header lets a hardware
mailbox read barrier identity and the plan commitment without parsing the
payload.  The format is bit-for-bit the reference's (reference:
pccl/ocs/protocol.py:23-32 header, :54-70 enum ids, :77-99 digests,
:215-320 encode/decode, :323-408 builders).

Header fields, in order::

    magic[4] version:u8 msg_type:u8 status:u8 route_mode:u8 job_id_hash:u64
    group_id:u32 barrier_id:u64 epoch_id:u64 next_epoch_id:u64 src_rank:i32
    src_gpu_id:i32 participant_bitmap:u64 topology_id:u32 algorithm:u8 backend:u8
    reserved:u16 route_plan_id:u64 sequence:u64 send_time_us:u64
    plan_digest[32] payload_len:u32
"""

from __future__ import annotations

import hashlib
import json
import struct
import time
import zlib
from dataclasses import dataclass, fields
from enum import IntEnum
from typing import Optional, Tuple

from .exceptions import OCSProtocolError
from .plan import OCSPlan

OCS_CONTROL_MAGIC = b"OCSB"
OCS_CONTROL_VERSION = 1
OCS_CONTROL_MAX_PAYLOAD_BYTES = 1 << 20

_HEADER = struct.Struct("!4sBBBBQIQQQiiQIBBHQQQ32sI")
_CRC = struct.Struct("!I")
_ACK_TARGET = struct.Struct("!BiQ")
assert _HEADER.size == 128


class OCSControlMessageType(IntEnum):
    READY = 1
    RELEASE = 2
    ABORT = 3
    ACK = 4


class OCSControlStatus(IntEnum):
    OK = 0
    LINK_NOT_READY = 1
    PLAN_MISMATCH = 2
    TIMEOUT = 3
    INTERNAL_ERROR = 4


def _two_way(mapping):
    return mapping, {v: k for k, v in mapping.items()}


_ROUTE_MODE_TO_ID, _ROUTE_MODE_FROM_ID = _two_way(
    {"STATIC_PLAN": 1, "ID_ROUTE": 2, "SEGMENT_ROUTE": 3, "USER_PLAN": 4})
_ALGORITHM_TO_ID, _ALGORITHM_FROM_ID = _two_way(
    {"ring": 1, "rhd": 2, "tree": 3, "auto": 4, "torch_native": 5})
_BACKEND_TO_ID, _BACKEND_FROM_ID = _two_way({"torch": 1, "pccl": 2})


def _time_us() -> int:
    return time.time_ns() // 1000


def _job_id_hash(job_id: str) -> int:
    """64-bit BLAKE2b of the job name (big-endian)."""
    return int.from_bytes(hashlib.blake2b(str(job_id).encode("utf-8"), digest_size=8).digest(), "big")


def plan_digest(plan: OCSPlan) -> bytes:
    """SHA-256 over the canonical JSON of every plan field, payload included."""
    canonical = {
        "algorithm": plan.algorithm, "backend": plan.backend, "barrier_id": plan.barrier_id,
        "epoch_id": plan.epoch_id, "group_id": plan.group_id, "job_id": plan.job_id,
        "next_epoch_id": plan.next_epoch_id, "participant_ranks": plan.participant_ranks,
        "payload_hex": plan.payload.hex(), "route_mode": plan.route_mode,
        "route_plan_id": plan.route_plan_id, "topology_id": plan.topology_id,
    }
    text = json.dumps(canonical, sort_keys=True, separators=(",", ":"))
    return hashlib.sha256(text.encode("utf-8")).digest()


@dataclass(frozen=True)
class OCSControlMessageKey:
    """Identifies one logical message; retransmissions share the key."""

    job_id_hash: int
    group_id: int
    barrier_id: int
    epoch_id: int
    src_rank: int
    sequence: int
    message_type: OCSControlMessageType


#: plan attributes a message must echo unchanged
_PLAN_ECHO = ("group_id", "barrier_id", "epoch_id", "next_epoch_id", "participant_bitmap",
              "topology_id", "route_mode", "algorithm", "backend", "route_plan_id")


@dataclass(frozen=True)
class OCSControlMessage:
    message_type: OCSControlMessageType
    status: OCSControlStatus
    job_id_hash: int
    group_id: int
    barrier_id: int
    epoch_id: int
    next_epoch_id: int
    src_rank: int
    src_gpu_id: int
    participant_bitmap: int
    topology_id: int
    route_mode: str
    algorithm: str
    backend: str
    route_plan_id: int
    sequence: int
    send_time_us: int
    plan_digest: bytes
    payload: bytes = b""

    def __post_init__(self) -> None:
        if len(self.plan_digest) != 32:
            raise ValueError("plan_digest must be a SHA-256 digest")
        if not isinstance(self.payload, bytes):
            object.__setattr__(self, "payload", bytes(self.payload))
        if len(self.payload) > OCS_CONTROL_MAX_PAYLOAD_BYTES:
            raise ValueError(
                f"OCS control payload exceeds {OCS_CONTROL_MAX_PAYLOAD_BYTES} bytes")

    @property
    def key(self) -> OCSControlMessageKey:
        return OCSControlMessageKey(self.job_id_hash, self.group_id, self.barrier_id,
                                    self.epoch_id, self.src_rank, self.sequence,
                                    self.message_type)

    @classmethod
    def from_plan(cls, message_type: OCSControlMessageType, plan: OCSPlan, src_rank: int,
                  src_gpu_id: Optional[int] = None, sequence: int = 0,
                  status: OCSControlStatus = OCSControlStatus.OK,
                  payload: Optional[bytes] = None,
                  send_time_us: Optional[int] = None) -> "OCSControlMessage":
        """A message committing to ``plan``; READY carries the plan payload by default."""
        if payload is None:
            payload = plan.payload if message_type == OCSControlMessageType.READY else b""
        echo = {name: getattr(plan, name) for name in _PLAN_ECHO}
        return cls(message_type=message_type, status=status,
                   job_id_hash=_job_id_hash(plan.job_id), src_rank=int(src_rank),
                   src_gpu_id=int(src_rank if src_gpu_id is None else src_gpu_id),
                   sequence=int(sequence),
                   send_time_us=_time_us() if send_time_us is None else int(send_time_us),
                   plan_digest=plan_digest(plan), payload=bytes(payload), **echo)

    def matches_plan(self, plan: OCSPlan) -> bool:
        return (self.job_id_hash == _job_id_hash(plan.job_id)
                and all(getattr(self, name) == getattr(plan, name) for name in _PLAN_ECHO)
                and self.plan_digest == plan_digest(plan))

    def encode(self) -> bytes:
        try:
            head = _HEADER.pack(
                OCS_CONTROL_MAGIC, OCS_CONTROL_VERSION, int(self.message_type), int(self.status),
                _ROUTE_MODE_TO_ID[self.route_mode], self.job_id_hash, self.group_id,
                self.barrier_id, self.epoch_id, self.next_epoch_id, self.src_rank,
                self.src_gpu_id, self.participant_bitmap, self.topology_id,
                _ALGORITHM_TO_ID[self.algorithm], _BACKEND_TO_ID[self.backend], 0,
                self.route_plan_id, self.sequence, self.send_time_us, self.plan_digest,
                len(self.payload))
        except struct.error as err:
            raise OCSProtocolError(f"OCS control header field is out of range: {err}") from err
        body = head + self.payload
        return body + _CRC.pack(zlib.crc32(body) & 0xFFFFFFFF)

    @classmethod
    def decode(cls, wire: bytes) -> "OCSControlMessage":
        """Validate length, magic, version, payload length and CRC, then parse."""
        wire = bytes(wire)
        if len(wire) < _HEADER.size + _CRC.size:
            raise OCSProtocolError("OCS control message is shorter than its fixed header")
        (magic, version, msg_type, status, route_mode, job_hash, group_id, barrier_id, epoch_id,
         next_epoch_id, src_rank, src_gpu_id, bitmap, topology_id, algorithm, backend, _reserved,
         route_plan_id, sequence, send_time_us, digest, payload_len) = _HEADER.unpack_from(wire)
        if magic != OCS_CONTROL_MAGIC:
            raise OCSProtocolError("invalid OCS control message magic")
        if version != OCS_CONTROL_VERSION:
            raise OCSProtocolError(
                f"unsupported OCS control version {version}; expected {OCS_CONTROL_VERSION}")
        if payload_len > OCS_CONTROL_MAX_PAYLOAD_BYTES:
            raise OCSProtocolError("OCS control payload exceeds the protocol maximum")
        if len(wire) != _HEADER.size + payload_len + _CRC.size:
            raise OCSProtocolError("OCS control payload length does not match the wire size")
        body, (crc,) = wire[:-_CRC.size], _CRC.unpack(wire[-_CRC.size:])
        if zlib.crc32(body) & 0xFFFFFFFF != crc:
            raise OCSProtocolError("OCS control CRC32 mismatch")
        try:
            return cls(message_type=OCSControlMessageType(msg_type),
                       status=OCSControlStatus(status), job_id_hash=job_hash, group_id=group_id,
                       barrier_id=barrier_id, epoch_id=epoch_id, next_epoch_id=next_epoch_id,
                       src_rank=src_rank, src_gpu_id=src_gpu_id, participant_bitmap=bitmap,
                       topology_id=topology_id, route_mode=_ROUTE_MODE_FROM_ID[route_mode],
                       algorithm=_ALGORITHM_FROM_ID[algorithm], backend=_BACKEND_FROM_ID[backend],
                       route_plan_id=route_plan_id, sequence=sequence, send_time_us=send_time_us,
                       plan_digest=digest, payload=body[_HEADER.size:])
        except (KeyError, ValueError) as err:
            raise OCSProtocolError(f"invalid OCS control enum value: {err}") from err


def build_ready(plan: OCSPlan, src_rank: int, src_gpu_id: Optional[int] = None,
                sequence: int = 0) -> OCSControlMessage:
    return OCSControlMessage.from_plan(OCSControlMessageType.READY, plan, src_rank=src_rank,
                                       src_gpu_id=src_gpu_id, sequence=sequence)


def build_release(plan: OCSPlan, controller_rank: int = -1, sequence: int = 0,
                  status: OCSControlStatus = OCSControlStatus.OK) -> OCSControlMessage:
    """RELEASE when ``status`` is OK, otherwise ABORT carrying the status."""
    kind = (OCSControlMessageType.RELEASE if status == OCSControlStatus.OK
            else OCSControlMessageType.ABORT)
    return OCSControlMessage.from_plan(kind, plan, src_rank=controller_rank, src_gpu_id=-1,
                                       sequence=sequence, status=status, payload=b"")


def build_ack(acknowledged: OCSControlMessage, src_rank: int, src_gpu_id: Optional[int] = None,
              sequence: int = 0, status: OCSControlStatus = OCSControlStatus.OK) -> OCSControlMessage:
    """ACK whose payload names the acknowledged message (type, sender, sequence)."""
    inherited = {f.name: getattr(acknowledged, f.name) for f in fields(acknowledged)}
    inherited.update(
        message_type=OCSControlMessageType.ACK, status=status, src_rank=int(src_rank),
        src_gpu_id=int(src_rank if src_gpu_id is None else src_gpu_id), sequence=int(sequence),
        send_time_us=_time_us(),
        payload=_ACK_TARGET.pack(int(acknowledged.message_type), acknowledged.src_rank,
                                 acknowledged.sequence))
    return OCSControlMessage(**inherited)


def ack_target(message: OCSControlMessage) -> Tuple[OCSControlMessageType, int, int]:
    if message.message_type != OCSControlMessageType.ACK:
        raise ValueError("ack_target requires an ACK message")
    if len(message.payload) != _ACK_TARGET.size:
        raise OCSProtocolError("ACK payload has an invalid target key")
    kind, src_rank, sequence = _ACK_TARGET.unpack(message.payload)
    try:
        return OCSControlMessageType(kind), src_rank, sequence
    except ValueError as err:
        raise OCSProtocolError(f"ACK references an invalid message type: {kind}") from err
