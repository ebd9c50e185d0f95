"""Binary-tree allreduce (power-of-two ranks, root = rank 0).

Up-sweep: at level k a rank whose bit k is set hands its whole vector to the
partner across that bit (the partner pulls and reduces it) and drops out.
Down-sweep: the same pairs in reverse order, the upper rank pulling the
finished vector.  2*log2(N) steps, but the root moves the full vector each
time, so it only wins for small messages (reference:
pccl/dsl/algorithms/tree.py:19-123; same primitive sequence).
"""

from __future__ import annotations

from ..decorators import CommunicationOp, Stream
from ..graph import PrimitiveIRGraph
from ..nodes import DeviceType
from .base import CollectiveAlgorithm, finish, is_power_of_two


class TreeAllreduce(CollectiveAlgorithm):
    name: str = "tree"

    @property
    def step_count(self) -> str:
        return "O(2 log N)"

    @property
    def bandwidth_optimal(self) -> bool:
        return False

    def build_allreduce(self, rank, world_size, tensor_size, dtype="bfloat16", executor="tma",
                        num_channels=1) -> PrimitiveIRGraph:
        if not is_power_of_two(world_size):
            raise ValueError(f"TreeAllreduce requires power-of-2 world_size, got {world_size}")
        levels = world_size.bit_length() - 1
        tma = executor == "tma"

        with CommunicationOp(name=f"tree_ar_{executor}_rank{rank}", device=DeviceType.CUDA) as op:
            op.tensor(dtype=dtype, shape=(tensor_size,))
            with Stream("main"):
                op.set_channel(0)

                for k in range(levels):                        # up-sweep
                    partner = rank ^ (1 << k)
                    if rank >> k & 1:
                        # Child: announce "my vector is ready", wait until it was consumed.
                        op.notify(signal_id=rank, target_rank=partner)
                        op.wait_notify(signal_id=partner, source_rank=partner)
                        break
                    op.wait_notify(signal_id=partner, source_rank=partner)
                    (op.tma_reduce if tma else op.sm_reduce)(
                        reduce_op="sum", source_rank=partner, src_offset=0, dst_offset=0,
                        remote_offset=0, count=tensor_size)
                    op.notify(signal_id=rank, target_rank=partner)

                for k in reversed(range(levels)):              # down-sweep
                    if rank % (1 << k):
                        continue                               # not active at this level
                    partner = rank ^ (1 << k)
                    if rank >> k & 1:
                        op.wait_notify(signal_id=partner, source_rank=partner)
                        (op.tma_copy if tma else op.sm_copy)(
                            source_rank=partner, src_offset=0, dst_offset=0, size=tensor_size)
                        op.notify(signal_id=rank, target_rank=partner)
                    else:
                        op.notify(signal_id=rank, target_rank=partner)
                        op.wait_notify(signal_id=partner, source_rank=partner)
            return finish(op, "allreduce", "tree")
