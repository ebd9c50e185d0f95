"""Step-level software pipelining of a plan across channels.

``Pipeline(depth)`` rotates successive *stages* over ``depth`` channels: stage
``i`` is emitted on channel ``i % depth`` inside the stream ``__pipe_ch{c}``,
so primitives of the same channel stay chained while different channels are
free to overlap (reference: pccl/dsl/pipeline.py:34-103).

    with CommunicationOp("ar") as op:
        op.tensor("bfloat16", (n,))
        with Pipeline(depth=2).bind(op) as pipe:
            for step in range(steps):
                with pipe.stage():
                    op.sm_reduce(...); op.notify(...)
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Iterator, Optional

from .decorators import CommunicationOp, Stream


class Pipeline:
    def __init__(self, depth: int = 2):
        if depth < 1:
            raise ValueError(f"Pipeline depth must be >= 1, got {depth}")
        self.depth = depth
        self._comm_op: Optional[CommunicationOp] = None
        self._iteration = 0

    @contextmanager
    def bind(self, comm_op: CommunicationOp) -> Iterator["Pipeline"]:
        """Attach to ``comm_op`` for the duration of the block; the stage
        counter restarts at zero."""
        self._comm_op, self._iteration = comm_op, 0
        try:
            yield self
        finally:
            self._comm_op = None

    @contextmanager
    def stage(self) -> Iterator["Pipeline"]:
        """One pipeline iteration: selects the channel and its stream."""
        op = self._comm_op
        if op is None:
            raise RuntimeError("Pipeline.stage() must be used inside Pipeline.bind()")
        channel = self._iteration % self.depth
        self._iteration += 1
        op.set_channel(channel)
        with Stream(f"__pipe_ch{channel}"):
            yield self
