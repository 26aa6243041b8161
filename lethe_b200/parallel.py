"""Multi-GPU use of the path: one process per GPU, ``torch.distributed`` for the plumbing.

Two ways to split a problem (BASELINE configuration 4):

* **(batch x head) sharding** -- every (batch, head) pair is an independent recurrence, so ranks take
  disjoint slices and never talk.  ``shard_batch_heads`` computes the slices; each rank then calls
  the ordinary op on its slice.

* **Sequence parallel** -- for one very long sequence, rank r owns tokens ``[r L/N, (r+1) L/N)``.  The
  chunk-parallel kernels of all ranks run concurrently; only the chunk-to-chunk state scan is
  serial, so the state entering a rank's first chunk is received from rank r-1 (forward) and the
  adjoint state entering its last chunk from rank r+1 (backward) with point-to-point messages of one
  ``[B, H, K, V]`` fp32 tensor.  The received tensor lands in this GPU's own memory before any kernel
  reads it.  ``sp_forward`` / ``sp_backward`` are the protocol, written against three callables so
  that the same code runs with the CUDA kernels (``SequenceParallelGdn``) and, in the CPU tests,
  with the oracle over gloo.

The reference has no distributed layer on this path (its only ``torch.distributed`` use is a DDP
trainer elsewhere), so there is no reference file to cite for the protocol itself.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist
from torch import Tensor

from . import ops


def shard_batch_heads(B: int, H: int, rank: int, world: int) -> tuple[slice, slice]:
    """Slices of the batch and head axes that `rank` owns.  Splits the batch when it divides by the
    world size, else the heads; raises if neither does (no padding, no imbalance)."""
    if B % world == 0:
        n = B // world
        return slice(rank * n, (rank + 1) * n), slice(0, H)
    if H % world == 0:
        n = H // world
        return slice(0, B), slice(rank * n, (rank + 1) * n)
    raise ValueError(f"neither B={B} nor H={H} divides by the world size {world}")


class HandoffTimeout(ops.GdnError):
    """A neighbouring rank did not deliver its boundary state in time."""


def _peer(group, r: int) -> int:
    return dist.get_global_rank(group, r) if group is not None else r


def _wait_state(work, what: str, src: int, timeout_s: float | None) -> None:
    """Completes a posted receive.  On the CPU (gloo) the wait is bounded on the host: a neighbour that
    died, never joined the step or never sent surfaces as ``HandoffTimeout`` after ``timeout_s`` instead of
    a hang.  On NCCL the wait only orders the current stream behind the receive (the host does not
    block); there the process group's own timeout ends a receive whose sender is gone."""
    try:
        if timeout_s is not None and dist.get_backend() == "gloo":
            import datetime
            work.wait(timeout=datetime.timedelta(seconds=timeout_s))
        else:
            work.wait()
    except RuntimeError as e:       # gloo reports an expired wait as RuntimeError / DistBackendError
        raise HandoffTimeout(f"lethe_gdn: no {what} from rank {src} within {timeout_s} s: {e}") from e


def sp_forward(prepare: Callable[[], None], scan: Callable[[Tensor | None], Tensor],
               output: Callable[[], None], h0: Tensor | None, state_like: Tensor, group=None,
               timeout_s: float | None = None) -> Tensor:
    """Sequence-parallel forward.  `scan(h_in)` runs this rank's state scan from `h_in` (None = zero)
    and returns the state leaving the rank.  Returns that state (the global final state on the last
    rank).  The receive of the incoming state is posted before this rank's chunk-parallel work is
    enqueued, so the transfer does not queue up behind it; the outgoing state is sent, and the send
    completed, as soon as the scan has produced it, before the output kernels are enqueued."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    work, h_in = None, h0
    if rank > 0:
        h_in = torch.empty_like(state_like)
        work = dist.irecv(h_in, src=_peer(group, rank - 1), group=group)
    prepare()
    if work is not None:
        _wait_state(work, "chunk-boundary state", rank - 1, timeout_s)
    h_out = scan(h_in)
    if rank + 1 < world:
        # The next rank's scan waits for this message, so it goes out before this rank enqueues anything
        # else: a send issued with the output kernels already queued behind the scan found no free SM
        # until their grid had drained (measured on 4 GPUs: every hand-off 0.24 ms late in the forward and
        # 0.68 ms late in the backward, 2.8 ms of an 8.7 ms step).  The stream idles for the transfer
        # (2 MB over NVLink, tens of microseconds) instead.
        dist.isend(h_out, dst=_peer(group, rank + 1), group=group).wait()
    output()
    return h_out


def sp_backward(pre: Callable[[], None], scan: Callable[[Tensor | None], Tensor], main: Callable[[], None],
                dhT: Tensor | None, state_like: Tensor, group=None, timeout_s: float | None = None) -> Tensor:
    """Sequence-parallel backward: the adjoint state flows from the last rank to the first.
    `scan(dh_in)` returns the adjoint of the state entering this rank (dh0 on rank 0)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    work, dh_in = None, dhT
    if rank < world - 1:
        dh_in = torch.empty_like(state_like)
        work = dist.irecv(dh_in, src=_peer(group, rank + 1), group=group)
    pre()
    if work is not None:
        _wait_state(work, "adjoint state", rank + 1, timeout_s)
    dh_out = scan(dh_in)
    if rank > 0:
        dist.isend(dh_out, dst=_peer(group, rank - 1), group=group).wait()      # before Stage B / WY: see sp_forward
    main()
    return dh_out


class SequenceParallelGdn:
    """The CUDA kernels under the sequence-parallel protocol.  One instance per problem size keeps the
    buffers; ``forward`` / ``backward`` take this rank's token slice of every tensor."""

    def __init__(self, B, L_local, H, K, V, gate: int, delta: bool, device, group=None):
        self.buf = ops.GdnBuffers(B, L_local, H, K, V, gate, delta, device)
        self.group = group
        self.state_like = torch.empty(B, H, K, V, dtype=torch.float32, device=device)

    def forward(self, q, k, v, g, beta, h0, scale: float):
        """Returns (o_local, state leaving this rank).  `h0` is used on rank 0 only."""
        self._in = (q, k, v, g, beta)
        self._scale = scale
        self._h_in = None

        def prepare():
            ops.forward_into(self.buf, q, k, v, g, beta, None, scale, kernel_mask=1)

        def scan(h_in):
            self._h_in = h_in
            ops.forward_into(self.buf, q, k, v, g, beta, h_in, scale, kernel_mask=2)
            return self.buf.hT

        def output():
            ops.forward_into(self.buf, q, k, v, g, beta, self._h_in, scale, kernel_mask=4)

        hT = sp_forward(prepare, scan, output, h0, self.state_like, self.group)
        return self.buf.o, hT

    def backward(self, do, dhT):
        """Returns (dq, dk, dv, dg, dbeta, adjoint of the state entering this rank).  `dhT` is used on
        the last rank only."""
        q, k, v, g, beta = self._in
        scale = self._scale

        def pre():
            ops.backward_into(self.buf, q, k, v, g, beta, self._h_in, do, None, scale, kernel_mask=1)

        def scan(dh_in):
            ops.backward_into(self.buf, q, k, v, g, beta, self._h_in, do, dh_in, scale, kernel_mask=2)
            return self.buf.dh0

        def main():
            ops.backward_into(self.buf, q, k, v, g, beta, self._h_in, do, None, scale, kernel_mask=12)

        dh0 = sp_backward(pre, scan, main, dhT, self.state_like, self.group)
        b = self.buf
        return b.dq, b.dk, b.dv, b.dg, b.dbeta, dh0
