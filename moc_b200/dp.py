"""Token-sharded data parallelism for the MoC FFN: one process per GPU, each rank runs its own
tokens, parameter gradients are summed (averaged) across ranks with one all-reduce per weight.

The reference has no distributed code; the FFN is token-wise, so forward and dX need no
communication and only dW_gate, dW_up, dW_down are reduced. ``GradAllReducer`` starts the three
all-reduces on a side stream behind an event of the backward pass: by default the event after its
last kernel; with ``overlap=True`` the event that ``moc_ffn_bwd`` records as soon as the
weight-gradient GEMM is done, so that the transfers run beside the dX GEMM. Works with any ``torch.distributed`` backend (NCCL over NVLink on GPUs; gloo in
the CPU tests of the bookkeeping).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ffn as _ffn


def shard_bounds(total_tokens: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous token range [begin, end) owned by `rank`; the first `total % world` ranks get
    one extra token."""
    base, extra = divmod(total_tokens, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class GradAllReducer:
    """Overlapped gradient all-reduce for MoC FFN modules.

    Usage::

        reducer = GradAllReducer(average=True)
        with reducer:                 # installs the grad-ready hook
            loss.backward()
        # leaving the block waits (stream-wise, not host-wise) for all reductions
    """

    def __init__(self, group=None, average: bool = True, overlap: bool = False):
        self.group = group
        self.average = average
        # overlap=True starts the reductions behind the weight-gradient GEMM, beside the dX GEMM; the default
        # starts them after the backward pass (see moc_b200.ffn._grad_ready_early for the measurement)
        self.overlap = overlap
        self.comm_stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.launched = 0

    def _on_grad_ready(self, name: str, grad: torch.Tensor, event) -> None:
        world = dist.get_world_size(self.group)
        if world == 1:
            return
        if grad.is_cuda:
            self.comm_stream.wait_event(event)
            grad.record_stream(self.comm_stream)
            with torch.cuda.stream(self.comm_stream):
                self._reduce(grad, world)
        else:
            self._reduce(grad, world)
        self.launched += 1

    def _reduce(self, grad: torch.Tensor, world: int) -> None:
        if self.average and dist.get_backend(self.group) == "nccl":
            dist.all_reduce(grad, op=dist.ReduceOp.AVG, group=self.group)
        else:
            dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=self.group)
            if self.average:
                grad.div_(world)

    def reduce_now(self, name: str, grad: torch.Tensor) -> None:
        """Synchronous-path entry for tensors that did not come through the hook."""
        self._on_grad_ready(name, grad, None if not grad.is_cuda else _recorded_event())

    def __enter__(self):
        self.launched = 0
        _ffn.set_grad_ready_hook(self._on_grad_ready, early=self.overlap)
        return self

    def __exit__(self, *exc):
        _ffn.set_grad_ready_hook(None)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        return False


def _recorded_event():
    ev = torch.cuda.Event()
    ev.record()
    return ev
