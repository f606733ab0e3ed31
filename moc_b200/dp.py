"""Token-sharded data parallelism for the MoC FFN: one process per GPU, each rank runs its own
tokens, parameter gradients are summed (averaged) across ranks with one all-reduce per weight.

The reference has no distributed code; the FFN is token-wise, so forward and dX need no
communication and only dW_gate, dW_up, dW_down are reduced: the autograd node hands them over as one
[3, d_ffn * d] bucket and ``GradAllReducer`` runs one all-reduce on a side stream behind an event of the
backward pass: by default the event after its last kernel; with ``overlap=True`` the event that
``moc_ffn_bwd`` records as soon as the weight-gradient GEMM is done, so that the transfer runs beside the
dX GEMM, which then leaves ``reserve_sms`` SMs free for the collective's CTAs. Measured on 2 x B200 (67 MB
bucket as three 22 MB calls): serialised 0.23 ms after the backward pass; overlapped with 16 SMs reserved the
reduction ends 0.02 ms after the (0.05 ms slower) dX GEMM; without a reserve it cannot start before the GEMM
ends. Works with any ``torch.distributed`` backend (NCCL over NVLink on GPUs; gloo in
the CPU tests of the bookkeeping).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
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

    The reduction runs in place on the gradient tensors that the autograd node returns, which become the
    parameters' ``.grad`` only when those are unset: call ``zero_grad(set_to_none=True)`` before every backward
    pass. With gradient accumulation into existing ``.grad`` tensors, reduce after the last micro-batch with
    ``reduce_now`` instead.
    """

    def __init__(self, group=None, average: bool = True, overlap: bool = False, reserve_sms: int = 0):
        self.group = group
        self.average = average
        # with overlap: SMs that the dX GEMM leaves free for the collective's CTAs (moc_set_overlap_sm_reserve)
        self.reserve_sms = int(reserve_sms) if overlap else 0
        # overlap=True starts the reduction behind the weight-gradient GEMM, beside the dX GEMM; the default
        # starts it after the backward pass
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
        if self.reserve_sms:
            _lib.check(_lib.lib().moc_set_overlap_sm_reserve(self.reserve_sms), "moc_set_overlap_sm_reserve")
        return self

    def __exit__(self, *exc):
        _ffn.set_grad_ready_hook(None)
        if self.reserve_sms:
            _lib.lib().moc_set_overlap_sm_reserve(0)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        return False


def _recorded_event():
    ev = torch.cuda.Event()
    ev.record()
    return ev
