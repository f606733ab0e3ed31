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

import ctypes
import os

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


class SymmGradReducer(GradAllReducer):
    """Gradient reduction by the library's own kernel over NVLink peer memory (``moc_symm_allreduce``) instead of
    an NCCL call: one process per GPU of one node, at most 8 ranks, NCCL only for the set-up rendezvous.

    The reducer owns the gradient buffers: each FFN layer's [3, d_ffn * d] bucket is a symmetric allocation
    (``torch.distributed._symmetric_memory``) that every rank maps, handed to the backward pass through
    ``moc_b200.ffn.set_bucket_provider``, so the weight-gradient GEMM writes straight into memory the peers can
    reach. When the GEMM is done, one small kernel per rank (``ctas`` CTAs, by default three per reserved SM) reduces
    the rank's slice in the NVSwitch (``multimem.ld_reduce`` / ``multimem.st``; plain peer loads and stores when the
    allocation has no multicast mapping) beside the dX GEMM, which leaves ``reserve_sms`` SMs free. Its CTA count
    is fixed by this process, unlike a library collective's, so the two kernels always fit side by side.

    Because the buffers persist, the gradients of one step are overwritten by the next backward pass: call
    ``zero_grad(set_to_none=True)`` before every backward pass and do not keep references to old gradients.
    Every rank must run the same layers in the same order (allocation is a collective). Gradients that do not come
    as a bucket (parameter dtype different from the compute dtype) fall back to the NCCL path of the base class.
    """

    def __init__(self, group=None, average: bool = True, overlap: bool = True, reserve_sms: int = 8,
                 ctas: int | None = None, use_multicast: bool = True):
        super().__init__(group=group, average=average, overlap=overlap, reserve_sms=reserve_sms)
        self.use_multicast = use_multicast      # False: plain peer loads / stores even when a multicast mapping exists
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self._group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self._group)
        self.world = dist.get_world_size(self._group)
        if self.world > 8:
            raise ValueError("SymmGradReducer handles at most 8 ranks (one node)")
        self.ctas = int(ctas) if ctas else (3 * reserve_sms if overlap and reserve_sms else 96)
        self._buckets: dict = {}       # key -> (tensor, handle)
        self._flags = None
        self._flag_handle = None
        self._calls = 0
        self.multicast = None

    def _alloc(self, numel: int, dtype: torch.dtype, device) -> tuple:
        if os.environ.get("MOC_B200_SYMM_DISABLE") == "1":     # lets a caller exercise its fallback path
            raise RuntimeError("symmetric memory disabled by MOC_B200_SYMM_DISABLE=1")
        t = self._symm.empty(numel, dtype=dtype, device=device)
        return t, self._symm.rendezvous(t, self._group)

    def _provide(self, key, numel: int, dtype: torch.dtype, device):
        if self.world == 1 or (numel * dtype.itemsize) % 16 != 0 or dtype not in (torch.bfloat16, torch.float32):
            return None
        entry = self._buckets.get((key, numel, dtype))
        if entry is None:
            if self._flags is None:
                nflag = _lib.lib().moc_symm_allreduce_flag_bytes() // 4
                self._flags, self._flag_handle = self._alloc(nflag, torch.int32, device)
                self._flags.zero_()
                torch.cuda.synchronize(device)
                dist.barrier(group=self._group)       # nobody signals before every rank's flags are zero
            entry = self._alloc(numel, dtype, device)
            self._buckets[(key, numel, dtype)] = entry
            self.multicast = bool(entry[1].multicast_ptr) and self.use_multicast
        return entry[0]

    def _on_grad_ready(self, name: str, grad: torch.Tensor, event) -> None:
        entry = None
        if name == "bucket" and grad.is_cuda:
            for (key, numel, dtype), e in self._buckets.items():
                if e[0].data_ptr() == grad.data_ptr() and numel == grad.numel():
                    entry = e
                    break
        if entry is None:
            return super()._on_grad_ready(name, grad, event)
        handle = entry[1]
        ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in handle.buffer_ptrs])
        flags = (ctypes.c_void_p * self.world)(*[int(p) for p in self._flag_handle.buffer_ptrs])
        self._calls += 1
        self.comm_stream.wait_event(event)
        with torch.cuda.device(grad.device):
            rc = _lib.lib().moc_symm_allreduce(_lib.dtype_code(grad.dtype), self.rank, self.world, ptrs,
                                               (int(handle.multicast_ptr) or None) if self.use_multicast else None, flags,
                                               grad.numel() * grad.element_size(), 1 if self.average else 0,
                                               self._calls, self.ctas, self.comm_stream.cuda_stream)
        _lib.check(rc, "moc_symm_allreduce")
        self.launched += 1

    def check(self) -> None:
        """Synchronises the reduction stream and raises if a wait for another rank timed out."""
        if self._flags is not None:
            with torch.cuda.device(self._flags.device):
                _lib.check(_lib.lib().moc_symm_allreduce_status(self._flags.data_ptr(), self.comm_stream.cuda_stream),
                           "moc_symm_allreduce")

    def __enter__(self):
        _ffn.set_bucket_provider(self._provide)
        return super().__enter__()

    def __exit__(self, *exc):
        _ffn.set_bucket_provider(None)
        return super().__exit__(*exc)
