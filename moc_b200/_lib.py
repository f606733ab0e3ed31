"""ctypes binding of libmoc_b200.so (the C ABI declared in include/moc_b200.h).

There is no fallback: if the shared library is missing or a call fails, a RuntimeError is
raised. The library is built in-tree by ``python -m moc_b200.build``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libmoc_b200.so"

MOC_BF16, MOC_F32 = 0, 1
SELECT_TOPK, SELECT_2OF8, SELECT_POST_SILU_ABS = 0, 1, 2
ERR_DEVICE_TIMEOUT = -6

_DTYPES = {torch.bfloat16: MOC_BF16, torch.float32: MOC_F32}

# name -> (restype, argtypes); mirrors include/moc_b200.h one to one
_P = c_void_p
SIGNATURES = {
    "moc_b200_abi_version": (c_int, []),
    "moc_last_error": (c_char_p, []),
    "moc_ffn_ld": (c_int64, [c_int64]),
    "moc_mask_words": (c_int64, [c_int64]),
    "moc_select_2of8_k": (c_int64, [c_int64]),
    "moc_ffn_fwd_workspace_bytes": (c_int64, [c_int, c_int64, c_int64]),
    "moc_ffn_fwd_workspace_bytes_select": (c_int64, [c_int, c_int, c_int64, c_int64]),
    "moc_ffn_bwd_workspace_bytes": (c_int64, [c_int, c_int64, c_int64]),
    "moc_transpose": (c_int, [c_int, _P, _P, c_int64, c_int64, _P]),
    "moc_topk_select": (c_int, [c_int, _P, c_int64, c_int64, c_int64, c_int64, _P, _P, _P, _P, _P]),
    "moc_select_2of8": (c_int, [c_int, _P, c_int64, c_int64, c_int64, _P, _P, _P, _P, _P]),
    "moc_gemm": (c_int, [c_int, c_int, c_int64, c_int64, c_int64, _P, c_int64, c_int, _P, c_int64, c_int, _P,
                         c_int64, c_int, _P, _P]),
    "moc_ffn_fwd": (c_int, [c_int, c_int, c_int64, c_int64, c_int64, c_int64] + [_P] * 13 + [c_int64, _P]),
    "moc_ffn_bwd": (c_int, [c_int, c_int64, c_int64, c_int64, c_int64] + [_P] * 15 + [c_int64, _P, _P, _P, _P]),
    "moc_profile_begin": (c_int, [_P, c_int]),
    "moc_profile_end": (c_int, [_P, c_int]),
    "moc_side_launch_count": (c_int64, []),
    "moc_set_overlap_sm_reserve": (c_int, [c_int]),
    "moc_read_status": (c_int, [_P, _P]),
    "moc_dense_ffn_fwd": (c_int, [c_int, c_int64, c_int64, c_int64] + [_P] * 8 + [c_int64, _P]),
    "moc_dense_ffn_bwd": (c_int, [c_int, c_int64, c_int64, c_int64] + [_P] * 12 + [c_int64, _P]),
    "moc_decode_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "moc_decode_global": (c_int, [c_int64] * 4 + [_P] * 6 + [c_int64, _P]),
    "moc_decode_after_gate": (c_int, [c_int64] * 4 + [_P] * 6 + [c_int64, _P]),
    "moc_decode_2of8": (c_int, [c_int64] * 3 + [_P] * 6 + [c_int64, _P]),
    "moc_decode_dense": (c_int, [c_int64] * 3 + [_P] * 6 + [c_int64, _P]),
    "moc_decode_global_static": (c_int, [c_int64] * 4 + [_P] * 5 + [_P]),
    "moc_decode_static_max_batch": (c_int64, []),
    "moc_decode_static_max_d": (c_int64, []),
    "moc_decode_static_max_d_ffn": (c_int64, []),
    "moc_decode_selected_down": (c_int, [c_int64] * 4 + [_P] * 5 + [c_int64, _P]),
    "moc_decode_selected_up": (c_int, [c_int64] * 4 + [_P] * 6),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared library once and declare every symbol of the header."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m moc_b200.build` "
                "(there is no CPU or PyTorch fallback for the MoC kernels)")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            if not hasattr(handle, name):
                continue   # optional entry points are checked where they are used
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        if handle.moc_b200_abi_version() != 1:
            raise RuntimeError("libmoc_b200.so has an unexpected ABI version")
        _lib = handle
    return _lib


def exported(name: str) -> bool:
    return hasattr(lib(), name)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"moc_b200 supports torch.bfloat16 and torch.float32 tensors, got {dtype}") from None


def last_error() -> str:
    msg = lib().moc_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}: {last_error()}")


def ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    return t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class _StatusRing:
    """Always-on detection of bounded-wait time-outs without a host synchronisation.

    Every kernel wait of the library is bounded; a wait that runs out sets the status word at the start of
    the call's workspace and the kernel returns early, leaving its outputs incomplete. After each call the
    wrappers copy that word into a small ring of pinned host slots (one asynchronous 4-byte copy on the
    caller's stream plus an event); at the next call the slots whose events have completed are read, and a
    non-zero word raises ``RuntimeError`` (MOC_ERR_DEVICE_TIMEOUT), at the latest one call after the failure.
    ``flush`` synchronises and checks everything that is pending. Nothing is enqueued while the stream is being
    captured into a CUDA graph."""

    SLOTS = 16

    def __init__(self, device):
        self.device = device
        self.host = torch.zeros(self.SLOTS, dtype=torch.int32).pin_memory()
        self.events = [None] * self.SLOTS
        self.what = [""] * self.SLOTS
        self.next = 0

    def _check_slot(self, i: int, wait: bool) -> None:
        ev = self.events[i]
        if ev is None:
            return
        if wait:
            ev.synchronize()
        elif not ev.query():
            return
        self.events[i] = None
        word = int(self.host[i])
        if word != 0:
            self.host[i] = 0
            raise RuntimeError(
                f"{self.what[i]} failed with code {ERR_DEVICE_TIMEOUT}: device-side wait timed out "
                f"(role {(word >> 24) & 0xFF}, detail 0x{word & 0xFFFFFF:x}); the outputs of that call are incomplete")

    def poll(self) -> None:
        for i in range(self.SLOTS):
            self._check_slot(i, wait=False)

    def push(self, ws: torch.Tensor, what: str) -> None:
        if torch.cuda.is_current_stream_capturing():
            return
        self.poll()
        i = self.next
        self._check_slot(i, wait=True)       # the ring wrapped around a copy that is still in flight
        self.next = (i + 1) % self.SLOTS
        self.host[i:i + 1].copy_(ws[:4].view(torch.int32), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.events[i] = ev
        self.what[i] = what

    def flush(self) -> None:
        for i in range(self.SLOTS):
            self._check_slot(i, wait=True)


_rings: dict = {}


def watch_status(ws: torch.Tensor, what: str) -> None:
    """Queue the status word of the call that just used workspace ``ws`` for the asynchronous time-out check and
    raise for any earlier call whose word came back non-zero."""
    key = ws.device.index
    ring = _rings.get(key)
    if ring is None:
        ring = _rings[key] = _StatusRing(ws.device)
    ring.push(ws, what)


def flush_status() -> None:
    """Wait for every queued status word and raise if one reports a time-out."""
    for ring in _rings.values():
        ring.flush()


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("MoC B200 kernels require CUDA tensors.")
