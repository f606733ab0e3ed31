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
    "moc_symm_allreduce": (c_int, [c_int, c_int, c_int, _P, _P, _P, c_int64, c_int, ctypes.c_uint32, c_int, _P]),
    "moc_symm_allreduce_flag_bytes": (c_int64, []),
    "moc_host_rmsnorm": (c_int, [c_int64, c_int64, _P, _P, _P, _P, ctypes.c_float, _P]),
    "moc_host_rope_cache": (c_int, [c_int64] * 4 + [_P] * 8),
    "moc_host_attn_step": (c_int, [c_int64] * 4 + [_P] * 6),
    "moc_symm_allreduce_status": (c_int, [_P, _P]),
    "moc_read_status": (c_int, [_P, _P]),
    "moc_publish_status": (c_int, [_P, _P, _P]),
    "moc_debug_set_wait_cycles": (c_int, [c_int64]),
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


class _StatusSink:
    """Always-on detection of bounded-wait time-outs without a host synchronisation and without a copy.

    Every kernel wait of the library is bounded; a wait that runs out sets the status word at the start of
    the call's workspace and the kernel returns early, leaving its outputs incomplete. After each call the
    wrappers enqueue ``moc_publish_status``: a one-thread kernel that stores a non-zero status word into one
    pinned host word per device (the GPU reaches pinned host memory directly; nothing is written in the normal
    case, and no copy engine is involved, so the check never queues behind a large transfer). At the next call
    the host word is read, and a non-zero word raises ``RuntimeError`` (MOC_ERR_DEVICE_TIMEOUT). Calls
    recorded into a CUDA graph are not followed by the publish kernel (replays are unchecked)."""

    def __init__(self, device):
        self.device = device
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.view = self.host.numpy()
        self.what = ""

    def check(self) -> None:
        word = int(self.view[0])
        if word != 0:
            self.view[0] = 0
            raise RuntimeError(
                f"{self.what or 'a moc_b200 call'} failed with code {ERR_DEVICE_TIMEOUT}: device-side wait timed out "
                f"(role {(word >> 24) & 0xFF}, detail 0x{word & 0xFFFFFF:x}); the outputs of that call are incomplete")

    def push(self, ws: torch.Tensor, what: str) -> None:
        self.check()
        if torch.cuda.is_current_stream_capturing():
            return      # a dependent one-thread node would cost a decode graph about 2 us per FFN call
        with torch.cuda.device(self.device):
            check(lib().moc_publish_status(ws.data_ptr(), self.host.data_ptr(), stream_ptr(self.device)),
                  "moc_publish_status")
        self.what = what


_sinks: dict = {}


def watch_status(ws: torch.Tensor, what: str) -> None:
    """Queue the status word of the call that just used workspace ``ws`` for the asynchronous time-out check and
    raise for any earlier call whose word came back non-zero."""
    key = ws.device.index
    sink = _sinks.get(key)
    if sink is None:
        sink = _sinks[key] = _StatusSink(ws.device)
    sink.push(ws, what)


def flush_status() -> None:
    """Wait for the queued work of every device that ran a call and raise if one reported a time-out."""
    for sink in _sinks.values():
        torch.cuda.synchronize(sink.device)
        sink.check()


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("MoC B200 kernels require CUDA tensors.")
