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


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("MoC B200 kernels require CUDA tensors.")
