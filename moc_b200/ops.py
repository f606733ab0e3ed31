"""torch.library custom ops over the C ABI: the dispatcher-visible form of the decode entry points.

The reference exposes its decode kernels as dispatcher ops so that they can sit inside ``torch.compile``d
models: ``moc_native::optimized_global_topk_bf16``, ``..._selected_up_silu_bf16``, ``..._selected_down_bf16``,
``..._after_gate_bf16`` (optimized_global_moc_ext.cpp:88-100, optimized_global_moc_ops.py:53-93) and
``moc::fused_grouped_top2_up_silu`` / ``moc::selected_grouped_down`` (triton_grouped_moc_ops.py:26-143).
This module registers the same operations, with the same argument meaning, in the ``moc_b200`` namespace; each
has a fake (meta) kernel, so FakeTensor tracing and ``torch.compile`` see shapes and dtypes without running the
CUDA code. The eager modules (``InferenceMoCSwiGLUFFN``) call the C ABI directly and do not pay the
dispatcher's per-call cost; these ops are for callers that need a traceable graph.

Differences from the reference ops: selected channel indices come back in ascending channel order (the
reference's are in ``torch.topk`` order), ties at the K-th score go to the lower channel, and bf16 is the only
dtype, as in the reference.
"""
from __future__ import annotations

import torch

from . import _lib
from .ffn import _moc_2_8_effective_k

_BF16 = torch.bfloat16


def _check_bf16_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("MoC fused helper kernels require CUDA tensors.")
        if t.dtype != _BF16:
            raise TypeError(f"moc_b200 decode ops compute in bfloat16, got {t.dtype}")


def _workspace(batch: int, d: int, d_ffn: int, device) -> tuple[torch.Tensor, int]:
    n = _lib.lib().moc_decode_workspace_bytes(batch, d, d_ffn)
    return torch.empty(n, device=device, dtype=torch.uint8), n


@torch.library.custom_op("moc_b200::global_topk", mutates_args=())
def global_topk(scores: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Row-wise Top-K of [batch, d_ffn] gate scores: (values [batch, k], int64 indices [batch, k])."""
    _check_bf16_cuda(scores)
    scores = scores.contiguous()
    batch, d_ffn = scores.shape
    lib = _lib.lib()
    words = lib.moc_mask_words(d_ffn)
    idx = torch.empty(batch, k, device=scores.device, dtype=torch.int16)
    vals = torch.empty(batch, k, device=scores.device, dtype=_BF16)
    bitmap = torch.empty(batch, words, device=scores.device, dtype=torch.int32)
    rank0 = torch.empty(batch, words, device=scores.device, dtype=torch.int16)
    rc = lib.moc_topk_select(_lib.dtype_code(_BF16), scores.data_ptr(), d_ffn, batch, d_ffn, k, idx.data_ptr(),
                             vals.data_ptr(), bitmap.data_ptr(), rank0.data_ptr(), _lib.stream_ptr(scores.device))
    _lib.check(rc, "moc_topk_select")
    return vals, idx.to(torch.int64)


@global_topk.register_fake
def _(scores, k):
    batch = scores.shape[0]
    return scores.new_empty(batch, k), scores.new_empty(batch, k, dtype=torch.int64)


@torch.library.custom_op("moc_b200::selected_up_silu", mutates_args=())
def selected_up_silu(x: torch.Tensor, topk_vals: torch.Tensor, topk_idx: torch.Tensor,
                     up_weight: torch.Tensor) -> torch.Tensor:
    """sparse_z[b, j] = SiLU(topk_vals[b, j]) * (x[b] . up_weight[topk_idx[b, j]])."""
    _check_bf16_cuda(x, topk_vals, up_weight)
    x, topk_vals, up_weight = x.contiguous(), topk_vals.contiguous(), up_weight.contiguous()
    idx16 = topk_idx.to(torch.int16).contiguous()
    batch, d = x.shape
    k = topk_vals.shape[1]
    z = torch.empty(batch, k, device=x.device, dtype=_BF16)
    rc = _lib.lib().moc_decode_selected_up(batch, k, d, up_weight.shape[0], x.data_ptr(), topk_vals.data_ptr(),
                                           idx16.data_ptr(), up_weight.data_ptr(), z.data_ptr(),
                                           _lib.stream_ptr(x.device))
    _lib.check(rc, "moc_decode_selected_up")
    return z


@selected_up_silu.register_fake
def _(x, topk_vals, topk_idx, up_weight):
    return torch.empty_like(topk_vals, dtype=x.dtype)


@torch.library.custom_op("moc_b200::selected_down", mutates_args=())
def selected_down(sparse_z: torch.Tensor, topk_idx: torch.Tensor, down_weight_t: torch.Tensor) -> torch.Tensor:
    """y[b] = sum_j sparse_z[b, j] * down_weight_t[topk_idx[b, j]]; down_weight_t is W_down^T [d_ffn, d]."""
    _check_bf16_cuda(sparse_z, down_weight_t)
    sparse_z, down_weight_t = sparse_z.contiguous(), down_weight_t.contiguous()
    idx16 = topk_idx.to(torch.int16).contiguous()
    batch, k = sparse_z.shape
    d_ffn, d = down_weight_t.shape
    y = torch.empty(batch, d, device=sparse_z.device, dtype=_BF16)
    ws, n = _workspace(batch, d, d_ffn, sparse_z.device)
    rc = _lib.lib().moc_decode_selected_down(batch, k, d, d_ffn, sparse_z.data_ptr(), idx16.data_ptr(),
                                             down_weight_t.data_ptr(), y.data_ptr(), ws.data_ptr(), n,
                                             _lib.stream_ptr(sparse_z.device))
    _lib.check(rc, "moc_decode_selected_down")
    return y


@selected_down.register_fake
def _(sparse_z, topk_idx, down_weight_t):
    return sparse_z.new_empty(sparse_z.shape[0], down_weight_t.shape[1])


@torch.library.custom_op("moc_b200::global_after_gate", mutates_args=())
def global_after_gate(x: torch.Tensor, gate_scores: torch.Tensor, up_weight: torch.Tensor,
                      down_weight_t: torch.Tensor, k: int) -> torch.Tensor:
    """Global MoC decode FFN after the gate projection, one op: Top-K on gate_scores, selected up + SiLU,
    gathered down projection."""
    _check_bf16_cuda(x, gate_scores, up_weight, down_weight_t)
    x, gate_scores = x.contiguous(), gate_scores.contiguous()
    up_weight, down_weight_t = up_weight.contiguous(), down_weight_t.contiguous()
    batch, d = x.shape
    d_ffn = up_weight.shape[0]
    y = torch.empty(batch, d, device=x.device, dtype=_BF16)
    ws, n = _workspace(batch, d, d_ffn, x.device)
    rc = _lib.lib().moc_decode_after_gate(batch, d, d_ffn, k, x.data_ptr(), gate_scores.data_ptr(),
                                          up_weight.data_ptr(), down_weight_t.data_ptr(), y.data_ptr(),
                                          ws.data_ptr(), n, _lib.stream_ptr(x.device))
    _lib.check(rc, "moc_decode_after_gate")
    return y


@global_after_gate.register_fake
def _(x, gate_scores, up_weight, down_weight_t, k):
    return x.new_empty(x.shape[0], down_weight_t.shape[1])


@torch.library.custom_op("moc_b200::global_ffn", mutates_args=())
def global_ffn(x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor, down_weight_t: torch.Tensor,
               k: int) -> torch.Tensor:
    """Whole global-MoC decode FFN including the gate projection (one cooperative launch at batch 1)."""
    _check_bf16_cuda(x, gate_weight, up_weight, down_weight_t)
    x, gate_weight = x.contiguous(), gate_weight.contiguous()
    up_weight, down_weight_t = up_weight.contiguous(), down_weight_t.contiguous()
    batch, d = x.shape
    d_ffn = up_weight.shape[0]
    y = torch.empty(batch, d, device=x.device, dtype=_BF16)
    ws, n = _workspace(batch, d, d_ffn, x.device)
    rc = _lib.lib().moc_decode_global(batch, d, d_ffn, k, x.data_ptr(), gate_weight.data_ptr(), up_weight.data_ptr(),
                                      down_weight_t.data_ptr(), y.data_ptr(), ws.data_ptr(), n,
                                      _lib.stream_ptr(x.device))
    _lib.check(rc, "moc_decode_global")
    return y


@global_ffn.register_fake
def _(x, gate_weight, up_weight, down_weight_t, k):
    return x.new_empty(x.shape[0], down_weight_t.shape[1])


@torch.library.custom_op("moc_b200::grouped_2of8_ffn", mutates_args=())
def grouped_2of8_ffn(x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor,
                     down_weight_t: torch.Tensor) -> torch.Tensor:
    """MoC 2:8 decode FFN: top-2 of every 8 consecutive gate channels, up + SiLU, gathered down projection (the
    pair moc::fused_grouped_top2_up_silu + moc::selected_grouped_down of the reference as one op; d_ffn need
    not be a multiple of 8, the tail group keeps min(2, tail) channels)."""
    _check_bf16_cuda(x, gate_weight, up_weight, down_weight_t)
    x, gate_weight = x.contiguous(), gate_weight.contiguous()
    up_weight, down_weight_t = up_weight.contiguous(), down_weight_t.contiguous()
    batch, d = x.shape
    d_ffn = up_weight.shape[0]
    y = torch.empty(batch, d, device=x.device, dtype=_BF16)
    ws, n = _workspace(batch, d, d_ffn, x.device)
    rc = _lib.lib().moc_decode_2of8(batch, d, d_ffn, x.data_ptr(), gate_weight.data_ptr(), up_weight.data_ptr(),
                                    down_weight_t.data_ptr(), y.data_ptr(), ws.data_ptr(), n, _lib.stream_ptr(x.device))
    _lib.check(rc, "moc_decode_2of8")
    return y


@grouped_2of8_ffn.register_fake
def _(x, gate_weight, up_weight, down_weight_t):
    return x.new_empty(x.shape[0], down_weight_t.shape[1])


def grouped_2of8_k(d_ffn: int) -> int:
    """Channels the 2:8 rule keeps for a given width (moc/ffn.py:62-65)."""
    return _moc_2_8_effective_k(d_ffn)
