"""Dense SwiGLU FFN on the B200 GEMM core: the comparison row of the reference
(``StandardSwiGLUFFN``, moc/ffn.py:111-121) with the same module surface, running
``moc_dense_ffn_fwd`` / ``moc_dense_ffn_bwd`` instead of three ``nn.Linear`` calls plus autograd."""
from __future__ import annotations

import torch

from . import _lib
from .ffn import _maybe_check_status, transpose_weight


class _DenseSwiGLUFunction(torch.autograd.Function):
    """Saves x and the rounded gate / up activations G, U (what autograd keeps for the reference's
    dense FFN besides SiLU(G) and Z, which are recomputed here)."""

    @staticmethod
    def forward(ctx, x, gate_w, up_w, down_w, down_w_t=None):
        if not x.is_cuda:
            raise ValueError("The B200 dense SwiGLU kernels require CUDA tensors.")
        lib = _lib.lib()
        compute_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled() else x.dtype
        code = _lib.dtype_code(compute_dtype)
        x2d = x.reshape(-1, x.shape[-1]).to(compute_dtype).contiguous()
        gw = gate_w.detach().to(compute_dtype).contiguous()
        uw = up_w.detach().to(compute_dtype).contiguous()
        wdt = down_w_t
        if wdt is None or wdt.dtype != compute_dtype:
            wdt = transpose_weight(down_w.detach().to(compute_dtype))
        tokens, d = x2d.shape
        d_ffn = gw.shape[0]
        ld = lib.moc_ffn_ld(d_ffn)
        dev = x2d.device
        y = torch.empty(tokens, d, device=dev, dtype=compute_dtype)
        g = torch.empty(tokens, ld, device=dev, dtype=compute_dtype)
        u = torch.empty(tokens, ld, device=dev, dtype=compute_dtype)
        nbytes = lib.moc_ffn_fwd_workspace_bytes(code, tokens, d_ffn)
        ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
        with torch.cuda.device(dev):
            _lib.check(lib.moc_dense_ffn_fwd(code, tokens, d, d_ffn, x2d.data_ptr(), gw.data_ptr(), uw.data_ptr(),
                                             wdt.data_ptr(), y.data_ptr(), g.data_ptr(), u.data_ptr(), ws.data_ptr(),
                                             nbytes, _lib.stream_ptr(dev)), "moc_dense_ffn_fwd")
        _maybe_check_status(ws, dev, "moc_dense_ffn_fwd")
        ctx.save_for_backward(x2d, gw, uw, wdt, g, u)
        ctx.x_shape, ctx.x_dtype = x.shape, x.dtype
        ctx.w_dtypes = (gate_w.dtype, up_w.dtype, down_w.dtype)
        return y.reshape(x.shape)   # compute dtype, as nn.Linear under autocast

    @staticmethod
    def backward(ctx, grad_out):
        lib = _lib.lib()
        x2d, gw, uw, wdt, g, u = ctx.saved_tensors
        tokens, d = x2d.shape
        d_ffn = gw.shape[0]
        dt, dev = x2d.dtype, x2d.device
        code = _lib.dtype_code(dt)
        go = grad_out.reshape(-1, d).to(dt).contiguous()
        dx = torch.empty(tokens, d, device=dev, dtype=dt)
        d_gate = torch.empty(d_ffn, d, device=dev, dtype=dt)
        d_up = torch.empty(d_ffn, d, device=dev, dtype=dt)
        d_down = torch.empty(d, d_ffn, device=dev, dtype=dt)
        nbytes = lib.moc_ffn_bwd_workspace_bytes(code, tokens, d_ffn)
        ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
        with torch.cuda.device(dev):
            _lib.check(lib.moc_dense_ffn_bwd(code, tokens, d, d_ffn, go.data_ptr(), x2d.data_ptr(), gw.data_ptr(),
                                             uw.data_ptr(), wdt.data_ptr(), g.data_ptr(), u.data_ptr(), dx.data_ptr(),
                                             d_gate.data_ptr(), d_up.data_ptr(), d_down.data_ptr(), ws.data_ptr(),
                                             nbytes, _lib.stream_ptr(dev)), "moc_dense_ffn_bwd")
        _maybe_check_status(ws, dev, "moc_dense_ffn_bwd")
        return (dx.reshape(ctx.x_shape).to(ctx.x_dtype), d_gate.to(ctx.w_dtypes[0]), d_up.to(ctx.w_dtypes[1]),
                d_down.to(ctx.w_dtypes[2]), None)


def dense_swiglu(x, gate_w, up_w, down_w, down_w_t=None):
    """down(silu(gate(x)) * up(x)) (moc/ffn.py:120-121) through the B200 kernels. ``down_w_t``: optional cached
    W_down^T [d_ffn, d] in the compute dtype (the kernels read the down weight in that layout); built per call
    when absent."""
    if not x.is_cuda:
        raise ValueError("The B200 dense SwiGLU kernels require CUDA tensors.")
    return _DenseSwiGLUFunction.apply(x, gate_w, up_w, down_w, down_w_t)
