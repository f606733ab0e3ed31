"""B200-native Mixture-of-Channels SwiGLU FFN behind the reference's plugin surface.

Mirrors ``moc/ffn.py`` of xiaohuangji/MoC: ``build_ffn`` (ffn.py:584-609), ``MoCSwiGLUFFN``
(ffn.py:500-581) and ``StandardSwiGLUFFN`` (ffn.py:111-121) keep their names, constructor
arguments, attributes, parameter names/shapes and error behaviour, so the modules drop into
``moc/model.py`` (``TransformerBlock`` calls ``build_ffn(d, d_ffn, ffn_type=..., k=...)``,
model.py:81) and load the reference's checkpoints. What differs is what runs: every mode
launches the hand-written sm_100a kernels of libmoc_b200 through its C ABI. There is no
Triton, no PyTorch fallback and no CPU path; CPU tensors raise ``ValueError`` exactly like
the reference's fused modes do (ffn.py:135-136).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib

_MOC_MODES = (
    "moc",
    "moc_gcp",
    "moc_triton_aux",
    "moc_gcp_triton_aux",
    "moc_2_8",
    "moc_2_8_triton_aux",
    "moc_post_silu_abs",
    "moc_post_silu_abs_triton_aux",
)


def _moc_2_8_effective_k(intermediate_size: int) -> int:
    """K' of the 2:8 rule (moc/ffn.py:62-65)."""
    full_groups, tail = divmod(intermediate_size, 8)
    return full_groups * 2 + min(2, tail)


# ------------------------------------------------------------------------------------------
# thin op layer over the C ABI (tensors in, tensors out; allocation by PyTorch's caching allocator)
# ------------------------------------------------------------------------------------------


def transpose_weight(w: torch.Tensor) -> torch.Tensor:
    """W [rows, cols] -> W^T [cols, rows] contiguous, by the library's transpose kernel."""
    _lib.require_cuda(w)
    w = w.contiguous()
    out = torch.empty(w.shape[1], w.shape[0], device=w.device, dtype=w.dtype)
    with torch.cuda.device(w.device):
        _lib.check(_lib.lib().moc_transpose(_lib.dtype_code(w.dtype), w.data_ptr(), out.data_ptr(), w.shape[0],
                                            w.shape[1], _lib.stream_ptr(w.device)), "moc_transpose")
    return out


def moc_ffn_forward(x2d, gate_w, up_w, down_w_t, k: int, select: int, save_sz: bool):
    """One MoC FFN forward through ``moc_ffn_fwd``. Returns
    (y, idx, g_sel, u_sel, s_sel | None, z_sel | None, bitmap, rank0)."""
    lib = _lib.lib()
    _lib.require_cuda(x2d, gate_w, up_w, down_w_t)
    tokens, d = x2d.shape
    d_ffn = gate_w.shape[0]
    dt = x2d.dtype
    code = _lib.dtype_code(dt)
    dev = x2d.device
    words = lib.moc_mask_words(d_ffn)
    y = torch.empty(tokens, d, device=dev, dtype=dt)
    idx = torch.empty(tokens, k, device=dev, dtype=torch.int16)
    g_sel = torch.empty(tokens, k, device=dev, dtype=dt)
    u_sel = torch.empty(tokens, k, device=dev, dtype=dt)
    s_sel = torch.empty(tokens, k, device=dev, dtype=dt) if save_sz else None
    z_sel = torch.empty(tokens, k, device=dev, dtype=dt) if save_sz else None
    bitmap = torch.empty(tokens, words, device=dev, dtype=torch.int32)
    rank0 = torch.empty(tokens, words, device=dev, dtype=torch.int16)
    ws_bytes = lib.moc_ffn_fwd_workspace_bytes_select(code, select, tokens, d_ffn)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):       # the library launches on the current device
        rc = _call_fwd(lib, code, select, tokens, d, d_ffn, k, x2d, gate_w, up_w, down_w_t, y, idx, g_sel, u_sel, s_sel,
                       z_sel, bitmap, rank0, ws, ws_bytes, dev)
    _lib.check(rc, "moc_ffn_fwd")
    _maybe_check_status(ws, dev, "moc_ffn_fwd")
    return y, idx, g_sel, u_sel, s_sel, z_sel, bitmap, rank0


def _call_fwd(lib, code, select, tokens, d, d_ffn, k, x2d, gate_w, up_w, down_w_t, y, idx, g_sel, u_sel, s_sel, z_sel,
              bitmap, rank0, ws, ws_bytes, dev):
    return lib.moc_ffn_fwd(code, select, tokens, d, d_ffn, k, x2d.data_ptr(), gate_w.data_ptr(), up_w.data_ptr(),
                         down_w_t.data_ptr(), y.data_ptr(), idx.data_ptr(), g_sel.data_ptr(), u_sel.data_ptr(),
                         _lib.ptr(s_sel), _lib.ptr(z_sel), bitmap.data_ptr(), rank0.data_ptr(), ws.data_ptr(),
                         ws_bytes, _lib.stream_ptr(dev))


def moc_ffn_backward(grad_y2d, x2d, gate_w, up_w, down_w_t, idx, g_sel, u_sel, s_sel, z_sel,
                     grad_events=None):
    """One MoC FFN backward through ``moc_ffn_bwd``. Returns (dx, d_gate_w, d_up_w, d_down_w) in
    the dtype of the inputs. ``grad_events``: optional (ev_down, ev_gate, ev_up) torch.cuda.Event
    objects recorded as soon as each weight gradient is final."""
    lib = _lib.lib()
    tokens, d = x2d.shape
    d_ffn = gate_w.shape[0]
    k = g_sel.shape[1]
    dt = x2d.dtype
    code = _lib.dtype_code(dt)
    dev = x2d.device
    dx = torch.empty(tokens, d, device=dev, dtype=dt)
    # the three weight gradients are views of one buffer, so that a data-parallel caller can reduce them with a
    # single collective (moc_b200.dp)
    bucket = _bucket_provider(gate_w.data_ptr(), 3 * d_ffn * d, dt, dev) if _bucket_provider is not None else None
    bucket = torch.empty(3, d_ffn * d, device=dev, dtype=dt) if bucket is None else bucket.view(3, d_ffn * d)
    d_down = bucket[0].view(d, d_ffn)
    d_gate = bucket[1].view(d_ffn, d)
    d_up = bucket[2].view(d_ffn, d)
    ws_bytes = lib.moc_ffn_bwd_workspace_bytes(code, tokens, d_ffn)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
    evs = [None, None, None]
    if grad_events is not None:
        evs = [e.cuda_event if e is not None else None for e in grad_events]
    with torch.cuda.device(dev):       # the library launches on the current device
        rc = lib.moc_ffn_bwd(code, tokens, d, d_ffn, k, grad_y2d.data_ptr(), x2d.data_ptr(), gate_w.data_ptr(),
                             up_w.data_ptr(), down_w_t.data_ptr(), idx.data_ptr(), g_sel.data_ptr(),
                             u_sel.data_ptr(), _lib.ptr(s_sel), _lib.ptr(z_sel), dx.data_ptr(), d_gate.data_ptr(),
                             d_up.data_ptr(), d_down.data_ptr(), ws.data_ptr(), ws_bytes, evs[0], evs[1], evs[2],
                             _lib.stream_ptr(dev))
    _lib.check(rc, "moc_ffn_bwd")
    _maybe_check_status(ws, dev, "moc_ffn_bwd")
    return dx, d_gate, d_up, d_down, bucket


_CHECK_STATUS = False


def set_status_checks(enabled: bool) -> None:
    """When enabled, every op synchronises and raises if a kernel recorded a bounded-wait
    time-out (costs a stream sync per call; meant for tests and debugging). When disabled (the default) the
    same check runs asynchronously and raises one call later (moc_b200._lib.watch_status)."""
    global _CHECK_STATUS
    _CHECK_STATUS = bool(enabled)


def _maybe_check_status(ws: torch.Tensor, dev, what: str = "moc_b200 call") -> None:
    """Time-out detection after a call that used workspace ``ws``: synchronous when ``set_status_checks(True)``,
    otherwise through the pinned status word of the device (raises at the next call, or at ``flush_status``)."""
    if _CHECK_STATUS:
        _lib.check(_lib.lib().moc_read_status(ws.data_ptr(), _lib.stream_ptr(dev)), "device status")
    else:
        _lib.watch_status(ws, what)


# ------------------------------------------------------------------------------------------
# autograd
# ------------------------------------------------------------------------------------------

# Hook for data-parallel training: when set, it is called right after the backward kernels were enqueued, as
# hook("bucket", flat, event) with the [3, d_ffn * d] buffer that the three returned weight gradients are views
# of (down, gate, up), or, when a parameter dtype differs from the compute dtype, as hook(name, grad, event) for
# name in ("down", "gate", "up"). `event` is recorded on the compute stream at the point where the gradient is
# final. The hook may reduce the tensor in place. See moc_b200.dp.
_grad_ready_hook = None
# True: events fire as soon as the weight-gradient GEMM is done, so a reduction can run beside the dX GEMM.
# False (default): one event after the whole backward pass. The dX GEMM hands out its tiles in arrival order, so a
# collective that takes SMs away only makes it proportionally slower; for the collective to find free SMs while
# the GEMM runs, the caller also reserves some (moc_set_overlap_sm_reserve, see moc_b200.dp.GradAllReducer).
_grad_ready_early = False


# Optional source of the [3 * d_ffn * d] gradient buffer of a backward call: provider(key, numel, dtype, device) ->
# flat tensor or None (None: a fresh allocation). `key` identifies the layer (address of its gate weight). A data-
# parallel reducer that needs the gradients in memory its peers can reach hands out its own buffers here
# (moc_b200.dp.SymmGradReducer).
_bucket_provider = None


def set_bucket_provider(provider) -> None:
    global _bucket_provider
    _bucket_provider = provider


def set_grad_ready_hook(hook, early: bool = False) -> None:
    global _grad_ready_hook, _grad_ready_early
    _grad_ready_hook = hook
    _grad_ready_early = bool(early)


class _MoCB200Function(torch.autograd.Function):
    """Autograd node of the MoC FFN; stands where _MoCFunction / _MoCGCPFunction / _MoC28Function
    stand in the reference (moc/ffn.py:124-259, :262-310, :372-497).

    Saved for backward: x, the selected channel indices (int16), g_sel and u_sel: the compact
    [tokens, k] activation layout of moc/ffn.py:417, never a dense [tokens, d_ffn] tensor. The
    reference's `moc` mode additionally keeps s_sel = SiLU(g_sel) and z_sel = s_sel * u_sel
    (moc/ffn.py:166-169) to skip their recomputation; here the backward kernels rebuild both
    bit-identically inside their own passes at no extra cost, so `moc` and `moc_gcp` share the
    smaller saved set unless ``materialize_sz`` asks for the reference's one.
    """

    @staticmethod
    def forward(ctx, x, gate_w, up_w, down_w, down_w_t, k, select, recompute_sz):
        if not x.is_cuda:
            raise ValueError("MoC fused helper kernels require CUDA tensors.")
        compute_dtype = x.dtype
        if torch.is_autocast_enabled():
            compute_dtype = torch.get_autocast_dtype("cuda")
        if compute_dtype not in (torch.bfloat16, torch.float32):
            raise TypeError(f"moc_b200 computes in bfloat16 or float32, got {compute_dtype}")
        x2d = x.reshape(-1, x.shape[-1]).to(compute_dtype).contiguous()
        gw = gate_w.detach().to(compute_dtype).contiguous()
        uw = up_w.detach().to(compute_dtype).contiguous()
        if down_w_t is None or down_w_t.dtype != compute_dtype:
            down_w_t = transpose_weight(down_w.detach().to(compute_dtype))
        y, idx, g_sel, u_sel, s_sel, z_sel, bitmap, rank0 = moc_ffn_forward(
            x2d, gw, uw, down_w_t, k, select, save_sz=not recompute_sz)
        saved = [x2d, gw, uw, down_w_t, idx, g_sel, u_sel]
        if not recompute_sz:
            saved += [s_sel, z_sel]
        ctx.save_for_backward(*saved)
        ctx.recompute_sz = recompute_sz
        ctx.set_materialize_grads(False)   # no zero-filled gradient tensor for the integer index output
        ctx.x_shape = x.shape
        ctx.x_dtype = x.dtype
        ctx.w_dtypes = (gate_w.dtype, up_w.dtype, down_w.dtype)
        ctx.mark_non_differentiable(idx)
        # like the reference's matmuls under autocast, the output has the compute dtype (moc/ffn.py:163)
        return y.reshape(x.shape), idx.reshape(*x.shape[:-1], k)

    @staticmethod
    def backward(ctx, grad_out, _grad_idx):
        if grad_out is None:
            return (None,) * 8
        saved = ctx.saved_tensors
        x2d, gw, uw, down_w_t, idx, g_sel, u_sel = saved[:7]
        s_sel, z_sel = (None, None) if ctx.recompute_sz else saved[7:9]
        go = grad_out.reshape(-1, grad_out.shape[-1]).to(x2d.dtype).contiguous()
        hook = _grad_ready_hook
        events = None
        if hook is not None and _grad_ready_early:
            events = tuple(torch.cuda.Event() for _ in range(3))
            for ev in events:
                ev.record()   # PyTorch creates the CUDA event lazily; the library re-records it
        dx, d_gate, d_up, d_down, bucket = moc_ffn_backward(go, x2d, gw, uw, down_w_t, idx, g_sel, u_sel, s_sel,
                                                            z_sel, events)
        same_dtype = all(dt == bucket.dtype for dt in ctx.w_dtypes)
        d_gate = d_gate.to(ctx.w_dtypes[0])
        d_up = d_up.to(ctx.w_dtypes[1])
        d_down = d_down.to(ctx.w_dtypes[2])
        if hook is not None and (events is None or not same_dtype):
            # after the last backward kernel; also when the gradients were converted to another parameter dtype:
            # the converted tensors are written by cast kernels queued behind the dX GEMM, so the early events
            # (recorded behind the weight-gradient GEMM) do not cover them
            done = torch.cuda.Event()
            done.record()
            events = (done, done, done)
        if hook is not None and same_dtype:
            hook("bucket", bucket, events[2])      # one collective over the three gradients (views of `bucket`)
        elif hook is not None:
            hook("down", d_down, events[0])
            hook("gate", d_gate, events[1])
            hook("up", d_up, events[2])
        return dx.reshape(ctx.x_shape).to(ctx.x_dtype), d_gate, d_up, d_down, None, None, None, None


# ------------------------------------------------------------------------------------------
# modules
# ------------------------------------------------------------------------------------------


class StandardSwiGLUFFN(nn.Module):
    """Standard LLaMA-style SwiGLU FFN (moc/ffn.py:111-121): down(silu(gate(x)) * up(x))."""

    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        # W_down^T [d_ffn, d] copy the kernels read, refreshed whenever the parameter changes (as in MoCSwiGLUFFN)
        self._down_weight_t: torch.Tensor | None = None
        self._down_weight_t_key = None

    def _ensure_down_weight_t(self, dtype: torch.dtype) -> torch.Tensor:
        w = self.down_proj.weight
        key = (w.data_ptr(), w._version, dtype, w.device)
        if self._down_weight_t is None or self._down_weight_t_key != key:
            with torch.no_grad():
                self._down_weight_t = transpose_weight(w.detach().to(dtype))
            self._down_weight_t_key = key
        return self._down_weight_t

    def forward(self, x):
        from .dense import dense_swiglu
        if not x.is_cuda:
            raise ValueError("The B200 dense SwiGLU kernels require CUDA tensors.")
        compute_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled() else x.dtype
        return dense_swiglu(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight,
                            self._ensure_down_weight_t(compute_dtype))


class MoCSwiGLUFFN(nn.Module):
    """MoC SwiGLU FFN (moc/ffn.py:500-581) running on the B200 kernels.

    mode='moc' (alias 'moc_triton_aux')         : keep s, z of the selected channels for backward.
    mode='moc_gcp' (alias 'moc_gcp_triton_aux') : recompute them in backward.
    mode='moc_2_8' (alias 'moc_2_8_triton_aux') : structured top-2-of-8 selection; `k` is ignored.
    mode='moc_post_silu_abs' (alias '..._triton_aux') : Top-K on |SiLU(gate)| instead of the gate (moc/ffn.py:313-369).
    """

    def __init__(self, hidden_size: int, intermediate_size: int, k: int | None = None,
                 mode: str = "moc", index_save_dtype=None):
        super().__init__()
        if mode not in _MOC_MODES:
            raise ValueError(
                f"Unknown mode '{mode}'. Use 'moc', 'moc_gcp', "
                "'moc_triton_aux', 'moc_gcp_triton_aux', "
                "'moc_2_8', 'moc_2_8_triton_aux', "
                "'moc_post_silu_abs', or 'moc_post_silu_abs_triton_aux'."
            )
        self.mode = mode
        self.requested_k = k
        if mode.startswith("moc_2_8"):
            self.k_effective = _moc_2_8_effective_k(intermediate_size)
        else:
            if k is None:
                raise ValueError("MoC FFN requires `k` outside moc_2_8 modes.")
            self.k_effective = k
        self.k = self.k_effective
        if self.k < 1 or self.k > intermediate_size:
            raise ValueError(f"k={self.k} must be in [1, {intermediate_size}]")
        if intermediate_size - 1 > torch.iinfo(torch.int16).max:
            # same limit as _pack_topk_idx with int16 indices (moc/ffn.py:27-41)
            raise ValueError(
                f"topk_idx range [0, {intermediate_size - 1}] cannot be stored as {torch.int16}")
        self.index_save_dtype = index_save_dtype
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        # W_down^T [d_ffn, d] copy the kernels read (d_ffn may be odd, which rules out TMA on
        # W_down's own rows); refreshed whenever the parameter changes, never saved.
        self._down_weight_t: torch.Tensor | None = None
        self._down_weight_t_key = None
        # record_topk_idx = True keeps the selected channel indices [..., k] (int16) of the latest forward call in
        # last_topk_idx, for inspection and tests; off by default: it would pin tokens * k * 2 bytes per layer
        self.record_topk_idx = False
        self.last_topk_idx: torch.Tensor | None = None
        # True: also write and keep s_sel, z_sel like the reference's `moc` mode (moc/ffn.py:166-169)
        self.materialize_sz = False

    def _ensure_down_weight_t(self, dtype: torch.dtype) -> torch.Tensor:
        w = self.down_proj.weight
        key = (w.data_ptr(), w._version, dtype, w.device)
        if self._down_weight_t is None or self._down_weight_t_key != key:
            with torch.no_grad():
                self._down_weight_t = transpose_weight(w.detach().to(dtype))
            self._down_weight_t_key = key
        return self._down_weight_t

    def forward(self, x):
        if not x.is_cuda:
            raise ValueError("MoC fused helper kernels require CUDA tensors.")
        compute_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled() else x.dtype
        down_w_t = self._ensure_down_weight_t(compute_dtype)
        if self.mode.startswith("moc_2_8"):
            select = _lib.SELECT_2OF8
        elif self.mode.startswith("moc_post_silu_abs"):
            select = _lib.SELECT_POST_SILU_ABS
        else:
            select = _lib.SELECT_TOPK
        y, idx = _MoCB200Function.apply(
            x,
            self.gate_proj.weight,
            self.up_proj.weight,
            self.down_proj.weight,
            down_w_t,
            self.k,
            select,
            not self.materialize_sz,
        )
        self.last_topk_idx = idx if self.record_topk_idx else None
        return y


def build_ffn(hidden_size: int, intermediate_size: int, ffn_type: str = "dense", k=None):
    """Factory for Dense FFN, MoC, MoC+GCP and MoC 2:8 (moc/ffn.py:584-609): same arguments,
    same accepted ``ffn_type`` strings, same errors."""
    if ffn_type == "dense":
        return StandardSwiGLUFFN(hidden_size, intermediate_size)
    if ffn_type in ("moc", "moc_gcp", "moc_2_8", "moc_post_silu_abs"):
        if k is None and ffn_type != "moc_2_8":
            raise ValueError("MoC FFN requires `k`")
        mode = {
            "moc": "moc_triton_aux",
            "moc_gcp": "moc_gcp_triton_aux",
            "moc_2_8": "moc_2_8_triton_aux",
            "moc_post_silu_abs": "moc_post_silu_abs_triton_aux",
        }[ffn_type]
        return MoCSwiGLUFFN(
            hidden_size,
            intermediate_size,
            k,
            mode=mode,
            index_save_dtype=torch.int16,
        )
    raise ValueError(f"Unknown ffn_type '{ffn_type}'")


def install_into(moc_module) -> None:
    """Rebind the reference package's factory so that ``moc.build_model`` / ``LLaMAModel``
    (moc/model.py:81, :147) construct the B200 modules: ``install_into(moc)`` after
    ``import moc``."""
    import sys

    model_mod = sys.modules.get(moc_module.__name__ + ".model")
    ffn_mod = sys.modules.get(moc_module.__name__ + ".ffn")
    for mod in (moc_module, model_mod, ffn_mod):
        if mod is None:
            continue
        for name, obj in (("build_ffn", build_ffn), ("MoCSwiGLUFFN", MoCSwiGLUFFN),
                          ("StandardSwiGLUFFN", StandardSwiGLUFFN)):
            if hasattr(mod, name):
                setattr(mod, name, obj)
