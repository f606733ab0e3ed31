"""Decode-time MoC FFN on the B200 kernels, behind the surface of the reference's
``moc/inference/inference_ffn.py`` (``InferenceMoCSwiGLUFFN``, inference_ffn.py:30-315).

Same constructor, configuration object, parameter names and mode strings; the fast modes launch
libmoc_b200's decode kernels (``moc_decode_global`` / ``moc_decode_2of8`` / ``moc_decode_dense``)
instead of cuBLAS + the CUDA extension + Triton. ``masked_reference`` stays what it is in the
reference: the dense-masking definition written with PyTorch ops, used to check the fast modes.
Differences: grouped 2:8 accepts an intermediate size that is not a multiple of 8 (the tail group
contributes top-min(2, tail) channels, as the training path does, moc/ffn.py:62-108), and the
fast modes need bf16 CUDA tensors and raise otherwise (there is no fallback).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from .ffn import _moc_2_8_effective_k, transpose_weight


@dataclass(frozen=True)
class InferenceMoCConfig:
    hidden_size: int
    intermediate_size: int
    k: int
    grouped_a: Optional[int] = None
    grouped_b: Optional[int] = None

    @property
    def grouped(self) -> bool:
        return self.grouped_a is not None and self.grouped_b is not None


def _check_fast_inputs(x_2d: torch.Tensor, *weights: torch.Tensor) -> None:
    for t in (x_2d, *weights):
        if not t.is_cuda:
            raise ValueError("all tensors must be CUDA")
        if t.dtype != torch.bfloat16:
            raise ValueError("x and the weights must be BF16")


class InferenceMoCSwiGLUFFN(nn.Module):
    """Inference-only MoC FFN (inference_ffn.py:30-315).

    Modes (``forward(x, mode=...)``):
      - dense_baseline: dense SwiGLU FFN (inference_ffn.py:164-167)
      - masked_reference: dense masking reference in PyTorch ops (inference_ffn.py:169-180)
      - moc_inference_optimized_global_after_gate_native: global Top-K MoC (inference_ffn.py:182-196)
      - moc_inference_grouped_top2of8: MoC 2:8 (inference_ffn.py:281-298)
      - auto: the fast mode matching the configuration
    """

    def __init__(self, hidden_size: int, intermediate_size: int, k: int,
                 grouped_a: Optional[int] = None, grouped_b: Optional[int] = None):
        super().__init__()
        if k < 1 or k > intermediate_size:
            raise ValueError(f"k={k} must be in [1, {intermediate_size}]")
        if (grouped_a is None) != (grouped_b is None):
            raise ValueError("grouped_a and grouped_b must be set together")
        if grouped_a is not None:
            if (grouped_a, grouped_b) != (2, 8):
                raise ValueError("grouped MoC supports grouped_a=2, grouped_b=8")
            expected_k = _moc_2_8_effective_k(intermediate_size)
            if k != expected_k:
                raise ValueError(f"grouped MoC requires k=intermediate_size*a/b={expected_k}, got {k}")
        self.config = InferenceMoCConfig(hidden_size, intermediate_size, k, grouped_a, grouped_b)
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        self._down_weight_t: torch.Tensor | None = None
        self._down_weight_t_source_ptr: int | None = None
        self._compile_frozen: bool = False
        self._workspaces: dict = {}

    # ---- caches -------------------------------------------------------------------------------
    def _ensure_down_weight_t(self) -> None:
        """Keep W_down^T [d_ffn, d] contiguous next to the parameter (inference_ffn.py:104-110)."""
        if getattr(self, "_compile_frozen", False):
            return
        w = self.down_proj.weight
        key = (w.data_ptr(), w._version, w.dtype)
        if self._down_weight_t is None or self._down_weight_t_source_ptr != key:
            with torch.no_grad():
                self._down_weight_t = transpose_weight(w.detach()) if w.is_cuda else w.detach().t().contiguous()
            self._down_weight_t_source_ptr = key

    def freeze_for_compile(self, device: torch.device | None = None) -> None:
        """Refresh the cached transposed down weight and stop tracking parameter changes
        (inference_ffn.py:112-129)."""
        self._compile_frozen = False
        self._ensure_down_weight_t()
        self._compile_frozen = True

    def _workspace(self, batch: int, device) -> torch.Tensor:
        key = (batch, str(device))
        ws = self._workspaces.get(key)
        if ws is None:
            nbytes = _lib.lib().moc_decode_workspace_bytes(batch, self.config.hidden_size,
                                                           self.config.intermediate_size)
            ws = torch.empty(nbytes, device=device, dtype=torch.uint8)
            self._workspaces[key] = ws
        return ws

    # ---- shape helpers (inference_ffn.py:131-143) -------------------------------------------------
    def _flatten_decode_input(self, x: torch.Tensor) -> tuple[torch.Tensor, tuple[int, ...]]:
        if x.dim() == 2:
            return x, tuple(x.shape)
        if x.dim() == 3 and x.shape[1] == 1:
            return x[:, 0, :], tuple(x.shape)
        raise ValueError(f"expected decode shape [batch, hidden] or [batch, 1, hidden], got {tuple(x.shape)}")

    def _restore_output_shape(self, y_2d: torch.Tensor, original_shape: tuple[int, ...]) -> torch.Tensor:
        if len(original_shape) == 2:
            return y_2d
        return y_2d.unsqueeze(1)

    # ---- reference-definition modes ----------------------------------------------------------------
    def _select_channels(self, gate_values: torch.Tensor):
        """Selection of masked_reference (inference_ffn.py:145-162), extended by the tail rule."""
        if not self.config.grouped:
            return torch.topk(gate_values, self.config.k, dim=-1, largest=True, sorted=False)
        inter = self.config.intermediate_size
        full, tail = divmod(inter, 8)
        vals, idxs = [], []
        if full:
            grouped = gate_values[:, : full * 8].reshape(gate_values.shape[0], full, 8)
            v, local = torch.topk(grouped, 2, dim=-1)
            base = (torch.arange(full, device=gate_values.device, dtype=torch.int64) * 8).view(1, full, 1)
            vals.append(v.reshape(gate_values.shape[0], -1))
            idxs.append((local + base).reshape(gate_values.shape[0], -1))
        if tail:
            v, local = torch.topk(gate_values[:, full * 8:], min(2, tail), dim=-1)
            vals.append(v)
            idxs.append(local + full * 8)
        return torch.cat(vals, dim=-1), torch.cat(idxs, dim=-1)

    def masked_reference(self, x: torch.Tensor) -> torch.Tensor:
        x_2d, original_shape = self._flatten_decode_input(x)
        gate_full = self.gate_proj(x_2d)
        up_full = self.up_proj(x_2d)
        topk_vals, topk_idx = self._select_channels(gate_full)
        sparse_z = F.silu(topk_vals) * torch.gather(up_full, -1, topk_idx)
        z_full = torch.zeros_like(gate_full)
        z_full.scatter_(-1, topk_idx, sparse_z)
        return self._restore_output_shape(self.down_proj(z_full), original_shape)

    # ---- fast modes -----------------------------------------------------------------------------
    def _run(self, fn_name: str, x: torch.Tensor, with_k: bool) -> torch.Tensor:
        lib = _lib.lib()
        self._ensure_down_weight_t()
        x_2d, original_shape = self._flatten_decode_input(x)
        x_2d = x_2d.contiguous()
        wg, wu, wdt = self.gate_proj.weight, self.up_proj.weight, self._down_weight_t
        _check_fast_inputs(x_2d, wg, wu, wdt)
        batch, d = x_2d.shape
        d_ffn = self.config.intermediate_size
        y = torch.empty(batch, d, device=x_2d.device, dtype=x_2d.dtype)
        ws = self._workspace(batch, x_2d.device)
        args = [batch, d, d_ffn]
        if with_k:
            args.append(self.config.k)
        args += [x_2d.data_ptr(), wg.data_ptr(), wu.data_ptr(), wdt.data_ptr(), y.data_ptr(), ws.data_ptr(),
                 ws.numel(), _lib.stream_ptr(x_2d.device)]
        with torch.cuda.device(x_2d.device):       # the library launches on the current device
            _lib.check(getattr(lib, fn_name)(*args), fn_name)
        _lib.watch_status(ws, fn_name)             # asynchronous time-out check (one tiny launch; not recorded into graphs)
        return self._restore_output_shape(y, original_shape)

    def dense_baseline(self, x: torch.Tensor) -> torch.Tensor:
        return self._run("moc_decode_dense", x, with_k=False)

    def moc_inference_optimized_global_after_gate_native(self, x: torch.Tensor) -> torch.Tensor:
        """Global MoC: gate projection, Top-K and the selected projections in one call."""
        if self.config.grouped:
            raise ValueError("moc_inference_optimized_global_after_gate_native requires ungrouped global MoC")
        return self._run("moc_decode_global", x, with_k=True)

    def moc_inference_grouped_top2of8(self, x: torch.Tensor) -> torch.Tensor:
        if not (self.config.grouped and self.config.grouped_a == 2 and self.config.grouped_b == 8):
            raise ValueError(
                "moc_inference_grouped_top2of8 requires grouped MoC with grouped_a=2, grouped_b=8.")
        return self._run("moc_decode_2of8", x, with_k=False)

    def make_graph_runner(self, batch_size: int, mode: str = "auto"):
        """Capture one decode call of `mode` for a fixed batch size in a CUDA graph (the reference builds
        such runners per mode: inference_ffn.py:205-279, optimized_global_moc_ops.py:106-162). Returns
        runner(x) -> y; y is a persistent buffer that the next call overwrites."""
        dev = self.gate_proj.weight.device
        dtype = self.gate_proj.weight.dtype
        x_buf = torch.zeros(batch_size, self.config.hidden_size, device=dev, dtype=dtype)
        self._ensure_down_weight_t()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                y_buf = self.forward(x_buf, mode=mode)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_buf = self.forward(x_buf, mode=mode)

        def runner(x_in: torch.Tensor) -> torch.Tensor:
            x_2d, original_shape = self._flatten_decode_input(x_in)
            if x_2d.shape[0] != batch_size:
                raise ValueError(f"graph runner built for batch_size={batch_size}, got {x_2d.shape[0]}")
            x_buf.copy_(x_2d)
            graph.replay()
            return self._restore_output_shape(y_buf, original_shape)

        return runner

    def make_moc2_8_graph_runner(self, batch_size: int, **_unused):
        """inference_ffn.py:205-279 (the tile-size keyword arguments of the Triton kernels have no meaning here)."""
        if not (self.config.grouped and self.config.grouped_a == 2 and self.config.grouped_b == 8):
            raise ValueError("graph runner requires grouped MoC with grouped_a=2, grouped_b=8.")
        return self.make_graph_runner(batch_size, mode="moc_inference_grouped_top2of8")

    def forward(self, x: torch.Tensor, mode: str = "auto") -> torch.Tensor:
        if mode == "auto":
            mode = ("moc_inference_grouped_top2of8" if self.config.grouped
                    else "moc_inference_optimized_global_after_gate_native")
        if mode == "dense_baseline":
            return self.dense_baseline(x)
        if mode == "masked_reference":
            return self.masked_reference(x)
        if mode == "moc_inference_optimized_global_after_gate_native":
            return self.moc_inference_optimized_global_after_gate_native(x)
        if mode == "moc_inference_grouped_top2of8":
            return self.moc_inference_grouped_top2of8(x)
        raise ValueError(f"unknown mode={mode}")
