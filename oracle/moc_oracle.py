"""CPU oracle for the MoC sparse SwiGLU FFN path.

TEST INFRASTRUCTURE ONLY. This file restates, in plain PyTorch-on-CPU / numpy, the algorithm
of the reference implementation (xiaohuangji/MoC) for the FFN hot path so that the CUDA
kernels can be checked against it. Only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it; the product
package ``moc_b200`` never does.

Pinning: the reference ships no tests and no golden vectors, so the oracle is pinned against
outputs of the reference itself: ``tests/golden/make_golden.py`` imports the reference's own
``moc.ffn.MoCSwiGLUFFN`` / ``moc.inference.inference_ffn.InferenceMoCSwiGLUFFN`` (pure PyTorch
paths, CPU), runs them on seeded inputs and stores the results under ``tests/golden``;
``tests/test_oracle_golden.py`` checks every function here against those fixtures.

Each function cites the reference lines it follows (paths inside the reference project).

Tie rule. ``torch.topk`` leaves the choice among equal values unspecified (with bf16 gates,
ties at the K-th value are the norm). The oracle fixes it the way the reference's own CUDA
decode kernel does (stable descending radix sort of order keys,
moc/inference/cuda/optimized_global_moc_ext.cu:26-29, :85-125): among equal values the lower
channel index wins, values are compared in the IEEE total order (-0 < +0).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

# --------------------------------------------------------------------------------------
# order keys and channel selection
# --------------------------------------------------------------------------------------


def order_keys(g: torch.Tensor) -> torch.Tensor:
    """Order-preserving integer keys (int64) of a bf16 or fp32 tensor.

    bf16: moc/inference/cuda/optimized_global_moc_ext.cu:26-29 (bf16_order_key); the fp32
    variant applies the same sign-flip map to 32-bit patterns.
    """
    if g.dtype == torch.bfloat16:
        bits = g.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
        neg = (bits & 0x8000) != 0
        return torch.where(neg, bits ^ 0xFFFF, bits ^ 0x8000)
    if g.dtype == torch.float32:
        bits = g.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        neg = (bits & 0x80000000) != 0
        return torch.where(neg, bits ^ 0xFFFFFFFF, bits ^ 0x80000000)
    raise TypeError(f"order_keys: unsupported dtype {g.dtype}")


def canonical_topk(g: torch.Tensor, k: int, dim: int = -1, largest: bool = True, sorted: bool = False):
    """Row-wise Top-K with the canonical tie rule; drop-in for ``torch.topk`` as the reference
    calls it (moc/ffn.py:144, :392; moc/inference/inference_ffn.py:147-153).

    Returns (values, indices[int64]) with indices in ascending channel order.
    """
    assert dim in (-1, g.dim() - 1) and largest
    keys = order_keys(g)
    # stable descending sort: equal keys keep ascending index order
    order = torch.sort(keys, dim=-1, descending=True, stable=True).indices
    idx = torch.sort(order[..., :k], dim=-1).values
    return torch.gather(g, -1, idx), idx


def select_2of8(g: torch.Tensor):
    """Top-2 of every 8 consecutive channels, top-min(2, tail) of the tail group
    (moc/ffn.py:68-108); lower index wins ties
    (moc/inference/triton_fused_ffn_kernels.py:103-114). Ascending channel order."""
    inter = g.shape[-1]
    full, tail = divmod(inter, 8)
    parts = []
    if full:
        grouped = g[..., : full * 8].reshape(*g.shape[:-1], full, 8)
        _, local = canonical_topk(grouped, 2)
        base = (torch.arange(full, dtype=torch.int64) * 8).view(*([1] * (g.dim() - 1)), full, 1)
        parts.append((local + base).reshape(*g.shape[:-1], full * 2))
    if tail:
        _, local = canonical_topk(g[..., full * 8:], min(2, tail))
        parts.append(local + full * 8)
    idx = torch.cat(parts, dim=-1)
    return torch.gather(g, -1, idx), idx


def effective_k_2of8(inter: int) -> int:
    """moc/ffn.py:62-65."""
    full, tail = divmod(inter, 8)
    return full * 2 + min(2, tail)


def selection_bitmap(idx: torch.Tensor, inter: int) -> np.ndarray:
    """uint32 mask words [rows, ceil128(inter)/32] of a selected index set (layout of the CUDA
    kernels' bitmap output; no counterpart in the reference, which keeps indices only)."""
    rows = idx.reshape(-1, idx.shape[-1]).numpy()
    words = (inter + 127) // 128 * 4
    out = np.zeros((rows.shape[0], words), dtype=np.uint32)
    r = np.repeat(np.arange(rows.shape[0]), rows.shape[1])
    c = rows.reshape(-1)
    np.bitwise_or.at(out, (r, c // 32), (np.uint32(1) << (c % 32).astype(np.uint32)))
    return out


# --------------------------------------------------------------------------------------
# training path
# --------------------------------------------------------------------------------------


def _select(g, k, select):
    if select == "topk":
        return canonical_topk(g, k)
    if select == "2of8":
        return select_2of8(g)
    if select == "post_silu_abs":
        # moc/ffn.py:336-339: the K largest |SiLU(g)|; the values handed on are the pre-SiLU gates there
        _, idx = canonical_topk(F.silu(g).abs(), k)
        return torch.gather(g, -1, idx), idx
    raise ValueError(select)


def moc_forward(x, gate_w, up_w, down_w, k, select="topk", idx_override=None):
    """MoC forward, pure-PyTorch branch of the reference (moc/ffn.py:141-163 for `moc`,
    :389-414 for `moc_gcp`, :277-298 for `moc_2_8`, :333-354 for `moc_post_silu_abs`). All tensors share one dtype (fp32 or
    bf16); every op rounds to that dtype exactly where the reference's tensor ops do.

    ``idx_override`` (int64 [..., k]) replaces the selection step by a given channel set; the
    tests use it to compare the remaining arithmetic under an identical mask when the gate
    values of two implementations differ in their last bit.

    Returns a dict: y, idx (int64, ascending), g_sel, u_sel, s_sel, z_sel, g (dense gate).
    """
    inter = gate_w.shape[0]
    g = x @ gate_w.t()                                   # ffn.py:141
    if idx_override is None:
        g_sel, idx = _select(g, k, select)               # ffn.py:144
    else:
        idx = idx_override
        g_sel = torch.gather(g, -1, idx)
    u = x @ up_w.t()                                     # ffn.py:146
    u_sel = torch.gather(u, -1, idx)                     # ffn.py:156
    s_sel = F.silu(g_sel)                                # ffn.py:157
    z_sel = s_sel * u_sel                                # ffn.py:158
    z_full = torch.zeros(*x.shape[:-1], inter, dtype=z_sel.dtype)
    z_full.scatter_(-1, idx, z_sel)                      # ffn.py:160-161
    y = z_full @ down_w.t()                              # ffn.py:163
    return dict(y=y, idx=idx, g_sel=g_sel, u_sel=u_sel, s_sel=s_sel, z_sel=z_sel, g=g)


def moc_backward(grad_y, x, gate_w, up_w, down_w, idx, g_sel, u_sel, s_sel=None, z_sel=None):
    """MoC backward (moc/ffn.py:176-259). With s_sel/z_sel = None this is the moc_gcp variant
    (moc/ffn.py:424-497): it recomputes them first (:435-436) and forms dX with one fused
    addmm_ (:491-494) instead of two rounded products. Returns (dx, d_gate_w, d_up_w, d_down_w)."""
    inter = gate_w.shape[0]
    gcp = s_sel is None
    if s_sel is None:
        s_sel = F.silu(g_sel)                            # ffn.py:435
    if z_sel is None:
        z_sel = s_sel * u_sel                            # ffn.py:436
    z_full = torch.zeros(*x.shape[:-1], inter, dtype=z_sel.dtype)
    z_full.scatter_(-1, idx, z_sel)                      # ffn.py:198-199
    z_2d = z_full.reshape(-1, inter)
    go_2d = grad_y.reshape(-1, grad_y.shape[-1])
    d_down_w = go_2d.t() @ z_2d                          # ffn.py:203
    grad_z_full = grad_y @ down_w                        # ffn.py:206
    x_2d = x.reshape(-1, x.shape[-1])
    grad_z = torch.gather(grad_z_full, -1, idx)          # ffn.py:219
    grad_s = u_sel * grad_z                              # ffn.py:222
    grad_u_sel = s_sel * grad_z                          # ffn.py:223
    sig = torch.sigmoid(g_sel)                           # ffn.py:226
    silu_deriv = sig * (1.0 + g_sel * (1.0 - sig))       # ffn.py:227
    grad_g_sel = grad_s * silu_deriv                     # ffn.py:229
    grad_g = torch.zeros(*x.shape[:-1], inter, dtype=grad_g_sel.dtype)
    grad_g.scatter_(-1, idx, grad_g_sel)                 # ffn.py:232-233
    grad_u = torch.zeros(*x.shape[:-1], inter, dtype=grad_u_sel.dtype)
    grad_u.scatter_(-1, idx, grad_u_sel)                 # ffn.py:235-236
    d_gate_w = grad_g.reshape(-1, inter).t() @ x_2d      # ffn.py:239
    dx_g = grad_g @ gate_w                               # ffn.py:245
    d_up_w = grad_u.reshape(-1, inter).t() @ x_2d        # ffn.py:248
    if gcp:
        dx = dx_g
        dx.reshape(-1, dx.shape[-1]).addmm_(grad_u.reshape(-1, inter), up_w)   # ffn.py:491-494
    else:
        dx_u = grad_u @ up_w                             # ffn.py:254
        dx = (dx_g + dx_u).to(x.dtype)                   # ffn.py:255
    return dx, d_gate_w, d_up_w, d_down_w


def dense_forward(x, gate_w, up_w, down_w):
    """Dense SwiGLU (moc/ffn.py:120-121)."""
    return (F.silu(x @ gate_w.t()) * (x @ up_w.t())) @ down_w.t()


def dense_forward_backward(x, gate_w, up_w, down_w, grad_y):
    """Dense SwiGLU forward + autograd backward, as nn.Linear + autograd compute it for
    StandardSwiGLUFFN (moc/ffn.py:111-121). Returns (y, dx, d_gate_w, d_up_w, d_down_w)."""
    xs = x.detach().clone().requires_grad_(True)
    ws = [w.detach().clone().requires_grad_(True) for w in (gate_w, up_w, down_w)]
    y = dense_forward(xs, *ws)
    y.backward(grad_y)
    return y.detach(), xs.grad, ws[0].grad, ws[1].grad, ws[2].grad


# --------------------------------------------------------------------------------------
# decode path
# --------------------------------------------------------------------------------------


def masked_reference(x, gate_w, up_w, down_w, k=None, select="topk"):
    """Decode-time MoC FFN, dense masking form (moc/inference/inference_ffn.py:169-180);
    x is [batch, hidden]."""
    gate_full = F.linear(x, gate_w)
    up_full = F.linear(x, up_w)
    vals, idx = _select(gate_full, k, select)
    sparse_z = F.silu(vals) * torch.gather(up_full, -1, idx)
    z_full = torch.zeros_like(gate_full)
    z_full.scatter_(-1, idx, sparse_z)
    return F.linear(z_full, down_w)


def dense_baseline(x, gate_w, up_w, down_w):
    """moc/inference/inference_ffn.py:164-167."""
    return F.linear(F.silu(F.linear(x, gate_w)) * F.linear(x, up_w), down_w)


# --------------------------------------------------------------------------------------
# seeded synthetic inputs (shared by tests, smoke and bench so that all sides see the same data)
# --------------------------------------------------------------------------------------


def make_inputs(tokens, d, d_ffn, dtype, seed=1234, weight_seed=0):
    """x, grad_y ~ N(0,1) (seed), weights ~ N(0, 0.02) (weight_seed), generated in fp32 on
    the CPU generator and rounded to `dtype` (benchmarks/training/benchmark_training_latency.py:112-124;
    moc/model.py:117-122)."""
    gw = torch.Generator().manual_seed(weight_seed)
    gate_w = (torch.randn(d_ffn, d, generator=gw) * 0.02).to(dtype)
    up_w = (torch.randn(d_ffn, d, generator=gw) * 0.02).to(dtype)
    down_w = (torch.randn(d, d_ffn, generator=gw) * 0.02).to(dtype)
    gx = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, d, generator=gx).to(dtype)
    grad_y = torch.randn(tokens, d, generator=gx).to(dtype)
    return x, grad_y, gate_w, up_w, down_w
