"""Channel selection kernels (moc_topk_select, moc_select_2of8) through the C ABI against the
oracle's canonical rule on the SAME gate tensor: indices, gathered gate values, bitmap and
ranks must be bit-exact."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from moc_b200 import _lib
from oracle import moc_oracle as O

pytestmark = pytest.mark.gpu


def _run_select(g_cpu: torch.Tensor, k: int, ld: int | None = None, rule="topk"):
    lib = _lib.lib()
    tokens, d_ffn = g_cpu.shape
    dev = torch.device("cuda")
    ld = d_ffn if ld is None else ld
    buf = torch.full((tokens, ld), float("nan"), dtype=g_cpu.dtype)
    buf[:, :d_ffn] = g_cpu
    g = buf.to(dev)
    words = lib.moc_mask_words(d_ffn)
    if rule == "2of8":
        k = lib.moc_select_2of8_k(d_ffn)
    idx = torch.full((tokens, k), -1, device=dev, dtype=torch.int16)
    g_sel = torch.zeros(tokens, k, device=dev, dtype=g_cpu.dtype)
    bitmap = torch.zeros(tokens, words, device=dev, dtype=torch.int32)
    rank0 = torch.zeros(tokens, words, device=dev, dtype=torch.int16)
    code = _lib.dtype_code(g_cpu.dtype)
    if rule == "topk":
        rc = lib.moc_topk_select(code, g.data_ptr(), ld, tokens, d_ffn, k, idx.data_ptr(), g_sel.data_ptr(),
                                 bitmap.data_ptr(), rank0.data_ptr(), _lib.stream_ptr())
    else:
        rc = lib.moc_select_2of8(code, g.data_ptr(), ld, tokens, d_ffn, idx.data_ptr(), g_sel.data_ptr(),
                                 bitmap.data_ptr(), rank0.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "select")
    torch.cuda.synchronize()
    return idx.cpu(), g_sel.cpu(), bitmap.cpu(), rank0.cpu()


def _check(g_cpu, k, ld=None, rule="topk"):
    idx, g_sel, bitmap, rank0 = _run_select(g_cpu, k, ld, rule)
    if rule == "topk":
        ref_vals, ref_idx = O.canonical_topk(g_cpu, k)
    else:
        ref_vals, ref_idx = O.select_2of8(g_cpu)
    assert torch.equal(idx.to(torch.int64), ref_idx)
    bits = lambda t: t.view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32)
    assert torch.equal(bits(g_sel), bits(ref_vals.contiguous()))
    ref_bm = O.selection_bitmap(ref_idx, g_cpu.shape[1])
    got_bm = bitmap.numpy().view(np.uint32)
    assert np.array_equal(got_bm, ref_bm)
    pop = np.array([[bin(int(w)).count("1") for w in row] for row in ref_bm])
    ref_rank = np.cumsum(pop, axis=1) - pop
    assert np.array_equal(rank0.numpy().view(np.uint16).astype(np.int64), ref_rank)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tokens,d_ffn,k", [(5, 173, 40), (3, 1376, 256), (4, 5461, 1024), (2, 8, 1), (2, 9, 9),
                                             (1, 9000, 33), (2, 2048, 384)])
def test_topk_random(dtype, tokens, d_ffn, k):
    g = torch.randn(tokens, d_ffn, generator=torch.Generator().manual_seed(d_ffn + k)).to(dtype)
    _check(g, k)
    _check(g, k, ld=_lib.lib().moc_ffn_ld(d_ffn))     # padded rows, NaN in the padding


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_topk_heavy_ties(dtype):
    gen = torch.Generator().manual_seed(5)
    g = torch.randint(-3, 4, (6, 777), generator=gen).to(dtype)      # 7 distinct values
    for k in (1, 100, 400, 776, 777):
        _check(g, k)
    z = torch.zeros(2, 300, dtype=dtype)                               # all equal: lowest indices win
    z[1, ::2] = -0.0
    _check(z, 17)
    _check(z, 151)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_topk_extremes(dtype):
    g = torch.randn(3, 500, generator=torch.Generator().manual_seed(9)).to(dtype)
    g[0, 7] = float("inf")
    g[0, 8] = float("-inf")
    g[1, :] = -g[1, :].abs()          # all negative
    g[2, 100] = torch.finfo(dtype).max
    g[2, 101] = torch.finfo(dtype).tiny
    _check(g, 50)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tokens,d_ffn", [(3, 173), (2, 5461), (2, 5464), (4, 8), (1, 9), (1, 11), (600, 173),
                                            (515, 5461)])   # 512 rows and more: the warp-per-row vector kernel
def test_select_2of8(dtype, tokens, d_ffn):
    g = torch.randn(tokens, d_ffn, generator=torch.Generator().manual_seed(d_ffn)).to(dtype)
    _check(g, None, rule="2of8")
    gi = torch.randint(-1, 2, (tokens, d_ffn), generator=torch.Generator().manual_seed(1)).to(dtype)
    _check(gi, None, rule="2of8")
    # rows padded to the mask width (NaN in the padding): the bf16 vector kernel, one group of 8 per 16-byte load
    ld = _lib.lib().moc_ffn_ld(d_ffn)
    _check(g, None, ld=ld, rule="2of8")
    _check(gi, None, ld=ld, rule="2of8")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tokens,d_ffn,k", [(1100, 173, 40), (1030, 1376, 256), (1025, 5461, 1024)])
def test_topk_many_rows(dtype, tokens, d_ffn, k):
    """More than 1024 rows: the one-warp-per-row kernels (generic, and the bf16 vector path on padded rows)
    instead of the one-CTA-per-row kernel that small calls use."""
    g = torch.randn(tokens, d_ffn, generator=torch.Generator().manual_seed(tokens)).to(dtype)
    g[3, : d_ffn // 2] = 0.25                      # a row that ties heavily at the threshold
    _check(g, k)
    _check(g, k, ld=_lib.lib().moc_ffn_ld(d_ffn))


# ---- the fused selection of the forward pass at more than 1024 rows (the persistent shared-memory-staged kernel) ----
def _crafted_gate_rows(d_ffn: int, k: int, n_patterns: int = 64) -> torch.Tensor:
    """[n_patterns, d_ffn] bf16 gate rows that stress the selection: plain normal rows, rows drawn from very few
    distinct values (long runs of ties at the threshold), constant rows, mostly-negative rows (negative threshold),
    huge and tiny magnitudes, and a row whose K-th value ties across the word and chunk boundaries."""
    gen = torch.Generator().manual_seed(1234 + d_ffn + k)
    rows = []
    for p in range(n_patterns):
        kind = p % 8
        if kind == 0:
            r = torch.randn(d_ffn, generator=gen) * 0.9
        elif kind == 1:
            vals = torch.tensor([-1.0, -0.5, 0.25, 0.5, 2.0])
            r = vals[torch.randint(0, 5, (d_ffn,), generator=gen)]
        elif kind == 2:
            r = torch.full((d_ffn,), 0.75 if p % 16 == 2 else -3.0)
        elif kind == 3:
            r = -torch.rand(d_ffn, generator=gen) - 0.01
            r[torch.randint(0, d_ffn, (max(1, k // 3),), generator=gen)] = 1.5
        elif kind == 4:
            r = torch.randn(d_ffn, generator=gen) * 1e30
        elif kind == 5:
            r = torch.randn(d_ffn, generator=gen) * 1e-30
        elif kind == 6:
            r = torch.randn(d_ffn, generator=gen).round()          # integers: many ties in every bin
        else:
            r = torch.zeros(d_ffn)
            r[: max(1, k // 2)] = 1.0                                # ties at zero fill the rest, lowest channels win
        rows.append(r + 0.0)        # no negative zeros: a one-hot product sum gives +0 for them
    return torch.stack(rows).to(torch.bfloat16)


@pytest.mark.parametrize("save_sz", [False, True])
@pytest.mark.parametrize("tokens,d_ffn,k", [(1100, 5461, 1024), (1030, 173, 40), (1025, 1000, 1000), (1040, 2049, 1),
                                            (1026, 8192, 2048), (1027, 1376, 37), (2500, 6200, 777)])
def test_fused_forward_selection_bit_exact(tokens, d_ffn, k, save_sz):
    """moc_ffn_fwd with one-hot token rows: the gate row of token t is exactly column t % 64 of W_gate, so the
    selection input is known bit for bit. idx, g_sel, u_sel, bitmap and ranks must equal the oracle's canonical
    Top-K of those rows; the Z' rows left in the workspace must be zero outside the selected channels and
    round(round(SiLU(g)) * u) on them (one bf16 ulp allowed: the device sigmoid uses ex2/rcp approximations)."""
    from moc_b200 import ffn as F

    lib = _lib.lib()
    dev = torch.device("cuda")
    d = 64
    g_rows = _crafted_gate_rows(d_ffn, k)                                   # [64, d_ffn]
    gen = torch.Generator().manual_seed(99)
    u_rows = (torch.randn(64, d_ffn, generator=gen) * 0.7).to(torch.bfloat16)
    wg = g_rows.t().contiguous().to(dev)                                    # [d_ffn, 64]
    wu = u_rows.t().contiguous().to(dev)
    wdt = (torch.randn(d_ffn, d, generator=gen) * 0.02).to(torch.bfloat16).to(dev)
    pat = torch.arange(tokens) % 64
    x = torch.zeros(tokens, d, dtype=torch.bfloat16)
    x[torch.arange(tokens), pat] = 1.0
    x = x.to(dev)
    words = lib.moc_mask_words(d_ffn)
    ld = lib.moc_ffn_ld(d_ffn)
    y = torch.empty(tokens, d, device=dev, dtype=torch.bfloat16)
    idx = torch.full((tokens, k), -1, device=dev, dtype=torch.int16)
    g_sel = torch.zeros(tokens, k, device=dev, dtype=torch.bfloat16)
    u_sel = torch.zeros_like(g_sel)
    s_sel = torch.zeros_like(g_sel) if save_sz else None
    z_sel = torch.zeros_like(g_sel) if save_sz else None
    bitmap = torch.zeros(tokens, words, device=dev, dtype=torch.int32)
    rank0 = torch.zeros(tokens, words, device=dev, dtype=torch.int16)
    ws_bytes = lib.moc_ffn_fwd_workspace_bytes(0, tokens, d_ffn)
    ws = torch.zeros(ws_bytes, device=dev, dtype=torch.uint8)
    rc = F._call_fwd(lib, 0, 0, tokens, d, d_ffn, k, x, wg, wu, wdt, y, idx, g_sel, u_sel, s_sel, z_sel, bitmap, rank0,
                     ws, ws_bytes, dev)
    _lib.check(rc, "moc_ffn_fwd")
    _lib.check(lib.moc_read_status(ws.data_ptr(), _lib.stream_ptr()), "device status")
    torch.cuda.synchronize()

    ref_vals, ref_idx = O.canonical_topk(g_rows, k)                          # per pattern
    ref_vals, ref_idx = ref_vals[pat], ref_idx[pat]
    bits = lambda t: t.contiguous().view(torch.int16)
    assert torch.equal(idx.cpu().to(torch.int64), ref_idx)
    assert torch.equal(bits(g_sel.cpu()), bits(ref_vals))
    ref_u = torch.gather(u_rows[pat], 1, ref_idx)
    assert torch.equal(bits(u_sel.cpu()), bits(ref_u))
    ref_bm = O.selection_bitmap(ref_idx[:64], d_ffn)
    assert np.array_equal(bitmap.cpu().numpy().view(np.uint32)[:64], ref_bm)
    pop = np.array([[bin(int(w)).count("1") for w in row] for row in ref_bm])
    assert np.array_equal(rank0.cpu().numpy().view(np.uint16)[:64].astype(np.int64), np.cumsum(pop, axis=1) - pop)
    assert torch.equal(bitmap.cpu()[64:128], bitmap.cpu()[:64]) if tokens >= 128 else True
    # Z' rows: first dense scratch matrix of the workspace, [tokens, ld]
    zdense = ws[256:256 + tokens * ld * 2].view(torch.bfloat16).view(tokens, ld).cpu().float()
    s_ref = torch.nn.functional.silu(ref_vals.float()).to(torch.bfloat16).float()
    z_ref = (s_ref * ref_u.float()).to(torch.bfloat16).float()
    z_got = torch.gather(zdense[:, :d_ffn], 1, ref_idx)
    ulp = torch.maximum(z_ref.abs(), torch.tensor(1e-37)) * 2.0 ** -7
    assert bool(((z_got - z_ref).abs() <= 2 * ulp).all())
    mask = torch.zeros(tokens, ld, dtype=torch.bool)
    mask.scatter_(1, ref_idx, True)
    assert bool((zdense[~mask] == 0).all())
    if save_sz:
        assert bool(((z_sel.cpu().float() - z_ref).abs() <= 2 * ulp).all())
        assert torch.equal(bits(z_sel.cpu()), bits(z_got.to(torch.bfloat16)))
        s_ulp = torch.maximum(s_ref.abs(), torch.tensor(1e-37)) * 2.0 ** -7
        assert bool(((s_sel.cpu().float() - s_ref).abs() <= s_ulp).all())


@pytest.mark.parametrize("k", [40, 700])
def test_fused_forward_selection_with_inf_and_nan(k):
    """Rows with +inf, -inf and NaN through the fused selection of moc_ffn_fwd (every token row is the same one-hot
    vector and the other columns of W_gate are zero, so no 0 * inf arises): NaN counts as the largest value and
    +inf comes next, as in torch.topk and the oracle's key order. The packed floating-point compares of the kernel's
    fast path are not valid for such rows; this checks that it steps aside."""
    from moc_b200 import ffn as F

    lib = _lib.lib()
    dev = torch.device("cuda")
    tokens, d, d_ffn = 1030, 64, 1376
    gen = torch.Generator().manual_seed(5)
    g_row = (torch.randn(d_ffn, generator=gen) * 0.9).to(torch.bfloat16)
    g_row[[3, 500, 1375]] = float("inf")
    g_row[[4, 77]] = float("-inf")
    g_row[[9, 640, 1001]] = float("nan")
    wg = torch.zeros(d_ffn, d, dtype=torch.bfloat16)
    wg[:, 0] = g_row
    wu = (torch.randn(d_ffn, d, generator=gen) * 0.5).to(torch.bfloat16)
    wdt = (torch.randn(d_ffn, d, generator=gen) * 0.02).to(torch.bfloat16)
    x = torch.zeros(tokens, d, dtype=torch.bfloat16)
    x[:, 0] = 1.0
    words = lib.moc_mask_words(d_ffn)
    y = torch.empty(tokens, d, device=dev, dtype=torch.bfloat16)
    idx = torch.full((tokens, k), -1, device=dev, dtype=torch.int16)
    g_sel = torch.zeros(tokens, k, device=dev, dtype=torch.bfloat16)
    u_sel = torch.zeros_like(g_sel)
    bitmap = torch.zeros(tokens, words, device=dev, dtype=torch.int32)
    rank0 = torch.zeros(tokens, words, device=dev, dtype=torch.int16)
    ws_bytes = lib.moc_ffn_fwd_workspace_bytes(0, tokens, d_ffn)
    ws = torch.zeros(ws_bytes, device=dev, dtype=torch.uint8)
    rc = F._call_fwd(lib, 0, 0, tokens, d, d_ffn, k, x.to(dev), wg.to(dev), wu.to(dev), wdt.to(dev), y, idx, g_sel, u_sel,
                     None, None, bitmap, rank0, ws, ws_bytes, dev)
    _lib.check(rc, "moc_ffn_fwd")
    _lib.check(lib.moc_read_status(ws.data_ptr(), _lib.stream_ptr()), "device status")
    torch.cuda.synchronize()
    _, ref_idx = O.canonical_topk(g_row[None, :], k)
    assert torch.equal(idx.cpu().to(torch.int64), ref_idx.expand(tokens, k))
    for ch in (3, 500, 1375, 9, 640, 1001):
        assert ch in ref_idx[0].tolist()
    ref_bm = O.selection_bitmap(ref_idx, d_ffn)
    assert np.array_equal(bitmap.cpu().numpy().view(np.uint32), np.repeat(ref_bm, tokens, axis=0))
