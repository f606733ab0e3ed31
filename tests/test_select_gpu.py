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
