"""torch.library ops of moc_b200.ops: schema / fake-kernel checks (torch.library.opcheck) and agreement with the
oracle's decode restatement and with the composed pipeline."""
from __future__ import annotations

import pytest
import torch

from conftest import rel_l2
from moc_b200 import ops
from moc_b200.ffn import transpose_weight
from oracle import moc_oracle as O

BF = torch.bfloat16


def _inputs(batch, d, d_ffn, seed):
    x, _, wg, wu, wd = O.make_inputs(batch, d, d_ffn, BF, seed=seed)
    return x.cuda(), wg.cuda(), wu.cuda(), wd.cuda()


def test_fake_kernels_trace_without_a_gpu():
    """FakeTensor tracing sees shapes and dtypes of every op without running CUDA code (CPU-only test)."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(3, 64, dtype=BF)
        wg = torch.empty(176, 64, dtype=BF)
        wdt = torch.empty(176, 64, dtype=BF)
        scores = torch.empty(3, 176, dtype=BF)
        vals, idx = torch.ops.moc_b200.global_topk(scores, 40)
        assert vals.shape == (3, 40) and idx.dtype == torch.int64
        z = torch.ops.moc_b200.selected_up_silu(x, vals, idx, wg)
        assert z.shape == (3, 40) and z.dtype == BF
        assert torch.ops.moc_b200.selected_down(z, idx, wdt).shape == (3, 64)
        assert torch.ops.moc_b200.global_after_gate(x, scores, wg, wdt, 40).shape == (3, 64)
        assert torch.ops.moc_b200.global_ffn(x, wg, wg, wdt, 40).shape == (3, 64)
        assert torch.ops.moc_b200.grouped_2of8_ffn(x, wg, wg, wdt).shape == (3, 64)


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [1, 5])
def test_ops_match_oracle_and_compose(batch):
    d, d_ffn, k = 256, 1001, 200
    x, wg, wu, wd = _inputs(batch, d, d_ffn, seed=31 + batch)
    wdt = transpose_weight(wd)
    scores = (x.float() @ wg.float().t()).to(BF)          # torch product only to feed the ops a score tensor
    vals, idx = ops.global_topk(scores, k)
    ref_vals, ref_idx = O.canonical_topk(scores.cpu(), k)
    assert torch.equal(idx.cpu(), ref_idx) and torch.equal(vals.cpu(), ref_vals)
    z = ops.selected_up_silu(x, vals, idx, wu)
    y_parts = ops.selected_down(z, idx, wdt)
    y_one = ops.global_after_gate(x, scores, wu, wdt, k)
    assert rel_l2(y_parts.float().cpu(), y_one.float().cpu()) < 1e-2
    # oracle with the same selection
    u = (x.float().cpu() @ wu.float().cpu().t()).to(BF)
    z_ref = (torch.nn.functional.silu(ref_vals) * torch.gather(u, -1, ref_idx))
    assert rel_l2(z.float().cpu(), z_ref.float()) < 1e-2
    y_ref = O.masked_reference(x.cpu(), wg.cpu(), wu.cpu(), wd.cpu(), k)
    y_full = ops.global_ffn(x, wg, wu, wdt, k)
    assert rel_l2(y_full.float().cpu(), y_ref.float()) < 5e-2
    y28 = ops.grouped_2of8_ffn(x, wg, wu, wdt)
    y28_ref = O.masked_reference(x.cpu(), wg.cpu(), wu.cpu(), wd.cpu(), select="2of8")
    assert rel_l2(y28.float().cpu(), y28_ref.float()) < 5e-2


@pytest.mark.gpu
def test_opcheck():
    x, wg, wu, wd = _inputs(2, 64, 176, seed=9)
    wdt = transpose_weight(wd)
    scores = (x.float() @ wg.float().t()).to(BF)
    vals, idx = ops.global_topk(scores, 40)
    z = ops.selected_up_silu(x, vals, idx, wu)
    checks = ("test_schema", "test_faketensor")
    torch.library.opcheck(torch.ops.moc_b200.global_topk.default, (scores, 40), test_utils=checks)
    torch.library.opcheck(torch.ops.moc_b200.selected_up_silu.default, (x, vals, idx, wu), test_utils=checks)
    torch.library.opcheck(torch.ops.moc_b200.selected_down.default, (z, idx, wdt), test_utils=checks)
    torch.library.opcheck(torch.ops.moc_b200.global_after_gate.default, (x, scores, wu, wdt, 40), test_utils=checks)
    torch.library.opcheck(torch.ops.moc_b200.global_ffn.default, (x, wg, wu, wdt, 40), test_utils=checks)
    torch.library.opcheck(torch.ops.moc_b200.grouped_2of8_ffn.default, (x, wg, wu, wdt), test_utils=checks)
