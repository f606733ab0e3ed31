"""Pin the CPU oracle against fixtures produced by the reference implementation itself
(tests/golden/make_golden.py). CPU only."""
from __future__ import annotations

import pytest
import torch

from conftest import load_golden, max_abs, rel_l2
from oracle import moc_oracle as O

torch.set_num_threads(1)


def _tiny_inputs(gold, dtype):
    return O.make_inputs(gold["meta.tokens"], gold["meta.d"], gold["meta.d_ffn"], dtype, seed=gold["meta.seed"])


@pytest.mark.parametrize("dtype,name", [(torch.float32, "tiny_fp32"), (torch.bfloat16, "tiny_bf16")])
@pytest.mark.parametrize("mode", ["moc", "moc_gcp", "moc_2_8", "moc_post_silu_abs"])
def test_training_matches_reference(dtype, name, mode):
    gold = load_golden(name)
    x, grad_y, wg, wu, wd = _tiny_inputs(gold, dtype)
    k = gold["meta.k"]
    select = {"moc_2_8": "2of8", "moc_post_silu_abs": "post_silu_abs"}.get(mode, "topk")
    fwd = O.moc_forward(x, wg, wu, wd, k, select=select)
    assert fwd["idx"].shape[-1] == gold[f"{mode}.k_effective"]
    # selected channel sets are bit-exact
    assert torch.equal(fwd["idx"].to(torch.int32), gold[f"{mode}.idx_sorted"])
    if mode == "moc_gcp":
        grads = O.moc_backward(grad_y, x, wg, wu, wd, fwd["idx"], fwd["g_sel"], fwd["u_sel"])
    else:
        grads = O.moc_backward(grad_y, x, wg, wu, wd, fwd["idx"], fwd["g_sel"], fwd["u_sel"], fwd["s_sel"],
                               fwd["z_sel"])
    got = dict(y=fwd["y"], dx=grads[0], d_gate_w=grads[1], d_up_w=grads[2], d_down_w=grads[3])
    # The restatement runs the same PyTorch ops in the same order; the only freedom is the order of
    # the selected channels inside a row (ascending here, torch.topk's order in the fp32 reference
    # run), which does not change any value. fp32: tolerance 1e-6 relative; bf16: bit-exact.
    for key, val in got.items():
        ref = gold[f"{mode}.{key}"]
        assert val.dtype == ref.dtype and val.shape == ref.shape
        if dtype == torch.bfloat16:
            assert torch.equal(val, ref), f"{mode}.{key}: max abs diff {max_abs(val, ref)}"
        else:
            assert rel_l2(val, ref) < 1e-6, f"{mode}.{key}: rel l2 {rel_l2(val, ref)}"


def test_bf16_selection_matches_unpatched_topk_multiset():
    """With bf16 ties torch.topk may pick other channels, but the multiset of selected gate
    values cannot differ from the canonical rule's."""
    gold = load_golden("tiny_bf16")
    x, _, wg, wu, wd = _tiny_inputs(gold, torch.bfloat16)
    fwd = O.moc_forward(x, wg, wu, wd, gold["meta.k"])
    vals = torch.sort(fwd["g_sel"].float(), dim=-1).values
    assert torch.equal(vals, gold["moc.unpatched_topk_vals_sorted"])


def test_cfg1_matches_reference():
    """BASELINE config 1 (60m shape, fp32, X [2,256,512]) against the reference's own CPU run."""
    gold = load_golden("cfg1_60m_fp32")
    x, grad_y, wg, wu, wd = O.make_inputs(gold["meta.tokens"], gold["meta.d"], gold["meta.d_ffn"], torch.float32,
                                           seed=gold["meta.seed"])
    fwd = O.moc_forward(x, wg, wu, wd, gold["meta.k"])
    dx, dwg, dwu, dwd = O.moc_backward(grad_y, x, wg, wu, wd, fwd["idx"], fwd["g_sel"], fwd["u_sel"], fwd["s_sel"],
                                       fwd["z_sel"])
    rows, wrows = gold["rows"].long(), gold["wrows"].long()
    assert torch.equal(fwd["idx"][rows].to(torch.int16), gold["idx_sorted_rows"])
    assert int(fwd["idx"].sum()) == gold["idx_checksum"]
    # The fixture was produced with the batch as [2,256,512]; the oracle runs it flattened, so the
    # BLAS blocking may differ: fp32 tolerance 2e-5 relative L2.
    tol = 2e-5
    assert rel_l2(fwd["y"][rows], gold["y_rows"]) < tol
    assert rel_l2(dx[rows], gold["dx_rows"]) < tol
    assert rel_l2(dwg[wrows], gold["d_gate_w_rows"]) < tol
    assert rel_l2(dwu[wrows], gold["d_up_w_rows"]) < tol
    assert rel_l2(dwd[:, wrows], gold["d_down_w_cols"]) < tol
    for key, val in dict(y=fwd["y"], dx=dx, d_gate_w=dwg, d_up_w=dwu, d_down_w=dwd).items():
        v = val.double()
        assert abs((v * v).sum().item() - gold[f"sumsq.{key}"]) <= 1e-5 * gold[f"sumsq.{key}"]


@pytest.mark.parametrize("dtype,name", [(torch.float32, "decode_fp32"), (torch.bfloat16, "decode_bf16")])
def test_decode_matches_reference(dtype, name):
    gold = load_golden(name)
    d, d_ffn, k = gold["meta.d"], gold["meta.d_ffn"], gold["meta.k"]
    for batch in (1, 3):
        x, _, wg, wu, wd = O.make_inputs(batch, d, d_ffn, dtype, seed=77 + batch)
        got = {
            "global.masked_reference": O.masked_reference(x, wg, wu, wd, k=k),
            "g2of8.masked_reference": O.masked_reference(x, wg, wu, wd, select="2of8"),
            "dense_baseline": O.dense_baseline(x, wg, wu, wd),
        }
        for key, val in got.items():
            ref = gold[f"b{batch}.{key}"]
            if dtype == torch.bfloat16:
                assert torch.equal(val, ref), f"{key}: {max_abs(val, ref)}"
            else:
                assert rel_l2(val, ref) < 1e-6


def test_canonical_topk_tie_rule():
    g = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0, -0.0, 0.0]], dtype=torch.bfloat16)
    vals, idx = O.canonical_topk(g, 2)
    assert idx.tolist() == [[1, 2]]            # lowest indices among the three 3.0
    _, idx = O.canonical_topk(g, 4)
    assert idx.tolist() == [[1, 2, 3, 4]]
    _, idx = O.canonical_topk(g, 6)
    assert idx.tolist() == [[0, 1, 2, 3, 4, 6]]   # +0 ranks above -0 in the total order
    _, idx = O.canonical_topk(g, 7)
    assert idx.tolist() == [[0, 1, 2, 3, 4, 5, 6]]


def test_select_2of8_tail_and_ties():
    g = torch.zeros(1, 11)
    g[0, 3] = 1.0
    g[0, 9] = -1.0
    vals, idx = O.select_2of8(g)
    # group 0: channel 3 and, among equal zeros, channel 0; tail (8,9,10): the two zeros
    assert idx.tolist() == [[0, 3, 8, 10]]
    assert O.effective_k_2of8(11) == 4 and O.effective_k_2of8(5461) == 1366 and O.effective_k_2of8(9) == 3
