"""The real drop-in: the reference's own model code (moc/model.py, installed unmodified under baseline/_ref by
baseline/install_ref.py) with the B200 FFN modules bound into it by ``moc_b200.install_into``. The fixture
tests/golden/host_tiny_fp32.npz holds the reference model's state_dict, inputs, logits, loss and gradients
from its CPU run with its own pure-PyTorch FFN (tests/golden/make_golden.py); the same model object, now
constructing this package's modules through ``build_ffn`` (moc/model.py:81), must reproduce them on the GPU.
Skipped when baseline/_ref is absent."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

import moc_b200
from conftest import load_golden, rel_l2

REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF / "moc" / "model.py").exists(), reason="baseline/_ref is not installed")]


def _reference_package():
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import moc
    return moc


@pytest.mark.parametrize("ffn_type", ["dense", "moc"])
def test_reference_model_runs_on_the_b200_ffn(ffn_type):
    moc = _reference_package()
    originals = (moc.model.build_ffn, moc.build_ffn)
    moc_b200.install_into(moc)
    try:
        cfg = moc.MoCConfig(hidden_size=64, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
                            vocab_size=97, max_seq_len=16, k=40)
        model = moc.build_model(cfg, ffn_type)
        expected = moc_b200.StandardSwiGLUFFN if ffn_type == "dense" else moc_b200.MoCSwiGLUFFN
        assert all(type(b.ffn) is expected for b in model.blocks)
        assert ffn_type == "dense" or model.blocks[0].ffn.k_effective == 40     # read by the reference's train script
        gold = load_golden("host_tiny_fp32")
        model.load_state_dict({k[len("state."):]: v for k, v in gold.items() if k.startswith("state.")}, strict=True)
        model = model.cuda()
        out = model(gold["ids"].cuda(), labels=gold["labels"].cuda())
        logits, loss = (out["logits"], out["loss"]) if isinstance(out, dict) else out
        loss.backward()
        moc_b200.flush_status()
        assert rel_l2(logits.detach().cpu(), gold[f"{ffn_type}.logits"]) < 1e-4
        assert abs(loss.item() - float(gold[f"{ffn_type}.loss"])) < 1e-4
        params = dict(model.named_parameters())
        for name in ("tok_emb.weight", "blocks.0.ffn.gate_proj.weight", "blocks.1.ffn.down_proj.weight",
                     "blocks.0.attn.qkv_proj.weight", "lm_head.weight"):
            assert rel_l2(params[name].grad.cpu(), gold[f"{ffn_type}.grad.{name}"]) < 2e-4, name
    finally:
        moc.model.build_ffn, moc.build_ffn = originals
