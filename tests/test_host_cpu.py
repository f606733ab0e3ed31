"""CPU-only checks: the C-ABI library loads and exports every symbol the header declares, the
host-side plugin surface mirrors the reference's (names, attributes, errors), and the token-sharded
data-parallel bookkeeping works across two gloo ranks. No kernel is launched here."""
from __future__ import annotations

import os
import re
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import moc_b200  # noqa: E402
from moc_b200 import _lib, dp  # noqa: E402
from moc_b200.ffn import MoCSwiGLUFFN, StandardSwiGLUFFN, build_ffn  # noqa: E402
from oracle import moc_oracle as O  # noqa: E402


def _declared_functions():
    text = (ROOT / "include" / "moc_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_functions()
    assert len(names) >= 15
    lib = _lib.lib()
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/moc_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in moc_b200/_lib.py"
    for name in _lib.SIGNATURES:
        assert name in names, f"{name} is bound in _lib.py but not declared in the header"
    assert lib.moc_b200_abi_version() == 1


def test_layout_helpers_without_gpu():
    lib = _lib.lib()
    assert lib.moc_ffn_ld(5461) == 5504 and lib.moc_ffn_ld(128) == 128 and lib.moc_ffn_ld(129) == 256
    assert lib.moc_mask_words(5461) == 172
    for f in (8, 9, 11, 173, 1376, 5461, 5464):
        assert lib.moc_select_2of8_k(f) == O.effective_k_2of8(f)
    assert lib.moc_ffn_fwd_workspace_bytes(_lib.MOC_BF16, 16384, 5461) == 256 + 2 * 16384 * 5504 * 2
    assert lib.moc_ffn_bwd_workspace_bytes(_lib.MOC_F32, 3, 100) == 256 + 3 * 1536
    assert lib.moc_decode_workspace_bytes(8, 2048, 5461) > 0


def test_argument_errors_are_reported_not_raised_in_c():
    lib = _lib.lib()
    rc = lib.moc_topk_select(_lib.MOC_BF16, None, 8, 1, 8, 2, None, None, None, None, None)
    assert rc == -1 and "null" in _lib.last_error()
    rc = lib.moc_ffn_fwd(7, 0, 1, 8, 8, 2, *([None] * 13), 0, None)
    assert rc == -1 and "dtype" in _lib.last_error()
    rc = lib.moc_gemm(_lib.MOC_BF16, 0, 4, 4, 0, None, 0, 0, None, 0, 0, None, 0, 0, None, None)
    assert rc == -1
    with pytest.raises(RuntimeError, match="code -1"):
        _lib.check(rc, "moc_gemm")


def test_build_ffn_surface_matches_reference():
    d = build_ffn(64, 173)
    assert isinstance(d, StandardSwiGLUFFN)
    m = build_ffn(64, 173, "moc", k=40)
    assert isinstance(m, MoCSwiGLUFFN) and m.mode == "moc_triton_aux" and m.index_save_dtype == torch.int16
    assert (m.k, m.k_effective, m.requested_k) == (40, 40, 40)
    g = build_ffn(64, 173, "moc_gcp", k=40)
    assert g.mode == "moc_gcp_triton_aux"
    s = build_ffn(64, 173, "moc_2_8", k=99)
    assert s.k_effective == 44 and s.requested_k == 99 and s.mode == "moc_2_8_triton_aux"
    for mod in (d, m, g, s):
        assert [n for n, _ in mod.named_parameters()] == ["gate_proj.weight", "up_proj.weight", "down_proj.weight"]
        assert mod.gate_proj.weight.shape == (173, 64) and mod.down_proj.weight.shape == (64, 173)
        assert mod.gate_proj.bias is None
    with pytest.raises(ValueError, match="requires `k`"):
        build_ffn(64, 173, "moc")
    with pytest.raises(ValueError, match="Unknown ffn_type"):
        build_ffn(64, 173, "sparse")
    with pytest.raises(ValueError, match="Unknown mode"):
        MoCSwiGLUFFN(64, 173, 40, mode="nope")
    with pytest.raises(ValueError, match="requires `k`"):
        MoCSwiGLUFFN(64, 173, None, mode="moc")
    with pytest.raises(ValueError, match="cannot be stored"):
        MoCSwiGLUFFN(8, 40000, 10, mode="moc")
    with pytest.raises(ValueError, match="require CUDA"):
        m(torch.randn(2, 64))
    with pytest.raises(ValueError, match="require CUDA"):
        d(torch.randn(2, 64))


def test_install_into_rebinds_a_reference_like_package(tmp_path):
    pkg = tmp_path / "fakemoc"
    pkg.mkdir()
    (pkg / "__init__.py").write_text("from .ffn import build_ffn\nfrom .model import make\n")
    (pkg / "ffn.py").write_text("def build_ffn(*a, **k):\n    return 'reference'\n")
    (pkg / "model.py").write_text("from .ffn import build_ffn\n\ndef make():\n    return build_ffn(8, 16, 'moc', k=4)\n")
    sys.path.insert(0, str(tmp_path))
    try:
        import fakemoc
        assert fakemoc.make() == "reference"
        moc_b200.install_into(fakemoc)
        assert isinstance(fakemoc.make(), MoCSwiGLUFFN)
    finally:
        sys.path.remove(str(tmp_path))
        for name in [n for n in sys.modules if n.startswith("fakemoc")]:
            del sys.modules[name]


def test_shard_bounds_cover_all_tokens():
    for total, world in ((16384, 8), (10, 4), (3, 8), (0, 2)):
        spans = [dp.shard_bounds(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    tokens, d, d_ffn, k = 48, 32, 72, 16
    x, dy, wg, wu, wd = O.make_inputs(tokens, d, d_ffn, torch.float32, seed=5)
    b, e = dp.shard_bounds(tokens, world, rank)
    fwd = O.moc_forward(x[b:e], wg, wu, wd, k)
    grads = O.moc_backward(dy[b:e], x[b:e], wg, wu, wd, fwd["idx"], fwd["g_sel"], fwd["u_sel"], fwd["s_sel"],
                           fwd["z_sel"])
    reducer = dp.GradAllReducer(average=False)
    with reducer:
        for name, g in zip(("gate", "up", "down"), grads[1:]):
            reducer._on_grad_ready(name, g, None)   # what the autograd node does after the backward kernels
    assert reducer.launched == 3
    if rank == 0:
        torch.save([g.clone() for g in grads[1:]], out)
    dist.destroy_process_group()


def test_two_rank_gradient_reduction_matches_full_batch(tmp_path):
    """Token sharding: the sum of the per-shard weight gradients equals the full-batch gradients."""
    out = tmp_path / "grads.pt"
    mp.spawn(_dp_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    got = torch.load(out)
    tokens, d, d_ffn, k = 48, 32, 72, 16
    x, dy, wg, wu, wd = O.make_inputs(tokens, d, d_ffn, torch.float32, seed=5)
    fwd = O.moc_forward(x, wg, wu, wd, k)
    ref = O.moc_backward(dy, x, wg, wu, wd, fwd["idx"], fwd["g_sel"], fwd["u_sel"], fwd["s_sel"], fwd["z_sel"])[1:]
    for a, b in zip(got, ref):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
