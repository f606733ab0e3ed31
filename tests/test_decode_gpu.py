"""Decode-time MoC FFN kernels through the C ABI and the InferenceMoCSwiGLUFFN surface, against the
CPU oracle's masked_reference / dense_baseline and the reference-generated fixtures.

Tolerances (bf16): with the SAME gate scores on both sides (moc_decode_after_gate fed with the
oracle's scores) the channel sets are identical and y must agree to relative L2 <= 1e-2 and 4 bf16
ulps of the largest magnitude. With each side's own gate projection a 1-ulp difference in a score
at the threshold can swap one channel of a row, so that path is held to relative L2 <= 5e-2."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from conftest import load_golden, max_abs, rel_l2
from moc_b200 import _lib
from moc_b200.ffn import transpose_weight
from moc_b200.inference import InferenceMoCSwiGLUFFN
from oracle import moc_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _ws(batch, d, d_ffn):
    n = _lib.lib().moc_decode_workspace_bytes(batch, d, d_ffn)
    return torch.empty(n, device="cuda", dtype=torch.uint8)


def _call(name, batch, d, d_ffn, k, x, a, wu, wdt):
    """a = w_gate (or gate scores for moc_decode_after_gate)."""
    y = torch.full((batch, d), float("nan"), device="cuda", dtype=BF)
    ws = _ws(batch, d, d_ffn)
    args = [batch, d, d_ffn] + ([k] if k is not None else [])
    args += [x.data_ptr(), a.data_ptr(), wu.data_ptr(), wdt.data_ptr(), y.data_ptr(), ws.data_ptr(), ws.numel(),
             _lib.stream_ptr()]
    _lib.check(getattr(_lib.lib(), name)(*args), name)
    torch.cuda.synchronize()
    return y.cpu()


def _close(got, ref, tol, label):
    assert torch.isfinite(got.float()).all(), label
    r, a = rel_l2(got, ref), max_abs(got, ref)
    print(f"{label}: rel_l2={r:.3e} max_abs={a:.3e}")
    assert r <= tol, f"{label}: rel_l2 {r:.3e}"


SHAPES = [(64, 176, 40), (256, 1000, 200), (512, 1376, 256), (2048, 5461, 1024)]


@pytest.mark.parametrize("batch", [1, 2, 3, 8, 13, 64])
@pytest.mark.parametrize("d,d_ffn,k", SHAPES)
def test_decode_global_and_after_gate(batch, d, d_ffn, k):
    if d_ffn == 5461 and batch not in (1, 8, 64):
        pytest.skip("1b shape: batches of BASELINE config 3 only")
    x, _, wg, wu, wd = O.make_inputs(batch, d, d_ffn, BF, seed=batch + d)
    ref = O.masked_reference(x, wg, wu, wd, k=k)
    xc, wgc, wuc = x.cuda(), wg.cuda(), wu.cuda()
    wdt = transpose_weight(wd.cuda())
    scores = F.linear(x, wg).cuda()            # the oracle's own bf16 gate scores
    got = _call("moc_decode_after_gate", batch, d, d_ffn, k, xc, scores, wuc, wdt)
    _close(got, ref, 1e-2, f"after_gate[{batch},{d},{d_ffn}]")
    scale = ref.float().abs().max().item()
    assert max_abs(got, ref) <= 4 * scale * 2 ** -8 + 1e-6
    got2 = _call("moc_decode_global", batch, d, d_ffn, k, xc, wgc, wuc, wdt)
    _close(got2, ref, 5e-2, f"global[{batch},{d},{d_ffn}]")
    again = _call("moc_decode_global", batch, d, d_ffn, k, xc, wgc, wuc, wdt)
    assert torch.equal(got2, again), "decode must be run-to-run deterministic"


@pytest.mark.parametrize("batch", [1, 5, 8, 64])
@pytest.mark.parametrize("d,d_ffn", [(64, 176), (256, 1001), (2048, 5461), (2048, 5464)])
def test_decode_2of8_and_dense(batch, d, d_ffn):
    x, _, wg, wu, wd = O.make_inputs(batch, d, d_ffn, BF, seed=batch + d_ffn)
    xc, wgc, wuc = x.cuda(), wg.cuda(), wu.cuda()
    wdt = transpose_weight(wd.cuda())
    ref = O.masked_reference(x, wg, wu, wd, select="2of8")
    got = _call("moc_decode_2of8", batch, d, d_ffn, None, xc, wgc, wuc, wdt)
    _close(got, ref, 5e-2, f"2of8[{batch},{d},{d_ffn}]")
    refd = O.dense_baseline(x, wg, wu, wd)
    gotd = _call("moc_decode_dense", batch, d, d_ffn, None, xc, wgc, wuc, wdt)
    _close(gotd, refd, 1e-2, f"dense[{batch},{d},{d_ffn}]")


@pytest.mark.parametrize("batch", [8, 64])
def test_decode_dense_widest_d_ffn(batch):
    """d_ffn = 32768 (the widest the int16 channel indices address) with a small hidden size: here the split-K
    products of the dense baseline have more 128-row tiles than the device has SMs, so each keeps a single
    partial block of d_ffn rows; the gate and up blocks must not overlap and must stay inside the workspace.
    A canary behind the workspace must survive."""
    d, d_ffn = 64, 32768
    x, _, wg, wu, wd = O.make_inputs(batch, d, d_ffn, BF, seed=batch)
    n = _lib.lib().moc_decode_workspace_bytes(batch, d, d_ffn)
    buf = torch.full((n + 4096,), 0x5A, device="cuda", dtype=torch.uint8)
    y = torch.full((batch, d), float("nan"), device="cuda", dtype=BF)
    xc, wgc, wuc = x.cuda(), wg.cuda(), wu.cuda()
    wdt = transpose_weight(wd.cuda())
    _lib.check(_lib.lib().moc_decode_dense(batch, d, d_ffn, xc.data_ptr(), wgc.data_ptr(), wuc.data_ptr(),
                                           wdt.data_ptr(), y.data_ptr(), buf.data_ptr(), n, _lib.stream_ptr()),
               "moc_decode_dense")
    torch.cuda.synchronize()
    assert bool((buf[n:] == 0x5A).all()), "write beyond the workspace"
    _close(y.cpu(), O.dense_baseline(x, wg, wu, wd), 1e-2, f"dense[{batch},{d},{d_ffn}]")


def test_bounded_wait_runs_out_and_the_next_call_recovers():
    """Every device-side wait of the library is bounded. With the grid-barrier limit lowered to one cycle
    (moc_debug_set_wait_cycles) the persistent decode kernel's first barrier gives up in the CTAs that do not
    arrive last: the kernel must return (no trap, no endless spin), the status word must report the time-out
    through both the synchronous and the asynchronous reader, and the next call with the normal limit must be
    correct again."""
    lib = _lib.lib()
    batch, d, d_ffn, k = 1, 2048, 5461, 1024
    x, _, wg, wu, wd = O.make_inputs(batch, d, d_ffn, BF, seed=5)
    xc, wgc, wuc = x.cuda(), wg.cuda(), wu.cuda()
    wdt = transpose_weight(wd.cuda())
    y = torch.zeros(batch, d, device="cuda", dtype=BF)
    ws = _ws(batch, d, d_ffn)
    sink = torch.zeros(1, dtype=torch.int32).pin_memory()
    args = [batch, d, d_ffn, k, xc.data_ptr(), wgc.data_ptr(), wuc.data_ptr(), wdt.data_ptr(), y.data_ptr(),
            ws.data_ptr(), ws.numel(), _lib.stream_ptr()]
    _lib.check(lib.moc_debug_set_wait_cycles(1), "moc_debug_set_wait_cycles")
    try:
        _lib.check(lib.moc_decode_global(*args), "moc_decode_global")
        _lib.check(lib.moc_publish_status(ws.data_ptr(), sink.data_ptr(), _lib.stream_ptr()), "moc_publish_status")
        rc = lib.moc_read_status(ws.data_ptr(), _lib.stream_ptr())
    finally:
        lib.moc_debug_set_wait_cycles(0)
    assert rc == _lib.ERR_DEVICE_TIMEOUT and "timed out" in _lib.last_error()
    torch.cuda.synchronize()
    assert int(sink[0]) != 0
    _lib.check(lib.moc_decode_global(*args), "moc_decode_global")
    assert lib.moc_read_status(ws.data_ptr(), _lib.stream_ptr()) == 0
    _close(y.cpu(), O.masked_reference(x, wg, wu, wd, k=k), 5e-2, "after a time-out")


def test_decode_golden_fixture():
    """tests/golden/decode_bf16.npz: the reference's masked_reference / dense_baseline on CPU."""
    gold = load_golden("decode_bf16")
    d, d_ffn, k = gold["meta.d"], gold["meta.d_ffn"], gold["meta.k"]
    for batch in (1, 3):
        x, _, wg, wu, wd = O.make_inputs(batch, d, d_ffn, BF, seed=77 + batch)
        xc, wuc = x.cuda(), wu.cuda()
        wdt = transpose_weight(wd.cuda())
        scores = F.linear(x, wg).cuda()
        got = _call("moc_decode_after_gate", batch, d, d_ffn, k, xc, scores, wuc, wdt)
        _close(got, gold[f"b{batch}.global.masked_reference"], 1e-2, f"golden global b{batch}")
        got = _call("moc_decode_dense", batch, d, d_ffn, None, xc, wg.cuda(), wuc, wdt)
        _close(got, gold[f"b{batch}.dense_baseline"], 1e-2, f"golden dense b{batch}")
        got = _call("moc_decode_2of8", batch, d, d_ffn, None, xc, wg.cuda(), wuc, wdt)
        _close(got, gold[f"b{batch}.g2of8.masked_reference"], 5e-2, f"golden 2of8 b{batch}")


def test_selected_down_alone():
    batch, k, d, d_ffn = 3, 37, 256, 500
    g = torch.Generator().manual_seed(3)
    z = torch.randn(batch, k, generator=g).to(BF)
    idx = torch.stack([torch.randperm(d_ffn, generator=g)[:k].sort().values for _ in range(batch)]).to(torch.int16)
    wdt = (torch.randn(d_ffn, d, generator=g) * 0.05).to(BF)
    y = torch.empty(batch, d, device="cuda", dtype=BF)
    ws = _ws(batch, d, d_ffn)
    zc, ic, wc = z.cuda(), idx.cuda(), wdt.cuda()
    _lib.check(_lib.lib().moc_decode_selected_down(batch, k, d, d_ffn, zc.data_ptr(), ic.data_ptr(), wc.data_ptr(),
                                                   y.data_ptr(), ws.data_ptr(), ws.numel(), _lib.stream_ptr()),
               "moc_decode_selected_down")
    ref = torch.einsum("bk,bkd->bd", z.float(), wdt.float()[idx.long()]).to(BF)
    _close(y.cpu(), ref, 1e-2, "selected_down")


def test_module_surface():
    m = InferenceMoCSwiGLUFFN(256, 1000, 200)
    assert m.config.k == 200 and not m.config.grouped and m.config.hidden_size == 256
    assert list(m.state_dict().keys()) == ["gate_proj.weight", "up_proj.weight", "down_proj.weight"]
    with pytest.raises(ValueError):
        InferenceMoCSwiGLUFFN(256, 1000, 0)
    with pytest.raises(ValueError):
        InferenceMoCSwiGLUFFN(256, 1000, 200, grouped_a=2)
    with pytest.raises(ValueError):
        InferenceMoCSwiGLUFFN(256, 1000, 200, grouped_a=2, grouped_b=8)   # k must be 250
    with pytest.raises(ValueError, match="CUDA"):
        m.bfloat16()(torch.randn(2, 256).bfloat16())
    m = m.cuda().bfloat16()
    with pytest.raises(ValueError, match="BF16"):
        m.float()(torch.randn(2, 256, device="cuda"))
    m = m.bfloat16()
    x = torch.randn(4, 1, 256, device="cuda", dtype=BF)
    y = m(x)
    assert y.shape == (4, 1, 256)
    ref = m(x, mode="masked_reference")
    assert rel_l2(y.cpu(), ref.cpu()) < 5e-2
    with pytest.raises(ValueError):
        m(x, mode="moc_inference_grouped_top2of8")
    with pytest.raises(ValueError):
        m(torch.randn(4, 2, 256, device="cuda", dtype=BF))
    yd = m(x, mode="dense_baseline")
    refd = m.down_proj(F.silu(m.gate_proj(x)) * m.up_proj(x))
    assert rel_l2(yd.cpu(), refd.cpu()) < 1e-2
    # in-place weight updates are picked up through the cached transposed copy
    with torch.no_grad():
        m.down_proj.weight.mul_(-1.0)
    assert rel_l2(m(x).cpu(), (-y).cpu()) < 1e-3
    g = InferenceMoCSwiGLUFFN(256, 1001, 251, grouped_a=2, grouped_b=8).cuda().bfloat16()
    xg = torch.randn(3, 256, device="cuda", dtype=BF)
    assert rel_l2(g(xg).cpu(), g(xg, mode="masked_reference").cpu()) < 5e-2
    runner = g.make_moc2_8_graph_runner(3)
    assert torch.equal(runner(xg), g(xg))
    runner2 = m.make_graph_runner(4)
    assert torch.equal(runner2(x), m(x))
