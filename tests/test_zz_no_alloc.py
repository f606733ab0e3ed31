"""moc_decode_global_static: the decode FFN for callers that cannot hand the library any scratch memory
(for example a host whose device-memory budget is fully handed out, or whose allocator is frozen while it
serves requests). The library keeps the scratch in a fixed array of its own, so the call needs inputs and
outputs only. Checked here through the C ABI against moc_decode_global (which takes a caller workspace)
on the same inputs, twice in a row, because every call reuses the same built-in scratch and must not
depend on what the previous call left there. This file sorts last on purpose, so that a run that stops
at the first failure has already run every other test."""
from __future__ import annotations

import pytest
import torch

from moc_b200 import _lib
from moc_b200.ffn import transpose_weight
from oracle import moc_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _workspace_call(batch, d, d_ffn, k, x, wg, wu, wdt):
    lib = _lib.lib()
    y = torch.empty(batch, d, device="cuda", dtype=BF)
    n = lib.moc_decode_workspace_bytes(batch, d, d_ffn)
    ws = torch.empty(n, device="cuda", dtype=torch.uint8)
    _lib.check(lib.moc_decode_global(batch, d, d_ffn, k, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), wdt.data_ptr(),
                                     y.data_ptr(), ws.data_ptr(), n, _lib.stream_ptr()), "moc_decode_global")
    return y


def _static_call(batch, d, d_ffn, k, x, wg, wu, wdt):
    y = torch.full((batch, d), float("nan"), device="cuda", dtype=BF)
    _lib.check(_lib.lib().moc_decode_global_static(batch, d, d_ffn, k, x.data_ptr(), wg.data_ptr(), wu.data_ptr(),
                                                   wdt.data_ptr(), y.data_ptr(), _lib.stream_ptr()),
               "moc_decode_global_static")
    return y


def test_static_scratch_entry_matches_workspace_entry_twice():
    for call, (batch, d, d_ffn, k, seed) in enumerate([(8, 2048, 5461, 1024, 11), (3, 256, 1000, 200, 12),
                                                        (1, 2048, 5461, 1024, 13), (1, 256, 1000, 200, 14)]):
        x, _, wg, wu, wd = O.make_inputs(batch, d, d_ffn, BF, seed=seed)
        xc, wgc, wuc = x.cuda(), wg.cuda(), wu.cuda()
        wdt = transpose_weight(wd.cuda())
        ref = _workspace_call(batch, d, d_ffn, k, xc, wgc, wuc, wdt)
        got = _static_call(batch, d, d_ffn, k, xc, wgc, wuc, wdt)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # same kernels, same launch plan: the tolerance of the decode tests (relative L2 <= 1e-2) is met exactly
        err = (got.double() - ref.double()).norm() / ref.double().norm()
        assert err <= 1e-2, f"call {call}: relative L2 {err:.3e}"
        assert torch.equal(got, ref), f"call {call}: results differ bitwise"


def test_static_scratch_entry_rejects_sizes_beyond_its_limits():
    lib = _lib.lib()
    assert (lib.moc_decode_static_max_batch(), lib.moc_decode_static_max_d(), lib.moc_decode_static_max_d_ffn()) == \
        (8, 4096, 8192)
    t = torch.zeros(16, device="cuda", dtype=BF)
    for batch, d, d_ffn in ((9, 2048, 5461), (1, 8192, 5461), (1, 2048, 16384)):
        rc = lib.moc_decode_global_static(batch, d, d_ffn, 8, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                          t.data_ptr(), _lib.stream_ptr())
        assert rc == -2 and "exceed the built-in scratch" in _lib.last_error()
