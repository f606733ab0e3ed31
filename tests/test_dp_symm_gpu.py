"""Gradient reduction on two GPUs: the reduced weight gradients of an MoC FFN must equal the mean of the two ranks'
local gradients - by the library's own NVLink kernel (moc_symm_allreduce through moc_b200.dp.SymmGradReducer) in
the multicast (in-switch) form and in the plain peer load/store form, over several steps in a row (the flag words
are never reset between calls), and by the NCCL path of moc_b200.dp.GradAllReducer (ReduceOp.AVG beside the dX
GEMM). Needs two GPUs; ranks are child processes, one per GPU."""
from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, kind: str, overlap: bool, out_dir: str):
    import torch.distributed as dist

    import moc_b200
    from moc_b200.dp import GradAllReducer, SymmGradReducer

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"     # NCCL only carries the rendezvous and the comparison data here
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    d, d_ffn, k, tokens = 256, 1000, 200, 640
    torch.manual_seed(0)
    module = moc_b200.build_ffn(d, d_ffn, "moc", k=k).to(device=dev, dtype=torch.bfloat16)
    use_multicast = kind == "multicast"
    if kind == "nccl":
        reducer = GradAllReducer(average=True, overlap=overlap, reserve_sms=16)
    else:
        reducer = SymmGradReducer(average=True, overlap=overlap, reserve_sms=16, use_multicast=use_multicast)
    worst = 0.0
    for step in range(3):
        g = torch.Generator().manual_seed(100 * step + rank)
        x = torch.randn(tokens, d, generator=g).bfloat16().to(dev).requires_grad_(True)
        dy = torch.randn(tokens, d, generator=g).bfloat16().to(dev)
        module.zero_grad(set_to_none=True)
        module(x).backward(dy)                       # local gradients, no reduction
        torch.cuda.synchronize()
        local = [p.grad.float().clone() for p in module.parameters()]
        want = []
        for t in local:
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            want.append(sum(parts) / world)
        module.zero_grad(set_to_none=True)
        with reducer:
            module(x).backward(dy)
        torch.cuda.synchronize()
        if kind != "nccl":
            reducer.check()
        for p, w in zip(module.parameters(), want):
            err = float((p.grad.float() - w).norm() / w.norm().clamp_min(1e-30))
            worst = max(worst, err)
    # bf16 sums of two bf16 values are rounded once more than the fp32 mean: one part in 2^8
    multicast = getattr(reducer, "multicast", None)
    ok = worst <= 2.0 ** -7 and reducer.launched == 1 and (multicast or not use_multicast)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{int(ok)} worst={worst:.3e} multicast={multicast} launched={reducer.launched}\n")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("kind,overlap", [("multicast", True), ("peer", True), ("multicast", False), ("nccl", True)])
def test_gradient_reduction_two_gpus(kind, overlap, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), kind, overlap, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        line = (tmp_path / f"rank{r}.txt").read_text()
        assert line.startswith("1 "), line


def test_wait_for_an_absent_rank_runs_out_and_is_reported():
    """One GPU plays rank 0 of a two-rank reduction whose rank 1 never shows up (its buffer and flag words are local
    stand-ins that nothing ever signals): the kernel's bounded wait runs out after about a second, the kernel returns,
    moc_symm_allreduce_status reports MOC_ERR_DEVICE_TIMEOUT, and a following one-rank call on fresh flags works.
    Nothing traps or spins without limit."""
    import ctypes
    import time

    from moc_b200 import _lib

    lib = _lib.lib()
    dev = torch.device("cuda:0")
    n = 4096
    bufs = [torch.ones(n, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    nflag = lib.moc_symm_allreduce_flag_bytes() // 4
    flags = [torch.zeros(nflag, device=dev, dtype=torch.int32) for _ in range(2)]
    ptrs = (ctypes.c_void_p * 2)(*[b.data_ptr() for b in bufs])
    fptrs = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
    stream = _lib.stream_ptr()
    t0 = time.perf_counter()
    _lib.check(lib.moc_symm_allreduce(0, 0, 2, ptrs, None, fptrs, n * 2, 1, 1, 4, stream), "moc_symm_allreduce")
    rc = lib.moc_symm_allreduce_status(flags[0].data_ptr(), stream)
    took = time.perf_counter() - t0
    assert rc == _lib.ERR_DEVICE_TIMEOUT and "timed out" in _lib.last_error(), (rc, _lib.last_error())
    assert took < 20.0, took
    # the device is still usable: a one-rank mean over fresh flags leaves the values as they are
    solo = torch.full((n,), 3.0, device=dev, dtype=torch.bfloat16)
    f1 = torch.zeros(nflag, device=dev, dtype=torch.int32)
    p1 = (ctypes.c_void_p * 1)(solo.data_ptr())
    q1 = (ctypes.c_void_p * 1)(f1.data_ptr())
    _lib.check(lib.moc_symm_allreduce(0, 0, 1, p1, None, q1, n * 2, 1, 1, 4, stream), "moc_symm_allreduce")
    assert lib.moc_symm_allreduce_status(f1.data_ptr(), stream) == 0
    assert bool((solo == 3.0).all())
