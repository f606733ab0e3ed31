"""GEMM cores through the C ABI (moc_gemm) against a plain PyTorch fp32 product.

Covers every operand-major combination the FFN path uses, tile tails in M, N and K, and the
transposed store. bf16 inputs: the fp32 reference product of the same bf16 values, rounded
once to bf16, must match within 1 bf16 ulp of accumulation-order noise (rtol 2^-7, atol 1e-2
at these magnitudes)."""
from __future__ import annotations

import pytest
import torch

from moc_b200 import _lib

pytestmark = pytest.mark.gpu


def _run_gemm(dtype, impl, m, n, k, a_mn, b_mn, c_t, seed=0):
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(seed)
    a_log = torch.randn(m, k, generator=g).to(dtype)
    b_log = torch.randn(n, k, generator=g).to(dtype)
    # memory layouts: K-major = [mn][k], MN-major = [k][mn]; leading dims padded to a multiple of 8
    def lay(t, mn_major):
        t = t.t().contiguous() if mn_major else t.contiguous()
        rows, cols = t.shape
        ld = (cols + 7) // 8 * 8
        buf = torch.zeros(rows, ld, dtype=dtype)
        buf[:, :cols] = t
        return buf.to(dev), ld
    a_dev, lda = lay(a_log, a_mn)
    b_dev, ldb = lay(b_log, b_mn)
    if c_t:
        c = torch.full((n, m), float("nan"), device=dev, dtype=dtype)
        ldc = m
    else:
        c = torch.full((m, n), float("nan"), device=dev, dtype=dtype)
        ldc = n
    status = torch.zeros(64, device=dev, dtype=torch.int32)
    rc = _lib.lib().moc_gemm(_lib.dtype_code(dtype), impl, m, n, k, a_dev.data_ptr(), lda, int(a_mn),
                             b_dev.data_ptr(), ldb, int(b_mn), c.data_ptr(), ldc, int(c_t), status.data_ptr(),
                             _lib.stream_ptr())
    _lib.check(rc, "moc_gemm")
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0, f"device status {int(status[0].item()):#x}"
    ref = a_log.float() @ b_log.float().t()
    got = (c.t() if c_t else c).float().cpu()
    return got, ref


CASES = [
    # m, n, k
    (128, 256, 64),
    (128, 256, 256),
    (256, 512, 320),
    (130, 300, 100),     # tails in M, N and K
    (1, 8, 8),
    (3, 5461, 2048),     # odd N (d_ffn of the 1b preset), tiny M
    (640, 384, 5461),    # odd K
    (1000, 777, 1200),   # several 256-row tile pairs with a tail in each dimension
    (4693, 1024, 192),   # 18 tile pairs + 85 rows on 148 SMs: impl 0 runs the tail rows as a second kernel on a side stream
]

# bf16 tensor-core cores: 0 = automatic choice, 2 = CTA-pair kernel (256-row tiles), 3 = single-CTA kernel
TC_IMPLS = [0, 2, 3]


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("m,n,k", CASES)
@pytest.mark.parametrize("impl", TC_IMPLS)
def test_tcgen05_gemm_bf16(impl, m, n, k, a_mn, b_mn):
    got, ref = _run_gemm(torch.bfloat16, impl, m, n, k, a_mn, b_mn, 0, seed=m + n + k)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, ref.bfloat16().float(), rtol=2 ** -7, atol=1e-2 * max(1.0, (k / 64) ** 0.5))


@pytest.mark.parametrize("m,n,k", [(130, 300, 100), (256, 512, 320), (4693, 1024, 192)])
@pytest.mark.parametrize("impl", TC_IMPLS)
def test_tcgen05_gemm_transposed_store(impl, m, n, k):
    got, ref = _run_gemm(torch.bfloat16, impl, m, n, k, 1, 1, 1, seed=7)
    torch.testing.assert_close(got, ref.bfloat16().float(), rtol=2 ** -7, atol=2e-2)


@pytest.mark.parametrize("c_t", [0, 1])
@pytest.mark.parametrize("a_mn", [0, 1])
@pytest.mark.parametrize("m,n,k", [(5461, 64, 2048), (300, 40, 200), (257, 100, 320), (129, 128, 64), (2048, 9, 5461),
                                   (700, 16, 72)])
def test_tcgen05_gemm_few_columns(m, n, k, a_mn, c_t):
    """Products with at most 128 columns and a K-major B (the decode projections: weights as the M operand, batch
    rows as N) run on the single-CTA kernel with an MMA and a B tile as narrow as N allows and a deeper operand
    ring."""
    got, ref = _run_gemm(torch.bfloat16, 3, m, n, k, a_mn, 0, c_t, seed=m + n)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, ref.bfloat16().float(), rtol=2 ** -7, atol=1e-2 * max(1.0, (k / 64) ** 0.5))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("a_mn,b_mn,c_t", [(0, 0, 0), (0, 1, 0), (1, 1, 1)])
def test_simt_gemm(dtype, a_mn, b_mn, c_t):
    got, ref = _run_gemm(dtype, 1, 130, 300, 100, a_mn, b_mn, c_t, seed=3)
    if dtype == torch.float32:
        torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-4)
    else:
        torch.testing.assert_close(got, ref.bfloat16().float(), rtol=2 ** -7, atol=2e-2)


def test_pair_and_single_cta_kernels_agree_bitwise():
    """Both tensor-core kernels add the same K blocks in the same order into fp32 TMEM accumulators, so their
    bf16 results are identical bit for bit."""
    a, _ = _run_gemm(torch.bfloat16, 2, 1000, 777, 1200, 0, 1, 0, seed=13)
    b, _ = _run_gemm(torch.bfloat16, 3, 1000, 777, 1200, 0, 1, 0, seed=13)
    assert torch.equal(a, b)


@pytest.mark.parametrize("impl", TC_IMPLS)
def test_tcgen05_matches_simt_bitwise_class(impl):
    """Same bf16 inputs through both cores: both accumulate in fp32, results may differ only by
    the final rounding of slightly different fp32 sums."""
    a, ref = _run_gemm(torch.bfloat16, impl, 256, 512, 512, 0, 0, 0, seed=11)
    b, _ = _run_gemm(torch.bfloat16, 1, 256, 512, 512, 0, 0, 0, seed=11)
    diff = (a - b).abs()
    assert (diff > 0).float().mean().item() < 0.05
    torch.testing.assert_close(a, b, rtol=2 ** -7, atol=2e-2)
